// Launchers of the child-sum Tree-GRU cell kernels (kernels/gru.cu).  Level rows are [off, off+rows) of
// arenas in tensor-id order; child [K, n_total], parent [n_total]; state is [n_total, H] (h only);
// A is the per-token input projection [tokens, 3H] (blocks r,z,n) read through a_row (NULL: one row per
// vertex); PR [rows,K,H], PZ / PN [rows,H] are the level's recurrent products.  bf16: storage type of
// A, PR, PZ, PN, M, dA, ZR (else fp32).
#ifndef CAVS_B200_KERNELS_GRU_H_
#define CAVS_B200_KERNELS_GRU_H_

#include <cuda_runtime.h>

#include <cstdint>

namespace cavs_b200 {

int LaunchGruGateR(float* R, void* M, bool bf16, const void* A, const void* PR, const float* bias, const float* state,
                   const int32_t* child, const int32_t* a_row, int n_total, int off, int rows, int H, int K, cudaStream_t st);
int LaunchGruOut(float* state, float* ZN, bool bf16, const void* A, const void* PZ, const void* PN, const float* bias,
                 const int32_t* child, const int32_t* a_row, int n_total, int off, int rows, int H, int K, bool leaf,
                 cudaStream_t st);
int LaunchGruBwdA(void* dA, float* dHt, bool bf16, const float* mailbox, const float* dOut, const float* ZN, const float* state,
                  const int32_t* child, const int32_t* parent, int n_total, int off, int rows, int H, int K, bool leaf,
                  cudaStream_t st);
int LaunchGruBwdB1(void* dA, void* ZR, bool bf16, const float* dm, const float* R, const float* state, const int32_t* child,
                   int n_total, int off, int rows, int H, int K, cudaStream_t st);
int LaunchGruBwdB2(float* mailbox, const float* dHt, const float* dsz, const float* dm, const float* dqr, const float* R,
                   const int32_t* child, int n_total, int off, int rows, int H, int K, cudaStream_t st);

}  // namespace cavs_b200
#endif
