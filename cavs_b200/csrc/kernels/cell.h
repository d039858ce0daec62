// Internal launchers of the fused Tree-LSTM cell kernels (kernels/cell.cu) and of the
// other per-step kernels (embedding, loss head, reductions, optimizers).
#ifndef CAVS_B200_KERNELS_CELL_H_
#define CAVS_B200_KERNELS_CELL_H_

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace cavs_b200 {

// child: [K, n_total] tensor-id of each child slot or -1; parent: [n_total] or -1.
// Level rows are [off, off + rows).  S is [n_total, H], HK / ZF are [n_total, K, H],
// P is [rows, 3H] and Q / dq are [rows, K, H] (level-local), A / dA are [n_total, 4H].
// state_pitch: floats per state row (h first); 0 = 2H (the Tree-LSTM's h|c rows).
int LaunchGatherChildH(void* S, void* HK, bool bf16, const float* state, const int32_t* child, int n_total, int off,
                       int rows, int H, int K, cudaStream_t st, int state_pitch = 0);
// A, P, Q are fp32, or bf16 when preact_bf16 is set.
// gates: fp32, or fp16 when preact_bf16 / bf16 is set (the bf16-GEMM configurations).
// a_row (optional): [n_total] row of A for each vertex (A then holds one row per distinct token).
int LaunchCellFwd(float* state, void* gates, const void* A, const void* P, const void* Q, bool preact_bf16, const float* bias,
                  const int32_t* child, const int32_t* a_row, int n_total, int off, int rows, int H, int K, bool leaf, cudaStream_t st,
                  bool store_leaf_gates = true, int tok_base = -1, void* gates_f = nullptr, int* status = nullptr);
// gates_f (here and in LaunchCellBwd): NULL = the saved gates are one array [n_total, (3+K)H] (i|o|u|f_0..f_{K-1});
// else `gates` is [n_total, 3H] (i|o|u) and gates_f [n_total, K, H] holds the forget gates -- the layout the gate
// products write when their epilogue finishes the gates (bf16 mode).
// The rest of the forward cell on finished gates: c = i o u + sum_c f_c o c_c, h = o o tanh(c) (fp16 gates).
int LaunchCellFwdGated(float* state, const void* gates3, const void* gates_f, const int32_t* child, int n_total, int off, int rows,
                       int H, int K, cudaStream_t st);
// tok_base >= 0 (internal level whose children are all leaves with per-token states): `child` holds state rows
// tok_base + token row, P is [tokens, 4H] = h_tok.U_iou | h_tok.U_f, Q is unused; the level's own P / Q are never formed.
// store_leaf_gates = false (leaf levels): the gates are not saved; the backward pass must then be given A, a_row and
// bias and recomputes them (a leaf's gates depend on its input-projection row only).
// dB_part (optional): [CellBwdMaxGrid(), 4H] fp32, zeroed by the caller before the first level of a
// backward sweep; every launch adds its per-CTA column sums of (zi, zo, zu, sum zf) into it, and a
// final column sum over its rows gives the bias gradient.  Needs CellBwdFusesBias(H).
constexpr int kHeadDzPitch = 8;
int CellBwdMaxGrid();
bool CellBwdFusesBias(int H);
int LaunchCellBwd(void* dA, void* ZF, bool bf16, float* mailbox, float* dB_part, const float* dOut, const void* gates,
                  const float* state, const int32_t* child, const int32_t* parent, int n_total, int off, int rows, int H,
                  int K, bool leaf, cudaStream_t st, const float* dz = nullptr, const float* Wc = nullptr, int C = 0,
                  const void* A = nullptr, const int32_t* a_row = nullptr, const float* bias = nullptr,
                  const int32_t* child_state = nullptr, const void* gates_f = nullptr, int* status = nullptr);
// child_state (optional, [K, n_total]): rows of `state` holding the children's cell state when they differ from
// the children's tensor ids (leaf states shared per token); the mailbox is always addressed by `child`.
// status (optional): device word raised when a bounded wait of the streaming form expires.
// A / a_row / bias (optional, leaf levels only): recompute i, o, u and c from the input-projection rows instead of
// reading the saved gates and cell state (A in the same precision as dA).
// dz / Wc / C (optional): rebuild d(pushed h) = dz[t,:] . Wc inside the kernel instead of reading dOut
// (dz: [n_total, kHeadDzPitch] rows from LaunchLossHead's dz_out; Wc: [C, H], C <= 8); dOut may then be NULL.
// First pass of the per-token sums of dA with the leaf level's backward cell folded in (kernels/cell.cu,
// TokenGradChunks): chunk_out / chunk_seg [n_chunks] give a single-chunk token's output row (else -1) and every
// chunk's token row; leaves are the rows below n_leaf (every scheduled leaf has a parent, so its mailbox row is
// valid) and are recomputed from A, bias, the mailbox and dz (or dOut); internal rows are read from dA.  partial: [n_chunks, 4H] fp32, always written; out: [tokens, 4H].
// The second pass over multi-chunk tokens is LaunchSegmentedRowSumFinal.
int LaunchTokenGradChunks(float* partial, void* out, bool bf16, const int32_t* chunk_out, const void* dA, const void* A,
                          const int32_t* order, const int32_t* chunk_off, const int32_t* chunk_seg, int n_chunks,
                          const float* mailbox, const float* dOut, const float* dz, const float* Wc, int C, const float* bias,
                          int n_leaf, int H, cudaStream_t st, const float* ptok = nullptr, const int32_t* label = nullptr,
                          float inv_rows = 0.0f, const float* dh_tok = nullptr, const int32_t* seg_first_chunk = nullptr);
// An entry of `order` with this bit set is a leaf whose mailbox row holds no d(h) (its parent's level hands d(h) down
// per token): only the c half of the row is read.  dh_tok [tokens, H] (optional) is that per-token d(h), added once per
// token by the chunk seg_first_chunk[token row].
constexpr int32_t kOrderNoDh = 1 << 30;
// Per-token sums over parent-child links of a level whose children are all leaves: link t * K + c contributes
// [ dA[t, 0:3H] | ZF[t * K + c, :] ]; chunks of <= 256 links of one child token; a single-chunk token's sum goes straight
// to out[chunk_out[chunk], 4H], the other chunks write partial [chunk, 4H] fp32 for LaunchSegmentedRowSumFinal.
int LaunchLinkSumChunks(float* partial, void* out, bool bf16, const int32_t* chunk_out, const void* dA, const void* ZF,
                        const int32_t* order, const int32_t* chunk_off, int n_chunks, int H, int K, cudaStream_t st);
// ptok / label / inv_rows (optional, instead of dz): a leaf's d(logits) is (ptok[token] - onehot(label)) * inv_rows.
// loss[t] = -log ptok[tok_slot[t]][label[t]] for the leaves t < n_leaf (0 without a label): fills in what the loss
// head's token rows do not write.
int LaunchLeafLossFill(float* loss, const float* ptok, const int32_t* tok_slot, const int32_t* label, int n_leaf, int C,
                       cudaStream_t st);
int LaunchSegmentedRowSumFinal(void* out, bool out_bf16, const float* partial, const int32_t* seg_first_chunk,
                               const int32_t* multi_seg, int n_multi, int width, cudaStream_t st);
int LaunchScatterChildGrad(float* mailbox, const float* ds, const float* dq, const int32_t* child, int n_total, int off,
                           int rows, int H, int K, cudaStream_t st);

// Embedding lookup out[t,:] = table[tok[t],:] (fp32 table; fp32 or bf16 output).
int LaunchEmbedFwd(void* out, bool bf16, const float* table, const int32_t* tok, int rows, int E, int vocab, cudaStream_t st);
// Deterministic segmented embedding gradient.  order: row indices sorted by token (stable);
// seg_off: [n_seg+1] offsets into order; seg_tok: [n_seg] token of each segment.  Long
// segments are split into chunks of kEmbedChunk rows whose partial sums go to scratch
// ([n_chunks, E] fp32) before a fixed-order second pass.
constexpr int kEmbedChunk = 256;
int LaunchEmbedBwd(float* dtable, const float* dX, const int32_t* order, const int32_t* chunk_seg, const int32_t* chunk_off,
                   int n_chunks, const int32_t* seg_first_chunk, const int32_t* seg_tok, int n_seg, float* scratch, int E,
                   cudaStream_t st);

// out[s,:] = sum over the rows of segment s of x[row,:] (rows listed in `order`, cut into chunks as for
// LaunchEmbedBwd); fp32 accumulation in a fixed order; scratch: [n_chunks, width] fp32.
int LaunchSegmentedRowSum(void* out, bool out_bf16, const void* x, bool in_bf16, long long pitch, int width, const int32_t* order,
                          const int32_t* chunk_off, int n_chunks, const int32_t* seg_first_chunk, int n_seg, float* scratch,
                          cudaStream_t st, const int32_t* chunk_out = nullptr, const int32_t* multi_seg = nullptr,
                          int n_multi = 0);
// chunk_out (optional, [n_chunks]): segment index for a chunk that is its segment's only chunk, else -1; such
// chunks write their output row in the first pass.  multi_seg (optional with chunk_out, [n_multi]): the segments
// with more than one chunk; the second pass then runs only over them, several CTAs per segment.

// Fused classifier + softmax cross-entropy for small class counts (C <= 32), forward and backward
// in one pass over the pushed hidden rows.  h rows are read with pitch h_pitch (state is [n,2H]).
// Writes loss[t], dOut[t,:] = dz Wc; per-CTA partials of dWc / dbc / loss sum go to scratch and are
// reduced in fixed order.  inv_rows scales dz (the reference divides by the logits' row count).
size_t LossHeadScratchBytes(int H, int C);
// Token rows of the loss head (streaming form): loss rows at and above rows_v each stand for all leaves that carry one
// token (they share a hidden row).  hist [tokens, 8] (int32): how many of the token's leaves have each label; ptok
// [tokens, 8] receives the token's class probabilities, from which each leaf's own d(logits) and loss follow.  No
// loss / dz row is written for a token row; its d(logits) = (count * p - hist) / rows feeds dWc, dbc and the loss sum.
struct LossTokenRows {
  const int32_t* hist = nullptr;
  float* ptok = nullptr;
  int rows_v = 0;
};
int LaunchLossHead(float* loss, float* loss_sum, float* dOut, float* dWc, float* dbc, const float* h, long long h_pitch,
                   const int32_t* label, const float* Wc, const float* bc, int rows, int H, int C, float inv_rows,
                   float* scratch, cudaStream_t st, bool accumulate = false,    // accumulate: add into dWc / dbc / loss_sum
                   float* dz_out = nullptr, int* status = nullptr, const int32_t* row_index = nullptr,
                   LossTokenRows token_rows = LossTokenRows());
// row_index (optional, [rows]): loss row t reads its hidden row at h[row_index[t]] (streaming form only).
bool LossHeadStreams(const float* h, long long h_pitch, int H);   // would this shape take the streaming form?
// status (optional, device): raised to 1 if a bounded wait on an asynchronous row copy expires.
// dz_out (optional, [rows, 8]): d(logits) rows zero-padded to 8 floats.  With dz_out set, dOut may be NULL:
// the cell-gradient kernel then rebuilds d(hidden) = dz Wc on the fly (LaunchCellBwd's head arguments)
// instead of reading it back from memory.

// Softmax cross-entropy over wide rows: z [rows, C] (pitch ldz) holds logits WITHOUT bias on entry
// (bias, optional, is added here) and dz = (softmax - onehot) * inv_rows on exit; dz_bf16 (optional,
// same pitch) receives a bf16 copy for the gradient GEMMs; loss[r] = -log softmax(z_r)[label_r].
int LaunchSoftmaxXentRows(float* loss, float* z, void* dz_bf16, long long ldz, const float* bias, const int32_t* label, int rows,
                          int C, float inv_rows, cudaStream_t st);

// Column sums of a [rows, cols] matrix (fp32 or bf16) into out[perm(col)], deterministic two-stage.
size_t ColumnSumScratchBytes(int cols);
// block > 0 (cols == 4*block): source column block b is written to destination block m_b.
int LaunchColumnSum(float* out, const void* x, bool bf16, long long pitch, int rows, int cols, float* scratch, cudaStream_t st,
                    int block = 0, int m0 = 0, int m1 = 1, int m2 = 2, int m3 = 3);

int LaunchSgd(float* w, const float* g, size_t n, float lr, cudaStream_t st);
int LaunchAdagrad(float* w, float* acc, const float* g, size_t n, float lr, float eps, cudaStream_t st);
// w[rows[i], :width] takes gradient row g[i, :width]: SGD, or Adagrad when acc (same shape as w) is given.
int LaunchUpdateRows(float* w, float* acc, const float* g, const int32_t* rows, int n_rows, int width, float lr, float eps,
                     cudaStream_t st);
// dst_bf16[i] = bf16(src[i])
int LaunchCastBf16(void* dst, const float* src, size_t n, cudaStream_t st);
// dst [rows, cols] (dense, bf16) = src [rows, cols] with row pitch src_pitch (fp32)
int LaunchCastRowsBf16(void* dst, const float* src, long long rows, int cols, long long src_pitch, cudaStream_t st);

}  // namespace cavs_b200
#endif
