/*
 * cavs_b200 -- C ABI of the B200-native level-batched vertex-function path.
 *
 * Plain C: pointers, sizes and int status returns; no C++ or torch types.  Every
 * device pointer is a CUDA device address owned by the caller; every `stream`
 * argument is a cudaStream_t passed as void* (NULL = the legacy default stream).
 * Unless a function says otherwise it allocates nothing and only enqueues work on
 * `stream`.  Functions return CAVS_OK or an error code; cavs_last_error() gives
 * the message of the calling thread's most recent failure.
 *
 * Citations name the file:line of the reference (zhisbug/Cavs) interface that an
 * entry point replaces.
 */
#ifndef CAVS_B200_H_
#define CAVS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Exported symbol marker: the library is built with hidden default visibility. */
#define CAVS_API __attribute__((visibility("default")))

enum cavs_status {
  CAVS_OK = 0,
  CAVS_ERR_BAD_ARG = 1,     /* null pointer, negative size, unsupported shape            */
  CAVS_ERR_BAD_GRAPH = 2,   /* malformed parent array (no terminator, range, fan-in, cycle) */
  CAVS_ERR_CAPACITY = 3,    /* caller-provided buffer too small                          */
  CAVS_ERR_TIMEOUT = 4,     /* a bounded device-side wait expired                         */
  CAVS_ERR_CUDA = 5,        /* a CUDA runtime / driver call failed                        */
  CAVS_ERR_UNSUPPORTED = 6  /* valid request this build does not implement                */
};

CAVS_API const char* cavs_status_string(int status);
CAVS_API const char* cavs_last_error(void);
/* Library version and the GPU architecture the kernels were compiled for ("sm_100a"). */
CAVS_API const char* cavs_build_info(void);
/* Kernels this library has launched in this process so far (every launch is counted). */
CAVS_API unsigned long long cavs_launch_count(void);

/* ------------------------------------------------------------------------ */
/* Level scheduler (host only; no CUDA call)                                 */
/* Replaces GraphSchedulerBase::LoadGraph + BatchGraphScheduler::Initialize /  */
/* ActivateNext / ReverseGraph, cavs/midend/graph_scheduler.cc:12-81,169-258.  */
/* ------------------------------------------------------------------------ */
typedef struct cavs_sched cavs_sched;

CAVS_API int cavs_sched_create(cavs_sched** out);
CAVS_API void cavs_sched_destroy(cavs_sched* s);
/* parents: host int32 [batch, max_len]; entry j of a sample is the local index of
 * vertex j's parent, the root holds -1 and is the sample's last vertex; trailing
 * slots are ignored.  n_slots = child slots per vertex (the reference has 2; 1..4
 * accepted).  Builds every level of the batch in one pass. */
CAVS_API int cavs_sched_load(cavs_sched* s, const int32_t* parents, int batch, int max_len, int n_slots);
/* n_total: vertices in the batch (LoadGraph's return value); n_scheduled: vertices
 * that execute (single-vertex samples never do, graph_scheduler.cc:180). */
CAVS_API int cavs_sched_counts(const cavs_sched* s, int* n_total, int* n_scheduled, int* n_levels, int* max_level_rows);
/* level_off: [n_levels+1] first tensor id of each level (round2offset_, graph_scheduler.cc:203-204). */
CAVS_API int cavs_sched_level_offsets(const cavs_sched* s, int32_t* level_off, int capacity);
/* t2j: tensor id -> job id (TensorIdsToJobIds(), graph_scheduler.h:51); j2t: inverse, -1 if never scheduled. */
CAVS_API int cavs_sched_maps(const cavs_sched* s, int32_t* t2j, int32_t* j2t, int capacity);
/* Per-row index tables in tensor-id space, each [n_total] or [n_slots*n_total] slot-major:
 *   fg[c][t] forward Gather(Child=c) source row in the mailbox, -1 = zero row
 *   fs[t]    forward Scatter target row, -1 = none (roots)
 *   bg[t]    backward Gather source row, -1 = zero row (roots)
 *   bs[c][t] backward Scatter(Child=c) target row, -1 = none
 * mode 0 = aligned; mode 1 = ref_compat: the reference's positional pairing of its compact
 * per-round lists with level rows (op_impl_graphop.cu:62-76,144-157), which shifts rows on
 * levels that mix vertices with and without a given child slot / parent. */
CAVS_API int cavs_sched_tables(const cavs_sched* s, int mode, int32_t* fg, int32_t* fs, int32_t* bg, int32_t* bs, int capacity);
/* The reference's own per-round lists, as CurrentRoundTensorIdsForGather/Scatter would
 * return them in forward round `level` (graph_scheduler.h:44-49).  Returns the count in *n. */
CAVS_API int cavs_sched_ref_gather(const cavs_sched* s, int level, int slot, int32_t* ids, int capacity, int* n);
CAVS_API int cavs_sched_ref_scatter(const cavs_sched* s, int level, int32_t* ids, int capacity, int* n);
/* Whole forward + backward schedule serialised as one int32 stream (layout documented in
 * oracle/refsched_driver.cc); *n receives the length, CAVS_ERR_CAPACITY if it does not fit. */
CAVS_API int cavs_sched_ref_stream(const cavs_sched* s, int32_t* out, int capacity, int* n);

/* Round order of the NEXT cavs_sched_load: 0 = one round per level of the batch (default), 1 = one
 * vertex per round, sample after sample -- the execution order of SerialGraphScheduler
 * (graph_scheduler.cc:83-167), i.e. the reference's Session without OPT_BATCHING
 * (cavs/proto/opt.proto:3-8).  Tensor ids follow execution order in both modes, every "level" then
 * holds one row, and single-vertex samples are skipped (never truncating the sweep).  The engines run
 * such a schedule unchanged; it exists to measure what batching buys. */
CAVS_API int cavs_sched_set_order(cavs_sched* s, int order);
/* Job-id-space adjacency of the loaded batch: parent_job[g] or -1; child_job[c*capacity + g] = the
 * slot-c child or -1 (children_ / parents_, graph_scheduler.cc:44-59).  Either pointer may be null. */
CAVS_API int cavs_sched_adjacency(const cavs_sched* s, int32_t* parent_job, int32_t* child_job, int capacity);
/* The reference's SerialGraphScheduler itself, where tensor id == job id: jobs[r] is the vertex of
 * round r of the forward (backward = 0) or backward sweep and init[r] (optional) the single entry of
 * CurrentRoundTensorIdsForGatherInitialization() in that round, -1 for none.  A round's gather /
 * scatter lists follow from the adjacency: forward gather(c) = the slot-c child, scatter(0) = the
 * vertex itself if it has a parent; backward the reverse.  The sweep reproduces the reference's
 * work-list order, including its early end at a single-vertex sample. */
CAVS_API int cavs_sched_serial_rounds(const cavs_sched* s, int backward, int32_t* jobs, int32_t* init, int capacity, int* n);
/* Both serial sweeps serialised as one int32 stream (layout documented in oracle/refsched_driver.cc). */
CAVS_API int cavs_sched_ref_serial_stream(const cavs_sched* s, int32_t* out, int capacity, int* n);

/* ------------------------------------------------------------------------ */
/* Row movement behind the graph ops (device).  HBM-bound, 128-bit accesses. */
/* ------------------------------------------------------------------------ */
/* out[b,:] = inp[ids[b],:] for b < n_ids.  Replaces BatchedDynamicSelectedInputSliceCopyKernel
 * as launched by GraphGatherOp / GraphPullOp (functor_batched_memcpy.cuh:34-47,
 * op_impl_graphop.cu:62-76,243-249).  ids is a DEVICE array (the reference re-uploads a host
 * vector before every launch).  Extension: ids[b] < 0 writes a zero row.  row_bytes must be a
 * multiple of 4; rows that are multiples of 16 bytes in 16-byte aligned buffers take the
 * 128-bit path. */
CAVS_API int cavs_gather_rows(void* out, const void* inp, const int32_t* ids, int n_ids, size_t row_bytes, void* stream);
/* out[ids[b],:] = inp[b,:] for b < n_ids.  Replaces BatchedDynamicSelectedOutputSliceCopyKernel
 * as launched by GraphScatterOp / FunctionPopRetOp (functor_batched_memcpy.cuh:49-62,
 * op_impl_graphop.cu:144-157,304-318).  Extension: ids[b] < 0 skips the row.  Target rows must
 * be distinct (they are: one mailbox row per vertex). */
CAVS_API int cavs_scatter_rows(void* out, const int32_t* ids, const void* inp, int n_ids, size_t row_bytes, void* stream);
/* The strided form behind vertex functions that are executed op by op (Slice / Concat views of wider rows,
 * cavs/backend/op_impl_slice_join.cu:35-149): for b < rows, dst[dst_ids[b], :width] (+)= src[src_ids[b], :width], fp32,
 * pitches in floats; a NULL index list means row b itself, a negative source row reads zeros, a negative target row is
 * skipped.  Target rows must be distinct. */
CAVS_API int cavs_copy_rows_2d(float* dst, long long dst_pitch, const int32_t* dst_ids, const float* src, long long src_pitch,
                               const int32_t* src_ids, int rows, int width, int accumulate, void* stream);
/* out[b,:] = 0 for b < n_rows.  Replaces BatchedDynamicSelectedAssignZeroKernel, which ignores
 * the id values it is given and clears the first n rows (functor_batched_memcpy.cuh:64-75,
 * op_impl_graphop.cu:77-86). */
CAVS_API int cavs_zero_rows(void* out, int n_rows, size_t row_bytes, void* stream);

/* ------------------------------------------------------------------------ */
/* Dense contractions (device).                                              */
/* ------------------------------------------------------------------------ */
/* bf16 x bf16 -> fp32-accumulate GEMM on the tcgen05 tensor cores (TMA-fed, TMEM accumulator).
 * Replaces the cublasSgemm calls behind MatMul (cavs/backend/cublas_wrapper.cc:13-28,
 * cavs/backend/op_impl_blas3_cublas.cc:35-70) for the bf16 configurations.
 *   a_major 0: A is [m,k] row-major (pitch lda);  1: A is [k,m] row-major (used transposed)
 *   b_major 0: B is [n,k] row-major (pitch ldb);  1: B is [k,n] row-major
 *   out_mode 0: C (fp32) = A.B   1: C (fp32) += A.B   2: C (bf16) = A.B;  C is [m,n], pitch ldc.
 * a and b need 16-byte aligned bases and pitches that are multiples of 8 elements.
 * splits > 1 cuts K across CTAs: partials go to `scratch` (cavs_gemm_bf16_scratch_bytes) and are
 * reduced in a fixed order.  status: optional device int raised if a bounded wait inside the
 * kernel expires. */
CAVS_API int cavs_gemm_bf16(void* c, long long ldc, int out_mode, const void* a, long long lda, int a_major,
                            const void* b, long long ldb, int b_major, int m, int n, int k, int splits, void* scratch,
                            size_t scratch_bytes, int* status, void* stream);
CAVS_API size_t cavs_gemm_bf16_scratch_bytes(int m, int n, int splits);
/* Self-test of the kernel's bounded waits.  Launches the same kernel as cavs_gemm_bf16 (A [m,k] and B [k,n]
 * row-major, C fp32) with its operand loads withheld and a poll limit of a few milliseconds, so that every wait
 * inside it runs out: the kernel must raise *status, free its tensor memory and return without writing C, and the
 * context must stay usable.  For tests of the error path (CAVS_ERR_TIMEOUT); no counterpart in the reference, whose
 * kernels never wait on one another. */
CAVS_API int cavs_gemm_bf16_wait_selftest(void* c, long long ldc, const void* a, long long lda, const void* b, long long ldb,
                                          int m, int n, int k, int* status, void* stream);
/* fp32 GEMM on the CUDA cores with element strides (any transpose without a copy):
 * C[i,j] (+)= sum_p A[i*a_row_stride + p*a_col_stride] * B[p*b_row_stride + j*b_col_stride].
 * The fp32 configurations use it to stay within 1e-5 of the reference's cublasSgemm. */
CAVS_API int cavs_gemm_f32(float* c, long long ldc, int accumulate, const float* a, long long a_row_stride,
                           long long a_col_stride, const float* b, long long b_row_stride, long long b_col_stride, int m,
                           int n, int k, void* stream);

/* ------------------------------------------------------------------------ */
/* Fused vertex-function kernels (device).  Level rows are [off, off+rows) of */
/* arenas in tensor-id order; child is [n_slots, n_total], parent [n_total].  */
/* ------------------------------------------------------------------------ */
/* S[t] = sum_c h(child_c(t)), HK[t,c] = h(child_c(t)) for the level's rows, fp32 or bf16 output:
 * Gather(Child=c) + Slice + Add of the vertex function (apps/paper/tree-lstm-cavs.cc:131-136,
 * cavs/backend/op_impl_graphop.cu:32-90).  state is [n_total, 2*hidden] (h|c). */
CAVS_API int cavs_gather_child_h(void* S, void* HK, int bf16, const float* state, const int32_t* child, int n_total,
                                 int off, int rows, int hidden, int n_slots, void* stream);
/* Fused child-sum Tree-LSTM cell forward (apps/paper/tree-lstm-cavs.cc:159-171; stands in for the
 * NVRTC-fused elementwise groups, cavs/backend/op_impl_fused_kernel.cu:62-64, plus the forward
 * Scatter and Push, cavs/backend/op_impl_graphop.cu:108-202).  A [n_total,4H] = x.W (i,o,u,f),
 * P [rows,3H] = (sum h).U_iou, Q [rows,n_slots,H] = h_c.U_f, bias [4H] (i,f,u,o).  Writes
 * gates [n_total,(3+n_slots)H] and state [n_total,2H].  leaf != 0: no children (P, Q unused, the
 * forget gates are neither computed nor stored).  preact_bf16 != 0: A, P, Q hold bf16 (the GEMM
 * epilogue's rounded output) and gates are stored as fp16; else both are fp32.  a_row (optional,
 * [n_total]): row of A to use for each vertex -- x.W depends on a vertex only through its token, so A may
 * hold one row per distinct token; NULL: one row per vertex. */
CAVS_API int cavs_treelstm_cell_fwd(float* state, void* gates, const void* A, const void* P, const void* Q, int preact_bf16,
                                    const float* bias, const int32_t* child, const int32_t* a_row, int n_total, int off, int rows,
                                    int hidden, int n_slots, int leaf, void* stream);
/* Fused gate-gradient backward of the cell: reads d(pushed h) dOut [n_total,H], the parent's
 * d(h|c) from mailbox [n_total,2H] (zeros for roots), saved gates and states; writes
 * dA [n_total,4H] (zi|zo|zu|sum zf), ZF [n_total,n_slots,H] (fp32, or bf16 with fp16 gates when bf16 != 0)
 * and d(c_child) into the
 * children's mailbox rows (Scatter(Child=c), cavs/backend/op_decl_graphop.cc:25-41). */
CAVS_API int cavs_treelstm_cell_bwd(void* dA, void* ZF, int bf16, float* mailbox, const float* dOut, const void* gates,
                                    const float* state, const int32_t* child, const int32_t* parent, int n_total, int off,
                                    int rows, int hidden, int n_slots, int leaf, void* stream);
/* The fused cell in operator form, for hosts that keep the reference's op-by-op dataflow inside Node(): every
 * input is a dense level-local tensor (fp32, like all of the reference's ops).  Forward: A [rows,4H] = x.W
 * (i,o,u,f), P [rows,3H] = (sum h).U_iou, Q[c] [rows,H] = h_c.U_f, child_hc[c] [rows,2H] = Gather(Child=c) (h|c);
 * a NULL entry of Q / child_hc stands for a slot without children in this level (zeros, as the zero-filled Gather
 * gives, op_impl_graphop.cu:77-86).  Writes hc [rows,2H] (what Scatter takes) and gates [rows,(3+n_slots)H].
 * One launch instead of the elementwise / slice / concat ops of apps/paper/tree-lstm-cavs.cc:150-171.
 * Backward: d_hc [rows,2H] = the gradient the parents left (NULL for a level of roots), dOut [rows,H] = the pushed
 * h's gradient (NULL if none); writes dA [rows,4H] (zi|zo|zu|sum zf: the gradients of A; its first 3H columns are
 * the gradient of P), ZF[c] [rows,H] (gradient of Q[c]) and d_child_c[c] [rows,H] (the c half of what is scattered
 * to child c; the h half is the sum of the MatMul gradients of P and Q[c]).  NULL entries are not written. */
CAVS_API int cavs_treelstm_cell_dense_fwd(float* hc, float* gates, const float* A, const float* P, const float* const* Q,
                                          const float* const* child_hc, const float* bias, int rows, int hidden, int n_slots,
                                          void* stream);
CAVS_API int cavs_treelstm_cell_dense_bwd(float* dA, float* const* ZF, float* const* d_child_c, const float* d_hc,
                                          const float* dOut, const float* gates, const float* hc, const float* const* child_hc,
                                          int rows, int hidden, int n_slots, void* stream);
/* mailbox[child_c(t)].h = ds[b] + dq[b,c]: the child-state gradient scatter. */
CAVS_API int cavs_scatter_child_grad(float* mailbox, const float* ds, const float* dq, const int32_t* child, int n_total,
                                     int off, int rows, int hidden, int n_slots, void* stream);

/* ------------------------------------------------------------------------ */
/* Around the vertex function (device).                                      */
/* ------------------------------------------------------------------------ */
/* out[t,:] = table[tok[t],:], fp32 or bf16 output.  Replaces BatchedCopy
 * (cavs/backend/op_impl_embedding_lookup.cu:23-35); ids are int32, out-of-range ids read row 0. */
CAVS_API int cavs_embed_fwd(void* out, int bf16, const float* table, const int32_t* tok, int rows, int embed, int vocab,
                            void* stream);
/* Deterministic segmented embedding gradient; replaces BatchedSparseUpdate's atomicAdd
 * (cavs/backend/op_impl_embedding_lookup.cu:91-103).  order: row indices grouped by token;
 * chunk_off [n_chunks+1]: ranges of `order`, at most 256 rows each, never spanning two tokens;
 * seg_first_chunk [n_seg+1]: first chunk of each token group; seg_tok [n_seg]: its token;
 * scratch: [n_chunks, embed] fp32.  Rows of dtable for absent tokens are left untouched. */
CAVS_API int cavs_embed_bwd_segmented(float* dtable, const float* dX, const int32_t* order, const int32_t* chunk_off,
                                      int n_chunks, const int32_t* seg_first_chunk, const int32_t* seg_tok, int n_seg,
                                      float* scratch, int embed, void* stream);
/* Classifier + softmax cross-entropy, forward and backward in one pass (classes <= 8).  Replaces
 * FullyConnected + SoftmaxEntropyLoss and their gradients
 * (cavs/backend/op_impl_fullyconnected_cublas.cc:33-85,104-176,
 * cavs/backend/op_impl_softmax_entropy_logits_loss.cu:106-140,213-250): loss[t] = -log softmax(h Wc^T + bc)[label],
 * dz = (softmax - onehot) * inv_rows (the reference divides by the row count and ignores the
 * upstream gradient), dH = dz Wc, dWc = dz^T h, dbc = sum dz, *loss_sum = sum loss.  label < 0 marks a
 * row without a loss term.  h has row pitch h_pitch.  Scratch holds per-CTA partials reduced in order. */
CAVS_API size_t cavs_fc_softmax_xent_scratch_bytes(int hidden, int classes);
CAVS_API int cavs_fc_softmax_xent(float* loss, float* loss_sum, float* dH, float* dWc, float* dbc, const float* h,
                                  long long h_pitch, const int32_t* label, const float* Wc, const float* bc, int rows,
                                  int hidden, int classes, float inv_rows, float* scratch, void* stream);
/* The same loss head for callers that cannot allocate device memory -- for example a host program
 * that gave the whole GPU to its own memory pool at start-up, or a running step loop in which
 * cudaMalloc / cudaFree are forbidden because they stall the device.  It takes no scratch argument:
 * the per-CTA partial records live in a fixed array inside the library (about 12 MB per GPU, held
 * by every GPU that loads the library until the process exits), and the call uses no allocating
 * routine.  This entry point has no counterpart in the reference.
 *   Limit: classes*hidden + classes + 1 <= 10240 floats per record (e.g. 5 x 1024, 8 x 1024);
 *   larger shapes return CAVS_ERR_CAPACITY -- use cavs_fc_softmax_xent with your own scratch.
 *   Sharing: every call on a device uses the same array.  Calls that can overlap on the GPU
 *   (different streams or threads) race; keep them on one stream or order them yourself.  Nothing
 *   in the array needs to start at zero: each launch rewrites every record it later reads.
 *   First call: the first call on each device looks up the array's device address (with that device
 *   current) and caches it; make that call before you begin any stream capture. */
CAVS_API int cavs_fc_softmax_xent_static(float* loss, float* loss_sum, float* dH, float* dWc, float* dbc, const float* h,
                                         long long h_pitch, const int32_t* label, const float* Wc, const float* bc, int rows,
                                         int hidden, int classes, float inv_rows, void* stream);
/* out[j] = sum_r x[r,j] (fp32 or bf16 input), two-stage fixed-order reduction.  Replaces the
 * per-thread serial column loop used for bias gradients (cavs/backend/op_impl_elementwise.cuh:31-37). */
CAVS_API size_t cavs_column_sum_scratch_bytes(int cols);
CAVS_API int cavs_column_sum(float* out, const void* x, int bf16, long long pitch, int rows, int cols, float* scratch,
                             void* stream);
/* w <- w - lr*g.  Replaces SGDKernel (cavs/backend/op_impl_sgd.cu:15-47). */
CAVS_API int cavs_sgd(float* w, const float* g, size_t count, float lr, void* stream);
/* acc += g^2; w <- w - lr*g/(sqrt(acc)+eps).  No counterpart in the reference (it registers only SGD). */
CAVS_API int cavs_adagrad(float* w, float* acc, const float* g, size_t count, float lr, float eps, void* stream);
/* *out = sum |x[i]|: what the reference's Reduce_sum computes (cublasSasum, cavs/backend/op_impl_blas1_cublas.cc:48-77).
 * Fixed reduction order; scratch: 1024 floats. */
CAVS_API int cavs_abs_sum(float* out, const float* x, size_t count, float* scratch, void* stream);
/* x[i] = value (the gradient seed ConstOp / Fill, cavs/midend/graph_util.cc:106-112, cavs/backend/op_decl_reduction.cc:19-28). */
CAVS_API int cavs_fill(float* x, size_t count, float value, void* stream);
/* y += alpha * x. */
CAVS_API int cavs_axpy(float* y, const float* x, size_t count, float alpha, void* stream);
/* Gradient clipping as Sym::Optimizer(vars, lr, clip) asks for it (cavs/backend/op_impl_clip.cu:25-45,
 * cavs/midend/graph_util.cc:209-225): s = the SUM of the L2 norms of the gradient blocks (one block per variable;
 * block_offsets is a HOST array of n_blocks + 1 offsets into g), then g *= clip / max(s, clip).  The reference takes the
 * norms with a host-synchronous cublasSnrm2; here nothing leaves the device.  scratch: cavs_clip_gradients_scratch_bytes. */
CAVS_API size_t cavs_clip_gradients_scratch_bytes(int n_blocks);
CAVS_API int cavs_clip_gradients(float* g, const unsigned long long* block_offsets, int n_blocks, float clip, float* scratch,
                                 void* stream);
/* dst (bf16) = src (fp32): shadow copies of the GEMM weights after an update. */
CAVS_API int cavs_cast_bf16(void* dst, const float* src, size_t count, void* stream);

/* ------------------------------------------------------------------------ */
/* Data-parallel training: one process per GPU, gradients summed with NCCL.   */
/* Replaces MPIAllReduce through host memory                                  */
/* (cavs/backend/op_impl_mpi.cc:29-49, inserted per variable gradient by       */
/* MPISession, cavs/midend/session_mpi.cc:31-80) and the start-up broadcast of */
/* the variables from rank 0 (cavs/backend/op_impl_variable.h:151-159).        */
/* ------------------------------------------------------------------------ */
typedef struct cavs_comm cavs_comm;
/* Rank 0 makes a 128-byte id and hands it to every rank by whatever channel the host program has (the reference
 * uses MPI; a PyTorch host its process-group store); every rank then creates its communicator with the device it
 * will compute on current.  NCCL is bound on first use; CAVS_ERR_UNSUPPORTED if it cannot be loaded. */
CAVS_API int cavs_comm_unique_id(void* id, size_t bytes);
CAVS_API int cavs_comm_create(const void* id, size_t bytes, int rank, int world, cavs_comm** out);
CAVS_API void cavs_comm_destroy(cavs_comm* comm);
CAVS_API int cavs_comm_info(const cavs_comm* comm, int* rank, int* world, int* nccl_version);
/* buf (fp32, device) <- sum over ranks, in place, on `stream`; a no-op for a world of one. */
CAVS_API int cavs_allreduce(float* buf, size_t count, cavs_comm* comm, void* stream);
/* buf <- rank `root`'s buf (parameters at start-up). */
CAVS_API int cavs_broadcast(void* buf, size_t bytes, int root, cavs_comm* comm, void* stream);
/* recv [world, bytes_per_rank] <- every rank's send [bytes_per_rank]. */
CAVS_API int cavs_allgather(const void* send, void* recv, size_t bytes_per_rank, cavs_comm* comm, void* stream);

/* ------------------------------------------------------------------------ */
/* Tree-LSTM engine: the level loop, forward and backward.                   */
/* Replaces GraphStatement::Run / GraphGradStatement::Run                    */
/* (cavs/midend/statement.cc:43-123) for the child-sum Tree-LSTM vertex       */
/* function (apps/paper/tree-lstm-cavs.cc:107-172; n_slots = 1 with permuted  */
/* parameter blocks is the chain LSTM of apps/paper/seq-lstm-cavs.cc:45-86).  */
/* ------------------------------------------------------------------------ */
typedef struct cavs_treelstm cavs_treelstm;
typedef struct cavs_treelstm_config {
  int hidden, embed, vocab, classes, n_slots;
  int gemm_bf16;       /* 1: gate GEMMs on tcgen05 with bf16 operands; 0: fp32 GEMMs on the CUDA cores */
  int max_vertices;    /* capacity: vertices per batch */
  int max_level_rows;  /* capacity: rows of the widest level */
} cavs_treelstm_config;
/* Parameters and gradients are ONE flat fp32 device buffer each, laid out
 * Emb [vocab,embed] | W [embed,4H] (i,o,u,f) | U = U_iou [H,3H] then U_f [H,H] | B [4H] (i,f,u,o) | Wc [classes,H] | bc [classes]. */
CAVS_API size_t cavs_treelstm_param_count(const cavs_treelstm_config* cfg);
CAVS_API size_t cavs_treelstm_workspace_bytes(const cavs_treelstm_config* cfg);
/* workspace: caller-owned device memory, 256-byte aligned.  Allocates only a pinned host staging
 * buffer for the per-batch index upload. */
CAVS_API int cavs_treelstm_create(const cavs_treelstm_config* cfg, void* workspace, size_t workspace_bytes, cavs_treelstm** out);
CAVS_API void cavs_treelstm_destroy(cavs_treelstm* e);
CAVS_API int cavs_treelstm_bind(cavs_treelstm* e, float* params, float* grads);
/* Refreshes the bf16 shadow copies of W and U (call after every parameter update; no-op in fp32 mode). */
CAVS_API int cavs_treelstm_refresh_weights(cavs_treelstm* e, void* stream);
/* tok_job / label_job: host int32 per vertex in job order (compact, sample-major).  Reorders them to
 * tensor-id order (the Pull and FunctionPopRet permutations, cavs/backend/op_impl_graphop.cu:214-254,275-327),
 * builds the embedding-gradient segments and uploads all tables with one async copy on an internal
 * copy stream (the `stream` argument is ignored); the next cavs_treelstm_forward waits for it.  Two
 * table slots alternate, so the batch after the one in flight can be loaded while it executes.
 * loss_rows: divisor of the loss gradient (0 = this batch's vertex count). */
CAVS_API int cavs_treelstm_load_batch(cavs_treelstm* e, const cavs_sched* s, const int32_t* tok_job, const int32_t* label_job,
                                      int loss_rows, void* stream);
/* Sparse exchange of the embedding gradient.  rows: the table rows that ANY rank's shard of the coming batch touches
 * (strictly ascending, every token of this rank's shard among them), identical on every rank -- a data-parallel loader
 * that reads the global batch's token ids has them.  The list is consumed by the next cavs_treelstm_load_batch /
 * _stage / _stage_async.  For that batch the embedding block of the gradient buffer then holds ONE ROW PER LISTED ROW,
 * in list order (row i = d(Emb[rows[i]])): backward clears and fills only those rows, cavs_treelstm_step all-reduces
 * n_rows * embed floats instead of vocab * embed and updates the listed rows of the table only.  A list that differs
 * between ranks makes their reductions differ in size: the caller's contract, as with any collective.  Without a list
 * (or n_rows = 0) the block is dense.  Embedding width must be a multiple of 4.  The reference reduces every variable's
 * whole gradient (cavs/midend/session_mpi.cc:31-80) and scatters the embedding gradient into the dense table-sized
 * tensor (cavs/backend/op_impl_embedding_lookup.cu:91-103). */
CAVS_API int cavs_treelstm_set_exchange_rows(cavs_treelstm* e, const int32_t* rows, int n_rows);
/* Level scheduling of a batch (cavs_sched_load into `s`, with the engine's slot count) and cavs_treelstm_load_batch
 * in one call: everything the host does per batch before the device step.  parents == NULL (here and in
 * cavs_treelstm_stage_async): `s` already holds the batch's schedule -- the caller ran cavs_sched_load itself, for
 * instance on a thread of its own while the previous batch was being packed -- and only the tables are packed. */
CAVS_API int cavs_treelstm_stage(cavs_treelstm* e, cavs_sched* s, const int32_t* parents, int batch, int max_len,
                                 const int32_t* tok_job, const int32_t* label_job, int loss_rows);
/* The same on a helper thread of the engine: returns at once, so that the caller's thread can enqueue the step of the
 * batch in flight while this one is scheduled and packed (the host side of a step is then the longer of the two, not
 * their sum).  The arrays must stay valid until the request has finished; the next cavs_treelstm_forward / _step (or
 * cavs_treelstm_stage_wait, which also reports the request's status) waits for it.  One request at a time; `s` must not
 * be used by the caller until then. */
CAVS_API int cavs_treelstm_stage_async(cavs_treelstm* e, cavs_sched* s, const int32_t* parents, int batch, int max_len,
                                       const int32_t* tok_job, const int32_t* label_job, int loss_rows);
CAVS_API int cavs_treelstm_stage_wait(cavs_treelstm* e);
/* Joins a request in flight and makes the staged batch the current one (what the next forward would do by itself).
 * For a loop that keeps the helper thread busy DURING the enqueueing of a step:
 *     promote(batch i);  stage_async(batch i+1);  step();        -- host side per step = max(schedule, enqueue)
 * instead of stage_async(batch i+1) only after step i has been enqueued (their sum, when the device step is shorter).
 * After the first call the engine no longer promotes by itself: forward / step run the batch last promoted and leave
 * a staged one (or a request in flight) alone.  No counterpart in the reference, which schedules inside Session::Run. */
CAVS_API int cavs_treelstm_promote(cavs_treelstm* e, void* stream);
/* One training step in one call: forward, backward, the sum of the gradients over the ranks of `comm` (NULL or a
 * world of one: none) and the update of the flat parameter buffer -- optimizer 0: none (gradients only), 1: SGD,
 * 2: Adagrad with accumulator opt_state [param_count] -- followed by the refresh of the bf16 weight copies.  What
 * Session::Run does for a fetched train op (cavs/midend/session_mpi.cc:84-138).  For the summed gradient to equal
 * the single-GPU gradient of the global batch, every rank passes the GLOBAL loss-row count to load_batch / stage.
 * The embedding block of the gradient is reduced on an internal stream while the weight gradients are still being
 * computed; with exchange rows (cavs_treelstm_set_exchange_rows) only the listed rows travel and are updated.
 * Enqueues only; the loss of this rank's shard is read with cavs_treelstm_read_loss or peek array 6. */
CAVS_API int cavs_treelstm_step(cavs_treelstm* e, cavs_comm* comm, int optimizer, float* opt_state, float lr, float eps,
                                void* stream);
/* Embedding lookup and input projection over the batch's distinct tokens, then the forward level loop. */
CAVS_API int cavs_treelstm_forward(cavs_treelstm* e, void* stream);
/* Loss head, level loop in reverse, deferred weight / bias / embedding gradients (overwrites grads). */
CAVS_API int cavs_treelstm_backward(cavs_treelstm* e, void* stream);
/* Copies the loss sum and the device status word to the host; synchronises `stream`. */
/* Layer stacking (apps/lstm stacks LSTM layers by feeding a layer's h to the next layer's input).  An engine
 * created with vocab == 0 has no embedding table: its inputs are dense rows x [n, embed] in tensor-id order
 * (pitch in floats), set here before forward -- typically the h columns of the layer below (cavs_treelstm_peek
 * array 0, pitch 2*hidden).  Its backward leaves d(loss)/d(x) in peek array 5 ([n, embed], dense).  An engine
 * created with classes == 0 has no loss head: d(loss)/d(h) [n, hidden] (dense) is set here before backward --
 * typically array 5 of the layer above.  Flat parameter layout is unchanged; the absent blocks are empty.
 * Both engines load the same schedule; tokens may be NULL for a dense layer, labels for a headless one. */
CAVS_API int cavs_treelstm_set_dense_input(cavs_treelstm* e, const float* x, long long pitch);
CAVS_API int cavs_treelstm_set_output_grad(cavs_treelstm* e, const float* dh);
/* With an embedding table and a fused loss head the engine keeps ONE state row per distinct leaf token (a leaf's h|c
 * depends on nothing else) and reads leaf states through remapped row indices; the per-vertex rows of the leaves in
 * peek array 0 are then not written by forward, and the leaves' entries of peek array 1 (per-vertex loss) not by
 * backward (the loss head runs once per distinct leaf token).  This call fills both in on `stream`, for callers
 * that want to look at every vertex's state or loss.  A no-op for engines that keep per-vertex leaf rows (dense inputs, no
 * loss head, more than 8 classes, hidden not a multiple of 4 or above 1024, or CAVS_LEAF_BY_TOKEN=0). */
CAVS_API int cavs_treelstm_materialize_state(cavs_treelstm* e, void* stream);
/* Makes `stream` wait until the embedding-gradient block (the first vocab*embed floats of the bound gradient
 * buffer) written by the most recent cavs_treelstm_backward is complete.  backward produces that block before
 * the weight gradients, so a data-parallel caller can start its cross-GPU reduction on another stream
 * while the rest of backward is still running.  Does not block the host. */
CAVS_API int cavs_treelstm_wait_embed_grad(cavs_treelstm* e, void* stream);
/* Bytes of index tables the most recent cavs_treelstm_load_batch copied from pinned host memory to the device. */
CAVS_API size_t cavs_treelstm_upload_bytes(const cavs_treelstm* e);
CAVS_API int cavs_treelstm_read_loss(cavs_treelstm* e, float* loss_sum_host, int* status_host, void* stream);
/* Per-kernel-class timing with CUDA events on the launching stream.  While enabled, every launch
 * of forward / backward is bracketed by two events.  profile_read sums, per class, the elapsed
 * milliseconds, the algorithmic work (flops for class 0, bytes otherwise) and the launch count
 * since the last read.  Classes: 0 gate GEMMs, 1 cell forward, 2 cell backward, 3 child-h gather,
 * 4 child-gradient scatter, 5 loss head, 6 embedding forward, 7 embedding backward, 8 column sum; from
 * cavs_treelstm_step: 9 all-reduce of the embedding block (on the side stream), 10 all-reduce of the other blocks,
 * 11 time the compute stream waited for 9 to finish (its part that was not hidden), 12 optimizer.  n_classes >= 13. */
CAVS_API int cavs_treelstm_profile(cavs_treelstm* e, int enable);
CAVS_API int cavs_treelstm_profile_read(cavs_treelstm* e, double* ms, double* work, int* launches, int n_classes);
/* Device views for inspection: 0 state [n,2H], 1 loss [n], 2 dOut [n,H] (classes > 8 only: the fused
 * loss head does not materialise it), 3 mailbox [n,2H], 4 saved gates (fp32 mode: float [n,(3+K)H] = i|o|u|f_0..f_{K-1};
 * bf16 mode with hidden a multiple of 64: half, the whole arena, G3 [max_vertices,3H] = i|o|u followed by
 * GF [max_vertices,K,H] = the forget gates), 5 d(x) [n,E] (dense-input engines),
 * 6 the two words cavs_treelstm_read_loss copies: loss sum (float) and status (int) -- for callers that fetch
 * them with their own asynchronous copy instead of the blocking read. */
CAVS_API int cavs_treelstm_peek(cavs_treelstm* e, int what, const void** dev_ptr, size_t* bytes);

/* ------------------------------------------------------------------------ */
/* Child-sum Tree-GRU engine: the same level loop over a second vertex        */
/* function.  The reference ships LSTM vertex functions only (apps/paper/     */
/* tree-lstm-cavs.cc, apps/lstm/); this shows what a user-defined F costs on  */
/* top of the shared tables, input projection, loss head and weight-gradient  */
/* passes.  Per vertex with children h_k: ht = sum h_k; r_k = sigmoid(a_r +   */
/* h_k U_r + b_r); z = sigmoid(a_z + ht U_z + b_z); n = tanh(a_n + (sum r_k o */
/* h_k) U_n + b_n); h = (1-z) o ht + z o n, with a = Emb[tok] W.              */
/* Flat parameters: Emb [V,E] | W [E,3H] (r,z,n) | U [3,H,H] | B [3H] |       */
/* Wc [C,H] | bc [C].  Same config struct and call sequence as cavs_treelstm; */
/* classes <= 8; one batch at a time, tables uploaded on the caller's stream. */
/* ------------------------------------------------------------------------ */
typedef struct cavs_treegru cavs_treegru;
CAVS_API size_t cavs_treegru_param_count(const cavs_treelstm_config* cfg);
CAVS_API size_t cavs_treegru_workspace_bytes(const cavs_treelstm_config* cfg);
CAVS_API int cavs_treegru_create(const cavs_treelstm_config* cfg, void* workspace, size_t workspace_bytes, cavs_treegru** out);
CAVS_API void cavs_treegru_destroy(cavs_treegru* e);
CAVS_API int cavs_treegru_bind(cavs_treegru* e, float* params, float* grads);
CAVS_API int cavs_treegru_refresh_weights(cavs_treegru* e, void* stream);
CAVS_API int cavs_treegru_load_batch(cavs_treegru* e, const cavs_sched* s, const int32_t* tok_job, const int32_t* label_job,
                                     int loss_rows, void* stream);
CAVS_API int cavs_treegru_forward(cavs_treegru* e, void* stream);
CAVS_API int cavs_treegru_backward(cavs_treegru* e, void* stream);
CAVS_API int cavs_treegru_read_loss(cavs_treegru* e, float* loss_sum_host, int* status_host, void* stream);
/* Device views: 0 state [n,H], 1 loss [n], 2 dOut [n,H], 3 mailbox [n,H]. */
CAVS_API int cavs_treegru_peek(cavs_treegru* e, int what, const void** dev_ptr, size_t* bytes);

/* ------------------------------------------------------------------------ */
/* Synthetic workloads (host only).  One SplitMix64 stream per (seed, stream).*/
/* ------------------------------------------------------------------------ */
/* Random trees: leaves ~ U{leaf_lo..leaf_hi}; every internal vertex has 2 children when
 * max_arity == 2, else U{1..max_arity} (a unary vertex never has a unary child); vertices
 * are numbered in post-order so the root is last.  parents: [batch, max_len] filled with -1
 * padding; max_len must be >= the largest tree.  is_leaf (optional): [batch, max_len]. */
CAVS_API int cavs_synth_trees(uint64_t seed, int batch, int leaf_lo, int leaf_hi, int max_arity, int max_len,
                     int32_t* parents, uint8_t* is_leaf);
/* Chains: lengths ~ U{len_lo..len_hi}; vertex t's parent is t+1. */
CAVS_API int cavs_synth_chains(uint64_t seed, int batch, int len_lo, int len_hi, int max_len, int32_t* parents);
/* Zipf(s) token ids over [0, vocab) by inverse-CDF lookup. */
CAVS_API int cavs_synth_zipf(uint64_t seed, double s, int vocab, int32_t* out, size_t count);
/* Uniform ints in [0, bound) and uniform floats in [-scale, scale). */
CAVS_API int cavs_synth_uniform_int(uint64_t seed, int bound, int32_t* out, size_t count);
CAVS_API int cavs_synth_uniform_float(uint64_t seed, float scale, float* out, size_t count);

#ifdef __cplusplus
}
#endif
#endif /* CAVS_B200_H_ */
