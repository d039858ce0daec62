// C ABI wrappers of the per-level and per-step kernels (see include/cavs_b200.h).
#include "abi_common.h"
#include "kernels/cell.h"

using namespace cavs_b200;

static cudaStream_t St(void* s) { return static_cast<cudaStream_t>(s); }

extern "C" int cavs_gather_child_h(void* S, void* HK, int bf16, const float* state, const int32_t* child, int n_total,
                                   int off, int rows, int hidden, int n_slots, void* stream) {
  CAVS_REQUIRE((S && HK && state && child) || rows == 0, CAVS_ERR_BAD_ARG, "gather_child_h: null pointer");
  return LaunchGatherChildH(S, HK, bf16 != 0, state, child, n_total, off, rows, hidden, n_slots, St(stream));
}
extern "C" int cavs_treelstm_cell_fwd(float* state, void* gates, const void* A, const void* P, const void* Q, int preact_bf16,
                                      const float* bias, const int32_t* child, const int32_t* a_row, int n_total, int off, int rows,
                                      int hidden, int n_slots, int leaf, void* stream) {
  CAVS_REQUIRE((state && gates && A && bias && (leaf || (P && Q && child))) || rows == 0, CAVS_ERR_BAD_ARG,
               "treelstm_cell_fwd: null pointer");
  return LaunchCellFwd(state, gates, A, P, Q, preact_bf16 != 0, bias, child, a_row, n_total, off, rows, hidden, n_slots, leaf != 0, St(stream));
}
extern "C" int cavs_treelstm_cell_bwd(void* dA, void* ZF, int bf16, float* mailbox, const float* dOut, const void* gates,
                                      const float* state, const int32_t* child, const int32_t* parent, int n_total, int off,
                                      int rows, int hidden, int n_slots, int leaf, void* stream) {
  CAVS_REQUIRE((dA && mailbox && dOut && gates && state && parent && (leaf || (ZF && child))) || rows == 0, CAVS_ERR_BAD_ARG,
               "treelstm_cell_bwd: null pointer");
  return LaunchCellBwd(dA, ZF, bf16 != 0, mailbox, nullptr, dOut, gates, state, child, parent, n_total, off, rows, hidden, n_slots,
                       leaf != 0, St(stream));
}
extern "C" int cavs_scatter_child_grad(float* mailbox, const float* ds, const float* dq, const int32_t* child, int n_total,
                                       int off, int rows, int hidden, int n_slots, void* stream) {
  CAVS_REQUIRE((mailbox && ds && dq && child) || rows == 0, CAVS_ERR_BAD_ARG, "scatter_child_grad: null pointer");
  return LaunchScatterChildGrad(mailbox, ds, dq, child, n_total, off, rows, hidden, n_slots, St(stream));
}
extern "C" int cavs_embed_fwd(void* out, int bf16, const float* table, const int32_t* tok, int rows, int embed, int vocab,
                              void* stream) {
  return LaunchEmbedFwd(out, bf16 != 0, table, tok, rows, embed, vocab, St(stream));
}
extern "C" int cavs_embed_bwd_segmented(float* dtable, const float* dX, const int32_t* order, const int32_t* chunk_off,
                                        int n_chunks, const int32_t* seg_first_chunk, const int32_t* seg_tok, int n_seg,
                                        float* scratch, int embed, void* stream) {
  return LaunchEmbedBwd(dtable, dX, order, nullptr, chunk_off, n_chunks, seg_first_chunk, seg_tok, n_seg, scratch, embed, St(stream));
}
extern "C" size_t cavs_fc_softmax_xent_scratch_bytes(int hidden, int classes) { return LossHeadScratchBytes(hidden, classes); }
extern "C" int cavs_fc_softmax_xent(float* loss, float* loss_sum, float* dH, float* dWc, float* dbc, const float* h,
                                    long long h_pitch, const int32_t* label, const float* Wc, const float* bc, int rows,
                                    int hidden, int classes, float inv_rows, float* scratch, void* stream) {
  return LaunchLossHead(loss, loss_sum, dH, dWc, dbc, h, h_pitch, label, Wc, bc, rows, hidden, classes, inv_rows, scratch, St(stream));
}
extern "C" size_t cavs_column_sum_scratch_bytes(int cols) { return ColumnSumScratchBytes(cols); }
extern "C" int cavs_column_sum(float* out, const void* x, int bf16, long long pitch, int rows, int cols, float* scratch,
                               void* stream) {
  return LaunchColumnSum(out, x, bf16 != 0, pitch, rows, cols, scratch, St(stream));
}
extern "C" int cavs_sgd(float* w, const float* g, size_t count, float lr, void* stream) { return LaunchSgd(w, g, count, lr, St(stream)); }
extern "C" int cavs_adagrad(float* w, float* acc, const float* g, size_t count, float lr, float eps, void* stream) {
  return LaunchAdagrad(w, acc, g, count, lr, eps, St(stream));
}
extern "C" int cavs_cast_bf16(void* dst, const float* src, size_t count, void* stream) { return LaunchCastBf16(dst, src, count, St(stream)); }
