// Level-batched execution of the child-sum Tree-LSTM vertex function, forward and
// backward: the host-side level loop.
//
// Replaces GraphStatement::Run / GraphGradStatement::Run (cavs/midend/statement.cc:43-123)
// and the per-op prologue ExprStatement::Run (statement.cc:8-41).  Differences that matter:
//   * the input projection x.W does not depend on children and depends on a vertex only through
//     its token (x is an embedding row), so it is one GEMM over the batch's DISTINCT tokens before
//     the loop -- (Emb.W)[tok] instead of Emb[tok].W per vertex per level (tree-lstm-cavs.cc:139-146);
//     the cell reads its row through a per-vertex index.  Symmetrically, d(pre-activation) rows are
//     summed per token before the input-weight and embedding gradients, which turns the three
//     largest GEMMs of a step into one segmented row sum plus GEMMs over distinct tokens;
//   * level 0 holds only leaves, whose recurrent GEMMs multiply zero rows in the reference
//     (op_impl_graphop.cu:77-86); they are skipped, which is exact;
//   * per level the forward pass is 4 launches (gather, 2 GEMMs, fused cell) and the
//     backward pass 4 (fused cell-grad, 2 GEMMs, scatter) instead of ~46 / ~90;
//   * weight, bias and embedding gradients are deferred to one pass over all vertices after
//     the loop, as BatchingWeightUpdater does (cavs/midend/batch_weight_updater.h:10-85);
//   * all index tables of the batch arrive in one pinned upload; no per-op host-to-device
//     copy and no device synchronisation inside a step.
// Per-vertex tensors live in tensor-id (execution) order, so a level is a contiguous row
// range [level_off[l], level_off[l+1]) of every arena (cf. graph_session.cc:27-43).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "abi_common.h"
#include "host/sched_handle.h"
#include "host/threads.h"
#include "kernels/cell.h"
#include "kernels/gemm.h"
#include "kernels/launch.h"

using namespace cavs_b200;

struct cavs_treelstm {
  cavs_treelstm_config cfg{};
  bool bf16 = false;
  size_t elt = 4;               // bytes per GEMM-operand element
  // ---- device workspace views ----
  int32_t* d_idx = nullptr;     // two index blobs of idx_ints each, mirrored by h_idx (pinned)
  int32_t* h_idx = nullptr;
  size_t idx_ints = 0;
  uint8_t *X = nullptr, *S = nullptr, *HK = nullptr, *dA = nullptr, *ZF = nullptr;   // GEMM operands (fp32 or bf16)
  uint8_t* dAtok = nullptr;     // [distinct tokens, 4H] per-token sums of dA (GEMM operand precision)
  uint8_t *A = nullptr, *P = nullptr, *Q = nullptr;   // gate pre-activations: fp32, or bf16 in bf16 mode
  uint8_t* gates = nullptr;                           // saved gates: fp32, or fp16 in bf16 mode
  float *state = nullptr, *mailbox = nullptr;
  float *dOut = nullptr, *dz8 = nullptr, *ds = nullptr, *dq = nullptr, *dX = nullptr, *loss = nullptr, *dB_tmp = nullptr;
  float* tail = nullptr;        // [0] loss sum, [1] status word (int)
  float *loss_scratch = nullptr, *col_scratch = nullptr, *emb_scratch = nullptr, *splitk_scratch = nullptr;
  size_t splitk_bytes = 0;
  uint8_t *W_bf = nullptr, *U_bf = nullptr, *Wc_bf = nullptr;
  // wide loss head (classes > 8): logits / dz [N, Cp] fp32, bf16 copies of dz and of the pushed h rows
  float* logits = nullptr;
  uint8_t *dz_bf = nullptr, *h_bf = nullptr;
  // Layer stacking: dense per-vertex inputs instead of an embedding table (cfg.vocab == 0) and an
  // output gradient handed in by the layer above instead of a loss head (cfg.classes == 0).
  const float* x_dense = nullptr;   // [n, embed] rows in tensor-id order, pitch x_pitch
  long long x_pitch = 0;
  const float* dh_ext = nullptr;    // [n, hidden] dense
  // Leaf states per token: a leaf's h|c depends only on its token, so the leaf level is computed once per distinct
  // token into rows [max_vertices, max_vertices + tokens) of `state`, and everything that reads a leaf's state
  // (the parents' gather and cell kernels, the loss head) goes through remapped row indices.  Needs the
  // streaming loss head (it reads rows by index) and a caller that does not read `state` rows directly.
  bool leaf_tok = false;
  bool LeafTokEligible() const {
    return cfg.vocab > 0 && cfg.classes > 0 && !WideHead() && cfg.hidden % 4 == 0 && cfg.hidden <= 1024 && OffWc() % 4 == 0;
  }
  // Token inputs with hidden a multiple of 4: the leaf level's backward cell is folded into the per-token sums of dA
  // (the leaves' dA rows are never stored) and the bias gradient is the column sum of the chunk partials.
  bool TokGrad() const { return cfg.vocab > 0 && cfg.hidden % 4 == 0; }
  // With per-token leaf states, a fused loss head and token gradient sums, the loss head also runs once per distinct
  // leaf token instead of once per leaf (weighted by the token's label histogram).
  bool TokHead() const { return leaf_tok && FusedDh() && TokGrad(); }
  float* ptok = nullptr;        // [tokens, 8] class probabilities of the leaf tokens (TokHead)
  // Level 1 by token (l1_tok): every child of a level-1 vertex is a leaf, and a leaf's h depends on its token
  // only, so every product of that level with the recurrent weights is formed once per distinct token instead of
  // once per vertex -- forward h_tok.U (PQT), backward the per-token sums of the parents' gate gradients over
  // parent-child links (ZT), d(h) per token (dh_tok = ZT.U^T) and the level's share of dU (h_tok^T ZT).  Exact
  // algebra (linearity of the products), like the per-token input projection.
  bool l1_tok = false, l1_always = false;
  uint8_t *htok_bf = nullptr, *PQT = nullptr, *ZT = nullptr;   // [tokens, H], [tokens, 4H], [tokens, 4H] (GEMM element type)
  float *dh_tok = nullptr, *link_scratch = nullptr;            // [tokens, H]; [link chunks, 4H]
  bool Dense() const { return cfg.vocab == 0; }
  bool Headless() const { return cfg.classes == 0; }
  int Cp() const { return (cfg.classes + 7) & ~7; }
  bool WideHead() const { return cfg.classes > 8; }
  // d(pushed h) is rebuilt inside the cell gradient from d(logits) rows when the classifier fits its shared-memory copy
  bool FusedDh() const { return !Headless() && !WideHead() && static_cast<long long>(cfg.classes) * cfg.hidden <= 8192; }
  // TMA maps of the per-level GEMM operands, encoded once over whole arenas (bf16 mode).
  TcOperandMap map_S, map_HK, map_dA3, map_ZF;              // K-major A operands: [rows, k]
  TcOperandMap map_Uiou_mn, map_Uf_mn, map_Uiou_k, map_Uf_k; // weights as B: [k,n] for forward, [n,k] for dgrad
  TcOperandMap map_Uiou_k64, map_Uf_k64;                     // the dgrad maps again for 64-column tiles (small levels)
  TcOperandMap map_P, map_Q, map_ds;                         // level-local outputs (rows past a level's end are scratch)
  // Gate epilogue (bf16 mode, hidden a multiple of 64): the gate products' epilogue adds the input projection and the
  // bias, applies sigmoid / tanh and stores the finished gates (fp16) straight into the saved-gate arena, split into
  // G3 [N,3H] (i|o|u, the head of `gates`) and GF [N,K,H] (forget gates, behind it); P and Q are never stored, and
  // the forward cell only forms c and h.  CAVS_GATE_EPILOGUE=0 keeps the separate pre-activation arrays.
  bool gate_epi = false;
  bool dual_gemm = true;       // small levels: both products of a level in one launch (CAVS_DUAL_GEMM=0: never)
  uint8_t* gates_f = nullptr;
  TcOperandMap map_G3, map_GF;
  float *params = nullptr, *grads = nullptr;   // flat fp32: Emb | W | U | B | Wc | bc
  // ---- batches: two slots so the tables of the next batch can be packed and uploaded while the
  // current one executes; forward() promotes the staged slot ----
  struct Batch {
    int n = 0, n_total = 0, n_levels = 0, loss_rows = 0, n_chunks = 0, n_seg = 0;
    std::vector<int32_t> level_off;
    int32_t *child_st = nullptr, *state_row = nullptr;   // leaf_tok: state rows of the children / of every vertex
    int32_t *tok_hist = nullptr, *head_row = nullptr;    // TokHead: label histogram per token; state rows of the loss rows
    int32_t *child = nullptr, *parent = nullptr, *tok = nullptr, *label = nullptr, *order = nullptr, *chunk_off = nullptr,
            *seg_first_chunk = nullptr, *seg_tok = nullptr, *tok_slot = nullptr, *chunk_out = nullptr, *multi_seg = nullptr, *chunk_seg = nullptr;
    int n_multi = 0;
    int shared_chunk = -1;   // chunk whose partial row is the column sum over the internal vertices, or -1
    // l1_tok: links (t, c) of level 1 as t * K + c, grouped by the child's token row and cut into chunks
    int32_t *l_order = nullptr, *l_chunk_off = nullptr, *l_chunk_out = nullptr, *l_seg_first = nullptr, *l_multi = nullptr;
    int n_l_chunks = 0, n_l_multi = 0, n_links = 0;
    bool l1 = false;         // this batch runs level 1 by token (it has a level 1)
    // exchange rows (cavs_treelstm_set_exchange_rows): the embedding rows whose gradients exist for this batch, in
    // ascending order, and for each token segment its position in that list; n_xrows == 0: dense gradient block
    int32_t *xrows = nullptr, *seg_pos = nullptr;
    int n_xrows = 0;
  };
  Batch slot[2];
  int active = -1, staged = -1;
  size_t last_upload_bytes = 0;   // size of the table blob the most recent load_batch sent to the device
  // The table upload runs on its own stream so it overlaps the step in flight: copied[s] marks the
  // upload into slot s, slot_done[s] the end of the last pass (forward, backward or state fill) that read slot s.
  cudaStream_t copy_stream = nullptr;
  cudaEvent_t copied[2] = {nullptr, nullptr}, slot_done[2] = {nullptr, nullptr};
  cudaEvent_t emb_ready = nullptr;   // recorded in backward once the embedding gradient is complete
  // cavs_treelstm_step: the embedding block of the gradient is reduced across GPUs on its own stream while the
  // weight-gradient products still run; comm_done marks the end of that reduction
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t comm_done = nullptr;
  // cavs_treelstm_stage_async: one helper thread per engine schedules and packs the next batch while the caller's
  // thread enqueues the current step; forward() joins the pending request before it promotes the staged tables.
  struct Stager {
    std::thread thread;
    std::mutex mu;
    std::condition_variable cv;
    bool has_job = false, busy = false, quit = false;
    int device = 0, status = CAVS_OK;
    std::string error;
    cavs_sched* sched = nullptr;
    const int32_t *parents = nullptr, *tok = nullptr, *label = nullptr;
    int batch = 0, max_len = 0, loss_rows = 0;
  };
  Stager* stager = nullptr;
  bool slot_used[2] = {false, false};
  std::vector<int32_t> pending_xrows;   // consumed by the next load_batch
  bool explicit_promote = false;   // set by cavs_treelstm_promote: forward() then leaves the staged batch alone
  std::vector<int32_t> bucket, slot_of_token, leaf_count, link_bucket;
  // ---- optional per-kernel-class timing (cavs_treelstm_profile) ----
  bool prof_on = false;
  std::vector<cudaEvent_t> ev_pool;
  size_t ev_used = 0;
  struct Rec { int cls; cudaEvent_t a, b; double work; };
  std::vector<Rec> recs;
  cudaEvent_t NextEvent() {
    if (ev_used == ev_pool.size()) { cudaEvent_t ev; cudaEventCreate(&ev); ev_pool.push_back(ev); }
    return ev_pool[ev_used++];
  }

  size_t OffW() const { return static_cast<size_t>(cfg.vocab) * cfg.embed; }
  size_t OffU() const { return OffW() + static_cast<size_t>(cfg.embed) * 4 * cfg.hidden; }
  size_t OffB() const { return OffU() + static_cast<size_t>(4) * cfg.hidden * cfg.hidden; }
  size_t OffWc() const { return OffB() + static_cast<size_t>(4) * cfg.hidden; }
  size_t Offbc() const { return OffWc() + static_cast<size_t>(cfg.classes) * cfg.hidden; }
  size_t ParamCount() const { return Offbc() + cfg.classes; }
  int* Status() const { return reinterpret_cast<int*>(tail + 1); }
};

namespace {

size_t Align(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

// Host-side packing of a batch's tables runs next to the device step of the previous batch; its loops over vertices
// that touch disjoint outputs are split over a few threads (CAVS_HOST_THREADS, default: the host's threads shared out
// among its GPUs, at most 8; short loops stay on the caller's thread).
int PackThreads() {
  static const int n = HostThreadBudget(8);
  return n;
}
template <typename F>
void ParallelRanges(int n, F fn) {
  const int threads = std::max(1, std::min(PackThreads(), n / 32768));
  if (threads <= 1) { fn(0, n); return; }
  const int step = (n + threads - 1) / threads;
  std::vector<std::thread> pool;
  for (int w = 1; w < threads; ++w) {
    const int b = w * step, e2 = std::min(n, b + step);
    if (b < e2) pool.emplace_back([=] { fn(b, e2); });
  }
  fn(0, std::min(n, step));
  for (auto& th : pool) th.join();
}

struct Carver {
  uint8_t* base;
  size_t used = 0;
  explicit Carver(void* b) : base(static_cast<uint8_t*>(b)) {}
  template <typename T> T* Take(size_t count) {
    T* p = base ? reinterpret_cast<T*>(base + used) : nullptr;
    used += Align(count * sizeof(T));
    return p;
  }
};

// Kernel classes reported by cavs_treelstm_profile_read.  "work" is algorithmic flops for the
// GEMM class and algorithmic bytes (the kernel interface's inputs + outputs) for the others.
// Levels of at most this many rows release their successors early whatever they are (chained launches).
constexpr int kChainSmallRows = 4096;

enum ProfClass { kProfGemm = 0, kProfCellFwd, kProfCellBwd, kProfGatherH, kProfScatterGrad, kProfLossHead, kProfEmbedFwd,
                 kProfEmbedBwd, kProfColumnSum, kProfCommEmbed, kProfCommRest, kProfCommExposed, kProfOptimizer, kProfCount };

// Runs `call` (an int-returning launch) bracketed by events when profiling is on.
#define PROF(e, cls, work_expr, st, call)                                   \
  do {                                                                      \
    int _rc;                                                                \
    if ((e)->prof_on) {                                                     \
      cudaEvent_t _a = (e)->NextEvent(), _b = (e)->NextEvent();             \
      cudaEventRecord(_a, st);                                              \
      _rc = (call);                                                         \
      cudaEventRecord(_b, st);                                              \
      (e)->recs.push_back({cls, _a, _b, static_cast<double>(work_expr)});   \
    } else {                                                                \
      _rc = (call);                                                         \
    }                                                                       \
    if (_rc) return _rc;                                                    \
  } while (0)

int CheckConfig(const cavs_treelstm_config* c) {
  CAVS_REQUIRE(c, CAVS_ERR_BAD_ARG, "treelstm: null config");
  CAVS_REQUIRE(c->hidden > 0 && c->embed > 0 && c->vocab >= 0 && c->classes >= 0, CAVS_ERR_BAD_ARG,
               "treelstm: hidden and embed must be positive, vocab and classes non-negative");
  CAVS_REQUIRE(c->n_slots >= 1 && c->n_slots <= kMaxSlots, CAVS_ERR_BAD_ARG, "treelstm: child slots must be 1..4");
  CAVS_REQUIRE(c->max_vertices > 0 && c->max_level_rows > 0 && c->max_level_rows <= c->max_vertices, CAVS_ERR_BAD_ARG,
               "treelstm: capacities must be positive and max_level_rows <= max_vertices");
  if (c->gemm_bf16)
    CAVS_REQUIRE(c->hidden % 8 == 0 && c->embed % 8 == 0, CAVS_ERR_BAD_ARG,
                 "treelstm: the tensor-core path needs hidden and embed to be multiples of 8 (16-byte TMA rows)");
  return CAVS_OK;
}

// Rows of the input projection: distinct tokens of a batch, or every vertex with dense inputs.
size_t MaxSegments(const cavs_treelstm_config& c) { return c.vocab == 0 ? c.max_vertices : std::min<size_t>(c.max_vertices, c.vocab); }
// A token's rows are cut into chunks of kEmbedChunk, separately for its leaves and its internal vertices.
size_t MaxChunks(const cavs_treelstm_config& c) { return 2 * MaxSegments(c) + c.max_vertices / kEmbedChunk + 2; }
// Parent-child links of one level, grouped by the child's token: one chunk list per token plus the overflow chunks.
size_t MaxLinkChunks(const cavs_treelstm_config& c) {
  return MaxSegments(c) + static_cast<size_t>(c.n_slots) * c.max_vertices / kEmbedChunk + 2;
}
size_t IdxInts(const cavs_treelstm_config& c) {
  const size_t n = c.max_vertices;
  return (2 * c.n_slots + 7) * n + 4 * (MaxChunks(c) + 1) + (MaxSegments(c) + 1) + 10 * MaxSegments(c) + 64 +
         c.n_slots * n + 2 * (MaxLinkChunks(c) + 1) + 2 * (MaxSegments(c) + 1) +   // link lists (level 1 by token)
         static_cast<size_t>(std::max(c.vocab, 0)) + MaxSegments(c) + 2;            // exchange rows and their positions
}

// Split-K scratch large enough for the three weight-gradient GEMMs at full capacity.
size_t SplitKBytes(const cavs_treelstm_config& c) {
  // fp32 mode: room for the k-split partials of a narrow level's products (up to 16 slabs of 64 rows x 4H)
  if (!c.gemm_bf16) return static_cast<size_t>(16) * 64 * 4 * c.hidden * sizeof(float);
  const int N = c.max_vertices, H = c.hidden, E = c.embed, K = c.n_slots;
  size_t b = GemmBf16ScratchBytes(E, 4 * H, 32);
  b = std::max(b, GemmBf16ScratchBytes(H, 3 * H, 32));
  b = std::max(b, GemmBf16ScratchBytes(H, H, 32));
  if (c.classes > 8) b = std::max(b, GemmBf16ScratchBytes(c.classes, H, 16));
  (void)N; (void)K;
  return b;
}

// Everything about an engine that follows from its configuration (and the environment) alone.
void InitModes(cavs_treelstm* e, const cavs_treelstm_config& cfg) {
  e->cfg = cfg;
  e->bf16 = cfg.gemm_bf16 != 0;
  e->elt = e->bf16 ? 2 : 4;
  const char* v = std::getenv("CAVS_LEAF_BY_TOKEN");   // "0": keep one state row per leaf vertex
  e->leaf_tok = e->LeafTokEligible() && !(v != nullptr && v[0] == '0');
  // "0": level 1 runs per vertex like every other level; "1": by token whenever possible; unset: by token for batches
  // whose level 1 has at least twice as many rows as the batch has distinct tokens (below that the handful of extra
  // launches costs what the smaller products save)
  const char* v1 = std::getenv("CAVS_LEVEL1_BY_TOKEN");
  e->l1_tok = e->TokHead() && e->bf16 && !(v1 != nullptr && v1[0] == '0');
  e->l1_always = v1 != nullptr && v1[0] == '1';
  const char* v3 = std::getenv("CAVS_DUAL_GEMM");
  e->dual_gemm = !(v3 != nullptr && v3[0] == '0');
  const char* v2 = std::getenv("CAVS_GATE_EPILOGUE");
  e->gate_epi = e->bf16 && cfg.hidden % 64 == 0 && !(v2 != nullptr && v2[0] == '0');
}

// Carves every device array out of the workspace; with base == nullptr it only sizes it.
size_t Carve(cavs_treelstm* e, void* base) {
  const cavs_treelstm_config& c = e->cfg;
  const size_t N = c.max_vertices, L = c.max_level_rows, H = c.hidden, E = c.embed, K = c.n_slots;
  const size_t elt = c.gemm_bf16 ? 2 : 4;
  Carver w(base);
  e->d_idx = w.Take<int32_t>(2 * IdxInts(c));
  const size_t T = MaxSegments(c);   // distinct tokens per batch
  e->X = w.Take<uint8_t>(T * E * elt);
  e->S = w.Take<uint8_t>(N * H * elt);
  e->HK = w.Take<uint8_t>(N * K * H * elt);
  e->dA = w.Take<uint8_t>(N * 4 * H * elt);
  e->ZF = w.Take<uint8_t>(N * K * H * elt);
  e->A = w.Take<uint8_t>(T * 4 * H * elt);
  e->dAtok = w.Take<uint8_t>(c.vocab == 0 ? 0 : T * 4 * H * elt);
  e->P = w.Take<uint8_t>(L * 3 * H * elt);
  e->Q = w.Take<uint8_t>(L * K * H * elt);
  e->gates = w.Take<uint8_t>(N * (3 + K) * H * elt);
  e->gates_f = (e->gate_epi && e->gates) ? e->gates + N * 3 * H * elt : nullptr;
  e->state = w.Take<float>((N + (e->leaf_tok ? T : 0)) * 2 * H);   // per-token leaf rows follow the vertex rows
  e->mailbox = w.Take<float>(N * 2 * H);
  // d(pushed h): materialised only by the wide loss head; the fused head hands d(logits) rows (dz8) to the cell gradient
  e->dOut = w.Take<float>(e->FusedDh() || e->Headless() ? 0 : N * H);
  e->dz8 = w.Take<float>(e->FusedDh() ? N * kHeadDzPitch : 0);
  e->ptok = w.Take<float>(e->TokHead() ? T * kHeadDzPitch : 0);
  e->htok_bf = w.Take<uint8_t>(e->l1_tok ? T * H * elt : 0);
  e->PQT = w.Take<uint8_t>(e->l1_tok ? T * 4 * H * elt : 0);
  e->ZT = w.Take<uint8_t>(e->l1_tok ? T * 4 * H * elt : 0);
  e->dh_tok = w.Take<float>(e->l1_tok ? T * H : 0);
  e->link_scratch = w.Take<float>(e->l1_tok ? MaxLinkChunks(c) * 4 * H : 0);
  e->ds = w.Take<float>(L * H);
  e->dq = w.Take<float>(c.gemm_bf16 ? 0 : L * K * H);   // bf16 mode: the dq product is scattered by its own epilogue
  e->dX = w.Take<float>(T * E);
  e->loss = w.Take<float>(N);
  e->dB_tmp = w.Take<float>(CellBwdFusesBias(c.hidden) ? static_cast<size_t>(CellBwdMaxGrid()) * 4 * H : 4 * H);
  e->tail = w.Take<float>(4);
  const bool wide = c.classes > 8;
  const size_t Cp = (c.classes + 7) & ~static_cast<size_t>(7);
  e->loss_scratch = w.Take<float>(wide || c.classes == 0 ? 0 : LossHeadScratchBytes(c.hidden, c.classes) / sizeof(float));
  e->logits = w.Take<float>(wide ? N * Cp : 0);
  e->dz_bf = w.Take<uint8_t>(wide && c.gemm_bf16 ? N * Cp * 2 : 0);
  e->h_bf = w.Take<uint8_t>(wide && c.gemm_bf16 ? N * H * 2 : 0);
  e->Wc_bf = w.Take<uint8_t>(wide && c.gemm_bf16 ? static_cast<size_t>(c.classes) * H * 2 : 0);
  e->col_scratch = w.Take<float>(ColumnSumScratchBytes(std::max(4 * c.hidden, c.classes)) / sizeof(float));
  e->emb_scratch = w.Take<float>(c.vocab == 0 ? 0 : MaxChunks(c) * 4 * H);
  e->splitk_bytes = SplitKBytes(c);
  e->splitk_scratch = w.Take<float>(e->splitk_bytes / sizeof(float));
  e->W_bf = w.Take<uint8_t>(c.gemm_bf16 ? static_cast<size_t>(E) * 4 * H * 2 : 0);
  e->U_bf = w.Take<uint8_t>(c.gemm_bf16 ? static_cast<size_t>(4) * H * H * 2 : 0);
  return w.used;
}

// One GEMM of the step in either precision.  `a_t` / `b_t`: operand is used transposed
// relative to its row-major storage (a_t: A stored [k,m]; b_t: B stored [n,k]).
// `accumulate`: 0 store, 1 add into C, 2 store C as bf16 (bf16 mode only; the fp32 path always writes fp32).
int Gemm(cavs_treelstm* e, void* c, long long ldc, int accumulate, const void* a, long long lda, bool a_t, const void* b,
         long long ldb, bool b_t, int m, int n, int k, bool split_ok, cudaStream_t st, const TcOperandMap* amap = nullptr,
         int a_row_off = 0, const TcOperandMap* bmap = nullptr, const TcOperandMap* cmap = nullptr,
         const TcOperandMap* bmap_small = nullptr) {
  if (m == 0 || n == 0 || k == 0) return CAVS_OK;
  if (e->bf16 && amap && bmap) {
    // Per-level GEMM through pre-encoded arena maps: `a` is not used, the level is a row offset.
    GemmBf16MappedArgs g;
    g.c = c; g.ldc = ldc; g.out_mode = accumulate;
    g.a = amap; g.a_row_off = a_row_off; g.b = bmap; g.b_small = bmap_small; g.c_map = cmap;
    g.m = m; g.n = n; g.k = k;
    g.status = e->Status();
    PROF(e, kProfGemm, 2.0 * m * n * k, st, GemmBf16Mapped(g, st));
    return CAVS_OK;
  }
  if (e->bf16) {
    GemmBf16Args g;
    g.c = c; g.ldc = ldc; g.out_mode = accumulate;
    g.a = a; g.lda = lda; g.a_major = a_t ? 1 : 0;   // stored [k,m] = MN-major
    g.b = b; g.ldb = ldb; g.b_major = b_t ? 0 : 1;   // stored [n,k] = K-major, [k,n] = MN-major
    g.m = m; g.n = n; g.k = k;
    g.status = e->Status();
    if (split_ok) {
      g.splits = GemmBf16SplitsFor(m, n, k);
      g.scratch = e->splitk_scratch; g.scratch_bytes = e->splitk_bytes;
    }
    PROF(e, kProfGemm, 2.0 * m * n * k, st, GemmBf16(g, st));
    return CAVS_OK;
  }
  GemmF32Args g;
  g.c = static_cast<float*>(c); g.ldc = ldc; g.accumulate = accumulate == 1;
  g.a = static_cast<const float*>(a); g.a_rs = a_t ? 1 : lda; g.a_cs = a_t ? lda : 1;
  g.b = static_cast<const float*>(b); g.b_rs = b_t ? 1 : ldb; g.b_cs = b_t ? ldb : 1;
  g.m = m; g.n = n; g.k = k;
  g.scratch = e->splitk_scratch; g.scratch_bytes = e->splitk_bytes;
  PROF(e, kProfGemm, 2.0 * m * n * k, st, GemmF32(g, st));
  return CAVS_OK;
}

}  // namespace

extern "C" size_t cavs_treelstm_param_count(const cavs_treelstm_config* cfg) {
  if (CheckConfig(cfg) != CAVS_OK) return 0;
  cavs_treelstm tmp; tmp.cfg = *cfg;
  return tmp.ParamCount();
}

extern "C" size_t cavs_treelstm_workspace_bytes(const cavs_treelstm_config* cfg) {
  if (CheckConfig(cfg) != CAVS_OK) return 0;
  cavs_treelstm tmp;
  InitModes(&tmp, *cfg);
  return Carve(&tmp, nullptr);
}

extern "C" int cavs_treelstm_create(const cavs_treelstm_config* cfg, void* workspace, size_t workspace_bytes,
                                    cavs_treelstm** out) {
  if (int rc = CheckConfig(cfg)) return rc;
  CAVS_REQUIRE(out && workspace, CAVS_ERR_BAD_ARG, "treelstm_create: null pointer");
  CAVS_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, CAVS_ERR_BAD_ARG, "treelstm_create: workspace must be 256-byte aligned");
  auto* e = new cavs_treelstm();
  InitModes(e, *cfg);
  const size_t need = Carve(e, workspace);
  if (need > workspace_bytes) {
    delete e;
    return Fail(CAVS_ERR_CAPACITY, "treelstm_create: workspace needs " + std::to_string(need) + " bytes");
  }
  e->idx_ints = IdxInts(*cfg);
  if (e->bf16) {
    const long long N = cfg->max_vertices, H = cfg->hidden, K = cfg->n_slots;
    const uint8_t* Uf = e->U_bf + static_cast<size_t>(3) * H * H * 2;
    int rc = EncodeTcOperand(&e->map_S, e->S, N, H, H, 0, 128);
    if (!rc) rc = EncodeTcOperand(&e->map_HK, e->HK, N * K, H, H, 0, 128);
    if (!rc) rc = EncodeTcOperand(&e->map_dA3, e->dA, N, 3 * H, 4 * H, 0, 128);
    if (!rc) rc = EncodeTcOperand(&e->map_ZF, e->ZF, N * K, H, H, 0, 128);
    if (!rc) rc = EncodeTcOperand(&e->map_Uiou_mn, e->U_bf, 3 * H, H, 3 * H, 1, 0);                        // [k=H, n=3H]
    if (!rc) rc = EncodeTcOperand(&e->map_Uf_mn, Uf, H, H, H, 1, 0);                                       // [k=H, n=H]
    if (!rc) rc = EncodeTcOperand(&e->map_Uiou_k, e->U_bf, H, 3 * H, 3 * H, 0, GemmBf16TileN(static_cast<int>(H)));  // [n=H, k=3H]
    if (!rc) rc = EncodeTcOperand(&e->map_Uf_k, Uf, H, H, H, 0, GemmBf16TileN(static_cast<int>(H)));       // [n=H, k=H]
    if (!rc) rc = EncodeTcOperand(&e->map_Uiou_k64, e->U_bf, H, 3 * H, 3 * H, 0, 64);
    if (!rc) rc = EncodeTcOperand(&e->map_Uf_k64, Uf, H, H, H, 0, 64);
    const long long L = cfg->max_level_rows;
    if (!rc) rc = EncodeTcOutput(&e->map_P, e->P, L, 3 * H, 3 * H, true);
    if (!rc) rc = EncodeTcOutput(&e->map_Q, e->Q, L * K, H, H, true);
    if (!rc) rc = EncodeTcOutput(&e->map_ds, e->ds, L, H, H, false);
    if (!rc && e->gate_epi) rc = EncodeTcOutput(&e->map_G3, e->gates, N, 3 * H, 3 * H, true);      // fp16: 16-bit elements
    if (!rc && e->gate_epi) rc = EncodeTcOutput(&e->map_GF, e->gates_f, N * K, H, H, true);
    if (rc) { delete e; return rc; }
  }
  cudaError_t err = cudaHostAlloc(reinterpret_cast<void**>(&e->h_idx), 2 * e->idx_ints * sizeof(int32_t), cudaHostAllocDefault);
  if (err != cudaSuccess) {
    delete e;
    return Fail(CAVS_ERR_CUDA, std::string("treelstm_create: pinned staging: ") + cudaGetErrorString(err));
  }
  if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&e->copy_stream, cudaStreamNonBlocking);
  for (int i = 0; i < 2 && err == cudaSuccess; ++i) {
    err = cudaEventCreateWithFlags(&e->copied[i], cudaEventDisableTiming);
    if (err == cudaSuccess) err = cudaEventCreateWithFlags(&e->slot_done[i], cudaEventDisableTiming);
  }
  if (err == cudaSuccess) err = cudaEventCreateWithFlags(&e->emb_ready, cudaEventDisableTiming);
  if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&e->comm_stream, cudaStreamNonBlocking);
  if (err == cudaSuccess) err = cudaEventCreateWithFlags(&e->comm_done, cudaEventDisableTiming);
  if (err == cudaSuccess) err = cudaMemset(e->tail, 0, 4 * sizeof(float));
  if (err != cudaSuccess) {
    cudaFreeHost(e->h_idx);
    delete e;
    return Fail(CAVS_ERR_CUDA, std::string("treelstm_create: ") + cudaGetErrorString(err));
  }
  *out = e;
  return CAVS_OK;
}

extern "C" void cavs_treelstm_destroy(cavs_treelstm* e) {
  if (!e) return;
  if (e->stager) {
    {
      std::lock_guard<std::mutex> lock(e->stager->mu);
      e->stager->quit = true;
    }
    e->stager->cv.notify_all();
    if (e->stager->thread.joinable()) e->stager->thread.join();
    delete e->stager;
  }
  if (e->h_idx) cudaFreeHost(e->h_idx);
  for (cudaEvent_t ev : e->ev_pool) cudaEventDestroy(ev);
  for (int i = 0; i < 2; ++i) {
    if (e->copied[i]) cudaEventDestroy(e->copied[i]);
    if (e->slot_done[i]) cudaEventDestroy(e->slot_done[i]);
  }
  if (e->emb_ready) cudaEventDestroy(e->emb_ready);
  if (e->comm_done) cudaEventDestroy(e->comm_done);
  if (e->comm_stream) cudaStreamDestroy(e->comm_stream);
  if (e->copy_stream) cudaStreamDestroy(e->copy_stream);
  delete e;
}

extern "C" int cavs_treelstm_bind(cavs_treelstm* e, float* params, float* grads) {
  CAVS_REQUIRE(e && params && grads, CAVS_ERR_BAD_ARG, "treelstm_bind: null pointer");
  CAVS_REQUIRE(((reinterpret_cast<uintptr_t>(params) | reinterpret_cast<uintptr_t>(grads)) & 15u) == 0, CAVS_ERR_BAD_ARG,
               "treelstm_bind: buffers must be 16-byte aligned");
  e->params = params;
  e->grads = grads;
  return CAVS_OK;
}

extern "C" int cavs_treelstm_refresh_weights(cavs_treelstm* e, void* stream) {
  CAVS_REQUIRE(e && e->params, CAVS_ERR_BAD_ARG, "treelstm_refresh_weights: parameters not bound");
  if (!e->bf16) return CAVS_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t H = e->cfg.hidden, E = e->cfg.embed;
  // W and U are adjacent in the flat buffer, and so are their bf16 shadows only logically;
  // cast them separately into their own 16-byte aligned arrays.
  if (int rc = LaunchCastBf16(e->W_bf, e->params + e->OffW(), E * 4 * H, st)) return rc;
  if (e->WideHead())
    if (int rc = LaunchCastBf16(e->Wc_bf, e->params + e->OffWc(), static_cast<size_t>(e->cfg.classes) * H, st)) return rc;
  return LaunchCastBf16(e->U_bf, e->params + e->OffU(), 4 * H * H, st);
}

extern "C" int cavs_treelstm_set_exchange_rows(cavs_treelstm* e, const int32_t* rows, int n_rows) {
  CAVS_REQUIRE(e && n_rows >= 0 && (rows || n_rows == 0), CAVS_ERR_BAD_ARG, "treelstm_set_exchange_rows: bad arguments");
  CAVS_REQUIRE(!e->Dense(), CAVS_ERR_BAD_ARG, "treelstm_set_exchange_rows: the engine has no embedding table");
  if (int rc = cavs_treelstm_stage_wait(e)) return rc;   // the helper thread may be reading the previous list
  CAVS_REQUIRE(n_rows <= e->cfg.vocab, CAVS_ERR_BAD_ARG, "treelstm_set_exchange_rows: more rows than the table has");
  CAVS_REQUIRE(e->cfg.embed % 4 == 0, CAVS_ERR_UNSUPPORTED, "treelstm_set_exchange_rows: embedding width must be a multiple of 4");
  for (int i = 0; i < n_rows; ++i)
    CAVS_REQUIRE(rows[i] >= 0 && rows[i] < e->cfg.vocab && (i == 0 || rows[i] > rows[i - 1]), CAVS_ERR_BAD_ARG,
                 "treelstm_set_exchange_rows: rows must be table indices in strictly ascending order");
  e->pending_xrows.assign(rows, rows + n_rows);
  return CAVS_OK;
}

extern "C" int cavs_treelstm_load_batch(cavs_treelstm* e, const cavs_sched* s, const int32_t* tok_job,
                                        const int32_t* label_job, int loss_rows, void* stream) {
  CAVS_REQUIRE(e && s && s->loaded, CAVS_ERR_BAD_ARG, "treelstm_load_batch: null pointer or empty schedule");
  CAVS_REQUIRE((tok_job || e->Dense()) && (label_job || e->Headless()), CAVS_ERR_BAD_ARG,
               "treelstm_load_batch: tokens are required with an embedding table, labels with a loss head");
  const LevelSchedule& sch = s->impl;
  const int n = sch.n_scheduled(), nt = sch.n_total(), K = e->cfg.n_slots;
  CAVS_REQUIRE(sch.n_slots() == K, CAVS_ERR_BAD_ARG, "treelstm_load_batch: schedule was built with a different slot count");
  CAVS_REQUIRE(nt <= e->cfg.max_vertices, CAVS_ERR_CAPACITY,
               "treelstm_load_batch: batch has " + std::to_string(nt) + " vertices, capacity " + std::to_string(e->cfg.max_vertices));
  CAVS_REQUIRE(sch.max_level_rows() <= e->cfg.max_level_rows, CAVS_ERR_CAPACITY,
               "treelstm_load_batch: widest level has " + std::to_string(sch.max_level_rows()) + " rows, capacity " +
                   std::to_string(e->cfg.max_level_rows));
  const int which = e->active < 0 ? 0 : 1 - e->active;
  cavs_treelstm::Batch& bt = e->slot[which];
  // The pinned half of this slot is free once its previous upload has finished.
  CAVS_CUDA(cudaEventSynchronize(e->copied[which]));
  bt.n = n; bt.n_total = nt; bt.n_levels = sch.n_levels();
  bt.loss_rows = loss_rows > 0 ? loss_rows : std::max(n, 1);
  bt.level_off = sch.level_off();

  // Pack the blob: child | parent | tok | label | order | chunk_off | seg_first_chunk | seg_tok.
  int32_t* h = e->h_idx + static_cast<size_t>(which) * e->idx_ints;
  int32_t* d = e->d_idx + static_cast<size_t>(which) * e->idx_ints;
  size_t o = 0;
  auto view = [&](size_t count, int32_t** dev) { int32_t* p = h + o; *dev = d + o; o += count; return p; };
  int32_t* h_child = view(static_cast<size_t>(K) * nt, &bt.child);
  int32_t* h_parent = view(nt, &bt.parent);
  int32_t* h_tok = view(nt, &bt.tok);
  int32_t* h_label = view(nt, &bt.label);
  int32_t* h_order = view(nt, &bt.order);
  int32_t* h_slot = view(nt, &bt.tok_slot);
  int32_t* h_child_st = e->leaf_tok ? view(static_cast<size_t>(K) * nt, &bt.child_st) : nullptr;
  int32_t* h_state_row = e->leaf_tok ? view(nt, &bt.state_row) : nullptr;
  const int32_t* t2j = sch.t2j().data();
  const int V = e->cfg.vocab;
  {
    const int32_t* src_child = sch.child_t().data();
    const int32_t* src_parent = sch.parent_t().data();
    // Pull (op_impl_graphop.cu:214-254) and the label permutation FunctionPopRet implies
    // (:275-327) are folded into this host-side reorder to tensor-id order.
    ParallelRanges(nt, [=](int b0, int b1) {
      for (int c = 0; c < K; ++c)
        std::memcpy(h_child + static_cast<size_t>(c) * nt + b0, src_child + static_cast<size_t>(c) * nt + b0, sizeof(int32_t) * (b1 - b0));
      std::memcpy(h_parent + b0, src_parent + b0, sizeof(int32_t) * (b1 - b0));
      for (int t = b0; t < std::min(b1, n); ++t) {
        const int id = tok_job ? tok_job[t2j[t]] : 0;
        h_tok[t] = (id < 0 || id >= V) ? 0 : id;
        h_label[t] = label_job ? label_job[t2j[t]] : -1;
      }
    });
  }
  int n_seg = 0, n_chunks = 0;
  if (e->Dense()) {
    // Dense inputs: one projection row per vertex, no token grouping.
    bt.chunk_off = bt.seg_first_chunk = bt.seg_tok = bt.chunk_out = bt.multi_seg = nullptr;
    bt.n_multi = 0;
    bt.shared_chunk = -1;
    bt.tok_slot = nullptr;
    n_seg = n;
    CAVS_REQUIRE(o <= e->idx_ints, CAVS_ERR_CAPACITY, "treelstm_load_batch: index blob overflow");
  } else {
    // Stable counting sort of rows by token -> segments and chunks for the per-token gradient sums.  Within a
    // token the rows are in tensor-id order, so its leaves (level 0) come first; leaves and internal vertices get
    // separate chunks.
    const int n_leaf = sch.n_levels() > 0 ? bt.level_off[1] : 0;
    // When every internal vertex carries the same token (the reference's zero-filled inputs: only leaves have
    // words) and the backward cell keeps per-CTA column sums, the sum of dA over the internal vertices is exactly
    // those column sums: the internal rows are left out of the lists below, and the token gets one extra, empty
    // chunk whose partial row backward fills from the column sums.
    int shared_tok = -1;
    if (e->TokGrad() && CellBwdFusesBias(e->cfg.hidden) && n > n_leaf) {
      shared_tok = h_tok[n_leaf];
      for (int t = n_leaf + 1; t < n && shared_tok >= 0; ++t)
        if (h_tok[t] != shared_tok) shared_tok = -1;
    }
    const int n_listed = shared_tok >= 0 ? n_leaf : n;   // rows that appear in `order`
    e->bucket.assign(static_cast<size_t>(V) + 1, 0);
    e->leaf_count.assign(static_cast<size_t>(V), 0);
    for (int t = 0; t < n_listed; ++t) ++e->bucket[h_tok[t] + 1];
    for (int t = 0; t < n_leaf; ++t) ++e->leaf_count[h_tok[t]];
    auto chunks_of = [](int rows) { return (rows + kEmbedChunk - 1) / kEmbedChunk; };
    for (int v = 0; v < V; ++v) {
      const int cnt = e->bucket[v + 1];
      if (cnt || v == shared_tok) {
        ++n_seg;
        n_chunks += chunks_of(e->leaf_count[v]) + chunks_of(cnt - e->leaf_count[v]) + (v == shared_tok ? 1 : 0);
      }
      e->bucket[v + 1] += e->bucket[v];
    }
    int32_t* h_chunk_off = view(static_cast<size_t>(n_chunks) + 1, &bt.chunk_off);
    int32_t* h_seg_first = view(static_cast<size_t>(n_seg) + 1, &bt.seg_first_chunk);
    int32_t* h_seg_tok = view(n_seg, &bt.seg_tok);
    int32_t* h_chunk_out = view(static_cast<size_t>(n_chunks) + 1, &bt.chunk_out);
    int32_t* h_chunk_seg = view(static_cast<size_t>(n_chunks) + 1, &bt.chunk_seg);
    int32_t* h_multi = view(static_cast<size_t>(n_chunks) + 1, &bt.multi_seg);   // segments folded by the second pass
    CAVS_REQUIRE(o <= e->idx_ints, CAVS_ERR_CAPACITY, "treelstm_load_batch: index blob overflow");
    int si = 0, ci = 0, n_multi = 0;
    bt.shared_chunk = -1;
    e->slot_of_token.resize(V);
    for (int v = 0; v < V; ++v) {
      const int b0 = e->bucket[v], b1 = e->bucket[v + 1];
      if (b0 == b1 && v != shared_tok) continue;
      e->slot_of_token[v] = si;
      h_seg_tok[si] = v;
      h_seg_first[si] = ci;
      const int mid = b0 + e->leaf_count[v];                    // leaves [b0, mid), internal vertices [mid, b1)
      // a token whose rows form one chunk gets its sum written by the first pass of the segmented sums
      const bool single = v != shared_tok && chunks_of(mid - b0) + chunks_of(b1 - mid) == 1;
      if (!single) h_multi[n_multi++] = si;
      for (int part = 0; part < 2; ++part)
        for (int b = part ? mid : b0; b < (part ? b1 : mid); b += kEmbedChunk) {
          h_chunk_out[ci] = single ? si : -1;
          h_chunk_seg[ci] = si;
          h_chunk_off[ci++] = b;
        }
      if (v == shared_tok) {   // the empty chunk that receives the internal vertices' column sums
        bt.shared_chunk = ci;
        h_chunk_out[ci] = -1;
        h_chunk_seg[ci] = si;
        h_chunk_off[ci++] = b1;
      }
      ++si;
    }
    h_seg_first[si] = ci;
    h_chunk_off[ci] = n_listed;
    bt.n_multi = n_multi;
    for (int t = 0; t < n_listed; ++t) h_order[e->bucket[h_tok[t]]++] = t;   // bucket[v] advances to bucket end
    {
      const int32_t* slot_of = e->slot_of_token.data();
      ParallelRanges(n, [=](int b0, int b1) { for (int t = b0; t < b1; ++t) h_slot[t] = slot_of[h_tok[t]]; });
    }
  }
  if (e->leaf_tok) {
    // State rows: a leaf (level 0) lives in its token's row behind the vertex rows, every other vertex in its own.
    const int n_leaf = sch.n_levels() > 0 ? bt.level_off[1] : 0;
    const int base = e->cfg.max_vertices;
    ParallelRanges(nt, [=](int b0, int b1) { for (int t = b0; t < b1; ++t) h_state_row[t] = t < n_leaf ? base + h_slot[t] : t; });
    ParallelRanges(nt, [=](int b0, int b1) {
      for (int c = 0; c < K; ++c)
        for (size_t i = static_cast<size_t>(c) * nt + b0, end = static_cast<size_t>(c) * nt + b1; i < end; ++i) {
          const int ch = h_child[i];
          h_child_st[i] = ch >= 0 ? h_state_row[ch] : ch;
        }
    });
  }
  if (e->TokHead()) {
    // Loss rows: the internal vertices in tensor-id order, then one row per distinct token standing for its leaves.
    const int n_leaf = sch.n_levels() > 0 ? bt.level_off[1] : 0;
    int32_t* h_hist = view(static_cast<size_t>(n_seg) * kHeadDzPitch, &bt.tok_hist);
    int32_t* h_head_row = view(static_cast<size_t>(n - n_leaf) + n_seg, &bt.head_row);
    CAVS_REQUIRE(o <= e->idx_ints, CAVS_ERR_CAPACITY, "treelstm_load_batch: index blob overflow");
    std::memset(h_hist, 0, sizeof(int32_t) * n_seg * kHeadDzPitch);
    for (int t = 0; t < n_leaf; ++t) {
      const int y = h_label[t];
      if (y >= 0 && y < e->cfg.classes) ++h_hist[static_cast<size_t>(h_slot[t]) * kHeadDzPitch + y];
    }
    for (int t = n_leaf; t < n; ++t) h_head_row[t - n_leaf] = t;
    for (int sidx = 0; sidx < n_seg; ++sidx) h_head_row[n - n_leaf + sidx] = e->cfg.max_vertices + sidx;
  }
  bt.l1 = e->l1_tok && sch.n_levels() >= 2 &&
          (e->l1_always || static_cast<long long>(bt.level_off[2] - bt.level_off[1]) >= 2LL * n_seg);
  bt.n_l_chunks = bt.n_l_multi = bt.n_links = 0;
  if (bt.l1) {
    // Links of level 1 grouped by the token row of the child (stable counting sort: within a token, links stay in
    // (vertex, slot) order), cut into chunks of kEmbedChunk; and the leaves below level 1 marked in `order`: their
    // d(h) arrives per token, the h half of their mailbox rows is never written.
    const int off1 = bt.level_off[1], off2 = bt.level_off[2];
    e->link_bucket.assign(static_cast<size_t>(n_seg) + 1, 0);
    for (int t = off1; t < off2; ++t)
      for (int c = 0; c < K; ++c) {
        const int ch = h_child[static_cast<size_t>(c) * nt + t];
        if (ch >= 0) ++e->link_bucket[h_slot[ch] + 1];
      }
    int n_lc = 0, n_lm = 0;
    for (int sidx = 0; sidx < n_seg; ++sidx) n_lc += (e->link_bucket[sidx + 1] + kEmbedChunk - 1) / kEmbedChunk;
    int32_t* h_l_order = view(static_cast<size_t>(K) * (off2 - off1), &bt.l_order);
    int32_t* h_l_chunk_off = view(static_cast<size_t>(n_lc) + 1, &bt.l_chunk_off);
    int32_t* h_l_chunk_out = view(static_cast<size_t>(n_lc) + 1, &bt.l_chunk_out);
    int32_t* h_l_seg_first = view(static_cast<size_t>(n_seg) + 1, &bt.l_seg_first);
    int32_t* h_l_multi = view(static_cast<size_t>(n_seg) + 1, &bt.l_multi);
    CAVS_REQUIRE(o <= e->idx_ints, CAVS_ERR_CAPACITY, "treelstm_load_batch: index blob overflow");
    int ci = 0, pos = 0;
    for (int sidx = 0; sidx < n_seg; ++sidx) {
      const int cnt = e->link_bucket[sidx + 1];
      const int chunks = (cnt + kEmbedChunk - 1) / kEmbedChunk;
      h_l_seg_first[sidx] = ci;
      if (chunks > 1) h_l_multi[n_lm++] = sidx;
      for (int b = 0; b < chunks; ++b) {
        h_l_chunk_out[ci] = chunks == 1 ? sidx : -1;
        h_l_chunk_off[ci++] = pos + b * kEmbedChunk;
      }
      e->link_bucket[sidx + 1] = pos;   // becomes the running write position of token row sidx
      pos += cnt;
    }
    h_l_seg_first[n_seg] = ci;
    h_l_chunk_off[ci] = pos;
    for (int t = off1; t < off2; ++t)
      for (int c = 0; c < K; ++c) {
        const int ch = h_child[static_cast<size_t>(c) * nt + t];
        if (ch >= 0) h_l_order[e->link_bucket[h_slot[ch] + 1]++] = t * K + c;
      }
    bt.n_l_chunks = n_lc; bt.n_l_multi = n_lm; bt.n_links = pos;
    const int n_leaf = bt.level_off[1];
    // `order` holds every leaf, and the internal vertices too unless they all share one token
    ParallelRanges(bt.shared_chunk >= 0 ? n_leaf : n, [=](int b0, int b1) {
      for (int i = b0; i < b1; ++i) {
        const int t = h_order[i];
        if (t < n_leaf && h_parent[t] >= off1 && h_parent[t] < off2) h_order[i] = t | kOrderNoDh;
      }
    });
  }
  bt.n_seg = n_seg; bt.n_chunks = n_chunks;
  // Exchange rows given for this batch: every token segment's position in the list (both ascending: one merge).
  bt.n_xrows = 0;
  bt.xrows = bt.seg_pos = nullptr;
  if (!e->pending_xrows.empty()) {
    std::vector<int32_t> rows;
    rows.swap(e->pending_xrows);          // consumed by this load, whatever its outcome
    CAVS_REQUIRE(!e->Dense(), CAVS_ERR_BAD_ARG, "treelstm_load_batch: exchange rows need an embedding table");
    const int U = static_cast<int>(rows.size());
    int32_t* h_xrows = view(U, &bt.xrows);
    int32_t* h_seg_pos = view(n_seg, &bt.seg_pos);
    CAVS_REQUIRE(o <= e->idx_ints, CAVS_ERR_CAPACITY, "treelstm_load_batch: index blob overflow");
    std::memcpy(h_xrows, rows.data(), sizeof(int32_t) * U);
    const int32_t* h_seg_tok_c = h + (bt.seg_tok - d);
    int pos = 0;
    for (int si = 0; si < n_seg; ++si) {
      while (pos < U && rows[pos] < h_seg_tok_c[si]) ++pos;
      CAVS_REQUIRE(pos < U && rows[pos] == h_seg_tok_c[si], CAVS_ERR_BAD_ARG,
                   "treelstm_load_batch: token " + std::to_string(h_seg_tok_c[si]) + " of the batch is not among the exchange rows");
      h_seg_pos[si] = pos;
    }
    bt.n_xrows = U;
  }
  // The device half is free once the last pass that read it has finished.
  (void)stream;
  if (e->slot_used[which]) CAVS_CUDA(cudaStreamWaitEvent(e->copy_stream, e->slot_done[which], 0));
  CAVS_CUDA(cudaMemcpyAsync(d, h, o * sizeof(int32_t), cudaMemcpyHostToDevice, e->copy_stream));
  CAVS_CUDA(cudaEventRecord(e->copied[which], e->copy_stream));
  e->staged = which;
  e->last_upload_bytes = o * sizeof(int32_t);
  return CAVS_OK;
}

namespace {
// Joins a staging request in flight and makes the staged batch (if any) the current one.
int PromoteStaged(cavs_treelstm* e, cudaStream_t st) {
  if (int rc = cavs_treelstm_stage_wait(e)) return rc;
  if (e->staged >= 0) {
    e->active = e->staged;
    e->staged = -1;
    CAVS_CUDA(cudaStreamWaitEvent(st, e->copied[e->active], 0));   // tables of this batch are in place
  }
  return CAVS_OK;
}
}  // namespace

extern "C" int cavs_treelstm_promote(cavs_treelstm* e, void* stream) {
  CAVS_REQUIRE(e, CAVS_ERR_BAD_ARG, "treelstm_promote: null handle");
  e->explicit_promote = true;
  return PromoteStaged(e, static_cast<cudaStream_t>(stream));
}

extern "C" int cavs_treelstm_forward(cavs_treelstm* e, void* stream) {
  CAVS_REQUIRE(e && e->params, CAVS_ERR_BAD_ARG, "treelstm_forward: parameters not bound");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Without explicit promotion the pass takes the staged batch itself, after joining a request still on the helper
  // thread; a caller that promotes explicitly may have the batch after this one on the helper thread right now.
  if (!e->explicit_promote)
    if (int rc = PromoteStaged(e, st)) return rc;
  CAVS_REQUIRE(e->active >= 0, CAVS_ERR_BAD_ARG, "treelstm_forward: no batch loaded");
  const cavs_treelstm::Batch& bt = e->slot[e->active];
  const int n = bt.n, nt = bt.n_total, H = e->cfg.hidden, E = e->cfg.embed, K = e->cfg.n_slots;
  if (n == 0) return CAVS_OK;
  const float* Emb = e->params;
  const uint8_t* W = e->bf16 ? e->W_bf : reinterpret_cast<const uint8_t*>(e->params + e->OffW());
  const uint8_t* U = e->bf16 ? e->U_bf : reinterpret_cast<const uint8_t*>(e->params + e->OffU());
  const void* U_iou = U;
  const void* U_f = U + static_cast<size_t>(3) * H * H * e->elt;
  const float* B = e->params + e->OffB();
  int rc;
  const double elt = static_cast<double>(e->elt);
  const int n_tok = bt.n_seg;        // distinct tokens of the batch
  ChainHint(false);
  const int pre = e->bf16 ? 2 : 0;   // pre-activations are stored in the GEMM operand precision
  const void* Xop = e->X;
  long long ldx = E;
  if (e->Dense()) {
    // Dense inputs (a stacked layer): one projection row per vertex, A = x.W over all rows.
    CAVS_REQUIRE(e->x_dense, CAVS_ERR_BAD_ARG, "treelstm_forward: dense inputs not set (cavs_treelstm_set_dense_input)");
    if (e->bf16) {
      if ((rc = LaunchCastRowsBf16(e->X, e->x_dense, n, E, e->x_pitch, st))) return rc;
    } else {
      Xop = e->x_dense; ldx = e->x_pitch;
    }
  } else {
    // X = Emb[distinct tokens]; A = X.W: one row per token, shared by every vertex carrying it.
    PROF(e, kProfEmbedFwd, static_cast<double>(n_tok) * (4 + 4.0 * E + elt * E), st,
         LaunchEmbedFwd(e->X, e->bf16, Emb, bt.seg_tok, n_tok, E, e->cfg.vocab, st));
  }
  if ((rc = Gemm(e, e->A, 4 * H, pre, Xop, ldx, false, W, 4 * H, false, n_tok, 4 * H, E, false, st))) return rc;
  for (int l = 0; l < bt.n_levels; ++l) {
    const int off = bt.level_off[l], rows = bt.level_off[l + 1] - off;
    if (l == 0) {
      // leaf rows: read the token row's i,o,u blocks (3H) + its index, write h|c (2H); the gates are recomputed by
      // the backward pass, not stored
      PROF(e, kProfCellFwd, static_cast<double>(e->leaf_tok ? n_tok : rows) * (H * (elt * 3 + 4.0 * 2) + 4), st,
           e->leaf_tok
               // one state row per distinct token (row s of A -> row max_vertices + s of state), not per leaf
               ? LaunchCellFwd(e->state + static_cast<size_t>(e->cfg.max_vertices) * 2 * H, e->gates, e->A, nullptr, nullptr, e->bf16,
                               B, bt.child, nullptr, n_tok, 0, n_tok, H, K, true, st, false)
               : LaunchCellFwd(e->state, e->gates, e->A, nullptr, nullptr, e->bf16, B, bt.child, bt.tok_slot, nt, off, rows, H, K,
                               true, st, false));
      if (bt.l1) {
        // h_tok.U_iou | h_tok.U_f, one row per distinct leaf token: everything level 1 needs from the recurrent weights
        float* h_tok = e->state + static_cast<size_t>(e->cfg.max_vertices) * 2 * H;
        if ((rc = LaunchCastRowsBf16(e->htok_bf, h_tok, n_tok, H, 2 * H, st))) return rc;
        if ((rc = Gemm(e, e->PQT, 4 * H, pre, e->htok_bf, H, false, U_iou, 3 * H, false, n_tok, 3 * H, H, false, st))) return rc;
        if ((rc = Gemm(e, e->PQT + static_cast<size_t>(3) * H * e->elt, 4 * H, pre, e->htok_bf, H, false, U_f, H, false, n_tok, H, H, false, st)))
          return rc;
      }
      continue;
    }
    if (l == 1 && bt.l1) {
      // no gather, no per-row products: the cell reads its children's per-token product rows
      ChainHint(rows <= kChainSmallRows);
      PROF(e, kProfCellFwd, static_cast<double>(rows) * (H * (elt * (4 + 4 * K + 3 + K) + 4.0 * (K + 2)) + 4), st,
           LaunchCellFwd(e->state, e->gates, e->A, e->PQT, nullptr, e->bf16, B, bt.child_st, bt.tok_slot, nt, off, rows, H, K, false, st,
                         true, e->cfg.max_vertices, e->gates_f, e->Status()));
      continue;
    }
    // Chained launches: a kernel releases its successor early when that successor is a GEMM (one CTA per
    // SM) or the level is small enough that placement does not matter.
    const bool small = rows <= kChainSmallRows;
    ChainHint(true);       // gather -> P GEMM -> Q GEMM
    // read K child h rows (fp32) + K indices, write S and HK
    PROF(e, kProfGatherH, static_cast<double>(rows) * (4.0 * K * H + 4.0 * K + elt * (1 + K) * H), st,
         LaunchGatherChildH(e->S, e->HK, e->bf16, e->state, e->leaf_tok ? bt.child_st : bt.child, nt, off, rows, H, K, st));
    if (e->gate_epi) {
      // The two gate products finish the gates in their epilogues: G3[t] = act((S.U_iou + A[row(t), :3H]) + b),
      // GF[t,c] = sigmoid((HK[t,c].U_f + A[row(t), 3H:]) + b_f); the cell then reads them back once.
      GemmBf16MappedArgs gp[2];
      for (int part = 0; part < 2; ++part) {
        GemmBf16MappedArgs& ga = gp[part];
        ga.out_mode = 4;
        ga.a = part == 0 ? &e->map_S : &e->map_HK;
        ga.b = part == 0 ? &e->map_Uiou_mn : &e->map_Uf_mn;
        ga.a_row_off = part == 0 ? off : off * K;
        ga.c = part == 0 ? e->gates : e->gates_f;
        ga.ldc = part == 0 ? 3 * H : H;
        ga.c_map = part == 0 ? &e->map_G3 : &e->map_GF;
        ga.c_row_off = ga.a_row_off;
        ga.m = part == 0 ? rows : rows * K; ga.n = part == 0 ? 3 * H : H; ga.k = H;
        ga.status = e->Status();
        ga.act_a = e->A; ga.act_a_row = bt.tok_slot; ga.act_bias = B;
        ga.act_col0 = part == 0 ? 0 : 3 * H; ga.act_hidden = H; ga.act_rows_per_vertex = part == 0 ? 1 : K; ga.act_t_off = off;
      }
      // The two products go out as ONE launch: a small level pays launch and pipeline-fill latency once, a large one
      // has one partial last wave of tiles instead of two (measured at every size: 2.45 -> 2.41 ms for a 512-tree
      // shard against pairing only levels of up to three waves, 12.06 -> 12.02 ms for the 4096-tree batch).
      if (e->dual_gemm) {
        ChainHint(small);     // the launch is followed by the cell: a wide grid-stride kernel
        PROF(e, kProfGemm, 2.0 * gp[0].m * gp[0].n * gp[0].k + 2.0 * gp[1].m * gp[1].n * gp[1].k, st, GemmBf16MappedDual(gp[0], gp[1], st));
      } else {
        PROF(e, kProfGemm, 2.0 * gp[0].m * gp[0].n * gp[0].k, st, GemmBf16Mapped(gp[0], st));
        ChainHint(small);     // second product -> cell -> next level's gather: wide grid-stride kernels
        PROF(e, kProfGemm, 2.0 * gp[1].m * gp[1].n * gp[1].k, st, GemmBf16Mapped(gp[1], st));
      }
      // read the finished gates ((3+K)H fp16) and child c (KH); write h|c (2H)
      PROF(e, kProfCellFwd, static_cast<double>(rows) * (H * (2.0 * (3 + K) + 4.0 * (K + 2))), st,
           LaunchCellFwdGated(e->state, e->gates, e->gates_f, e->leaf_tok ? bt.child_st : bt.child, nt, off, rows, H, K, st));
      continue;
    }
    const uint8_t* S_l = e->S + static_cast<size_t>(off) * H * e->elt;
    const uint8_t* HK_l = e->HK + static_cast<size_t>(off) * K * H * e->elt;
    if ((rc = Gemm(e, e->P, 3 * H, pre, S_l, H, false, U_iou, 3 * H, false, rows, 3 * H, H, false, st, &e->map_S, off, &e->map_Uiou_mn, &e->map_P))) return rc;
    ChainHint(small);      // Q GEMM -> cell -> next level's gather: wide grid-stride kernels
    if ((rc = Gemm(e, e->Q, H, pre, HK_l, H, false, U_f, H, false, rows * K, H, H, false, st, &e->map_HK, off * K, &e->map_Uf_mn, &e->map_Q))) return rc;
    // read the token row (4H) + index, P (3H), Q (KH), child c (KH); write gates ((3+K)H), h|c (2H)
    PROF(e, kProfCellFwd, static_cast<double>(rows) * (H * (elt * (4 + 3 + K + 3 + K) + 4.0 * (K + 2)) + 4), st,
         LaunchCellFwd(e->state, e->gates, e->A, e->P, e->Q, e->bf16, B, e->leaf_tok ? bt.child_st : bt.child, bt.tok_slot, nt, off, rows,
                       H, K, false, st));
  }
  ChainHint(false);
  (void)rc;
  // a forward-only caller may load the batch after next into this slot without ever running backward
  CAVS_CUDA(cudaEventRecord(e->slot_done[e->active], st));
  e->slot_used[e->active] = true;
  return CAVS_OK;
}

extern "C" int cavs_treelstm_backward(cavs_treelstm* e, void* stream) {
  CAVS_REQUIRE(e && e->params && e->grads, CAVS_ERR_BAD_ARG, "treelstm_backward: parameters / gradients not bound");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CAVS_REQUIRE(e->active >= 0, CAVS_ERR_BAD_ARG, "treelstm_backward: no batch loaded");
  const cavs_treelstm::Batch& bt = e->slot[e->active];
  const int n = bt.n, nt = bt.n_total, H = e->cfg.hidden, E = e->cfg.embed, K = e->cfg.n_slots, C = e->cfg.classes;
  float* g = e->grads;
  if (n == 0) {
    CAVS_CUDA(cudaMemsetAsync(g, 0, e->ParamCount() * sizeof(float), st));
    CAVS_CUDA(cudaEventRecord(e->emb_ready, st));
    return CAVS_OK;
  }
  const uint8_t* W = e->bf16 ? e->W_bf : reinterpret_cast<const uint8_t*>(e->params + e->OffW());
  const uint8_t* U = e->bf16 ? e->U_bf : reinterpret_cast<const uint8_t*>(e->params + e->OffU());
  const void* U_iou = U;
  const void* U_f = U + static_cast<size_t>(3) * H * H * e->elt;
  int rc;
  const double elt = static_cast<double>(e->elt);
  ChainHint(false);
  if (e->Headless()) {
    // No loss head: d(h) of every vertex comes from the layer above.
    CAVS_REQUIRE(e->dh_ext, CAVS_ERR_BAD_ARG, "treelstm_backward: output gradient not set (cavs_treelstm_set_output_grad)");
    CAVS_CUDA(cudaMemsetAsync(e->tail, 0, sizeof(float), st));
    CAVS_CUDA(cudaMemsetAsync(e->loss, 0, static_cast<size_t>(n) * sizeof(float), st));
  } else if (!e->WideHead()) {
    // Fused loss head over the pushed rows (h part of the state), in tensor-id order: read h (H), label,
    // write loss and the d(logits) row; d(h) = dz Wc is rebuilt inside the cell gradient, never stored.
    const bool fdh = e->FusedDh();
    if (e->TokHead()) {
      // internal vertices one by one, leaves once per distinct token
      const int n_leaf = bt.n_levels > 0 ? bt.level_off[1] : 0;
      const int rows_v = n - n_leaf, rows = rows_v + bt.n_seg;
      LossTokenRows tr;
      tr.hist = bt.tok_hist; tr.ptok = e->ptok; tr.rows_v = rows_v;
      PROF(e, kProfLossHead, static_cast<double>(rows) * (4.0 * H + 8 + 4.0 * kHeadDzPitch), st,
           LaunchLossHead(e->loss + n_leaf, e->tail, nullptr, g + e->OffWc(), g + e->Offbc(), e->state, 2 * H, bt.label + n_leaf,
                          e->params + e->OffWc(), e->params + e->Offbc(), rows, H, C, 1.0f / static_cast<float>(bt.loss_rows),
                          e->loss_scratch, st, false, e->dz8 + static_cast<size_t>(n_leaf) * kHeadDzPitch, e->Status(),
                          bt.head_row, tr));
    } else {
    PROF(e, kProfLossHead, static_cast<double>(n) * (4.0 * H + 8 + (fdh ? 4.0 * kHeadDzPitch : 4.0 * H)), st,
         LaunchLossHead(e->loss, e->tail, fdh ? nullptr : e->dOut, g + e->OffWc(), g + e->Offbc(), e->state, 2 * H, bt.label,
                        e->params + e->OffWc(), e->params + e->Offbc(), n, H, C, 1.0f / static_cast<float>(bt.loss_rows),
                        e->loss_scratch, st, false, fdh ? e->dz8 : nullptr, e->Status(), e->leaf_tok ? bt.state_row : nullptr));
    }
  } else {
    // Wide head (vocabulary-sized class count): logits = h Wc^T, row softmax cross-entropy, then
    // dH = dz Wc, dWc = dz^T h, dbc = column sums of dz -- FullyConnected + SoftmaxEntropyLoss and their
    // gradients (op_impl_fullyconnected_cublas.cc:33-176, op_impl_softmax_entropy_logits_loss.cu:106-250).
    const int Cp = e->Cp();
    const void* hA = e->state;      // h rows: fp32 view of the state with pitch 2H, or a dense bf16 copy
    long long ldh = 2 * H;
    const void* Wc = e->params + e->OffWc();
    if (e->bf16) {
      if ((rc = LaunchCastRowsBf16(e->h_bf, e->state, n, H, 2 * H, st))) return rc;
      hA = e->h_bf; ldh = H; Wc = e->Wc_bf;
    }
    if ((rc = Gemm(e, e->logits, Cp, 0, hA, ldh, false, Wc, H, true, n, C, H, false, st))) return rc;
    PROF(e, kProfLossHead, static_cast<double>(n) * (8.0 * C + 8), st,
         LaunchSoftmaxXentRows(e->loss, e->logits, e->bf16 ? e->dz_bf : nullptr, Cp, e->params + e->Offbc(), bt.label, n, C,
                               1.0f / static_cast<float>(bt.loss_rows), st));
    const void* dz = e->bf16 ? static_cast<const void*>(e->dz_bf) : e->logits;
    if ((rc = Gemm(e, e->dOut, H, 0, dz, Cp, false, Wc, H, false, n, H, C, false, st))) return rc;
    if ((rc = Gemm(e, g + e->OffWc(), H, 0, dz, Cp, true, hA, ldh, false, C, H, n, true, st))) return rc;
    if ((rc = LaunchColumnSum(g + e->Offbc(), e->logits, false, Cp, n, C, e->col_scratch, st))) return rc;
    if ((rc = LaunchColumnSum(e->tail, e->loss, false, 1, n, 1, e->col_scratch, st))) return rc;
  }
  // With token inputs (TokGrad) the leaf level has no backward cell launch of its own: its gate gradients are
  // formed inside the per-token sums below, and the bias gradient is the column sum of those sums' partials.
  const bool tok_grad = e->TokGrad();
  // The backward cell keeps per-CTA column sums of dA either for the bias gradient (no token sums) or, when all
  // internal vertices share one token, as that token's sum over the internal vertices.
  const bool fuse_bias = tok_grad ? bt.shared_chunk >= 0 : CellBwdFusesBias(H);
  const size_t dB_rows = static_cast<size_t>(CellBwdMaxGrid());
  if (fuse_bias) CAVS_CUDA(cudaMemsetAsync(e->dB_tmp, 0, dB_rows * 4 * H * sizeof(float), st));
  for (int l = bt.n_levels - 1; l >= (tok_grad ? 1 : 0); --l) {
    const int off = bt.level_off[l], rows = bt.level_off[l + 1] - off;
    // read d(h) (H; or the dz row with the fused head), mailbox (2H), gates, own c (H) [+ child c (KH)];
    // write dA (4H) [+ ZF (KH), child dc (KH)]
    const double dh_bytes = e->FusedDh() ? 4.0 * kHeadDzPitch : 4.0 * H;
    // leaves: mailbox (2H) and the token row's i,o,u blocks (3H) in, dA (4H) out
    const double cell_bytes = l == 0 ? rows * (H * (4.0 * 2 + elt * (3 + 4)) + dh_bytes + 4)
                                     : rows * (H * (4.0 * (2 + 1 + K + K) + elt * (3 + K + 4 + K)) + dh_bytes);
    ChainHint(l > 0);      // cell gradient -> ds GEMM -> dq GEMM
    PROF(e, kProfCellBwd, cell_bytes, st,
         LaunchCellBwd(e->dA, e->ZF, e->bf16, e->mailbox, fuse_bias ? e->dB_tmp : nullptr, e->FusedDh() ? nullptr : (e->Headless() ? e->dh_ext : e->dOut),
                       e->gates, e->state, bt.child, bt.parent, nt, off, rows, H, K, l == 0, st,
                       e->FusedDh() ? e->dz8 : nullptr, e->params + e->OffWc(), C, l == 0 ? e->A : nullptr,
                       l == 0 ? bt.tok_slot : nullptr, l == 0 ? e->params + e->OffB() : nullptr,
                       e->leaf_tok ? bt.child_st : nullptr, e->gates_f, e->Status()));
    if (l == 0) break;
    if (l == 1 && bt.l1) {
      // The children are leaves: what they receive is summed per token first (fixed order), and the two products
      // with the transposed recurrent weights run once per token.  dh_tok joins the leaves' other gradients inside
      // the per-token sums of the tail below.
      ChainHint(false);
      CAVS_CUDA(cudaMemsetAsync(e->ZT, 0, static_cast<size_t>(bt.n_seg) * 4 * H * e->elt, st));
      // each parent's i,o,u gradient row (3H) once, each link's forget-gate row (H) and index; per chunk 4H fp32 out, per
      // token 4H out
      PROF(e, kProfEmbedBwd,
           static_cast<double>(rows) * 3 * H * elt + static_cast<double>(bt.n_links) * (H * elt + 4) +
               static_cast<double>(bt.n_l_chunks) * 16.0 * H + static_cast<double>(bt.n_seg) * 4 * H * elt,
           st,
           LaunchLinkSumChunks(e->link_scratch, e->ZT, e->bf16, bt.l_chunk_out, e->dA, e->ZF, bt.l_order, bt.l_chunk_off, bt.n_l_chunks,
                               H, K, st));
      if ((rc = LaunchSegmentedRowSumFinal(e->ZT, e->bf16, e->link_scratch, bt.l_seg_first, bt.l_multi, bt.n_l_multi, 4 * H, st))) return rc;
      if ((rc = Gemm(e, e->dh_tok, H, 0, e->ZT, 4 * H, false, U_iou, 3 * H, true, bt.n_seg, H, 3 * H, false, st))) return rc;
      if ((rc = Gemm(e, e->dh_tok, H, 1, e->ZT + static_cast<size_t>(3) * H * e->elt, 4 * H, false, U_f, H, true, bt.n_seg, H, H, false, st)))
        return rc;
      continue;
    }
    const uint8_t* dA_l = e->dA + static_cast<size_t>(off) * 4 * H * e->elt;
    const uint8_t* ZF_l = e->ZF + static_cast<size_t>(off) * K * H * e->elt;
    // ds = dP U_iou^T, dq = Zf U_f^T  (dX = dY W^T, cavs/backend/op_decl_matmul.cc:21-31)
    // (Cutting a narrow level's ds product into K slices on more SMs, the partial products left unreduced for the dq
    // product's epilogue to add, was measured: 2.68 against 2.69 ms on a 512-tree shard -- not worth its code.)
    if ((rc = Gemm(e, e->ds, H, 0, dA_l, 4 * H, false, U_iou, 3 * H, true, rows, H, 3 * H, false, st, &e->map_dA3, off, &e->map_Uiou_k, &e->map_ds, &e->map_Uiou_k64))) return rc;
    ChainHint(rows <= kChainSmallRows);   // dq GEMM (-> scatter) -> next level's cell gradient
    if (e->bf16) {
      // dq = Zf U_f^T with the child-gradient scatter in its epilogue: row (t, c) of the product plus ds[t] goes
      // straight to the h half of mailbox[child_c(t)] (Scatter(Child=c), cavs/backend/op_decl_graphop.cc:25-41),
      // so dq is never stored and no separate scatter pass runs.  (Making the two products independent -- the
      // readers of a child's mailbox row adding their parent's ds row themselves -- so that they could share one
      // launch was measured: the extra gathered read per vertex cost more than the saved launch.)
      GemmBf16MappedArgs ga;
      ga.c = e->mailbox; ga.ldc = 2 * H; ga.out_mode = 3;
      ga.a = &e->map_ZF; ga.a_row_off = off * K; ga.b = &e->map_Uf_k; ga.b_small = &e->map_Uf_k64;
      ga.m = rows * K; ga.n = H; ga.k = H;
      ga.status = e->Status();
      ga.scatter_child = bt.child; ga.scatter_n_total = nt; ga.scatter_off = off; ga.scatter_slots = K;
      ga.scatter_addend = e->ds; ga.scatter_addend_ld = H;
      // work: the product's flops; the bytes the separate scatter used to move are no longer moved
      PROF(e, kProfGemm, 2.0 * rows * K * H * H, st, GemmBf16Mapped(ga, st));
    } else {
      if ((rc = Gemm(e, e->dq, H, 0, ZF_l, H, false, U_f, H, true, rows * K, H, H, false, st, &e->map_ZF, off * K, &e->map_Uf_k, nullptr, &e->map_Uf_k64))) return rc;
      PROF(e, kProfScatterGrad, static_cast<double>(rows) * (4.0 * H * (1 + K + K) + 4.0 * K), st,
           LaunchScatterChildGrad(e->mailbox, e->ds, e->dq, bt.child, nt, off, rows, H, K, st));
    }
  }
  ChainHint(false);
  // Deferred gradients, one pass per weight over all rows (cavs/midend/batch_weight_updater.h:10-85).  The
  // embedding gradient -- by far the largest block of the flat gradient buffer -- comes first and is
  // announced by an event, so a data-parallel caller can start reducing it across GPUs while the weight
  // gradients below are still being computed (cavs_treelstm_wait_embed_grad).
  // dA rows are first summed per distinct token (fixed order); dEmb[token] = dAtok W^T and dW = X^T dAtok
  // then run over tokens, not vertices.
  const int n_tok = bt.n_seg;
  if (e->Dense()) {
    // Dense inputs: d(x) = dA W^T for every vertex (the layer below takes it as its output gradient) and
    // dW = x^T dA over all rows.
    const void* Xop = e->bf16 ? static_cast<const void*>(e->X) : e->x_dense;
    const long long ldx = e->bf16 ? E : e->x_pitch;
    if ((rc = Gemm(e, e->dX, E, 0, e->dA, 4 * H, false, W, 4 * H, true, n, E, 4 * H, false, st))) return rc;
    CAVS_CUDA(cudaEventRecord(e->emb_ready, st));
    if ((rc = Gemm(e, g + e->OffW(), 4 * H, 0, Xop, ldx, true, e->dA, 4 * H, false, E, 4 * H, n, true, st))) return rc;
  } else {
    if (tok_grad) {
      const int n_leaf = bt.n_levels > 0 ? bt.level_off[1] : 0;
      const bool fdh = e->FusedDh();
      // leaves: mailbox (2H) + d(logits) row (or d(h)) in; internal rows: dA (4H) in; per chunk 4H fp32 out;
      // per token 4H out
      // (a leaf under level 1 by token has no d(h) half to read; with per-token loss rows no leaf reads a d(logits) row)
      const double leaf_head = e->TokHead() ? 0.0 : (fdh ? 4.0 * kHeadDzPitch : 4.0 * H);
      const double bytes = static_cast<double>(n_leaf - bt.n_links) * (4.0 * 2 * H + leaf_head + 4) +
                           static_cast<double>(bt.n_links) * (4.0 * H + leaf_head + 4) +
                           (bt.shared_chunk >= 0 ? 0.0 : static_cast<double>(n - n_leaf) * (4 + 4.0 * H * elt)) +
                           static_cast<double>(bt.n_chunks) * (16.0 * H + 3.0 * H * elt) + static_cast<double>(n_tok) * 4 * H * elt;
      PROF(e, kProfEmbedBwd, bytes, st,
           LaunchTokenGradChunks(e->emb_scratch, e->dAtok, e->bf16, bt.chunk_out, e->dA, e->A, bt.order, bt.chunk_off, bt.chunk_seg,
                                 bt.n_chunks, e->mailbox, fdh ? nullptr : (e->Headless() ? e->dh_ext : e->dOut),
                                 fdh ? e->dz8 : nullptr, e->params + e->OffWc(), C, e->params + e->OffB(), n_leaf, H, st,
                                 e->TokHead() ? e->ptok : nullptr, bt.tok_hist, 1.0f / static_cast<float>(bt.loss_rows),
                                 bt.l1 ? e->dh_tok : nullptr, bt.seg_first_chunk));
      if (bt.shared_chunk >= 0) {
        // the internal vertices' column sums become the partial row of their token's extra chunk
        if ((rc = LaunchColumnSum(e->emb_scratch + static_cast<size_t>(bt.shared_chunk) * 4 * H, e->dB_tmp, false, 4 * H,
                                  static_cast<int>(dB_rows), 4 * H, e->col_scratch, st)))
          return rc;
      }
      if ((rc = LaunchSegmentedRowSumFinal(e->dAtok, e->bf16, e->emb_scratch, bt.seg_first_chunk, bt.multi_seg, bt.n_multi, 4 * H, st)))
        return rc;
    } else {
      PROF(e, kProfEmbedBwd, static_cast<double>(n) * (4 + 4.0 * H * elt) + static_cast<double>(n_tok) * 4 * H * elt, st,
           LaunchSegmentedRowSum(e->dAtok, e->bf16, e->dA, e->bf16, 4 * H, 4 * H, bt.order, bt.chunk_off, bt.n_chunks,
                                 bt.seg_first_chunk, n_tok, e->emb_scratch, st, bt.chunk_out, bt.multi_seg, bt.n_multi));
    }
    if ((rc = Gemm(e, e->dX, E, 0, e->dAtok, 4 * H, false, W, 4 * H, true, n_tok, E, 4 * H, false, st))) return rc;
    // The embedding block of the gradient buffer: row v = d(Emb[v]) -- or, with exchange rows, row i = d(Emb[xrows[i]]):
    // only those rows are cleared, filled, exchanged between the ranks and applied.
    const bool compact = bt.n_xrows > 0;
    CAVS_CUDA(cudaMemsetAsync(g, 0, static_cast<size_t>(compact ? bt.n_xrows : e->cfg.vocab) * E * sizeof(float), st));
    if ((rc = cavs_scatter_rows(g, compact ? bt.seg_pos : bt.seg_tok, e->dX, n_tok, static_cast<size_t>(E) * sizeof(float), st))) return rc;
    CAVS_CUDA(cudaEventRecord(e->emb_ready, st));
    if ((rc = Gemm(e, g + e->OffW(), 4 * H, 0, e->X, E, true, e->dAtok, 4 * H, false, E, 4 * H, n_tok, true, st))) return rc;
  }
  // first row of the per-vertex weight-gradient products: the first internal row, or with level 1 by token the
  // first row of level 2
  const int off1 = bt.l1 ? (bt.n_levels > 2 ? bt.level_off[2] : n) : (bt.n_levels > 1 ? bt.level_off[1] : n);
  const int n_int = n - off1;
  float* dU = g + e->OffU();
  if (n_int > 0) {
    const uint8_t* S1 = e->S + static_cast<size_t>(off1) * H * e->elt;
    const uint8_t* dA1 = e->dA + static_cast<size_t>(off1) * 4 * H * e->elt;
    const uint8_t* HK1 = e->HK + static_cast<size_t>(off1) * K * H * e->elt;
    const uint8_t* ZF1 = e->ZF + static_cast<size_t>(off1) * K * H * e->elt;
    if ((rc = Gemm(e, dU, 3 * H, 0, S1, H, true, dA1, 4 * H, false, H, 3 * H, n_int, true, st))) return rc;
    if ((rc = Gemm(e, dU + static_cast<size_t>(3) * H * H, H, 0, HK1, H, true, ZF1, H, false, H, H, n_int * K, true, st))) return rc;
  } else {
    CAVS_CUDA(cudaMemsetAsync(dU, 0, static_cast<size_t>(4) * H * H * sizeof(float), st));
  }
  if (bt.l1) {
    // level 1's share: sum over links of h_child^T dz = sum over tokens of h_tok^T (the token's link sums)
    if ((rc = Gemm(e, dU, 3 * H, 1, e->htok_bf, H, true, e->ZT, 4 * H, false, H, 3 * H, bt.n_seg, true, st))) return rc;
    if ((rc = Gemm(e, dU + static_cast<size_t>(3) * H * H, H, 1, e->htok_bf, H, true, e->ZT + static_cast<size_t>(3) * H * e->elt, 4 * H, false,
                   H, H, bt.n_seg, true, st)))
      return rc;
  }
  // Bias gradient: column sums of dA, gate order i,o,u,f -> bias order i,f,u,o.
  if (tok_grad) {
    PROF(e, kProfColumnSum, static_cast<double>(bt.n_chunks) * 4 * H * 4, st,
         LaunchColumnSum(g + e->OffB(), e->emb_scratch, false, 4 * H, bt.n_chunks, 4 * H, e->col_scratch, st, H, 0, 3, 2, 1));
  } else if (fuse_bias) {   // no token sums: the column sums are the bias gradient
    PROF(e, kProfColumnSum, static_cast<double>(dB_rows) * 4 * H * 4, st,
         LaunchColumnSum(g + e->OffB(), e->dB_tmp, false, 4 * H, static_cast<int>(dB_rows), 4 * H, e->col_scratch, st, H, 0, 3, 2, 1));
  } else {
    PROF(e, kProfColumnSum, static_cast<double>(n) * 4 * H * elt, st,
         LaunchColumnSum(g + e->OffB(), e->dA, e->bf16, 4 * H, n, 4 * H, e->col_scratch, st, H, 0, 3, 2, 1));
  }
  (void)rc;
  CAVS_CUDA(cudaEventRecord(e->slot_done[e->active], st));
  e->slot_used[e->active] = true;
  return CAVS_OK;
}

extern "C" int cavs_treelstm_stage(cavs_treelstm* e, cavs_sched* s, const int32_t* parents, int batch, int max_len,
                                   const int32_t* tok_job, const int32_t* label_job, int loss_rows) {
  CAVS_REQUIRE(e && s, CAVS_ERR_BAD_ARG, "treelstm_stage: null handle");
  // parents == NULL: `s` already holds the batch's schedule (the caller ran cavs_sched_load itself, e.g. on a thread
  // of its own beside the packing of the previous batch); only the tables are packed and uploaded
  if (parents != nullptr)
    if (int rc = cavs_sched_load(s, parents, batch, max_len, e->cfg.n_slots)) return rc;
  return cavs_treelstm_load_batch(e, s, tok_job, label_job, loss_rows, nullptr);
}

extern "C" int cavs_treelstm_stage_async(cavs_treelstm* e, cavs_sched* s, const int32_t* parents, int batch, int max_len,
                                         const int32_t* tok_job, const int32_t* label_job, int loss_rows) {
  CAVS_REQUIRE(e && s, CAVS_ERR_BAD_ARG, "treelstm_stage_async: null handle");
  if (int rc = cavs_treelstm_stage_wait(e)) return rc;   // one request at a time
  if (e->stager == nullptr) {
    e->stager = new cavs_treelstm::Stager();
    CAVS_CUDA(cudaGetDevice(&e->stager->device));
    cavs_treelstm::Stager* w = e->stager;
    w->thread = std::thread([e, w] {
      cudaSetDevice(w->device);
      std::unique_lock<std::mutex> lock(w->mu);
      for (;;) {
        w->cv.wait(lock, [w] { return w->has_job || w->quit; });
        if (w->quit) return;
        w->has_job = false;
        lock.unlock();
        const int rc = cavs_treelstm_stage(e, w->sched, w->parents, w->batch, w->max_len, w->tok, w->label, w->loss_rows);
        const std::string msg = rc ? cavs_last_error() : "";
        lock.lock();
        w->status = rc;
        w->error = msg;
        w->busy = false;
        w->cv.notify_all();
      }
    });
  }
  cavs_treelstm::Stager* w = e->stager;
  {
    std::lock_guard<std::mutex> lock(w->mu);
    w->sched = s; w->parents = parents; w->tok = tok_job; w->label = label_job;
    w->batch = batch; w->max_len = max_len; w->loss_rows = loss_rows;
    w->has_job = true; w->busy = true;
  }
  w->cv.notify_all();
  return CAVS_OK;
}

extern "C" int cavs_treelstm_stage_wait(cavs_treelstm* e) {
  CAVS_REQUIRE(e, CAVS_ERR_BAD_ARG, "treelstm_stage_wait: null handle");
  if (e->stager == nullptr) return CAVS_OK;
  cavs_treelstm::Stager* w = e->stager;
  std::unique_lock<std::mutex> lock(w->mu);
  w->cv.wait(lock, [w] { return !w->busy; });
  const int rc = w->status;
  w->status = CAVS_OK;
  if (rc) return Fail(rc, "treelstm_stage_async: " + w->error);
  return CAVS_OK;
}

extern "C" int cavs_treelstm_step(cavs_treelstm* e, cavs_comm* comm, int optimizer, float* opt_state, float lr, float eps,
                                  void* stream) {
  CAVS_REQUIRE(e && e->params && e->grads, CAVS_ERR_BAD_ARG, "treelstm_step: parameters / gradients not bound");
  CAVS_REQUIRE(optimizer == 0 || optimizer == 1 || optimizer == 2, CAVS_ERR_BAD_ARG, "treelstm_step: optimizer must be 0 (none), 1 (SGD) or 2 (Adagrad)");
  CAVS_REQUIRE(optimizer != 2 || opt_state, CAVS_ERR_BAD_ARG, "treelstm_step: Adagrad needs its accumulator");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int world = 1;
  if (comm) cavs_comm_info(comm, nullptr, &world, nullptr);
  if (int rc = cavs_treelstm_forward(e, stream)) return rc;
  if (int rc = cavs_treelstm_backward(e, stream)) return rc;
  const size_t n_all = e->ParamCount(), n_emb = e->OffW();
  // With exchange rows the embedding block holds one gradient row per listed table row: that is what travels and what
  // the update walks.  Every rank must have been given the same list, or the ranks' reductions differ in size.
  const cavs_treelstm::Batch& bt = e->slot[e->active];
  const bool compact = bt.n_xrows > 0;
  const size_t n_emb_x = compact ? static_cast<size_t>(bt.n_xrows) * e->cfg.embed : n_emb;
  if (world > 1) {
    // Sum of the per-GPU gradients (cavs/midend/session_mpi.cc:31-80 inserts one all-reduce per variable gradient;
    // here the flat buffer goes in two pieces).  backward finishes the embedding block -- the bulk of the buffer --
    // first and announces it, so its reduction runs on a second stream under the weight-gradient products; the
    // remaining blocks follow on the compute stream, which then waits for the first piece.
    cudaEvent_t a0 = nullptr, a1 = nullptr, x0 = nullptr, x1 = nullptr;
    CAVS_CUDA(cudaStreamWaitEvent(e->comm_stream, e->emb_ready, 0));
    if (e->prof_on) { a0 = e->NextEvent(); a1 = e->NextEvent(); CAVS_CUDA(cudaEventRecord(a0, e->comm_stream)); }
    if (int rc = cavs_allreduce(e->grads, n_emb_x, comm, e->comm_stream)) return rc;
    if (e->prof_on) {
      CAVS_CUDA(cudaEventRecord(a1, e->comm_stream));
      e->recs.push_back({kProfCommEmbed, a0, a1, 4.0 * static_cast<double>(n_emb_x)});
    }
    CAVS_CUDA(cudaEventRecord(e->comm_done, e->comm_stream));
    PROF(e, kProfCommRest, 4.0 * static_cast<double>(n_all - n_emb), st, cavs_allreduce(e->grads + n_emb, n_all - n_emb, comm, st));
    // what the compute stream loses waiting for the embedding block's reduction (the part of it that was not hidden)
    if (e->prof_on) { x0 = e->NextEvent(); x1 = e->NextEvent(); CAVS_CUDA(cudaEventRecord(x0, st)); }
    CAVS_CUDA(cudaStreamWaitEvent(st, e->comm_done, 0));
    if (e->prof_on) {
      CAVS_CUDA(cudaEventRecord(x1, st));
      e->recs.push_back({kProfCommExposed, x0, x1, 0.0});
    }
  }
  if (optimizer != 0) {
    // w <- w - lr g (SGD, cavs/backend/op_impl_sgd.cu:15-47) or the Adagrad form, over the whole flat buffer, then the
    // bf16 shadows of the GEMM weights
    const double per = optimizer == 2 ? 20.0 : 12.0;
    if (compact) {
      // listed rows of the table, then the other blocks
      PROF(e, kProfOptimizer, per * static_cast<double>(n_emb_x), st,
           LaunchUpdateRows(e->params, optimizer == 2 ? opt_state : nullptr, e->grads, bt.xrows, bt.n_xrows, e->cfg.embed, lr, eps, st));
      PROF(e, kProfOptimizer, per * static_cast<double>(n_all - n_emb), st,
           optimizer == 2 ? LaunchAdagrad(e->params + n_emb, opt_state + n_emb, e->grads + n_emb, n_all - n_emb, lr, eps, st)
                          : LaunchSgd(e->params + n_emb, e->grads + n_emb, n_all - n_emb, lr, st));
    } else {
      PROF(e, kProfOptimizer, per * static_cast<double>(n_all), st,
           optimizer == 2 ? LaunchAdagrad(e->params, opt_state, e->grads, n_all, lr, eps, st) : LaunchSgd(e->params, e->grads, n_all, lr, st));
    }
    if (int rc = cavs_treelstm_refresh_weights(e, stream)) return rc;
  }
  // The update of listed rows reads the slot's tables (the row list) after backward's own mark: only now may the
  // upload of the batch after next overwrite them.
  CAVS_CUDA(cudaEventRecord(e->slot_done[e->active], st));
  return CAVS_OK;
}

extern "C" int cavs_treelstm_set_dense_input(cavs_treelstm* e, const float* x, long long pitch) {
  CAVS_REQUIRE(e && e->Dense(), CAVS_ERR_BAD_ARG, "treelstm_set_dense_input: the engine was created with an embedding table (vocab > 0)");
  CAVS_REQUIRE(x && pitch >= e->cfg.embed && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && pitch % 4 == 0, CAVS_ERR_BAD_ARG,
               "treelstm_set_dense_input: rows must be 16-byte aligned with pitch >= embed");
  e->x_dense = x;
  e->x_pitch = pitch;
  return CAVS_OK;
}

extern "C" int cavs_treelstm_set_output_grad(cavs_treelstm* e, const float* dh) {
  CAVS_REQUIRE(e && e->Headless(), CAVS_ERR_BAD_ARG, "treelstm_set_output_grad: the engine was created with a loss head (classes > 0)");
  CAVS_REQUIRE(dh && (reinterpret_cast<uintptr_t>(dh) & 15u) == 0, CAVS_ERR_BAD_ARG, "treelstm_set_output_grad: rows must be 16-byte aligned");
  e->dh_ext = dh;
  return CAVS_OK;
}

extern "C" int cavs_treelstm_materialize_state(cavs_treelstm* e, void* stream) {
  CAVS_REQUIRE(e, CAVS_ERR_BAD_ARG, "treelstm_materialize_state: null handle");
  if (!e->leaf_tok || e->active < 0) return CAVS_OK;
  const cavs_treelstm::Batch& bt = e->slot[e->active];
  const int n_leaf = bt.n_levels > 0 ? bt.level_off[1] : 0;
  // leaf vertex t <- its token's row: rows [0, n_leaf) of state_row are exactly those source rows
  if (int rc = cavs_gather_rows(e->state, e->state, bt.state_row, n_leaf, static_cast<size_t>(2) * e->cfg.hidden * sizeof(float), stream))
    return rc;
  // and the leaves' loss values, which the loss head's token rows do not write (valid after backward)
  if (e->TokHead())
    if (int rc = LaunchLeafLossFill(e->loss, e->ptok, bt.tok_slot, bt.label, n_leaf, e->cfg.classes, static_cast<cudaStream_t>(stream)))
      return rc;
  CAVS_CUDA(cudaEventRecord(e->slot_done[e->active], static_cast<cudaStream_t>(stream)));   // these launches read the slot's tables
  e->slot_used[e->active] = true;
  return CAVS_OK;
}

extern "C" size_t cavs_treelstm_upload_bytes(const cavs_treelstm* e) { return e ? e->last_upload_bytes : 0; }

extern "C" int cavs_treelstm_wait_embed_grad(cavs_treelstm* e, void* stream) {
  CAVS_REQUIRE(e, CAVS_ERR_BAD_ARG, "treelstm_wait_embed_grad: null handle");
  CAVS_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), e->emb_ready, 0));
  return CAVS_OK;
}

extern "C" int cavs_treelstm_profile(cavs_treelstm* e, int enable) {
  CAVS_REQUIRE(e, CAVS_ERR_BAD_ARG, "treelstm_profile: null handle");
  e->prof_on = enable != 0;
  e->recs.clear();
  e->ev_used = 0;
  return CAVS_OK;
}

extern "C" int cavs_treelstm_profile_read(cavs_treelstm* e, double* ms, double* work, int* launches, int n_classes) {
  CAVS_REQUIRE(e && ms && work && launches && n_classes >= kProfCount, CAVS_ERR_BAD_ARG,
               "treelstm_profile_read: need arrays of at least 13 entries");
  for (int i = 0; i < n_classes; ++i) { ms[i] = 0; work[i] = 0; launches[i] = 0; }
  const bool dump = std::getenv("CAVS_PROF_DUMP") != nullptr;   // one line per launch on stderr
  for (const auto& r : e->recs) {
    CAVS_CUDA(cudaEventSynchronize(r.b));
    float t = 0;
    CAVS_CUDA(cudaEventElapsedTime(&t, r.a, r.b));
    if (dump) std::fprintf(stderr, "prof cls=%d work=%.4g ms=%.4f\n", r.cls, r.work, t);
    ms[r.cls] += t; work[r.cls] += r.work; launches[r.cls] += 1;
  }
  e->recs.clear();
  e->ev_used = 0;
  return CAVS_OK;
}

extern "C" int cavs_treelstm_read_loss(cavs_treelstm* e, float* loss_sum_host, int* status_host, void* stream) {
  CAVS_REQUIRE(e && loss_sum_host, CAVS_ERR_BAD_ARG, "treelstm_read_loss: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float host[2];
  CAVS_CUDA(cudaMemcpyAsync(host, e->tail, sizeof(host), cudaMemcpyDeviceToHost, st));
  CAVS_CUDA(cudaStreamSynchronize(st));
  *loss_sum_host = host[0];
  int status;
  std::memcpy(&status, &host[1], sizeof(int));
  if (status_host) *status_host = status;
  CAVS_REQUIRE(status == 0, CAVS_ERR_TIMEOUT, "treelstm: a bounded device-side wait expired during the step");
  return CAVS_OK;
}

extern "C" int cavs_treelstm_peek(cavs_treelstm* e, int what, const void** dev_ptr, size_t* bytes) {
  CAVS_REQUIRE(e && dev_ptr && bytes, CAVS_ERR_BAD_ARG, "treelstm_peek: null pointer");
  const size_t n = e->active >= 0 ? e->slot[e->active].n : 0, H = e->cfg.hidden;
  switch (what) {
    case 0: *dev_ptr = e->state; *bytes = n * 2 * H * sizeof(float); break;      // h|c per vertex, tensor-id order
    case 1: *dev_ptr = e->loss; *bytes = n * sizeof(float); break;               // per-vertex loss
    case 2:                                                                      // d(loss)/d(pushed h), wide head only
      if (e->FusedDh()) return Fail(CAVS_ERR_UNSUPPORTED, "treelstm_peek: d(h) is not materialised with the fused loss head");
      *dev_ptr = e->dOut; *bytes = n * H * sizeof(float); break;
    case 3: *dev_ptr = e->mailbox; *bytes = n * 2 * H * sizeof(float); break;    // child-gradient mailbox
    case 4: {                                                                    // saved gates; leaf rows are not written
      // with the gate epilogue the arena is split at its capacity: G3 [max_vertices, 3H], then GF [max_vertices, K, H]
      const size_t rows = e->gate_epi ? static_cast<size_t>(e->cfg.max_vertices) : n;
      *dev_ptr = e->gates; *bytes = rows * (3 + e->cfg.n_slots) * H * e->elt; break;
    }
    case 6: *dev_ptr = e->tail; *bytes = 2 * sizeof(float); break;               // [0] loss sum, [1] status word (int)
    case 5:                                                                      // d(loss)/d(dense input)
      if (!e->Dense()) return Fail(CAVS_ERR_UNSUPPORTED, "treelstm_peek: d(x) exists only with dense inputs");
      *dev_ptr = e->dX; *bytes = n * e->cfg.embed * sizeof(float); break;
    default: return Fail(CAVS_ERR_BAD_ARG, "treelstm_peek: unknown array id");
  }
  return CAVS_OK;
}
