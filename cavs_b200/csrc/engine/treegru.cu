// Level-batched execution of a child-sum Tree-GRU vertex function, forward and backward.
//
// The reference ships LSTM vertex functions only (apps/paper/tree-lstm-cavs.cc, apps/lstm/*); this
// engine is the same level loop (cavs/midend/statement.cc:43-123) over a second cell type, to show
// that the scheduler tables, the per-token input projection, the loss head and the deferred weight
// gradients are not tied to one vertex function.  The cell is defined in kernels/gru.cu.
//
// Parameters, flat fp32: Emb [V,E] | W [E,3H] (r,z,n) | U [3,H,H] (U_r|U_z|U_n) | B [3H] | Wc [C,H] | bc [C].
// Per level, forward: gather child h -> (sum h).U_z and h_k.U_r -> reset gates and m -> m.U_n -> z, n, h;
// backward: gate gradients -> zn.U_n^T and zz.U_z^T -> reset-gate gradients -> zr.U_r^T -> child messages.
// One batch at a time (tables are uploaded on the caller's stream); classes <= 8.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <string>
#include <vector>

#include "abi_common.h"
#include "host/sched_handle.h"
#include "kernels/cell.h"
#include "kernels/gemm.h"
#include "kernels/gru.h"

using namespace cavs_b200;

struct cavs_treegru {
  cavs_treelstm_config cfg{};
  bool bf16 = false;
  size_t elt = 4;
  int32_t *d_idx = nullptr, *h_idx = nullptr;
  size_t idx_ints = 0;
  uint8_t *X = nullptr, *A = nullptr, *S = nullptr, *HK = nullptr, *M = nullptr;   // GEMM operands / pre-activations
  uint8_t *dA = nullptr, *ZR = nullptr, *dAtok = nullptr, *PR = nullptr, *PZ = nullptr, *PN = nullptr;
  float *R = nullptr, *ZN = nullptr, *state = nullptr, *mailbox = nullptr, *dOut = nullptr;
  float *dHt = nullptr, *dm = nullptr, *dsz = nullptr, *dqr = nullptr, *dX = nullptr, *loss = nullptr, *tail = nullptr;
  float *loss_scratch = nullptr, *col_scratch = nullptr, *emb_scratch = nullptr, *splitk_scratch = nullptr;
  size_t splitk_bytes = 0;
  uint8_t *W_bf = nullptr, *U_bf = nullptr;
  float *params = nullptr, *grads = nullptr;
  // current batch
  int n = 0, n_total = 0, n_levels = 0, loss_rows = 0, n_chunks = 0, n_seg = 0;
  std::vector<int32_t> level_off, bucket, slot_of_token;
  int32_t *child = nullptr, *parent = nullptr, *label = nullptr, *order = nullptr, *tok_slot = nullptr, *chunk_off = nullptr,
          *seg_first_chunk = nullptr, *seg_tok = nullptr;
  cudaEvent_t copied = nullptr;

  size_t OffW() const { return static_cast<size_t>(cfg.vocab) * cfg.embed; }
  size_t OffU() const { return OffW() + static_cast<size_t>(cfg.embed) * 3 * cfg.hidden; }
  size_t OffB() const { return OffU() + static_cast<size_t>(3) * cfg.hidden * cfg.hidden; }
  size_t OffWc() const { return OffB() + static_cast<size_t>(3) * cfg.hidden; }
  size_t Offbc() const { return OffWc() + static_cast<size_t>(cfg.classes) * cfg.hidden; }
  size_t ParamCount() const { return Offbc() + cfg.classes; }
  int* Status() const { return reinterpret_cast<int*>(tail + 1); }
};

namespace {

size_t Align(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

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

int CheckConfig(const cavs_treelstm_config* c) {
  CAVS_REQUIRE(c, CAVS_ERR_BAD_ARG, "treegru: null config");
  CAVS_REQUIRE(c->hidden > 0 && c->embed > 0 && c->vocab > 0 && c->classes > 0, CAVS_ERR_BAD_ARG, "treegru: sizes must be positive");
  CAVS_REQUIRE(c->classes <= 8, CAVS_ERR_UNSUPPORTED, "treegru: at most 8 classes (fused loss head)");
  CAVS_REQUIRE(c->n_slots >= 1 && c->n_slots <= kMaxSlots, CAVS_ERR_BAD_ARG, "treegru: child slots must be 1..4");
  CAVS_REQUIRE(c->max_vertices > 0 && c->max_level_rows > 0 && c->max_level_rows <= c->max_vertices, CAVS_ERR_BAD_ARG,
               "treegru: capacities must be positive and max_level_rows <= max_vertices");
  if (c->gemm_bf16)
    CAVS_REQUIRE(c->hidden % 8 == 0 && c->embed % 8 == 0, CAVS_ERR_BAD_ARG,
                 "treegru: the tensor-core path needs hidden and embed to be multiples of 8 (16-byte TMA rows)");
  return CAVS_OK;
}

size_t MaxSegments(const cavs_treelstm_config& c) { return std::min<size_t>(c.max_vertices, c.vocab); }
size_t MaxChunks(const cavs_treelstm_config& c) { return MaxSegments(c) + c.max_vertices / kEmbedChunk + 2; }
size_t IdxInts(const cavs_treelstm_config& c) {
  const size_t n = c.max_vertices;
  return (c.n_slots + 5) * n + (MaxChunks(c) + 1) + (MaxSegments(c) + 1) + MaxSegments(c) + 64;
}

size_t Carve(cavs_treegru* e, void* base) {
  const cavs_treelstm_config& c = e->cfg;
  const size_t N = c.max_vertices, L = c.max_level_rows, H = c.hidden, E = c.embed, K = c.n_slots, T = MaxSegments(c);
  const size_t elt = c.gemm_bf16 ? 2 : 4;
  Carver w(base);
  e->d_idx = w.Take<int32_t>(IdxInts(c));
  e->X = w.Take<uint8_t>(T * E * elt);
  e->A = w.Take<uint8_t>(T * 3 * H * elt);
  e->S = w.Take<uint8_t>(N * H * elt);
  e->HK = w.Take<uint8_t>(N * K * H * elt);
  e->M = w.Take<uint8_t>(N * H * elt);
  e->dA = w.Take<uint8_t>(N * 3 * H * elt);
  e->ZR = w.Take<uint8_t>(N * K * H * elt);
  e->dAtok = w.Take<uint8_t>(T * 3 * H * elt);
  e->PR = w.Take<uint8_t>(L * K * H * elt);
  e->PZ = w.Take<uint8_t>(L * H * elt);
  e->PN = w.Take<uint8_t>(L * H * elt);
  e->R = w.Take<float>(N * K * H);
  e->ZN = w.Take<float>(N * 2 * H);
  e->state = w.Take<float>(N * H);
  e->mailbox = w.Take<float>(N * H);
  e->dOut = w.Take<float>(N * H);
  e->dHt = w.Take<float>(L * H);
  e->dm = w.Take<float>(L * H);
  e->dsz = w.Take<float>(L * H);
  e->dqr = w.Take<float>(L * K * H);
  e->dX = w.Take<float>(T * E);
  e->loss = w.Take<float>(N);
  e->tail = w.Take<float>(4);
  e->loss_scratch = w.Take<float>(LossHeadScratchBytes(c.hidden, c.classes) / sizeof(float));
  e->col_scratch = w.Take<float>(ColumnSumScratchBytes(3 * c.hidden) / sizeof(float));
  e->emb_scratch = w.Take<float>(MaxChunks(c) * 3 * H);
  e->splitk_bytes = c.gemm_bf16 ? std::max(GemmBf16ScratchBytes(c.embed, 3 * c.hidden, 32), GemmBf16ScratchBytes(c.hidden, c.hidden, 32)) : 0;
  e->splitk_scratch = w.Take<float>(e->splitk_bytes / sizeof(float));
  e->W_bf = w.Take<uint8_t>(c.gemm_bf16 ? E * 3 * H * 2 : 0);
  e->U_bf = w.Take<uint8_t>(c.gemm_bf16 ? 3 * H * H * 2 : 0);
  return w.used;
}

// C (+)= op(A) op(B) in the engine's precision.  a_t: A stored [k,m]; b_t: B stored [n,k].
// mode: 0 store fp32, 1 accumulate fp32, 2 store bf16 (bf16 mode only; fp32 mode stores fp32).
int Gemm(cavs_treegru* e, void* c, long long ldc, int mode, const void* a, long long lda, bool a_t, const void* b, long long ldb,
         bool b_t, int m, int n, int k, bool split_ok, cudaStream_t st) {
  if (m == 0 || n == 0 || k == 0) return CAVS_OK;
  if (e->bf16) {
    GemmBf16Args g;
    g.c = c; g.ldc = ldc; g.out_mode = mode;
    g.a = a; g.lda = lda; g.a_major = a_t ? 1 : 0;
    g.b = b; g.ldb = ldb; g.b_major = b_t ? 0 : 1;
    g.m = m; g.n = n; g.k = k;
    g.status = e->Status();
    if (split_ok) {
      g.splits = GemmBf16SplitsFor(m, n, k);
      g.scratch = e->splitk_scratch; g.scratch_bytes = e->splitk_bytes;
    }
    return GemmBf16(g, st);
  }
  GemmF32Args g;
  g.c = static_cast<float*>(c); g.ldc = ldc; g.accumulate = mode == 1;
  g.a = static_cast<const float*>(a); g.a_rs = a_t ? 1 : lda; g.a_cs = a_t ? lda : 1;
  g.b = static_cast<const float*>(b); g.b_rs = b_t ? 1 : ldb; g.b_cs = b_t ? ldb : 1;
  g.m = m; g.n = n; g.k = k;
  return GemmF32(g, st);
}

#define GRU_TRY(call) do { if (int _rc = (call)) return _rc; } while (0)

}  // namespace

extern "C" size_t cavs_treegru_param_count(const cavs_treelstm_config* cfg) {
  if (CheckConfig(cfg) != CAVS_OK) return 0;
  cavs_treegru tmp; tmp.cfg = *cfg;
  return tmp.ParamCount();
}

extern "C" size_t cavs_treegru_workspace_bytes(const cavs_treelstm_config* cfg) {
  if (CheckConfig(cfg) != CAVS_OK) return 0;
  cavs_treegru tmp; tmp.cfg = *cfg;
  return Carve(&tmp, nullptr);
}

extern "C" int cavs_treegru_create(const cavs_treelstm_config* cfg, void* workspace, size_t workspace_bytes, cavs_treegru** out) {
  if (int rc = CheckConfig(cfg)) return rc;
  CAVS_REQUIRE(out && workspace, CAVS_ERR_BAD_ARG, "treegru_create: null pointer");
  CAVS_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, CAVS_ERR_BAD_ARG, "treegru_create: workspace must be 256-byte aligned");
  auto* e = new cavs_treegru();
  e->cfg = *cfg;
  e->bf16 = cfg->gemm_bf16 != 0;
  e->elt = e->bf16 ? 2 : 4;
  const size_t need = Carve(e, workspace);
  if (need > workspace_bytes) {
    delete e;
    return Fail(CAVS_ERR_CAPACITY, "treegru_create: workspace needs " + std::to_string(need) + " bytes");
  }
  e->idx_ints = IdxInts(*cfg);
  cudaError_t err = cudaHostAlloc(reinterpret_cast<void**>(&e->h_idx), e->idx_ints * sizeof(int32_t), cudaHostAllocDefault);
  if (err == cudaSuccess) err = cudaEventCreateWithFlags(&e->copied, cudaEventDisableTiming);
  if (err == cudaSuccess) err = cudaMemset(e->tail, 0, 4 * sizeof(float));
  if (err != cudaSuccess) {
    if (e->h_idx) cudaFreeHost(e->h_idx);
    if (e->copied) cudaEventDestroy(e->copied);
    delete e;
    return Fail(CAVS_ERR_CUDA, std::string("treegru_create: ") + cudaGetErrorString(err));
  }
  *out = e;
  return CAVS_OK;
}

extern "C" void cavs_treegru_destroy(cavs_treegru* e) {
  if (!e) return;
  if (e->h_idx) cudaFreeHost(e->h_idx);
  if (e->copied) cudaEventDestroy(e->copied);
  delete e;
}

extern "C" int cavs_treegru_bind(cavs_treegru* e, float* params, float* grads) {
  CAVS_REQUIRE(e && params && grads, CAVS_ERR_BAD_ARG, "treegru_bind: null pointer");
  CAVS_REQUIRE(((reinterpret_cast<uintptr_t>(params) | reinterpret_cast<uintptr_t>(grads)) & 15u) == 0, CAVS_ERR_BAD_ARG,
               "treegru_bind: buffers must be 16-byte aligned");
  e->params = params;
  e->grads = grads;
  return CAVS_OK;
}

extern "C" int cavs_treegru_refresh_weights(cavs_treegru* e, void* stream) {
  CAVS_REQUIRE(e && e->params, CAVS_ERR_BAD_ARG, "treegru_refresh_weights: parameters not bound");
  if (!e->bf16) return CAVS_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t H = e->cfg.hidden, E = e->cfg.embed;
  GRU_TRY(LaunchCastBf16(e->W_bf, e->params + e->OffW(), E * 3 * H, st));
  return LaunchCastBf16(e->U_bf, e->params + e->OffU(), 3 * H * H, st);
}

extern "C" int cavs_treegru_load_batch(cavs_treegru* e, const cavs_sched* s, const int32_t* tok_job, const int32_t* label_job,
                                       int loss_rows, void* stream) {
  CAVS_REQUIRE(e && s && s->loaded && tok_job && label_job, CAVS_ERR_BAD_ARG, "treegru_load_batch: null pointer or empty schedule");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const LevelSchedule& sch = s->impl;
  const int n = sch.n_scheduled(), nt = sch.n_total(), K = e->cfg.n_slots, V = e->cfg.vocab;
  CAVS_REQUIRE(sch.n_slots() == K, CAVS_ERR_BAD_ARG, "treegru_load_batch: schedule was built with a different slot count");
  CAVS_REQUIRE(nt <= e->cfg.max_vertices, CAVS_ERR_CAPACITY,
               "treegru_load_batch: batch has " + std::to_string(nt) + " vertices, capacity " + std::to_string(e->cfg.max_vertices));
  CAVS_REQUIRE(sch.max_level_rows() <= e->cfg.max_level_rows, CAVS_ERR_CAPACITY,
               "treegru_load_batch: widest level has " + std::to_string(sch.max_level_rows()) + " rows, capacity " +
                   std::to_string(e->cfg.max_level_rows));
  // The pinned staging array is reused: wait for the previous upload to have left it.
  CAVS_CUDA(cudaEventSynchronize(e->copied));
  e->n = n; e->n_total = nt; e->n_levels = sch.n_levels();
  e->loss_rows = loss_rows > 0 ? loss_rows : std::max(n, 1);
  e->level_off = sch.level_off();
  int32_t *h = e->h_idx, *d = e->d_idx;
  size_t o = 0;
  auto view = [&](size_t count, int32_t** dev) { int32_t* p = h + o; *dev = d + o; o += count; return p; };
  int32_t* dev_tok = nullptr;
  int32_t* h_child = view(static_cast<size_t>(K) * nt, &e->child);
  int32_t* h_parent = view(nt, &e->parent);
  int32_t* h_tok = view(nt, &dev_tok);
  int32_t* h_label = view(nt, &e->label);
  int32_t* h_order = view(nt, &e->order);
  int32_t* h_slot = view(nt, &e->tok_slot);
  std::memcpy(h_child, sch.child_t().data(), sizeof(int32_t) * K * nt);
  std::memcpy(h_parent, sch.parent_t().data(), sizeof(int32_t) * nt);
  const int32_t* t2j = sch.t2j().data();
  for (int t = 0; t < n; ++t) {
    const int id = tok_job[t2j[t]];
    h_tok[t] = (id < 0 || id >= V) ? 0 : id;
    h_label[t] = label_job[t2j[t]];
  }
  // Rows grouped by token (stable counting sort): segments = distinct tokens, chunks of at most
  // kEmbedChunk rows for the fixed-order segmented sums.
  e->bucket.assign(static_cast<size_t>(V) + 1, 0);
  for (int t = 0; t < n; ++t) ++e->bucket[h_tok[t] + 1];
  int n_seg = 0, n_chunks = 0;
  for (int v = 0; v < V; ++v) {
    const int cnt = e->bucket[v + 1];
    if (cnt) ++n_seg;
    n_chunks += (cnt + kEmbedChunk - 1) / kEmbedChunk;
    e->bucket[v + 1] += e->bucket[v];
  }
  int32_t* h_chunk_off = view(static_cast<size_t>(n_chunks) + 1, &e->chunk_off);
  int32_t* h_seg_first = view(static_cast<size_t>(n_seg) + 1, &e->seg_first_chunk);
  int32_t* h_seg_tok = view(n_seg, &e->seg_tok);
  CAVS_REQUIRE(o <= e->idx_ints, CAVS_ERR_CAPACITY, "treegru_load_batch: index blob overflow");
  e->slot_of_token.resize(V);
  int si = 0, ci = 0;
  for (int v = 0; v < V; ++v) {
    const int b0 = e->bucket[v], b1 = e->bucket[v + 1];
    if (b0 == b1) continue;
    e->slot_of_token[v] = si;
    h_seg_tok[si] = v;
    h_seg_first[si++] = ci;
    for (int b = b0; b < b1; b += kEmbedChunk) h_chunk_off[ci++] = b;
  }
  h_seg_first[si] = ci;
  h_chunk_off[ci] = n;
  for (int t = 0; t < n; ++t) {
    h_order[e->bucket[h_tok[t]]++] = t;
    h_slot[t] = e->slot_of_token[h_tok[t]];
  }
  e->n_seg = n_seg; e->n_chunks = n_chunks;
  CAVS_CUDA(cudaMemcpyAsync(d, h, o * sizeof(int32_t), cudaMemcpyHostToDevice, st));
  CAVS_CUDA(cudaEventRecord(e->copied, st));
  return CAVS_OK;
}

extern "C" int cavs_treegru_forward(cavs_treegru* e, void* stream) {
  CAVS_REQUIRE(e && e->params, CAVS_ERR_BAD_ARG, "treegru_forward: parameters not bound");
  CAVS_REQUIRE(!e->level_off.empty(), CAVS_ERR_BAD_ARG, "treegru_forward: no batch loaded");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int n = e->n, nt = e->n_total, H = e->cfg.hidden, E = e->cfg.embed, K = e->cfg.n_slots;
  if (n == 0) return CAVS_OK;
  const size_t elt = e->elt;
  const uint8_t* W = e->bf16 ? e->W_bf : reinterpret_cast<const uint8_t*>(e->params + e->OffW());
  const uint8_t* U = e->bf16 ? e->U_bf : reinterpret_cast<const uint8_t*>(e->params + e->OffU());
  const uint8_t *U_r = U, *U_z = U + static_cast<size_t>(H) * H * elt, *U_n = U + static_cast<size_t>(2) * H * H * elt;
  const float* B = e->params + e->OffB();
  const int pre = e->bf16 ? 2 : 0;
  GRU_TRY(LaunchEmbedFwd(e->X, e->bf16, e->params, e->seg_tok, e->n_seg, E, e->cfg.vocab, st));
  GRU_TRY(Gemm(e, e->A, 3 * H, pre, e->X, E, false, W, 3 * H, false, e->n_seg, 3 * H, E, false, st));
  for (int l = 0; l < e->n_levels; ++l) {
    const int off = e->level_off[l], rows = e->level_off[l + 1] - off;
    if (l == 0) {
      GRU_TRY(LaunchGruOut(e->state, e->ZN, e->bf16, e->A, nullptr, nullptr, B, e->child, e->tok_slot, nt, off, rows, H, K, true, st));
      continue;
    }
    GRU_TRY(LaunchGatherChildH(e->S, e->HK, e->bf16, e->state, e->child, nt, off, rows, H, K, st, H));
    const uint8_t* S_l = e->S + static_cast<size_t>(off) * H * elt;
    const uint8_t* HK_l = e->HK + static_cast<size_t>(off) * K * H * elt;
    const uint8_t* M_l = e->M + static_cast<size_t>(off) * H * elt;
    GRU_TRY(Gemm(e, e->PZ, H, pre, S_l, H, false, U_z, H, false, rows, H, H, false, st));
    GRU_TRY(Gemm(e, e->PR, H, pre, HK_l, H, false, U_r, H, false, rows * K, H, H, false, st));
    GRU_TRY(LaunchGruGateR(e->R, e->M, e->bf16, e->A, e->PR, B, e->state, e->child, e->tok_slot, nt, off, rows, H, K, st));
    GRU_TRY(Gemm(e, e->PN, H, pre, M_l, H, false, U_n, H, false, rows, H, H, false, st));
    GRU_TRY(LaunchGruOut(e->state, e->ZN, e->bf16, e->A, e->PZ, e->PN, B, e->child, e->tok_slot, nt, off, rows, H, K, false, st));
  }
  return CAVS_OK;
}

extern "C" int cavs_treegru_backward(cavs_treegru* e, void* stream) {
  CAVS_REQUIRE(e && e->params && e->grads, CAVS_ERR_BAD_ARG, "treegru_backward: parameters / gradients not bound");
  CAVS_REQUIRE(!e->level_off.empty(), CAVS_ERR_BAD_ARG, "treegru_backward: no batch loaded");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int n = e->n, nt = e->n_total, H = e->cfg.hidden, E = e->cfg.embed, K = e->cfg.n_slots, C = e->cfg.classes;
  float* g = e->grads;
  if (n == 0) {
    CAVS_CUDA(cudaMemsetAsync(g, 0, e->ParamCount() * sizeof(float), st));
    return CAVS_OK;
  }
  const size_t elt = e->elt;
  const uint8_t* W = e->bf16 ? e->W_bf : reinterpret_cast<const uint8_t*>(e->params + e->OffW());
  const uint8_t* U = e->bf16 ? e->U_bf : reinterpret_cast<const uint8_t*>(e->params + e->OffU());
  const uint8_t *U_r = U, *U_z = U + static_cast<size_t>(H) * H * elt, *U_n = U + static_cast<size_t>(2) * H * H * elt;
  GRU_TRY(LaunchLossHead(e->loss, e->tail, e->dOut, g + e->OffWc(), g + e->Offbc(), e->state, H, e->label, e->params + e->OffWc(),
                         e->params + e->Offbc(), n, H, C, 1.0f / static_cast<float>(e->loss_rows), e->loss_scratch, st));
  for (int l = e->n_levels - 1; l >= 0; --l) {
    const int off = e->level_off[l], rows = e->level_off[l + 1] - off;
    GRU_TRY(LaunchGruBwdA(e->dA, e->dHt, e->bf16, e->mailbox, e->dOut, e->ZN, e->state, e->child, e->parent, nt, off, rows, H, K,
                          l == 0, st));
    if (l == 0) break;
    const uint8_t* dA_l = e->dA + static_cast<size_t>(off) * 3 * H * elt;
    const uint8_t* ZR_l = e->ZR + static_cast<size_t>(off) * K * H * elt;
    // dm = zn U_n^T, dsz = zz U_z^T: the z / n blocks of dA are GEMM operands in place (row pitch 3H).
    GRU_TRY(Gemm(e, e->dm, H, 0, dA_l + static_cast<size_t>(2) * H * elt, 3 * H, false, U_n, H, true, rows, H, H, false, st));
    GRU_TRY(Gemm(e, e->dsz, H, 0, dA_l + static_cast<size_t>(H) * elt, 3 * H, false, U_z, H, true, rows, H, H, false, st));
    GRU_TRY(LaunchGruBwdB1(e->dA, e->ZR, e->bf16, e->dm, e->R, e->state, e->child, nt, off, rows, H, K, st));
    GRU_TRY(Gemm(e, e->dqr, H, 0, ZR_l, H, false, U_r, H, true, rows * K, H, H, false, st));
    GRU_TRY(LaunchGruBwdB2(e->mailbox, e->dHt, e->dsz, e->dm, e->dqr, e->R, e->child, nt, off, rows, H, K, st));
  }
  // Deferred weight gradients over all internal rows (leaves have no recurrent operands).
  const int off1 = e->n_levels > 1 ? e->level_off[1] : n;
  const int n_int = n - off1;
  float* dU = g + e->OffU();
  if (n_int > 0) {
    const uint8_t* S1 = e->S + static_cast<size_t>(off1) * H * elt;
    const uint8_t* HK1 = e->HK + static_cast<size_t>(off1) * K * H * elt;
    const uint8_t* M1 = e->M + static_cast<size_t>(off1) * H * elt;
    const uint8_t* dA1 = e->dA + static_cast<size_t>(off1) * 3 * H * elt;
    const uint8_t* ZR1 = e->ZR + static_cast<size_t>(off1) * K * H * elt;
    GRU_TRY(Gemm(e, dU, H, 0, HK1, H, true, ZR1, H, false, H, H, n_int * K, true, st));
    GRU_TRY(Gemm(e, dU + static_cast<size_t>(H) * H, H, 0, S1, H, true, dA1 + static_cast<size_t>(H) * elt, 3 * H, false, H, H, n_int, true, st));
    GRU_TRY(Gemm(e, dU + static_cast<size_t>(2) * H * H, H, 0, M1, H, true, dA1 + static_cast<size_t>(2) * H * elt, 3 * H, false, H, H, n_int, true, st));
  } else {
    CAVS_CUDA(cudaMemsetAsync(dU, 0, static_cast<size_t>(3) * H * H * sizeof(float), st));
  }
  GRU_TRY(LaunchColumnSum(g + e->OffB(), e->dA, e->bf16, 3 * H, n, 3 * H, e->col_scratch, st));
  const int n_tok = e->n_seg;
  GRU_TRY(LaunchSegmentedRowSum(e->dAtok, e->bf16, e->dA, e->bf16, 3 * H, 3 * H, e->order, e->chunk_off, e->n_chunks,
                                e->seg_first_chunk, n_tok, e->emb_scratch, st));
  GRU_TRY(Gemm(e, g + e->OffW(), 3 * H, 0, e->X, E, true, e->dAtok, 3 * H, false, E, 3 * H, n_tok, true, st));
  GRU_TRY(Gemm(e, e->dX, E, 0, e->dAtok, 3 * H, false, W, 3 * H, true, n_tok, E, 3 * H, false, st));
  CAVS_CUDA(cudaMemsetAsync(g, 0, static_cast<size_t>(e->cfg.vocab) * E * sizeof(float), st));
  GRU_TRY(cavs_scatter_rows(g, e->seg_tok, e->dX, n_tok, static_cast<size_t>(E) * sizeof(float), st));
  return CAVS_OK;
}

extern "C" int cavs_treegru_read_loss(cavs_treegru* e, float* loss_sum_host, int* status_host, void* stream) {
  CAVS_REQUIRE(e && loss_sum_host, CAVS_ERR_BAD_ARG, "treegru_read_loss: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float host[2];
  CAVS_CUDA(cudaMemcpyAsync(host, e->tail, sizeof(host), cudaMemcpyDeviceToHost, st));
  CAVS_CUDA(cudaStreamSynchronize(st));
  *loss_sum_host = host[0];
  int status;
  std::memcpy(&status, &host[1], sizeof(int));
  if (status_host) *status_host = status;
  CAVS_REQUIRE(status == 0, CAVS_ERR_TIMEOUT, "treegru: a bounded device-side wait expired during the step");
  return CAVS_OK;
}

extern "C" int cavs_treegru_peek(cavs_treegru* e, int what, const void** dev_ptr, size_t* bytes) {
  CAVS_REQUIRE(e && dev_ptr && bytes, CAVS_ERR_BAD_ARG, "treegru_peek: null pointer");
  const size_t n = e->n, H = e->cfg.hidden;
  switch (what) {
    case 0: *dev_ptr = e->state; *bytes = n * H * sizeof(float); break;       // h per vertex, tensor-id order
    case 1: *dev_ptr = e->loss; *bytes = n * sizeof(float); break;            // per-vertex loss
    case 2: *dev_ptr = e->dOut; *bytes = n * H * sizeof(float); break;        // d(loss)/d(h)
    case 3: *dev_ptr = e->mailbox; *bytes = n * H * sizeof(float); break;     // child-gradient mailbox
    default: return Fail(CAVS_ERR_BAD_ARG, "treegru_peek: unknown array id");
  }
  return CAVS_OK;
}
