/*
 * TEST INFRASTRUCTURE -- CPU oracle for the level-batched vertex-function path.
 *
 * Plain-C restatement of the reference's algorithm.  Only the test-suite, the
 * smoke check and the benchmark's CPU-baseline leg may link or call this file;
 * the product library never does.
 *
 * Parity status
 *   - schedule / index tables: PINNED.  cavs_oracle_schedule_stream() is checked
 *     stream-for-stream against the reference's own graph scheduler compiled from
 *     cavs/midend/graph_scheduler.{h,cc} (see refsched_driver.cc).
 *   - numerics (Tree-LSTM / chain-LSTM forward, loss, backward, SGD): PARITY
 *     UNPINNED by any reference test or golden vector (the reference has none for
 *     this path and has no CPU implementation of its ops).  The maths below
 *     follows the cited source lines and is cross-checked against PyTorch CPU
 *     autograd in the test-suite.
 *   - Adagrad, more than two child slots, bf16-rounded GEMM operands, Tree-GRU:
 *     extensions the reference lacks; defined here, parity unpinned.
 *
 * Everything is fp32 with int32 indices, as in the reference.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_MAX_SLOTS 4

/* ------------------------------------------------------------------------- */
/* Schedule: restatement of GraphSchedulerBase::LoadGraph                     */
/* (cavs/midend/graph_scheduler.cc:12-71) and BatchGraphScheduler::Initialize */
/* / ActivateNext (graph_scheduler.cc:169-258).                               */
/* ------------------------------------------------------------------------- */

typedef struct {
  int n_total;      /* vertices over all samples (LoadGraph's return value)          */
  int n_levels;
  int n_slots;
  int *parent;      /* [n_total] global id of the parent, -1 for a root              */
  int *n_child;     /* [n_total]                                                     */
  int *child;       /* [n_total * n_slots] children in ascending id, -1 padded       */
  int *level_off;   /* [n_levels + 1]                                                */
  int *t2j;         /* [n_total] tensor id (execution order) -> job id (global id)   */
  int *j2t;         /* [n_total] job id -> tensor id, -1 when never scheduled        */
  int *level_of;    /* [n_total] level of each tensor id                             */
} oracle_sched;

static void oracle_sched_free(oracle_sched *s) {
  free(s->parent); free(s->n_child); free(s->child); free(s->level_off);
  free(s->t2j); free(s->j2t); free(s->level_of);
  memset(s, 0, sizeof(*s));
}

/* Returns 0 on success, <0 on malformed input (the reference would CHECK-abort or
 * read out of bounds on these). */
static int oracle_sched_build(const int *parents, int batch, int max_len, int n_slots, oracle_sched *s) {
  memset(s, 0, sizeof(*s));
  if (batch < 0 || max_len <= 0 || n_slots < 1 || n_slots > ORACLE_MAX_SLOTS) return -1;
  /* graph_scheduler.cc:39 -- a sample's length is the position of its first -1, plus one. */
  int *len = (int *)malloc(sizeof(int) * (size_t)(batch > 0 ? batch : 1));
  int *base = (int *)malloc(sizeof(int) * (size_t)(batch > 0 ? batch : 1));
  int total = 0;
  for (int i = 0; i < batch; i++) {
    const int *row = parents + (size_t)i * max_len;
    int k = 0;
    while (k < max_len && row[k] != -1) k++;
    if (k == max_len) { free(len); free(base); return -2; } /* no terminator */
    len[i] = k + 1;
    base[i] = total;                                        /* graph_scheduler.cc:40, compact ids */
    total += len[i];
  }
  s->n_total = total;
  s->n_slots = n_slots;
  size_t nt = (size_t)(total > 0 ? total : 1);
  s->parent = (int *)malloc(sizeof(int) * nt);
  s->n_child = (int *)calloc(nt, sizeof(int));
  s->child = (int *)malloc(sizeof(int) * nt * n_slots);
  s->t2j = (int *)calloc(nt, sizeof(int));
  s->j2t = (int *)malloc(sizeof(int) * nt);
  s->level_of = (int *)calloc(nt, sizeof(int));
  for (size_t i = 0; i < nt * n_slots; i++) s->child[i] = -1;
  for (size_t i = 0; i < nt; i++) { s->parent[i] = -1; s->j2t[i] = -1; }
  int bad = 0;
  for (int i = 0; i < batch && !bad; i++) {
    const int *row = parents + (size_t)i * max_len;
    /* graph_scheduler.cc:44-50: every vertex but the last has one parent. */
    for (int j = 0; j < len[i] - 1; j++) {
      if (row[j] < 0 || row[j] >= len[i] || row[j] == j) { bad = 1; break; }
      s->parent[base[i] + j] = base[i] + row[j];
    }
    /* graph_scheduler.cc:52-59: children recorded in ascending id order. */
    for (int j = 0; j < len[i] - 1 && !bad; j++) {
      int p = s->parent[base[i] + j];
      if (s->n_child[p] >= n_slots) { bad = 1; break; }
      s->child[(size_t)p * n_slots + s->n_child[p]++] = base[i] + j;
    }
  }
  free(len); free(base);
  if (bad) { oracle_sched_free(s); return -3; }

  /* Wavefront.  Level 0 = childless vertices that have a parent, ascending id
   * (graph_scheduler.cc:178-188); later levels in discovery order
   * (graph_scheduler.cc:215-238). */
  int *ready = (int *)malloc(sizeof(int) * nt), *next = (int *)malloc(sizeof(int) * nt);
  int *hits = (int *)calloc(nt, sizeof(int));
  int *offs = (int *)malloc(sizeof(int) * (nt + 2));
  int n_ready = 0, levels = 0, placed = 0;
  for (int g = 0; g < total; g++)
    if (s->n_child[g] == 0 && s->parent[g] >= 0) ready[n_ready++] = g;
  while (n_ready > 0) {
    offs[levels] = placed;
    for (int b = 0; b < n_ready; b++) {
      s->t2j[placed + b] = ready[b];
      s->j2t[ready[b]] = placed + b;
      s->level_of[placed + b] = levels;
    }
    placed += n_ready;
    levels++;
    int n_next = 0;
    for (int b = 0; b < n_ready; b++) {
      int p = s->parent[ready[b]];
      if (p >= 0 && ++hits[p] == s->n_child[p]) next[n_next++] = p;
    }
    int *tmp = ready; ready = next; next = tmp;
    n_ready = n_next;
  }
  offs[levels] = placed;
  s->n_levels = levels;
  s->level_off = (int *)malloc(sizeof(int) * (size_t)(levels + 1));
  memcpy(s->level_off, offs, sizeof(int) * (size_t)(levels + 1));
  free(ready); free(next); free(hits); free(offs);
  if (placed != total) {
    /* Either single-vertex samples (never scheduled, graph_scheduler.cc:180) or a
     * cycle.  Single-vertex samples are legal; a cycle is not. */
    for (int g = 0; g < total; g++)
      if (s->j2t[g] < 0 && !(s->n_child[g] == 0 && s->parent[g] < 0)) { oracle_sched_free(s); return -4; }
  }
  return 0;
}

/* Lists of one forward level, in the reference's compact form. */
static int lvl_gather(const oracle_sched *s, int lvl, int slot, int *out) {
  /* graph_scheduler.cc:222-227: a slot's list only receives an entry from jobs
   * that own a child in that slot, so it can be shorter than the job list. */
  int n = 0;
  if (lvl == 0) return 0;
  for (int t = s->level_off[lvl]; t < s->level_off[lvl + 1]; t++) {
    int g = s->t2j[t];
    if (slot < s->n_child[g]) out[n++] = s->j2t[s->child[(size_t)g * s->n_slots + slot]];
  }
  return n;
}
static int lvl_scatter(const oracle_sched *s, int lvl, int *out) {
  /* graph_scheduler.cc:184,228-235: own tensor ids, roots excluded (level 0 never
   * holds a root). */
  int n = 0;
  for (int t = s->level_off[lvl]; t < s->level_off[lvl + 1]; t++)
    if (s->parent[s->t2j[t]] >= 0) out[n++] = t;
  return n;
}

#define EMIT(v) do { if (w < capacity) out[w] = (v); w++; } while (0)
#define EMIT_LIST(ptr, cnt) do { EMIT(cnt); for (int _i = 0; _i < (cnt); _i++) EMIT((ptr)[_i]); } while (0)

/* Serialises the schedule in the layout documented in refsched_driver.cc.
 * Returns the stream length, or -(needed length) if capacity is too small, or
 * -1000000-k for malformed graphs. */
int cavs_oracle_schedule_stream(const int *parents, int batch, int max_len, int *out, int capacity) {
  oracle_sched s;
  int rc = oracle_sched_build(parents, batch, max_len, 2, &s);
  if (rc < 0) return -1000000 + rc;
  long w = 0;
  int nt = s.n_total > 0 ? s.n_total : 1;
  int *tmp = (int *)malloc(sizeof(int) * (size_t)nt);
  int *roots = (int *)malloc(sizeof(int) * (size_t)nt);
  int n_roots = 0;
  EMIT(s.n_total);
  EMIT(s.n_levels);
  for (int l = 0; l <= s.n_levels; l++) EMIT(s.level_off[l]);
  int n0 = s.n_levels > 0 ? s.level_off[1] : 0;
  for (int l = 0; l < s.n_levels; l++) {
    EMIT_LIST(s.t2j + s.level_off[l], s.level_off[l + 1] - s.level_off[l]);
    for (int c = 0; c < 2; c++) { int n = lvl_gather(&s, l, c, tmp); EMIT_LIST(tmp, n); }
    { int n = lvl_scatter(&s, l, tmp); EMIT_LIST(tmp, n); }
    /* graph_scheduler.cc:190: the forward "gather initialisation" list is the level-0
     * job list and is never refreshed on later levels. */
    EMIT_LIST(s.t2j, n0);
  }
  for (int t = 0; t < s.n_total; t++) EMIT(s.t2j[t]);
  /* Roots' tensor ids accumulate in discovery order (graph_scheduler.cc:229-230). */
  for (int t = 0; t < s.level_off[s.n_levels]; t++)
    if (s.parent[s.t2j[t]] < 0) roots[n_roots++] = t;
  /* Backward replay (graph_scheduler.cc:194-198,246-257): gather := forward scatter
   * list, scatter := forward gather lists, last level first. */
  for (int l = s.n_levels - 1; l >= 0; l--) {
    EMIT(s.level_off[l]);
    EMIT_LIST(s.t2j + s.level_off[l], s.level_off[l + 1] - s.level_off[l]);
    { int n = lvl_scatter(&s, l, tmp); EMIT_LIST(tmp, n); }
    for (int c = 0; c < 2; c++) { int n = lvl_gather(&s, l, c, tmp); EMIT_LIST(tmp, n); }
    EMIT_LIST(roots, n_roots);
  }
  free(tmp); free(roots);
  oracle_sched_free(&s);
  if (w > capacity) return (int)-w;
  return (int)w;
}

/* ------------------------------------------------------------------------- */
/* Serial (one vertex per round) sweep: restatement of SerialGraphScheduler   */
/* (cavs/midend/graph_scheduler.cc:83-167, graph_scheduler.h:122-138).        */
/* Tensor id == job id there (:90,138), a round's offset is its job id.       */
/* ------------------------------------------------------------------------- */

/* One sweep.  `up` are the edges a finished vertex follows to wake others, `down` the
 * edges that must all have finished before a vertex runs: forward up = parent, down =
 * children; after ReverseGraph (graph_scheduler.cc:73-81) the two swap.  The work list is
 * first-in first-out (:89,131,139-142).  A sample enters the list when the previous
 * sample's last vertex (one without `up` edges) leaves it (:135-137) -- so in the backward
 * sweep every forward leaf pulls in the next sample -- and a sample contributes its
 * vertices that have no `down` but some `up` edge (:110-114), which is nothing for a
 * single-vertex sample: if the list is empty at that point the sweep ends early (:141).
 * Emits, per round: job id, then the four lists in the order the caller asks for. */
static long serial_sweep(const oracle_sched *s, const int *base, const int *len, int batch, int backward,
                         int *out, long w, long capacity, int *n_rounds, int *seen) {
  const int K = s->n_slots;
  int nt = s->n_total > 0 ? s->n_total : 1;
  int *queue = (int *)malloc(sizeof(int) * (size_t)nt * 2);
  int *hits = (int *)calloc((size_t)nt, sizeof(int));
  int head = 0, tail = 0, sample = 0, rounds = 0;
  int last_init = -1;
#define N_UP(g) (backward ? s->n_child[g] : (s->parent[g] >= 0 ? 1 : 0))
#define N_DOWN(g) (backward ? (s->parent[g] >= 0 ? 1 : 0) : s->n_child[g])
#define UP(g, i) (backward ? s->child[(size_t)(g) * K + (i)] : s->parent[g])
#define DOWN(g, i) (backward ? s->parent[g] : s->child[(size_t)(g) * K + (i)])
#define ENTER(sid) do { for (int _j = 0; _j < len[sid]; _j++) { int _g = base[sid] + _j; \
      if (N_DOWN(_g) == 0 && N_UP(_g) > 0) queue[tail++] = _g; } } while (0)
  if (batch > 0) ENTER(0);
  while (head < tail) {
    const int g = queue[head];
    if (N_DOWN(g) == 0) last_init = g;                       /* :101,105,153,165: never cleared otherwise */
    EMIT(g);
    if (!backward) {
      for (int c = 0; c < 2; c++) { if (c < N_DOWN(g)) { EMIT(1); EMIT(DOWN(g, c)); } else EMIT(0); }   /* :150-152 */
      { int n = N_UP(g); EMIT(n); for (int i = 0; i < n; i++) EMIT(g); }                                 /* :146-149 */
    } else {
      { int n = N_DOWN(g); EMIT(n); for (int i = 0; i < n; i++) EMIT(g); }                               /* :157-160 */
      for (int c = 0; c < 2; c++) { if (c < N_UP(g)) { EMIT(1); EMIT(UP(g, c)); } else EMIT(0); }        /* :161-163 */
    }
    if (last_init >= 0) { EMIT(1); EMIT(last_init); } else EMIT(0);
    if (seen) seen[g] = 1;
    rounds++;
    /* ActivateNext, :121-139 */
    if (N_UP(g) > 0) {
      for (int i = 0; i < N_UP(g); i++) { int p = UP(g, i); if (++hits[p] == N_DOWN(p)) queue[tail++] = p; }
    } else if (++sample < batch) {
      ENTER(sample);
    }
    head++;
  }
#undef N_UP
#undef N_DOWN
#undef UP
#undef DOWN
#undef ENTER
  free(queue); free(hits);
  *n_rounds = rounds;
  return w;
}

/* Stream layout ("serial schedule stream"), all int32 (lists are written as count, entries):
 *   N
 *   RF, then per forward round:  job  gather(0)  gather(1)  scatter(0)  gather-initialisation
 *   t2j[N]                       identity for vertices that ran, 0 otherwise (a fresh scheduler)
 *   RB, then per backward round: job  gather(0)  scatter(0)  scatter(1)  gather-initialisation
 * Returns the length, -(needed) if capacity is too small, -1000000-k for malformed graphs. */
int cavs_oracle_serial_stream(const int *parents, int batch, int max_len, int *out, int capacity) {
  oracle_sched s;
  int rc = oracle_sched_build(parents, batch, max_len, 2, &s);
  if (rc < 0) return -1000000 + rc;
  int nb = batch > 0 ? batch : 1;
  int *base = (int *)malloc(sizeof(int) * (size_t)nb), *len = (int *)malloc(sizeof(int) * (size_t)nb);
  int total = 0;
  for (int i = 0; i < batch; i++) {
    const int *row = parents + (size_t)i * max_len;
    int k = 0;
    while (row[k] != -1) k++;
    base[i] = total; len[i] = k + 1; total += k + 1;
  }
  int *seen = (int *)calloc((size_t)(total > 0 ? total : 1), sizeof(int));
  long w = 0;
  int rounds = 0;
  EMIT(s.n_total);
  long at = w; EMIT(0);
  w = serial_sweep(&s, base, len, batch, 0, out, w, capacity, &rounds, seen);
  if (at < capacity) out[at] = rounds;
  for (int g = 0; g < s.n_total; g++) EMIT(seen[g] ? g : 0);
  at = w; EMIT(0);
  if (rounds > 0) w = serial_sweep(&s, base, len, batch, 1, out, w, capacity, &rounds, NULL);
  else rounds = 0;
  if (at < capacity) out[at] = rounds;
  free(base); free(len); free(seen);
  oracle_sched_free(&s);
  if (w > capacity) return (int)-w;
  return (int)w;
}

/* Per-vertex index tables in tensor-id space, the form the numerics below (and the
 * product engine) consume.  All arrays are [n] or [n_slots * n] (slot-major).
 *   fg[c][t]  forward gather source: mailbox row read into row t's slot-c child state, -1 = zeros
 *   fs[t]     forward scatter target: mailbox row that receives row t's h|c, -1 = none
 *   bg[t]     backward gather source: mailbox row holding d(h|c) for row t, -1 = zeros
 *   bs[c][t]  backward scatter target for the slot-c child gradient, -1 = none
 * mode 0 ("aligned"): row b of a level always talks to its own children / itself.
 * mode 1 ("ref_compat"): reproduces the reference, where the compact lists are applied
 *   positionally -- list entry b pairs with arena row b of the level
 *   (functor_batched_memcpy.cuh:34-61, op_impl_graphop.cu:62-76,144-157) -- so rows of a
 *   level whose jobs lack a child slot / a parent are shifted; rows past the end of a
 *   list keep the zero fill the allocator gave them (allocator.cu:17-22).
 * Also returns tok_perm-free helpers: t2j, j2t, level_off.  Returns n_levels or <0. */
int cavs_oracle_tables(const int *parents, int batch, int max_len, int n_slots, int mode,
                       int *n_total_out, int *level_off /* [max possible levels+1] or NULL */, int level_cap,
                       int *t2j, int *j2t, int *fg, int *fs, int *bg, int *bs) {
  oracle_sched s;
  int rc = oracle_sched_build(parents, batch, max_len, n_slots, &s);
  if (rc < 0) return rc;
  int n = s.n_total;
  if (s.n_levels + 1 > level_cap) { oracle_sched_free(&s); return -10; }
  *n_total_out = n;
  memcpy(level_off, s.level_off, sizeof(int) * (size_t)(s.n_levels + 1));
  memcpy(t2j, s.t2j, sizeof(int) * (size_t)n);
  memcpy(j2t, s.j2t, sizeof(int) * (size_t)n);
  for (size_t i = 0; i < (size_t)n * n_slots; i++) { fg[i] = -1; bs[i] = -1; }
  for (int t = 0; t < n; t++) { fs[t] = -1; bg[t] = -1; }
  int *tmp = (int *)malloc(sizeof(int) * (size_t)(n > 0 ? n : 1));
  for (int l = 0; l < s.n_levels; l++) {
    int off = s.level_off[l], cnt = s.level_off[l + 1] - off;
    if (mode == 0) {
      for (int b = 0; b < cnt; b++) {
        int g = s.t2j[off + b];
        for (int c = 0; c < s.n_child[g]; c++) {
          int ct = s.j2t[s.child[(size_t)g * n_slots + c]];
          fg[(size_t)c * n + off + b] = ct;
          bs[(size_t)c * n + off + b] = ct;
        }
        if (s.parent[g] >= 0) { fs[off + b] = off + b; bg[off + b] = off + b; }
      }
    } else {
      for (int c = 0; c < n_slots; c++) {
        int m = lvl_gather(&s, l, c, tmp);
        for (int b = 0; b < m; b++) { fg[(size_t)c * n + off + b] = tmp[b]; bs[(size_t)c * n + off + b] = tmp[b]; }
      }
      int m = lvl_scatter(&s, l, tmp);
      for (int b = 0; b < m; b++) { fs[off + b] = tmp[b]; bg[off + b] = tmp[b]; }
    }
  }
  free(tmp);
  int levels = s.n_levels;
  oracle_sched_free(&s);
  return levels;
}

/* ------------------------------------------------------------------------- */
/* Graph ops on rows: restatement of the three row-copy kernels               */
/* (cavs/backend/functor_batched_memcpy.cuh:34-75).                            */
/* ------------------------------------------------------------------------- */

void cavs_oracle_gather_rows(float *out, const float *inp, const int *ids, int n_ids, int row) {
  for (int b = 0; b < n_ids; b++) memcpy(out + (size_t)b * row, inp + (size_t)ids[b] * row, sizeof(float) * (size_t)row);
}
void cavs_oracle_scatter_rows(float *out, const int *ids, const float *inp, int n_ids, int row) {
  for (int b = 0; b < n_ids; b++) memcpy(out + (size_t)ids[b] * row, inp + (size_t)b * row, sizeof(float) * (size_t)row);
}
/* The zero-fill kernel ignores the id values and clears the first n_ids rows
 * (functor_batched_memcpy.cuh:64-75). */
void cavs_oracle_zero_rows(float *out, int n_ids, int row) {
  memset(out, 0, sizeof(float) * (size_t)n_ids * (size_t)row);
}

/* ------------------------------------------------------------------------- */
/* Numerics helpers                                                           */
/* ------------------------------------------------------------------------- */

static inline float bf16_round(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return x; /* NaN */
  u += 0x7fffu + ((u >> 16) & 1u);
  u &= 0xffff0000u;
  memcpy(&x, &u, 4);
  return x;
}
static void round_copy(float *dst, const float *src, size_t n, int bf16) {
  if (!bf16) { memcpy(dst, src, n * sizeof(float)); return; }
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; i++) dst[i] = bf16_round(src[i]);
}
static inline float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); } /* expression.h:40-72 */

/* C[m,n] (+)= A[m,k] * B[k,n], row-major.  Every C[i,j] is accumulated in ascending k order starting from its
 * old value (or zero), exactly like the three-loop form; the loops are only blocked for the caches (C blocks of
 * GEMM_MC x GEMM_NC, K in steps of GEMM_KC, register tiles of 4 rows x 16 columns that the compiler keeps in
 * vector registers), so that the timed CPU baseline is bound by arithmetic, not by re-reading B from memory. */
#define GEMM_MC 64
#define GEMM_NC 256
#define GEMM_KC 256
typedef float gemm_v8 __attribute__((vector_size(32), aligned(4)));   /* eight floats, unaligned loads allowed */
static void gemm_block(float *C, const float *A, const float *B, int n, int k, int i0, int i1, int j0, int j1, int p0, int p1) {
  int i = i0;
  for (; i + 4 <= i1; i += 4) {
    const float *a0 = A + (size_t)i * k, *a1 = a0 + k, *a2 = a1 + k, *a3 = a2 + k;
    int j = j0;
    for (; j + 16 <= j1; j += 16) {
      float *c0 = C + (size_t)i * n + j, *c1 = c0 + n, *c2 = c1 + n, *c3 = c2 + n;
      gemm_v8 r00 = *(gemm_v8 *)c0, r01 = *(gemm_v8 *)(c0 + 8), r10 = *(gemm_v8 *)c1, r11 = *(gemm_v8 *)(c1 + 8);
      gemm_v8 r20 = *(gemm_v8 *)c2, r21 = *(gemm_v8 *)(c2 + 8), r30 = *(gemm_v8 *)c3, r31 = *(gemm_v8 *)(c3 + 8);
      for (int p = p0; p < p1; p++) {
        const float *b = B + (size_t)p * n + j;
        const gemm_v8 b0 = *(const gemm_v8 *)b, b1 = *(const gemm_v8 *)(b + 8);
        r00 += a0[p] * b0; r01 += a0[p] * b1;
        r10 += a1[p] * b0; r11 += a1[p] * b1;
        r20 += a2[p] * b0; r21 += a2[p] * b1;
        r30 += a3[p] * b0; r31 += a3[p] * b1;
      }
      *(gemm_v8 *)c0 = r00; *(gemm_v8 *)(c0 + 8) = r01; *(gemm_v8 *)c1 = r10; *(gemm_v8 *)(c1 + 8) = r11;
      *(gemm_v8 *)c2 = r20; *(gemm_v8 *)(c2 + 8) = r21; *(gemm_v8 *)c3 = r30; *(gemm_v8 *)(c3 + 8) = r31;
    }
    for (; j < j1; j++)
      for (int r = 0; r < 4; r++) {
        float acc = C[(size_t)(i + r) * n + j];
        for (int p = p0; p < p1; p++) acc += A[(size_t)(i + r) * k + p] * B[(size_t)p * n + j];
        C[(size_t)(i + r) * n + j] = acc;
      }
  }
  for (; i < i1; i++) {
    float *c = C + (size_t)i * n;
    for (int p = p0; p < p1; p++) {
      const float av = A[(size_t)i * k + p];
      const float *b = B + (size_t)p * n;
      for (int j = j0; j < j1; j++) c[j] += av * b[j];
    }
  }
}
static void gemm_nn(float *C, const float *A, const float *B, int m, int n, int k, int accumulate) {
  const int mb = (m + GEMM_MC - 1) / GEMM_MC, nb = (n + GEMM_NC - 1) / GEMM_NC;
#pragma omp parallel for schedule(dynamic)
  for (int blk = 0; blk < mb * nb; blk++) {
    const int i0 = (blk / nb) * GEMM_MC, j0 = (blk % nb) * GEMM_NC;
    const int i1 = i0 + GEMM_MC < m ? i0 + GEMM_MC : m, j1 = j0 + GEMM_NC < n ? j0 + GEMM_NC : n;
    if (!accumulate)
      for (int i = i0; i < i1; i++) memset(C + (size_t)i * n + j0, 0, sizeof(float) * (size_t)(j1 - j0));
    for (int p0 = 0; p0 < k; p0 += GEMM_KC)
      gemm_block(C, A, B, n, k, i0, i1, j0, j1, p0, p0 + GEMM_KC < k ? p0 + GEMM_KC : k);
  }
}
/* dst[c,r] = src[r,c] for src [rows,cols] */
static float *transposed(const float *src, int rows, int cols) {
  float *dst = (float *)malloc(sizeof(float) * (size_t)rows * (size_t)cols + 4);
#pragma omp parallel for schedule(static)
  for (int c0 = 0; c0 < cols; c0 += 32)
    for (int r = 0; r < rows; r++)
      for (int c = c0; c < c0 + 32 && c < cols; c++) dst[(size_t)c * rows + r] = src[(size_t)r * cols + c];
  return dst;
}
/* C[m,n] = A[m,k] * B[n,k]^T: B is transposed once, then the same k-ordered sums as gemm_nn. */
static void gemm_nt(float *C, const float *A, const float *B, int m, int n, int k, int accumulate) {
  float *Bt = transposed(B, n, k);
  gemm_nn(C, A, Bt, m, n, k, accumulate);
  free(Bt);
}
/* C[m,n] (+)= A[k,m]^T * B[k,n]  (weight gradients: reduction over rows, in row order) */
static void gemm_tn(float *C, const float *A, const float *B, int m, int n, int k, int accumulate) {
  float *At = transposed(A, k, m);
  gemm_nn(C, At, B, m, n, k, accumulate);
  free(At);
}

/* ------------------------------------------------------------------------- */
/* Child-sum Tree-LSTM with n_slots child slots; n_slots = 2 is the reference */
/* vertex function (apps/paper/tree-lstm-cavs.cc:107-172); n_slots = 1 with    */
/* permuted parameter blocks is the chain LSTM                                */
/* (apps/paper/seq-lstm-cavs.cc:45-86).                                        */
/*                                                                             */
/* Parameter layout (tree-lstm-cavs.cc:107-127):                               */
/*   Emb [V,E]; W [E,4H] column blocks i,o,u,f; U = U_iou [H,3H] (i,o,u)       */
/*   followed by U_f [H,H]; B [4H] blocks i,f,u,o; Wc [C,H]; bc [C].           */
/* Loss head: FullyConnected + SoftmaxEntropyLoss                              */
/*   (op_impl_fullyconnected_cublas.cc:33-85,                                  */
/*    op_impl_softmax_entropy_logits_loss.cu:106-140,213-250).                 */
/* ------------------------------------------------------------------------- */

typedef struct {
  int n;          /* vertices (rows), tensor-id order                    */
  int n_levels;
  int hidden;     /* H */
  int embed;      /* E */
  int vocab;      /* V */
  int classes;    /* C */
  int n_slots;    /* K */
  int gemm_bf16;  /* round every GEMM operand to bf16 first (extension)  */
  int loss_rows;  /* divisor of the loss gradient; the reference uses the row count of the logits */
  int preact_bf16; /* also round the forward GEMM outputs (gate pre-activations) to bf16 (extension) */
} cavs_oracle_cfg;

typedef struct {
  /* saved by forward for backward, all [n, ...] in tensor-id order */
  float *x;      /* [n,E]    embedded inputs                              */
  float *gath;   /* [K][n,2H] gathered child states h|c                   */
  float *gates;  /* [n,(3+K)H] i,o,u,f_0..f_{K-1}                         */
  float *state;  /* [n,2H]   h|c                                          */
} oracle_saved;

/* Forward + loss + backward.  Outputs: state [n,2H], loss [n], and the gradients
 * (overwritten, not accumulated).  label < 0 marks a row without a loss term
 * (root-only losses, an extension).  Returns 0. */
/* One layer of a stack (apps/lstm stacks layers by feeding a layer's h into the next one's input):
 *   x_dense != NULL: the inputs are the rows x_dense[t,:] ([n,E], tensor-id order) instead of Emb[tok[t]];
 *                    tok, Emb and dEmb are ignored; dx_out ([n,E], optional) receives d(loss)/d(x_dense);
 *   dh_ext  != NULL: d(loss)/d(h) of every vertex comes from the layer above ([n,H]) and the loss head is
 *                    skipped; label, Wc, bc, dWc, dbc are ignored and loss_out is zero. */
static int treelstm_layer(const cavs_oracle_cfg *cfg, const int *level_off, const int *fg, const int *fs,
                          const int *bg, const int *bs, const int *tok, const int *label, const float *Emb,
                          const float *W, const float *U, const float *B, const float *Wc, const float *bc,
                          float *state_out, float *loss_out, float *dEmb, float *dW, float *dU, float *dB,
                          float *dWc, float *dbc, float *dstate_dbg, const float *x_dense, const float *dh_ext,
                          float *dx_out);

int cavs_oracle_treelstm_fwd_bwd(const cavs_oracle_cfg *cfg, const int *level_off, const int *fg, const int *fs,
                                 const int *bg, const int *bs, const int *tok, const int *label, const float *Emb,
                                 const float *W, const float *U, const float *B, const float *Wc, const float *bc,
                                 float *state_out, float *loss_out, float *dEmb, float *dW, float *dU, float *dB,
                                 float *dWc, float *dbc, float *dstate_dbg /* optional [n,2H]: d(h|c) seen by each row */) {
  return treelstm_layer(cfg, level_off, fg, fs, bg, bs, tok, label, Emb, W, U, B, Wc, bc, state_out, loss_out, dEmb, dW, dU,
                        dB, dWc, dbc, dstate_dbg, NULL, NULL, NULL);
}

int cavs_oracle_treelstm_layer(const cavs_oracle_cfg *cfg, const int *level_off, const int *fg, const int *fs,
                               const int *bg, const int *bs, const int *tok, const int *label, const float *Emb,
                               const float *W, const float *U, const float *B, const float *Wc, const float *bc,
                               float *state_out, float *loss_out, float *dEmb, float *dW, float *dU, float *dB,
                               float *dWc, float *dbc, const float *x_dense, const float *dh_ext, float *dx_out) {
  return treelstm_layer(cfg, level_off, fg, fs, bg, bs, tok, label, Emb, W, U, B, Wc, bc, state_out, loss_out, dEmb, dW, dU,
                        dB, dWc, dbc, NULL, x_dense, dh_ext, dx_out);
}

static int treelstm_layer(const cavs_oracle_cfg *cfg, const int *level_off, const int *fg, const int *fs,
                          const int *bg, const int *bs, const int *tok, const int *label, const float *Emb,
                          const float *W, const float *U, const float *B, const float *Wc, const float *bc,
                          float *state_out, float *loss_out, float *dEmb, float *dW, float *dU, float *dB,
                          float *dWc, float *dbc, float *dstate_dbg, const float *x_dense, const float *dh_ext,
                          float *dx_out) {
  const int n = cfg->n, H = cfg->hidden, E = cfg->embed, C = cfg->classes, K = cfg->n_slots, V = cfg->vocab;
  const int bf = cfg->gemm_bf16;
  const size_t G = (size_t)(3 + K) * H;
  const float *U_iou = U, *U_f = U + (size_t)3 * H * H;
  const float *b_i = B, *b_f = B + H, *b_u = B + 2 * H, *b_o = B + 3 * H;

  float *Wr = (float *)malloc(sizeof(float) * (size_t)E * 4 * H);
  float *Ur = (float *)malloc(sizeof(float) * (size_t)4 * H * H);
  round_copy(Wr, W, (size_t)E * 4 * H, bf);
  round_copy(Ur, U, (size_t)4 * H * H, bf);
  const float *Ur_iou = Ur, *Ur_f = Ur + (size_t)3 * H * H;
  (void)U_iou; (void)U_f;

  size_t nn = (size_t)(n > 0 ? n : 1);
  float *x = (float *)calloc(nn * E, sizeof(float));
  float *a = (float *)calloc(nn * 4 * H, sizeof(float));
  float *gath = (float *)calloc(nn * 2 * H * K, sizeof(float));
  float *gates = (float *)calloc(nn * G, sizeof(float));
  float *state = (float *)calloc(nn * 2 * H, sizeof(float));
  float *mailbox = (float *)calloc(nn * 2 * H, sizeof(float)); /* graph_session.cc:173-185 */
  float *s = (float *)calloc(nn * H, sizeof(float));
  float *hk = (float *)calloc(nn * H * K, sizeof(float));
  float *p = (float *)calloc(nn * 3 * H, sizeof(float));
  float *q = (float *)calloc(nn * H * K, sizeof(float));

  /* Embedding lookup for every vertex, leaf or not (op_impl_embedding_lookup.cu:23-35),
   * then the input projection.  x does not depend on the level, so one product over
   * all rows equals the reference's per-level products row for row. */
#pragma omp parallel for schedule(static)
  for (int t = 0; t < n; t++) {
    const float *src;
    if (x_dense) {
      src = x_dense + (size_t)t * E;
    } else {
      int id = tok[t];
      if (id < 0 || id >= V) id = 0;
      src = Emb + (size_t)id * E;
    }
    for (int e = 0; e < E; e++) x[(size_t)t * E + e] = bf ? bf16_round(src[e]) : src[e];
  }
  gemm_nn(a, x, Wr, n, 4 * H, E, 0);
  if (cfg->preact_bf16) round_copy(a, a, (size_t)n * 4 * H, 1);

  for (int l = 0; l < cfg->n_levels; l++) {
    const int off = level_off[l], cnt = level_off[l + 1] - off;
    /* Gather (op_impl_graphop.cu:32-90): child state rows out of the mailbox. */
    for (int c = 0; c < K; c++)
#pragma omp parallel for schedule(static)
      for (int t = off; t < off + cnt; t++) {
        float *dst = gath + ((size_t)c * n + t) * 2 * H;
        int src = fg[(size_t)c * n + t];
        if (src >= 0) memcpy(dst, mailbox + (size_t)src * 2 * H, sizeof(float) * 2 * H);
        else memset(dst, 0, sizeof(float) * 2 * H);
      }
    /* h_lr = h_l + h_r (tree-lstm-cavs.cc:136) and the recurrent products. */
#pragma omp parallel for schedule(static)
    for (int t = off; t < off + cnt; t++)
      for (int j = 0; j < H; j++) {
        float acc = gath[((size_t)0 * n + t) * 2 * H + j];
        for (int c = 1; c < K; c++) acc += gath[((size_t)c * n + t) * 2 * H + j];
        s[(size_t)t * H + j] = bf ? bf16_round(acc) : acc;
        for (int c = 0; c < K; c++) {
          float hv = gath[((size_t)c * n + t) * 2 * H + j];
          hk[((size_t)c * n + t) * H + j] = bf ? bf16_round(hv) : hv;
        }
      }
    gemm_nn(p + (size_t)off * 3 * H, s + (size_t)off * H, Ur_iou, cnt, 3 * H, H, 0);
    for (int c = 0; c < K; c++)
      gemm_nn(q + ((size_t)c * n + off) * H, hk + ((size_t)c * n + off) * H, Ur_f, cnt, H, H, 0);
    if (cfg->preact_bf16) {
      round_copy(p + (size_t)off * 3 * H, p + (size_t)off * 3 * H, (size_t)cnt * 3 * H, 1);
      for (int c = 0; c < K; c++)
        round_copy(q + ((size_t)c * n + off) * H, q + ((size_t)c * n + off) * H, (size_t)cnt * H, 1);
    }
    /* Gates and cell (tree-lstm-cavs.cc:159-168), add order (xW + hU) + b. */
#pragma omp parallel for schedule(static)
    for (int t = off; t < off + cnt; t++) {
      const float *at = a + (size_t)t * 4 * H, *pt = p + (size_t)t * 3 * H;
      float *gt = gates + (size_t)t * G, *st = state + (size_t)t * 2 * H;
      for (int j = 0; j < H; j++) {
        float gi = sigmoidf_((at[j] + pt[j]) + b_i[j]);
        float go = sigmoidf_((at[H + j] + pt[H + j]) + b_o[j]);
        float gu = tanhf((at[2 * H + j] + pt[2 * H + j]) + b_u[j]);
        float cc = gi * gu;
        for (int c = 0; c < K; c++) {
          float gf = sigmoidf_((at[3 * H + j] + q[((size_t)c * n + t) * H + j]) + b_f[j]);
          gt[(size_t)(3 + c) * H + j] = gf;
          cc = cc + gf * gath[((size_t)c * n + t) * 2 * H + H + j];
        }
        gt[j] = gi; gt[H + j] = go; gt[2 * H + j] = gu;
        st[H + j] = cc;
        st[j] = go * tanhf(cc);
      }
    }
    /* Scatter (op_impl_graphop.cu:108-161): h|c into the mailbox (one target row per vertex). */
#pragma omp parallel for schedule(static)
    for (int t = off; t < off + cnt; t++)
      if (fs[t] >= 0) memcpy(mailbox + (size_t)fs[t] * 2 * H, state + (size_t)t * 2 * H, sizeof(float) * 2 * H);
  }
  if (state_out) memcpy(state_out, state, sizeof(float) * (size_t)n * 2 * H);

  /* Loss head over the pushed h rows. */
  float *dOut = (float *)calloc(nn * H, sizeof(float));
  float *dz = (float *)calloc(nn * (size_t)(C > 0 ? C : 1), sizeof(float));
  const float inv_rows = 1.0f / (float)(cfg->loss_rows > 0 ? cfg->loss_rows : (n > 0 ? n : 1));
  if (dh_ext) {
    memcpy(dOut, dh_ext, sizeof(float) * (size_t)n * H);
    if (loss_out) memset(loss_out, 0, sizeof(float) * (size_t)n);
  }
#pragma omp parallel for schedule(static)
  for (int t = 0; t < (dh_ext ? 0 : n); t++) {
    float z[64];
    float *zz = C <= 64 ? z : (float *)malloc(sizeof(float) * C);
    const float *h = state + (size_t)t * 2 * H;
    float mx = -INFINITY;
    for (int c = 0; c < C; c++) {
      float acc = 0.0f;
      for (int j = 0; j < H; j++) acc += h[j] * Wc[(size_t)c * H + j];
      zz[c] = acc + bc[c];
      if (zz[c] > mx) mx = zz[c];
    }
    float den = 0.0f;
    for (int c = 0; c < C; c++) { zz[c] = expf(zz[c] - mx); den += zz[c]; }
    int y = label[t];
    if (y >= 0) {
      if (loss_out) loss_out[t] = -logf(zz[y] / den);
      /* dx = (softmax - onehot) / rows, upstream gradient ignored
       * (op_impl_softmax_entropy_logits_loss.cu:151-160,244-245). */
      for (int c = 0; c < C; c++) dz[(size_t)t * C + c] = (zz[c] / den - (c == y ? 1.0f : 0.0f)) * inv_rows;
    } else {
      if (loss_out) loss_out[t] = 0.0f;
    }
    for (int j = 0; j < H; j++) {
      float acc = 0.0f;
      for (int c = 0; c < C; c++) acc += dz[(size_t)t * C + c] * Wc[(size_t)c * H + j];
      dOut[(size_t)t * H + j] = acc;
    }
    if (zz != z) free(zz);
  }
  /* dWc = dz^T h, dbc = column sums (op_impl_fullyconnected_cublas.cc:157-167). */
  for (int c = 0; c < (dh_ext ? 0 : C); c++) {
    float accb = 0.0f;
    for (int t = 0; t < n; t++) accb += dz[(size_t)t * C + c];
    dbc[c] = accb;
#pragma omp parallel for schedule(static)
    for (int j = 0; j < H; j++) {
      float acc = 0.0f;
      for (int t = 0; t < n; t++) acc += dz[(size_t)t * C + c] * state[(size_t)t * 2 * H + j];
      dWc[(size_t)c * H + j] = acc;
    }
  }

  /* Backward sweep, last level first (statement.cc:87-123). */
  float *dA = (float *)calloc(nn * 4 * H, sizeof(float));   /* zi|zo|zu|sum_c zf_c */
  float *zf = (float *)calloc(nn * H * K, sizeof(float));
  float *dck = (float *)calloc(nn * H * K, sizeof(float));
  float *ds = (float *)calloc(nn * H, sizeof(float));
  float *dq = (float *)calloc(nn * H * K, sizeof(float));
  float *dP_r = (float *)calloc(nn * 3 * H, sizeof(float));
  float *zf_r = (float *)calloc(nn * H * K, sizeof(float));
  for (int l = cfg->n_levels - 1; l >= 0; l--) {
    const int off = level_off[l], cnt = level_off[l + 1] - off;
#pragma omp parallel for schedule(static)
    for (int t = off; t < off + cnt; t++) {
      const float *gt = gates + (size_t)t * G, *st = state + (size_t)t * 2 * H;
      const float *m = bg[t] >= 0 ? mailbox + (size_t)bg[t] * 2 * H : NULL;
      float *dat = dA + (size_t)t * 4 * H;
      for (int j = 0; j < H; j++) {
        float mh = m ? m[j] : 0.0f, mc = m ? m[H + j] : 0.0f;
        float dh = dOut[(size_t)t * H + j] + mh;
        if (dstate_dbg) { dstate_dbg[(size_t)t * 2 * H + j] = dh; }
        float gi = gt[j], go = gt[H + j], gu = gt[2 * H + j];
        float th = tanhf(st[H + j]);
        float d_o = dh * th;
        float dc = mc + (dh * go) * (1.0f - th * th);
        if (dstate_dbg) { dstate_dbg[(size_t)t * 2 * H + H + j] = dc; }
        float zi = (dc * gu) * gi * (1.0f - gi);
        float zo = d_o * go * (1.0f - go);
        float zu = (dc * gi) * (1.0f - gu * gu);
        float zfs = 0.0f;
        for (int c = 0; c < K; c++) {
          float gf = gt[(size_t)(3 + c) * H + j];
          float cchild = gath[((size_t)c * n + t) * 2 * H + H + j];
          float z = (dc * cchild) * gf * (1.0f - gf);
          zf[((size_t)c * n + t) * H + j] = z;
          zf_r[((size_t)c * n + t) * H + j] = bf ? bf16_round(z) : z;
          dck[((size_t)c * n + t) * H + j] = dc * gf;
          zfs += z;
        }
        dat[j] = zi; dat[H + j] = zo; dat[2 * H + j] = zu; dat[3 * H + j] = zfs;
        dP_r[(size_t)t * 3 * H + j] = bf ? bf16_round(zi) : zi;
        dP_r[(size_t)t * 3 * H + H + j] = bf ? bf16_round(zo) : zo;
        dP_r[(size_t)t * 3 * H + 2 * H + j] = bf ? bf16_round(zu) : zu;
      }
    }
    /* dX = dY W^T (op_decl_matmul.cc:21-31). */
    gemm_nt(ds + (size_t)off * H, dP_r + (size_t)off * 3 * H, Ur_iou, cnt, H, 3 * H, 0);
    for (int c = 0; c < K; c++)
      gemm_nt(dq + ((size_t)c * n + off) * H, zf_r + ((size_t)c * n + off) * H, Ur_f, cnt, H, H, 0);
    /* Scatter(Child=c) of d(h_c|c_c) (op_decl_graphop.cc:25-41); a vertex has one parent, so targets are distinct. */
    for (int c = 0; c < K; c++)
#pragma omp parallel for schedule(static)
      for (int t = off; t < off + cnt; t++) {
        int dst = bs[(size_t)c * n + t];
        if (dst < 0) continue;
        float *mrow = mailbox + (size_t)dst * 2 * H;
        for (int j = 0; j < H; j++) {
          mrow[j] = ds[(size_t)t * H + j] + dq[((size_t)c * n + t) * H + j];
          mrow[H + j] = dck[((size_t)c * n + t) * H + j];
        }
      }
  }

  /* Deferred weight gradients over all rows at once (batch_weight_updater.h:10-85,
   * statement.cc:112-117). */
  float *dA_r = (float *)malloc(sizeof(float) * nn * 4 * H);
  round_copy(dA_r, dA, (size_t)n * 4 * H, bf);
  gemm_tn(dW, x, dA_r, E, 4 * H, n, 0);
  /* dU_iou = S^T dP ; dU_f = sum_c H_c^T Zf_c.  Operands are strided views: gather
   * the i,o,u block of dA (= dP). */
  gemm_tn(dU, s, dP_r, H, 3 * H, n, 0);
  for (int c = 0; c < K; c++)
    gemm_tn(dU + (size_t)3 * H * H, hk + (size_t)c * n * H, zf_r + (size_t)c * n * H, H, H, n, c > 0);
  /* Bias gradient = column sums, bias order i,f,u,o (tree-lstm-cavs.cc:120-123). */
#pragma omp parallel for schedule(static)
  for (int j = 0; j < H; j++) {
    float si = 0, so = 0, su = 0, sf = 0;
    for (int t = 0; t < n; t++) {
      const float *d = dA + (size_t)t * 4 * H;
      si += d[j]; so += d[H + j]; su += d[2 * H + j]; sf += d[3 * H + j];
    }
    dB[j] = si; dB[H + j] = sf; dB[2 * H + j] = su; dB[3 * H + j] = so;
  }
  /* dx = dA W^T, accumulated into the embedding rows in ascending row order
   * (the reference uses atomicAdd, op_impl_embedding_lookup.cu:91-103; the sum is the
   * same up to fp32 reassociation). */
  float *dX = (float *)malloc(sizeof(float) * nn * E);
  gemm_nt(dX, dA_r, Wr, n, E, 4 * H, 0);
  if (dx_out) memcpy(dx_out, dX, sizeof(float) * (size_t)n * E);
  if (!x_dense) {
    memset(dEmb, 0, sizeof(float) * (size_t)V * E);
    /* column blocks in parallel; within a column the rows are still added in ascending order */
#pragma omp parallel for schedule(static)
    for (int e0 = 0; e0 < E; e0 += 64)
      for (int t = 0; t < n; t++) {
        int id = tok[t];
        if (id < 0 || id >= V) id = 0;
        for (int e = e0; e < e0 + 64 && e < E; e++) dEmb[(size_t)id * E + e] += dX[(size_t)t * E + e];
      }
  }

  free(Wr); free(Ur); free(x); free(a); free(gath); free(gates); free(state); free(mailbox);
  free(s); free(hk); free(p); free(q); free(dOut); free(dz); free(dA); free(zf); free(dck);
  free(ds); free(dq); free(dP_r); free(zf_r); free(dA_r); free(dX);
  return 0;
}

/* ------------------------------------------------------------------------- */
/* Child-sum Tree-GRU with n_slots child slots (EXTENSION: the reference has   */
/* no GRU; this definition is the contract, parity unpinned).                  */
/*   a = x W  (W [E,3H], column blocks r,z,n);  ht = sum_k h_k                 */
/*   r_k = sigmoid((a_r + h_k U_r) + b_r)       z = sigmoid((a_z + ht U_z) + b_z) */
/*   m = sum_k r_k o h_k                        n = tanh((a_n + m U_n) + b_n)  */
/*   h = (1 - z) o ht + z o n                                                  */
/* U = U_r [H,H] | U_z [H,H] | U_n [H,H]; B [3H] blocks r,z,n; state row = h.  */
/* Missing children contribute zero rows.  Same loss head and index tables as  */
/* the Tree-LSTM; the mailbox row is d(h) only.                                */
/* ------------------------------------------------------------------------- */
int cavs_oracle_treegru_fwd_bwd(const cavs_oracle_cfg *cfg, const int *level_off, const int *fg, const int *fs,
                                const int *bg, const int *bs, const int *tok, const int *label, const float *Emb,
                                const float *W, const float *U, const float *B, const float *Wc, const float *bc,
                                float *state_out, float *loss_out, float *dEmb, float *dW, float *dU, float *dB,
                                float *dWc, float *dbc) {
  const int n = cfg->n, H = cfg->hidden, E = cfg->embed, C = cfg->classes, K = cfg->n_slots, V = cfg->vocab;
  const int bf = cfg->gemm_bf16;
  const size_t nn = (size_t)(n > 0 ? n : 1);
  const float *b_r = B, *b_z = B + H, *b_n = B + 2 * H;
  float *Wr = (float *)malloc(sizeof(float) * (size_t)E * 3 * H);
  float *Ur = (float *)malloc(sizeof(float) * (size_t)3 * H * H);
  round_copy(Wr, W, (size_t)E * 3 * H, bf);
  round_copy(Ur, U, (size_t)3 * H * H, bf);
  const float *U_r = Ur, *U_z = Ur + (size_t)H * H, *U_n = Ur + (size_t)2 * H * H;

  float *x = (float *)calloc(nn * E, sizeof(float));
  float *a = (float *)calloc(nn * 3 * H, sizeof(float));
  float *hk = (float *)calloc(nn * H * K, sizeof(float));      /* [K][n,H] gathered child h (fp32)     */
  float *hk_r = (float *)calloc(nn * H * K, sizeof(float));    /* GEMM-operand copy                    */
  float *ht = (float *)calloc(nn * H, sizeof(float));
  float *ht_r = (float *)calloc(nn * H, sizeof(float));
  float *pr = (float *)calloc(nn * H * K, sizeof(float));
  float *pz = (float *)calloc(nn * H, sizeof(float));
  float *pn = (float *)calloc(nn * H, sizeof(float));
  float *rk = (float *)calloc(nn * H * K, sizeof(float));
  float *m = (float *)calloc(nn * H, sizeof(float));
  float *m_r = (float *)calloc(nn * H, sizeof(float));
  float *zg = (float *)calloc(nn * H, sizeof(float));
  float *ng = (float *)calloc(nn * H, sizeof(float));
  float *state = (float *)calloc(nn * H, sizeof(float));
  float *mailbox = (float *)calloc(nn * H, sizeof(float));

  for (int t = 0; t < n; t++) {
    int id = tok[t];
    if (id < 0 || id >= V) id = 0;
    for (int e = 0; e < E; e++) x[(size_t)t * E + e] = bf ? bf16_round(Emb[(size_t)id * E + e]) : Emb[(size_t)id * E + e];
  }
  gemm_nn(a, x, Wr, n, 3 * H, E, 0);
  if (cfg->preact_bf16) for (size_t i = 0; i < (size_t)n * 3 * H; i++) a[i] = bf16_round(a[i]);

  for (int l = 0; l < cfg->n_levels; l++) {
    const int off = level_off[l], cnt = level_off[l + 1] - off;
    for (int t = off; t < off + cnt; t++)
      for (int j = 0; j < H; j++) {
        float acc = 0.0f;
        for (int c = 0; c < K; c++) {
          int src = fg[(size_t)c * n + t];
          float hv = src >= 0 ? mailbox[(size_t)src * H + j] : 0.0f;
          hk[((size_t)c * n + t) * H + j] = hv;
          hk_r[((size_t)c * n + t) * H + j] = bf ? bf16_round(hv) : hv;
          acc = (c == 0) ? hv : acc + hv;
        }
        ht[(size_t)t * H + j] = acc;
        ht_r[(size_t)t * H + j] = bf ? bf16_round(acc) : acc;
      }
    gemm_nn(pz + (size_t)off * H, ht_r + (size_t)off * H, U_z, cnt, H, H, 0);
    for (int c = 0; c < K; c++)
      gemm_nn(pr + ((size_t)c * n + off) * H, hk_r + ((size_t)c * n + off) * H, U_r, cnt, H, H, 0);
    if (cfg->preact_bf16) {
      for (size_t i = (size_t)off * H; i < (size_t)(off + cnt) * H; i++) pz[i] = bf16_round(pz[i]);
      for (int c = 0; c < K; c++)
        for (size_t i = ((size_t)c * n + off) * H; i < ((size_t)c * n + off + cnt) * H; i++) pr[i] = bf16_round(pr[i]);
    }
    for (int t = off; t < off + cnt; t++)
      for (int j = 0; j < H; j++) {
        float acc = 0.0f;
        for (int c = 0; c < K; c++) {
          float r = sigmoidf_((a[(size_t)t * 3 * H + j] + pr[((size_t)c * n + t) * H + j]) + b_r[j]);
          rk[((size_t)c * n + t) * H + j] = r;
          acc += r * hk[((size_t)c * n + t) * H + j];
        }
        m[(size_t)t * H + j] = acc;
        m_r[(size_t)t * H + j] = bf ? bf16_round(acc) : acc;
      }
    gemm_nn(pn + (size_t)off * H, m_r + (size_t)off * H, U_n, cnt, H, H, 0);
    if (cfg->preact_bf16) for (size_t i = (size_t)off * H; i < (size_t)(off + cnt) * H; i++) pn[i] = bf16_round(pn[i]);
    for (int t = off; t < off + cnt; t++)
      for (int j = 0; j < H; j++) {
        float z = sigmoidf_((a[(size_t)t * 3 * H + H + j] + pz[(size_t)t * H + j]) + b_z[j]);
        float g = tanhf((a[(size_t)t * 3 * H + 2 * H + j] + pn[(size_t)t * H + j]) + b_n[j]);
        zg[(size_t)t * H + j] = z;
        ng[(size_t)t * H + j] = g;
        state[(size_t)t * H + j] = (1.0f - z) * ht[(size_t)t * H + j] + z * g;
      }
    for (int t = off; t < off + cnt; t++)
      if (fs[t] >= 0) memcpy(mailbox + (size_t)fs[t] * H, state + (size_t)t * H, sizeof(float) * H);
  }
  if (state_out) memcpy(state_out, state, sizeof(float) * (size_t)n * H);

  /* Loss head (same as the Tree-LSTM's). */
  float *dOut = (float *)calloc(nn * H, sizeof(float));
  float *dz = (float *)calloc(nn * C, sizeof(float));
  const float inv_rows = 1.0f / (float)(cfg->loss_rows > 0 ? cfg->loss_rows : (n > 0 ? n : 1));
  for (int t = 0; t < n; t++) {
    float *zz = (float *)malloc(sizeof(float) * C);
    const float *h = state + (size_t)t * H;
    float mx = -INFINITY;
    for (int c = 0; c < C; c++) {
      float acc = 0.0f;
      for (int j = 0; j < H; j++) acc += h[j] * Wc[(size_t)c * H + j];
      zz[c] = acc + bc[c];
      if (zz[c] > mx) mx = zz[c];
    }
    float den = 0.0f;
    for (int c = 0; c < C; c++) { zz[c] = expf(zz[c] - mx); den += zz[c]; }
    int y = label[t];
    if (loss_out) loss_out[t] = (y >= 0) ? -logf(zz[y] / den) : 0.0f;
    if (y >= 0) for (int c = 0; c < C; c++) dz[(size_t)t * C + c] = (zz[c] / den - (c == y ? 1.0f : 0.0f)) * inv_rows;
    for (int j = 0; j < H; j++) {
      float acc = 0.0f;
      for (int c = 0; c < C; c++) acc += dz[(size_t)t * C + c] * Wc[(size_t)c * H + j];
      dOut[(size_t)t * H + j] = acc;
    }
    free(zz);
  }
  for (int c = 0; c < C; c++) {
    float accb = 0.0f;
    for (int t = 0; t < n; t++) accb += dz[(size_t)t * C + c];
    dbc[c] = accb;
    for (int j = 0; j < H; j++) {
      float acc = 0.0f;
      for (int t = 0; t < n; t++) acc += dz[(size_t)t * C + c] * state[(size_t)t * H + j];
      dWc[(size_t)c * H + j] = acc;
    }
  }

  /* Backward sweep. */
  float *dA = (float *)calloc(nn * 3 * H, sizeof(float));      /* sum_k zr_k | zz | zn */
  float *zz_r = (float *)calloc(nn * H, sizeof(float));
  float *zn_r = (float *)calloc(nn * H, sizeof(float));
  float *zr_r = (float *)calloc(nn * H * K, sizeof(float));
  float *dht = (float *)calloc(nn * H, sizeof(float));
  float *dm = (float *)calloc(nn * H, sizeof(float));
  float *dsz = (float *)calloc(nn * H, sizeof(float));
  float *dqr = (float *)calloc(nn * H * K, sizeof(float));
  for (int l = cfg->n_levels - 1; l >= 0; l--) {
    const int off = level_off[l], cnt = level_off[l + 1] - off;
    for (int t = off; t < off + cnt; t++) {
      const float *mb = bg[t] >= 0 ? mailbox + (size_t)bg[t] * H : NULL;
      for (int j = 0; j < H; j++) {
        float dh = dOut[(size_t)t * H + j] + (mb ? mb[j] : 0.0f);
        float z = zg[(size_t)t * H + j], g = ng[(size_t)t * H + j];
        float zz = (dh * (g - ht[(size_t)t * H + j])) * z * (1.0f - z);
        float zn = (dh * z) * (1.0f - g * g);
        dht[(size_t)t * H + j] = dh * (1.0f - z);
        dA[(size_t)t * 3 * H + H + j] = zz;
        dA[(size_t)t * 3 * H + 2 * H + j] = zn;
        zz_r[(size_t)t * H + j] = bf ? bf16_round(zz) : zz;
        zn_r[(size_t)t * H + j] = bf ? bf16_round(zn) : zn;
      }
    }
    gemm_nt(dm + (size_t)off * H, zn_r + (size_t)off * H, U_n, cnt, H, H, 0);
    gemm_nt(dsz + (size_t)off * H, zz_r + (size_t)off * H, U_z, cnt, H, H, 0);
    for (int t = off; t < off + cnt; t++)
      for (int j = 0; j < H; j++) {
        float acc = 0.0f;
        for (int c = 0; c < K; c++) {
          float r = rk[((size_t)c * n + t) * H + j];
          float zr = (dm[(size_t)t * H + j] * hk[((size_t)c * n + t) * H + j]) * r * (1.0f - r);
          zr_r[((size_t)c * n + t) * H + j] = bf ? bf16_round(zr) : zr;
          acc += zr;
        }
        dA[(size_t)t * 3 * H + j] = acc;
      }
    for (int c = 0; c < K; c++)
      gemm_nt(dqr + ((size_t)c * n + off) * H, zr_r + ((size_t)c * n + off) * H, U_r, cnt, H, H, 0);
    for (int c = 0; c < K; c++)
      for (int t = off; t < off + cnt; t++) {
        int dst = bs[(size_t)c * n + t];
        if (dst < 0) continue;
        for (int j = 0; j < H; j++)
          mailbox[(size_t)dst * H + j] = ((dht[(size_t)t * H + j] + dsz[(size_t)t * H + j]) +
                                          dm[(size_t)t * H + j] * rk[((size_t)c * n + t) * H + j]) +
                                         dqr[((size_t)c * n + t) * H + j];
      }
  }
  /* Deferred weight gradients. */
  float *dA_r = (float *)malloc(sizeof(float) * nn * 3 * H);
  round_copy(dA_r, dA, (size_t)n * 3 * H, bf);
  gemm_tn(dW, x, dA_r, E, 3 * H, n, 0);
  for (int c = 0; c < K; c++) gemm_tn(dU, hk_r + (size_t)c * n * H, zr_r + (size_t)c * n * H, H, H, n, c > 0);
  gemm_tn(dU + (size_t)H * H, ht_r, zz_r, H, H, n, 0);
  gemm_tn(dU + (size_t)2 * H * H, m_r, zn_r, H, H, n, 0);
  for (int j = 0; j < 3 * H; j++) {
    float acc = 0.0f;
    for (int t = 0; t < n; t++) acc += dA[(size_t)t * 3 * H + j];
    dB[j] = acc;
  }
  float *dX = (float *)malloc(sizeof(float) * nn * E);
  gemm_nt(dX, dA_r, Wr, n, E, 3 * H, 0);
  memset(dEmb, 0, sizeof(float) * (size_t)V * E);
  for (int t = 0; t < n; t++) {
    int id = tok[t];
    if (id < 0 || id >= V) id = 0;
    for (int e = 0; e < E; e++) dEmb[(size_t)id * E + e] += dX[(size_t)t * E + e];
  }
  free(Wr); free(Ur); free(x); free(a); free(hk); free(hk_r); free(ht); free(ht_r); free(pr); free(pz); free(pn); free(rk);
  free(m); free(m_r); free(zg); free(ng); free(state); free(mailbox); free(dOut); free(dz); free(dA); free(zz_r); free(zn_r);
  free(zr_r); free(dht); free(dm); free(dsz); free(dqr); free(dA_r); free(dX);
  return 0;
}

/* SGD (op_impl_sgd.cu:15-47): w <- w - lr * g. */
void cavs_oracle_sgd(float *w, const float *g, size_t count, float lr) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < (long)count; i++) w[i] -= lr * g[i];
}
/* Adagrad (extension; the reference registers only SGD): acc += g^2;
 * w <- w - lr * g / (sqrt(acc) + eps). */
void cavs_oracle_adagrad(float *w, float *acc, const float *g, size_t count, float lr, float eps) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < (long)count; i++) {
    float a = acc[i] + g[i] * g[i];
    acc[i] = a;
    w[i] -= lr * g[i] / (sqrtf(a) + eps);
  }
}

int cavs_oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
