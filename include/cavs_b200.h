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
