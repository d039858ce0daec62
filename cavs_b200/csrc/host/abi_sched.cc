// C ABI of the host-side level scheduler, plus status / error plumbing.
#include <atomic>
#include <cstring>
#include <string>
#include <vector>

#include "abi_common.h"
#include "host/sched_handle.h"

namespace cavs_b200 {
namespace {
thread_local std::string g_last_error;
std::atomic<unsigned long long> g_launches{0};
}
void CountLaunch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
int Fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}
}  // namespace cavs_b200


using cavs_b200::Fail;

extern "C" const char* cavs_status_string(int status) {
  switch (status) {
    case CAVS_OK: return "ok";
    case CAVS_ERR_BAD_ARG: return "bad argument";
    case CAVS_ERR_BAD_GRAPH: return "malformed graph";
    case CAVS_ERR_CAPACITY: return "buffer too small";
    case CAVS_ERR_TIMEOUT: return "device wait timed out";
    case CAVS_ERR_CUDA: return "CUDA error";
    case CAVS_ERR_UNSUPPORTED: return "unsupported";
    default: return "unknown status";
  }
}
extern "C" const char* cavs_last_error(void) { return cavs_b200::g_last_error.c_str(); }
extern "C" unsigned long long cavs_launch_count(void) { return cavs_b200::g_launches.load(); }
extern "C" const char* cavs_build_info(void) { return "cavs_b200 0.1 (sm_100a)"; }

extern "C" int cavs_sched_create(cavs_sched** out) {
  CAVS_REQUIRE(out, CAVS_ERR_BAD_ARG, "sched_create: null out");
  *out = new cavs_sched();
  return CAVS_OK;
}
extern "C" void cavs_sched_destroy(cavs_sched* s) { delete s; }

extern "C" int cavs_sched_load(cavs_sched* s, const int32_t* parents, int batch, int max_len, int n_slots) {
  CAVS_REQUIRE(s, CAVS_ERR_BAD_ARG, "sched_load: null handle");
  s->loaded = false;
  std::string err;
  const int rc = s->impl.Load(parents, batch, max_len, n_slots, &err);
  if (rc != CAVS_OK) return Fail(rc, err);
  s->loaded = true;
  return CAVS_OK;
}

extern "C" int cavs_sched_set_order(cavs_sched* s, int order) {
  CAVS_REQUIRE(s, CAVS_ERR_BAD_ARG, "sched_set_order: null handle");
  CAVS_REQUIRE(order == 0 || order == 1, CAVS_ERR_BAD_ARG, "sched_set_order: order must be 0 (batched) or 1 (one vertex per round)");
  s->impl.SetOrder(order == 1 ? cavs_b200::kUnbatched : cavs_b200::kBatched);
  return CAVS_OK;
}

#define SCHED_READY(name) CAVS_REQUIRE(s && s->loaded, CAVS_ERR_BAD_ARG, name ": no graph loaded")

extern "C" int cavs_sched_counts(const cavs_sched* s, int* n_total, int* n_scheduled, int* n_levels, int* max_level_rows) {
  SCHED_READY("sched_counts");
  if (n_total) *n_total = s->impl.n_total();
  if (n_scheduled) *n_scheduled = s->impl.n_scheduled();
  if (n_levels) *n_levels = s->impl.n_levels();
  if (max_level_rows) *max_level_rows = s->impl.max_level_rows();
  return CAVS_OK;
}
extern "C" int cavs_sched_level_offsets(const cavs_sched* s, int32_t* level_off, int capacity) {
  SCHED_READY("sched_level_offsets");
  const auto& v = s->impl.level_off();
  CAVS_REQUIRE(level_off && capacity >= static_cast<int>(v.size()), CAVS_ERR_CAPACITY, "sched_level_offsets: capacity");
  std::memcpy(level_off, v.data(), v.size() * sizeof(int32_t));
  return CAVS_OK;
}
extern "C" int cavs_sched_maps(const cavs_sched* s, int32_t* t2j, int32_t* j2t, int capacity) {
  SCHED_READY("sched_maps");
  const int n = s->impl.n_total();
  CAVS_REQUIRE(capacity >= n, CAVS_ERR_CAPACITY, "sched_maps: capacity");
  if (t2j) std::memcpy(t2j, s->impl.t2j().data(), sizeof(int32_t) * n);
  if (j2t) std::memcpy(j2t, s->impl.j2t().data(), sizeof(int32_t) * n);
  return CAVS_OK;
}
extern "C" int cavs_sched_tables(const cavs_sched* s, int mode, int32_t* fg, int32_t* fs, int32_t* bg, int32_t* bs, int capacity) {
  SCHED_READY("sched_tables");
  CAVS_REQUIRE(fg && fs && bg && bs, CAVS_ERR_BAD_ARG, "sched_tables: null output");
  CAVS_REQUIRE(mode == 0 || mode == 1, CAVS_ERR_BAD_ARG, "sched_tables: mode must be 0 (aligned) or 1 (ref_compat)");
  CAVS_REQUIRE(capacity >= s->impl.n_total(), CAVS_ERR_CAPACITY, "sched_tables: capacity");
  s->impl.Tables(static_cast<cavs_b200::TableMode>(mode), fg, fs, bg, bs);
  return CAVS_OK;
}
extern "C" int cavs_sched_ref_gather(const cavs_sched* s, int level, int slot, int32_t* ids, int capacity, int* n) {
  SCHED_READY("sched_ref_gather");
  CAVS_REQUIRE(level >= 0 && level < s->impl.n_levels() && slot >= 0 && slot < cavs_b200::kMaxSlots && n, CAVS_ERR_BAD_ARG,
               "sched_ref_gather: level/slot out of range");
  std::vector<int32_t> v;
  s->impl.RefGather(level, slot, &v);
  *n = static_cast<int>(v.size());
  CAVS_REQUIRE(capacity >= *n && (ids || *n == 0), CAVS_ERR_CAPACITY, "sched_ref_gather: capacity");
  if (*n) std::memcpy(ids, v.data(), v.size() * sizeof(int32_t));
  return CAVS_OK;
}
extern "C" int cavs_sched_ref_scatter(const cavs_sched* s, int level, int32_t* ids, int capacity, int* n) {
  SCHED_READY("sched_ref_scatter");
  CAVS_REQUIRE(level >= 0 && level < s->impl.n_levels() && n, CAVS_ERR_BAD_ARG, "sched_ref_scatter: level out of range");
  std::vector<int32_t> v;
  s->impl.RefScatter(level, &v);
  *n = static_cast<int>(v.size());
  CAVS_REQUIRE(capacity >= *n && (ids || *n == 0), CAVS_ERR_CAPACITY, "sched_ref_scatter: capacity");
  if (*n) std::memcpy(ids, v.data(), v.size() * sizeof(int32_t));
  return CAVS_OK;
}
extern "C" int cavs_sched_ref_stream(const cavs_sched* s, int32_t* out, int capacity, int* n) {
  SCHED_READY("sched_ref_stream");
  CAVS_REQUIRE(n, CAVS_ERR_BAD_ARG, "sched_ref_stream: null n");
  std::vector<int32_t> v;
  s->impl.RefStream(&v);
  *n = static_cast<int>(v.size());
  CAVS_REQUIRE(out && capacity >= *n, CAVS_ERR_CAPACITY, "sched_ref_stream: capacity");
  std::memcpy(out, v.data(), v.size() * sizeof(int32_t));
  return CAVS_OK;
}

extern "C" int cavs_sched_adjacency(const cavs_sched* s, int32_t* parent_job, int32_t* child_job, int capacity) {
  SCHED_READY("sched_adjacency");
  const int n = s->impl.n_total();
  CAVS_REQUIRE(capacity >= n, CAVS_ERR_CAPACITY, "sched_adjacency: capacity below n_total");
  if (parent_job && n) std::memcpy(parent_job, s->impl.parent_j().data(), sizeof(int32_t) * n);
  if (child_job && n) {
    // the library's arrays are packed at pitch n_total; the caller's at pitch `capacity`
    for (int c = 0; c < s->impl.n_slots(); ++c)
      std::memcpy(child_job + static_cast<size_t>(c) * capacity, s->impl.child_j().data() + static_cast<size_t>(c) * n, sizeof(int32_t) * n);
  }
  return CAVS_OK;
}
extern "C" int cavs_sched_serial_rounds(const cavs_sched* s, int backward, int32_t* jobs, int32_t* init, int capacity, int* n) {
  SCHED_READY("sched_serial_rounds");
  CAVS_REQUIRE(n, CAVS_ERR_BAD_ARG, "sched_serial_rounds: null n");
  std::vector<cavs_b200::LevelSchedule::SerialRound> rounds;
  s->impl.SerialSweep(backward != 0, &rounds);
  *n = static_cast<int>(rounds.size());
  CAVS_REQUIRE(capacity >= *n && (jobs || *n == 0), CAVS_ERR_CAPACITY, "sched_serial_rounds: capacity");
  for (int r = 0; r < *n; ++r) {
    jobs[r] = rounds[r].job;
    if (init) init[r] = rounds[r].init;
  }
  return CAVS_OK;
}
extern "C" int cavs_sched_ref_serial_stream(const cavs_sched* s, int32_t* out, int capacity, int* n) {
  SCHED_READY("sched_ref_serial_stream");
  CAVS_REQUIRE(n, CAVS_ERR_BAD_ARG, "sched_ref_serial_stream: null n");
  std::vector<int32_t> v;
  s->impl.RefSerialStream(&v);
  *n = static_cast<int>(v.size());
  CAVS_REQUIRE(out && capacity >= *n, CAVS_ERR_CAPACITY, "sched_ref_serial_stream: capacity");
  std::memcpy(out, v.data(), v.size() * sizeof(int32_t));
  return CAVS_OK;
}
