// TEST INFRASTRUCTURE (oracle).  Drives the reference's own BatchGraphScheduler
// (cavs/midend/graph_scheduler.{h,cc}, compiled unmodified from the reference
// checkout against the stand-in headers in refsched_shim/) through one forward
// and one backward sweep, exactly as GraphStatement::Run / GraphGradStatement::Run
// do (cavs/midend/statement.cc:43-123), and serialises every table the graph ops
// read into one int32 stream.  Only tests and the oracle build may link this.
//
// Stream layout ("schedule stream"), all int32:
//   N  L
//   level_off[0..L]                      forward GetCurrentRoundOffset() per round, then the scheduled total
//   per forward round r = 0..L-1:
//     n jobs[n]                          GetJobId()
//     n ids[n]   (x2, child slot 0, 1)   CurrentRoundTensorIdsForGather(slot)
//     n ids[n]                           CurrentRoundTensorIdsForScatter(0)
//     n ids[n]                           CurrentRoundTensorIdsForGatherInitialization()
//   t2j[N]                               TensorIdsToJobIds() after the forward sweep
//   per backward round (L of them, last forward level first):
//     off n jobs[n]
//     n ids[n]                           CurrentRoundTensorIdsForGather(0)
//     n ids[n]   (x2, child slot 0, 1)   CurrentRoundTensorIdsForScatter(slot)
//     n ids[n]                           CurrentRoundTensorIdsForGatherInitialization()
#include "cavs/midend/graph_scheduler.h"

#include <vector>

namespace {
void put(std::vector<int>* s, const std::vector<int>& v) {
  s->push_back(static_cast<int>(v.size()));
  s->insert(s->end(), v.begin(), v.end());
}
}  // namespace

extern "C" int refsched_stream(const int* parents, int batch, int max_len, int* out, int capacity) {
  midend::Tensor graph(parents, batch, max_len);
  midend::BatchGraphScheduler gs;
  const int total = gs.LoadGraph(graph);

  std::vector<int> offsets, body;
  int levels = 0, scheduled = 0;
  gs.Initialize();
  while (!gs.Terminate()) {
    offsets.push_back(gs.GetCurrentRoundOffset());
    scheduled = gs.GetCurrentRoundOffset() + static_cast<int>(gs.GetJobId().size());
    put(&body, gs.GetJobId());
    put(&body, gs.CurrentRoundTensorIdsForGather(0));
    put(&body, gs.CurrentRoundTensorIdsForGather(1));
    put(&body, gs.CurrentRoundTensorIdsForScatter(0));
    put(&body, gs.CurrentRoundTensorIdsForGatherInitialization());
    gs.ActivateNext();
    ++levels;
  }
  offsets.push_back(scheduled);
  const std::vector<int>& t2j = gs.TensorIdsToJobIds();
  body.insert(body.end(), t2j.begin(), t2j.end());

  if (levels > 0) {
    gs.ReverseGraph();
    gs.Initialize();
    while (!gs.Terminate()) {
      body.push_back(gs.GetCurrentRoundOffset());
      put(&body, gs.GetJobId());
      put(&body, gs.CurrentRoundTensorIdsForGather(0));
      put(&body, gs.CurrentRoundTensorIdsForScatter(0));
      put(&body, gs.CurrentRoundTensorIdsForScatter(1));
      put(&body, gs.CurrentRoundTensorIdsForGatherInitialization());
      gs.ActivateNext();
    }
  }

  const int need = 2 + static_cast<int>(offsets.size() + body.size());
  if (need > capacity) return -need;
  int* w = out;
  *w++ = total;
  *w++ = levels;
  for (int v : offsets) *w++ = v;
  for (int v : body) *w++ = v;
  return need;
}

// The same for the reference's SerialGraphScheduler (one vertex per round, tensor id == job id).
// Stream layout ("serial schedule stream"), all int32:
//   N
//   RF, then per forward round:  job  gather(0)  gather(1)  scatter(0)  gather-initialisation
//   t2j[N]
//   RB, then per backward round: job  gather(0)  scatter(0)  scatter(1)  gather-initialisation
// A first sample of one vertex would make the reference read the front of an empty list
// (graph_scheduler.cc:89); the driver reports zero rounds for it instead of calling in.
extern "C" int refsched_serial_stream(const int* parents, int batch, int max_len, int* out, int capacity) {
  midend::Tensor graph(parents, batch, max_len);
  midend::SerialGraphScheduler gs;
  const int total = gs.LoadGraph(graph);
  std::vector<int> fwd, bwd;
  int rf = 0, rb = 0;
  const bool runnable = batch > 0 && parents[0] != -1;
  if (runnable) {
    gs.Initialize();
    while (!gs.Terminate()) {
      fwd.push_back(gs.GetCurrentRoundOffset());
      put(&fwd, gs.CurrentRoundTensorIdsForGather(0));
      put(&fwd, gs.CurrentRoundTensorIdsForGather(1));
      put(&fwd, gs.CurrentRoundTensorIdsForScatter(0));
      put(&fwd, gs.CurrentRoundTensorIdsForGatherInitialization());
      gs.ActivateNext();
      ++rf;
    }
  }
  std::vector<int> t2j = gs.TensorIdsToJobIds();
  if (rf > 0) {
    gs.ReverseGraph();
    gs.Initialize();
    while (!gs.Terminate()) {
      bwd.push_back(gs.GetCurrentRoundOffset());
      put(&bwd, gs.CurrentRoundTensorIdsForGather(0));
      put(&bwd, gs.CurrentRoundTensorIdsForScatter(0));
      put(&bwd, gs.CurrentRoundTensorIdsForScatter(1));
      put(&bwd, gs.CurrentRoundTensorIdsForGatherInitialization());
      gs.ActivateNext();
      ++rb;
    }
  }
  const int need = 3 + static_cast<int>(fwd.size() + t2j.size() + bwd.size());
  if (need > capacity) return -need;
  int* w = out;
  *w++ = total;
  *w++ = rf;
  for (int v : fwd) *w++ = v;
  for (int v : t2j) *w++ = v;
  *w++ = rb;
  for (int v : bwd) *w++ = v;
  return need;
}
