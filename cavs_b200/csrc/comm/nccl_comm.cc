// Cross-GPU reduction of gradients for data-parallel training: one process per GPU, NCCL over NVLink.
//
// Replaces the reference's per-variable MPIAllReduce through host memory (cavs/backend/op_impl_mpi.cc:29-49,
// inserted by MPISession, cavs/midend/session_mpi.cc:31-80) and the start-up broadcast of the variables from
// rank 0 (cavs/backend/op_impl_variable.h:151-159).  The collectives run on device buffers, in place, on the
// caller's stream.  NCCL is bound at run time (dlopen of libnccl.so.2 on first use) so that the library loads on
// hosts that never train data-parallel; inside a process that already holds an NCCL (a PyTorch host) that same
// copy is used.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstring>
#include <mutex>
#include <string>

#include "abi_common.h"

namespace {

// The slice of NCCL's C interface used here (nccl.h: stable across the 2.x series).
struct NcclUniqueId { char internal[128]; };
using NcclComm = void*;
constexpr int kNcclSuccess = 0;
constexpr int kNcclInt8 = 0, kNcclInt32 = 2, kNcclFloat32 = 7;
constexpr int kNcclSum = 0;

struct NcclApi {
  int (*GetUniqueId)(NcclUniqueId*) = nullptr;
  int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
  int (*Broadcast)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  int (*GetVersion)(int*) = nullptr;
  bool ok = false;
  std::string why;
};

NcclApi& Api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    if (!h) { api.why = std::string("libnccl.so.2 could not be loaded: ") + dlerror(); return; }
    auto sym = [&](const char* name) {
      void* p = dlsym(h, name);
      if (!p && api.why.empty()) api.why = std::string("libnccl lacks ") + name;
      return p;
    };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.Broadcast = reinterpret_cast<decltype(api.Broadcast)>(sym("ncclBroadcast"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    api.GetVersion = reinterpret_cast<decltype(api.GetVersion)>(sym("ncclGetVersion"));
    api.ok = api.why.empty();
  });
  return api;
}

int NcclFail(const char* what, int rc) {
  NcclApi& api = Api();
  return cavs_b200::Fail(CAVS_ERR_CUDA, std::string(what) + ": " + (api.GetErrorString ? api.GetErrorString(rc) : "NCCL error") + " (" +
                                            std::to_string(rc) + ")");
}

}  // namespace

struct cavs_comm {
  NcclComm comm = nullptr;
  int rank = 0, world = 1, device = 0;
};

#define CAVS_NCCL_READY()                                                                    \
  do {                                                                                       \
    if (!Api().ok) return cavs_b200::Fail(CAVS_ERR_UNSUPPORTED, "nccl: " + Api().why);       \
  } while (0)

extern "C" int cavs_comm_unique_id(void* id, size_t bytes) {
  CAVS_REQUIRE(id && bytes >= sizeof(NcclUniqueId), CAVS_ERR_BAD_ARG, "comm_unique_id: the id buffer must hold 128 bytes");
  CAVS_NCCL_READY();
  NcclUniqueId u;
  if (int rc = Api().GetUniqueId(&u)) return NcclFail("ncclGetUniqueId", rc);
  std::memcpy(id, &u, sizeof(u));
  return CAVS_OK;
}

extern "C" int cavs_comm_create(const void* id, size_t bytes, int rank, int world, cavs_comm** out) {
  CAVS_REQUIRE(id && out && bytes >= sizeof(NcclUniqueId), CAVS_ERR_BAD_ARG, "comm_create: null pointer or short id");
  CAVS_REQUIRE(world >= 1 && rank >= 0 && rank < world, CAVS_ERR_BAD_ARG, "comm_create: rank must lie in [0, world)");
  CAVS_NCCL_READY();
  auto* c = new cavs_comm();
  c->rank = rank; c->world = world;
  if (cudaGetDevice(&c->device) != cudaSuccess) { delete c; return cavs_b200::Fail(CAVS_ERR_CUDA, "comm_create: no current CUDA device"); }
  NcclUniqueId u;
  std::memcpy(&u, id, sizeof(u));
  if (int rc = Api().CommInitRank(&c->comm, world, u, rank)) { delete c; return NcclFail("ncclCommInitRank", rc); }
  *out = c;
  return CAVS_OK;
}

extern "C" void cavs_comm_destroy(cavs_comm* c) {
  if (!c) return;
  if (c->comm && Api().ok) Api().CommDestroy(c->comm);
  delete c;
}

extern "C" int cavs_comm_info(const cavs_comm* c, int* rank, int* world, int* nccl_version) {
  CAVS_REQUIRE(c, CAVS_ERR_BAD_ARG, "comm_info: null handle");
  if (rank) *rank = c->rank;
  if (world) *world = c->world;
  if (nccl_version) { *nccl_version = 0; if (Api().ok) Api().GetVersion(nccl_version); }
  return CAVS_OK;
}

extern "C" int cavs_allreduce(float* buf, size_t count, cavs_comm* c, void* stream) {
  CAVS_REQUIRE(c && (buf || count == 0), CAVS_ERR_BAD_ARG, "allreduce: null pointer");
  if (count == 0 || c->world == 1) return CAVS_OK;
  if (int rc = Api().AllReduce(buf, buf, count, kNcclFloat32, kNcclSum, c->comm, static_cast<cudaStream_t>(stream)))
    return NcclFail("ncclAllReduce", rc);
  return CAVS_OK;
}

extern "C" int cavs_broadcast(void* buf, size_t bytes, int root, cavs_comm* c, void* stream) {
  CAVS_REQUIRE(c && (buf || bytes == 0) && root >= 0 && root < c->world, CAVS_ERR_BAD_ARG, "broadcast: bad argument");
  if (bytes == 0 || c->world == 1) return CAVS_OK;
  if (int rc = Api().Broadcast(buf, buf, bytes, kNcclInt8, root, c->comm, static_cast<cudaStream_t>(stream)))
    return NcclFail("ncclBroadcast", rc);
  return CAVS_OK;
}

extern "C" int cavs_allgather(const void* send, void* recv, size_t bytes_per_rank, cavs_comm* c, void* stream) {
  CAVS_REQUIRE(c && ((send && recv) || bytes_per_rank == 0), CAVS_ERR_BAD_ARG, "allgather: null pointer");
  if (bytes_per_rank == 0) return CAVS_OK;
  if (c->world == 1) {
    if (send != recv &&
        cudaMemcpyAsync(recv, send, bytes_per_rank, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)) != cudaSuccess)
      return cavs_b200::Fail(CAVS_ERR_CUDA, "allgather: device copy failed");
    return CAVS_OK;
  }
  if (int rc = Api().AllGather(send, recv, bytes_per_rank, kNcclInt8, c->comm, static_cast<cudaStream_t>(stream)))
    return NcclFail("ncclAllGather", rc);
  return CAVS_OK;
}
