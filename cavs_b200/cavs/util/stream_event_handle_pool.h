// Stream lookup by small integer id, same entry point the reference's operators call
// (cavs/util/stream_event_handle_pool.h): id -1 means the default stream.
#ifndef CAVS_UTIL_STREAM_EVENT_HANDLE_POOL_H_
#define CAVS_UTIL_STREAM_EVENT_HANDLE_POOL_H_
#include <cuda_runtime.h>
class StreamEventHandlePool {
 public:
  static cudaStream_t GetCudaStream(int id);
};
#endif
