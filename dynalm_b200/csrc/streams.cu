// Two kernels of one step that do not depend on each other, side by side: the second stream waits for what the
// first has been given so far (fork), runs its kernel, and the first stream waits for that (join). In a step that
// holds decode rows and prompt portions, the split-KV attention of the decode rows and the flash attention of the
// prompt rows each fill a part of the GPU only.
//
// One pair of events per process: cudaStreamWaitEvent takes the event's latest record at the time of the call, so
// an event may be recorded again as soon as the wait has been issued.
//
// The reference runs its attention rows in one call (dynacore/cpu/cpu_device.cpp:1717-1776).
#include "common.cuh"

namespace dl {

static cudaEvent_t stream_event(int which) {
  static cudaEvent_t events[2] = {nullptr, nullptr};
  if (events[which] == nullptr && cudaEventCreateWithFlags(&events[which], cudaEventDisableTiming) != cudaSuccess)
    events[which] = nullptr;
  return events[which];
}

static int order_after(cudaStream_t first, cudaStream_t then, int which) {
  cudaEvent_t e = stream_event(which);
  if (e == nullptr) return DL_ERR_UNSUPPORTED;
  cudaError_t rc = cudaEventRecord(e, first);
  if (rc != cudaSuccess) return static_cast<int>(rc);
  rc = cudaStreamWaitEvent(then, e, 0);
  return static_cast<int>(rc);
}

}  // namespace dl

// What `side` is given from now on runs after everything `main` has been given so far.
DL_EXPORT int dl_stream_fork(cudaStream_t main, cudaStream_t side) { return dl::order_after(main, side, 0); }

// What `main` is given from now on runs after everything `side` has been given so far.
DL_EXPORT int dl_stream_join(cudaStream_t main, cudaStream_t side) { return dl::order_after(side, main, 1); }
