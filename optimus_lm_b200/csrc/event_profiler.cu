// Device time stamps for the region profiler: a one-thread kernel writes %globaltimer into a
// (pinned, device-visible) slot at the point of the stream where it was enqueued.  The
// reference's native profiler shim enqueues SYCL profiling tags
// (pytorch_xpu_extensions/pcl.xpu.profiler/csrc/profiler/profile.dp.cpp:8-69).
#include "olb_api.h"
#include "ptx.cuh"

namespace olb {
__global__ void stamp_kernel(unsigned long long* slot) { *slot = globaltimer_ns(); }
}  // namespace olb

extern "C" int olb_stamp_globaltimer(unsigned long long* slot, cudaStream_t stream) {
  olb::stamp_kernel<<<1, 1, 0, stream>>>(slot);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
