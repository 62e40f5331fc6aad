// Device status words: kernels record soft failures (a wait that ran out, a bounds check
// that tripped) here instead of trapping, and the host turns them into exceptions.
#pragma once
#include <cstdint>

namespace nt {

enum StatusCode : uint32_t {
  kStatusOk = 0,
  kStatusWaitTimeout = 1,   // a bounded spin on an mbarrier / flag gave up
  kStatusBounds = 2,        // a checked index was out of range (access skipped)
  kStatusBadArgument = 3,
};

// One record per device, in managed-free plain device memory: [0]=code, [1]=kernel id,
// [2]=detail (barrier id / peer / index), [3]=count of events.
struct StatusWord {
  uint32_t code, kernel, detail, count;
};

enum KernelId : uint32_t {
  kKernelGemm = 1,
  kKernelAttnFwd = 2,
  kKernelAttnBwd = 3,
  kKernelAllReduce = 4,
  kKernelEpDispatch = 5,
  kKernelEpCombine = 6,
  kKernelProbe = 7,
  kKernelPack = 8,
  kKernelCombine = 9,
};

#ifdef __CUDACC__
__device__ __forceinline__ void report_status(StatusWord* sw, uint32_t code, uint32_t kernel, uint32_t detail) {
  if (sw == nullptr) return;
  if (atomicAdd(&sw->count, 1u) == 0u) {
    sw->kernel = kernel;
    sw->detail = detail;
    __threadfence();
    sw->code = code;
  }
}
#endif

}  // namespace nt
