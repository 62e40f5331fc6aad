// Self-test of the soft-failure path: a kernel waits on an mbarrier that nothing will ever
// complete, with a short cycle limit; the wait gives up, records a status word and the kernel
// returns normally, so the context stays usable.  This is how the bounded waits of the tcgen05
// and NVLink kernels are exercised without faulting, trapping or hanging the GPU.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <ATen/ATen.h>

#include "cuda_check.h"
#include "ops.h"
#include "sm100.cuh"

namespace nt {

namespace {

__global__ void bounded_wait_probe_kernel(StatusWord* status, long long limit_cycles, int* gave_up) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    sm100::mbar_init(&bar, 1);
    abort_flag = 0u;
    sm100::fence_barrier_init();
  }
  __syncthreads();
  // same loop as sm100::mbar_wait, with the limit as a parameter
  bool ok = false;
  const long long start = clock64();
  while (true) {
    if (sm100::mbar_try_wait(&bar, 0)) { ok = true; break; }
    if (*reinterpret_cast<volatile uint32_t*>(&abort_flag) != 0u) break;
    if (clock64() - start > limit_cycles) {
      abort_flag = 1u;
      report_status(status, kStatusWaitTimeout, kKernelProbe, threadIdx.x);
      break;
    }
  }
  if (!ok) atomicAdd(gave_up, 1);
}

}  // namespace

// Returns how many threads abandoned the wait (all of them).  The device status word is set.
int64_t bounded_wait_probe(double limit_ms) {
  TORCH_CHECK(limit_ms > 0 && limit_ms <= 1000.0, "bounded_wait_probe: limit in (0, 1000] ms");
  auto counter = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA));
  bounded_wait_probe_kernel<<<1, 64, 0, at::cuda::getCurrentCUDAStream()>>>(device_status_word(), static_cast<long long>(limit_ms * 1.9e6),
                                                                            counter.data_ptr<int>());
  NT_KERNEL_CHECK();
  return counter.item<int>();
}

}  // namespace nt
