// Cross-GPU flag barrier used inside kernels that exchange data over NVLink peer memory (the reference has no
// device-side synchronisation between GPUs: every exchange is an NCCL call, src/model/moe_ops.py:139-145).
// Every rank owns a pad of 32-bit words that all peers can write; "arriving" means storing the
// current epoch (release, system scope) into one's own word of every peer's pad, "waiting" means
// polling one's own pad (acquire, system scope) until every peer's word has reached the epoch.
// Epochs only grow, so pads are never reset.  Waits are bounded: on time-out the status word is
// written and the caller gets `false`.
//
// The epoch of a launch is not a kernel argument: it is read from a counter word in this rank's
// own memory (`epoch_counter`, last value used) and the kernel's last block writes the new value
// back before it exits.  Every rank launches the same kernels in the same order, so the counters
// agree, and a launch has the same arguments every time - it can be replayed from a CUDA graph.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "status.h"

namespace nt {

constexpr int XR_MAX_RANKS = 16;

struct XRank {
  uint32_t* flag_local;
  uint32_t* flag_peer[XR_MAX_RANKS];
  int rank, N;
  uint32_t* epoch_counter;  // local word: epoch of the previous launch on this pad
  int word_base;            // first word of this barrier's two phases: [phase][XR_MAX_RANKS]
  long long wait_cycles;
  StatusWord* status;
};

__device__ __forceinline__ void xr_store_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t xr_load_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Every block calls this first (any thread; the value is the same for all blocks of the launch,
// because the counter is only advanced by xr_end, which runs after every block has started).
__device__ __forceinline__ uint32_t xr_begin(const XRank& x) {
  return *reinterpret_cast<volatile uint32_t*>(x.epoch_counter) + 1u;
}
// The launch's last block, once nothing of the launch needs the old value any more.
__device__ __forceinline__ void xr_end(const XRank& x, uint32_t epoch) { *reinterpret_cast<volatile uint32_t*>(x.epoch_counter) = epoch; }

// Threads [0, N) of the calling block take part (others return true at once).
__device__ __forceinline__ bool xr_barrier(const XRank& x, uint32_t epoch, int phase, bool signal, uint32_t kernel_id) {
  const int t = threadIdx.x;
  if (t >= x.N) return true;
  const int word = x.word_base + phase * XR_MAX_RANKS;
  if (signal) xr_store_release(x.flag_peer[t] + word + x.rank, epoch);
  const uint32_t* mine = x.flag_local + word + t;
  const long long start = clock64();
  while (static_cast<int32_t>(xr_load_acquire(mine) - epoch) < 0) {
    if (clock64() - start > x.wait_cycles) {
      report_status(x.status, kStatusWaitTimeout, kernel_id, 1000u * static_cast<uint32_t>(phase) + static_cast<uint32_t>(t));
      return false;
    }
    __nanosleep(64);
  }
  return true;
}

}  // namespace nt
