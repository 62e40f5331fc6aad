// Gradient-bucket all-reduce fused with the 1/N scale and the AdamW update, over NVLink.
//
// One launch per bucket, on a side stream, as soon as the bucket's last gradient is written:
//   1. entry barrier: every rank raises a flag in every peer's flag pad (release, system scope)
//      and waits (bounded) until all peers have raised theirs - the peers' gradients are then
//      complete and visible;
//   2. rank r owns slice r of the bucket.  It sums that slice over all replicas - one
//      `multimem.ld_reduce` per 16 bytes when the buffers are bound to an NVLS multicast object
//      (the switch adds with fp32 accumulation), else plain loads from every peer's buffer - and
//      scales by 1/N;
//   3. with an optimizer bound it applies AdamW to its slice of the fp32 master weights and
//      moments (the state tensors hold that slice only: optimizer state is sharded over the
//      ranks) and broadcasts the new bf16 parameters to every replica (`multimem.st` or peer
//      stores); without one it broadcasts the mean gradient back into every replica's bucket;
//   4. exit barrier (last block of the grid): nobody leaves before all peers' stores into its
//      memory are done.
// The reference does this as copy-in, NCCL all-reduce, divide, copy-back and a separate
// optimizer pass (src/parallel/reducer.py:103-145, src/optim.py).  Per-GPU NVLink traffic here
// is one bucket out and one bucket in; HBM sees the gradient once and the optimizer state of a
// 1/N slice.
// No TMA and no multicast *loads through TMA* are involved: `multimem.*` are plain
// load/store/reduce instructions on a multicast address.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <ATen/ATen.h>

#include "cuda_check.h"
#include "ops.h"
#include "status.h"

namespace nt {

namespace {

constexpr int AR_THREADS = 512;
constexpr int AR_MAX_RANKS = 16;
constexpr int AR_UNROLL = 4;

struct ArArgs {
  // gradients
  uint16_t* grad_local;
  uint16_t* grad_mc;  // multicast address or null
  uint16_t* grad_peer[AR_MAX_RANKS];
  // parameters (optimizer mode)
  uint16_t* param_mc;
  uint16_t* param_peer[AR_MAX_RANKS];
  float *master, *m, *v;  // state of this rank's slice: element i of the bucket is at [i - state_lo]
  long long state_lo;
  // flags: [slot][phase (2)][AR_MAX_RANKS] uint32 in every rank's pad
  uint32_t* flag_local;
  uint32_t* flag_peer[AR_MAX_RANKS];
  uint32_t* block_counter;  // local, one word per slot
  int rank, N, slot;
  uint32_t* epoch_counter;  // local, one word per slot: epoch of the slot's previous launch
  const float* bc_dev;      // optional {1 - beta1^t, 1 / sqrt(1 - beta2^t)} in device memory (CUDA-graph replays)
  long long n;  // elements, multiple of 8
  int fuse_adam, dtype;
  float lr, beta1, beta2, eps, wd, bc1, rsqrt_bc2;
  long long wait_cycles;
  StatusWord* status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// 8 bf16 summed over all replicas by the switch, fp32 accumulation.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16(const void* mc) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
  return r;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_f16(const void* mc) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
  return r;
}
__device__ __forceinline__ void multimem_st(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

__device__ __forceinline__ void unpack8(uint4 q, int dtype, float (&f)[8]) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (dtype == 1) {
      float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    } else {
      float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8], int dtype) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (dtype == 1) {
      __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&t);
    } else {
      __half2 t = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&t);
    }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// All ranks meet: raise my flag in every pad, wait for every flag in mine.  `phase` 0 = entry, 1 = exit.
// Called by threads [0, N) of one block (`signal` = this block raises the flags).  Returns false on time-out.
__device__ __forceinline__ bool cross_rank_barrier(const ArArgs& a, uint32_t epoch, int phase, bool signal) {
  const int t = threadIdx.x;
  bool ok = true;
  if (t < a.N) {
    const int word = (a.slot * 2 + phase) * AR_MAX_RANKS;
    if (signal) st_release_sys(a.flag_peer[t] + word + a.rank, epoch);
    const uint32_t* mine = a.flag_local + word + t;
    const long long start = clock64();
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if (clock64() - start > a.wait_cycles) {
        report_status(a.status, kStatusWaitTimeout, kKernelAllReduce, 1000u * static_cast<uint32_t>(phase) + static_cast<uint32_t>(t));
        ok = false;
        break;
      }
      __nanosleep(64);
    }
  }
  return ok;
}

__global__ void __launch_bounds__(AR_THREADS)
bucket_allreduce_kernel(const ArArgs a) {
  __shared__ int s_ok;
  __shared__ unsigned s_last;
  __shared__ float s_bc[2];
  // The epoch is the slot's launch count: read here by every block, advanced by the last block to
  // finish (after every block has read it), so the launch arguments are the same every step.
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.epoch_counter + a.slot) + 1u;
  if (threadIdx.x == 0) {
    s_ok = 1;
    if (a.bc_dev != nullptr) {  // bias corrections that change per step without changing the launch
      s_bc[0] = a.bc_dev[0];
      s_bc[1] = a.bc_dev[1];
    } else {
      s_bc[0] = a.bc1;
      s_bc[1] = a.rsqrt_bc2;
    }
  }
  __syncthreads();
  const float bc1 = s_bc[0], rsqrt_bc2 = s_bc[1];
  // ---- 1. entry barrier (every block waits; block 0 raises the flags)
  if (blockIdx.x == 0 && threadIdx.x == 0) __threadfence_system();
  if (!cross_rank_barrier(a, epoch, 0, blockIdx.x == 0)) s_ok = 0;
  __syncthreads();
  const bool ok = s_ok != 0;

  // ---- 2./3. my slice
  if (ok) {
    const long long per = ((a.n / 8 + a.N - 1) / a.N) * 8;
    const long long lo = min(a.n, per * a.rank), hi = min(a.n, lo + per);
    const float inv_n = 1.f / static_cast<float>(a.N);
    // Each thread keeps AR_UNROLL 16-byte reductions in flight: one `multimem.ld_reduce` (or one load per
    // peer) has a round-trip latency of microseconds through the switch, and a single outstanding request
    // per thread would cap the kernel far below the links.
    const long long stride = static_cast<long long>(gridDim.x) * AR_THREADS * 8;
    for (long long i0 = lo + (static_cast<long long>(blockIdx.x) * AR_THREADS + threadIdx.x) * 8; i0 < hi; i0 += stride * AR_UNROLL) {
      uint4 q[AR_UNROLL];
      float g[AR_UNROLL][8];
      if (a.grad_mc != nullptr) {
#pragma unroll
        for (int u = 0; u < AR_UNROLL; ++u) {
          const long long i = i0 + u * stride;
          if (i < hi) q[u] = a.dtype == 1 ? multimem_ld_reduce_bf16(a.grad_mc + i) : multimem_ld_reduce_f16(a.grad_mc + i);
        }
#pragma unroll
        for (int u = 0; u < AR_UNROLL; ++u) unpack8(q[u], a.dtype, g[u]);
      } else {
#pragma unroll
        for (int u = 0; u < AR_UNROLL; ++u)
#pragma unroll
          for (int j = 0; j < 8; ++j) g[u][j] = 0.f;
        for (int p = 0; p < a.N; ++p) {  // fixed order: identical sums whichever rank owns the slice
#pragma unroll
          for (int u = 0; u < AR_UNROLL; ++u) {
            const long long i = i0 + u * stride;
            q[u] = i < hi ? *reinterpret_cast<const uint4*>(a.grad_peer[p] + i) : make_uint4(0u, 0u, 0u, 0u);
          }
#pragma unroll
          for (int u = 0; u < AR_UNROLL; ++u) {
            float f[8];
            unpack8(q[u], a.dtype, f);
#pragma unroll
            for (int j = 0; j < 8; ++j) g[u][j] += f[j];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < AR_UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i >= hi) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) g[u][j] *= inv_n;
        uint4 out;
        if (a.fuse_adam) {
          // the slice's fp32 state, 32 bytes at a time (slices start on multiples of 8 elements)
          const long long s = i - a.state_lo;
          float4 pw[2], mm[2], vv[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            pw[h] = *reinterpret_cast<const float4*>(a.master + s + 4 * h);
            mm[h] = *reinterpret_cast<const float4*>(a.m + s + 4 * h);
            vv[h] = *reinterpret_cast<const float4*>(a.v + s + 4 * h);
          }
          float* pwf = reinterpret_cast<float*>(pw);
          float* mmf = reinterpret_cast<float*>(mm);
          float* vvf = reinterpret_cast<float*>(vv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            pwf[j] *= 1.f - a.lr * a.wd;
            mmf[j] = a.beta1 * mmf[j] + (1.f - a.beta1) * g[u][j];
            vvf[j] = a.beta2 * vvf[j] + (1.f - a.beta2) * g[u][j] * g[u][j];
            pwf[j] -= (a.lr / bc1) * mmf[j] / (sqrtf(vvf[j]) * rsqrt_bc2 + a.eps);
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            *reinterpret_cast<float4*>(a.master + s + 4 * h) = pw[h];
            *reinterpret_cast<float4*>(a.m + s + 4 * h) = mm[h];
            *reinterpret_cast<float4*>(a.v + s + 4 * h) = vv[h];
          }
          float w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) w[j] = pwf[j];
          out = pack8(w, a.dtype);
          if (a.param_mc != nullptr) multimem_st(a.param_mc + i, out);
          else for (int p = 0; p < a.N; ++p) *reinterpret_cast<uint4*>(a.param_peer[p] + i) = out;
        } else {
          out = pack8(g[u], a.dtype);
          if (a.grad_mc != nullptr) multimem_st(a.grad_mc + i, out);
          else for (int p = 0; p < a.N; ++p) *reinterpret_cast<uint4*>(a.grad_peer[p] + i) = out;
        }
      }
    }
  }
  // ---- 4. exit barrier by the last block to finish
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned ticket = atomicAdd(a.block_counter + a.slot, 1u);
    s_last = (ticket == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) a.block_counter[a.slot] = 0u;
    if (ok) cross_rank_barrier(a, epoch, 1, true);
    __syncthreads();
    if (threadIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(a.epoch_counter + a.slot) = epoch;
  }
}

}  // namespace

// ptr tables are int64 CPU tensors of length N (device addresses); mc pointers are 0 when NVLS is unavailable.
void bucket_allreduce(at::Tensor grad_local, int64_t grad_mc, const at::Tensor& grad_peers, int64_t param_mc,
                      const at::Tensor& param_peers, const c10::optional<at::Tensor>& master, const c10::optional<at::Tensor>& m,
                      const c10::optional<at::Tensor>& v, at::Tensor flag_local, const at::Tensor& flag_peers, at::Tensor block_counter,
                      int64_t rank, int64_t world, int64_t slot, at::Tensor epoch_counters, int64_t step,
                      const c10::optional<at::Tensor>& bc_dev, double lr, double beta1, double beta2,
                      double eps, double wd, int64_t blocks, double wait_ms) {
  TORCH_CHECK(grad_local.is_cuda() && grad_local.is_contiguous(), "bucket_allreduce: contiguous CUDA bucket");
  TORCH_CHECK(grad_local.scalar_type() == at::kBFloat16 || grad_local.scalar_type() == at::kHalf, "bucket_allreduce: bf16 / fp16 buckets");
  TORCH_CHECK(world >= 1 && world <= AR_MAX_RANKS, "bucket_allreduce: 1..", AR_MAX_RANKS, " ranks");
  TORCH_CHECK(grad_local.numel() % 8 == 0 && reinterpret_cast<uintptr_t>(grad_local.data_ptr()) % 16 == 0, "bucket_allreduce: 16-byte aligned, length % 8 == 0");
  TORCH_CHECK(grad_peers.numel() == world && flag_peers.numel() == world && grad_peers.scalar_type() == at::kLong, "bucket_allreduce: peer tables");
  c10::cuda::CUDAGuard guard(grad_local.device());
  ArArgs a{};
  a.grad_local = reinterpret_cast<uint16_t*>(grad_local.data_ptr());
  a.grad_mc = reinterpret_cast<uint16_t*>(grad_mc);
  a.param_mc = reinterpret_cast<uint16_t*>(param_mc);
  const auto* gp = grad_peers.data_ptr<int64_t>();
  const auto* fp = flag_peers.data_ptr<int64_t>();
  for (int i = 0; i < world; ++i) {
    a.grad_peer[i] = reinterpret_cast<uint16_t*>(gp[i]);
    a.flag_peer[i] = reinterpret_cast<uint32_t*>(fp[i]);
  }
  a.fuse_adam = master.has_value();
  if (a.fuse_adam) {
    TORCH_CHECK(m.has_value() && v.has_value() && param_peers.numel() == world, "bucket_allreduce: optimizer mode needs master, m, v and parameter peers");
    const long long n_all = grad_local.numel();
    const long long per = ((n_all / 8 + world - 1) / world) * 8;
    const long long lo = std::min(n_all, per * rank), hi = std::min(n_all, lo + per);
    // state tensors cover the whole bucket or exactly this rank's slice [lo, hi)
    const bool whole = master->numel() == n_all;
    TORCH_CHECK((whole || master->numel() == hi - lo) && m->numel() == master->numel() && v->numel() == master->numel(),
                "bucket_allreduce: optimizer state must have the bucket's length or the owned slice's (", hi - lo, ")");
    a.state_lo = whole ? 0 : lo;
    TORCH_CHECK(reinterpret_cast<uintptr_t>(master->data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(m->data_ptr()) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(v->data_ptr()) % 16 == 0, "bucket_allreduce: optimizer state must be 16-byte aligned");
    const auto* pp = param_peers.data_ptr<int64_t>();
    for (int i = 0; i < world; ++i) a.param_peer[i] = reinterpret_cast<uint16_t*>(pp[i]);
    a.master = master->data_ptr<float>();
    a.m = m->data_ptr<float>();
    a.v = v->data_ptr<float>();
  }
  a.flag_local = reinterpret_cast<uint32_t*>(flag_local.data_ptr());
  a.block_counter = reinterpret_cast<uint32_t*>(block_counter.data_ptr());
  a.rank = static_cast<int>(rank);
  a.N = static_cast<int>(world);
  a.slot = static_cast<int>(slot);
  TORCH_CHECK(epoch_counters.is_cuda() && epoch_counters.scalar_type() == at::kInt && slot < epoch_counters.numel(), "bucket_allreduce: epoch counters");
  a.epoch_counter = reinterpret_cast<uint32_t*>(epoch_counters.data_ptr());
  if (bc_dev.has_value()) {
    TORCH_CHECK(bc_dev->is_cuda() && bc_dev->scalar_type() == at::kFloat && bc_dev->numel() == 2, "bucket_allreduce: bc_dev is two fp32 on the device");
    a.bc_dev = bc_dev->data_ptr<float>();
  }
  a.n = grad_local.numel();
  a.dtype = grad_local.scalar_type() == at::kBFloat16 ? 1 : 0;
  a.lr = static_cast<float>(lr); a.beta1 = static_cast<float>(beta1); a.beta2 = static_cast<float>(beta2);
  a.eps = static_cast<float>(eps); a.wd = static_cast<float>(wd);
  a.bc1 = 1.f - static_cast<float>(std::pow(beta1, static_cast<double>(std::max<int64_t>(step, 1))));
  a.rsqrt_bc2 = 1.f / std::sqrt(1.f - static_cast<float>(std::pow(beta2, static_cast<double>(std::max<int64_t>(step, 1)))));
  a.wait_cycles = static_cast<long long>(wait_ms * 1.9e6);
  a.status = device_status_word();
  const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(blocks, 148)));
  bucket_allreduce_kernel<<<grid, AR_THREADS, 0, at::cuda::getCurrentCUDAStream()>>>(a);
  NT_KERNEL_CHECK();
}

}  // namespace nt
