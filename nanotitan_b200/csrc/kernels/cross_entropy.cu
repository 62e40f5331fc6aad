// Token cross-entropy over a padded logits matrix, forward and backward in one kernel (the reference calls
// F.cross_entropy on fp32-cast logits and lets autograd build the backward, src/parallel/pp.py:76).
//
// One block per row.  Pass 1 streams the row once with an online (max, sum-exp) pair; pass 2
// (the row is then in L2) overwrites the logits in place with
//   dlogits = (softmax - onehot(target)) * grad_scale
// so no second [T, V] buffer exists.  Per-row losses are written to a vector and summed by the
// caller in a fixed order.  Columns >= V (row padding kept for TMA alignment) are zeroed.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <ATen/ATen.h>

#include "cuda_check.h"
#include "ops.h"
#include "vec.cuh"

namespace nt {

namespace {

constexpr int CE_THREADS = 512;

__device__ __forceinline__ void online_merge(float& m, float& s, float om, float os) {
  const float nm = fmaxf(m, om);
  if (nm == -INFINITY) { m = nm; s = 0.f; return; }
  s = s * __expf(m - nm) + os * __expf(om - nm);
  m = nm;
}

template <typename T, int VEC>
__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_bwd_kernel(T* __restrict__ logits, const long long* __restrict__ targets, float* __restrict__ row_loss,
                  long long ld, int V, float grad_scale, int write_grad) {
  __shared__ float sm[CE_THREADS / 32], ss[CE_THREADS / 32];
  __shared__ float s_max, s_sum;
  const long long row = blockIdx.x;
  T* lr = logits + row * ld;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float m = -INFINITY, s = 0.f;
  const int v_vec = (V / VEC) * VEC;
  for (int c = threadIdx.x * VEC; c < v_vec; c += CE_THREADS * VEC) {
    float v[VEC];
    load_vec<T, VEC>(lr + c, v);
    float cm = v[0];
#pragma unroll
    for (int i = 1; i < VEC; ++i) cm = fmaxf(cm, v[i]);
    float cs = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) cs += __expf(v[i] - cm);
    online_merge(m, s, cm, cs);
  }
  for (int c = v_vec + threadIdx.x; c < V; c += CE_THREADS) online_merge(m, s, elem_to_float<T>(lr[c]), 1.f);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
    online_merge(m, s, om, os);
  }
  if (lane == 0) { sm[warp] = m; ss[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    m = lane < CE_THREADS / 32 ? sm[lane] : -INFINITY;
    s = lane < CE_THREADS / 32 ? ss[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
      online_merge(m, s, om, os);
    }
    if (lane == 0) { s_max = m; s_sum = s; }
  }
  __syncthreads();
  const float row_max = s_max, inv_sum = 1.f / s_sum;
  const long long tgt = targets[row];
  const bool tgt_ok = tgt >= 0 && tgt < V;  // out-of-range targets (e.g. -100) contribute nothing
  if (threadIdx.x == 0) row_loss[row] = tgt_ok ? (logf(s_sum) + row_max - elem_to_float<T>(lr[tgt])) : 0.f;
  if (!write_grad) return;
  __syncthreads();  // the target logit was read above; now the row may be overwritten
  const float scale = tgt_ok ? grad_scale : 0.f;
  for (int c = threadIdx.x * VEC; c < v_vec; c += CE_THREADS * VEC) {
    float v[VEC];
    load_vec<T, VEC>(lr + c, v);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      float p = __expf(v[i] - row_max) * inv_sum;
      if (c + i == tgt) p -= 1.f;
      v[i] = p * scale;
    }
    store_vec<T, VEC>(lr + c, v);
  }
  for (int c = v_vec + threadIdx.x; c < ld; c += CE_THREADS) {
    float p = 0.f;
    if (c < V) {
      p = __expf(elem_to_float<T>(lr[c]) - row_max) * inv_sum;
      if (c == tgt) p -= 1.f;
    }
    lr[c] = float_to_elem<T>(p * scale);
  }
}

}  // namespace

// logits [rows, ld >= V] is overwritten with dlogits when write_grad; returns per-row losses [rows] f32.
at::Tensor cross_entropy_fwd_bwd(at::Tensor logits, const at::Tensor& targets, int64_t V, double grad_scale, bool write_grad) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "cross_entropy: logits [rows, ld] with contiguous rows");
  TORCH_CHECK(targets.scalar_type() == at::kLong && targets.is_contiguous() && targets.numel() == logits.size(0), "cross_entropy: int64 targets, one per row");
  TORCH_CHECK(V <= logits.size(1), "cross_entropy: V exceeds the row length");
  c10::cuda::CUDAGuard guard(logits.device());
  const long long rows = logits.size(0), ld = logits.stride(0);
  auto row_loss = at::empty({rows}, logits.options().dtype(at::kFloat));
  if (rows == 0) return row_loss;
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  NT_DISPATCH_FLOAT(logits.scalar_type(), "cross_entropy", [&] {
    constexpr int VEC = 16 / sizeof(scalar_t);
    const bool vec = ld % VEC == 0 && is_aligned16(logits.data_ptr());
    if (vec)
      ce_fwd_bwd_kernel<scalar_t, VEC><<<static_cast<unsigned>(rows), CE_THREADS, 0, stream>>>(logits.data_ptr<scalar_t>(), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()),
          row_loss.data_ptr<float>(), ld, static_cast<int>(V), static_cast<float>(grad_scale), write_grad);
    else
      ce_fwd_bwd_kernel<scalar_t, 1><<<static_cast<unsigned>(rows), CE_THREADS, 0, stream>>>(logits.data_ptr<scalar_t>(), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()),
          row_loss.data_ptr<float>(), ld, static_cast<int>(V), static_cast<float>(grad_scale), write_grad);
  });
  NT_KERNEL_CHECK();
  return row_loss;
}

}  // namespace nt
