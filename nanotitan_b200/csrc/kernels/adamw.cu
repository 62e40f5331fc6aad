// Fused AdamW over a flat bucket: one pass reads the gradient and the fp32 master/moment
// state, writes the state back and the parameter in its storage dtype.  Same update rule as
// torch.optim.AdamW (decoupled weight decay, bias-corrected moments); `grad_scale` folds the
// 1/N of a data-parallel mean in.  Optionally emits per-block sums of grad^2 for a gradient
// norm, reduced in a fixed order by the caller.
// The reference steps `torch.optim.AdamW(lr, weight_decay=0.1)` per parameter tensor (src/optim.py:6-10) with no
// master weights.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <ATen/ATen.h>

#include "cuda_check.h"
#include "ops.h"
#include "vec.cuh"

namespace nt {

namespace {

constexpr int AD_THREADS = 256;

template <typename T, int VEC>
__global__ void __launch_bounds__(AD_THREADS)
adamw_kernel(T* __restrict__ param, const T* __restrict__ grad, float* __restrict__ master, float* __restrict__ m,
             float* __restrict__ v, long long n, float lr, float beta1, float beta2, float eps, float wd,
             float bc1, float rsqrt_bc2, float grad_scale, float* __restrict__ sq_partial, const float* __restrict__ bc_dev) {
  float local_sq = 0.f;
  if (bc_dev != nullptr) {
    bc1 = bc_dev[0];
    rsqrt_bc2 = bc_dev[1];
  }
  for (long long i = (static_cast<long long>(blockIdx.x) * AD_THREADS + threadIdx.x) * VEC; i < n;
       i += static_cast<long long>(gridDim.x) * AD_THREADS * VEC) {
    float g[VEC];
    load_vec<T, VEC>(grad + i, g);
#pragma unroll
    for (int j = 0; j < VEC; j += 4) {
      float4 pw = *reinterpret_cast<float4*>(master + i + j);
      float4 mm = *reinterpret_cast<float4*>(m + i + j);
      float4 vv = *reinterpret_cast<float4*>(v + i + j);
      float* pp = reinterpret_cast<float*>(&pw);
      float* pm = reinterpret_cast<float*>(&mm);
      float* pv = reinterpret_cast<float*>(&vv);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float gr = g[j + q] * grad_scale;
        local_sq += gr * gr;
        pp[q] *= 1.f - lr * wd;
        pm[q] = beta1 * pm[q] + (1.f - beta1) * gr;
        pv[q] = beta2 * pv[q] + (1.f - beta2) * gr * gr;
        const float denom = sqrtf(pv[q]) * rsqrt_bc2 + eps;
        pp[q] -= (lr / bc1) * pm[q] / denom;
        g[j + q] = pp[q];
      }
      *reinterpret_cast<float4*>(master + i + j) = pw;
      *reinterpret_cast<float4*>(m + i + j) = mm;
      *reinterpret_cast<float4*>(v + i + j) = vv;
    }
    store_vec<T, VEC>(param + i, g);
  }
  if (sq_partial != nullptr) {
    __shared__ float red[AD_THREADS / 32];
    local_sq = warp_sum(local_sq);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local_sq;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.f;
      for (int w = 0; w < AD_THREADS / 32; ++w) s += red[w];
      sq_partial[blockIdx.x] = s;
    }
  }
}

}  // namespace

// All buffers flat, same length (a multiple of 8), 16-byte aligned.  Returns sum(grad^2) partials or an empty tensor.
at::Tensor adamw_step(at::Tensor param, const at::Tensor& grad, at::Tensor master, at::Tensor m, at::Tensor v, int64_t step,
                      double lr, double beta1, double beta2, double eps, double wd, double grad_scale, bool want_sq,
                      const c10::optional<at::Tensor>& bc_dev) {
  TORCH_CHECK(param.is_cuda() && param.is_contiguous() && grad.is_contiguous() && master.is_contiguous() && m.is_contiguous() && v.is_contiguous(), "adamw_step: contiguous CUDA buffers");
  TORCH_CHECK(grad.scalar_type() == param.scalar_type() && master.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat, "adamw_step: dtypes");
  const long long n = param.numel();
  TORCH_CHECK(grad.numel() == n && master.numel() == n && m.numel() == n && v.numel() == n, "adamw_step: length mismatch");
  TORCH_CHECK(n % 8 == 0 && is_aligned16(param.data_ptr()) && is_aligned16(grad.data_ptr()) && is_aligned16(master.data_ptr()) &&
              is_aligned16(m.data_ptr()) && is_aligned16(v.data_ptr()), "adamw_step: buffers must be 16-byte aligned with length % 8 == 0");
  c10::cuda::CUDAGuard guard(param.device());
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>((n / 8 + AD_THREADS - 1) / AD_THREADS, 8LL * sms)));
  auto partial = want_sq ? at::empty({grid}, master.options()) : at::empty({0}, master.options());
  if (n == 0) return partial;
  const float bc1 = 1.f - static_cast<float>(std::pow(beta1, static_cast<double>(step)));
  const float bc2 = 1.f - static_cast<float>(std::pow(beta2, static_cast<double>(step)));
  const float* bcp = nullptr;
  if (bc_dev.has_value()) {
    TORCH_CHECK(bc_dev->is_cuda() && bc_dev->scalar_type() == at::kFloat && bc_dev->numel() == 2, "adamw_step: bc_dev is two fp32 on the device");
    bcp = bc_dev->data_ptr<float>();
  }
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  NT_DISPATCH_FLOAT(param.scalar_type(), "adamw_step", [&] {
    constexpr int VEC = sizeof(scalar_t) == 4 ? 4 : 8;
    adamw_kernel<scalar_t, VEC><<<grid, AD_THREADS, 0, stream>>>(param.data_ptr<scalar_t>(), grad.data_ptr<scalar_t>(), master.data_ptr<float>(),
        m.data_ptr<float>(), v.data_ptr<float>(), n, static_cast<float>(lr), static_cast<float>(beta1), static_cast<float>(beta2),
        static_cast<float>(eps), static_cast<float>(wd), bc1, 1.f / std::sqrt(bc2), static_cast<float>(grad_scale),
        want_sq ? partial.data_ptr<float>() : nullptr, bcp);
  });
  NT_KERNEL_CHECK();
  return partial;
}

}  // namespace nt
