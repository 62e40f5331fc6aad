// LayerNorm forward / backward with the model's semantics: biased variance, eps inside the
// square root, affine gamma/beta (src/model/model.py:92-105 of the reference).
// Memory-bound: one warp per row, 16-byte vector loads when the row allows, fp32 statistics.
// Backward produces dx plus per-block partial sums of dgamma/dbeta that a second kernel folds
// in a fixed order (no atomics, run-to-run deterministic).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <ATen/ATen.h>

#include "cuda_check.h"
#include "ops.h"
#include "vec.cuh"

namespace nt {

namespace {

constexpr int LN_WARPS = 4;

template <typename T, int VEC>
__global__ void __launch_bounds__(LN_WARPS * 32)
ln_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ y,
              float* __restrict__ mean_out, float* __restrict__ rstd_out, long long rows, int d, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * LN_WARPS + warp;
  if (row >= rows) return;
  const T* xr = x + row * d;
  T* yr = y + row * d;
  float sum = 0.f;
  for (int c = lane * VEC; c < d; c += 32 * VEC) {
    float v[VEC];
    load_vec<T, VEC>(xr + c, v);
#pragma unroll
    for (int i = 0; i < VEC; ++i) sum += v[i];
  }
  const float mean = warp_sum(sum) / d;
  float sq = 0.f;
  for (int c = lane * VEC; c < d; c += 32 * VEC) {
    float v[VEC];
    load_vec<T, VEC>(xr + c, v);
#pragma unroll
    for (int i = 0; i < VEC; ++i) sq += (v[i] - mean) * (v[i] - mean);
  }
  const float rstd = rsqrtf(warp_sum(sq) / d + eps);
  for (int c = lane * VEC; c < d; c += 32 * VEC) {
    float v[VEC], g[VEC], b[VEC];
    load_vec<T, VEC>(xr + c, v);
    load_vec<T, VEC>(gamma + c, g);
    load_vec<T, VEC>(beta + c, b);
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[i] = (v[i] - mean) * rstd * g[i] + b[i];
    store_vec<T, VEC>(yr + c, v);
  }
  if (lane == 0) {
    mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
}

// Register-resident forward for d <= CHUNKS * 32 * VEC: the row is read from memory once (all of a
// lane's 16-byte pieces requested before the first is used) and the two reductions run on registers.
template <typename T, int VEC, int CHUNKS>
__global__ void __launch_bounds__(LN_WARPS * 32)
ln_fwd_reg_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ y,
                  float* __restrict__ mean_out, float* __restrict__ rstd_out, long long rows, int d, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * LN_WARPS + warp;
  if (row >= rows) return;
  float v[CHUNKS][VEC];
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) {
    const int c = (j * 32 + lane) * VEC;
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[j][i] = 0.f;
    if (c < d) load_vec<T, VEC>(x + row * d + c, v[j]);
  }
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j)
#pragma unroll
    for (int i = 0; i < VEC; ++i) sum += v[j][i];
  const float mean = warp_sum(sum) / d;
  float sq = 0.f;
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) {
    const int c = (j * 32 + lane) * VEC;
    if (c < d) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) sq += (v[j][i] - mean) * (v[j][i] - mean);
    }
  }
  const float rstd = rsqrtf(warp_sum(sq) / d + eps);
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) {
    const int c = (j * 32 + lane) * VEC;
    if (c < d) {
      float g[VEC], b[VEC];
      load_vec<T, VEC>(gamma + c, g);
      load_vec<T, VEC>(beta + c, b);
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[j][i] = (v[j][i] - mean) * rstd * g[i] + b[i];
      store_vec<T, VEC>(y + row * d + c, v[j]);
    }
  }
  if (lane == 0) {
    mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
}

// dx = rstd * (gy - mean(gy) - xhat * mean(gy * xhat)), gy = gamma * dy.
template <typename T, int VEC>
__global__ void __launch_bounds__(LN_WARPS * 32)
ln_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
              const float* __restrict__ mean_in, const float* __restrict__ rstd_in, T* __restrict__ dx,
              const T* __restrict__ dres, float* __restrict__ part_gamma, float* __restrict__ part_beta, long long rows, int d) {
  extern __shared__ float acc[];  // [2][LN_WARPS][d]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* ag = acc + warp * d;
  float* ab = acc + (LN_WARPS + warp) * d;
  for (int c = lane; c < d; c += 32) { ag[c] = 0.f; ab[c] = 0.f; }
  __syncwarp();
  for (long long row = static_cast<long long>(blockIdx.x) * LN_WARPS + warp; row < rows;
       row += static_cast<long long>(gridDim.x) * LN_WARPS) {
    const T* xr = x + row * d;
    const T* dyr = dy + row * d;
    const float mean = mean_in[row], rstd = rstd_in[row];
    float s1 = 0.f, s2 = 0.f;
    for (int c = lane * VEC; c < d; c += 32 * VEC) {
      float xv[VEC], gv[VEC], dv[VEC];
      load_vec<T, VEC>(xr + c, xv);
      load_vec<T, VEC>(gamma + c, gv);
      load_vec<T, VEC>(dyr + c, dv);
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float xhat = (xv[i] - mean) * rstd;
        const float gy = gv[i] * dv[i];
        s1 += gy;
        s2 += gy * xhat;
        ag[c + i] += dv[i] * xhat;
        ab[c + i] += dv[i];
      }
    }
    s1 = warp_sum(s1) / d;
    s2 = warp_sum(s2) / d;
    for (int c = lane * VEC; c < d; c += 32 * VEC) {
      float xv[VEC], gv[VEC], dv[VEC];
      load_vec<T, VEC>(xr + c, xv);
      load_vec<T, VEC>(gamma + c, gv);
      load_vec<T, VEC>(dyr + c, dv);
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float xhat = (xv[i] - mean) * rstd;
        xv[i] = rstd * (gv[i] * dv[i] - s1 - xhat * s2);
      }
      if (dres != nullptr) {  // gradient that reached x on the path around the normalisation
        load_vec<T, VEC>(dres + row * d + c, dv);
#pragma unroll
        for (int i = 0; i < VEC; ++i) xv[i] += dv[i];
      }
      store_vec<T, VEC>(dx + row * d + c, xv);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float g = 0.f, b = 0.f;
#pragma unroll
    for (int w = 0; w < LN_WARPS; ++w) {
      g += acc[w * d + c];
      b += acc[(LN_WARPS + w) * d + c];
    }
    part_gamma[static_cast<long long>(blockIdx.x) * d + c] = g;
    part_beta[static_cast<long long>(blockIdx.x) * d + c] = b;
  }
}

// Register-resident variant for d <= CHUNKS * 32 * VEC: lane l owns columns (j*32 + l)*VEC.. of
// every row its warp visits, so dgamma/dbeta partial sums never leave registers until the end
// and each row is read from memory once.
template <typename T, int VEC, int CHUNKS>
__global__ void __launch_bounds__(LN_WARPS * 32)
ln_bwd_reg_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                  const float* __restrict__ mean_in, const float* __restrict__ rstd_in, T* __restrict__ dx,
                  const T* __restrict__ dres, float* __restrict__ part_gamma, float* __restrict__ part_beta, long long rows, int d) {
  extern __shared__ float acc[];  // [2][LN_WARPS][d], used once at the end
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float gv[CHUNKS][VEC], ag[CHUNKS][VEC], ab[CHUNKS][VEC];
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) {
    const int c = (j * 32 + lane) * VEC;
#pragma unroll
    for (int i = 0; i < VEC; ++i) { ag[j][i] = 0.f; ab[j][i] = 0.f; gv[j][i] = 0.f; }
    if (c < d) load_vec<T, VEC>(gamma + c, gv[j]);
  }
  // While a row is reduced, the warp's next row is pulled into L2 (one request per 128-byte line,
  // no registers held), so its loads in the next iteration do not wait for DRAM.
  const long long stride = static_cast<long long>(gridDim.x) * LN_WARPS;
  for (long long row = static_cast<long long>(blockIdx.x) * LN_WARPS + warp; row < rows; row += stride) {
    if (row + stride < rows && (lane & 7) == 0) {
#pragma unroll
      for (int j = 0; j < CHUNKS; ++j) {
        const int c = (j * 32 + lane) * VEC;
        if (c < d) {
          const long long o = (row + stride) * d + c;
          asm volatile("prefetch.global.L2 [%0];" ::"l"(x + o));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(dy + o));
          if (dres != nullptr) asm volatile("prefetch.global.L2 [%0];" ::"l"(dres + o));
        }
      }
    }
    const float mean = mean_in[row], rstd = rstd_in[row];
    float xh[CHUNKS][VEC], dv[CHUNKS][VEC];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
      const int c = (j * 32 + lane) * VEC;
      if (c < d) {
        load_vec<T, VEC>(x + row * d + c, xh[j]);
        load_vec<T, VEC>(dy + row * d + c, dv[j]);
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          xh[j][i] = (xh[j][i] - mean) * rstd;
          const float gy = gv[j][i] * dv[j][i];
          s1 += gy;
          s2 += gy * xh[j][i];
          ag[j][i] += dv[j][i] * xh[j][i];
          ab[j][i] += dv[j][i];
        }
      }
    }
    s1 = warp_sum(s1) / d;
    s2 = warp_sum(s2) / d;
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
      const int c = (j * 32 + lane) * VEC;
      if (c < d) {
        float out[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) out[i] = rstd * (gv[j][i] * dv[j][i] - s1 - xh[j][i] * s2);
        if (dres != nullptr) {  // gradient that reached x on the path around the normalisation
          float extra[VEC];
          load_vec<T, VEC>(dres + row * d + c, extra);
#pragma unroll
          for (int i = 0; i < VEC; ++i) out[i] += extra[i];
        }
        store_vec<T, VEC>(dx + row * d + c, out);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < CHUNKS; ++j) {
    const int c = (j * 32 + lane) * VEC;
    if (c < d) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        acc[warp * d + c + i] = ag[j][i];
        acc[(LN_WARPS + warp) * d + c + i] = ab[j][i];
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float g = 0.f, b = 0.f;
#pragma unroll
    for (int w = 0; w < LN_WARPS; ++w) {
      g += acc[w * d + c];
      b += acc[(LN_WARPS + w) * d + c];
    }
    part_gamma[static_cast<long long>(blockIdx.x) * d + c] = g;
    part_beta[static_cast<long long>(blockIdx.x) * d + c] = b;
  }
}

// out[c] = sum over `parts` rows of in[p][c].  Block = 32 columns x 8 row groups; each group adds
// its rows in index order and the 8 group sums are added in group order, so the result does not
// depend on scheduling.
template <typename TOut>
__global__ void column_sum_kernel(const float* __restrict__ in0, const float* __restrict__ in1, TOut* __restrict__ out0,
                                  TOut* __restrict__ out1, int parts, int d) {
  // blockIdx.y picks the array (dgamma partials / dbeta partials): one launch folds both
  const float* in = blockIdx.y == 0 ? in0 : in1;
  TOut* out = blockIdx.y == 0 ? out0 : out1;
  __shared__ float red[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < d)
    for (int p = threadIdx.y; p < parts; p += 8) s += in[static_cast<long long>(p) * d + c];
  red[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < d) {
    float t = 0.f;
#pragma unroll
    for (int y = 0; y < 8; ++y) t += red[y][threadIdx.x];
    out[c] = float_to_elem<TOut>(t);
  }
}

}  // namespace

std::vector<at::Tensor> layer_norm_fwd(const at::Tensor& x, const at::Tensor& gamma, const at::Tensor& beta, double eps) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && gamma.is_contiguous() && beta.is_contiguous(), "layer_norm_fwd: contiguous CUDA tensors");
  TORCH_CHECK(gamma.scalar_type() == x.scalar_type() && beta.scalar_type() == x.scalar_type(), "gamma/beta must share x's dtype");
  c10::cuda::CUDAGuard guard(x.device());
  const int d = static_cast<int>(x.size(-1));
  const long long rows = x.numel() / d;
  auto y = at::empty_like(x);
  auto mean = at::empty({rows}, x.options().dtype(at::kFloat));
  auto rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  if (rows == 0) return {y, mean, rstd};
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const unsigned grid = static_cast<unsigned>((rows + LN_WARPS - 1) / LN_WARPS);
  NT_DISPATCH_FLOAT(x.scalar_type(), "layer_norm_fwd", [&] {
    constexpr int V = 16 / sizeof(scalar_t);
    const bool vec = d % V == 0 && is_aligned16(x.data_ptr()) && is_aligned16(gamma.data_ptr()) && is_aligned16(beta.data_ptr());
    auto launch = [&](auto kernel) {
      kernel<<<grid, LN_WARPS * 32, 0, stream>>>(x.data_ptr<scalar_t>(), gamma.data_ptr<scalar_t>(), beta.data_ptr<scalar_t>(),
          y.data_ptr<scalar_t>(), mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, d, static_cast<float>(eps));
    };
    if (vec && d <= 32 * V) launch(ln_fwd_reg_kernel<scalar_t, V, 1>);
    else if (vec && d <= 64 * V) launch(ln_fwd_reg_kernel<scalar_t, V, 2>);
    else if (vec && d <= 128 * V) launch(ln_fwd_reg_kernel<scalar_t, V, 4>);
    else if (vec)
      ln_fwd_kernel<scalar_t, V><<<grid, LN_WARPS * 32, 0, stream>>>(x.data_ptr<scalar_t>(), gamma.data_ptr<scalar_t>(), beta.data_ptr<scalar_t>(),
          y.data_ptr<scalar_t>(), mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, d, static_cast<float>(eps));
    else
      ln_fwd_kernel<scalar_t, 1><<<grid, LN_WARPS * 32, 0, stream>>>(x.data_ptr<scalar_t>(), gamma.data_ptr<scalar_t>(), beta.data_ptr<scalar_t>(),
          y.data_ptr<scalar_t>(), mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, d, static_cast<float>(eps));
  });
  NT_KERNEL_CHECK();
  return {y, mean, rstd};
}

std::vector<at::Tensor> layer_norm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& gamma,
                                       const at::Tensor& mean, const at::Tensor& rstd, const c10::optional<at::Tensor>& dres,
                                       const c10::optional<at::Tensor>& dgamma_out, const c10::optional<at::Tensor>& dbeta_out) {
  TORCH_CHECK(dy.is_cuda() && dy.is_contiguous() && x.is_contiguous() && gamma.is_contiguous(), "layer_norm_bwd: contiguous CUDA tensors");
  TORCH_CHECK(dy.scalar_type() == x.scalar_type(), "dy and x must share a dtype");
  if (dres.has_value())
    TORCH_CHECK(dres->is_cuda() && dres->is_contiguous() && dres->scalar_type() == x.scalar_type() && dres->numel() == x.numel(),
                "layer_norm_bwd: the extra gradient must match x");
  c10::cuda::CUDAGuard guard(x.device());
  const int d = static_cast<int>(x.size(-1));
  const long long rows = x.numel() / d;
  auto dx = at::empty_like(x);
  TORCH_CHECK(dgamma_out.has_value() == dbeta_out.has_value(), "layer_norm_bwd: give both gradient outputs or neither");
  at::Tensor dgamma, dbeta;
  if (dgamma_out.has_value()) {
    dgamma = *dgamma_out;
    dbeta = *dbeta_out;
    TORCH_CHECK(dgamma.is_cuda() && dgamma.is_contiguous() && dbeta.is_contiguous() && dgamma.numel() == d && dbeta.numel() == d &&
                    dgamma.scalar_type() == dbeta.scalar_type(), "layer_norm_bwd: gradient outputs must be contiguous [d] tensors of one dtype");
  } else {
    dgamma = at::empty({d}, x.options().dtype(at::kFloat));
    dbeta = at::empty({d}, x.options().dtype(at::kFloat));
  }
  if (rows == 0) {
    dgamma.zero_();
    dbeta.zero_();
    return {dx, dgamma, dbeta};
  }
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int grid = static_cast<int>(std::min<long long>((rows + LN_WARPS - 1) / LN_WARPS, 4LL * sms));
  const size_t smem = sizeof(float) * 2 * LN_WARPS * d;
  TORCH_CHECK(smem <= 200 * 1024, "layer_norm_bwd: d too large for the shared-memory accumulators");
  auto part_g = at::empty({grid, d}, x.options().dtype(at::kFloat));
  auto part_b = at::empty({grid, d}, x.options().dtype(at::kFloat));
  NT_DISPATCH_FLOAT(x.scalar_type(), "layer_norm_bwd", [&] {
    constexpr int V = 16 / sizeof(scalar_t);
    const scalar_t* extra = dres.has_value() ? dres->data_ptr<scalar_t>() : nullptr;
    const bool vec = d % V == 0 && is_aligned16(x.data_ptr()) && is_aligned16(dy.data_ptr()) && is_aligned16(gamma.data_ptr()) &&
                     is_aligned16(extra);
    auto launch = [&](auto kernel) {
      if (smem > 48 * 1024) NT_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
      kernel<<<grid, LN_WARPS * 32, smem, stream>>>(dy.data_ptr<scalar_t>(), x.data_ptr<scalar_t>(), gamma.data_ptr<scalar_t>(),
          mean.data_ptr<float>(), rstd.data_ptr<float>(), dx.data_ptr<scalar_t>(), extra, part_g.data_ptr<float>(), part_b.data_ptr<float>(), rows, d);
    };
    if (vec && d <= 32 * V) launch(ln_bwd_reg_kernel<scalar_t, V, 1>);
    else if (vec && d <= 64 * V) launch(ln_bwd_reg_kernel<scalar_t, V, 2>);
    else if (vec && d <= 128 * V) launch(ln_bwd_reg_kernel<scalar_t, V, 4>);
    else if (vec) launch(ln_bwd_kernel<scalar_t, V>);
    else launch(ln_bwd_kernel<scalar_t, 1>);
  });
  NT_KERNEL_CHECK();
  const dim3 fold_grid((d + 31) / 32, 2);
  if (dgamma.scalar_type() == at::kFloat) {
    column_sum_kernel<float><<<fold_grid, dim3(32, 8), 0, stream>>>(part_g.data_ptr<float>(), part_b.data_ptr<float>(), dgamma.data_ptr<float>(),
                                                                    dbeta.data_ptr<float>(), grid, d);
  } else if (dgamma.scalar_type() == at::kBFloat16) {
    column_sum_kernel<c10::BFloat16><<<fold_grid, dim3(32, 8), 0, stream>>>(part_g.data_ptr<float>(), part_b.data_ptr<float>(),
                                                                            dgamma.data_ptr<c10::BFloat16>(), dbeta.data_ptr<c10::BFloat16>(), grid, d);
  } else {
    TORCH_CHECK(dgamma.scalar_type() == at::kHalf, "layer_norm_bwd: gradient outputs must be fp32, bf16 or fp16");
    column_sum_kernel<c10::Half><<<fold_grid, dim3(32, 8), 0, stream>>>(part_g.data_ptr<float>(), part_b.data_ptr<float>(),
                                                                        dgamma.data_ptr<c10::Half>(), dbeta.data_ptr<c10::Half>(), grid, d);
  }
  NT_KERNEL_CHECK();
  return {dx, dgamma, dbeta};
}

}  // namespace nt
