// Token pack / combine and their backward passes as atomic-free gathers.
//
// All four kernels are "one warp per row, 16-byte vectors": they are pure data movement with a
// k-term sum.  Forward pack scatters each token row to its k slots (read once, written k
// times); combine, pack-backward gather the k rows of a token in a fixed order with fp32
// accumulation, so results are bit-reproducible - the reference sums with fp32 / bf16
// atomicAdd in arrival order (csrc/kernels/combine_kernels.cu:22-31,
// csrc/kernels/backward_pack_kernel.cu:28-40).
//
// Token -> rows maps are given either as a fixed fan-out (`slot_of [T,k]`) or in CSR form
// (`row_start [T+1]`, `rows [A]`), which is what the reference-style entry points build from
// an arbitrary `packed_tokenId`.
//
// Every index read from a map (a slot, a packed row, a token id) is range-checked before it is used
// as an address: an index outside its tensor is skipped and recorded in the device status word
// (kernel id, offending value) instead of faulting, so a corrupted routing table surfaces as a
// Python exception at the end of the step.  The checks are compares on values the kernels load
// anyway; they are always compiled in.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <ATen/ATen.h>

#include "cuda_check.h"
#include "ops.h"
#include "vec.cuh"

namespace nt {

namespace {

constexpr int PK_WARPS = 4;

// packed_x[slot_of[t,j]] = x[t]; packed_token / packed_gate / packed_expert alongside.
template <typename T, int VEC>
__global__ void __launch_bounds__(PK_WARPS * 32)
pack_fwd_kernel(const T* __restrict__ x, const float* __restrict__ gates, const int* __restrict__ idx,
                const int* __restrict__ slot_of, T* __restrict__ packed_x, int* __restrict__ packed_token,
                int* __restrict__ packed_expert, float* __restrict__ packed_gate, long long tokens, int d, int k,
                StatusWord* __restrict__ status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long t = static_cast<long long>(blockIdx.x) * PK_WARPS + warp;
  if (t >= tokens) return;
  const long long A = tokens * k;
  if (lane < k) {
    const int s = slot_of[t * k + lane];
    if (s < 0 || s >= A) {
      report_status(status, kStatusBounds, kKernelPack, static_cast<uint32_t>(s));
    } else {
      packed_token[s] = static_cast<int>(t);
      packed_expert[s] = idx[t * k + lane];
      packed_gate[s] = gates[t * k + lane];
    }
  }
  for (int c = lane * VEC; c < d; c += 32 * VEC) {
    float v[VEC];
    load_vec<T, VEC>(x + t * d + c, v);
    for (int j = 0; j < k; ++j) {
      const long long s = slot_of[t * k + j];
      if (s >= 0 && s < A) store_vec<T, VEC>(packed_x + s * d + c, v);
    }
  }
}

// out[t] = residual[t] + sum_j w[r_j] * y[r_j] over the rows r_j of token t.
template <typename T, typename OutT, int VEC>
__global__ void __launch_bounds__(PK_WARPS * 32)
combine_fwd_kernel(const T* __restrict__ y, const float* __restrict__ w, const int* __restrict__ rows,
                   const int* __restrict__ row_start, int k_fixed, const T* __restrict__ residual,
                   OutT* __restrict__ out, long long tokens, int d, long long y_rows, StatusWord* __restrict__ status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long t = static_cast<long long>(blockIdx.x) * PK_WARPS + warp;
  if (t >= tokens) return;
  const long long lo = k_fixed > 0 ? t * k_fixed : row_start[t];
  const long long hi = k_fixed > 0 ? lo + k_fixed : row_start[t + 1];
  for (int c = lane * VEC; c < d; c += 32 * VEC) {
    float acc[VEC];
    if (residual != nullptr) {
      load_vec<T, VEC>(residual + t * d + c, acc);
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
    }
    for (long long a = lo; a < hi; ++a) {
      const int r = rows[a];
      if (r < 0 || r >= y_rows) {
        if (c == 0) report_status(status, kStatusBounds, kKernelCombine, static_cast<uint32_t>(r));
        continue;
      }
      const float g = w[r];
      float v[VEC];
      load_vec<T, VEC>(y + static_cast<long long>(r) * d + c, v);
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] = fmaf(g, v[i], acc[i]);
    }
    store_vec<OutT, VEC>(out + t * d + c, acc);
  }
}

// dy[a] = w[a] * dout[token[a]];  dw[a] = <dout[token[a]], y[a]>.   One warp per packed row.
template <typename T, typename GT, int VEC>
__global__ void __launch_bounds__(PK_WARPS * 32)
combine_bwd_kernel(const T* __restrict__ y, const int* __restrict__ token, const float* __restrict__ w,
                   const GT* __restrict__ dout, T* __restrict__ dy, float* __restrict__ dw, long long assignments, int d,
                   long long tokens, StatusWord* __restrict__ status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long a = static_cast<long long>(blockIdx.x) * PK_WARPS + warp;
  if (a >= assignments) return;
  const long long t = token[a];
  if (t < 0 || t >= tokens) {
    if (lane == 0) {
      report_status(status, kStatusBounds, kKernelCombine, static_cast<uint32_t>(t));
      dw[a] = 0.f;
    }
    return;
  }
  const float g = w[a];
  float dot = 0.f;
  for (int c = lane * VEC; c < d; c += 32 * VEC) {
    float go[VEC], yv[VEC];
    load_vec<GT, VEC>(dout + t * d + c, go);
    load_vec<T, VEC>(y + a * d + c, yv);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      dot = fmaf(go[i], yv[i], dot);
      go[i] *= g;
    }
    store_vec<T, VEC>(dy + a * d + c, go);
  }
  dot = warp_sum(dot);
  if (lane == 0) dw[a] = dot;
}

// dx[t] = sum_j dpacked[r_j] (fp32 accumulate, fixed order).
template <typename T, int VEC>
__global__ void __launch_bounds__(PK_WARPS * 32)
pack_bwd_kernel(const T* __restrict__ dpacked, const int* __restrict__ rows, const int* __restrict__ row_start, int k_fixed,
                T* __restrict__ dx, long long tokens, int d, long long packed_rows, StatusWord* __restrict__ status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long t = static_cast<long long>(blockIdx.x) * PK_WARPS + warp;
  if (t >= tokens) return;
  const long long lo = k_fixed > 0 ? t * k_fixed : row_start[t];
  const long long hi = k_fixed > 0 ? lo + k_fixed : row_start[t + 1];
  for (int c = lane * VEC; c < d; c += 32 * VEC) {
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
    for (long long a = lo; a < hi; ++a) {
      float v[VEC];
      const long long r = rows[a];
      if (r < 0 || r >= packed_rows) {
        if (c == 0) report_status(status, kStatusBounds, kKernelPack, static_cast<uint32_t>(r));
        continue;
      }
      load_vec<T, VEC>(dpacked + r * d + c, v);
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] += v[i];
    }
    store_vec<T, VEC>(dx + t * d + c, acc);
  }
}

// dgate[t,j] = dpacked_gate[a] for the packed row a of token t whose expert equals topk[t,j].
__global__ void pack_bwd_gate_kernel(const float* __restrict__ dpacked_gate, const int* __restrict__ token,
                                     const int* __restrict__ expert, const int* __restrict__ topk, float* __restrict__ dgate,
                                     long long assignments, int k) {
  const long long a = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (a >= assignments) return;
  const long long t = token[a];
  const int e = expert[a];
  for (int j = 0; j < k; ++j)
    if (topk[t * k + j] == e) { dgate[t * k + j] = dpacked_gate[a]; break; }  // a token picks an expert once
}

bool vec_ok(int d, int elem, std::initializer_list<const void*> ptrs) {
  if (d % (16 / elem) != 0) return false;
  for (const void* p : ptrs)
    if (p != nullptr && !is_aligned16(p)) return false;
  return true;
}

// CSR (row_start [T+1], rows [A]) of `token` with rows of a token in ascending packed index.
std::pair<at::Tensor, at::Tensor> csr_from_tokens(const at::Tensor& token, int64_t tokens) {
  auto tok64 = token.to(at::kLong);
  auto order = std::get<1>(at::sort(tok64, /*stable=*/true, /*dim=*/0, /*descending=*/false));
  auto counts = at::bincount(tok64, {}, tokens);
  auto row_start = at::zeros({tokens + 1}, token.options().dtype(at::kInt));
  row_start.slice(0, 1).copy_(at::cumsum(counts, 0));
  return {row_start, order.to(at::kInt)};
}

}  // namespace

// -> packed_x [A,d], packed_token [A] i32, packed_expert [A] i32, packed_gate [A] f32
std::vector<at::Tensor> pack_fwd(const at::Tensor& x, const at::Tensor& gates, const at::Tensor& idx, const at::Tensor& slot_of) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous(), "pack_fwd: x [T,d] contiguous");
  TORCH_CHECK(gates.scalar_type() == at::kFloat && gates.is_contiguous() && idx.scalar_type() == at::kInt && idx.is_contiguous() &&
              slot_of.scalar_type() == at::kInt && slot_of.is_contiguous(), "pack_fwd: gates f32, idx/slot_of i32, contiguous");
  c10::cuda::CUDAGuard guard(x.device());
  const long long tokens = x.size(0);
  const int d = static_cast<int>(x.size(1)), k = static_cast<int>(idx.size(1));
  TORCH_CHECK(k <= 32, "pack_fwd: top_k <= 32");
  const long long A = tokens * k;
  auto packed_x = at::empty({A, d}, x.options());
  auto packed_token = at::empty({A}, idx.options());
  auto packed_expert = at::empty({A}, idx.options());
  auto packed_gate = at::empty({A}, gates.options());
  if (A == 0) return {packed_x, packed_token, packed_expert, packed_gate};
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const unsigned grid = static_cast<unsigned>((tokens + PK_WARPS - 1) / PK_WARPS);
  NT_DISPATCH_FLOAT(x.scalar_type(), "pack_fwd", [&] {
    constexpr int V = 16 / sizeof(scalar_t);
    auto run = [&](auto kernel) {
      kernel<<<grid, PK_WARPS * 32, 0, stream>>>(x.data_ptr<scalar_t>(), gates.data_ptr<float>(), idx.data_ptr<int>(), slot_of.data_ptr<int>(),
          packed_x.data_ptr<scalar_t>(), packed_token.data_ptr<int>(), packed_expert.data_ptr<int>(), packed_gate.data_ptr<float>(), tokens, d, k,
          device_status_word());
    };
    if (vec_ok(d, sizeof(scalar_t), {x.data_ptr(), packed_x.data_ptr()})) run(pack_fwd_kernel<scalar_t, V>);
    else run(pack_fwd_kernel<scalar_t, 1>);
  });
  NT_KERNEL_CHECK();
  return {packed_x, packed_token, packed_expert, packed_gate};
}

// rows/row_start: CSR map, or (slot_of [T,k], undefined) for a fixed fan-out.  out dtype: y's, or fp32.
at::Tensor combine_fwd(const at::Tensor& y, const at::Tensor& w, const at::Tensor& rows, const c10::optional<at::Tensor>& row_start,
                       int64_t tokens, const c10::optional<at::Tensor>& residual, bool out_f32) {
  TORCH_CHECK(y.is_cuda() && y.dim() == 2 && y.is_contiguous() && w.scalar_type() == at::kFloat && w.is_contiguous() &&
              rows.scalar_type() == at::kInt && rows.is_contiguous(), "combine_fwd: y [A,d], w f32 [A], rows i32");
  c10::cuda::CUDAGuard guard(y.device());
  const int d = static_cast<int>(y.size(1));
  const int k_fixed = row_start.has_value() ? 0 : static_cast<int>(rows.numel() / std::max<int64_t>(tokens, 1));
  if (residual.has_value()) TORCH_CHECK(residual->is_contiguous() && residual->scalar_type() == y.scalar_type() && residual->numel() == tokens * d, "combine_fwd: bad residual");
  auto out = at::empty({tokens, d}, y.options().dtype(out_f32 ? at::kFloat : y.scalar_type()));
  if (tokens == 0) return out;
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const unsigned grid = static_cast<unsigned>((tokens + PK_WARPS - 1) / PK_WARPS);
  const int* rs = row_start.has_value() ? row_start->data_ptr<int>() : nullptr;
  NT_DISPATCH_FLOAT(y.scalar_type(), "combine_fwd", [&] {
    constexpr int V = 16 / sizeof(scalar_t);
    const scalar_t* res = residual.has_value() ? residual->data_ptr<scalar_t>() : nullptr;
    const bool vec = vec_ok(d, sizeof(scalar_t), {y.data_ptr(), res}) && (out_f32 ? d % 4 == 0 : true) && is_aligned16(out.data_ptr());
    auto run = [&](auto kernel, auto* outp) {
      kernel<<<grid, PK_WARPS * 32, 0, stream>>>(y.data_ptr<scalar_t>(), w.data_ptr<float>(), rows.data_ptr<int>(), rs, k_fixed, res, outp, tokens, d,
                                                 static_cast<long long>(y.size(0)), device_status_word());
    };
    if (out_f32) {
      // fp32 rows are written 4 elements per 16-byte store; keep the scalar path for simplicity
      run(combine_fwd_kernel<scalar_t, float, 1>, out.data_ptr<float>());
    } else if (vec) {
      run(combine_fwd_kernel<scalar_t, scalar_t, V>, out.data_ptr<scalar_t>());
    } else {
      run(combine_fwd_kernel<scalar_t, scalar_t, 1>, out.data_ptr<scalar_t>());
    }
  });
  NT_KERNEL_CHECK();
  return out;
}

// -> dy [A,d] (y's dtype), dw [A] f32
std::vector<at::Tensor> combine_bwd(const at::Tensor& y, const at::Tensor& token, const at::Tensor& w, const at::Tensor& dout) {
  TORCH_CHECK(y.is_cuda() && y.is_contiguous() && dout.is_contiguous() && token.scalar_type() == at::kInt && token.is_contiguous() &&
              w.scalar_type() == at::kFloat && w.is_contiguous(), "combine_bwd: contiguous y/dout, token i32, w f32");
  TORCH_CHECK(dout.scalar_type() == y.scalar_type() || dout.scalar_type() == at::kFloat, "combine_bwd: dout must be y's dtype or fp32");
  c10::cuda::CUDAGuard guard(y.device());
  const long long A = y.size(0);
  const int d = static_cast<int>(y.size(1));
  auto dy = at::empty_like(y);
  auto dw = at::empty({A}, w.options());
  if (A == 0) return {dy, dw};
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const unsigned grid = static_cast<unsigned>((A + PK_WARPS - 1) / PK_WARPS);
  NT_DISPATCH_FLOAT(y.scalar_type(), "combine_bwd", [&] {
    constexpr int V = 16 / sizeof(scalar_t);
    const bool same = dout.scalar_type() == y.scalar_type();
    const bool vec = same && vec_ok(d, sizeof(scalar_t), {y.data_ptr(), dout.data_ptr(), dy.data_ptr()});
    if (same) {
      auto run = [&](auto kernel) {
        kernel<<<grid, PK_WARPS * 32, 0, stream>>>(y.data_ptr<scalar_t>(), token.data_ptr<int>(), w.data_ptr<float>(), dout.data_ptr<scalar_t>(),
            dy.data_ptr<scalar_t>(), dw.data_ptr<float>(), A, d, static_cast<long long>(dout.size(0)), device_status_word());
      };
      if (vec) run(combine_bwd_kernel<scalar_t, scalar_t, V>); else run(combine_bwd_kernel<scalar_t, scalar_t, 1>);
    } else {
      combine_bwd_kernel<scalar_t, float, 1><<<grid, PK_WARPS * 32, 0, stream>>>(y.data_ptr<scalar_t>(), token.data_ptr<int>(), w.data_ptr<float>(),
          dout.data_ptr<float>(), dy.data_ptr<scalar_t>(), dw.data_ptr<float>(), A, d, static_cast<long long>(dout.size(0)), device_status_word());
    }
  });
  NT_KERNEL_CHECK();
  return {dy, dw};
}

at::Tensor pack_bwd(const at::Tensor& dpacked, const at::Tensor& rows, const c10::optional<at::Tensor>& row_start, int64_t tokens) {
  TORCH_CHECK(dpacked.is_cuda() && dpacked.dim() == 2 && dpacked.is_contiguous() && rows.scalar_type() == at::kInt && rows.is_contiguous(), "pack_bwd: bad arguments");
  c10::cuda::CUDAGuard guard(dpacked.device());
  const int d = static_cast<int>(dpacked.size(1));
  const int k_fixed = row_start.has_value() ? 0 : static_cast<int>(rows.numel() / std::max<int64_t>(tokens, 1));
  auto dx = at::empty({tokens, d}, dpacked.options());
  if (tokens == 0) return dx;
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const unsigned grid = static_cast<unsigned>((tokens + PK_WARPS - 1) / PK_WARPS);
  const int* rs = row_start.has_value() ? row_start->data_ptr<int>() : nullptr;
  NT_DISPATCH_FLOAT(dpacked.scalar_type(), "pack_bwd", [&] {
    constexpr int V = 16 / sizeof(scalar_t);
    auto run = [&](auto kernel) {
      kernel<<<grid, PK_WARPS * 32, 0, stream>>>(dpacked.data_ptr<scalar_t>(), rows.data_ptr<int>(), rs, k_fixed, dx.data_ptr<scalar_t>(), tokens, d,
                                                 static_cast<long long>(dpacked.size(0)), device_status_word());
    };
    if (vec_ok(d, sizeof(scalar_t), {dpacked.data_ptr(), dx.data_ptr()})) run(pack_bwd_kernel<scalar_t, V>); else run(pack_bwd_kernel<scalar_t, 1>);
  });
  NT_KERNEL_CHECK();
  return dx;
}

// ------------------------------------------------------------------ entry points with the reference's signatures
// pack_tokens_kernel(X, w, e, offset_cpy) -> (packed_X, packed_tokenId, packed_expert, packed_w)
std::vector<at::Tensor> pack_tokens_kernel(const at::Tensor& X, const at::Tensor& w, const at::Tensor& e, const at::Tensor& offset_cpy) {
  TORCH_CHECK(X.is_contiguous(), "X must be contiguous");
  TORCH_CHECK(e.scalar_type() == at::kInt, "topk experts must be int32");
  const int64_t E = std::max<int64_t>(offset_cpy.numel() - 1, 1);
  auto mask = at::empty({0}, e.options());
  auto ec = e.contiguous();
  // offset_cpy may hold E or E+1 entries; count over the larger to be safe
  auto counts = count_expert_kernel(ec, mask, std::max<int64_t>(E, offset_cpy.numel()), e.size(1));
  auto plan = assign_slots(ec, counts);
  return pack_fwd(X, w.to(at::kFloat).contiguous(), ec, plan[1]);
}

// combine_tokens_kernel(Y, tokenId, w, T, d) -> fp32 [T, d]
at::Tensor combine_tokens_kernel(const at::Tensor& Y, const at::Tensor& tokenId, const at::Tensor& w, int64_t T, int64_t d) {
  TORCH_CHECK(Y.size(1) == d, "hidden_dim does not match Y");
  auto csr = csr_from_tokens(tokenId, T);
  return combine_fwd(Y.contiguous(), w.to(at::kFloat).contiguous(), csr.second, csr.first, T, c10::nullopt, /*out_f32=*/true);
}

// combine_kernel_backward(Y, tokenId, w, dOut fp32 [T,d], d) -> (dY [A,d] in Y's dtype, dw fp32 [A])
std::vector<at::Tensor> combine_kernel_backward(const at::Tensor& Y, const at::Tensor& tokenId, const at::Tensor& w, const at::Tensor& dOut, int64_t d) {
  TORCH_CHECK(Y.size(1) == d, "hidden_dim does not match Y");
  return combine_bwd(Y.contiguous(), tokenId.to(at::kInt).contiguous(), w.to(at::kFloat).contiguous(), dOut.contiguous());
}

// pack_kernel_backward(dPackedX, dPackedW, tokenId, expert, topk_experts) -> (dX [T,d], dw fp32 [T,k])
std::vector<at::Tensor> pack_kernel_backward(const at::Tensor& dPackedX, const at::Tensor& dPackedW, const at::Tensor& tokenId,
                                             const at::Tensor& expert, const at::Tensor& topk) {
  c10::cuda::CUDAGuard guard(dPackedX.device());
  const int64_t T = topk.size(0), k = topk.size(1);
  auto csr = csr_from_tokens(tokenId, T);
  auto dX = pack_bwd(dPackedX.contiguous(), csr.second, csr.first, T);
  auto dgate = at::zeros({T, k}, dPackedW.options().dtype(at::kFloat));
  const long long A = tokenId.numel();
  if (A > 0) {
    auto dpw = dPackedW.to(at::kFloat).contiguous();
    auto tok = tokenId.to(at::kInt).contiguous();
    auto ex = expert.to(at::kInt).contiguous();
    auto tk = topk.to(at::kInt).contiguous();
    pack_bwd_gate_kernel<<<static_cast<unsigned>((A + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
        dpw.data_ptr<float>(), tok.data_ptr<int>(), ex.data_ptr<int>(), tk.data_ptr<int>(), dgate.data_ptr<float>(), A, static_cast<int>(k));
    NT_KERNEL_CHECK();
  }
  return {dX, dgate};
}

}  // namespace nt
