// MoE routing kernels.
//  * router_topk: logits = x . W_r^T in fp32, softmax, top-k, renormalised gates and per-expert
//    counts in one kernel (the reference does this with
//    a Linear, softmax, topk, a division and a separate counting kernel,
//    src/model/cuda_backend.py:24-52 / csrc/kernels/count_experts.cu).
//  * assign_slots: exclusive scan of the counts plus, for every (token, choice), its position
//    in expert-major order with ascending token id inside an expert.  One block per expert
//    scans the assignment list, so the order is a pure function of the routing - no atomics
//    (the reference hands out slots with atomicAdd, csrc/kernels/pack_tokens.cu:26-31).
//  * count_experts: the standalone histogram with optional mask of the reference's API.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <ATen/ATen.h>

#include "cuda_check.h"
#include "ops.h"
#include "vec.cuh"

namespace nt {

namespace {

constexpr int RT_WARPS = 4;
constexpr int RT_TOK = 4;       // tokens per warp pass (amortises the reads of W_r)
constexpr int RT_MAX_E = 256;   // experts supported by the fused router
constexpr int RT_SLOTS = RT_MAX_E / 32;

template <typename T, typename WT>
__global__ void __launch_bounds__(RT_WARPS * 32)
router_topk_kernel(const T* __restrict__ x, const WT* __restrict__ w, float* __restrict__ gates, int* __restrict__ idx,
                   float* __restrict__ probs, int* __restrict__ counts, float* __restrict__ prob_parts,
                   long long tokens, int d, int E, int k, StatusWord* __restrict__ status) {
  extern __shared__ float sx[];  // [RT_WARPS][RT_TOK][d] token rows as fp32
  __shared__ int s_counts[RT_MAX_E];
  __shared__ float s_psum[RT_WARPS][RT_MAX_E];
  float psum[RT_SLOTS];  // this warp's running sum of the probabilities of expert (slot * 32 + lane)
#pragma unroll
  for (int s = 0; s < RT_SLOTS; ++s) psum[s] = 0.f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_counts[e] = 0;
  __syncthreads();
  float* xs = sx + static_cast<size_t>(warp) * RT_TOK * d;
  const long long per_block = RT_WARPS * RT_TOK;
  for (long long base = static_cast<long long>(blockIdx.x) * per_block + warp * RT_TOK; base < tokens;
       base += static_cast<long long>(gridDim.x) * per_block) {
    const int nt = static_cast<int>(min(static_cast<long long>(RT_TOK), tokens - base));
    for (int t = 0; t < RT_TOK; ++t)
      for (int c = lane; c < d; c += 32) xs[t * d + c] = t < nt ? elem_to_float<T>(x[(base + t) * d + c]) : 0.f;
    __syncwarp();
    // lane (e % 32) keeps the logit of expert e in slot e / 32
    float logit[RT_TOK][RT_SLOTS];
#pragma unroll
    for (int t = 0; t < RT_TOK; ++t)
#pragma unroll
      for (int s = 0; s < RT_SLOTS; ++s) logit[t][s] = -INFINITY;
    for (int e = 0; e < E; ++e) {
      float acc[RT_TOK];
#pragma unroll
      for (int t = 0; t < RT_TOK; ++t) acc[t] = 0.f;
      const WT* we = w + static_cast<long long>(e) * d;
      for (int c = lane; c < d; c += 32) {
        const float wv = elem_to_float<WT>(we[c]);
#pragma unroll
        for (int t = 0; t < RT_TOK; ++t) acc[t] = fmaf(xs[t * d + c], wv, acc[t]);
      }
#pragma unroll
      for (int t = 0; t < RT_TOK; ++t) {
        const float v = warp_sum(acc[t]);
        if (lane == (e & 31)) {
#pragma unroll
          for (int s = 0; s < RT_SLOTS; ++s)
            if (s == (e >> 5)) logit[t][s] = v;
        }
      }
    }
#pragma unroll
    for (int t = 0; t < RT_TOK; ++t) {
      if (t >= nt) break;
      const long long tok = base + t;
      float mx = -INFINITY;
#pragma unroll
      for (int s = 0; s < RT_SLOTS; ++s) mx = fmaxf(mx, logit[t][s]);
      mx = warp_max(mx);
      float p[RT_SLOTS];
      float sum = 0.f;
#pragma unroll
      for (int s = 0; s < RT_SLOTS; ++s) {
        p[s] = (s * 32 + lane < E) ? __expf(logit[t][s] - mx) : 0.f;
        sum += p[s];
      }
      sum = warp_sum(sum);
      const float inv = 1.f / sum;
#pragma unroll
      for (int s = 0; s < RT_SLOTS; ++s) {
        p[s] *= inv;
        psum[s] += p[s];
        const int e = s * 32 + lane;
        if (e < E) probs[tok * E + e] = p[s];
      }
      // k rounds of warp arg-max; ties go to the lower expert id (torch.topk order on distinct values)
      float taken_sum = 0.f;
      float my_gate = 0.f;
      int my_e = 0;
      for (int j = 0; j < k; ++j) {
        float best = -1.f;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int s = 0; s < RT_SLOTS; ++s) {
          const int e = s * 32 + lane;
          if (e < E && p[s] > best) { best = p[s]; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
          if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (best_e >= E) {
          // No expert has a comparable probability: the token row holds NaN (an earlier kernel of the
          // step failed).  Route it to expert j with a neutral weight and say so, instead of using
          // the sentinel as an index.
          best_e = j;
          best = 0.f;
          if (lane == 0) report_status(status, kStatusBadArgument, kKernelPack, static_cast<uint32_t>(tok));
        }
#pragma unroll
        for (int s = 0; s < RT_SLOTS; ++s)
          if (s * 32 + lane == best_e) p[s] = -2.f;  // remove from later rounds
        taken_sum += best;
        if (lane == j) { my_gate = best; my_e = best_e; }
      }
      if (!(taken_sum > 0.f)) {  // all-NaN row: equal weights
        my_gate = 1.f;
        taken_sum = static_cast<float>(k);
      }
      if (lane < k) {
        gates[tok * k + lane] = my_gate / taken_sum;
        idx[tok * k + lane] = my_e;
        atomicAdd(&s_counts[my_e], 1);
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int s = 0; s < RT_SLOTS; ++s)
    if (s * 32 + lane < E) s_psum[warp][s * 32 + lane] = psum[s];
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    if (s_counts[e] != 0) atomicAdd(&counts[e], s_counts[e]);
    float t = 0.f;  // warps in index order: the block's partial sum does not depend on scheduling
#pragma unroll
    for (int w2 = 0; w2 < RT_WARPS; ++w2) t += s_psum[w2][e];
    prob_parts[static_cast<long long>(blockIdx.x) * E + e] = t;
  }
}

// The routing half of router_topk_kernel for logits that were computed elsewhere (a tensor-core GEMM): softmax,
// top-k with the same tie rule, renormalised gates, per-expert counts and the per-block sums of the
// probabilities.  One warp per token; lane (e % 32) holds expert e in slot e / 32.
__global__ void __launch_bounds__(RT_WARPS * 32)
router_from_logits_kernel(const float* __restrict__ logits, float* __restrict__ gates, int* __restrict__ idx,
                          float* __restrict__ probs, int* __restrict__ counts, float* __restrict__ prob_parts,
                          long long tokens, int E, int k, StatusWord* __restrict__ status) {
  __shared__ int s_counts[RT_MAX_E];
  __shared__ float s_psum[RT_WARPS][RT_MAX_E];
  float psum[RT_SLOTS];
#pragma unroll
  for (int s = 0; s < RT_SLOTS; ++s) psum[s] = 0.f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_counts[e] = 0;
  __syncthreads();
  for (long long tok = static_cast<long long>(blockIdx.x) * RT_WARPS + warp; tok < tokens;
       tok += static_cast<long long>(gridDim.x) * RT_WARPS) {
    float p[RT_SLOTS];
    float mx = -INFINITY;
#pragma unroll
    for (int s = 0; s < RT_SLOTS; ++s) {
      const int e = s * 32 + lane;
      p[s] = e < E ? logits[tok * E + e] : -INFINITY;
      mx = fmaxf(mx, p[s]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int s = 0; s < RT_SLOTS; ++s) {
      p[s] = (s * 32 + lane < E) ? __expf(p[s] - mx) : 0.f;
      sum += p[s];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int s = 0; s < RT_SLOTS; ++s) {
      p[s] *= inv;
      psum[s] += p[s];
      const int e = s * 32 + lane;
      if (e < E) probs[tok * E + e] = p[s];
    }
    float taken_sum = 0.f;
    float my_gate = 0.f;
    int my_e = 0;
    for (int j = 0; j < k; ++j) {
      float best = -1.f;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int s = 0; s < RT_SLOTS; ++s) {
        const int e = s * 32 + lane;
        if (e < E && p[s] > best) { best = p[s]; best_e = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
      }
      if (best_e >= E) {  // a row of NaN: fixed experts, neutral weight, and a record of it (see router_topk_kernel)
        best_e = j;
        best = 0.f;
        if (lane == 0) report_status(status, kStatusBadArgument, kKernelPack, static_cast<uint32_t>(tok));
      }
#pragma unroll
      for (int s = 0; s < RT_SLOTS; ++s)
        if (s * 32 + lane == best_e) p[s] = -2.f;
      taken_sum += best;
      if (lane == j) { my_gate = best; my_e = best_e; }
    }
    if (!(taken_sum > 0.f)) {
      my_gate = 1.f;
      taken_sum = static_cast<float>(k);
    }
    if (lane < k) {
      gates[tok * k + lane] = my_gate / taken_sum;
      idx[tok * k + lane] = my_e;
      atomicAdd(&s_counts[my_e], 1);
    }
  }
#pragma unroll
  for (int s = 0; s < RT_SLOTS; ++s)
    if (s * 32 + lane < E) s_psum[warp][s * 32 + lane] = psum[s];
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    if (s_counts[e] != 0) atomicAdd(&counts[e], s_counts[e]);
    float t = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < RT_WARPS; ++w2) t += s_psum[w2][e];
    prob_parts[static_cast<long long>(blockIdx.x) * E + e] = t;
  }
}

// out[c] = scale * sum over `parts` rows of in[p][c]; 8 row groups per column, added in a fixed order.
__global__ void scaled_column_sum_kernel(const float* __restrict__ in, float* __restrict__ out, int parts, int cols, float scale) {
  __shared__ float red[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < cols)
    for (int p = threadIdx.y; p < parts; p += 8) s += in[static_cast<long long>(p) * cols + c];
  red[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int y = 0; y < 8; ++y) t += red[y][threadIdx.x];
    out[c] = t * scale;
  }
}

// Backward of softmax -> top-k -> renormalise, one thread per token.
//   dl_tok = gradient of the logits through the gates (reaches tokens and router weight);
//   dl_all = dl_tok + gradient through the probabilities themselves (load-balancing loss; router weight only).
// The probability gradient may come as a [T, E] tensor, as the gradient of the column means ([E], every
// token then gets d_mean[e] / T), both, or neither.
template <typename TOut>
__global__ void router_bwd_kernel(const float* __restrict__ gates, const int* __restrict__ idx, const float* __restrict__ probs,
                                  const float* __restrict__ dgates, const float* __restrict__ dprobs,
                                  const float* __restrict__ dprobs_mean, TOut* __restrict__ dl_tok, TOut* __restrict__ dl_all,
                                  long long tokens, int E, int k) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  const float* p = probs + t * E;
  const int* id = idx + t * k;
  float top_sum = 0.f, gd = 0.f;
  for (int j = 0; j < k; ++j) {
    top_sum += p[id[j]];
    if (dgates != nullptr) gd += dgates[t * k + j] * gates[t * k + j];
  }
  // d(prob of chosen expert j) and its dot product with the probabilities
  float dot = 0.f;
  if (dgates != nullptr)
    for (int j = 0; j < k; ++j) dot += (dgates[t * k + j] - gd) / top_sum * p[id[j]];
  const float inv_t = 1.f / static_cast<float>(tokens);
  float dot2 = 0.f;
  const bool aux = dprobs != nullptr || dprobs_mean != nullptr;
  if (aux)
    for (int e = 0; e < E; ++e) {
      float g = 0.f;
      if (dprobs != nullptr) g += dprobs[t * E + e];
      if (dprobs_mean != nullptr) g += dprobs_mean[e] * inv_t;
      dot2 += g * p[e];
    }
  for (int e = 0; e < E; ++e) {
    float dp = 0.f;
    if (dgates != nullptr)
      for (int j = 0; j < k; ++j)
        if (id[j] == e) dp = (dgates[t * k + j] - gd) / top_sum;
    const float tok = p[e] * (dp - dot);
    float all = tok;
    if (aux) {
      float g = 0.f;
      if (dprobs != nullptr) g += dprobs[t * E + e];
      if (dprobs_mean != nullptr) g += dprobs_mean[e] * inv_t;
      all += p[e] * (g - dot2);
    }
    dl_tok[t * E + e] = float_to_elem<TOut>(tok);
    dl_all[t * E + e] = float_to_elem<TOut>(all);
  }
}

// Block e: offsets by a serial scan of `counts`, then slot_of[a] for every assignment a routed to e.
constexpr int SL_THREADS = 512;
constexpr int SL_PER_THREAD = 8;

__global__ void __launch_bounds__(SL_THREADS)
assign_slots_kernel(const int* __restrict__ idx, const int* __restrict__ counts, int* __restrict__ offsets,
                    int* __restrict__ slot_of, long long assignments, int E) {
  __shared__ int warp_tot[SL_THREADS / 32];
  __shared__ int s_base;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    int run = 0;
    for (int i = 0; i < e; ++i) run += counts[i];
    s_base = run;
    if (e == 0) {
      int acc = 0;
      offsets[0] = 0;
      for (int i = 0; i < E; ++i) { acc += counts[i]; offsets[i + 1] = acc; }
    }
  }
  __syncthreads();
  int running = s_base;
  const long long chunk = static_cast<long long>(SL_THREADS) * SL_PER_THREAD;
  for (long long start = 0; start < assignments; start += chunk) {
    const long long a0 = start + static_cast<long long>(threadIdx.x) * SL_PER_THREAD;
    int flags = 0, mine = 0;
#pragma unroll
    for (int i = 0; i < SL_PER_THREAD; ++i) {
      const long long a = a0 + i;
      if (a < assignments && idx[a] == e) { flags |= 1 << i; ++mine; }
    }
    int incl = mine;  // inclusive scan over the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int before = 0, total = 0;
    for (int wI = 0; wI < SL_THREADS / 32; ++wI) {
      const int v = warp_tot[wI];
      if (wI < warp) before += v;
      total += v;
    }
    int pos = running + before + incl - mine;
#pragma unroll
    for (int i = 0; i < SL_PER_THREAD; ++i)
      if (flags & (1 << i)) slot_of[a0 + i] = pos++;
    running += total;
    __syncthreads();
  }
}

__global__ void count_experts_kernel(const int* __restrict__ topk, const int* __restrict__ mask, int* __restrict__ counts,
                                     long long tokens, int E, int k) {
  extern __shared__ int hist[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  for (long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < tokens;
       t += static_cast<long long>(gridDim.x) * blockDim.x) {
    if (mask != nullptr && mask[t] == 0) continue;
    for (int j = 0; j < k; ++j) {
      const int e = topk[t * k + j];
      if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    if (hist[e] != 0) atomicAdd(&counts[e], hist[e]);
}

}  // namespace

// -> gates [T,k] f32, idx [T,k] i32, probs [T,E] f32, counts [E] i32, probs_mean [E] f32 (column means of probs)
std::vector<at::Tensor> router_topk(const at::Tensor& x, const at::Tensor& w, int64_t k) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && w.is_contiguous() && w.dim() == 2, "router_topk: x [T,d], w [E,d], contiguous");
  TORCH_CHECK(w.size(1) == x.size(1), "router_topk: width mismatch");
  c10::cuda::CUDAGuard guard(x.device());
  const long long tokens = x.size(0);
  const int d = static_cast<int>(x.size(1)), E = static_cast<int>(w.size(0));
  TORCH_CHECK(E <= RT_MAX_E, "router_topk supports up to ", RT_MAX_E, " experts");
  TORCH_CHECK(k >= 1 && k <= E && k <= 32, "router_topk: 1 <= k <= min(E, 32)");
  auto f32 = x.options().dtype(at::kFloat);
  auto i32 = x.options().dtype(at::kInt);
  auto gates = at::empty({tokens, k}, f32);
  auto idx = at::empty({tokens, k}, i32);
  auto probs = at::empty({tokens, E}, f32);
  auto counts = at::zeros({E}, i32);
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const long long per_block = RT_WARPS * RT_TOK;
  const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>((tokens + per_block - 1) / per_block, 8LL * sms)));
  auto probs_mean = tokens > 0 ? at::empty({E}, f32) : at::zeros({E}, f32);
  if (tokens > 0) {
    auto parts = at::empty({grid, E}, f32);
    const size_t smem = sizeof(float) * RT_WARPS * RT_TOK * d;
    TORCH_CHECK(smem <= 160 * 1024, "router_topk: d too large");
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    NT_DISPATCH_FLOAT(x.scalar_type(), "router_topk", [&] {
      using x_t = scalar_t;
      NT_DISPATCH_FLOAT(w.scalar_type(), "router_topk(w)", [&] {
        auto kernel = router_topk_kernel<x_t, scalar_t>;
        if (smem > 48 * 1024) NT_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        kernel<<<grid, RT_WARPS * 32, smem, stream>>>(x.data_ptr<x_t>(), w.data_ptr<scalar_t>(), gates.data_ptr<float>(), idx.data_ptr<int>(),
            probs.data_ptr<float>(), counts.data_ptr<int>(), parts.data_ptr<float>(), tokens, d, E, static_cast<int>(k), device_status_word());
      });
    });
    NT_KERNEL_CHECK();
    scaled_column_sum_kernel<<<(E + 31) / 32, dim3(32, 8), 0, stream>>>(parts.data_ptr<float>(), probs_mean.data_ptr<float>(), grid, E,
                                                                         1.f / static_cast<float>(tokens));
    NT_KERNEL_CHECK();
  }
  return {gates, idx, probs, counts, probs_mean};
}

// The same five outputs as router_topk from fp32 logits [T, E] (e.g. of the tensor-core GEMM, which is the faster
// way to form them once experts x width no longer fits the caches router_topk_kernel reads the router matrix through).
std::vector<at::Tensor> router_from_logits(const at::Tensor& logits, int64_t k) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous() && logits.scalar_type() == at::kFloat,
              "router_from_logits: logits fp32 [T, E], contiguous");
  c10::cuda::CUDAGuard guard(logits.device());
  const long long tokens = logits.size(0);
  const int E = static_cast<int>(logits.size(1));
  TORCH_CHECK(E >= 1 && E <= RT_MAX_E, "router_from_logits supports up to ", RT_MAX_E, " experts");
  TORCH_CHECK(k >= 1 && k <= E && k <= 32, "router_from_logits: 1 <= k <= min(E, 32)");
  auto f32 = logits.options();
  auto i32 = logits.options().dtype(at::kInt);
  auto gates = at::empty({tokens, k}, f32);
  auto idx = at::empty({tokens, k}, i32);
  auto probs = at::empty({tokens, E}, f32);
  auto counts = at::zeros({E}, i32);
  auto probs_mean = tokens > 0 ? at::empty({E}, f32) : at::zeros({E}, f32);
  if (tokens > 0) {
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>((tokens + RT_WARPS - 1) / RT_WARPS, 8LL * sms)));
    auto parts = at::empty({grid, E}, f32);
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    router_from_logits_kernel<<<grid, RT_WARPS * 32, 0, stream>>>(logits.data_ptr<float>(), gates.data_ptr<float>(), idx.data_ptr<int>(),
                                                                  probs.data_ptr<float>(), counts.data_ptr<int>(), parts.data_ptr<float>(),
                                                                  tokens, E, static_cast<int>(k), device_status_word());
    NT_KERNEL_CHECK();
    scaled_column_sum_kernel<<<(E + 31) / 32, dim3(32, 8), 0, stream>>>(parts.data_ptr<float>(), probs_mean.data_ptr<float>(), grid, E,
                                                                         1.f / static_cast<float>(tokens));
    NT_KERNEL_CHECK();
  }
  return {gates, idx, probs, counts, probs_mean};
}

// Backward of the fused router up to the logits; see router_bwd_kernel.  `like` gives the output dtype.
std::vector<at::Tensor> router_bwd(const at::Tensor& gates, const at::Tensor& idx, const at::Tensor& probs,
                                   const c10::optional<at::Tensor>& dgates, const c10::optional<at::Tensor>& dprobs,
                                   const c10::optional<at::Tensor>& dprobs_mean, const at::Tensor& like) {
  TORCH_CHECK(gates.is_cuda() && gates.is_contiguous() && gates.scalar_type() == at::kFloat && idx.is_contiguous() &&
                  idx.scalar_type() == at::kInt && probs.is_contiguous() && probs.scalar_type() == at::kFloat,
              "router_bwd: gates f32 [T,k], idx i32 [T,k], probs f32 [T,E], contiguous");
  c10::cuda::CUDAGuard guard(probs.device());
  const long long tokens = probs.size(0);
  const int E = static_cast<int>(probs.size(1)), k = static_cast<int>(gates.size(1));
  auto check = [&](const c10::optional<at::Tensor>& t, long long n, const char* name) -> const float* {
    if (!t.has_value()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == at::kFloat && t->numel() == n, "router_bwd: bad ", name);
    return t->data_ptr<float>();
  };
  const float* dg = check(dgates, tokens * k, "dgates");
  const float* dp = check(dprobs, tokens * E, "dprobs");
  const float* dm = check(dprobs_mean, E, "dprobs_mean");
  auto dl_tok = at::empty({tokens, E}, like.options());
  auto dl_all = at::empty({tokens, E}, like.options());
  if (tokens == 0) return {dl_tok, dl_all};
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const unsigned grid = static_cast<unsigned>((tokens + 127) / 128);
  NT_DISPATCH_FLOAT(like.scalar_type(), "router_bwd", [&] {
    router_bwd_kernel<scalar_t><<<grid, 128, 0, stream>>>(gates.data_ptr<float>(), idx.data_ptr<int>(), probs.data_ptr<float>(), dg, dp, dm,
                                                          dl_tok.data_ptr<scalar_t>(), dl_all.data_ptr<scalar_t>(), tokens, E, k);
  });
  NT_KERNEL_CHECK();
  return {dl_tok, dl_all};
}

// -> offsets [E+1] i32, slot_of [T,k] i32
std::vector<at::Tensor> assign_slots(const at::Tensor& idx, const at::Tensor& counts) {
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kInt && idx.is_contiguous(), "assign_slots: idx int32 contiguous");
  TORCH_CHECK(counts.scalar_type() == at::kInt && counts.is_contiguous(), "assign_slots: counts int32");
  c10::cuda::CUDAGuard guard(idx.device());
  const int E = static_cast<int>(counts.numel());
  auto offsets = at::empty({E + 1}, counts.options());
  auto slot_of = at::empty_like(idx);
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  assign_slots_kernel<<<E, SL_THREADS, 0, stream>>>(idx.data_ptr<int>(), counts.data_ptr<int>(), offsets.data_ptr<int>(),
                                                     slot_of.data_ptr<int>(), idx.numel(), E);
  NT_KERNEL_CHECK();
  return {offsets, slot_of};
}

at::Tensor count_expert_kernel(const at::Tensor& topk, const at::Tensor& mask, int64_t E, int64_t k) {
  TORCH_CHECK(topk.is_cuda() && topk.scalar_type() == at::kInt && topk.is_contiguous(), "count_expert_kernel: topk must be int32 contiguous");
  TORCH_CHECK(mask.scalar_type() == at::kInt && mask.is_contiguous(), "count_expert_kernel: mask must be int32 contiguous");
  c10::cuda::CUDAGuard guard(topk.device());
  const long long tokens = topk.numel() / std::max<int64_t>(k, 1);
  auto counts = at::zeros({E}, topk.options());  // zero-fill is ordered on the current stream
  if (tokens == 0) return counts;
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const int grid = static_cast<int>(std::min<long long>((tokens + 255) / 256, 1184));
  count_experts_kernel<<<grid, 256, sizeof(int) * E, stream>>>(topk.data_ptr<int>(), mask.numel() ? mask.data_ptr<int>() : nullptr,
                                                                counts.data_ptr<int>(), tokens, static_cast<int>(E), static_cast<int>(k));
  NT_KERNEL_CHECK();
  return counts;
}

}  // namespace nt
