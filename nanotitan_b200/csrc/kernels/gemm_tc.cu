// Host side of the tcgen05 GEMM: shape bookkeeping, TMA descriptors, tile-size choice, launch.
// The dense, grouped-by-expert and weight-gradient products that the reference runs as nn.Linear / cuBLAS calls
// (src/model/model.py:79-89, 128-182; src/model/feed_fwd.py:19-46) and as its SIMT kernels (csrc/kernels/gemm.cu:38-110,
// grouped_gemm.cu:12-60, bwd_grouped_gemm_dX.cu, bwd_grouped_gemm_dW.cu) all come through `gemm_tc` here.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <ATen/ATen.h>

#include <cstdlib>
#include <cstring>

#include "cuda_check.h"
#include "gemm_tc.cuh"
#include "gemm_tc2.cuh"
#include "ops.h"
#include "tma_desc.h"

namespace nt {

namespace {

using gemm::Args;

int dtype_code(const at::Tensor& t) {
  if (t.scalar_type() == at::kBFloat16) return 1;
  if (t.scalar_type() == at::kHalf) return 0;
  TORCH_CHECK(false, "gemm_tc: operands must be bf16 or fp16, got ", t.scalar_type());
}

void check_operand(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.dim() == 2 || t.dim() == 3, name, " must be 2-D or 3-D");
  if (t.numel() == 0) return;  // an operand without rows never reaches a kernel; its strides mean nothing
  TORCH_CHECK(t.stride(-1) == 1, name, " must have a contiguous last dim");
  TORCH_CHECK(t.stride(-2) % 8 == 0, name, ": row stride must be a multiple of 8 elements (TMA needs 16-byte strides)");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, name, " must be 16-byte aligned");
  if (t.dim() == 3) TORCH_CHECK(t.stride(0) % 8 == 0, name, ": group stride must be a multiple of 8 elements");
}

CUtensorMap map_a(const at::Tensor& a, bool a_mn) {
  const uint64_t dims[2] = {static_cast<uint64_t>(a.size(1)), static_cast<uint64_t>(a.size(0))};
  const uint64_t strides[1] = {static_cast<uint64_t>(a.stride(0)) * 2};
  const uint32_t box[2] = {64, a_mn ? 64u : 128u};
  return make_tma_desc(a.data_ptr(), 2, 2, dims, strides, box, true);
}

CUtensorMap map_b(const at::Tensor& b, bool b_mn, int box_rows) {
  const bool three = b.dim() == 3;
  const uint64_t groups = three ? b.size(0) : 1;
  const uint64_t rows = b.size(-2), cols = b.size(-1);
  const uint64_t ld = b.stride(-2);
  const uint64_t gs = three ? static_cast<uint64_t>(b.stride(0)) : rows * ld;
  const uint64_t dims[3] = {cols, rows, groups};
  const uint64_t strides[2] = {ld * 2, gs * 2};
  const uint32_t box[3] = {64, b_mn ? 64u : static_cast<uint32_t>(box_rows), 1};
  return make_tma_desc(b.data_ptr(), 2, 3, dims, strides, box, true);
}

// Destination map for the staged stores of the epilogue: 32 x 32 boxes of 16-bit elements, 64-byte swizzle.
CUtensorMap map_c(const void* base, int64_t cols, int64_t rows, int64_t ld) {
  const uint64_t dims[2] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(rows)};
  const uint64_t strides[1] = {static_cast<uint64_t>(ld) * 2};
  const uint32_t box[2] = {32, 32};
  return make_tma_desc_sw(base, 2, 2, dims, strides, box, 64);
}

bool tma_storable(const void* base, int64_t ld) {
  return reinterpret_cast<uintptr_t>(base) % 16 == 0 && (ld * 2) % 16 == 0;
}

template <int BN, int EPI>
void launch(const CUtensorMap& tA, const CUtensorMap (&tB)[3], const CUtensorMap (&tC)[3], const Args& args, int tiles,
            cudaStream_t stream) {
  using S = gemm::Smem<BN>;
  auto kernel = gemm::gemm_tc_kernel<BN, EPI>;
  static bool configured = false;
  if (!configured) {
    NT_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    configured = true;
  }
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int grid = std::max(1, std::min(tiles, sms));
  kernel<<<grid, gemm::NUM_THREADS, S::TOTAL, stream>>>(tA, tB[0], tB[1], tB[2], tC[0], tC[1], tC[2], args);
  NT_KERNEL_CHECK_AS("gemm_tc_kernel");
}

template <int EPI>
void launch_pair(const CUtensorMap& tA, const CUtensorMap (&tB)[3], const CUtensorMap (&tC)[3], const Args& args, int tiles,
                 cudaStream_t stream) {
  auto kernel = gemm::gemm_tc_pair_kernel<EPI>;
  static bool configured = false;
  if (!configured) {
    NT_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm::PAIR_SMEM));
    configured = true;
  }
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount & ~1;
  const int grid = std::max(2, std::min(2 * tiles, sms));
  kernel<<<grid, gemm::NUM_THREADS, gemm::PAIR_SMEM, stream>>>(tA, tB[0], tB[1], tB[2], tC[0], tC[1], tC[2], args);  // clusters of 2 (compile-time attribute)
  NT_KERNEL_CHECK_AS("gemm_tc_pair_kernel");
}

bool pair_kernels_enabled() {
  static const bool v = [] { const char* e = std::getenv("NT_GEMM_PAIR"); return !(e != nullptr && e[0] == '0'); }();  // NT_GEMM_PAIR=0 turns it off
  return v;
}

// 256-wide tiles move 1.5x fewer bytes per flop through shared memory than 128-wide ones, and
// with ~190 KB of stages in flight the narrow tile is memory-latency bound (measured: 30% vs
// 55% tensor-pipe activity), hence the penalty on BN = 128.
int pick_bn(long long m_tiles, int N, int sms) {
  if (N <= 64) return 64;
  if (N <= 128) return 128;
  double best = 1e30;
  int best_bn = 256;
  for (int bn : {256, 128}) {
    const long long tiles = m_tiles * ((N + bn - 1) / bn);
    const long long waves = (tiles + sms - 1) / sms;
    const double cost = static_cast<double>(waves) * bn * (bn == 128 ? 1.6 : 1.0);
    if (cost < best) { best = cost; best_bn = bn; }
  }
  return best_bn;
}

// out[g][m][n] (+)= sum_s ws[s][g][m][n], parts added in index order; 4 columns per thread.
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, int splits, long long part_elems, int M, int N,
                                     void* c0, void* c1, void* c2, long long ldc, long long c_group_stride,
                                     int c_split_size, int out_f32, int dtype, int accumulate) {
  const long long i4 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i4 >= part_elems) return;
  float4 acc = *reinterpret_cast<const float4*>(ws + i4);
  for (int s = 1; s < splits; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(ws + s * part_elems + i4);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  const long long gm = i4 / N;
  const int n = static_cast<int>(i4 - gm * N);
  const long long g = gm / M, m = gm - g * M;
  void* dst = c0;
  int dn = n;
  if (c_split_size > 0) {
    const int d = n / c_split_size;
    dst = d == 0 ? c0 : (d == 1 ? c1 : c2);
    dn = n - d * c_split_size;
  }
  const long long off = g * c_group_stride + m * ldc + dn;
  if (out_f32) {
    float* p = reinterpret_cast<float*>(dst) + off;
    if (accumulate) { acc.x += p[0]; acc.y += p[1]; acc.z += p[2]; acc.w += p[3]; }
    p[0] = acc.x; p[1] = acc.y; p[2] = acc.z; p[3] = acc.w;
  } else {
    uint16_t* p = reinterpret_cast<uint16_t*>(dst) + off;
    if (accumulate) {
      float a, b;
      gemm::unpack2(*reinterpret_cast<uint32_t*>(p), dtype, a, b); acc.x += a; acc.y += b;
      gemm::unpack2(*reinterpret_cast<uint32_t*>(p + 2), dtype, a, b); acc.z += a; acc.w += b;
    }
    uint2 q;
    q.x = gemm::pack2(acc.x, acc.y, dtype);
    q.y = gemm::pack2(acc.z, acc.w, dtype);
    *reinterpret_cast<uint2*>(p) = q;
  }
}

}  // namespace

StatusWord* device_status_word() {
  static StatusWord* words[64] = {nullptr};
  int dev = 0;
  NT_CUDA_CHECK(cudaGetDevice(&dev));
  if (words[dev] == nullptr) {
    NT_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&words[dev]), sizeof(StatusWord)));
    NT_CUDA_CHECK(cudaMemset(words[dev], 0, sizeof(StatusWord)));
  }
  return words[dev];
}

std::vector<int64_t> read_status(bool clear) {
  StatusWord host;
  StatusWord* dev = device_status_word();
  NT_CUDA_CHECK(cudaDeviceSynchronize());
  NT_CUDA_CHECK(cudaMemcpy(&host, dev, sizeof(host), cudaMemcpyDeviceToHost));
  if (clear) NT_CUDA_CHECK(cudaMemset(dev, 0, sizeof(StatusWord)));
  return {host.code, host.kernel, host.detail, host.count};
}

// The device's status word as a [4] int32 CUDA tensor (code, kernel, detail, count), so that a caller can read
// it with a stream-ordered copy of its own instead of the synchronising `read_status`.
at::Tensor status_word_tensor() {
  int dev = 0;
  NT_CUDA_CHECK(cudaGetDevice(&dev));
  return at::from_blob(device_status_word(), {4}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, dev));
}

// See ops.h for the contract.
void gemm_tc(const at::Tensor& A, bool a_mn, const std::vector<at::Tensor>& Bs, bool b_mn, int64_t b_split,
             const std::vector<at::Tensor>& Cs, int64_t mode, const c10::optional<at::Tensor>& offsets,
             int64_t epilogue, bool accumulate, const c10::optional<at::Tensor>& aux,
             const c10::optional<at::Tensor>& aux_out, int64_t force_bn) {
  c10::cuda::CUDAGuard guard(A.device());
  check_operand(A, "A");
  TORCH_CHECK(A.dim() == 2, "A must be 2-D");
  TORCH_CHECK(!Bs.empty() && Bs.size() <= 3 && !Cs.empty() && Cs.size() <= 3, "1..3 B sources and C destinations");
  const int dt = dtype_code(A);
  for (const auto& b : Bs) {
    check_operand(b, "B");
    TORCH_CHECK(dtype_code(b) == dt, "A and B must share a dtype");
    TORCH_CHECK(b.sizes() == Bs[0].sizes(), "all B sources must have the same shape");
  }
  TORCH_CHECK((b_split == gemm::kBNone) == (Bs.size() == 1), "b_split and the number of B sources disagree");
  TORCH_CHECK(b_split != gemm::kBDual || Bs.size() == 2, "dual-B needs exactly two sources");

  Args args{};
  args.mode = static_cast<int>(mode);
  args.a_mn = a_mn;
  args.b_mn = b_mn;
  args.dtype = dt;
  args.b_split = static_cast<int>(b_split);
  args.accumulate = accumulate;
  args.status = device_status_word();

  const int64_t a_rows = A.size(0), a_cols = A.size(1);
  const int64_t b_n = b_mn ? Bs[0].size(-1) : Bs[0].size(-2);  // per source
  const int64_t b_k = b_mn ? Bs[0].size(-2) : Bs[0].size(-1);
  const int nsrc = static_cast<int>(Bs.size());

  if (mode == gemm::kGroupedK) {
    TORCH_CHECK(a_mn && b_mn, "grouped-K needs MN-major A and B");
    TORCH_CHECK(offsets.has_value(), "grouped modes need offsets");
    TORCH_CHECK(Bs[0].dim() == 2 && Bs.size() == 1 && Bs[0].size(0) == a_rows, "grouped-K: A and B share the segmented rows");
    args.M = static_cast<int>(a_cols);
    args.N = static_cast<int>(b_n);
    args.K = 0;
  } else {
    args.M = static_cast<int>(a_mn ? a_cols : a_rows);
    const int64_t K = a_mn ? a_rows : a_cols;
    args.K = static_cast<int>(K);
    if (b_split == gemm::kBSplitN) {
      args.N = static_cast<int>(b_n * nsrc);
      args.b_split_size = static_cast<int>(b_n);
      TORCH_CHECK(b_k == K, "B reduction extent ", b_k, " != A's ", K);
    } else if (b_split == gemm::kBSplitK) {
      args.N = static_cast<int>(b_n);
      args.b_split_size = static_cast<int>(b_k);
      TORCH_CHECK(b_k * nsrc == K, "sum of B reduction extents != A's K");
      TORCH_CHECK(b_k % gemm::BK == 0, "K-split sources must be multiples of 64 deep");
    } else {
      args.N = static_cast<int>(b_n);
      TORCH_CHECK(b_k == K, "B reduction extent ", b_k, " != A's ", K);
    }
  }
  if (mode != gemm::kDense) {
    TORCH_CHECK(offsets.has_value(), "grouped modes need offsets");
    const auto& off = *offsets;
    TORCH_CHECK(off.is_cuda() && off.scalar_type() == at::kInt && off.is_contiguous(), "offsets must be a contiguous int32 CUDA tensor");
    args.G = static_cast<int>(off.numel() - 1);
    TORCH_CHECK(args.G >= 1 && args.G <= gemm::MAX_GROUPS, "1..", gemm::MAX_GROUPS, " groups supported");
    args.offsets = off.data_ptr<int>();
    if (mode == gemm::kGroupedM) TORCH_CHECK(Bs[0].dim() == 3 && Bs[0].size(0) == args.G, "grouped-M: B must be [G, ., .]");
  } else {
    args.G = 1;
    TORCH_CHECK(Bs[0].dim() == 2, "dense: B must be 2-D");
  }

  // ---- destinations
  const int ndst = static_cast<int>(Cs.size());
  const auto& C0 = Cs[0];
  args.out_f32 = C0.scalar_type() == at::kFloat;
  TORCH_CHECK(args.out_f32 || dtype_code(C0) == dt, "C must be fp32 or the operand dtype");
  for (int i = 0; i < ndst; ++i) {
    TORCH_CHECK(Cs[i].is_cuda() && Cs[i].stride(-1) == 1 && Cs[i].sizes() == C0.sizes() && Cs[i].strides() == C0.strides() &&
                    Cs[i].scalar_type() == C0.scalar_type(), "C destinations must be same-shaped CUDA tensors");
    args.C[i] = Cs[i].data_ptr();
  }
  args.ldc = C0.stride(-2);
  int64_t c_cols_expected = args.N;
  if (epilogue == gemm::kEpiSwigluFwd || epilogue == gemm::kEpiSwigluBwd) c_cols_expected = 2 * args.N;
  if (ndst > 1) {
    TORCH_CHECK(epilogue == gemm::kEpiStore && args.N % ndst == 0, "C split needs the store epilogue and N divisible by the count");
    args.c_split_size = args.N / ndst;
    c_cols_expected = args.c_split_size;
  }
  TORCH_CHECK(C0.size(-1) == c_cols_expected, "C has ", C0.size(-1), " columns, expected ", c_cols_expected);
  if (mode == gemm::kGroupedK) {
    TORCH_CHECK(C0.dim() == 3 && C0.size(0) == args.G && C0.size(1) == args.M, "grouped-K: C must be [G, M, N]");
    args.c_group_stride = C0.stride(0);
  } else {
    TORCH_CHECK(C0.dim() == 2 && C0.size(0) >= args.M, "C must be [M, N]");
  }

  // ---- epilogue extras
  if (epilogue == gemm::kEpiStore) {
    if (aux.has_value()) {
      TORCH_CHECK(mode != gemm::kGroupedK && aux->stride(-1) == 1 && dtype_code(*aux) == dt && aux->size(-1) == args.N, "bad residual");
      args.R = aux->data_ptr();
      args.ldr = aux->stride(-2);
    }
  } else if (epilogue == gemm::kEpiSwigluFwd) {
    TORCH_CHECK(b_split == gemm::kBDual && aux_out.has_value() && !args.out_f32, "SwiGLU forward needs dual B and an H output");
    TORCH_CHECK(aux_out->stride(-1) == 1 && aux_out->size(-1) == args.N && dtype_code(*aux_out) == dt, "bad H output");
    args.C2 = aux_out->data_ptr();
    args.ldc2 = aux_out->stride(-2);
  } else {
    TORCH_CHECK(aux.has_value() && aux->stride(-1) == 1 && aux->size(-1) == 2 * args.N && dtype_code(*aux) == dt && !args.out_f32,
                "SwiGLU backward needs GV [rows, 2N]");
    args.R = aux->data_ptr();
    args.ldr = aux->stride(-2);
  }

  if (args.M == 0 || args.N == 0) return;
  if (mode == gemm::kGroupedK && a_rows == 0) {
    // An empty reduction (an expert that received no token this step): the products are zero.
    // A tensor map cannot describe a tensor without rows, so this case never reaches the kernel.
    if (!accumulate)
      for (const auto& c : Cs) c.zero_();
    return;
  }

  // ---- staged TMA stores of the epilogue (16-bit outputs of the dense and grouped-M shapes)
  CUtensorMap tC[3];
  std::memset(tC, 0, sizeof(tC));
  static const bool staged_ok = [] { const char* e = std::getenv("NT_GEMM_DIRECT_STORE"); return !(e != nullptr && e[0] == '1'); }();
  if (staged_ok && mode != gemm::kGroupedK && !args.out_f32 && tma_storable(C0.data_ptr(), args.ldc)) {
    bool ok = true;
    if (epilogue == gemm::kEpiStore) {
      const int64_t cols = ndst > 1 ? args.c_split_size : args.N;
      for (int i = 0; i < ndst; ++i) ok = ok && tma_storable(Cs[i].data_ptr(), args.ldc);
      ok = ok && (ndst == 1 || args.c_split_size % 32 == 0);
      if (ok)
        for (int i = 0; i < 3; ++i) tC[i] = map_c(Cs[std::min(i, ndst - 1)].data_ptr(), cols, args.M, args.ldc);
    } else {
      ok = args.N % 32 == 0;  // a gate chunk must not run into the value half
      if (ok && epilogue == gemm::kEpiSwigluFwd) ok = tma_storable(args.C2, args.ldc2);
      if (ok) {
        tC[0] = map_c(C0.data_ptr(), 2 * args.N, args.M, args.ldc);
        tC[1] = epilogue == gemm::kEpiSwigluFwd ? map_c(args.C2, args.N, args.M, args.ldc2) : tC[0];
        tC[2] = tC[0];
      }
    }
    args.c_tma = ok ? 1 : 0;
  }
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  int m_tiles;
  if (mode == gemm::kDense) m_tiles = (args.M + gemm::BM - 1) / gemm::BM;
  else if (mode == gemm::kGroupedM) m_tiles = (args.M + gemm::BM - 1) / gemm::BM + args.G;  // upper bound
  else m_tiles = args.G * ((args.M + gemm::BM - 1) / gemm::BM);

  // ---- CTA-pair kernel (256 x 256 tiles, cta_group::2) for the non-ragged-reduction shapes
  const bool pair_ok = mode != gemm::kGroupedK && args.N > 128 && args.M >= 256 && ndst == 1 &&
                       (b_split != gemm::kBSplitN || args.b_split_size % gemm::PAIR_BN == 0);
  // Measured on the training shapes: the pair kernel wins from K = 2048 up (it halves the B traffic
  // per SM), the one-CTA kernel on K = 512 (twice the tiles to balance over the SMs).
  const bool use_pair = force_bn == 512 || (force_bn == 0 && pair_ok && args.K >= 1024 && pair_kernels_enabled());
  if (use_pair) {
    TORCH_CHECK(pair_ok, "gemm_tc: this problem cannot run on the CTA-pair kernel");
    const int pm = mode == gemm::kDense ? (args.M + gemm::PAIR_BM - 1) / gemm::PAIR_BM
                                         : (args.M + gemm::PAIR_BM - 1) / gemm::PAIR_BM + args.G;
    const int ptn = epilogue == gemm::kEpiSwigluFwd ? gemm::PAIR_BN / 2 : gemm::PAIR_BN;
    const int ptiles = pm * ((args.N + ptn - 1) / ptn);
    args.k_splits = 1;
    const CUtensorMap ptA = map_a(A, a_mn);
    CUtensorMap ptB[3];
    for (int i = 0; i < 3; ++i) ptB[i] = map_b(Bs[std::min(i, nsrc - 1)], b_mn, gemm::PAIR_BN / 2);
    cudaStream_t pstream = at::cuda::getCurrentCUDAStream();
    if (epilogue == gemm::kEpiSwigluFwd) launch_pair<gemm::kEpiSwigluFwd>(ptA, ptB, tC, args, ptiles, pstream);
    else if (epilogue == gemm::kEpiSwigluBwd) launch_pair<gemm::kEpiSwigluBwd>(ptA, ptB, tC, args, ptiles, pstream);
    else launch_pair<gemm::kEpiStore>(ptA, ptB, tC, args, ptiles, pstream);
    return;
  }

  int bn = epilogue == gemm::kEpiSwigluFwd ? 256 : pick_bn(m_tiles, args.N, sms);
  if (mode == gemm::kGroupedK && args.N >= 256) bn = 256;  // split-K fills the GPU; keep the wide tile
  if (force_bn > 0) bn = static_cast<int>(force_bn);
  if (force_bn < 0) bn = epilogue == gemm::kEpiSwigluFwd ? 256 : pick_bn(m_tiles, args.N, sms);  // -1: one-CTA kernel, automatic tile
  TORCH_CHECK(bn == 64 || bn == 128 || bn == 256, "BN must be 64, 128 or 256");
  if (b_split == gemm::kBSplitN) {
    while (bn > 64 && args.b_split_size % bn != 0) bn /= 2;
    TORCH_CHECK(args.b_split_size % bn == 0, "N-split sources must be a multiple of the tile width");
  }
  if (ndst > 1) {
    while (bn > 64 && args.c_split_size % bn != 0) bn /= 2;
    TORCH_CHECK(args.c_split_size % 32 == 0, "C split width must be a multiple of 32");
  }
  const int tn = epilogue == gemm::kEpiSwigluFwd ? bn / 2 : bn;
  const int tiles = m_tiles * ((args.N + tn - 1) / tn);

  // ---- split-K (grouped-K only): cut every segment's reduction so the grid fills the GPU
  at::Tensor ws;
  args.k_splits = 1;
  if (mode == gemm::kGroupedK && epilogue == gemm::kEpiStore && args.N % 4 == 0 && C0.stride(-2) % 4 == 0 &&
      (ndst == 1 || args.c_split_size % 4 == 0)) {
    const long long rows_per_group = std::max<long long>(1, a_rows / args.G);
    const long long max_by_depth = std::max<long long>(1, rows_per_group / (8 * gemm::BK));  // >= 8 steps per part
    // two full rounds of work units over the SMs, never a few units into a third round
    long long want = tiles < sms ? std::max<long long>(1, 2LL * sms / tiles) : 1;
    want = std::min<long long>({want, 32, max_by_depth});
    if (want > 1) {
      args.k_splits = static_cast<int>(want);
      ws = at::empty({want, args.G, args.M, args.N}, A.options().dtype(at::kFloat));
      args.ws = ws.data_ptr<float>();
    }
  }
  const int launch_tiles = tiles * args.k_splits;

  const CUtensorMap tA = map_a(A, a_mn);
  CUtensorMap tB[3];
  const int box_rows = b_split == gemm::kBDual ? bn / 2 : bn;
  for (int i = 0; i < 3; ++i) tB[i] = map_b(Bs[std::min(i, nsrc - 1)], b_mn, box_rows);

  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
#define NT_LAUNCH(BN_, EPI_) launch<BN_, EPI_>(tA, tB, tC, args, launch_tiles, stream)
  if (epilogue == gemm::kEpiSwigluFwd) {
    TORCH_CHECK(bn == 256, "SwiGLU forward uses 256-wide tiles");
    NT_LAUNCH(256, gemm::kEpiSwigluFwd);
  } else if (epilogue == gemm::kEpiSwigluBwd) {
    if (bn == 256) NT_LAUNCH(256, gemm::kEpiSwigluBwd);
    else if (bn == 128) NT_LAUNCH(128, gemm::kEpiSwigluBwd);
    else NT_LAUNCH(64, gemm::kEpiSwigluBwd);
  } else {
    if (bn == 256) NT_LAUNCH(256, gemm::kEpiStore);
    else if (bn == 128) NT_LAUNCH(128, gemm::kEpiStore);
    else NT_LAUNCH(64, gemm::kEpiStore);
  }
#undef NT_LAUNCH
  if (args.k_splits > 1) {
    const long long part = static_cast<long long>(args.G) * args.M * args.N;
    const unsigned blocks = static_cast<unsigned>((part / 4 + 255) / 256);
    splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(args.ws, args.k_splits, part, args.M, args.N, args.C[0], args.C[1], args.C[2],
                                                     args.ldc, args.c_group_stride, args.c_split_size, args.out_f32, args.dtype,
                                                     args.accumulate);
    NT_KERNEL_CHECK_AS("splitk_reduce_kernel");
  }
}

}  // namespace nt
