// Grouped-GEMM entry points with the reference's signatures (csrc/bindings.cpp:43-57 there).
// bf16 / fp16 problems whose rows are 16-byte aligned run on the tcgen05 kernel; everything
// else (fp32, fp64, odd widths) runs on the CUDA-core fallback.  Neither path reads the offsets
// on the host: the reference's wrappers do 2*E blocking device-to-host reads per call
// (csrc/kernels/grouped_gemm.cu:58-62).
#include <c10/cuda/CUDAGuard.h>
#include <ATen/ATen.h>

#include "gemm_tc.cuh"
#include "ops.h"

namespace nt {

namespace {

bool tc_ok(const at::Tensor& t) {
  return (t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kHalf) && t.stride(-1) == 1 && t.stride(-2) % 8 == 0 &&
         reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0 && (t.dim() < 3 || t.stride(0) % 8 == 0) && t.size(-1) % 8 == 0;
}

at::Tensor offsets_i32(const at::Tensor& offset) {
  TORCH_CHECK(offset.is_cuda(), "expert offsets must live on the GPU");
  return offset.to(at::kInt).contiguous();
}

void check_common(const at::Tensor& a, const at::Tensor& b, const at::Tensor& offset, const char* name) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda(), name, ": CUDA tensors expected");
  TORCH_CHECK(a.scalar_type() == b.scalar_type(), name, ": operands must share a dtype");
  TORCH_CHECK(offset.dim() == 1 && offset.numel() >= 2, name, ": offsets must be a 1-D tensor of E+1 entries");
}

}  // namespace

at::Tensor grouped_gemm_kernel(const at::Tensor& X, const at::Tensor& offset, const at::Tensor& W) {
  check_common(X, W, offset, "grouped_gemm_kernel");
  TORCH_CHECK(X.dim() == 2 && W.dim() == 3 && X.size(1) == W.size(1) && offset.numel() == W.size(0) + 1, "grouped_gemm_kernel: X [A,K], W [E,K,N], offsets [E+1]");
  auto off = offsets_i32(offset);
  auto Xc = X.contiguous();
  auto Wc = W.contiguous();
  if (tc_ok(Xc) && tc_ok(Wc) && W.size(0) <= gemm::MAX_GROUPS) {
    // rows past offsets[E] (none in normal use) stay zero
    auto out = at::zeros({X.size(0), W.size(2)}, X.options());
    gemm_tc(Xc, false, {Wc}, true, gemm::kBNone, {out}, gemm::kGroupedM, off, gemm::kEpiStore, false, c10::nullopt, c10::nullopt, 0);
    return out;
  }
  return simt_grouped_fwd(Xc, off, Wc);
}

at::Tensor bwd_grouped_gemm_dX_kernel(const at::Tensor& W, const at::Tensor& offset, const at::Tensor& dOut) {
  check_common(dOut, W, offset, "bwd_grouped_gemm_dX_kernel");
  TORCH_CHECK(dOut.dim() == 2 && W.dim() == 3 && dOut.size(1) == W.size(2) && offset.numel() == W.size(0) + 1, "bwd_grouped_gemm_dX_kernel: W [E,K,N], dOut [A,N]");
  auto off = offsets_i32(offset);
  auto G = dOut.contiguous();
  auto Wc = W.contiguous();
  if (tc_ok(G) && tc_ok(Wc) && W.size(0) <= gemm::MAX_GROUPS) {
    auto dX = at::zeros({dOut.size(0), W.size(1)}, dOut.options());
    // W[e] is [K, N] with N contiguous: as the B operand of dX = dOut . W[e]^T it is K-major
    gemm_tc(G, false, {Wc}, false, gemm::kBNone, {dX}, gemm::kGroupedM, off, gemm::kEpiStore, false, c10::nullopt, c10::nullopt, 0);
    return dX;
  }
  return simt_grouped_dx(Wc, off, G);
}

at::Tensor bwd_grouped_gemm_dW_kernel(const at::Tensor& X, const at::Tensor& offset, const at::Tensor& dOut) {
  check_common(X, dOut, offset, "bwd_grouped_gemm_dW_kernel");
  TORCH_CHECK(X.dim() == 2 && dOut.dim() == 2 && X.size(0) == dOut.size(0), "bwd_grouped_gemm_dW_kernel: X [A,K], dOut [A,N]");
  auto off = offsets_i32(offset);
  auto Xc = X.contiguous();
  auto G = dOut.contiguous();
  const int64_t E = offset.numel() - 1;
  if (tc_ok(Xc) && tc_ok(G) && E <= gemm::MAX_GROUPS) {
    auto dW = at::empty({E, X.size(1), dOut.size(1)}, X.options());
    gemm_tc(Xc, true, {G}, true, gemm::kBNone, {dW}, gemm::kGroupedK, off, gemm::kEpiStore, false, c10::nullopt, c10::nullopt, 0);
    return dW;
  }
  return simt_grouped_dw(Xc, off, G);
}

}  // namespace nt
