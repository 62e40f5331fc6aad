// CUDA-core GEMMs: the `gemm_kernel(A, B, implementation)` learning kernels of the reference's
// API (csrc/kernels/gemm.cu) and the strided, segment-aware fallback used by the grouped-GEMM
// entry points for dtypes / shapes the tensor-core path does not take (fp32, fp64, rows whose
// byte stride is not a multiple of 16).  fp32 accumulation (fp64 for doubles).
#include <ATen/Dispatch.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <ATen/ATen.h>

#include "cuda_check.h"
#include "ops.h"

namespace nt {

namespace {

constexpr int TS = 32;

template <typename T> struct AccT { using type = float; };
template <> struct AccT<double> { using type = double; };

// C(m, n) = sum_k A(m, k) * B(k, n) with arbitrary element strides; blockIdx.z selects a segment:
//   seg_mode 0: one problem.
//   seg_mode 1: rows [off[z], off[z+1]) of A and C, B advanced by z * b_seg.
//   seg_mode 2: reduction rows [off[z], off[z+1]) of A and B, C advanced by z * c_seg.
template <typename T, bool TILED>
__global__ void simt_gemm_kernel(const T* __restrict__ A, long long a_m, long long a_k, const T* __restrict__ B, long long b_k,
                                 long long b_n, T* __restrict__ C, long long c_m, long long c_n, int M, int N, int K,
                                 const int* __restrict__ off, int seg_mode, long long b_seg, long long c_seg) {
  using Acc = typename AccT<T>::type;
  int m_lo = 0, m_hi = M, k_lo = 0, k_hi = K;
  if (seg_mode == 1) { m_lo = off[blockIdx.z]; m_hi = off[blockIdx.z + 1]; B += blockIdx.z * b_seg; }
  if (seg_mode == 2) { k_lo = off[blockIdx.z]; k_hi = off[blockIdx.z + 1]; C += blockIdx.z * c_seg; }
  const int row = m_lo + blockIdx.y * TS + threadIdx.y;
  const int col = blockIdx.x * TS + threadIdx.x;
  if (m_lo + static_cast<int>(blockIdx.y) * TS >= m_hi) return;  // whole tile past the segment (uniform)
  Acc acc = 0;
  if constexpr (TILED) {
    __shared__ T sa[TS][TS + 1];
    __shared__ T sb[TS][TS + 1];
    for (int k0 = k_lo; k0 < k_hi; k0 += TS) {
      const int ka = k0 + threadIdx.x, kb = k0 + threadIdx.y;
      sa[threadIdx.y][threadIdx.x] = (row < m_hi && ka < k_hi) ? A[row * a_m + ka * a_k] : T(0);
      sb[threadIdx.y][threadIdx.x] = (kb < k_hi && col < N) ? B[kb * b_k + col * b_n] : T(0);
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < TS; ++kk) acc += static_cast<Acc>(sa[threadIdx.y][kk]) * static_cast<Acc>(sb[kk][threadIdx.x]);
      __syncthreads();
    }
  } else {
    if (row < m_hi && col < N)
      for (int k = k_lo; k < k_hi; ++k) acc += static_cast<Acc>(A[row * a_m + k * a_k]) * static_cast<Acc>(B[k * b_k + col * b_n]);
  }
  if (row < m_hi && col < N) C[row * c_m + col * c_n] = static_cast<T>(acc);
}

template <bool TILED>
void run_simt(const at::Tensor& A, long long a_m, long long a_k, const at::Tensor& B, long long b_k, long long b_n, at::Tensor& C,
              long long c_m, long long c_n, int M, int N, int K, const int* off, int seg_mode, int segments, int max_rows,
              long long b_seg, long long c_seg) {
  if (N == 0 || max_rows == 0) return;
  dim3 block(TS, TS), grid((N + TS - 1) / TS, (max_rows + TS - 1) / TS, segments);
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  AT_DISPATCH_FLOATING_TYPES_AND2(at::kHalf, at::kBFloat16, A.scalar_type(), "simt_gemm", [&] {
    simt_gemm_kernel<scalar_t, TILED><<<grid, block, 0, stream>>>(A.data_ptr<scalar_t>(), a_m, a_k, B.data_ptr<scalar_t>(), b_k, b_n,
        C.data_ptr<scalar_t>(), c_m, c_n, M, N, K, off, seg_mode, b_seg, c_seg);
  });
  NT_KERNEL_CHECK();
}

void check_gemm_inputs(const at::Tensor& A, const at::Tensor& B) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda(), "A and B must be CUDA tensors");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2, "A and B must be 2-D");
  TORCH_CHECK(A.size(1) == B.size(0), "inner dimensions must match: A is ", A.sizes(), ", B is ", B.sizes());
  TORCH_CHECK(A.scalar_type() == B.scalar_type(), "A and B must have the same dtype");
  TORCH_CHECK(A.device() == B.device(), "A and B must be on the same device");
}

}  // namespace

at::Tensor tiled_gemm_kernel(const at::Tensor& A, const at::Tensor& B) {
  check_gemm_inputs(A, B);
  c10::cuda::CUDAGuard guard(A.device());
  auto C = at::empty({A.size(0), B.size(1)}, A.options());
  const int M = A.size(0), N = B.size(1), K = A.size(1);
  run_simt<true>(A, A.stride(0), A.stride(1), B, B.stride(0), B.stride(1), C, C.stride(0), 1, M, N, K, nullptr, 0, 1, M, 0, 0);
  return C;
}

at::Tensor naive_gemm_kernel(const at::Tensor& A, const at::Tensor& B) {
  check_gemm_inputs(A, B);
  c10::cuda::CUDAGuard guard(A.device());
  auto C = at::empty({A.size(0), B.size(1)}, A.options());
  const int M = A.size(0), N = B.size(1), K = A.size(1);
  run_simt<false>(A, A.stride(0), A.stride(1), B, B.stride(0), B.stride(1), C, C.stride(0), 1, M, N, K, nullptr, 0, 1, M, 0, 0);
  return C;
}

at::Tensor gemm_kernel(const at::Tensor& A, const at::Tensor& B, const std::string& implementation) {
  if (implementation == "tiled") return tiled_gemm_kernel(A, B);
  if (implementation == "naive") return naive_gemm_kernel(A, B);
  TORCH_CHECK(false, "implementation must be either 'tiled' or 'naive'");
}

// Segment-aware fallbacks.  `max_rows`: an upper bound of the longest segment (grid sizing only).
at::Tensor simt_grouped_fwd(const at::Tensor& X, const at::Tensor& off, const at::Tensor& W) {  // [A,K] x [E,K,N] -> [A,N]
  c10::cuda::CUDAGuard guard(X.device());
  auto out = at::zeros({X.size(0), W.size(2)}, X.options());
  const int E = W.size(0);
  run_simt<true>(X, X.stride(0), X.stride(1), W, W.stride(1), W.stride(2), out, out.stride(0), 1, X.size(0), W.size(2), X.size(1),
                 off.data_ptr<int>(), 1, E, X.size(0), W.stride(0), 0);
  return out;
}
at::Tensor simt_grouped_dx(const at::Tensor& W, const at::Tensor& off, const at::Tensor& dOut) {  // dX = dOut . W[e]^T
  c10::cuda::CUDAGuard guard(dOut.device());
  auto dX = at::zeros({dOut.size(0), W.size(1)}, dOut.options());
  const int E = W.size(0);
  // B(k = n index, n = K index) = W[e][K index][n index]
  run_simt<true>(dOut, dOut.stride(0), dOut.stride(1), W, W.stride(2), W.stride(1), dX, dX.stride(0), 1, dOut.size(0), W.size(1), W.size(2),
                 off.data_ptr<int>(), 1, E, dOut.size(0), W.stride(0), 0);
  return dX;
}
at::Tensor simt_grouped_dw(const at::Tensor& X, const at::Tensor& off, const at::Tensor& dOut) {  // dW[e] = X_e^T . dOut_e
  c10::cuda::CUDAGuard guard(X.device());
  const int E = off.numel() - 1;
  auto dW = at::zeros({E, X.size(1), dOut.size(1)}, X.options());
  // A(m = K index, k = row) = X[row][K index]
  run_simt<true>(X, X.stride(1), X.stride(0), dOut, dOut.stride(0), dOut.stride(1), dW, dW.stride(1), 1, X.size(1), dOut.size(1), X.size(0),
                 off.data_ptr<int>(), 2, E, X.size(1), 0, dW.stride(0));
  return dW;
}

}  // namespace nt
