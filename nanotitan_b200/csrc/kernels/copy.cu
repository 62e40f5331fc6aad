// Bandwidth microbenchmark kernels: element-wise copy, 16-byte vector copy and a peer copy
// (reference: csrc/kernels/copy_kernel.cu).  Unlike the reference they run on the current
// stream under a device guard, the vector copy handles a ragged tail, and the peer copy is
// bound to Python.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <ATen/ATen.h>

#include "cuda_check.h"
#include "ops.h"

namespace nt {

namespace {

template <typename T>
__global__ void copy_scalar_kernel(const T* __restrict__ src, T* __restrict__ dst, long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}

__global__ void copy_vector_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n_vec,
                                   const uint8_t* __restrict__ src_tail, uint8_t* __restrict__ dst_tail, int tail) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
  if (blockIdx.x == 0 && threadIdx.x < tail) dst_tail[threadIdx.x] = src_tail[threadIdx.x];
}

// dst[i] = src[i] for the first rows[0] rows only; the row count lives on the device, so the host
// launches without knowing it (rows past the count keep whatever dst held).
__global__ void copy_rows_prefix_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const int* __restrict__ rows,
                                        long long max_rows, long long vec_per_row) {
  const long long n = min(static_cast<long long>(rows[0]), max_rows) * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}

int copy_grid(long long work_items) {
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return static_cast<int>(std::max<long long>(1, std::min<long long>((work_items + 255) / 256, 16LL * sms)));
}

}  // namespace

void copy_scalar(const at::Tensor& src, at::Tensor dst, int64_t n) {
  TORCH_CHECK(src.is_cuda() && dst.is_cuda() && src.is_contiguous() && dst.is_contiguous(), "copy_scalar: contiguous CUDA tensors");
  TORCH_CHECK(src.scalar_type() == dst.scalar_type() && n <= src.numel() && n <= dst.numel(), "copy_scalar: dtype / length mismatch");
  c10::cuda::CUDAGuard guard(src.device());
  if (n == 0) return;
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const int grid = copy_grid(n);
  switch (src.element_size()) {
    case 1: copy_scalar_kernel<uint8_t><<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(src.data_ptr()), static_cast<uint8_t*>(dst.data_ptr()), n); break;
    case 2: copy_scalar_kernel<uint16_t><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(src.data_ptr()), static_cast<uint16_t*>(dst.data_ptr()), n); break;
    case 4: copy_scalar_kernel<uint32_t><<<grid, 256, 0, stream>>>(static_cast<const uint32_t*>(src.data_ptr()), static_cast<uint32_t*>(dst.data_ptr()), n); break;
    case 8: copy_scalar_kernel<uint64_t><<<grid, 256, 0, stream>>>(static_cast<const uint64_t*>(src.data_ptr()), static_cast<uint64_t*>(dst.data_ptr()), n); break;
    default: TORCH_CHECK(false, "copy_scalar: unsupported element size");
  }
  NT_KERNEL_CHECK();
}

void copy_vector(const at::Tensor& src, at::Tensor dst) {
  TORCH_CHECK(src.is_cuda() && dst.is_cuda() && src.is_contiguous() && dst.is_contiguous(), "copy_vector: contiguous CUDA tensors");
  TORCH_CHECK(src.nbytes() == dst.nbytes(), "copy_vector: byte size mismatch");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(src.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(dst.data_ptr()) % 16 == 0, "copy_vector: 16-byte aligned buffers");
  c10::cuda::CUDAGuard guard(src.device());
  const long long bytes = src.nbytes();
  if (bytes == 0) return;
  const long long n_vec = bytes / 16;
  const int tail = static_cast<int>(bytes % 16);
  const auto* s = static_cast<const uint8_t*>(src.data_ptr());
  auto* d = static_cast<uint8_t*>(dst.data_ptr());
  copy_vector_kernel<<<copy_grid(n_vec), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const uint4*>(s), reinterpret_cast<uint4*>(d), n_vec, s + n_vec * 16, d + n_vec * 16, tail);
  NT_KERNEL_CHECK();
}

// First `rows[0]` rows of src [R, d] -> dst [>= R', d] (rows: int32 CUDA tensor with one element; rows of 16-byte multiples).
void copy_rows_prefix(const at::Tensor& src, at::Tensor dst, const at::Tensor& rows) {
  TORCH_CHECK(src.is_cuda() && dst.is_cuda() && src.dim() == 2 && dst.dim() == 2 && src.is_contiguous() && dst.is_contiguous() &&
                  src.size(1) == dst.size(1) && src.scalar_type() == dst.scalar_type(), "copy_rows_prefix: contiguous [rows, d] CUDA tensors");
  TORCH_CHECK(rows.is_cuda() && rows.scalar_type() == at::kInt && rows.numel() == 1, "copy_rows_prefix: rows must be one int32 on the device");
  const long long row_bytes = src.size(1) * src.element_size();
  TORCH_CHECK(row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(src.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(dst.data_ptr()) % 16 == 0,
              "copy_rows_prefix: 16-byte aligned rows");
  c10::cuda::CUDAGuard guard(src.device());
  const long long max_rows = std::min<long long>(src.size(0), dst.size(0));
  if (max_rows == 0 || row_bytes == 0) return;
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  copy_rows_prefix_kernel<<<8 * sms, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      static_cast<const uint4*>(src.data_ptr()), static_cast<uint4*>(dst.data_ptr()), rows.data_ptr<int>(), max_rows, row_bytes / 16);
  NT_KERNEL_CHECK();
}

// Device-to-device copy between two GPUs over NVLink, ordered on the destination's current stream.
void peer_copy_scalar(const at::Tensor& src, at::Tensor dst) {
  TORCH_CHECK(src.is_cuda() && dst.is_cuda() && src.is_contiguous() && dst.is_contiguous() && src.nbytes() == dst.nbytes(), "peer_copy_scalar: contiguous CUDA tensors of equal size");
  c10::cuda::CUDAGuard guard(dst.device());
  NT_CUDA_CHECK(cudaMemcpyPeerAsync(dst.data_ptr(), dst.get_device(), src.data_ptr(), src.get_device(), src.nbytes(),
                                    at::cuda::getCurrentCUDAStream()));
}

// Toy op of the reference's API: a zero vector of length x with t's options (csrc/random.cpp).
at::Tensor random_op(const at::Tensor& t, int64_t x) { return at::zeros({x}, t.options()); }

}  // namespace nt
