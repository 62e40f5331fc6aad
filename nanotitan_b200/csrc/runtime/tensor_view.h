// Strided 2-D view usable on host and device (reference: csrc/runtime/tensor_view.h).
#pragma once
#include <cstdint>

namespace nt {

template <typename T>
struct Tensor2D {
  T* data;
  int64_t rows, cols;
  int64_t row_stride, col_stride;

  __host__ __device__ Tensor2D(T* p, int64_t r, int64_t c, int64_t rs, int64_t cs = 1)
      : data(p), rows(r), cols(c), row_stride(rs), col_stride(cs) {}
  __host__ __device__ T& operator()(int64_t i, int64_t j) const {
    return data[i * row_stride + j * col_stride];
  }
  __host__ __device__ bool in_bounds(int64_t i, int64_t j) const {
    return i >= 0 && i < rows && j >= 0 && j < cols;
  }
};

}  // namespace nt
