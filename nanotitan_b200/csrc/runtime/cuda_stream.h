// RAII CUDA stream (reference: csrc/runtime/cuda_stream.{h,cpp}); header-only and move-enabled.
#pragma once
#include "cuda_check.h"

namespace nt {

class CudaStream {
 public:
  explicit CudaStream(unsigned flags = cudaStreamNonBlocking, int priority = 0) {
    NT_CUDA_CHECK(cudaStreamCreateWithPriority(&stream_, flags, priority));
  }
  ~CudaStream() {
    if (stream_ != nullptr) cudaStreamDestroy(stream_);
  }
  CudaStream(const CudaStream&) = delete;
  CudaStream& operator=(const CudaStream&) = delete;
  CudaStream(CudaStream&& other) noexcept : stream_(other.stream_) { other.stream_ = nullptr; }
  CudaStream& operator=(CudaStream&& other) noexcept {
    if (this != &other) {
      if (stream_ != nullptr) cudaStreamDestroy(stream_);
      stream_ = other.stream_;
      other.stream_ = nullptr;
    }
    return *this;
  }
  cudaStream_t get() const { return stream_; }
  void synchronize() const { NT_CUDA_CHECK(cudaStreamSynchronize(stream_)); }

 private:
  cudaStream_t stream_ = nullptr;
};

}  // namespace nt
