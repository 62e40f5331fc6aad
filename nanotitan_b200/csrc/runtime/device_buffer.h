// RAII device allocation, move-only (reference: csrc/runtime/device_buffer.h).
#pragma once
#include <cstddef>
#include <utility>

#include "cuda_check.h"

namespace nt {

template <typename T>
class DeviceBuffer {
 public:
  DeviceBuffer() = default;
  explicit DeviceBuffer(std::size_t count) : size_(count) {
    if (count > 0) NT_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&data_), count * sizeof(T)));
  }
  ~DeviceBuffer() { release(); }
  DeviceBuffer(const DeviceBuffer&) = delete;
  DeviceBuffer& operator=(const DeviceBuffer&) = delete;
  DeviceBuffer(DeviceBuffer&& other) noexcept
      : data_(std::exchange(other.data_, nullptr)), size_(std::exchange(other.size_, 0)) {}
  DeviceBuffer& operator=(DeviceBuffer&& other) noexcept {
    if (this != &other) {
      release();
      data_ = std::exchange(other.data_, nullptr);
      size_ = std::exchange(other.size_, 0);
    }
    return *this;
  }
  T* data() { return data_; }
  const T* data() const { return data_; }
  std::size_t size() const { return size_; }
  std::size_t bytes() const { return size_ * sizeof(T); }
  void zero(cudaStream_t stream = nullptr) {
    if (data_ != nullptr) NT_CUDA_CHECK(cudaMemsetAsync(data_, 0, bytes(), stream));
  }

 private:
  void release() {
    if (data_ != nullptr) cudaFree(data_);
    data_ = nullptr;
    size_ = 0;
  }
  T* data_ = nullptr;
  std::size_t size_ = 0;
};

}  // namespace nt
