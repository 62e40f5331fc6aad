// RAII CUDA event, move-only (reference: csrc/runtime/cuda_event.h, whose move-assignment
// does not compile; this one does).
#pragma once
#include "cuda_check.h"

namespace nt {

class CudaEvent {
 public:
  explicit CudaEvent(bool timing = true) {
    NT_CUDA_CHECK(cudaEventCreateWithFlags(&event_, timing ? cudaEventDefault : cudaEventDisableTiming));
  }
  ~CudaEvent() {
    if (event_ != nullptr) cudaEventDestroy(event_);
  }
  CudaEvent(const CudaEvent&) = delete;
  CudaEvent& operator=(const CudaEvent&) = delete;
  CudaEvent(CudaEvent&& other) noexcept : event_(other.event_) { other.event_ = nullptr; }
  CudaEvent& operator=(CudaEvent&& other) noexcept {
    if (this != &other) {
      if (event_ != nullptr) cudaEventDestroy(event_);
      event_ = other.event_;
      other.event_ = nullptr;
    }
    return *this;
  }
  void record(cudaStream_t stream) { NT_CUDA_CHECK(cudaEventRecord(event_, stream)); }
  // Make `stream` wait (on the device) until this event has happened.
  void wait(cudaStream_t stream) const { NT_CUDA_CHECK(cudaStreamWaitEvent(stream, event_, 0)); }
  void synchronize() const { NT_CUDA_CHECK(cudaEventSynchronize(event_)); }
  float elapsed_ms_since(const CudaEvent& start) const {
    float ms = 0.f;
    NT_CUDA_CHECK(cudaEventElapsedTime(&ms, start.event_, event_));
    return ms;
  }
  cudaEvent_t get() const { return event_; }

 private:
  cudaEvent_t event_ = nullptr;
};

}  // namespace nt
