// Error checks that throw with file:line, and the process-wide kernel-launch counter.
// (Role of the reference's csrc/runtime/cuda_check.h:1-21.)
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <sstream>
#include <stdexcept>
#include <string>

namespace nt {

inline void cuda_check(cudaError_t err, const char* expr, const char* file, int line) {
  if (err == cudaSuccess) return;
  std::ostringstream os;
  os << "CUDA error " << static_cast<int>(err) << " (" << cudaGetErrorString(err) << ") at " << file
     << ":" << line << " in `" << expr << "`";
  throw std::runtime_error(os.str());
}

// Number of kernels of this library launched by this process (benchmarks report it).
inline std::atomic<long long>& launch_counter() {
  static std::atomic<long long> counter{0};
  return counter;
}

}  // namespace nt

#define NT_CUDA_CHECK(expr) ::nt::cuda_check((expr), #expr, __FILE__, __LINE__)
// After a <<<>>> launch: surfaces launch-configuration errors and counts the launch.
#define NT_KERNEL_CHECK()                                  \
  do {                                                     \
    ::nt::launch_counter().fetch_add(1);                   \
    NT_CUDA_CHECK(cudaGetLastError());                     \
  } while (0)
// Names kept for code written against the reference's macros.
#define CUDA_CHECK(expr) NT_CUDA_CHECK(expr)
#define CUDA_KERNEL_CHECK() NT_KERNEL_CHECK()
