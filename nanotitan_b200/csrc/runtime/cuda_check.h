// Error checks that throw with file:line, and the process-wide kernel-launch counter.
// (Role of the reference's csrc/runtime/cuda_check.h:1-21.)
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <map>
#include <mutex>
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

// Per-host-entry-point launch counters ("bucket_allreduce", "gemm_tc", ...): benchmarks print them
// so that a run shows which of this library's kernels it actually used.
struct LaunchSites {
  std::mutex mu;
  std::map<std::string, std::atomic<long long>*> by_name;
  std::atomic<long long>& at(const char* func) {
    std::lock_guard<std::mutex> lock(mu);
    auto it = by_name.find(func);
    if (it == by_name.end()) it = by_name.emplace(func, new std::atomic<long long>(0)).first;
    return *it->second;
  }
  std::map<std::string, long long> snapshot() {
    std::lock_guard<std::mutex> lock(mu);
    std::map<std::string, long long> out;
    for (auto& kv : by_name) out[kv.first] = kv.second->load();
    return out;
  }
};
inline LaunchSites& launch_sites() {
  static LaunchSites sites;
  return sites;
}

}  // namespace nt

#define NT_CUDA_CHECK(expr) ::nt::cuda_check((expr), #expr, __FILE__, __LINE__)
// After a <<<>>> launch: surfaces launch-configuration errors and counts the launch.
#define NT_KERNEL_CHECK()                                  \
  do {                                                     \
    static std::atomic<long long>& nt_site_ = ::nt::launch_sites().at(__func__); \
    nt_site_.fetch_add(1);                                 \
    ::nt::launch_counter().fetch_add(1);                   \
    NT_CUDA_CHECK(cudaGetLastError());                     \
  } while (0)
// Same, filed under an explicit name (for launches made from helper templates or lambdas).
#define NT_KERNEL_CHECK_AS(NAME)                           \
  do {                                                     \
    static std::atomic<long long>& nt_site_ = ::nt::launch_sites().at(NAME); \
    nt_site_.fetch_add(1);                                 \
    ::nt::launch_counter().fetch_add(1);                   \
    NT_CUDA_CHECK(cudaGetLastError());                     \
  } while (0)
// Names kept for code written against the reference's macros.
#define CUDA_CHECK(expr) NT_CUDA_CHECK(expr)
#define CUDA_KERNEL_CHECK() NT_KERNEL_CHECK()
