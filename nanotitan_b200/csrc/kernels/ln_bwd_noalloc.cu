// See ln_bwd_noalloc.h: LayerNorm backward whose scratch lives in a file-scope device array,
// for callers that cannot allocate.  Self-contained on purpose (CUDA runtime only, no PyTorch).
#include "ln_bwd_noalloc.h"

#include <atomic>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>

namespace {

constexpr int kWarps = 4;                                    // warps per block
constexpr int kPartialRows = NT_LN_NOALLOC_ROWS_OF_PARTIALS;  // one row of partial sums per warp
constexpr int kMaxBlocks = kPartialRows / kWarps;
constexpr int kMaxD = NT_LN_NOALLOC_MAX_D;

// [0 .. kPartialRows*kMaxD): partial dgamma rows, then the same for dbeta.  Part of the library
// image: present on every device that loads it, never freed.
static __device__ __align__(256) float g_scratch[2 * kPartialRows * kMaxD];

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_total(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per row; warp w of block b owns partial row b*kWarps + w, clears it, then adds into it.
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
ln_bwd_rows(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma, const float* __restrict__ mean,
            const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ scratch, long long rows, int d) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = blockIdx.x * kWarps + warp;
  float* pg = scratch + static_cast<long long>(slot) * d;
  float* pb = scratch + static_cast<long long>(kPartialRows) * kMaxD + static_cast<long long>(slot) * d;
  for (int c = lane; c < d; c += 32) { pg[c] = 0.f; pb[c] = 0.f; }
  for (long long row = static_cast<long long>(blockIdx.x) * kWarps + warp; row < rows;
       row += static_cast<long long>(gridDim.x) * kWarps) {
    const T* xr = x + row * d;
    const T* gr = dy + row * d;
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int c = lane; c < d; c += 32) {
      const float xhat = (to_f(xr[c]) - mu) * rs;
      const float g = to_f(gr[c]);
      const float gy = to_f(gamma[c]) * g;
      s1 += gy;
      s2 += gy * xhat;
      pg[c] += g * xhat;  // this lane is the only writer of column c of this partial row
      pb[c] += g;
    }
    s1 = warp_total(s1) / d;
    s2 = warp_total(s2) / d;
    for (int c = lane; c < d; c += 32) {
      const float xhat = (to_f(xr[c]) - mu) * rs;
      dx[row * d + c] = from_f<T>(rs * (to_f(gamma[c]) * to_f(gr[c]) - s1 - xhat * s2));
    }
  }
}

// dgamma[c], dbeta[c] = sum of the partial rows in index order.
__global__ void ln_bwd_fold(const float* __restrict__ scratch, float* __restrict__ dgamma, float* __restrict__ dbeta, int used_rows, int d) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= d) return;
  const float* pg = scratch;
  const float* pb = scratch + static_cast<long long>(kPartialRows) * kMaxD;
  float g = 0.f, b = 0.f;
  for (int r = 0; r < used_rows; ++r) {
    g += pg[static_cast<long long>(r) * d + c];
    b += pb[static_cast<long long>(r) * d + c];
  }
  dgamma[c] = g;
  dbeta[c] = b;
}

int fail(int code, const char* what, char* err, int err_len) {
  if (err != nullptr && err_len > 0) {
    std::strncpy(err, what, static_cast<size_t>(err_len) - 1);
    err[err_len - 1] = '\0';
  }
  return code;
}

// Device address of g_scratch, looked up once per device.  In host code the name `g_scratch` is only
// a handle for the runtime; the address a kernel can use comes from cudaGetSymbolAddress.
// Host threads may make their first calls at the same time: the entries are atomics, and two threads
// that both find an entry empty both look the address up and store the same value.
float* scratch_for_current_device(char* err, int err_len, int* rc) {
  static std::atomic<float*> table[64];  // zero-initialised (static storage)
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    *rc = fail(NT_LN_NOALLOC_CUDA_ERROR, "nt_layer_norm_bwd_noalloc: cudaGetDevice failed", err, err_len);
    return nullptr;
  }
  float* known = table[dev].load(std::memory_order_acquire);
  if (known == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      char msg[160];
      std::snprintf(msg, sizeof(msg), "nt_layer_norm_bwd_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      *rc = fail(NT_LN_NOALLOC_CUDA_ERROR, msg, err, err_len);
      return nullptr;
    }
    table[dev].store(ptr, std::memory_order_release);
    known = ptr;
  }
  return known;
}

template <typename T>
cudaError_t run(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx, float* dgamma,
                float* dbeta, long long rows, int d, float* scratch, cudaStream_t stream) {
  long long want = (rows + kWarps - 1) / kWarps;
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > kMaxBlocks ? kMaxBlocks : want));
  ln_bwd_rows<T><<<blocks, kWarps * 32, 0, stream>>>(static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const T*>(gamma),
                                                     mean, rstd, static_cast<T*>(dx), scratch, rows, d);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  ln_bwd_fold<<<(d + 127) / 128, 128, 0, stream>>>(scratch, dgamma, dbeta, blocks * kWarps, d);
  return cudaGetLastError();
}

}  // namespace

extern "C" int nt_layer_norm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                                         void* dx, float* dgamma, float* dbeta, long long rows, int d, int dtype, void* stream,
                                         char* err, int err_len) {
  if (dy == nullptr || x == nullptr || gamma == nullptr || mean == nullptr || rstd == nullptr || dx == nullptr ||
      dgamma == nullptr || dbeta == nullptr || rows < 0 || d < 1 || dtype < 0 || dtype > 2)
    return fail(NT_LN_NOALLOC_BAD_ARGUMENT, "nt_layer_norm_bwd_noalloc: null pointer, negative row count, d < 1 or unknown dtype", err, err_len);
  if (d > kMaxD) {
    char msg[160];
    std::snprintf(msg, sizeof(msg), "nt_layer_norm_bwd_noalloc: d = %d exceeds the built-in scratch (max d = %d)", d, kMaxD);
    return fail(NT_LN_NOALLOC_TOO_LARGE, msg, err, err_len);
  }
  int rc = NT_LN_NOALLOC_OK;
  float* scratch = scratch_for_current_device(err, err_len, &rc);
  if (scratch == nullptr) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = dtype == 0 ? run<float>(dy, x, gamma, mean, rstd, dx, dgamma, dbeta, rows, d, scratch, s)
                  : dtype == 1 ? run<__half>(dy, x, gamma, mean, rstd, dx, dgamma, dbeta, rows, d, scratch, s)
                               : run<__nv_bfloat16>(dy, x, gamma, mean, rstd, dx, dgamma, dbeta, rows, d, scratch, s);
  if (e != cudaSuccess) {
    char msg[160];
    std::snprintf(msg, sizeof(msg), "nt_layer_norm_bwd_noalloc: kernel launch failed: %s", cudaGetErrorString(e));
    return fail(NT_LN_NOALLOC_CUDA_ERROR, msg, err, err_len);
  }
  return NT_LN_NOALLOC_OK;
}
