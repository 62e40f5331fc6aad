// Vector load/store helpers (16-byte accesses on fp32/fp16/bf16 rows), warp reductions and the
// dtype dispatch macro shared by the memory-bound kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <c10/util/BFloat16.h>
#include <c10/util/Half.h>

#include <cstdint>

namespace nt {

inline bool is_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T>
__device__ __forceinline__ float elem_to_float(T v) { return static_cast<float>(v); }
template <>
__device__ __forceinline__ float elem_to_float<c10::BFloat16>(c10::BFloat16 v) {
  return __uint_as_float(static_cast<uint32_t>(v.x) << 16);
}
template <>
__device__ __forceinline__ float elem_to_float<c10::Half>(c10::Half v) {
  return __half2float(*reinterpret_cast<const __half*>(&v));
}
template <typename T>
__device__ __forceinline__ T float_to_elem(float v) { return static_cast<T>(v); }
template <>
__device__ __forceinline__ c10::BFloat16 float_to_elem<c10::BFloat16>(float v) {
  __nv_bfloat16 b = __float2bfloat16_rn(v);
  c10::BFloat16 out;
  out.x = *reinterpret_cast<uint16_t*>(&b);
  return out;
}
template <>
__device__ __forceinline__ c10::Half float_to_elem<c10::Half>(float v) {
  __half h = __float2half_rn(v);
  c10::Half out;
  out.x = *reinterpret_cast<uint16_t*>(&h);
  return out;
}

// VEC elements starting at p (p must be 16-byte aligned when VEC * sizeof(T) == 16).
template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T* p, float (&out)[VEC]) {
  if constexpr (VEC * sizeof(T) == 16) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < VEC; ++i) out[i] = elem_to_float<T>(e[i]);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) out[i] = elem_to_float<T>(p[i]);
  }
}
// A 16-byte piece kept in its stored form (four registers) until it is needed as floats.
template <typename T, int VEC>
__device__ __forceinline__ void unpack_vec(const uint4& raw, float (&out)[VEC]) {
  static_assert(VEC * sizeof(T) == 16, "unpack_vec is for 16-byte pieces");
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < VEC; ++i) out[i] = elem_to_float<T>(e[i]);
}
template <typename T, int VEC>
__device__ __forceinline__ void store_vec(T* p, const float (&v)[VEC]) {
  if constexpr (VEC * sizeof(T) == 16) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < VEC; ++i) e[i] = float_to_elem<T>(v[i]);
    *reinterpret_cast<uint4*>(p) = raw;
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) p[i] = float_to_elem<T>(v[i]);
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace nt

// fp32 / fp16 / bf16 dispatch; the lambda sees `scalar_t`.
#define NT_DISPATCH_FLOAT(TYPE, NAME, ...)                                        \
  [&] {                                                                           \
    switch (TYPE) {                                                               \
      case at::kFloat: { using scalar_t = float; return __VA_ARGS__(); }          \
      case at::kHalf: { using scalar_t = c10::Half; return __VA_ARGS__(); }       \
      case at::kBFloat16: { using scalar_t = c10::BFloat16; return __VA_ARGS__(); } \
      default: TORCH_CHECK(false, NAME, ": unsupported dtype ", TYPE);            \
    }                                                                             \
  }()
