// Host-side builder (with a small cache) for TMA tensor maps over bf16/fp16/fp32 tensors.
// The driver entry point is resolved at run time, so the library links without libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <array>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>

#include "cuda_check.h"

namespace nt {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    NT_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res));
    if (ptr == nullptr || res != cudaDriverEntryPointSuccess)
      throw std::runtime_error("cuTensorMapEncodeTiled is not available in this driver");
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

struct TmaKey {
  const void* base;
  uint32_t rank, elem_bytes, swizzle;
  std::array<uint64_t, 4> dims;
  std::array<uint64_t, 3> strides;  // bytes, for dims 1..3
  std::array<uint32_t, 4> box;
  bool operator==(const TmaKey& o) const { return std::memcmp(this, &o, sizeof(TmaKey)) == 0; }
};
struct TmaKeyHash {
  size_t operator()(const TmaKey& k) const {
    const auto* p = reinterpret_cast<const uint64_t*>(&k);
    size_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(TmaKey) / 8; ++i) h = (h ^ p[i]) * 1099511628211ull;
    return h;
  }
};

// dims / box are innermost-first.  strides_bytes[i] is the byte stride of dim i+1.
// Rules checked here (the hardware faults on the ones nothing else checks): base 16-byte
// aligned, strides multiples of 16 bytes, inner box extent * elem size <= swizzle span.
// swizzle_bytes: 0 (none), 64 or 128.
inline CUtensorMap make_tma_desc_sw(const void* base, int elem_bytes, int rank, const uint64_t* dims,
                                    const uint64_t* strides_bytes, const uint32_t* box, int swizzle_bytes) {
  static std::mutex mu;
  static std::unordered_map<TmaKey, CUtensorMap, TmaKeyHash> cache;
  TmaKey key;
  std::memset(&key, 0, sizeof(key));
  key.base = base;
  key.rank = rank;
  key.elem_bytes = elem_bytes;
  key.swizzle = swizzle_bytes;
  for (int i = 0; i < rank; ++i) {
    key.dims[i] = dims[i];
    key.box[i] = box[i];
    if (i > 0) key.strides[i - 1] = strides_bytes[i - 1];
  }
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
  }
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) throw std::runtime_error("TMA: base address not 16-byte aligned");
  for (int i = 0; i + 1 < rank; ++i)
    if (strides_bytes[i] % 16 != 0) throw std::runtime_error("TMA: global stride not a multiple of 16 bytes");
  if (swizzle_bytes && static_cast<int>(box[0]) * elem_bytes > swizzle_bytes) throw std::runtime_error("TMA: inner box exceeds the swizzle span");
  // The encoder is a driver call: make sure this thread (e.g. an autograd worker) has the
  // device's primary context bound before calling it.
  // Once per thread: the call is not allowed while a stream capture is open, and warm-up steps
  // have made it on every thread that launches kernels by then.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    NT_CUDA_CHECK(cudaFree(nullptr));
    context_bound = true;
  }
  if ((box[0] * elem_bytes) % 16 != 0) throw std::runtime_error("TMA: inner box extent not a multiple of 16 bytes");
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  cuuint64_t gdims[4] = {1, 1, 1, 1};
  cuuint64_t gstrides[3] = {0, 0, 0};
  cuuint32_t gbox[4] = {1, 1, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    if (i > 0) gstrides[i - 1] = strides_bytes[i - 1];
  }
  CUtensorMap map;
  CUresult rc = encode_tiled_fn()(&map, dt, rank, const_cast<void*>(base), gdims, gstrides, gbox, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                                  swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE),
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(rc)));
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, map);
  return map;
}

inline CUtensorMap make_tma_desc(const void* base, int elem_bytes, int rank, const uint64_t* dims,
                                 const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128) {
  return make_tma_desc_sw(base, elem_bytes, rank, dims, strides_bytes, box, swizzle128 ? 128 : 0);
}

// 4-D map over 2-byte elements (attention tensors [B, S, H, Dh] seen innermost-first).
inline CUtensorMap make_tma_desc4(const void* base, const uint64_t* dims, const uint64_t* strides_bytes,
                                  const uint32_t* box, int swizzle_bytes) {
  return make_tma_desc_sw(base, 2, 4, dims, strides_bytes, box, swizzle_bytes);
}

}  // namespace nt
