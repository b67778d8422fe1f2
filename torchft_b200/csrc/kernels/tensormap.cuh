// Host-side creation (and caching) of TMA tensor maps.  The driver entry point is
// resolved at run time so that the library links without libcuda on build machines.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <stdint.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <unordered_map>

namespace tft {

struct TmapKey {
  const void* ptr;
  uint64_t d0, d1, d2, s1, s2;
  uint32_t b0, b1, b2, esize, swizzle;
  bool operator==(const TmapKey& o) const { return std::memcmp(this, &o, sizeof(TmapKey)) == 0; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    const uint64_t* p = reinterpret_cast<const uint64_t*>(&k);
    size_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(TmapKey) / 8; ++i) h = (h ^ p[i]) * 1099511628211ull;
    return h;
  }
};

inline PFN_cuTensorMapEncodeTiled_v12000 tensormap_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }();
  return fn;
}

// Up to rank 3, innermost dimension first.  Strides in bytes (s1 for dim1, s2 for dim2).
// Returns false on failure.  swizzle: 0 = none, 1 = 128 B.
inline bool make_tensormap(CUtensorMap* out, const void* ptr, int rank, uint32_t esize,
                           uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2,
                           uint32_t b0, uint32_t b1, uint32_t b2, uint32_t swizzle) {
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  TmapKey key;
  std::memset(&key, 0, sizeof(key));
  key.ptr = ptr; key.d0 = d0; key.d1 = d1; key.d2 = d2; key.s1 = s1; key.s2 = s2;
  key.b0 = b0; key.b1 = b1; key.b2 = b2; key.esize = esize | (rank << 8); key.swizzle = swizzle;
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
  }
  auto fn = tensormap_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1, s2};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt = esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                         : esize == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                      : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  // The encoder is a driver call and needs a current context.  Threads that only ever
  // used the runtime API lazily (autograd worker threads, for one) may not have bound the
  // primary context yet; a no-op runtime call binds it.  Once per thread: the call is not allowed
  // while a stream capture is in progress, and after the first time it has nothing left to do.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  CUresult r = fn(out, dt, rank, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    std::fprintf(stderr,
                 "torchft_b200: cuTensorMapEncodeTiled failed (%d): ptr=%p rank=%d esize=%u dims=(%llu,%llu,%llu) "
                 "strides=(%llu,%llu) box=(%u,%u,%u)\n",
                 static_cast<int>(r), ptr, rank, esize, (unsigned long long)d0, (unsigned long long)d1,
                 (unsigned long long)d2, (unsigned long long)s1, (unsigned long long)s2, b0, b1, b2);
    return false;
  }
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return true;
}

}  // namespace tft
