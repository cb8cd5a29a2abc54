// Host-side helpers: status codes of the C ABI, launch checks, and TMA tensor-map
// encoding through the driver entry point (so the library does not link libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <unordered_map>
#include <unordered_set>

#include "../../include/b200pair.h"

namespace b200 {

inline thread_local char g_last_error[512] = "";

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

#define B200_CHECK_ARG(cond, ...) \
  do {                            \
    if (!(cond)) return ::b200::fail(B200_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)

#define B200_CUDA(call)                                                                                     \
  do {                                                                                                      \
    cudaError_t e__ = (call);                                                                               \
    if (e__ != cudaSuccess)                                                                                 \
      return ::b200::fail(B200_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), __FILE__, \
                          __LINE__);                                                                        \
  } while (0)

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Kernels launched by this library since it was loaded (all threads, all devices).
inline std::atomic<unsigned long long> g_launch_count{0};

// After every kernel launch: count it and pick up a launch error.
#define B200_AFTER_LAUNCH()                                   \
  do {                                                        \
    ::b200::g_launch_count.fetch_add(1, std::memory_order_relaxed); \
    B200_CUDA(cudaGetLastError());                            \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

// Encode a tensor map of rank 2..4.  dims/box innermost first; strides in BYTES for
// dims 1..rank-1 (dim 0 is contiguous).  Returns 0 on success.
// Encoded maps are kept in a small cache keyed by every argument: the trunk calls each entry point with the same
// buffers block after block, so after the first block a launch costs a hash lookup instead of a driver call.
struct TmapKey {
  uint64_t v[16];
  bool operator==(const TmapKey& o) const { return memcmp(v, o.v, sizeof(v)) == 0; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (uint64_t x : k.v) h = (h ^ x) * 1099511628211ull;
    return size_t(h);
  }
};

inline int make_tmap(CUtensorMap* out, CUtensorMapDataType dtype, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz) {
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  TmapKey key;
  memset(&key, 0, sizeof(key));
  key.v[0] = reinterpret_cast<uint64_t>(base);
  key.v[1] = (uint64_t(dtype) << 32) | (uint64_t(rank) << 8) | uint64_t(swz);
  for (int i = 0; i < rank; ++i) {
    key.v[2 + i] = dims[i];
    key.v[7 + i] = box[i];
    if (i > 0) key.v[11 + i] = strides_bytes[i - 1];
  }
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = fn(out, dtype, rank, const_cast<void*>(base), gdim, gstr, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", int(r));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() >= 8192) cache.clear();  // bounded: a caller that cycles through many buffers just re-encodes
    cache.emplace(key, *out);
  }
  return 0;
}

inline int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz) {
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, rank, dims, strides_bytes, box, swz);
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device) instead of on every launch.
inline int set_smem_once(const void* kernel, uint32_t bytes) {
  static std::mutex mu;
  static std::unordered_set<uint64_t> done;
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  const uint64_t key = reinterpret_cast<uint64_t>(kernel) * 64 + uint64_t(dev & 63);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (done.count(key)) return 0;
  }
  B200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)));
  std::lock_guard<std::mutex> lock(mu);
  done.insert(key);
  return 0;
}

inline int sm_count() {
  static int n = 0;
  if (n) return n;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  return n;
}

}  // namespace b200
