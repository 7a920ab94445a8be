// Host-side helpers: error codes, TMA tensor-map encoding through the driver
// entry point (no link-time libcuda dependency) and a small descriptor cache.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

#include "../../include/fox_b200.h"

namespace fox {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Description of a (B, H, T, D) tensor of 16-bit or 32-bit elements whose last
// dimension has unit stride; the other strides are in elements.
struct Tensor4 {
  void* ptr;
  int64_t B, H, T, D;
  int64_t sb, sh, st;
};

// Can TMA address this view?  (16-byte aligned base and byte strides.)
inline bool tma_compatible(const Tensor4& t, int elem_bytes) {
  if (reinterpret_cast<uintptr_t>(t.ptr) % 16) return false;
  const int64_t s[3] = {t.sb, t.sh, t.st};
  for (int i = 0; i < 3; ++i) {
    const int64_t bytes = s[i] * elem_bytes;
    if (bytes <= 0 || bytes % 16) return false;
  }
  return true;
}

// Tiled map with dims (D, T, H, B), box (box_d, box_t, 1, 1).  swizzle128 selects
// the 128-byte swizzle (box_d * elem_bytes must then be 128) or none.
inline int make_tmap_4d(CUtensorMap* out, const Tensor4& t, int elem_bytes, bool is_float32, bool is_bf16,
                        uint32_t box_d, uint32_t box_t, bool swizzle128) {
  EncodeTiledFn fn = get_encode_tiled();
  if (!fn) return FOX_ERR_DRIVER;
  // A dimension of extent 1 may carry any stride in a torch view; give it a legal one.
  cuuint64_t dims[4] = {(cuuint64_t)t.D, (cuuint64_t)t.T, (cuuint64_t)t.H, (cuuint64_t)t.B};
  int64_t st = t.st, sh = t.sh, sb = t.sb;
  if (t.T == 1 && (st * elem_bytes) % 16) st = t.D;
  if (t.H == 1 && (sh * elem_bytes) % 16) sh = t.D * t.T;
  if (t.B == 1 && (sb * elem_bytes) % 16) sb = t.D * t.T * t.H;
  cuuint64_t strides[3] = {(cuuint64_t)(st * elem_bytes), (cuuint64_t)(sh * elem_bytes),
                           (cuuint64_t)(sb * elem_bytes)};
  cuuint32_t box[4] = {box_d, box_t, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMapDataType dt = is_float32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                      : (is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  CUresult r = fn(out, dt, 4, t.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FOX_OK : FOX_ERR_TENSORMAP;
}

// ------------------------------------------------------------- tensor-map cache
struct TmapKey {
  uintptr_t ptr;
  int64_t v[7];
  uint32_t w[4];
  bool operator==(const TmapKey& o) const {
    if (ptr != o.ptr) return false;
    for (int i = 0; i < 7; ++i)
      if (v[i] != o.v[i]) return false;
    for (int i = 0; i < 4; ++i)
      if (w[i] != o.w[i]) return false;
    return true;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = 1469598103934665603ull ^ k.ptr;
    for (int i = 0; i < 7; ++i) h = (h ^ (uint64_t)k.v[i]) * 1099511628211ull;
    for (int i = 0; i < 4; ++i) h = (h ^ (uint64_t)k.w[i]) * 1099511628211ull;
    return (size_t)h;
  }
};

// Encoding a tensor map costs a few microseconds; training loops call with the
// same (pointer, shape, strides) over and over, so maps are memoised.
inline int cached_tmap_4d(CUtensorMap* out, const Tensor4& t, int elem_bytes, bool is_float32, bool is_bf16,
                          uint32_t box_d, uint32_t box_t, bool swizzle128) {
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  TmapKey k;
  k.ptr = reinterpret_cast<uintptr_t>(t.ptr);
  k.v[0] = t.B; k.v[1] = t.H; k.v[2] = t.T; k.v[3] = t.D; k.v[4] = t.sb; k.v[5] = t.sh; k.v[6] = t.st;
  k.w[0] = box_d; k.w[1] = box_t;
  k.w[2] = (uint32_t)elem_bytes | (is_float32 ? 16u : 0u) | (is_bf16 ? 32u : 0u) | (swizzle128 ? 64u : 0u);
  k.w[3] = 0;
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(k);
    if (it != cache.end()) {
      *out = it->second;
      return FOX_OK;
    }
  }
  int rc = make_tmap_4d(out, t, elem_bytes, is_float32, is_bf16, box_d, box_t, swizzle128);
  if (rc != FOX_OK) return rc;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(k, *out);
  return FOX_OK;
}

}  // namespace fox
