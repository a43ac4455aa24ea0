// Host-side helper: tensor maps (TMA descriptors) of paged K / V pools, cached by what defines them.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <unordered_map>

typedef CUresult (*UllmTmaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda); null if absent
static inline UllmTmaEncodeFn ullm_tma_encode() {
  static UllmTmaEncodeFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (UllmTmaEncodeFn)ptr;
  }
  return fn;
}

struct UllmKvMapKey {
  const void* ptr;
  long long pages;
  int page_size, num_kv, head_dim, box_tokens;
  bool operator==(const UllmKvMapKey& o) const {
    return ptr == o.ptr && pages == o.pages && page_size == o.page_size && num_kv == o.num_kv &&
           head_dim == o.head_dim && box_tokens == o.box_tokens;
  }
};
struct UllmKvMapKeyHash {
  size_t operator()(const UllmKvMapKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.pages) * 31) ^
           ((size_t)k.page_size * 131) ^ ((size_t)k.num_kv * 8191) ^ ((size_t)k.head_dim * 524287) ^
           ((size_t)k.box_tokens * 7919);
  }
};

// A bfloat16 pool [pages, page_size, num_kv, head_dim]; a box holds 64 elements (128 bytes, 128-byte swizzle)
// of one head for `box_tokens` consecutive tokens of one page.
static inline bool ullm_tma_map_kv(const void* pool, long long pages, int page_size, int num_kv, int head_dim,
                                   int box_tokens, CUtensorMap* out) {
  static std::unordered_map<UllmKvMapKey, CUtensorMap, UllmKvMapKeyHash> maps;
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  UllmKvMapKey key{pool, pages, page_size, num_kv, head_dim, box_tokens};
  auto it = maps.find(key);
  if (it != maps.end()) {
    *out = it->second;
    return true;
  }
  UllmTmaEncodeFn enc = ullm_tma_encode();
  if (enc == nullptr) return false;
  cuuint64_t dims[4] = {(cuuint64_t)head_dim, (cuuint64_t)num_kv, (cuuint64_t)page_size, (cuuint64_t)pages};
  cuuint64_t strides[3] = {(cuuint64_t)head_dim * 2, (cuuint64_t)num_kv * head_dim * 2,
                           (cuuint64_t)page_size * num_kv * head_dim * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_tokens, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMap m;
  if (enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(pool), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (maps.size() > 4096) maps.clear();
  maps[key] = m;
  *out = m;
  return true;
}
