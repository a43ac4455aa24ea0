// Pieces shared by the weight-streaming kernels (linear_stream.cu, layer_tail_fused.cu): the chunked tensor map
// that brings a whole 256-wide k block of a matrix with one TMA copy, and the mma.sync / ldmatrix wrappers.
#pragma once

#include "tcgen05_util.cuh"

#define LS_CONSUMER_WARPS 8
#define LS_THREADS (32 * (LS_CONSUMER_WARPS + 1))
#define LS_BK 256                 // k per stage
#define LS_W_STAGE_BYTES 16384    // 32 rows x 256 k x 2 bytes
#define LS_MAX_STAGES 16

// A matrix [rows, cols] with cols a multiple of 64, seen as [cols / 64][rows][64]: one box brings 64-wide k
// chunks c .. c + 3 of `box_rows` rows, laid out chunk after chunk, each chunk rows x 128 bytes (128-byte
// swizzle): the same layout as four two-dimensional boxes, for a quarter of the copies.
static inline bool ls_chunked_map(const void* ptr, long long rows, long long cols, int box_rows, CUtensorMap* out) {
  struct Key {
    const void* ptr;
    long long rows, cols;
    int box_rows;
    bool operator==(const Key& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
  };
  struct Hash {
    size_t operator()(const Key& k) const {
      return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.rows) * 31) ^
             (std::hash<long long>()(k.cols) * 131) ^ (size_t)k.box_rows * 7919;
    }
  };
  static std::unordered_map<Key, CUtensorMap, Hash> maps;
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  Key key{ptr, rows, cols, box_rows};
  auto it = maps.find(key);
  if (it != maps.end()) {
    *out = it->second;
    return true;
  }
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr || cols % 64) return false;
  cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)cols * 2, 128};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 4};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMap m;
  if (enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (maps.size() > 4096) maps.clear();
  maps[key] = m;
  *out = m;
  return true;
}

__device__ __forceinline__ void ls_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ls_ldmatrix4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ls_ldmatrix2(uint32_t& r0, uint32_t& r1, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ls_bar_sync_consumers() {
  asm volatile("bar.sync 1, %0;" ::"n"(LS_CONSUMER_WARPS * 32) : "memory");
}

