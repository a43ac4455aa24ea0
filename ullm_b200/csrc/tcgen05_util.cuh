// Device and host helpers shared by the tcgen05 matrix-product kernels (linear_tcgen05.cu for few rows,
// linear_tcgen05_large.cu for many): mbarriers with bounded waits, TMA loads, shared-memory and instruction
// descriptors of tcgen05.mma for bfloat16 operands in K-major 128-byte-swizzled tiles, tensor-memory loads, and
// the host-side cache of tensor maps.
#pragma once

#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

#define ULLM_STATUS_TIMEOUT 6
#define WAIT_LIMIT (1 << 20)

__device__ __forceinline__ uint32_t lin_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(lin_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(lin_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(lin_smem(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// false: gave up after `limit` polls (the caller records it and stops waiting).  test_wait first: it is the
// cheaper instruction when the phase is already complete, which is the common case while a ring drains.
__device__ __forceinline__ bool mbar_wait_limited(uint64_t* bar, uint32_t parity, int limit) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(lin_smem(bar)), "r"(parity)
      : "memory");
  if (ok) return true;
  for (int i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  return mbar_wait_limited(bar, parity, WAIT_LIMIT);
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(lin_smem(smem_dst)), "l"(map), "r"(lin_smem(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(lin_smem(smem_dst)), "l"(map), "r"(lin_smem(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// shared-memory matrix descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle,
// groups of 8 rows 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(const void* smem_tile) {
  const uint32_t addr = lin_smem(smem_tile);
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);       // start address
  d |= (uint64_t)1 << 16;                        // leading-dimension offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride between 8-row groups
  d |= (uint64_t)1 << 46;                        // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                        // 128-byte swizzle
  return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same instruction with the descriptors given as their low words (start address in 16-byte units,
// leading-dimension field) and the high word they share: stepping a descriptor is then one 32-bit add.
// ACC: a compile-time accumulate flag (1), or the run-time flag `acc` (-1).
template <int ACC>
__device__ __forceinline__ void umma_bf16_lo(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                             uint32_t acc = 1) {
  if (ACC == 1) {
    asm volatile(
        "{\n .reg .b64 da, db;\n .reg .pred p;\n mov.b64 da, {%1, %3};\n mov.b64 db, {%2, %3};\n"
        " setp.eq.b32 p, 0, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n}\n"
        ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc)
        : "memory");
  } else {
    asm volatile(
        "{\n .reg .b64 da, db;\n .reg .pred p;\n mov.b64 da, {%1, %3};\n mov.b64 db, {%2, %3};\n"
        " setp.ne.b32 p, %5, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n}\n"
        ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(acc)
        : "memory");
  }
}
__device__ __forceinline__ void umma_commit_addr(uint32_t bar_smem) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_smem) : "memory");
}
// wait with the barrier given by its shared-memory address
__device__ __forceinline__ bool mbar_wait_addr(uint32_t bar_smem, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar_smem), "r"(parity)
      : "memory");
  if (ok) return true;
  for (int i = 0; i < WAIT_LIMIT; ++i) {
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar_smem), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(lin_smem(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}


__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(lin_smem(bar)) : "memory");
}

// ---------------------------------------------------------------------------------------------
// host side: tensor maps
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

struct MapKey {
  const void* ptr;
  long long rows, cols;
  int box_rows;  // negative: the three-dimensional gate/up map
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.rows) * 31) ^
           (std::hash<long long>()(k.cols) * 131) ^ (size_t)k.box_rows * 7919;
  }
};

// tensor map of a row-major bf16 matrix [rows, cols], boxes of box_rows x 64 columns, 128-byte swizzle
// (box_rows < 0: the matrix seen as [2][rows / 2][cols], boxes of 2 x -box_rows x 64)
static inline bool get_map(const void* ptr, long long rows, long long cols, int box_rows, CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
  static std::mutex g_maps_mutex;
  std::lock_guard<std::mutex> lock(g_maps_mutex);
  MapKey key{ptr, rows, cols, box_rows};
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return true;
  }
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return false;
  CUtensorMap m;
  CUresult r;
  if (box_rows > 0) {
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    // [2][rows / 2][cols]: gate rows, then up rows; a box takes -box_rows rows of each
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows / 2, 2};
    cuuint64_t strides[2] = {(cuuint64_t)cols * 2, (cuuint64_t)(rows / 2) * cols * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)(-box_rows), 2};
    cuuint32_t estr[3] = {1, 1, 1};
    r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) return false;
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps[key] = m;
  *out = m;
  return true;
}

