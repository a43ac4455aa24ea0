// out[M, N] = x[M, K] . W[N, K]^T for few rows (M <= 64, the decode step's
// matrix products), bfloat16 in, 32-bit accumulate, bfloat16 or float32 out.
//
// The weight matrix is the big operand and is read exactly once; the kernel is a
// streaming pipeline around the 5th-generation tensor cores:
//
//   * W is the A operand of tcgen05.mma (M = 128 weight rows per block), x the B
//     operand (N = the batch rows padded to 16/32/48/64): "swap A/B", so that the
//     128-wide side of the instruction is filled by weight rows, not by the batch.
//   * One elected thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle)
//     of 128 x 64 weight tiles and Mpad x 64 activation tiles into a ring of
//     shared-memory stages; one elected thread issues the MMAs; the accumulator
//     [128 lanes x Mpad columns] lives in tensor memory.  mbarriers carry
//     "stage full" (TMA transaction bytes), "stage free" and "accumulator done"
//     (tcgen05.commit).
//   * K is split across the blocks of a thread-block cluster so that enough blocks
//     stream at once even when N is small; the partial accumulators meet in
//     distributed shared memory and are added in rank order (deterministic).
//   * Every load is issued by the block that uses it (no multicast).
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT polls the kernel records
// ULLM_STATUS_TIMEOUT in the status word, stops waiting, still frees its tensor
// memory and returns.
#include <cooperative_groups.h>
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace cg = cooperative_groups;

#define ULLM_STATUS_TIMEOUT 6
#define LIN_BM 128        // weight rows per block (UMMA M)
#define LIN_BK 64         // k elements per stage: 128 bytes of bf16 = one swizzle row
#define LIN_THREADS 128
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
// false: gave up (the caller records it and stops waiting)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (int i = 0; i < WAIT_LIMIT; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(lin_smem(smem_dst)), "l"(map), "r"(lin_smem(bar)), "r"(x), "r"(y)
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

struct LinParams {
  int M, N, K;          // rows of x, rows of W, shared dimension
  int m_pad;            // M rounded up to 16
  int k_blocks;         // ceil(K / 64)
  int splits;           // cluster size along K
  int stages;
  int out_f32;          // 1: float32 output, 0: bfloat16
  void* out;            // [M, N]
  const void* bias;     // [N] bf16 or null
  int* status;
};

// dynamic shared memory: [stages] x (A tile 16 KB | B tile m_pad*128 B), 1024-byte aligned; the
// first m_pad*128 floats are reused for the cluster reduction after the main loop
__global__ void __launch_bounds__(LIN_THREADS)
linear_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      const LinParams p) {
  extern __shared__ unsigned char lin_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[8], empty_bar[8], accum_bar;
  pdl_launch_dependents();
  __shared__ uint32_t tmem_base_slot;
  unsigned char* tiles = (unsigned char*)(((uintptr_t)lin_smem_raw + 1023) & ~(uintptr_t)1023);
  const int a_bytes = LIN_BM * 128, b_bytes = p.m_pad * 128, stage_bytes = a_bytes + ((b_bytes + 1023) & ~1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * LIN_BM;
  const int rank = blockIdx.y;  // position in the cluster = K split
  const int kb_per = (p.k_blocks + p.splits - 1) / p.splits;
  const int kb_begin = min(p.k_blocks, rank * kb_per), kb_end = min(p.k_blocks, kb_begin + kb_per);
  const int my_blocks = kb_end - kb_begin;
  const uint32_t tmem_cols = p.m_pad <= 32 ? 32 : 64;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    // The weights do not depend on the kernel before this one: the first ring of weight tiles is
    // requested at once, before tensor memory is set up and before pdl_wait().
    const int first = min(p.stages, my_blocks);
    for (int i = 0; i < first; ++i) {
      mbar_expect_tx(&full_bar[i], a_bytes + b_bytes);
      tma_load_2d(tiles + i * stage_bytes, &map_w, &full_bar[i], (kb_begin + i) * LIN_BK, n0);
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(lin_smem(&tmem_base_slot)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_base_slot;

  if (warp == 0 && lane == 0) {
    // ---- producer: TMA loads ---------------------------------------------------------------
    // (the first ring of weight tiles was requested at the top) the activation tiles follow once the
    // kernel before this one is complete
    const int first = min(p.stages, my_blocks);
    pdl_wait();
    for (int i = 0; i < first; ++i) {
      unsigned char* b = tiles + i * stage_bytes + a_bytes;
      tma_load_2d(b, &map_x, &full_bar[i], (kb_begin + i) * LIN_BK, 0);
    }
    for (int i = first; i < my_blocks; ++i) {
      const int s = i % p.stages;
      const uint32_t parity = ((i / p.stages) & 1) ^ 1;  // a fresh barrier passes a wait on parity 1
      if (!mbar_wait(&empty_bar[s], parity)) {
        ullm_report(p.status, ULLM_STATUS_TIMEOUT, 1, i);
        break;
      }
      unsigned char* a = tiles + s * stage_bytes;
      unsigned char* b = a + a_bytes;
      mbar_expect_tx(&full_bar[s], a_bytes + b_bytes);
      const int k = (kb_begin + i) * LIN_BK;
      tma_load_2d(a, &map_w, &full_bar[s], k, n0);
      tma_load_2d(b, &map_x, &full_bar[s], k, 0);
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer -------------------------------------------------------------------------
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.m_pad >> 3) << 17) |
                           ((uint32_t)(LIN_BM >> 4) << 24);
    bool ok = true;
    pdl_wait();  // the bounded waits below then cover TMA latency only, not the kernel before this one
    for (int i = 0; i < my_blocks && ok; ++i) {
      const int s = i % p.stages;
      const uint32_t parity = (i / p.stages) & 1;
      if (!mbar_wait(&full_bar[s], parity)) {
        ullm_report(p.status, ULLM_STATUS_TIMEOUT, 2, i);
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const unsigned char* a = tiles + s * stage_bytes;
      const unsigned char* b = a + a_bytes;
      const uint64_t adesc = umma_desc(a), bdesc = umma_desc(b);
#pragma unroll
      for (int kk = 0; kk < LIN_BK / 16; ++kk) {
        // 16 bf16 = 32 bytes further along the swizzled row: +2 in the 16-byte address field
        umma_bf16(tmem_d, adesc + 2 * kk, bdesc + 2 * kk, idesc, (i > 0 || kk > 0) ? 1u : 0u);
      }
      umma_commit(&empty_bar[s]);  // the stage is free once these MMAs have read it
    }
    umma_commit(&accum_bar);       // the accumulator is complete once every MMA above is
  }

  // ---- epilogue: all four warps; warp w owns accumulator lanes 32w .. 32w+31 ------------------------
  __syncwarp();
  pdl_wait();  // nothing of the previous kernel's may be overwritten before it is complete
  bool have = my_blocks > 0;
  if (have) {
    if (!mbar_wait(&accum_bar, 0)) {
      have = false;
      if (lane == 0) {
        ullm_report(p.status, ULLM_STATUS_TIMEOUT, 3, rank);
      }
    }
  }
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const int f = warp * 32 + lane;  // feature (weight row) inside the block
  float acc[64];
#pragma unroll
  for (int j = 0; j < 64; ++j) acc[j] = 0.f;
  if (have) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      if (c * 16 < p.m_pad) {
        float v[16];
        tmem_ld16(tmem_d + ((uint32_t)(warp * 32) << 16) + c * 16, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[c * 16 + j] = v[j];
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");

  const __nv_bfloat16* bias = (const __nv_bfloat16*)p.bias;
  if (p.splits == 1) {
    const int n = n0 + f;
    if (n < p.N) {
      const float bv = bias != nullptr ? __bfloat162float(bias[n]) : 0.f;
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        if (j < p.M) {
          const float v = acc[j] + bv;
          if (p.out_f32) ((float*)p.out)[(long long)j * p.N + n] = v;
          else ((__nv_bfloat16*)p.out)[(long long)j * p.N + n] = __float2bfloat16_rn(v);
        }
      }
    }
    __syncthreads();
  } else {
    // partial sums meet in distributed shared memory: red[j][f], j < m_pad
    cg::cluster_group cluster = cg::this_cluster();
    __syncthreads();  // every thread is past the main loop: the stage memory is free
    float* red = reinterpret_cast<float*>(tiles);
#pragma unroll
    for (int j = 0; j < 64; ++j)
      if (j < p.m_pad) red[j * LIN_BM + f] = acc[j];
    cluster.sync();
    const int per = LIN_BM / p.splits;  // features this block finishes
    for (int idx = threadIdx.x; idx < per * p.M; idx += LIN_THREADS) {
      const int j = idx / per, ff = rank * per + idx % per;
      const int n = n0 + ff;
      if (n >= p.N) continue;
      float sum = bias != nullptr ? __bfloat162float(bias[n]) : 0.f;
      for (int q = 0; q < p.splits; ++q) {
        const float* remote = cluster.map_shared_rank(red, q);
        sum += remote[j * LIN_BM + ff];
      }
      if (p.out_f32) ((float*)p.out)[(long long)j * p.N + n] = sum;
      else ((__nv_bfloat16*)p.out)[(long long)j * p.N + n] = __float2bfloat16_rn(sum);
    }
    cluster.sync();  // nobody leaves while a peer may still read its shared memory
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(tmem_cols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
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
  int box_rows;
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
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
static std::mutex g_maps_mutex;

// tensor map of a row-major bf16 matrix [rows, cols], boxes of box_rows x 64 columns, 128-byte swizzle
static bool get_map(const void* ptr, long long rows, long long cols, int box_rows, CUtensorMap* out) {
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
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {LIN_BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps[key] = m;
  *out = m;
  return true;
}

// Shapes this kernel takes: 1 <= M <= 64, K a multiple of 8 (16-byte rows for TMA), 16-byte aligned bases.
extern "C" int ullm_linear_tcgen05_supported(int M, int N, int K) {
  return M >= 1 && M <= 64 && N >= 1 && K >= 8 && K % 8 == 0;
}

static int g_lin_attr_set = 0;

extern "C" int ullm_linear_tcgen05(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                                   int out_f32, int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (!ullm_linear_tcgen05_supported(M, N, K)) return ULLM_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return ULLM_ERR_UNSUPPORTED;
  LinParams p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.m_pad = (M + 15) / 16 * 16;
  p.k_blocks = (K + LIN_BK - 1) / LIN_BK;
  p.out_f32 = out_f32;
  p.out = out;
  p.bias = bias;
  p.status = status;
  const int n_blocks = (N + LIN_BM - 1) / LIN_BM;
  // Split K across a cluster while all blocks still fit the GPU at once (two per SM) and each keeps at
  // least 4 k-blocks: one full wave streams, no tail wave.
  int splits = 1;
  while (splits < 8 && n_blocks * splits * 2 <= 296 && p.k_blocks / (splits * 2) >= 4) splits *= 2;
  p.splits = splits;
  const int b_bytes = ((p.m_pad * 128) + 1023) & ~1023;
  const int stage_bytes = LIN_BM * 128 + b_bytes;
  // Stages: the ring is what a block holds in flight, and what it has prefetched while it waits for
  // the kernel before it.  ULLM_B200_LIN_SMEM_KB bounds a block's ring (default 112 KB: two blocks per SM).
  static int ring_kb = 0;
  if (ring_kb == 0) {
    const char* e = getenv("ULLM_B200_LIN_SMEM_KB");
    ring_kb = e != nullptr ? atoi(e) : 112;
    if (ring_kb < 40 || ring_kb > 200) ring_kb = 112;
  }
  int stages = (ring_kb * 1024 - 1024) / stage_bytes;
  const int kb_per = (p.k_blocks + splits - 1) / splits;
  if (stages > kb_per) stages = kb_per < 2 ? 2 : kb_per;
  if (stages > 8) stages = 8;
  p.stages = stages;
  size_t smem = (size_t)stages * stage_bytes + 1024;
  const size_t red_bytes = (size_t)p.m_pad * LIN_BM * 4 + 1024;
  if (smem < red_bytes) smem = red_bytes;
  CUtensorMap map_w, map_x;
  if (!get_map(w, N, K, LIN_BM, &map_w) || !get_map(x, M, K, p.m_pad, &map_x)) return ULLM_ERR_LAUNCH;
  if (!g_lin_attr_set) {
    if (cudaFuncSetAttribute(linear_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) !=
        cudaSuccess)
      return ULLM_ERR_LAUNCH;
    cudaFuncSetAttribute(linear_tcgen05_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    g_lin_attr_set = 1;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_blocks, splits, 1);
  cfg.blockDim = dim3(LIN_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = splits;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_ullm_pdl ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, linear_tcgen05_kernel, map_w, map_x, p) != cudaSuccess) {
    cudaGetLastError();
    return ULLM_ERR_LAUNCH;
  }
  return ullm_launch_status();
}
