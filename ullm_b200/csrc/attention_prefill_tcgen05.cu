// Paged causal attention for bfloat16 prompt portions on the 5th-generation
// tensor cores (head size 128).  A block owns 128 rows of one kv head for one
// request (rows are (token, query head of the group) pairs, so one pass over K and
// V serves every head that shares them) and walks the request's keys in tiles of
// 64:
//
//   S[128 x 64]   = Q[128 x 128] K^T        tcgen05.mma, A and B K-major from shared memory,
//                                           accumulator in tensor memory (64 columns)
//   P             = 2^(S * scale - m)       four softmax warps, one thread per row, read S with
//                                           tcgen05.ld; 32-bit max, sum and exponent (ex2)
//   O[128 x 128] += P[128 x 64] V           P (bf16) goes to shared memory as the A operand, V is the
//                                           MN-major B operand; O stays in tensor memory (128 columns)
//                                           and is rescaled there when a row's maximum moves
//
// Q, K and V tiles are brought in by TMA (cp.async.bulk.tensor, 128-byte swizzle): Q as one 3-D box of
// the projection buffer that gathers (token, head) rows, K and V page by page (a page of 16 tokens is two
// swizzle groups of 8 rows) through 4-D maps of the cache.  One thread issues the loads, one thread the
// MMAs; mbarriers carry "tile landed", "scores ready", "P ready", "P.V done", "stage free".  Slots of a
// page past the request's length are zeroed in shared memory before V is used (they may hold anything).
// Every load is issued by the block that uses it.
//
// Every wait on an mbarrier is bounded; a wait that runs out records ULLM_STATUS_TIMEOUT, and the block
// stops waiting, frees its tensor memory and returns.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tma_host.cuh"

#define ULLM_STATUS_TIMEOUT 6
#define TA_ROWS 128
#define TA_KEYS 64
#define TA_D 128
#define TA_THREADS 192
#define TA_WAIT_LIMIT (1 << 20)
#define TA_TILE_Q (TA_ROWS * TA_D * 2)   // 32 KB: two halves of [128 rows x 128 B]
#define TA_TILE_KV (TA_KEYS * TA_D * 2)  // 16 KB: two halves of [64 keys x 128 B]
#define TA_TILE_P (TA_ROWS * TA_KEYS * 2)  // 16 KB: [128 rows x 128 B]
#define TA_STAGES 2
#define TA_BARRIER_BYTES 128  // mbarriers and the tensor-memory slot, behind the tiles
#define TA_TILES_BYTES (TA_TILE_Q + TA_STAGES * 2 * TA_TILE_KV + TA_TILE_P)  // 112 KB
#define TA_SMEM (TA_TILES_BYTES + TA_BARRIER_BYTES)

__device__ __forceinline__ uint32_t ta_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ta_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ta_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void ta_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ta_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ta_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ta_smem(bar)) : "memory");
}
__device__ __forceinline__ bool ta_mbar_wait(uint64_t* bar, uint32_t parity) {
  for (int i = 0; i < TA_WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(ta_smem(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void ta_tma_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(ta_smem(dst)), "l"(map), "r"(ta_smem(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void ta_tma_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z,
                                          int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(ta_smem(dst)), "l"(map), "r"(ta_smem(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
// K-major operand tile: rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t ta_desc_kmajor(const void* tile) {
  uint64_t d = (uint64_t)((ta_smem(tile) & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// MN-major operand tile (V as B: N = head dim, K = keys): a row of 128 bytes holds 64 neighbouring
// N elements of one key; 8-key groups 1024 bytes apart (stride offset); the next 64 N elements
// `lbo_bytes` further (leading offset)
__device__ __forceinline__ uint64_t ta_desc_mnmajor(const void* tile, uint32_t lbo_bytes) {
  uint64_t d = (uint64_t)((ta_smem(tile) & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo_bytes >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ void ta_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void ta_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ta_smem(bar))
               : "memory");
}
__device__ __forceinline__ void ta_tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// 64 columns of this thread's lane: two loads in flight, one wait
__device__ __forceinline__ void ta_tmem_ld64(uint32_t taddr, float (&v)[64]) {
  uint32_t r[64];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31}, [%32];"
      : "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
        "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
        "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
        "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr + 32));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void ta_tmem_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,"
      "%31,%32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
      "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
      "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
      "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
      "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])),
      "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
      "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
      "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])),
      "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])),
      "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float ta_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct TaParams {
  const int* block_table;
  const int* req_slots;
  const int* cu_q;
  const int* kv_len;
  __nv_bfloat16* out;
  int* status;
  int max_pages, num_requests, num_q, num_kv, page_size, window;
  float scale_log2;
  long long num_pages;
};

// 6 warps are scheduled like 8 (two per scheduler partition): the register budget for two blocks per SM is
// 65536 / (2 * 8 * 32) = 128 per thread.
__global__ void __launch_bounds__(256, 2)
prefill_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v, const TaParams p) {
  // No static shared memory and no slack: two blocks of 112 KB of tiles + 128 bytes of barriers fit one SM.
  // The tiles need a 1024-byte boundary (128-byte swizzle); the dynamic region of a block that has no static
  // shared memory starts on one.  If it ever did not, the block says so and leaves.
  extern __shared__ __align__(16) unsigned char ta_raw[];
  pdl_launch_dependents();
  if ((ta_smem(ta_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 10, (int)(ta_smem(ta_raw) & 1023u));
    return;
  }
  unsigned char* base = ta_raw;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ta_raw + TA_TILES_BYTES);
  // One barrier pair per K/V stage (separate pairs for K and V, to fetch K two tiles ahead, were slower).
  uint64_t& q_full = bars[0];
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = bars + 1 + TA_STAGES;
  uint64_t* s_full = bars + 1 + 2 * TA_STAGES;  // one per score buffer
  uint64_t& p_ready = bars[3 + 2 * TA_STAGES];
  uint64_t& pv_done = bars[4 + 2 * TA_STAGES];
  uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bars + 5 + 2 * TA_STAGES);
  unsigned char* q_s = base;
  unsigned char* kv_s = base + TA_TILE_Q;                       // stage s: K at s * 2 * KV, V right after it
  unsigned char* p_s = kv_s + TA_STAGES * 2 * TA_TILE_KV;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // A 1-D grid, numbered so that consecutive blocks are the same token tile of all kv heads: the block
  // scheduler then starts the heaviest tiles of EVERY head first (longest work first keeps the SMs level).
  const int kh = (int)(blockIdx.x % p.num_kv);
  const int G = p.num_q / p.num_kv;
  const int tpt = TA_ROWS / G;
  pdl_wait();

  // ---- which request and which of its token tiles (numbered from the back: heavy tiles first) ----------
  const int tile_id = (int)(gridDim.x / p.num_kv) - 1 - (int)(blockIdx.x / p.num_kv);
  int r = -1, first = 0, q_len = 0, q_begin = 0;
  {
    int running = 0;
    for (int i = 0; i < p.num_requests; ++i) {
      const int b = p.cu_q[i], n = p.cu_q[i + 1] - b;
      const int nt = (n + tpt - 1) / tpt;
      if (tile_id < running + nt) {
        r = i;
        first = (tile_id - running) * tpt;
        q_len = n;
        q_begin = b;
        break;
      }
      running += nt;
    }
  }
  if (r < 0) return;
  const int kvl = p.kv_len[r];
  const int ntok = min(tpt, q_len - first);
  const int rows_valid = ntok * G;
  const int p0 = kvl - q_len + first, p1 = p0 + ntok - 1;
  if (kvl <= 0 || p0 < 0) {
    for (int i = tid; i < rows_valid * TA_D; i += blockDim.x) {
      const int row = i / TA_D, d = i - row * TA_D;
      p.out[((long long)(q_begin + first + row / G) * p.num_q + kh * G + row % G) * TA_D + d] = __float2bfloat16_rn(0.f);
    }
    return;
  }
  const int key_lo = p.window > 0 ? max(0, p0 - p.window + 1) : 0;
  const int k_start = key_lo / TA_KEYS * TA_KEYS;
  const int tiles = (p1 - k_start) / TA_KEYS + 1;
  const int* bt = p.block_table + (long long)p.req_slots[r] * p.max_pages;
  const int pages_per_tile = TA_KEYS / p.page_size;

  if (tid == 0) {
    ta_mbar_init(&q_full, 1);
    for (int s = 0; s < TA_STAGES; ++s) {
      ta_mbar_init(&kv_full[s], 1);
      ta_mbar_init(&kv_empty[s], 1);
    }
    ta_mbar_init(&s_full[0], 1);
    ta_mbar_init(&s_full[1], 1);
    ta_mbar_init(&p_ready, 128);
    ta_mbar_init(&pv_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ta_smem(&tmem_slot)), "r"(256)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_s = tmem_slot;         // columns 0..63 and 64..127: two score buffers (tile t uses t & 1)
  const uint32_t tmem_o = tmem_slot + 128;   // columns 128..255: output accumulator

  if (warp == 4) {
    // ---- producer: the whole warp reads page ids (one coalesced load per tile, a tile ahead of their use),
    // lane 0 issues the TMA loads ---------------------------------------------------------------------------
    if (lane == 0) {
      ta_mbar_expect_tx(&q_full, TA_TILE_Q);
      ta_tma_3d(q_s, &map_q, &q_full, 0, kh * G, q_begin + first);
      ta_tma_3d(q_s + TA_TILE_Q / 2, &map_q, &q_full, 64, kh * G, q_begin + first);
    }
    auto page_of = [&](int t) -> int {  // lane pg holds the page of the pg-th page of tile t
      const int key = k_start + t * TA_KEYS + lane * p.page_size;
      int page = -1;
      if (lane < pages_per_tile && key < kvl) {
        // a tile may begin before the first key any row can see; pages there may have been given back
        // (entry -1): they are zero-filled and masked.  Only an id beyond the pool is an error.
        page = bt[key / p.page_size];
        if (page >= p.num_pages) {
          ullm_report(p.status, ULLM_STATUS_PAGE, r, page);
          page = -1;
        }
      }
      return page;
    };
    int pages_next = page_of(0);
    bool ok = true;
    for (int t = 0; t < tiles && ok; ++t) {
      const int s = t % TA_STAGES;
      const int pages_now = pages_next;
      if (t + 1 < tiles) pages_next = page_of(t + 1);  // in flight while this tile's stage is awaited
      unsigned char* k_t = kv_s + s * 2 * TA_TILE_KV;
      unsigned char* v_t = k_t + TA_TILE_KV;
      if (lane == 0 && !ta_mbar_wait(&kv_empty[s], ((t / TA_STAGES) & 1) ^ 1)) {
        ullm_report(p.status, ULLM_STATUS_TIMEOUT, 11, t);
        ok = false;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane == 0) ta_mbar_expect_tx(&kv_full[s], 2 * TA_TILE_KV);
      for (int pg = 0; pg < pages_per_tile; ++pg) {
        const int page = __shfl_sync(0xffffffffu, pages_now, pg);
        if (lane == 0) {
          // a page that is not there (-1) is out of the map's range: the box is filled with zeros
          const int pcoord = page >= 0 ? page : (int)p.num_pages;
          const int off = pg * p.page_size * 128;
          ta_tma_4d(k_t + off, &map_k, &kv_full[s], 0, kh, 0, pcoord);
          ta_tma_4d(k_t + TA_TILE_KV / 2 + off, &map_k, &kv_full[s], 64, kh, 0, pcoord);
          ta_tma_4d(v_t + off, &map_v, &kv_full[s], 0, kh, 0, pcoord);
          ta_tma_4d(v_t + TA_TILE_KV / 2 + off, &map_v, &kv_full[s], 64, kh, 0, pcoord);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // ---- MMA issuer -----------------------------------------------------------------------------------
      // S: M 128, N 64, both operands K-major.  O: M 128, N 128, A (P) K-major, B (V) MN-major.
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TA_KEYS >> 3) << 17) |
                               ((uint32_t)(TA_ROWS >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(TA_D >> 3) << 17) |
                               ((uint32_t)(TA_ROWS >> 4) << 24);
      bool ok = ta_mbar_wait(&q_full, 0);
      if (!ok) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 12, 0);
      // Two score buffers: the scores of tile t + 1 are issued right behind P.V of tile t, while the
      // softmax warps may still be reading the scores of tile t (issuing them BEFORE P.V was slower: with
      // two K/V stages the wait for tile t + 1 to land then sits in front of P.V).
      auto issue_scores = [&](int t) -> bool {
        const int s = t % TA_STAGES;
        if (!ta_mbar_wait(&kv_full[s], (t / TA_STAGES) & 1)) {
          ullm_report(p.status, ULLM_STATUS_TIMEOUT, 13, t);
          return false;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned char* k_t = kv_s + s * 2 * TA_TILE_KV;
#pragma unroll
        for (int kk = 0; kk < TA_D / 16; ++kk) {
          // d = 16 kk: half kk / 4 of the Q and K tiles, 32 bytes further per step inside a half
          const uint64_t a = ta_desc_kmajor(q_s + (kk >> 2) * (TA_TILE_Q / 2)) + 2 * (kk & 3);
          const uint64_t b = ta_desc_kmajor(k_t + (kk >> 2) * (TA_TILE_KV / 2)) + 2 * (kk & 3);
          ta_mma(tmem_s + (t & 1) * TA_KEYS, a, b, idesc_s, kk > 0 ? 1u : 0u);
        }
        ta_commit(&s_full[t & 1]);
        return true;
      };
      if (ok) ok = issue_scores(0);
      for (int t = 0; t < tiles && ok; ++t) {
        if (!ta_mbar_wait(&p_ready, t & 1)) {
          ullm_report(p.status, ULLM_STATUS_TIMEOUT, 14, t);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned char* v_t = kv_s + (t % TA_STAGES) * 2 * TA_TILE_KV + TA_TILE_KV;
#pragma unroll
        for (int ks = 0; ks < TA_KEYS / 16; ++ks) {
          // 16 keys = 32 bytes along a row of P; two 8-key groups = 2048 bytes down the V tile
          const uint64_t a = ta_desc_kmajor(p_s) + 2 * ks;
          const uint64_t b = ta_desc_mnmajor(v_t + ks * 2048, TA_TILE_KV / 2);
          ta_mma(tmem_o, a, b, idesc_o, (t > 0 || ks > 0) ? 1u : 0u);
        }
        ta_commit(&kv_empty[t % TA_STAGES]);
        ta_commit(&pv_done);
        if (t + 1 < tiles && !issue_scores(t + 1)) break;
      }
    }
  } else {
    // ---- softmax: thread `tid` owns row `tid` (tensor-memory lane `tid`) ------------------------------------
    const int row = tid;
    const bool row_ok = row < rows_valid;
    const int pos = row_ok ? p0 + row / G : -1;
    const int lo = p.window > 0 ? pos - p.window + 1 : 0;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int t = 0; t < tiles && ok; ++t) {
      const int key0 = k_start + t * TA_KEYS;
      if (!ta_mbar_wait(&s_full[t & 1], (t >> 1) & 1)) {
        if (lane == 0) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 15, t);
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float s[TA_KEYS];
      ta_tmem_ld64(tmem_s + (t & 1) * TA_KEYS + lane_base, s);
      const bool need_mask = rows_valid < TA_ROWS || key0 + TA_KEYS - 1 > p0 || (p.window > 0 && key0 < p1 - p.window + 1);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < TA_KEYS; ++i) {
          const int key = key0 + i;
          if (!(key <= pos && key >= lo)) s[i] = -INFINITY;
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < TA_KEYS; ++i) mx = fmaxf(mx, s[i]);
      // The reference point of the exponents only moves when the row's maximum grows by more than 2^8:
      // until then P is at most 256 (exact in bf16 range, sums in 32-bit), and O and l, which share the
      // reference, need no rescaling.  The result O / l does not depend on the reference.
      const float m_cand = fmaxf(m, mx * p.scale_log2);
      const float m_new = (m == -INFINITY || m_cand - m > 8.f) ? m_cand : m;
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = ta_ex2(m - m_use);
      m = m_new;
      // P in registers first (packed bf16): this part overlaps the P.V product of the tile before
      uint4 chunks[TA_KEYS / 8];
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int c = 0; c < TA_KEYS / 8; ++c) {
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&chunks[c]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float a = ta_ex2(fmaf(s[c * 8 + 2 * i], p.scale_log2, -m_use));
          const float b = ta_ex2(fmaf(s[c * 8 + 2 * i + 1], p.scale_log2, -m_use));
          sum0 += a;
          sum1 += b;
          h2[i] = __floats2bfloat162_rn(a, b);
        }
      }
      l = l * alpha + (sum0 + sum1);
      // the P tile in shared memory and O in tensor memory are in use until P.V of the tile before is done
      if (t > 0) {
        if (!ta_mbar_wait(&pv_done, (t - 1) & 1)) {
          if (lane == 0) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 16, t);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
      // P row -> shared memory, K-major, 128-byte swizzle: chunk c of row r at (r/8)*1024 + (r%8)*128 + ((c^(r%8))*16)
      unsigned char* prow = p_s + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
      for (int c = 0; c < TA_KEYS / 8; ++c) *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) * 16)) = chunks[c];
      // the last tile may hold slots past the request's length: whatever they contain must not reach O
      if (key0 + TA_KEYS > kvl) {
        // (the tile's scores exist, so its K and V, which share a barrier, have landed)
        unsigned char* v_t = kv_s + (t % TA_STAGES) * 2 * TA_TILE_KV + TA_TILE_KV;
        const int first_bad = max(0, kvl - key0);
        for (int i = tid; i < (TA_KEYS - first_bad) * 16; i += 128) {
          const int key = first_bad + i / 16, ch = i % 16;  // 16 chunks of 16 bytes per key: 8 per half
          *reinterpret_cast<uint4*>(v_t + (ch >> 3) * (TA_TILE_KV / 2) + key * 128 + (ch & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
      }
      if (t > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
        for (int c = 0; c < TA_D / 32; ++c) {
          float v[32];
          ta_tmem_ld32(tmem_o + lane_base + c * 32, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] *= alpha;
          ta_tmem_st32(tmem_o + lane_base + c * 32, v);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      ta_mbar_arrive(&p_ready);
    }
    if (ok && !ta_mbar_wait(&pv_done, (tiles - 1) & 1)) {
      if (lane == 0) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 17, tiles);
      ok = false;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat16* op = p.out + ((long long)(q_begin + first + row / G) * p.num_q + kh * G + row % G) * TA_D;
#pragma unroll
    for (int c = 0; c < TA_D / 32; ++c) {
      float v[32];
      ta_tmem_ld32(tmem_o + lane_base + c * 32, v);  // all lanes of the warp take part
      if (row_ok && ok) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 chunk;
          __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&chunk);
#pragma unroll
          for (int k = 0; k < 4; ++k) h2[k] = __floats2bfloat162_rn(v[i * 8 + 2 * k] * inv, v[i * 8 + 2 * k + 1] * inv);
          *reinterpret_cast<uint4*>(op + c * 32 + i * 8) = chunk;
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncwarp();  // the lanes of the single-thread role wait here for their lane 0 (the barrier counts warps)
  __syncthreads();
  if (warp == 5) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_slot), "r"(256) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef UllmTmaEncodeFn TaEncodeFn;
static TaEncodeFn ta_encode() { return ullm_tma_encode(); }

struct TaKey {
  const void* ptr;
  long long a, b, c;
  bool operator==(const TaKey& o) const { return ptr == o.ptr && a == o.a && b == o.b && c == o.c; }
};
struct TaKeyHash {
  size_t operator()(const TaKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.a) * 31) ^ (std::hash<long long>()(k.b) * 131) ^
           (std::hash<long long>()(k.c) * 8191);
  }
};
static std::unordered_map<TaKey, CUtensorMap, TaKeyHash> g_ta_maps;
static std::mutex g_ta_mutex;

// Q: the projection buffer [tokens, heads_total, 128]; a box gathers 64 columns x G heads x 128/G tokens
static bool ta_map_q(const void* q, long long tokens, long long row_stride_elems, int heads_total, int G,
                     CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_ta_mutex);
  TaKey key{q, tokens, row_stride_elems, (long long)heads_total * 1000 + G};
  auto it = g_ta_maps.find(key);
  if (it != g_ta_maps.end()) {
    *out = it->second;
    return true;
  }
  TaEncodeFn enc = ta_encode();
  if (enc == nullptr) return false;
  cuuint64_t dims[3] = {TA_D, (cuuint64_t)heads_total, (cuuint64_t)tokens};
  cuuint64_t strides[2] = {TA_D * 2, (cuuint64_t)row_stride_elems * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(TA_ROWS / G)};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMap m;
  if (enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (g_ta_maps.size() > 4096) g_ta_maps.clear();
  g_ta_maps[key] = m;
  *out = m;
  return true;
}
// K or V pages [pages, page_size, kv heads, 128]; a box is one page of one head, 64 columns
static bool ta_map_kv(const void* cache, long long pages, int page_size, int num_kv, CUtensorMap* out) {
  return ullm_tma_map_kv(cache, pages, page_size, num_kv, TA_D, page_size, out);
}

// bfloat16, head size 128, a power-of-two number (<= 16) of query heads per kv head, pages of 8, 16, 32 or 64 tokens
extern "C" int ullm_prefill_attention_tcgen05_supported(int head_dim, int num_q, int num_kv, int page_size) {
  if (num_kv <= 0 || num_q % num_kv) return 0;
  const int G = num_q / num_kv;
  if (head_dim != TA_D || G > 16 || (G & (G - 1))) return 0;
  return page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64;
}

static int g_ta_attr_set = 0;
static int g_ta_blocks_per_sm = -1;

// Blocks of the kernel that fit one SM (2 is the design point); -1 before the first launch.
extern "C" int ullm_prefill_attention_tcgen05_blocks_per_sm(void) { return g_ta_blocks_per_sm; }

extern "C" int ullm_prefill_attention_tcgen05(const void* q, long long q_row_stride, void* out, const void* k_cache,
                                              const void* v_cache, const int* block_table, int max_pages,
                                              const int* req_slots, const int* cu_q, const int* kv_len, int tokens,
                                              int num_requests, int num_q, int num_kv, int head_dim, int page_size,
                                              int window, float scale, long long num_pages, int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || num_requests <= 0 || max_pages <= 0 || window < 0) return ULLM_ERR_BAD_SIZE;
  if (!ullm_prefill_attention_tcgen05_supported(head_dim, num_q, num_kv, page_size)) return ULLM_ERR_UNSUPPORTED;
  if (q_row_stride % 8 || ((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) % 16)
    return ULLM_ERR_UNSUPPORTED;
  if (q_row_stride % TA_D) return ULLM_ERR_UNSUPPORTED;
  if (tokens == 0) return ULLM_OK;
  const int G = num_q / num_kv;
  CUtensorMap mq, mk, mv;
  if (!ta_map_q(q, tokens, q_row_stride, (int)(q_row_stride / TA_D), G, &mq) ||
      !ta_map_kv(k_cache, num_pages, page_size, num_kv, &mk) || !ta_map_kv(v_cache, num_pages, page_size, num_kv, &mv))
    return ULLM_ERR_LAUNCH;
  if (!g_ta_attr_set) {
    if (cudaFuncSetAttribute(prefill_attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TA_SMEM) !=
        cudaSuccess)
      return ULLM_ERR_LAUNCH;
    // ask for the largest shared-memory carve-out, so that two blocks of 112 KB share an SM
    cudaFuncSetAttribute(prefill_attention_tcgen05_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    g_ta_attr_set = 1;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&g_ta_blocks_per_sm, prefill_attention_tcgen05_kernel, TA_THREADS,
                                                  TA_SMEM);
  }
  TaParams p;
  p.block_table = block_table;
  p.req_slots = req_slots;
  p.cu_q = cu_q;
  p.kv_len = kv_len;
  p.out = (__nv_bfloat16*)out;
  p.status = status;
  p.max_pages = max_pages;
  p.num_requests = num_requests;
  p.num_q = num_q;
  p.num_kv = num_kv;
  p.page_size = page_size;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.num_pages = num_pages;
  const int tpt = TA_ROWS / G;
  dim3 grid(((tokens + tpt - 1) / tpt + num_requests) * num_kv);
  return ullm_launch_kernel(prefill_attention_tcgen05_kernel, grid, dim3(TA_THREADS), (size_t)TA_SMEM, st, mq, mk, mv, p);
}

// Blocks per SM the kernel would get with `smem_bytes` of dynamic shared memory (a sizing aid).
extern "C" int ullm_prefill_attention_tcgen05_occupancy_for(int smem_bytes) {
  int n = -1;
  cudaFuncSetAttribute(prefill_attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  cudaFuncSetAttribute(prefill_attention_tcgen05_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                       cudaSharedmemCarveoutMaxShared);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, prefill_attention_tcgen05_kernel, TA_THREADS, smem_bytes);
  cudaFuncAttributes a;
  if (cudaFuncGetAttributes(&a, prefill_attention_tcgen05_kernel) == cudaSuccess && smem_bytes < 0)
    return (int)a.sharedSizeBytes * 1000 + a.numRegs;
  return n;
}
