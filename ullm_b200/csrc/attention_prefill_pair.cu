// Paged causal attention for bfloat16 prompt portions on the 5th-generation tensor cores (head size 128),
// two query tiles per block.
//
// A block owns 256 rows of one kv head for one request: two query tiles of 128 rows (rows are (token, query
// head of the group) pairs, so one pass over K and V serves every head that shares them).  It walks the
// request's keys in tiles of 128; each K and V tile is loaded ONCE for both query tiles.
//
//   S_i[128 x 128]  = Q_i[128 x 128] K^T      tcgen05.mma, A and B K-major from shared memory, accumulator in
//                                             tensor memory (128 columns per query tile)
//   P_i             = 2^(S_i * scale - m)     one softmax warp group per query tile, one thread per row: reads S
//                                             with tcgen05.ld, keeps max, sum and exponent in 32-bit, and writes
//                                             P as packed bfloat16 back into the first 64 columns of S_i
//   O_i[128 x 128] += P_i[128 x 128] V        tcgen05.mma with the A operand in tensor memory; V is the MN-major
//                                             B operand from shared memory; O_i stays in tensor memory (128
//                                             columns per tile) and is rescaled there when a row's maximum moves
//
// The MMA thread issues   P.V_0(j), S_0(j+1), P.V_1(j), S_1(j+1), ...   so the tensor pipe works on one query
// tile while the other tile's warp group does its softmax.  Tensor memory: S_0, S_1, O_0, O_1 = 512 columns; one
// block per SM.  Shared memory: two Q tiles (64 KB), K tile 0, and two slots for the pairs (V_j, K_{j+1}): all
// that step j of the MMA thread reads, loaded under one barrier and given back by one commit.  (What this thread
// does between two products is on the critical path: its waits poll, its descriptors are stepped by adds, and a
// step has three commits: the two score barriers, which also cover the P.V products issued before them, and the
// pair's release.)
//
// Q, K and V tiles are brought in by TMA (cp.async.bulk.tensor, 128-byte swizzle): Q as 3-D boxes of the
// projection buffer that gather (token, head) rows, K and V page by page through 4-D maps of the cache.  Slots of
// a page past the request's length are zeroed in shared memory before V is used (they may hold anything).  Every
// load is issued by the block that uses it.
//
// Every wait on an mbarrier is bounded; a wait that runs out records ULLM_STATUS_TIMEOUT, and the block stops
// waiting, frees its tensor memory and returns.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tma_host.cuh"

#define ULLM_STATUS_TIMEOUT 6
#define TP_ROWS 128
#define TP_KEYS 128
#define TP_D 128
#define TP_THREADS 320  // warps 0-3: softmax of tile 0; 4-7: softmax of tile 1; 8: loads; 9: MMA
#define TP_WAIT_LIMIT (1 << 20)
#define TP_TILE_Q (TP_ROWS * TP_D * 2)    // 32 KB: two halves of [128 rows x 128 B]
#define TP_TILE_KV (TP_KEYS * TP_D * 2)   // 32 KB: two halves of [128 keys x 128 B]
#define TP_TILES_BYTES (2 * TP_TILE_Q + 5 * TP_TILE_KV)  // 224 KB: two Q tiles, K tile 0, two (V, K) pairs
#define TP_BARRIER_BYTES 256
#define TP_SMEM (TP_TILES_BYTES + TP_BARRIER_BYTES)
#define TP_TMEM_COLS 512


__device__ __forceinline__ uint32_t tp_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tp_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tp_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void tp_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tp_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tp_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tp_smem(bar)) : "memory");
}
// test_wait first: it is the cheaper instruction when the phase is already complete
__device__ __forceinline__ bool tp_mbar_wait(uint64_t* bar, uint32_t parity) {
  {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(tp_smem(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  for (int i = 0; i < TP_WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(tp_smem(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
// the same by polling without suspension (the MMA thread: its wake-up is on the critical path)
__device__ __forceinline__ bool tp_mbar_spin(uint64_t* bar, uint32_t parity) {
  for (int i = 0; i < TP_WAIT_LIMIT * 16; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(tp_smem(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void tp_tma_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(tp_smem(dst)), "l"(map), "r"(tp_smem(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tp_tma_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z,
                                          int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(tp_smem(dst)), "l"(map), "r"(tp_smem(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
// K-major operand tile: rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t tp_desc_kmajor(const void* tile) {
  uint64_t d = (uint64_t)((tp_smem(tile) & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// MN-major operand tile (V as B: N = head dim, K = keys): a row of 128 bytes holds 64 neighbouring N elements
// of one key; 8-key groups 1024 bytes apart (stride offset); the next 64 N elements `lbo_bytes` further
__device__ __forceinline__ uint64_t tp_desc_mnmajor(const void* tile, uint32_t lbo_bytes) {
  uint64_t d = (uint64_t)((tp_smem(tile) & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo_bytes >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// both operands from shared memory
__device__ __forceinline__ void tp_mma_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the A operand from tensor memory (row m in lane m, two bfloat16 per 32-bit column)
__device__ __forceinline__ void tp_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tp_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tp_smem(bar))
               : "memory");
}
// 32 columns of this thread's lane, no wait (the caller waits once for all loads in flight)
__device__ __forceinline__ void tp_tmem_ld32_nowait(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
// 8 columns at a time (the rescaling of O: a rare path that must not cost the common one its registers)
__device__ __forceinline__ void tp_tmem_ld8_nowait(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}
__device__ __forceinline__ void tp_tmem_st8_nowait(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tp_tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tp_tmem_st32_nowait(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,"
      "%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
      "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
      "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tp_tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float tp_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float tp_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// two floats to packed bfloat16 (round to nearest even): `lo` in the low half
__device__ __forceinline__ uint32_t tp_pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

struct TpParams {
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

__global__ void __launch_bounds__(TP_THREADS, 1)
prefill_attention_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                              const __grid_constant__ CUtensorMap map_v, const TpParams p) {
  // No static shared memory: the tiles need a 1024-byte boundary (128-byte swizzle), and the dynamic region of a
  // block without static shared memory starts on one.  If it ever did not, the block says so and leaves.
  extern __shared__ __align__(16) unsigned char tp_raw[];
  pdl_launch_dependents();
  if ((tp_smem(tp_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 20, (int)(tp_smem(tp_raw) & 1023u));
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(tp_raw + TP_TILES_BYTES);
  uint64_t& q_full = bars[0];
  uint64_t& k0_full = bars[1];                  // the first K tile has landed
  uint64_t* full = bars + 2;                    // [2] the pair (V_j, K_{j+1}) has landed in pair slot j & 1
  uint64_t* empty = bars + 4;                   // [2] the products that read the pair are done
  uint64_t* s_full = bars + 6;                  // [2] scores of query tile i are in tensor memory
  uint64_t* p_ready = bars + 8;                 // [2] P of query tile i is in tensor memory (one arrival per warp)
  uint64_t* pv_done = bars + 10;                // [2] the LAST P.V product of query tile i is done
  uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bars + 12);
  unsigned char* q_s = tp_raw;                  // query tile i at i * TP_TILE_Q
  unsigned char* k0_s = tp_raw + 2 * TP_TILE_Q;          // K tile 0
  unsigned char* pair_s = k0_s + TP_TILE_KV;             // pair slot s: V at s * 2 * TP_TILE_KV, K right behind it
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // A 1-D grid, numbered so that consecutive blocks are the same token block of all kv heads: the block
  // scheduler then starts the heaviest blocks of EVERY head first (longest work first keeps the SMs level).
  const int kh = (int)(blockIdx.x % p.num_kv);
  const int G = p.num_q / p.num_kv;
  const int tpt = TP_ROWS / G;  // tokens of a query tile
  const int tpb = 2 * tpt;      // tokens of a block
  pdl_wait();

  // ---- which request and which of its token blocks (numbered from the back: heavy blocks first) ---------
  const int block_id = (int)(gridDim.x / p.num_kv) - 1 - (int)(blockIdx.x / p.num_kv);
  int r = -1, first = 0, q_len = 0, q_begin = 0;
  {
    int running = 0;
    for (int i = 0; i < p.num_requests; ++i) {
      const int b = p.cu_q[i], n = p.cu_q[i + 1] - b;
      const int nb = (n + tpb - 1) / tpb;
      if (block_id < running + nb) {
        r = i;
        first = (block_id - running) * tpb;
        q_len = n;
        q_begin = b;
        break;
      }
      running += nb;
    }
  }
  if (r < 0) return;
  const int kvl = p.kv_len[r];
  const int ntok_all = min(tpb, q_len - first);
  const int ntok0 = min(tpt, ntok_all), ntok1 = ntok_all - ntok0;
  const int p0 = kvl - q_len + first;  // position of the block's first token
  if (kvl <= 0 || p0 < 0) {
    for (int i = tid; i < ntok_all * G * TP_D; i += blockDim.x) {
      const int row = i / TP_D, d = i - row * TP_D;
      p.out[((long long)(q_begin + first + row / G) * p.num_q + kh * G + row % G) * TP_D + d] = __float2bfloat16_rn(0.f);
    }
    return;
  }
  const int key_lo = p.window > 0 ? max(0, p0 - p.window + 1) : 0;
  const int k_start = key_lo / TP_KEYS * TP_KEYS;
  // key tiles each query tile walks (tile 1 sees later keys: tiles1 >= tiles0 when it has rows)
  const int tiles0 = (p0 + ntok0 - 1 - k_start) / TP_KEYS + 1;
  const int tiles1 = ntok1 > 0 ? (p0 + ntok_all - 1 - k_start) / TP_KEYS + 1 : 0;
  const int tiles = max(tiles0, tiles1);
  const int* bt = p.block_table + (long long)p.req_slots[r] * p.max_pages;
  const int pages_per_tile = TP_KEYS / p.page_size;

  if (tid == 0) {
    tp_mbar_init(&q_full, 1);
    tp_mbar_init(&k0_full, 1);
    for (int s = 0; s < 2; ++s) {
      tp_mbar_init(&full[s], 1);
      tp_mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tp_mbar_init(&s_full[i], 1);
      tp_mbar_init(&p_ready[i], 4);  // one arrival per warp of the group
      tp_mbar_init(&pv_done[i], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tp_smem(&tmem_slot)),
                 "r"(TP_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_slot;
  // columns: S_0 0..127 (P_0 in 0..63), S_1 128..255 (P_1 in 128..191), O_0 256..383, O_1 384..511

  if (warp == 8) {
    // ---- producer: the warp reads page ids (one coalesced load per key tile, a tile ahead of their use);
    // lane pg issues the loads of the tile's page pg -----------------------------------------------------------
    if (lane == 0) {
      tp_mbar_expect_tx(&q_full, 2 * TP_TILE_Q);
      for (int i = 0; i < 2; ++i) {
        tp_tma_3d(q_s + i * TP_TILE_Q, &map_q, &q_full, 0, kh * G, q_begin + first + i * tpt);
        tp_tma_3d(q_s + i * TP_TILE_Q + TP_TILE_Q / 2, &map_q, &q_full, 64, kh * G, q_begin + first + i * tpt);
      }
    }
    auto page_of = [&](int t) -> int {  // lane pg: the page that holds the pg-th page of key tile t
      const int key = k_start + t * TP_KEYS + lane * p.page_size;
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
    // K tile 0, then the pairs (V_j, K_{j+1}): what step j of the MMA thread reads
    int pages_now = page_of(0);
    int pages_next = tiles > 1 ? page_of(1) : -1;
    auto load_tile = [&](unsigned char* dst, const CUtensorMap* map, uint64_t* bar, int page) {
      // a page that is not there (-1) is out of the map's range: the box is filled with zeros
      if (lane < pages_per_tile) {
        const int pcoord = page >= 0 ? page : (int)p.num_pages;
        unsigned char* d = dst + lane * p.page_size * 128;
        tp_tma_4d(d, map, bar, 0, kh, 0, pcoord);
        tp_tma_4d(d + TP_TILE_KV / 2, map, bar, 64, kh, 0, pcoord);
      }
    };
    if (lane == 0) tp_mbar_expect_tx(&k0_full, TP_TILE_KV);
    __syncwarp();
    load_tile(k0_s, &map_k, &k0_full, pages_now);
    bool ok = true;
    for (int t = 0; t < tiles && ok; ++t) {
      const int s = t & 1;
      const bool has_k = t + 1 < tiles;
      const int pages_after = t + 2 < tiles ? page_of(t + 2) : -1;  // in flight while this pair's slot is awaited
      if (lane == 0 && !tp_mbar_wait(&empty[s], ((t >> 1) & 1) ^ 1)) {
        ullm_report(p.status, ULLM_STATUS_TIMEOUT, 21, t);
        ok = false;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane == 0) tp_mbar_expect_tx(&full[s], has_k ? 2 * TP_TILE_KV : TP_TILE_KV);
      __syncwarp();
      unsigned char* dst = pair_s + s * 2 * TP_TILE_KV;
      load_tile(dst, &map_v, &full[s], pages_now);
      if (has_k) load_tile(dst + TP_TILE_KV, &map_k, &full[s], pages_next);
      pages_now = pages_next;
      pages_next = pages_after;
    }
  } else if (warp == 9) {
    if (lane == 0) {
      // ---- MMA issuer -----------------------------------------------------------------------------------
      // S: M 128, N 128, both operands K-major.  O: M 128, N 128, A (P) from tensor memory, B (V) MN-major.
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TP_KEYS >> 3) << 17) |
                               ((uint32_t)(TP_ROWS >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(TP_D >> 3) << 17) |
                               ((uint32_t)(TP_ROWS >> 4) << 24);
      bool ok = tp_mbar_wait(&q_full, 0);
      if (!ok) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 22, 0);
      // This one thread's instruction stream paces the tensor pipe, so everything is kept to adds: descriptors as
      // their 32-bit halves (the high word is the same for all of them: 8-row groups 1024 bytes apart, version 1,
      // 128-byte swizzle; the low word holds the start address in 16-byte units and the leading-dimension field),
      // ring slots and parities stepped, not divided.
      const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
      const uint32_t k0_lo = ((tp_smem(k0_s) & 0x3FFFF) >> 4) | (1u << 16);
      const uint32_t pair_lo = (tp_smem(pair_s) & 0x3FFFF) >> 4;
      const uint32_t q_lo[2] = {((tp_smem(q_s) & 0x3FFFF) >> 4) | (1u << 16),
                                ((tp_smem(q_s + TP_TILE_Q) & 0x3FFFF) >> 4) | (1u << 16)};
      auto mma_ss = [&](uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t acc) {
        asm volatile(
            "{\n .reg .b64 da, db;\n .reg .pred p;\n mov.b64 da, {%1, %3};\n mov.b64 db, {%2, %3};\n"
            " setp.ne.b32 p, %5, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n}\n"
            ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc_s), "r"(acc)
            : "memory");
      };
      auto mma_ts = [&](uint32_t d, uint32_t a_tmem, uint32_t b_lo, uint32_t acc) {
        asm volatile(
            "{\n .reg .b64 db;\n .reg .pred p;\n mov.b64 db, {%2, %3};\n"
            " setp.ne.b32 p, %5, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n}\n"
            ::"r"(d), "r"(a_tmem), "r"(b_lo), "r"(desc_hi), "r"(idesc_o), "r"(acc)
            : "memory");
      };
      // scores of query tile i from the K tile whose descriptor low word is `b0`
      auto scores = [&](int i, uint32_t b0) {
#pragma unroll
        for (int kk = 0; kk < TP_D / 16; ++kk) {
          // d = 16 kk: half kk / 4 of the Q and K tiles (16 KB = 1024 units further), 32 bytes per step inside a half
          const uint32_t off = (kk >> 2) * ((TP_TILE_KV / 2) >> 4) + 2 * (kk & 3);
          mma_ss(tmem + i * TP_KEYS, q_lo[i] + off, b0 + off, kk > 0 ? 1u : 0u);
        }
        tp_commit(&s_full[i]);
      };
      // O_i += P_i V from the V tile at `v_lo` (16-byte units)
      auto p_times_v = [&](int i, int j, uint32_t v_lo) {
        // MN-major: the leading-dimension field is the distance of the two 64-column halves
        const uint32_t b0 = v_lo | ((uint32_t)((TP_TILE_KV / 2) >> 4) << 16);
#pragma unroll
        for (int ks = 0; ks < TP_KEYS / 16; ++ks)  // 16 keys: 8 columns of P; two 8-key groups = 2048 bytes down the V tile
          mma_ts(tmem + 2 * TP_KEYS + i * TP_D, tmem + i * TP_KEYS + ks * 8, b0 + ks * (2048 >> 4),
                 (j > 0 || ks > 0) ? 1u : 0u);
      };
      if (ok && !tp_mbar_wait(&k0_full, 0)) {
        ullm_report(p.status, ULLM_STATUS_TIMEOUT, 23, 0);
        ok = false;
      }
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        scores(0, k0_lo);
        if (tiles1 > 0) scores(1, k0_lo);
      }
      for (int j = 0; j < tiles && ok; ++j) {
        // the pair (V_j, K_{j+1}): all this step reads.  (The commits behind the score products also cover the
        // P.V products issued before them, so the softmax warps need no signal of their own for those.)
        if (!tp_mbar_wait(&full[j & 1], (j >> 1) & 1)) {
          ullm_report(p.status, ULLM_STATUS_TIMEOUT, 24, j);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t v_lo = pair_lo + (j & 1) * ((2 * TP_TILE_KV) >> 4);
        const uint32_t k_lo = (v_lo + (TP_TILE_KV >> 4)) | (1u << 16);
        for (int i = 0; i < 2 && ok; ++i) {
          const int tiles_i = i == 0 ? tiles0 : tiles1;
          if (j < tiles_i) {
            if (!tp_mbar_spin(&p_ready[i], j & 1)) {
              ullm_report(p.status, ULLM_STATUS_TIMEOUT, 26 + i, j);
              ok = false;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            p_times_v(i, j, v_lo);
            if (j + 1 == tiles_i) tp_commit(&pv_done[i]);
          }
          if (j + 1 < tiles_i) scores(i, k_lo);
        }
        if (!ok) break;
        tp_commit(&empty[j & 1]);  // every product that reads the pair has been issued
      }
    }
  } else {
    // ---- softmax: warp group i owns query tile i; thread `row` of the group owns row `row` (tensor-memory
    // lane `row`) -------------------------------------------------------------------------------------------------
    const int i = warp >> 2;
    const int row = tid & 127;
    const int ntok_i = i == 0 ? ntok0 : ntok1;
    const int tiles_i = i == 0 ? tiles0 : tiles1;
    const int rows_valid = ntok_i * G;
    const bool row_ok = row < rows_valid;
    const int pf = p0 + i * tpt;                 // position of the tile's first token
    const int pl = pf + ntok_i - 1;              // and of its last
    const int pos = row_ok ? pf + row / G : -1;
    const int lo = p.window > 0 ? pos - p.window + 1 : 0;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tmem_s = tmem + i * TP_KEYS + lane_base;
    const uint32_t tmem_o = tmem + 2 * TP_KEYS + i * TP_D + lane_base;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < tiles_i && ok; ++j) {
      const int key0 = k_start + j * TP_KEYS;
      if (!tp_mbar_wait(&s_full[i], j & 1)) {
        if (lane == 0) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 28 + i, j);
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t sr[TP_KEYS];
#pragma unroll
      for (int c = 0; c < TP_KEYS / 32; ++c) tp_tmem_ld32_nowait(tmem_s + c * 32, sr + c * 32);
      tp_tmem_ld_wait();
      const bool need_mask = rows_valid < TP_ROWS || key0 + TP_KEYS - 1 > pf || (p.window > 0 && key0 < pl - p.window + 1);
      if (need_mask) {
#pragma unroll
        for (int k = 0; k < TP_KEYS; ++k) {
          const int key = key0 + k;
          if (!(key <= pos && key >= lo)) sr[k] = 0xff800000u;  // -inf
        }
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int k = 0; k < TP_KEYS / 2; ++k)
        mx[k & 3] = tp_max3(mx[k & 3], __uint_as_float(sr[2 * k]), __uint_as_float(sr[2 * k + 1]));
      const float row_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      // The reference point of the exponents only moves when the row's maximum grows by more than 2^8:
      // until then P is at most 256 (exact in bf16 range, sums in 32-bit), and O and l, which share the
      // reference, need no rescaling.  The result O / l does not depend on the reference.
      const float m_cand = fmaxf(m, row_max * p.scale_log2);
      const float m_new = (m == -INFINITY || m_cand - m > 8.f) ? m_cand : m;
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = m == -INFINITY ? 1.f : tp_ex2(m - m_use);  // (no key seen yet: O and l are still zero)
      m = m_new;
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
      const float neg_m = -m_use;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t pk[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          const float a = tp_ex2(fmaf(__uint_as_float(sr[h * 64 + 2 * k]), p.scale_log2, neg_m));
          const float b = tp_ex2(fmaf(__uint_as_float(sr[h * 64 + 2 * k + 1]), p.scale_log2, neg_m));
          sum[(2 * k) & 3] += a;
          sum[(2 * k + 1) & 3] += b;
          pk[k] = tp_pack_bf16(a, b);
        }
        tp_tmem_st32_nowait(tmem_s + h * 32, pk);  // keys 64 h .. 64 h + 63 of this row
      }
      l = l * alpha + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
      // the last key tile may hold slots past the request's length: whatever they contain must not reach O.
      // The first warp group that works on this tile clears them (its P.V product is issued first).
      if (key0 + TP_KEYS > kvl && (i == 0 || j >= tiles0)) {
        if (!tp_mbar_wait(&full[j & 1], (j >> 1) & 1)) {
          if (lane == 0) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 30 + i, j);
          ok = false;
        } else {
          unsigned char* v_t = pair_s + (j & 1) * 2 * TP_TILE_KV;
          const int first_bad = max(0, kvl - key0);
          for (int x = row; x < (TP_KEYS - first_bad) * 16; x += 128) {
            const int key = first_bad + x / 16, ch = x % 16;  // 16 chunks of 16 bytes per key: 8 per half
            *reinterpret_cast<uint4*>(v_t + (ch >> 3) * (TP_TILE_KV / 2) + key * 128 + (ch & 7) * 16) = make_uint4(0, 0, 0, 0);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
      }
      if (ok && j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        // O shares the reference point.  P.V of the tile before is in it: this tile's scores were issued behind
        // that product, and their completion was awaited above.  Rescale this warp's rows.
#pragma unroll 1
        for (int c = 0; c < TP_D / 8; ++c) {
          uint32_t v[8];
          tp_tmem_ld8_nowait(tmem_o + c * 8, v);
          tp_tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 8; ++k) v[k] = __float_as_uint(__uint_as_float(v[k]) * alpha);
          tp_tmem_st8_nowait(tmem_o + c * 8, v);
        }
      }
      tp_tmem_st_wait();
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) tp_mbar_arrive(&p_ready[i]);  // (also after a failed wait: the MMA thread is not left waiting for this tile)
    }
    if (tiles_i > 0) {
      if (ok && !tp_mbar_wait(&pv_done[i], 0)) {
        if (lane == 0) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 34 + i, tiles_i);
        ok = false;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* op = p.out + ((long long)(q_begin + first + i * tpt + row / G) * p.num_q + kh * G + row % G) * TP_D;
#pragma unroll
      for (int c = 0; c < TP_D / 32; ++c) {
        uint32_t v[32];
        tp_tmem_ld32_nowait(tmem_o + c * 32, v);  // all lanes of the warp take part
        tp_tmem_ld_wait();
        if (row_ok && ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 chunk;
            chunk.x = tp_pack_bf16(__uint_as_float(v[q * 8 + 0]) * inv, __uint_as_float(v[q * 8 + 1]) * inv);
            chunk.y = tp_pack_bf16(__uint_as_float(v[q * 8 + 2]) * inv, __uint_as_float(v[q * 8 + 3]) * inv);
            chunk.z = tp_pack_bf16(__uint_as_float(v[q * 8 + 4]) * inv, __uint_as_float(v[q * 8 + 5]) * inv);
            chunk.w = tp_pack_bf16(__uint_as_float(v[q * 8 + 6]) * inv, __uint_as_float(v[q * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(op + c * 32 + q * 8) = chunk;
          }
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncwarp();  // the lanes of the single-thread role wait here for their lane 0 (the barrier counts warps)
  __syncthreads();
  if (warp == 9) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TP_TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
struct TpKey {
  const void* ptr;
  long long a, b, c;
  bool operator==(const TpKey& o) const { return ptr == o.ptr && a == o.a && b == o.b && c == o.c; }
};
struct TpKeyHash {
  size_t operator()(const TpKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.a) * 31) ^ (std::hash<long long>()(k.b) * 131) ^
           (std::hash<long long>()(k.c) * 8191);
  }
};
static std::unordered_map<TpKey, CUtensorMap, TpKeyHash> g_tp_maps;
static std::mutex g_tp_mutex;

// Q: the projection buffer [tokens, heads_total, 128]; a box gathers 64 columns x G heads x 128 / G tokens
static bool tp_map_q(const void* q, long long tokens, long long row_stride_elems, int heads_total, int G,
                     CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_tp_mutex);
  TpKey key{q, tokens, row_stride_elems, (long long)heads_total * 1000 + G};
  auto it = g_tp_maps.find(key);
  if (it != g_tp_maps.end()) {
    *out = it->second;
    return true;
  }
  UllmTmaEncodeFn enc = ullm_tma_encode();
  if (enc == nullptr) return false;
  cuuint64_t dims[3] = {TP_D, (cuuint64_t)heads_total, (cuuint64_t)tokens};
  cuuint64_t strides[2] = {TP_D * 2, (cuuint64_t)row_stride_elems * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(TP_ROWS / G)};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMap m;
  if (enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (g_tp_maps.size() > 4096) g_tp_maps.clear();
  g_tp_maps[key] = m;
  *out = m;
  return true;
}

// bfloat16, head size 128, a power-of-two number (<= 16) of query heads per kv head, pages of 8 to 128 tokens
extern "C" int ullm_prefill_attention_pair_supported(int head_dim, int num_q, int num_kv, int page_size) {
  if (num_kv <= 0 || num_q % num_kv) return 0;
  const int G = num_q / num_kv;
  if (head_dim != TP_D || G > 16 || (G & (G - 1))) return 0;
  return page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128;
}

static int g_tp_attr_set = 0;
extern "C" int ullm_prefill_attention_pair(const void* q, long long q_row_stride, void* out, const void* k_cache,
                                           const void* v_cache, const int* block_table, int max_pages,
                                           const int* req_slots, const int* cu_q, const int* kv_len, int tokens,
                                           int num_requests, int num_q, int num_kv, int head_dim, int page_size,
                                           int window, float scale, long long num_pages, int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || num_requests <= 0 || max_pages <= 0 || window < 0) return ULLM_ERR_BAD_SIZE;
  if (!ullm_prefill_attention_pair_supported(head_dim, num_q, num_kv, page_size)) return ULLM_ERR_UNSUPPORTED;
  if (q_row_stride % 8 || ((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) % 16)
    return ULLM_ERR_UNSUPPORTED;
  if (q_row_stride % TP_D) return ULLM_ERR_UNSUPPORTED;
  if (tokens == 0) return ULLM_OK;
  const int G = num_q / num_kv;
  CUtensorMap mq, mk, mv;
  if (!tp_map_q(q, tokens, q_row_stride, (int)(q_row_stride / TP_D), G, &mq) ||
      !ullm_tma_map_kv(k_cache, num_pages, page_size, num_kv, TP_D, page_size, &mk) ||
      !ullm_tma_map_kv(v_cache, num_pages, page_size, num_kv, TP_D, page_size, &mv))
    return ULLM_ERR_LAUNCH;
  if (!g_tp_attr_set) {
    if (cudaFuncSetAttribute(prefill_attention_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_SMEM) !=
        cudaSuccess)
      return ULLM_ERR_LAUNCH;
    g_tp_attr_set = 1;
  }
  TpParams p;
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
  const int tpb = 2 * (TP_ROWS / G);
  dim3 grid(((tokens + tpb - 1) / tpb + num_requests) * num_kv);
  return ullm_launch_kernel(prefill_attention_pair_kernel, grid, dim3(TP_THREADS), (size_t)TP_SMEM, st, mq, mk, mv, p);
}
