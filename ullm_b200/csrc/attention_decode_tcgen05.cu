// Paged decode attention for bfloat16 on the 5th-generation tensor cores (head size 128): one new token per
// request, the keys of the whole batch cut evenly over the blocks.
//
// The unit of work is a tile of 128 keys of one (request, kv head) pair.  The tiles of all pairs, in pair order,
// form one list that is cut into equal contiguous ranges, one per block, one block per SM (the grid never depends
// on the lengths).  With one query token there are only `group` (query heads per kv head) rows of Q, far fewer
// than a tensor-core tile is tall, so the products are taken transposed: the KEYS are the 128 rows.
//
//   S^T[128 keys x 16] = K[128 x 128] Q^T      tcgen05.mma M=128 N=16, K tile and Q both K-major from shared
//                                              memory, accumulator in tensor memory; column c is query head c
//   P^T               = 2^(S^T scale - m)      four softmax warps, thread = key (tensor-memory lane); the maximum
//                                              of a column is a reduction over the 128 threads
//   O^T[128 dims x 16] += V^T[128 x 128] P^T   V as the MN-major A operand (the cache's [key][dim] rows as they
//                                              are), P^T (bf16) through shared memory as the K-major B operand;
//                                              O^T stays in tensor memory, thread = output dimension
//
// K and V come in by TMA page by page (4-D boxes of one head's tokens of a page, 128-byte swizzle) into a ring
// of three 64 KB stages; Q rides with every tile (1 KB).  One thread issues the loads' bookkeeping (all lanes of
// its warp ask for a box each), one thread the MMAs; mbarriers carry "tile landed", "scores ready", "P ready",
// "P.V done / stage free".  A pair that lies whole inside a block's range is finished by the block; a pair that
// the range cuts leaves its part (max, sum, unnormalised output) in the scratch array for the merge kernel of
// decode_merge.cuh.  Keys outside a request's visible range are masked and their V rows zeroed in shared memory.
//
// Every wait on an mbarrier is bounded; a wait that runs out records ULLM_STATUS_TIMEOUT, the block stops
// waiting (all softmax threads leave together), frees its tensor memory and returns.
#include "decode_merge.cuh"
#include "tcgen05_util.cuh"
#include "tma_host.cuh"

#define DTC_KEYS 128
#define DTC_D 128
#define DTC_THREADS 192
#define DTC_STAGES 3
#define DTC_HALF (DTC_KEYS * 128)        // 16 KB: 128 rows x 64 elements of K or V
#define DTC_KV (2 * DTC_HALF)            // 32 KB
#define DTC_QP 4096                      // Q (or P^T) operand: two halves of [16 rows x 128 B]
#define DTC_STAGE_BYTES (2 * DTC_KV + DTC_QP)
#define DTC_SMEM (DTC_STAGES * DTC_STAGE_BYTES + 2 * DTC_QP + 1024)  // two P^T buffers behind the ring
#define DTC_MAX_BATCH 512
#define DTC_TMEM_COLS 128                // S^T buffers at columns 0 and 32, O^T at 64

__device__ __forceinline__ void dtc_tma_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(lin_smem(dst)), "l"(map), "r"(lin_smem(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
// MN-major operand tile (V^T as A: M = head dim, K = keys): a row of 128 bytes holds 64 neighbouring M elements
// of one key; 8-key groups 1024 bytes apart (stride offset); the next 64 M elements `lbo_bytes` further
__device__ __forceinline__ uint64_t dtc_desc_mnmajor(const void* tile, uint32_t lbo_bytes) {
  uint64_t d = (uint64_t)((lin_smem(tile) & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo_bytes >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// N consecutive columns of this thread's tensor-memory lane
template <int N>
__device__ __forceinline__ void dtc_tmem_ld(uint32_t taddr, float (&v)[N]) {
  static_assert(N == 4 || N == 8 || N == 16, "column counts of the loads written out here");
  uint32_t r[N];
  if constexpr (N == 4) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr));
  } else if constexpr (N == 8) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
  } else {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
  }
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = __uint_as_float(r[i]);
}
template <int N>
__device__ __forceinline__ void dtc_tmem_st(uint32_t taddr, const float (&v)[N]) {
  static_assert(N == 4 || N == 8 || N == 16, "column counts of the stores written out here");
  if constexpr (N == 4) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr), "r"(__float_as_uint(v[0])),
                 "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3]))
                 : "memory");
  } else if constexpr (N == 8) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr),
                 "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
                 "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
                 "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7]))
                 : "memory");
  } else {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
        : "memory");
  }
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float dtc_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// the 128 softmax threads meet (the two single-thread warps are not part of it)
__device__ __forceinline__ void dtc_softmax_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

struct DtcParams {
  const int* block_table;
  int max_pages;
  const int* req_slots;
  const int* kv_len;
  __nv_bfloat16* out;
  float* part;    // [ranges][2][group][D + 4]: unnormalised output, max, sum
  int* prefix;    // [batch + 1]: tiles of the requests before each (per kv head)
  int* flags;     // [batch * num_kv], zero between launches: set for a pair that was cut, cleared by the merge
  int batch, num_q, num_kv, page_size, page_shift, window;
  float scale_log2;
  long long num_pages;
  int* status;
};

// Where a role stands in the list of tiles.
struct DtcCursor {
  int b, kh;
  int tile, tiles;  // tile inside the pair, tiles of the pair
  int first;        // absolute index of the pair's tile 0 (a tile holds the keys 128 i .. 128 i + 127)
  int lo, end;      // the request's visible keys [lo, end)
};

// GP: columns of a tensor-memory load that hold the group's query heads (4, 8 or 16 >= group)
template <int GP>
__global__ void __launch_bounds__(DTC_THREADS, 1)
decode_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                const __grid_constant__ CUtensorMap map_v, const DtcParams p) {
  extern __shared__ unsigned char dtc_raw[];
  __shared__ int s_pre[DTC_MAX_BATCH + 1], s_lo[DTC_MAX_BATCH], s_end[DTC_MAX_BATCH], s_slot[DTC_MAX_BATCH];
  __shared__ __align__(8) uint64_t kv_full[DTC_STAGES], kv_empty[DTC_STAGES], s_full[2], p_ready, pv_done[2];
  __shared__ uint32_t tmem_slot;
  __shared__ float s_red[2][4][GP], s_lsum[4][GP];
  __shared__ int s_abort;
  pdl_launch_dependents();
  pdl_wait();
  unsigned char* smem = (unsigned char*)(((uintptr_t)dtc_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* p_s = smem + DTC_STAGES * DTC_STAGE_BYTES;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = p.num_q / p.num_kv;

  // ---- prologue: every request's visible keys, tiles and their running sum ---------------------------
  for (int b = tid; b < p.batch; b += blockDim.x) {
    const int pos = p.kv_len[b] - 1;
    const int lo = (p.window > 0 && pos >= 0) ? max(0, pos - p.window + 1) : 0;
    const int n = pos >= 0 ? pos - lo + 1 : 0;
    s_lo[b] = lo;
    s_end[b] = lo + n;
    s_slot[b] = p.req_slots[b];
    s_pre[b + 1] = n > 0 ? (lo + n + DTC_KEYS - 1) / DTC_KEYS - lo / DTC_KEYS : 0;
  }
  if (tid == 0) {
    for (int s = 0; s < DTC_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(&p_ready, 4);  // lane 0 of each softmax warp
    mbar_init(&pv_done[0], 1);
    mbar_init(&pv_done[1], 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  if (tid == 0) {
    s_pre[0] = 0;
    for (int b = 0; b < p.batch; ++b) s_pre[b + 1] += s_pre[b];
  }
  __syncthreads();
  if (blockIdx.x == 0)
    for (int b = tid; b <= p.batch; b += blockDim.x) p.prefix[b] = s_pre[b];
  // rows of requests that hold nothing (padding of a captured batch) are zero
  for (long long b = blockIdx.x; b < p.batch; b += gridDim.x) {
    if (s_pre[b + 1] == s_pre[b]) {
      __nv_bfloat16* o = p.out + b * p.num_q * DTC_D;
      for (int i = tid; i < p.num_q * DTC_D; i += blockDim.x) o[i] = __float2bfloat16_rn(0.f);
    }
  }
  const long long W = (long long)p.num_kv * s_pre[p.batch];
  const long long GW = decb_ranges(W, (long long)gridDim.x, 1);
  const long long gw = blockIdx.x;
  if (gw >= GW || W == 0) return;  // the whole block: nothing was allocated yet
  const long long u0 = gw * W / GW, u1 = (gw + 1) * W / GW;
  if (u0 >= u1) return;
  const int n_tiles = (int)(u1 - u0);

  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(lin_smem(&tmem_slot)),
                 "r"(DTC_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_s = tmem_slot;       // two score buffers, 32 columns apart (tile i uses i & 1)
  const uint32_t tmem_o = tmem_slot + 64;  // the output accumulator

  auto set_pair = [&](DtcCursor& c) {
    c.tiles = s_pre[c.b + 1] - s_pre[c.b];
    c.lo = s_lo[c.b];
    c.end = s_end[c.b];
    c.first = c.lo / DTC_KEYS;
  };
  auto advance = [&](DtcCursor& c) {  // to the next tile of the list (callers stop at the range's end)
    if (++c.tile < c.tiles) return;
    c.tile = 0;
    if (++c.kh == p.num_kv) {
      c.kh = 0;
      do ++c.b; while (c.b < p.batch - 1 && s_pre[c.b + 1] == s_pre[c.b]);
      if (c.b >= p.batch) c.b = p.batch - 1;
      set_pair(c);
    }
  };
  DtcCursor cur;
  {  // the request that tile u0 belongs to: the first b whose tiles end beyond u0
    int lo_b = 0, hi_b = p.batch - 1;
    while (lo_b < hi_b) {
      const int mid = (lo_b + hi_b) >> 1;
      if ((long long)p.num_kv * s_pre[mid + 1] > u0) hi_b = mid;
      else lo_b = mid + 1;
    }
    cur.b = lo_b;
    set_pair(cur);
    const long long rem = u0 - (long long)p.num_kv * s_pre[cur.b];
    cur.kh = (int)(rem / cur.tiles);
    cur.tile = (int)(rem % cur.tiles);
  }

  if (warp == 4) {
    // ---- producer: the warp reads the tile's page ids (one per lane, a tile ahead of their use), every lane
    // asks for boxes; lane 0 keeps the barriers ------------------------------------------------------------
    const int sh = p.page_shift, ps = p.page_size;
    const int ppt = DTC_KEYS >> sh;  // pages of a tile
    auto pages_of = [&](const DtcCursor& c) -> int {
      const int base = (c.first + c.tile) * DTC_KEYS;
      const int k0 = base + lane * ps;
      int page = -1;
      if (lane < ppt && k0 < c.end && k0 + ps > c.lo) {
        page = p.block_table[(long long)s_slot[c.b] * p.max_pages + (k0 >> sh)];
        if (page < 0 || page >= p.num_pages) {  // a page with visible keys must be there
          ullm_report(p.status, ULLM_STATUS_PAGE, c.b, page);
          page = -1;
        }
      }
      return page;
    };
    int pages_next = pages_of(cur);
    DtcCursor nxt = cur;
    bool ok = true;
    for (int i = 0; i < n_tiles && ok; ++i) {
      const int s = i % DTC_STAGES;
      const int pages_now = pages_next;
      const DtcCursor c = nxt;
      if (i + 1 < n_tiles) {
        advance(nxt);
        pages_next = pages_of(nxt);  // in flight while this tile's stage is awaited
      }
      if (lane == 0 && !mbar_wait(&kv_empty[s], ((i / DTC_STAGES) & 1) ^ 1)) {
        ullm_report(p.status, ULLM_STATUS_TIMEOUT, 30, i);
        ok = false;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      unsigned char* st = smem + s * DTC_STAGE_BYTES;
      if (lane == 0) {
        mbar_expect_tx(&kv_full[s], 2 * DTC_KV + 2 * (uint32_t)group * 128);
        // Q of the pair: `group` rows of 128 bytes per half, behind K and V
        tma_load_3d(st + 2 * DTC_KV, &map_q, &kv_full[s], 0, c.kh * group, c.b);
        tma_load_3d(st + 2 * DTC_KV + DTC_QP / 2, &map_q, &kv_full[s], 64, c.kh * group, c.b);
      }
      __syncwarp();
      // box = (page of the tile, K or V, half): all of them, a missing page as a coordinate beyond the pool
      // (the box is then filled with zeros and counts its bytes all the same)
      for (int b0 = 0; b0 < ppt * 4; b0 += 32) {
        const int box = b0 + lane, pg = box >> 2, kind = box & 3;
        const int page = __shfl_sync(0xffffffffu, pages_now, pg & 31);
        if (box < ppt * 4) {
          const int pcoord = page >= 0 ? page : (int)p.num_pages;
          dtc_tma_4d(st + (kind >> 1) * DTC_KV + (kind & 1) * DTC_HALF + pg * ps * 128, kind < 2 ? &map_k : &map_v,
                     &kv_full[s], (kind & 1) * 64, c.kh, 0, pcoord);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // ---- MMA issuer ---------------------------------------------------------------------------------------
      // S^T: M 128 (keys), N 16, both K-major.  O^T: M 128 (dims), N 16, A (V^T) MN-major, B (P^T) K-major.
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(16 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_o = idesc_s | (1u << 15);
      // K-major and MN-major descriptors differ in the low word only (the leading offset): one high word
      const uint64_t desc0 = umma_desc(smem);
      const uint32_t desc_hi = (uint32_t)(desc0 >> 32), kdesc_lo = (uint32_t)desc0;
      const uint32_t vdesc_lo = (uint32_t)dtc_desc_mnmajor(smem + DTC_KV, DTC_HALF), pdesc_lo = (uint32_t)umma_desc(p_s);
      bool ok = true;
      auto issue_scores = [&](int i) -> bool {
        const int s = i % DTC_STAGES;
        if (!mbar_wait(&kv_full[s], (i / DTC_STAGES) & 1)) {
          ullm_report(p.status, ULLM_STATUS_TIMEOUT, 31, i);
          return false;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // descriptors by their low words (address in 16-byte units): K at the stage's base, Q behind K and V
        const uint32_t k_lo = kdesc_lo + (uint32_t)s * (DTC_STAGE_BYTES >> 4), q_lo = k_lo + ((2 * DTC_KV) >> 4);
        const uint32_t d = tmem_s + (i & 1) * 32;
        // d = 16 kk: half kk / 4 of the K and Q tiles, 32 bytes further per step inside a half
        umma_bf16_lo<-1>(d, k_lo, q_lo, desc_hi, idesc_s, 0u);
#pragma unroll
        for (int kk = 1; kk < DTC_D / 16; ++kk)
          umma_bf16_lo<1>(d, k_lo + (kk >> 2) * (DTC_HALF >> 4) + 2 * (kk & 3),
                          q_lo + (kk >> 2) * ((DTC_QP / 2) >> 4) + 2 * (kk & 3), desc_hi, idesc_s);
        umma_commit(&s_full[i & 1]);
        return true;
      };
      ok = issue_scores(0);
      DtcCursor c = cur;
      bool share_start = true;  // the tile is the first of this block's share of its pair
      for (int i = 0; i < n_tiles && ok; ++i) {
        // The next tile's scores go in front of this tile's P.V when that tile has landed (it has, once the ring
        // runs ahead): the softmax warps then find them ready and work while P.V runs.
        const bool early = i + 1 < n_tiles && mbar_try_wait(&kv_full[(i + 1) % DTC_STAGES], ((i + 1) / DTC_STAGES) & 1);
        if (early && !issue_scores(i + 1)) break;
        if (!mbar_wait(&p_ready, i & 1)) {
          ullm_report(p.status, ULLM_STATUS_TIMEOUT, 32, i);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t v_lo = vdesc_lo + (uint32_t)(i % DTC_STAGES) * (DTC_STAGE_BYTES >> 4);
        const uint32_t p_lo = pdesc_lo + (uint32_t)(i & 1) * (DTC_QP >> 4);
        // 16 keys: two 8-key groups = 2048 bytes down the V tile; 32 bytes along a row of P^T (half ks / 4)
        umma_bf16_lo<-1>(tmem_o, v_lo, p_lo, desc_hi, idesc_o, share_start ? 0u : 1u);
#pragma unroll
        for (int ks = 1; ks < DTC_KEYS / 16; ++ks)
          umma_bf16_lo<1>(tmem_o, v_lo + ks * (2048 >> 4), p_lo + (ks >> 2) * ((DTC_QP / 2) >> 4) + 2 * (ks & 3), desc_hi,
                          idesc_o);
        umma_commit(&kv_empty[i % DTC_STAGES]);
        umma_commit(&pv_done[i & 1]);
        share_start = c.tile + 1 == c.tiles;
        if (i + 1 < n_tiles) {
          advance(c);
          if (!early && !issue_scores(i + 1)) break;
        }
      }
    }
  } else {
    // ---- softmax: thread `tid` owns key `tid` of a tile and output dimension `tid` -----------------------------
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    float m[GP], l[GP];
#pragma unroll
    for (int c = 0; c < GP; ++c) m[c] = -INFINITY, l[c] = 0.f;
    DtcCursor c = cur;
    bool share_start = true;
    int share_first_tile = cur.tile, shares = 0;
    for (int i = 0; i < n_tiles; ++i) {
      const int base = (c.first + c.tile) * DTC_KEYS;
      unsigned char* st = smem + (i % DTC_STAGES) * DTC_STAGE_BYTES;
      if (!mbar_wait(&s_full[i & 1], (i >> 1) & 1)) {
        if (lane == 0) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 33, i);
        s_abort = 1;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float s[GP];
      dtc_tmem_ld<GP>(tmem_s + (i & 1) * 32 + lane_base, s);
      const int key = base + tid;
      const bool visible = key >= c.lo && key < c.end;
      float mx[GP];
#pragma unroll
      for (int q = 0; q < GP; ++q) {
        s[q] = visible ? s[q] * p.scale_log2 : -INFINITY;
        mx[q] = s[q];
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
        for (int q = 0; q < GP; ++q) mx[q] = fmaxf(mx[q], __shfl_xor_sync(0xffffffffu, mx[q], off));
      }
      if (lane < GP) {
        float v = mx[0];
#pragma unroll
        for (int q = 1; q < GP; ++q) v = lane == q ? mx[q] : v;
        s_red[i & 1][warp][lane] = v;
      }
      // this tile's P^T buffer was last read by P.V two tiles ago (long done: its barrier takes every other tile,
      // so it cannot have moved past that phase)
      if (i > 1 && !mbar_wait(&pv_done[i & 1], ((i - 2) >> 1) & 1)) {
        if (lane == 0) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 34, i);
        s_abort = 1;
      }
      dtc_softmax_sync();
      if (s_abort) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // The reference point of a column's exponents only moves when its maximum grows by more than 2^8: until
      // then P is at most 256 and O^T and l, which share the reference, need no rescaling.
      float alpha[GP];
      bool moved = false;
#pragma unroll
      for (int q = 0; q < GP; ++q) {
        const float tmax = fmaxf(fmaxf(s_red[i & 1][0][q], s_red[i & 1][1][q]), fmaxf(s_red[i & 1][2][q], s_red[i & 1][3][q]));
        const float m_cand = fmaxf(m[q], tmax);
        const float m_new = (m[q] == -INFINITY || m_cand - m[q] > 8.f) ? m_cand : m[q];
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        alpha[q] = m[q] == -INFINITY ? 0.f : dtc_ex2(m[q] - m_use);
        moved = moved || (q < group && m_new != m[q] && m[q] != -INFINITY);
        m[q] = m_new;
        const float pr = dtc_ex2(s[q] - m_use);
        l[q] = l[q] * alpha[q] + pr;
        // P^T[q][key] (bf16): half tid / 64, row q, 16-byte chunk (tid % 64) / 8 swizzled by the row
        if (q < group) {
          const int kk = tid & 63;
          unsigned char* at = p_s + (i & 1) * DTC_QP + (tid >> 6) * (DTC_QP / 2) + (q >> 3) * 1024 + (q & 7) * 128 + (((kk >> 3) ^ (q & 7)) * 16) +
                              (kk & 7) * 2;
          *reinterpret_cast<__nv_bfloat16*>(at) = __float2bfloat16_rn(pr);
        }
      }
      // rows of V whose keys are not visible may hold anything: 0 * x must stay 0
      if (!visible) {
        unsigned char* v_t = st + DTC_KV + tid * 128;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          *reinterpret_cast<uint4*>(v_t + ch * 16) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(v_t + DTC_HALF + ch * 16) = make_uint4(0, 0, 0, 0);
        }
      }
      if (moved && !share_start) {  // the same in every thread: m is
        // O^T is complete up to the tile before once its P.V is done
        if (!mbar_wait(&pv_done[(i - 1) & 1], ((i - 1) >> 1) & 1)) {
          if (lane == 0) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 36, i);
          s_abort = 1;  // seen by all at their next meeting; this tile goes on with what is there
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float o[GP];
        dtc_tmem_ld<GP>(tmem_o + lane_base, o);
#pragma unroll
        for (int q = 0; q < GP; ++q) o[q] *= alpha[q];
        dtc_tmem_st<GP>(tmem_o + lane_base, o);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready);

      // ---- the pair ends here, or the range does: flush the softmax state -------------------------------
      const bool pair_ends = c.tile + 1 == c.tiles, range_ends = i + 1 == n_tiles;
      share_start = false;
      if (pair_ends || range_ends) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
          for (int q = 0; q < GP; ++q) l[q] += __shfl_xor_sync(0xffffffffu, l[q], off);
        }
        if (lane < GP) {
          float v = l[0];
#pragma unroll
          for (int q = 1; q < GP; ++q) v = lane == q ? l[q] : v;
          s_lsum[warp][lane] = v;
        }
        if (!mbar_wait(&pv_done[i & 1], (i >> 1) & 1)) {
          if (lane == 0) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 35, i);
          s_abort = 1;
        }
        dtc_softmax_sync();
        if (s_abort) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float o[GP];
        dtc_tmem_ld<GP>(tmem_o + lane_base, o);
        const bool whole = share_first_tile == 0 && pair_ends;
        float* part = p.part + ((gw * 2 + (shares == 0 ? 0 : 1)) * group) * DECB_ROW(DTC_D);
#pragma unroll
        for (int q = 0; q < GP; ++q) {
          if (q < group) {
            const float lsum = (s_lsum[0][q] + s_lsum[1][q]) + (s_lsum[2][q] + s_lsum[3][q]);
            if (whole) {
              const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
              p.out[((long long)c.b * p.num_q + c.kh * group + q) * DTC_D + tid] = __float2bfloat16_rn(o[q] * inv);
            } else {
              part[q * DECB_ROW(DTC_D) + tid] = o[q];
              if (tid == 0) *reinterpret_cast<float2*>(part + q * DECB_ROW(DTC_D) + DTC_D) = make_float2(m[q], lsum);
            }
          }
        }
        if (!whole && tid == 0) p.flags[c.b * p.num_kv + c.kh] = 1;  // this pair has parts to add
        ++shares;
        share_start = true;
        share_first_tile = 0;
#pragma unroll
        for (int q = 0; q < GP; ++q) m[q] = -INFINITY, l[q] = 0.f;
        // the next tile's P.V overwrites O^T: it waits for p_ready, which comes after these reads
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      }
      if (!range_ends) advance(c);
    }
  }
  __syncwarp();  // the lanes of the single-thread roles wait here for their lane 0 (the barrier counts warps)
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 5) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_slot), "r"(DTC_TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
struct DtcQKey {
  const void* ptr;
  long long rows, stride;
  int group;
  bool operator==(const DtcQKey& o) const { return ptr == o.ptr && rows == o.rows && stride == o.stride && group == o.group; }
};
struct DtcQKeyHash {
  size_t operator()(const DtcQKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.rows) * 31) ^ (std::hash<long long>()(k.stride) * 131) ^
           ((size_t)k.group * 8191);
  }
};
// Q: the projection buffer [rows, heads_total, 128]; a box is 64 columns of `group` neighbouring heads of one row
static bool dtc_map_q(const void* q, long long rows, long long row_stride_elems, int group, CUtensorMap* out) {
  static std::unordered_map<DtcQKey, CUtensorMap, DtcQKeyHash> maps;
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  DtcQKey key{q, rows, row_stride_elems, group};
  auto it = maps.find(key);
  if (it != maps.end()) {
    *out = it->second;
    return true;
  }
  UllmTmaEncodeFn enc = ullm_tma_encode();
  if (enc == nullptr) return false;
  cuuint64_t dims[3] = {DTC_D, (cuuint64_t)(row_stride_elems / DTC_D), (cuuint64_t)rows};
  cuuint64_t strides[2] = {DTC_D * 2, (cuuint64_t)row_stride_elems * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)group, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMap m;
  if (enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (maps.size() > 4096) maps.clear();
  maps[key] = m;
  *out = m;
  return true;
}

// bfloat16, head size 128, at most 16 query heads per kv head, at most 512 requests, pages of 8 to 128 tokens
// (a power of two: a tile of 128 keys is whole pages)
extern "C" int ullm_decode_attention_tcgen05_supported(int head_dim, int num_q, int num_kv, int batch, int page_size) {
  if (num_kv <= 0 || num_q % num_kv || batch > DTC_MAX_BATCH) return 0;
  if (page_size < 8 || page_size > DTC_KEYS || (page_size & (page_size - 1))) return 0;
  return head_dim == DTC_D && num_q / num_kv <= 16;
}

static int g_dtc_blocks = 0;

// Blocks of a launch (one per SM); 0: the kernel cannot be set up on this device.
extern "C" int ullm_decode_attention_tcgen05_blocks(void) {
  if (g_dtc_blocks == 0) {
    if (cudaFuncSetAttribute(decode_attention_tcgen05_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, DTC_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(decode_attention_tcgen05_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, DTC_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(decode_attention_tcgen05_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, DTC_SMEM) != cudaSuccess)
      return 0;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      return 0;
    g_dtc_blocks = sms;
  }
  return g_dtc_blocks;
}

// Floats of `part` a launch needs for `group` query heads per kv head (`prefix` takes batch + 1 ints, `flags`
// batch * num_kv ints that are zero before the first launch).
extern "C" long long ullm_decode_attention_tcgen05_scratch_floats(int group) {
  return (long long)ullm_decode_attention_tcgen05_blocks() * 2 * group * DECB_ROW(DTC_D);
}

extern "C" int ullm_decode_attention_tcgen05(const void* q, long long q_row_stride, const void* k_cache,
                                             const void* v_cache, const int* block_table, int max_pages,
                                             const int* req_slots, const int* kv_len, void* out, float* part,
                                             int* prefix, int* flags, int batch, int num_q, int num_kv, int head_dim,
                                             int page_size, int window, float scale, long long num_pages, int* status,
                                             void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (batch < 0 || num_q <= 0 || num_kv <= 0 || page_size <= 0 || max_pages <= 0 || window < 0) return ULLM_ERR_BAD_SIZE;
  if (!ullm_decode_attention_tcgen05_supported(head_dim, num_q, num_kv, batch, page_size)) return ULLM_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) return ULLM_ERR_UNSUPPORTED;
  if (q_row_stride % DTC_D) return ULLM_ERR_UNSUPPORTED;
  if (part == nullptr || prefix == nullptr || flags == nullptr) return ULLM_ERR_BAD_SIZE;
  if (batch == 0) return ULLM_OK;
  const int blocks = ullm_decode_attention_tcgen05_blocks();
  if (blocks <= 0) return ULLM_ERR_LAUNCH;
  const int group = num_q / num_kv;
  DtcParams p;
  p.block_table = block_table;
  p.max_pages = max_pages;
  p.req_slots = req_slots;
  p.kv_len = kv_len;
  p.out = (__nv_bfloat16*)out;
  p.part = part;
  p.prefix = prefix;
  p.flags = flags;
  p.batch = batch;
  p.num_q = num_q;
  p.num_kv = num_kv;
  p.page_size = page_size;
  p.page_shift = 0;
  while ((1 << p.page_shift) < page_size) ++p.page_shift;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.num_pages = num_pages;
  p.status = status;
  CUtensorMap mq, mk, mv;
  if (!dtc_map_q(q, batch, q_row_stride, group, &mq) ||
      !ullm_tma_map_kv(k_cache, num_pages, page_size, num_kv, head_dim, page_size, &mk) ||
      !ullm_tma_map_kv(v_cache, num_pages, page_size, num_kv, head_dim, page_size, &mv))
    return ULLM_ERR_LAUNCH;
  int rc;
  if (group <= 4)
    rc = ullm_launch_kernel(decode_attention_tcgen05_kernel<4>, dim3(blocks), dim3(DTC_THREADS), (size_t)DTC_SMEM, st, mq, mk, mv, p);
  else if (group <= 8)
    rc = ullm_launch_kernel(decode_attention_tcgen05_kernel<8>, dim3(blocks), dim3(DTC_THREADS), (size_t)DTC_SMEM, st, mq, mk, mv, p);
  else
    rc = ullm_launch_kernel(decode_attention_tcgen05_kernel<16>, dim3(blocks), dim3(DTC_THREADS), (size_t)DTC_SMEM, st, mq, mk, mv, p);
  if (rc == ULLM_OK)
    rc = ullm_launch_kernel(decode_balanced_merge_kernel<DTC_D>, dim3(batch * num_kv), dim3(DECB_MERGE_THREADS), 0, st,
                            (const float*)part, (const int*)prefix, flags, (__nv_bfloat16*)out, batch, num_q, num_kv,
                            (long long)blocks, 1);
  if (rc != ULLM_OK) return rc;
  return ullm_launch_status();
}
