// Paged decode attention for bfloat16 with the keys of the whole batch split evenly over the warps.
//
// attention_decode.cu gives every (request, kv head) the same number of blocks, whatever the request's
// length: a batch of one long and many short requests waits for the long one, a block count that is no
// multiple of what the GPU holds at once pays for a half-empty last wave, and every block pays its own
// start-up and merge.  Here the unit of work is a tile of 16 keys of one (request, kv head) pair; the tiles of
// all pairs, in pair order, form one list that is cut into equal contiguous ranges, one per warp, for as many
// warps as the GPU holds at once (the grid never depends on the lengths, so a captured launch stays valid).
//
// A warp streams its range through one ring of shared-memory stages without a break: one lane asks the TMA unit
// for a tile (cp.async.bulk.tensor boxes of one head's 16 tokens out of a page, 128-byte swizzle, completion on
// an mbarrier), two tiles ahead of the arithmetic (mma.sync m16n8k16 on ldmatrix fragments, as in
// decode_core.cuh), and the loads cross from one pair into the next; only the softmax state is flushed at a
// pair's end.  Tiles are aligned to absolute token positions, so that a tile is a whole page (or 16 / page_size
// pages, or half a 32-token page); keys outside the request's visible range are masked and their V rows zeroed.  A pair
// that lies whole inside the range is finished by the warp (it writes the output rows); a pair that the range
// cuts (at most the first and the last of a warp) leaves its partial (max, sum, unnormalised output) in the
// warp's slot 0 or 1 of the scratch array, and the merge kernel that follows adds the parts of such a pair in
// warp order.  No warp waits for another: after the prologue there is no block-wide barrier.  The waits on the
// mbarriers are bounded: after DECB_WAIT_LIMIT polls the warp records ULLM_STATUS_TIMEOUT and returns.
#include "decode_core.cuh"
#include "decode_merge.cuh"
#include "tma_host.cuh"

#define ULLM_STATUS_TIMEOUT 6
#define DECB_WAIT_LIMIT (1 << 20)
#define DECB_SUB 2048  // bytes of a sub-tile: 16 tokens x 64 elements
#ifndef DECB_STAGES
#define DECB_STAGES 2  // tiles of a warp's ring
#endif

__device__ __forceinline__ uint32_t decb_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void decb_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(decb_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void decb_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(decb_smem(bar)), "r"(bytes) : "memory");
}
// false: gave up
__device__ __forceinline__ bool decb_mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t a = decb_smem(bar);
  for (int i = 0; i < DECB_WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(a), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void decb_tma_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z,
                                            int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(decb_smem(dst)), "l"(map), "r"(decb_smem(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

#define DECB_MAX_BATCH 512
#ifndef DECB_WARPS
#define DECB_WARPS 4  // warps of a block
#endif
#define DECB_MIN_TILES 4  // ranges are not made shorter than this many tiles (fewer warps work instead)

struct DecbParams {
  const __nv_bfloat16* q;
  long long q_row_stride;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* block_table;
  int max_pages;
  const int* req_slots;
  const int* kv_len;
  __nv_bfloat16* out;
  float* part;    // [warps][2][group][D + 4]: unnormalised output, max, sum
  int* prefix;    // [batch + 1]: tiles of the requests before each (per kv head)
  int* flags;     // [batch * num_kv], zero between launches: set for a pair that was cut, cleared by the merge
  int batch, num_q, num_kv, page_size, page_shift, window;  // page_size = 1 << page_shift
  float scale_log2;
  long long num_pages;
  int* status;
};

// Where a warp stands in the list of tiles.
struct DecbCursor {
  int b, kh;       // the pair
  int tile, tiles; // tile inside the pair, tiles of the pair
  int first;       // absolute index of the pair's tile 0 (a tile holds the keys 16 i .. 16 i + 15)
  int lo, end;     // the request's visible keys [lo, end)
};

template <int D>
__global__ void __launch_bounds__(DECB_WARPS * 32, DECB_STAGES >= 4 ? 1 : 3)
decode_attention_balanced_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                                 const DecbParams p) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_pre[DECB_MAX_BATCH + 1], s_lo[DECB_MAX_BATCH], s_end[DECB_MAX_BATCH], s_slot[DECB_MAX_BATCH];
  __shared__ __align__(8) uint64_t s_full[DECB_WARPS][DECB_STAGES];
  pdl_launch_dependents();
  pdl_wait();
  constexpr int HALVES = D / 64;            // 64-element halves of a row
  constexpr int KSTEPS = D / 16;            // k-steps of the score product
  constexpr int NT_O = D / 8;               // n-tiles of the output
  constexpr int KV_BYTES = HALVES * DECB_SUB;  // a K (or V) tile: its halves one after the other
  constexpr int STAGE_BYTES = 2 * KV_BYTES;
  constexpr int WARP_BYTES = DECB_STAGES * STAGE_BYTES;
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.num_q / p.num_kv;

  // ---- prologue (the only block-wide part): every request's visible keys, tiles and their running sum -----
  for (int b = threadIdx.x; b < p.batch; b += blockDim.x) {
    const int pos = p.kv_len[b] - 1;
    const int lo = (p.window > 0 && pos >= 0) ? max(0, pos - p.window + 1) : 0;
    const int n = pos >= 0 ? pos - lo + 1 : 0;
    s_lo[b] = lo;
    s_end[b] = lo + n;
    s_slot[b] = p.req_slots[b];
    s_pre[b + 1] = n > 0 ? (lo + n + DEC_TILE - 1) / DEC_TILE - lo / DEC_TILE : 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    s_pre[0] = 0;
    for (int b = 0; b < p.batch; ++b) s_pre[b + 1] += s_pre[b];
  }
  __syncthreads();
  if (blockIdx.x == 0)
    for (int b = threadIdx.x; b <= p.batch; b += blockDim.x) p.prefix[b] = s_pre[b];
  // rows of requests that hold nothing (padding of a captured batch) are zero
  for (long long b = blockIdx.x; b < p.batch; b += gridDim.x) {
    if (s_pre[b + 1] == s_pre[b]) {
      __nv_bfloat16* o = p.out + b * p.num_q * D;
      for (int i = threadIdx.x; i < p.num_q * D; i += blockDim.x) o[i] = __float2bfloat16_rn(0.f);
    }
  }

  const long long W = (long long)p.num_kv * s_pre[p.batch];
  const long long GW = decb_ranges(W, (long long)gridDim.x * DECB_WARPS, DECB_MIN_TILES);
  const long long gw = (long long)blockIdx.x * DECB_WARPS + warp;
  if (gw >= GW || W == 0) return;
  const long long u0 = gw * W / GW, u1 = (gw + 1) * W / GW;
  if (u0 >= u1) return;
  unsigned char* ring = smem + warp * WARP_BYTES;
  uint64_t* full = s_full[warp];
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < DECB_STAGES; ++s) decb_mbar_init(&full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();

  auto set_pair = [&](DecbCursor& c) {
    c.tiles = s_pre[c.b + 1] - s_pre[c.b];
    c.lo = s_lo[c.b];
    c.end = s_end[c.b];
    c.first = c.lo / DEC_TILE;
  };
  auto advance = [&](DecbCursor& c) {  // to the next tile of the list (callers stop at the range's end)
    if (++c.tile < c.tiles) return;
    c.tile = 0;
    if (++c.kh == p.num_kv) {
      c.kh = 0;
      do ++c.b; while (c.b < p.batch - 1 && s_pre[c.b + 1] == s_pre[c.b]);
      if (c.b >= p.batch) c.b = p.batch - 1;
      set_pair(c);
    }
  };
  DecbCursor cur;
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
  DecbCursor ahead = cur;  // the cursor of the loads, two tiles ahead of the arithmetic

  // Block-table entries of the request the loads are in, 32 at a time, one per lane.  A tile is one group of
  // boxes of 16 tokens when a page holds 16 or more, else 16 / page_size groups of a whole page each.  A group is
  // the K and the V box of each 64-element half of the head: 2 HALVES boxes, asked for by as many lanes in one
  // instruction (lane = group * 2 HALVES + box).
  const int sh = p.page_shift;
  const int box_tokens = min(p.page_size, DEC_TILE), boxes = DEC_TILE / box_tokens;
  constexpr int PER_GROUP = 2 * HALVES;
  const int my_group = lane / PER_GROUP, my_box = lane % PER_GROUP;  // box: (K, V) x halves
  const CUtensorMap* my_map = my_box < HALVES ? &map_k : &map_v;
  const int my_off = (my_box < HALVES ? 0 : KV_BYTES) + (my_box % HALVES) * DECB_SUB + my_group * box_tokens * 128;
  const int my_x = (my_box % HALVES) * 64;
  const uint32_t group_bytes = (uint32_t)box_tokens * 128 * PER_GROUP;
  int win_b = -1, win_base = 0, win_page = -1;
  auto issue = [&](const DecbCursor& c, int stage) {
    const int base = (c.first + c.tile) * DEC_TILE;  // absolute position of the tile's row 0
    const int page0 = base >> sh;
    if (c.b != win_b || page0 + boxes - 1 > win_base + 31 || page0 < win_base) {
      win_b = c.b;
      win_base = page0;
      const int last = (c.end - 1) >> sh;
      win_page = win_base + lane <= last ? p.block_table[(long long)s_slot[c.b] * p.max_pages + win_base + lane] : -1;
    }
    // a group is loaded if any of its keys is visible; pages in front of a window may have been given back (-1).
    // 32 / PER_GROUP groups per pass (one pass unless pages are tiny): count first, then one expect_tx, then ask.
    constexpr int GROUPS_PER_PASS = 32 / PER_GROUP;
    int n_load = 0;
    for (int g0 = 0; g0 < boxes; g0 += GROUPS_PER_PASS) {
      const int grp = g0 + my_group;
      const int page = __shfl_sync(0xffffffffu, win_page, grp < boxes ? page0 + grp - win_base : 0);
      const int k0 = base + grp * box_tokens;
      bool load = grp < boxes && k0 < c.end && k0 + box_tokens > c.lo;
      if (load && (page < 0 || page >= p.num_pages)) {
        if (my_box == 0) ullm_report(p.status, ULLM_STATUS_PAGE, c.b, page);
        load = false;
      }
      n_load += __popc(__ballot_sync(0xffffffffu, load && my_box == 0));
    }
    if (lane == 0) decb_mbar_expect_tx(&full[stage], (uint32_t)n_load * group_bytes);
    __syncwarp();
    for (int g0 = 0; g0 < boxes; g0 += GROUPS_PER_PASS) {
      const int grp = g0 + my_group;
      const int page = __shfl_sync(0xffffffffu, win_page, grp < boxes ? page0 + grp - win_base : 0);
      const int k0 = base + grp * box_tokens;
      if (grp < boxes && k0 < c.end && k0 + box_tokens > c.lo && page >= 0 && page < p.num_pages)
        decb_tma_4d(ring + stage * STAGE_BYTES + my_off + g0 * box_tokens * 128, my_map, &full[stage], my_x, c.kh,
                    p.page_size >= DEC_TILE ? base & (p.page_size - 1) : 0, page);
    }
  };

  unsigned qa[KSTEPS][4];
  auto load_q = [&](const DecbCursor& c) {  // Q fragments (A operand) of the pair, rows >= group are zero
    const int r0 = lane >> 2, r1 = r0 + 8, cc = (lane & 3) * 2;
    const __nv_bfloat16* q0 = p.q + (long long)c.b * p.q_row_stride + (long long)(c.kh * group + r0) * D;
    const __nv_bfloat16* q1 = p.q + (long long)c.b * p.q_row_stride + (long long)(c.kh * group + r1) * D;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      qa[kk][0] = r0 < group ? *reinterpret_cast<const unsigned*>(q0 + kk * 16 + cc) : 0u;
      qa[kk][1] = r1 < group ? *reinterpret_cast<const unsigned*>(q1 + kk * 16 + cc) : 0u;
      qa[kk][2] = r0 < group ? *reinterpret_cast<const unsigned*>(q0 + kk * 16 + 8 + cc) : 0u;
      qa[kk][3] = r1 < group ? *reinterpret_cast<const unsigned*>(q1 + kk * 16 + 8 + cc) : 0u;
    }
  };

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[NT_O][4];
#pragma unroll
  for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

  const int n_tiles = (int)(u1 - u0);
  int next_issue = 0;  // the next tile of the range to ask for; `ahead` stands on it
  auto fill = [&](int upto) {  // asks for tiles while ring stages are free: tiles before `upto` have been used
    while (next_issue < n_tiles && next_issue < upto + DECB_STAGES) {
      issue(ahead, next_issue % DECB_STAGES);
      if (++next_issue < n_tiles) advance(ahead);
    }
  };
  fill(0);
  load_q(cur);
  int share_first_tile = cur.tile;  // where this warp's share of the current pair began
  int shares = 0;                   // shares flushed so far (the first partial goes to slot 0, a later one to slot 1)

  // Two tiles of the same pair are taken in one go where there are two: their score products are independent
  // chains of tensor instructions, which hides the instruction's latency that a single chain would expose.
  for (int it = 0; it < n_tiles;) {
    const int nt = (DECB_STAGES >= 4 && it + 1 < n_tiles && cur.tile + 1 < cur.tiles) ? 2 : 1;
    // every lane sees the phases complete (and with them the tiles); the warp gives up as one
    bool got = decb_mbar_wait(&full[it % DECB_STAGES], (it / DECB_STAGES) & 1);
    if (nt == 2) got = got && decb_mbar_wait(&full[(it + 1) % DECB_STAGES], ((it + 1) / DECB_STAGES) & 1);
    if (!__all_sync(0xffffffffu, got)) {
      if (lane == 0) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 20, it);
      return;
    }
    unsigned char* kbuf[2];
    unsigned char* vbuf[2];
    const int base = (cur.first + cur.tile) * DEC_TILE;  // absolute position of the first tile's row 0
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      kbuf[t] = ring + ((it + t) % DECB_STAGES) * STAGE_BYTES;
      vbuf[t] = kbuf[t] + KV_BYTES;
    }
    if (base < cur.lo || base + nt * DEC_TILE > cur.end) {
      // rows of keys that are not visible may hold anything (another request's old values, never-written
      // memory): their scores are masked below, their V rows are zeroed here so that 0 * x stays 0
      for (int t = 0; t < nt; ++t) {
        for (int i = lane; i < DEC_TILE * HALVES * 8; i += 32) {
          const int row = i / (HALVES * 8), rest = i % (HALVES * 8);
          const int key = base + t * DEC_TILE + row;
          if (key < cur.lo || key >= cur.end)
            *reinterpret_cast<uint4*>(vbuf[t] + (rest / 8) * DECB_SUB + row * 128 + (rest % 8) * 16) = make_uint4(0, 0, 0, 0);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // before the TMA unit writes these stages again
      __syncwarp();
    }
    // ---- scores: 2 n-tiles of 8 keys per tile ---------------------------------------------
    float sc[4][4];
#pragma unroll
    for (int t = 0; t < 4; ++t) sc[t][0] = sc[t][1] = sc[t][2] = sc[t][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      const int mat = lane >> 3, row = (mat >> 1) * 8 + (lane & 7), ch = 2 * kk + (mat & 1);
      const int at = (ch >> 3) * DECB_SUB + row * 128 + (((ch & 7) ^ (row & 7)) * 16);
      unsigned b0, b1, b2, b3;
      ldmatrix_x4(b0, b1, b2, b3, kbuf[0] + at);
      mma_bf16(sc[0], qa[kk], b0, b1);
      mma_bf16(sc[1], qa[kk], b2, b3);
      if (nt == 2) {
        ldmatrix_x4(b0, b1, b2, b3, kbuf[1] + at);
        mma_bf16(sc[2], qa[kk], b0, b1);
        mma_bf16(sc[3], qa[kk], b2, b3);
      }
    }
    // ---- mask (tiles at the ends of the visible range only), online softmax --------------------
    const bool edge = base < cur.lo || base + nt * DEC_TILE > cur.end;
    float mx[2] = {m[0], m[1]};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = sc[t][e] * p.scale_log2;
        if (t >= 2 && nt == 1) v = -INFINITY;
        if (edge) {
          const int key = base + t * 8 + (lane & 3) * 2 + (e & 1);
          if (key < cur.lo || key >= cur.end) v = -INFINITY;
        }
        sc[t][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    // the running maximum rarely moves after the first tiles: the output is rescaled only when it did
    const bool moved = __any_sync(0xffffffffu, mx[0] != m[0] || mx[1] != m[1]);
    float alpha[2] = {1.f, 1.f};
    if (moved) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        alpha[r] = mx[r] == -INFINITY ? 1.f : exp2f(m[r] - mx[r]);
        m[r] = mx[r];
        l[r] *= alpha[r];
      }
    }
    unsigned pa[2][4];
    {
      float pr[4][4];
#pragma unroll
      for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          pr[t][e] = m[e >> 1] == -INFINITY ? 0.f : exp2f(sc[t][e] - m[e >> 1]);
          l[e >> 1] += pr[t][e];
        }
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        pa[t][0] = pack_bf16(pr[2 * t][0], pr[2 * t][1]);
        pa[t][1] = pack_bf16(pr[2 * t][2], pr[2 * t][3]);
        pa[t][2] = pack_bf16(pr[2 * t + 1][0], pr[2 * t + 1][1]);
        pa[t][3] = pack_bf16(pr[2 * t + 1][2], pr[2 * t + 1][3]);
      }
    }
    // ---- O = alpha O + P V ------------------------------------------------------------
    if (moved) {
#pragma unroll
      for (int j = 0; j < NT_O; ++j) {
        o[j][0] *= alpha[0]; o[j][1] *= alpha[0]; o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
      }
    }
#pragma unroll
    for (int j = 0; j < NT_O; j += 2) {
      const int mat = lane >> 3, row = (mat & 1) * 8 + (lane & 7), ch = j + (mat >> 1);
      const int at = (ch >> 3) * DECB_SUB + row * 128 + (((ch & 7) ^ (row & 7)) * 16);
      unsigned b0, b1, b2, b3;
      ldmatrix_x4_trans(b0, b1, b2, b3, vbuf[0] + at);
      mma_bf16(o[j], pa[0], b0, b1);
      mma_bf16(o[j + 1], pa[0], b2, b3);
      if (nt == 2) {
        ldmatrix_x4_trans(b0, b1, b2, b3, vbuf[1] + at);
        mma_bf16(o[j], pa[1], b0, b1);
        mma_bf16(o[j + 1], pa[1], b2, b3);
      }
    }
    __syncwarp();
    if (nt == 2) advance(cur);  // onto the second of the two tiles: the flush below looks at the last tile taken
    it += nt;
    fill(it);  // the stages of the tiles just used are free

    // ---- the pair ends here, or the range does: flush the softmax state ------------------------
    const bool pair_ends = cur.tile + 1 == cur.tiles, range_ends = it == n_tiles;
    if (pair_ends || range_ends) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
      }
      const bool whole = share_first_tile == 0 && pair_ends;
      const int r0 = lane >> 2, r1 = r0 + 8, cc = (lane & 3) * 2;
      if (whole) {
        const float inv0 = l[0] > 0.f ? 1.f / l[0] : 0.f, inv1 = l[1] > 0.f ? 1.f / l[1] : 0.f;
        __nv_bfloat16* o0 = p.out + ((long long)cur.b * p.num_q + cur.kh * group + r0) * D + cc;
        __nv_bfloat16* o1 = p.out + ((long long)cur.b * p.num_q + cur.kh * group + r1) * D + cc;
#pragma unroll
        for (int j = 0; j < NT_O; ++j) {
          if (r0 < group) *reinterpret_cast<__nv_bfloat162*>(o0 + j * 8) = __floats2bfloat162_rn(o[j][0] * inv0, o[j][1] * inv0);
          if (r1 < group) *reinterpret_cast<__nv_bfloat162*>(o1 + j * 8) = __floats2bfloat162_rn(o[j][2] * inv1, o[j][3] * inv1);
        }
      } else {
        float* part = p.part + ((gw * 2 + (shares == 0 ? 0 : 1)) * group) * DECB_ROW(D);
#pragma unroll
        for (int j = 0; j < NT_O; ++j) {
          if (r0 < group) *reinterpret_cast<float2*>(part + r0 * DECB_ROW(D) + j * 8 + cc) = make_float2(o[j][0], o[j][1]);
          if (r1 < group) *reinterpret_cast<float2*>(part + r1 * DECB_ROW(D) + j * 8 + cc) = make_float2(o[j][2], o[j][3]);
        }
        if ((lane & 3) == 0) {
          if (r0 < group) *reinterpret_cast<float2*>(part + r0 * DECB_ROW(D) + D) = make_float2(m[0], l[0]);
          if (r1 < group) *reinterpret_cast<float2*>(part + r1 * DECB_ROW(D) + D) = make_float2(m[1], l[1]);
        }
        if (lane == 0) p.flags[cur.b * p.num_kv + cur.kh] = 1;  // tells the merge kernel that this pair has parts to add
      }
      ++shares;
      m[0] = m[1] = -INFINITY;
      l[0] = l[1] = 0.f;
#pragma unroll
      for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    }
    if (!range_ends) {
      advance(cur);
      if (pair_ends) {
        load_q(cur);
        share_first_tile = 0;
      }
    }
  }
}

static int g_decb_blocks[2] = {0, 0};

// dynamic shared memory of a block: the warps' rings, and room to align them to 1024 bytes
static constexpr int decb_smem_bytes(int head_dim) {
  return DECB_WARPS * DECB_STAGES * 2 * (head_dim / 64) * DECB_SUB + 1024;
}

// Blocks of a launch: as many as the GPU holds at once.  0: the kernel cannot be set up.
template <int D>
static int decb_blocks(int which) {
  if (g_decb_blocks[which] == 0) {
    constexpr int SMEM = decb_smem_bytes(D);
    if (cudaFuncSetAttribute(decode_attention_balanced_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM) != cudaSuccess)
      return 0;
    cudaFuncSetAttribute(decode_attention_balanced_kernel<D>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_attention_balanced_kernel<D>, DECB_WARPS * 32,
                                                      SMEM) != cudaSuccess ||
        sms <= 0 || per_sm <= 0)
      return 0;
    g_decb_blocks[which] = sms * per_sm;
  }
  return g_decb_blocks[which];
}

// Sizes: as ullm_decode_attention_supported, at most DECB_MAX_BATCH requests, and pages of a power of two of
// tokens (a tile of 16 tokens is then whole pages, or lies inside one; positions split by shifts).
extern "C" int ullm_decode_attention_balanced_supported(int head_dim, int num_q, int num_kv, int batch, int page_size) {
  if (num_kv <= 0 || num_q % num_kv || batch > DECB_MAX_BATCH) return 0;
  if (page_size <= 0 || (page_size & (page_size - 1))) return 0;
  return (head_dim == 64 || head_dim == 128) && (num_q / num_kv) <= 16;
}

// Blocks a launch uses on the current device (the scratch is sized by it): 0 on failure.
extern "C" int ullm_decode_attention_balanced_blocks(int head_dim) {
  return head_dim == 64 ? decb_blocks<64>(0) : head_dim == 128 ? decb_blocks<128>(1) : 0;
}

// Floats of `part` a launch needs for `group` query heads per kv head (`prefix` takes batch + 1 ints, `flags`
// batch * num_kv ints that are zero before the first launch).
extern "C" long long ullm_decode_attention_balanced_scratch_floats(int head_dim, int group) {
  return (long long)ullm_decode_attention_balanced_blocks(head_dim) * DECB_WARPS * 2 * group * DECB_ROW(head_dim);
}

extern "C" int ullm_decode_attention_balanced(const void* q, long long q_row_stride, const void* k_cache,
                                              const void* v_cache, const int* block_table, int max_pages,
                                              const int* req_slots, const int* kv_len, void* out, float* part,
                                              int* prefix, int* flags, int batch, int num_q, int num_kv, int head_dim,
                                              int page_size, int window, float scale, long long num_pages, int* status,
                                              void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (batch < 0 || num_q <= 0 || num_kv <= 0 || page_size <= 0 || max_pages <= 0 || window < 0) return ULLM_ERR_BAD_SIZE;
  if (!ullm_decode_attention_balanced_supported(head_dim, num_q, num_kv, batch, page_size)) return ULLM_ERR_UNSUPPORTED;
  if (((uintptr_t)k_cache | (uintptr_t)v_cache) & 15) return ULLM_ERR_UNSUPPORTED;
  if (part == nullptr || prefix == nullptr || flags == nullptr) return ULLM_ERR_BAD_SIZE;
  if (batch == 0) return ULLM_OK;
  const int blocks = ullm_decode_attention_balanced_blocks(head_dim);
  if (blocks <= 0) return ULLM_ERR_LAUNCH;
  DecbParams p;
  p.q = (const __nv_bfloat16*)q;
  p.q_row_stride = q_row_stride;
  p.k_cache = (const __nv_bfloat16*)k_cache;
  p.v_cache = (const __nv_bfloat16*)v_cache;
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
  const long long warps = (long long)blocks * DECB_WARPS;
  const int box_tokens = page_size < DEC_TILE ? page_size : DEC_TILE;
  CUtensorMap map_k, map_v;
  if (!ullm_tma_map_kv(k_cache, num_pages, page_size, num_kv, head_dim, box_tokens, &map_k) ||
      !ullm_tma_map_kv(v_cache, num_pages, page_size, num_kv, head_dim, box_tokens, &map_v))
    return ULLM_ERR_LAUNCH;
  int rc;
  if (head_dim == 64) {
    rc = ullm_launch_kernel(decode_attention_balanced_kernel<64>, dim3(blocks), dim3(DECB_WARPS * 32),
                            (size_t)decb_smem_bytes(64), st, map_k, map_v, p);
    if (rc == ULLM_OK)
      rc = ullm_launch_kernel(decode_balanced_merge_kernel<64>, dim3(batch * num_kv), dim3(DECB_MERGE_THREADS), 0, st,
                              (const float*)part, (const int*)prefix, flags, (__nv_bfloat16*)out, batch, num_q, num_kv, warps, DECB_MIN_TILES);
  } else {
    rc = ullm_launch_kernel(decode_attention_balanced_kernel<128>, dim3(blocks), dim3(DECB_WARPS * 32),
                            (size_t)decb_smem_bytes(128), st, map_k, map_v, p);
    if (rc == ULLM_OK)
      rc = ullm_launch_kernel(decode_balanced_merge_kernel<128>, dim3(batch * num_kv), dim3(DECB_MERGE_THREADS), 0, st,
                              (const float*)part, (const int*)prefix, flags, (__nv_bfloat16*)out, batch, num_q, num_kv, warps, DECB_MIN_TILES);
  }
  if (rc != ULLM_OK) return rc;
  return ullm_launch_status();
}
