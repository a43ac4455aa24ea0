// Paged decode attention for bfloat16: one query token per request, keys and
// values streamed once from the pages.  Split over the key range (grid.x) and,
// inside a block, over its four warps; every warp runs an online softmax over
// its own keys with tensor-core products (mma.sync m16n8k16, fp32 accumulate):
//
//   rows of the 16-row tile = the query heads that share one kv head (<= 16)
//   S[16 x 16 keys]  = Q[16 x D] K^T          (scores, fp32)
//   O[16 x D]       += P[16 x 16 keys] V      (P rounded to bf16, O fp32)
//
// K and V rows (one head of one token: D bf16) are gathered page by page with
// cp.async into a three-stage ring per warp (chunks of 16 bytes, XOR-swizzled by
// row so that ldmatrix reads are conflict-free).  Rows past the end of the range
// are zero-filled, never read.  The warps' partial (max, sum, O) are merged in
// shared memory; with more than one split the block writes its partial to the
// scratch arrays and a second kernel merges the splits.  Softmax and all
// accumulation are 32-bit; exp is ex2 on log2(e)-scaled scores.
//
// The grid depends on the batch size and the split count only, never on the
// lengths, so a captured launch stays valid as the requests grow.
//
// Given the rotation tables (DecFuse), the kernel also prepares its inputs from the
// raw projection: every block norms and rotates the q rows it holds as fragments,
// and the one warp whose keys end with the newest one norms and rotates the new
// key, copies the new value, writes both to the cache and, once its last tile has
// landed, into that tile's rows in shared memory.
#include <cooperative_groups.h>

#include "decode_core.cuh"

namespace cg = cooperative_groups;

// What the kernel needs to prepare q and the new key and value itself (cos == nullptr: they come prepared, as
// qk_rope_store.cu leaves them): per-head RMSNorm weights (or null), the rotation tables [positions, D / 2], the
// row's position and cache slot.  The arithmetic is that of qk_norm_rope_store_bf16_kernel: 32-bit sums and
// rotation, one rounding to bfloat16.
struct DecFuse {
  const float* q_w;
  const float* k_w;
  const float* cos_t;
  const float* sin_t;
  const int* positions;
  const int* slot_mapping;  // null: this execution does not write the cache
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  long long num_slots;
  int max_positions;
  float eps;
};

// 2^x by the hardware's unit alone (exp2f adds a range fix-up around the same instruction)
__device__ __forceinline__ float dec_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// CL: the splits of a (request, kv head) pair are the blocks of one thread-block cluster (at most 8) and merge
// their partials through distributed shared memory; no scratch arrays, no second kernel.
template <int D, bool CL>
__global__ void __launch_bounds__(DEC_WARPS * 32)
decode_attention_kernel(const __nv_bfloat16* __restrict__ q, long long q_row_stride,
                        const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                        const int* __restrict__ block_table, int max_pages, const int* __restrict__ req_slots,
                        const int* __restrict__ kv_len, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                        float* __restrict__ part_ml, int num_q, int num_kv, int page_size, int window,
                        float scale_log2, long long num_pages, int* status, const DecFuse fu) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ float cm[CL ? 16 * (D + 2) : 1];  // this block's merged partial (cluster form): [head][D outputs, max, sum]
  pdl_launch_dependents();
  constexpr int CHUNKS = D / 8;        // 16-byte chunks per row
  constexpr int KSTEPS = D / 16;       // k-steps of the score product
  constexpr int NT_O = D / 8;          // n-tiles of the output
  using S = DecodeSmem<D>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, num_splits = gridDim.x, kh = blockIdx.y, b = blockIdx.z;
  const int group = num_q / num_kv;
  const int kvl = kv_len[b];
  const int pos = kvl - 1;
  const int lo = (window > 0 && pos >= 0) ? max(0, pos - window + 1) : 0;
  const int n_keys = pos >= 0 ? pos - lo + 1 : 0;
  // this block's keys, then this warp's keys (both in whole tiles, except the last)
  int per_split = (n_keys + num_splits - 1) / num_splits;
  per_split = (per_split + DEC_TILE * DEC_WARPS - 1) / (DEC_TILE * DEC_WARPS) * (DEC_TILE * DEC_WARPS);
  const int s_begin = min(n_keys, split * per_split), s_end = min(n_keys, s_begin + per_split);
  const int per_warp = per_split / DEC_WARPS;
  const int w_begin = lo + min(s_end, s_begin + warp * per_warp), w_end = lo + min(s_end, s_begin + (warp + 1) * per_warp);
  const int tiles = (w_end - w_begin + DEC_TILE - 1) / DEC_TILE;
  const int* bt = block_table + (long long)req_slots[b] * max_pages;
  const long long kv_row = (long long)num_kv * D;

  unsigned char* ring = smem + warp * S::WARP_BYTES;
  auto issue = [&](int tile) {
    unsigned char* kbuf = ring + (tile % DEC_STAGES) * 2 * S::TILE_BYTES;
    unsigned char* vbuf = kbuf + S::TILE_BYTES;
    const int base = w_begin + tile * DEC_TILE;
    // lanes 0..15 look up the slot of row `lane`
    long long my_slot = -1;
    if (lane < DEC_TILE) {
      const int key = base + lane;
      if (key < w_end) {
        const int page = bt[key / page_size];
        if (page < 0 || page >= num_pages) ullm_report(status, ULLM_STATUS_PAGE, b, page);
        else my_slot = (long long)page * page_size + key % page_size;
      }
    }
#pragma unroll
    for (int i = 0; i < DEC_TILE * CHUNKS / 32; ++i) {
      const int c = i * 32 + lane;
      const int row = c / CHUNKS, ch = c % CHUNKS;
      const long long slot = __shfl_sync(0xffffffffu, my_slot, row);
      const bool ok = slot >= 0;
      const long long off = ok ? (slot * kv_row + (long long)kh * D + ch * 8) : 0;
      const int sw = row * S::ROW_BYTES + ((ch ^ (row & 7)) * 16);
      cp_async_16(kbuf + sw, k_cache + off, ok);
      cp_async_16(vbuf + sw, v_cache + off, ok);
    }
  };

  // Under programmatic dependent launch the kernel in front (the projection that writes q and the new key and
  // value) may still be running here.  The pages of the older keys do not depend on it (block tables and lengths
  // were staged before the step's first kernel; this layer's pages are written by this kernel alone), so a kernel
  // that prepares the new key itself starts its first tiles' copies now and waits only then.  What a copy finds
  // in the newest key's slot does not matter: that row is replaced in shared memory below.
  const bool early = fu.cos_t != nullptr;
  // What the preparation of q needs besides q itself does not depend on that kernel either (the positions are
  // staged with the block tables; tables and norm weights never change): fetched now, so that after the wait only
  // q's own loads stand before the first product.
  int qpos = 0;
  float2 q_cos[KSTEPS / 2][2], q_sin[KSTEPS / 2][2], q_nw[KSTEPS][2];
  if (early) {
#pragma unroll
    for (int s = 0; s < DEC_STAGES - 1; ++s) {
      if (s < tiles) issue(s);
      cp_async_commit();
    }
    qpos = kvl > 0 ? fu.positions[b] : 0;
    if (qpos < 0 || qpos >= fu.max_positions) {
      if (threadIdx.x == 0 && kvl > 0) ullm_report(status, ULLM_STATUS_POSITION, b, qpos);
      qpos = 0;
    }
    const int c = (lane & 3) * 2;
    const float* cr = fu.cos_t + (long long)qpos * (D / 2);
    const float* sr = fu.sin_t + (long long)qpos * (D / 2);
#pragma unroll
    for (int kk = 0; kk < KSTEPS / 2; ++kk) {
      q_cos[kk][0] = *reinterpret_cast<const float2*>(cr + kk * 16 + c);
      q_cos[kk][1] = *reinterpret_cast<const float2*>(cr + kk * 16 + 8 + c);
      q_sin[kk][0] = *reinterpret_cast<const float2*>(sr + kk * 16 + c);
      q_sin[kk][1] = *reinterpret_cast<const float2*>(sr + kk * 16 + 8 + c);
    }
    if (fu.q_w != nullptr) {
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        q_nw[kk][0] = *reinterpret_cast<const float2*>(fu.q_w + kk * 16 + c);
        q_nw[kk][1] = *reinterpret_cast<const float2*>(fu.q_w + kk * 16 + 8 + c);
      }
    }
  }
  pdl_wait();

  // ---- Q fragments (A operand), rows >= group are zero -------------------------------
  unsigned qa[KSTEPS][4];
  {
    const int r0 = lane >> 2, r1 = r0 + 8, c = (lane & 3) * 2;
    const __nv_bfloat16* q0 = q + (long long)b * q_row_stride + (long long)(kh * group + r0) * D;
    const __nv_bfloat16* q1 = q + (long long)b * q_row_stride + (long long)(kh * group + r1) * D;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      qa[kk][0] = r0 < group ? *reinterpret_cast<const unsigned*>(q0 + kk * 16 + c) : 0u;
      qa[kk][1] = r1 < group ? *reinterpret_cast<const unsigned*>(q1 + kk * 16 + c) : 0u;
      qa[kk][2] = r0 < group ? *reinterpret_cast<const unsigned*>(q0 + kk * 16 + 8 + c) : 0u;
      qa[kk][3] = r1 < group ? *reinterpret_cast<const unsigned*>(q1 + kk * 16 + 8 + c) : 0u;
    }
  }
  uint4 new_kv = make_uint4(0, 0, 0, 0);  // this lane's 16 bytes of the new key (lanes < D / 8) or value (the next D / 8)
  bool have_new = false;
  if (fu.cos_t != nullptr) {
    // ---- q: RMSNorm over the head, then the rotation; a thread holds, of rows r0 and r1, the columns
    // 16 kk + c, + 1, + 8, + 9 (c = 2 (lane % 4)) for every kk: the rotation partner (D / 2 further) is its own
    // kk + KSTEPS / 2 ----
    const float* cr = fu.cos_t + (long long)qpos * (D / 2);
    const float* sr = fu.sin_t + (long long)qpos * (D / 2);
#pragma unroll
    for (int half = 0; half < 2; ++half) {  // row r0 (fragment words 0, 2), then row r1 (words 1, 3)
      float y[KSTEPS][4];
      float ss = 0.f;
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&qa[kk][half]);
        const __nv_bfloat162 bb = *reinterpret_cast<const __nv_bfloat162*>(&qa[kk][half + 2]);
        y[kk][0] = __bfloat162float(a.x), y[kk][1] = __bfloat162float(a.y);
        y[kk][2] = __bfloat162float(bb.x), y[kk][3] = __bfloat162float(bb.y);
        ss += y[kk][0] * y[kk][0] + y[kk][1] * y[kk][1] + y[kk][2] * y[kk][2] + y[kk][3] * y[kk][3];
      }
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      if (fu.q_w != nullptr) {
        const float rstd = rsqrtf(ss / (float)D + fu.eps);
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
          const float2 w0 = q_nw[kk][0], w1 = q_nw[kk][1];
          y[kk][0] *= rstd * w0.x, y[kk][1] *= rstd * w0.y, y[kk][2] *= rstd * w1.x, y[kk][3] *= rstd * w1.y;
        }
      }
#pragma unroll
      for (int kk = 0; kk < KSTEPS / 2; ++kk) {
        const float2 c0 = q_cos[kk][0], c1 = q_cos[kk][1];
        const float2 s0 = q_sin[kk][0], s1 = q_sin[kk][1];
        const float cs[4] = {c0.x, c0.y, c1.x, c1.y}, sn[4] = {s0.x, s0.y, s1.x, s1.y};
        float lo4[4], hi4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float a = y[kk][i], p2 = y[kk + KSTEPS / 2][i];
          lo4[i] = a * cs[i] - p2 * sn[i];
          hi4[i] = p2 * cs[i] + a * sn[i];
        }
        qa[kk][half] = pack_bf16(lo4[0], lo4[1]);
        qa[kk][half + 2] = pack_bf16(lo4[2], lo4[3]);
        qa[kk + KSTEPS / 2][half] = pack_bf16(hi4[0], hi4[1]);
        qa[kk + KSTEPS / 2][half + 2] = pack_bf16(hi4[2], hi4[3]);
      }
      // (rows >= group were loaded as zeros and stay zeros: 0 * rstd * w, rotated, is 0)
    }
    // ---- the new key and value: the warp whose keys end with the newest one prepares them, writes them to the
    // cache for the steps to come, and keeps them to put them into its own last tile once that has landed (what
    // the tile's load finds in the slot meanwhile does not matter) ----------------------------------------------
    if (fu.slot_mapping != nullptr && n_keys > 0 && w_end == lo + n_keys && w_end > w_begin) {
      constexpr int LW = D / 8;  // lanes of a row
      long long slot = fu.slot_mapping[b];
      if (slot >= fu.num_slots) {
        if (lane == 0) ullm_report(status, ULLM_STATUS_SLOT, b, (int)slot);
        slot = -1;
      }
      if (slot >= 0) {
        const int sl = lane % LW, which = lane / LW;  // 0: the key row, 1: the value row (further lanes idle)
        const __nv_bfloat16* src = q + (long long)b * q_row_stride + (long long)(num_q + (which == 1 ? num_kv : 0) + kh) * D + sl * 8;
        const uint4 raw = which < 2 ? *reinterpret_cast<const uint4*>(src) : make_uint4(0, 0, 0, 0);
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
        float y[8];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          y[i] = __bfloat162float(e[i]);
          ss += y[i] * y[i];
        }
#pragma unroll
        for (int off = LW / 2; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);  // every lane takes part
        if (fu.k_w != nullptr) {
          const float rstd = rsqrtf(ss / (float)D + fu.eps);
          const float4 w0 = *reinterpret_cast<const float4*>(fu.k_w + sl * 8), w1 = *reinterpret_cast<const float4*>(fu.k_w + sl * 8 + 4);
          y[0] *= rstd * w0.x, y[1] *= rstd * w0.y, y[2] *= rstd * w0.z, y[3] *= rstd * w0.w;
          y[4] *= rstd * w1.x, y[5] *= rstd * w1.y, y[6] *= rstd * w1.z, y[7] *= rstd * w1.w;
        }
        const int j0 = (sl % (LW / 2)) * 8;
        const float4 c0 = *reinterpret_cast<const float4*>(cr + j0), c1 = *reinterpret_cast<const float4*>(cr + j0 + 4);
        const float4 s0 = *reinterpret_cast<const float4*>(sr + j0), s1 = *reinterpret_cast<const float4*>(sr + j0 + 4);
        const float c8[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float s8[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        uint4 ov;
        __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&ov);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float partner = __shfl_xor_sync(0xffffffffu, y[i], LW / 2);
          const float v = sl < LW / 2 ? y[i] * c8[i] - partner * s8[i] : y[i] * c8[i] + partner * s8[i];
          ob[i] = __float2bfloat16_rn(v);
        }
        new_kv = which == 0 ? ov : raw;
        have_new = which < 2;
        if (which == 0) *reinterpret_cast<uint4*>(fu.k_cache + (slot * num_kv + kh) * D + sl * 8) = ov;
        if (which == 1) *reinterpret_cast<uint4*>(fu.v_cache + (slot * num_kv + kh) * D + sl * 8) = raw;
      }
    }
  }

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[NT_O][4];
#pragma unroll
  for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

  if (!early) {
#pragma unroll
    for (int s = 0; s < DEC_STAGES - 1; ++s) {
      if (s < tiles) issue(s);
      cp_async_commit();
    }
  }
  for (int it = 0; it < tiles; ++it) {
    if (it + DEC_STAGES - 1 < tiles) issue(it + DEC_STAGES - 1);
    cp_async_commit();
    cp_async_wait<DEC_STAGES - 1>();
    __syncwarp();
    unsigned char* kbuf = ring + (it % DEC_STAGES) * 2 * S::TILE_BYTES;
    unsigned char* vbuf = kbuf + S::TILE_BYTES;
    if (it == tiles - 1 && __any_sync(0xffffffffu, have_new)) {
      // the newest key and value, prepared above, go into their row of this tile
      if (have_new) {
        constexpr int LW = D / 8;
        const int row = w_end - 1 - (w_begin + it * DEC_TILE), ch = lane % LW;
        *reinterpret_cast<uint4*>((lane < LW ? kbuf : vbuf) + row * S::ROW_BYTES + ((ch ^ (row & 7)) * 16)) = new_kv;
      }
      __syncwarp();
    }
    // ---- scores: 2 n-tiles of 8 keys ------------------------------------------------
    float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      // even and odd k steps into accumulators of their own (four chains of KSTEPS / 2 dependent products
      // instead of two of KSTEPS: with one or two warps per scheduler that chain is what a tile waits for)
      float sd[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        const int mat = lane >> 3, row = (mat >> 1) * 8 + (lane & 7), ch = 2 * kk + (mat & 1);
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, kbuf + row * S::ROW_BYTES + ((ch ^ (row & 7)) * 16));
        if (kk & 1) {
          mma_bf16(sd[0], qa[kk], b0, b1);
          mma_bf16(sd[1], qa[kk], b2, b3);
        } else {
          mma_bf16(sc[0], qa[kk], b0, b1);
          mma_bf16(sc[1], qa[kk], b2, b3);
        }
      }
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[t][e] += sd[t][e];
    }
    // ---- mask, online softmax -------------------------------------------------------
    const int base = w_begin + it * DEC_TILE;
    float mx[2] = {m[0], m[1]};
#pragma unroll
    for (int t = 0; t < 2; ++t) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = base + t * 8 + (lane & 3) * 2 + (e & 1);
        const float v = key < w_end ? sc[t][e] * scale_log2 : -INFINITY;
        sc[t][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      alpha[r] = mx[r] == -INFINITY ? 1.f : dec_ex2(m[r] - mx[r]);
      m[r] = mx[r];
      l[r] *= alpha[r];
    }
    unsigned pa[4];
    {
      float p[2][4];
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          p[t][e] = m[e >> 1] == -INFINITY ? 0.f : dec_ex2(sc[t][e] - m[e >> 1]);
          l[e >> 1] += p[t][e];
        }
      pa[0] = pack_bf16(p[0][0], p[0][1]);
      pa[1] = pack_bf16(p[0][2], p[0][3]);
      pa[2] = pack_bf16(p[1][0], p[1][1]);
      pa[3] = pack_bf16(p[1][2], p[1][3]);
    }
    // ---- O = alpha O + P V ------------------------------------------------------------
    if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {  // (most tiles leave the maxima where they are)
#pragma unroll
      for (int j = 0; j < NT_O; ++j) {
        o[j][0] *= alpha[0]; o[j][1] *= alpha[0]; o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
      }
    }
#pragma unroll
    for (int j = 0; j < NT_O; j += 2) {
      const int mat = lane >> 3, row = (mat & 1) * 8 + (lane & 7), ch = j + (mat >> 1);
      unsigned b0, b1, b2, b3;
      ldmatrix_x4_trans(b0, b1, b2, b3, vbuf + row * S::ROW_BYTES + ((ch ^ (row & 7)) * 16));
      mma_bf16(o[j], pa, b0, b1);
      mma_bf16(o[j + 1], pa, b2, b3);
    }
    __syncwarp();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }

  // ---- merge the four warps in shared memory -----------------------------------------
  __syncthreads();
  float* mo = reinterpret_cast<float*>(smem);  // [warp][row 16][D + 2]
  {
    float* mine = mo + warp * 16 * (D + 2);
    const int r0 = lane >> 2, r1 = r0 + 8, c = (lane & 3) * 2;
#pragma unroll
    for (int j = 0; j < NT_O; ++j) {
      mine[r0 * (D + 2) + j * 8 + c] = o[j][0];
      mine[r0 * (D + 2) + j * 8 + c + 1] = o[j][1];
      mine[r1 * (D + 2) + j * 8 + c] = o[j][2];
      mine[r1 * (D + 2) + j * 8 + c + 1] = o[j][3];
    }
    if ((lane & 3) == 0) {
      mine[r0 * (D + 2) + D] = m[0];
      mine[r0 * (D + 2) + D + 1] = l[0];
      mine[r1 * (D + 2) + D] = m[1];
      mine[r1 * (D + 2) + D + 1] = l[1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < group * D; idx += blockDim.x) {
    const int r = idx / D, d = idx - r * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, mo[(w * 16 + r) * (D + 2) + D]);
    float ll = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float mw = mo[(w * 16 + r) * (D + 2) + D];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - mm);
      ll += mo[(w * 16 + r) * (D + 2) + D + 1] * f;
      acc += mo[(w * 16 + r) * (D + 2) + d] * f;
    }
    const int h = kh * group + r;
    if (num_splits == 1) {
      out[((long long)b * num_q + h) * D + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
    } else if (CL) {
      cm[r * (D + 2) + d] = acc;
      if (d == 0) {
        cm[r * (D + 2) + D] = mm;
        cm[r * (D + 2) + D + 1] = ll;
      }
    } else {
      const long long p = ((long long)b * num_q + h) * num_splits + split;
      part_o[p * D + d] = acc;
      if (d == 0) {
        part_ml[p * 2] = mm;
        part_ml[p * 2 + 1] = ll;
      }
    }
  }
  if (CL && num_splits > 1) {
    // The splits' partials meet: block `split` of the cluster finishes every num_splits-th output element, reading
    // all partials (its peers' through distributed shared memory) and adding them in split order, as the merge
    // kernel does: out = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M).
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    for (int idx = split * blockDim.x + threadIdx.x; idx < group * D; idx += num_splits * blockDim.x) {
      const int r = idx / D, d = idx - r * D;
      // all peers' values first (the loads through distributed shared memory are then in flight together: a
      // loop that adds as it loads pays their latency once per peer), then the arithmetic, in split order
      float ms[8], ls[8], as[8];
#pragma unroll
      for (int s2 = 0; s2 < 8; ++s2) {
        ms[s2] = -INFINITY, ls[s2] = 0.f, as[s2] = 0.f;
        if (s2 < num_splits) {
          const float* peer = cluster.map_shared_rank(cm, s2) + r * (D + 2);
          ms[s2] = peer[D];
          ls[s2] = peer[D + 1];
          as[s2] = peer[d];
        }
      }
      float mm = -INFINITY;
#pragma unroll
      for (int s2 = 0; s2 < 8; ++s2) mm = fmaxf(mm, ms[s2]);
      float ll = 0.f, acc = 0.f;
#pragma unroll
      for (int s2 = 0; s2 < 8; ++s2) {
        const float f = ms[s2] == -INFINITY ? 0.f : exp2f(ms[s2] - mm);
        ll += ls[s2] * f;
        acc += as[s2] * f;
      }
      out[((long long)b * num_q + kh * group + r) * D + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
    }
    cluster.sync();  // no block leaves while a peer may still read its partial
  }
}

// out[b, h, :] = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)
template <int D>
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    __nv_bfloat16* __restrict__ out, int num_splits) {
  pdl_launch_dependents();
  pdl_wait();
  const long long bh = blockIdx.x;
  const int d = threadIdx.x;
  if (d >= D) return;
  // eight splits at a time, all their loads issued before they are used (the count is small, the latency of a
  // chain of dependent loads is what this kernel would otherwise spend its time on)
  const float* ml = part_ml + bh * num_splits * 2;
  const float* po = part_o + bh * num_splits * D + d;
  float mm = -INFINITY;
  for (int s0 = 0; s0 < num_splits; s0 += 8) {
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = s0 + i < num_splits ? ml[(s0 + i) * 2] : -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) mm = fmaxf(mm, v[i]);
  }
  float ll = 0.f, acc = 0.f;
  for (int s0 = 0; s0 < num_splits; s0 += 8) {
    float ms[8], ls[8], os[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const bool on = s0 + i < num_splits;
      ms[i] = on ? ml[(s0 + i) * 2] : -INFINITY;
      ls[i] = on ? ml[(s0 + i) * 2 + 1] : 0.f;
      os[i] = on ? po[(long long)(s0 + i) * D] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // in split order: the same sum in every launch
      const float f = ms[i] == -INFINITY ? 0.f : exp2f(ms[i] - mm);
      ll += ls[i] * f;
      acc += os[i] * f;
    }
  }
  out[bh * D + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
}

static int g_decode_attr_set[2] = {0, 0};
static int g_decode_cluster = 1;  // 1: splits of 2 to 8 merge inside a cluster; 0: always scratch arrays + merge kernel

// 0 switches the cluster form off (tests and measurements compare the two).
extern "C" void ullm_decode_attention_cluster_merge(int on) { g_decode_cluster = on ? 1 : 0; }
// What the last launch used: 1 the cluster form, 0 the merge kernel (or a single split).
static int g_decode_last_cluster = 0;
extern "C" int ullm_decode_attention_last_used_cluster(void) { return g_decode_last_cluster; }

template <int D>
static int launch_decode(int which, const void* q, long long q_row_stride, const void* k_cache, const void* v_cache,
                         const int* block_table, int max_pages, const int* req_slots, const int* kv_len, void* out,
                         float* part_o, float* part_ml, int batch, int num_q, int num_kv, int page_size, int window,
                         float scale, int num_splits, long long num_pages, int* status, cudaStream_t st,
                         const DecFuse& fu) {
  using S = DecodeSmem<D>;
  if (!g_decode_attr_set[which]) {
    if (cudaFuncSetAttribute(decode_attention_kernel<D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::BYTES) !=
            cudaSuccess ||
        cudaFuncSetAttribute(decode_attention_kernel<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::BYTES) !=
            cudaSuccess)
      return ULLM_ERR_LAUNCH;
    cudaFuncSetAttribute(decode_attention_kernel<D, false>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(decode_attention_kernel<D, true>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    g_decode_attr_set[which] = 1;
  }
  dim3 grid(num_splits, num_kv, batch);
  g_decode_last_cluster = 0;
  if (g_decode_cluster == 1 && num_splits > 1 && num_splits <= 8) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(DEC_WARPS * 32);
    cfg.dynamicSmemBytes = (size_t)S::BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)num_splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_ullm_pdl ? 2 : 1;
    if (cudaLaunchKernelEx(&cfg, decode_attention_kernel<D, true>, (const __nv_bfloat16*)q, q_row_stride,
                           (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_table, max_pages, req_slots,
                           kv_len, (__nv_bfloat16*)out, part_o, part_ml, num_q, num_kv, page_size, window,
                           scale * 1.4426950408889634f, num_pages, status, fu) == cudaSuccess) {
      g_decode_last_cluster = 1;
      return ULLM_OK;
    }
    cudaGetLastError();
    g_decode_cluster = -1;  // this device does not take the cluster launch: scratch arrays and merge kernel from now on
  }
  int rc = ullm_launch_kernel(decode_attention_kernel<D, false>, grid, dim3(DEC_WARPS * 32), (size_t)S::BYTES, st,
      (const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_table,
      max_pages, req_slots, kv_len, (__nv_bfloat16*)out, part_o, part_ml, num_q, num_kv, page_size, window,
      scale * 1.4426950408889634f, num_pages, status, fu);
  if (rc != ULLM_OK) return rc;
  if (num_splits > 1)
    rc = ullm_launch_kernel(decode_merge_kernel<D>, dim3(batch * num_q), dim3(D), 0, st, (const float*)part_o,
                            (const float*)part_ml, (__nv_bfloat16*)out, num_splits);
  return rc;
}

// Sizes this kernel takes: bfloat16, head_dim 64 or 128, at most 16 query heads per kv head.
extern "C" int ullm_decode_attention_supported(int head_dim, int num_q, int num_kv) {
  if (num_kv <= 0 || num_q % num_kv) return 0;
  return (head_dim == 64 || head_dim == 128) && (num_q / num_kv) <= 16;
}

// Floats of scratch the split partials need: part_o then part_ml.
extern "C" long long ullm_decode_attention_scratch_floats(int batch, int num_q, int head_dim, int num_splits) {
  return (long long)batch * num_q * num_splits * (head_dim + 2);
}

static int decode_attention_impl(const void* q, long long q_row_stride, const void* k_cache, const void* v_cache,
                                 const int* block_table, int max_pages, const int* req_slots, const int* kv_len,
                                 void* out, float* scratch, int batch, int num_q, int num_kv, int head_dim,
                                 int page_size, int window, float scale, int num_splits, long long num_pages,
                                 int* status, void* stream, const DecFuse& fu) {
  cudaStream_t st = (cudaStream_t)stream;
  if (batch < 0 || num_q <= 0 || num_kv <= 0 || page_size <= 0 || max_pages <= 0 || num_splits <= 0 || window < 0)
    return ULLM_ERR_BAD_SIZE;
  if (!ullm_decode_attention_supported(head_dim, num_q, num_kv)) return ULLM_ERR_UNSUPPORTED;
  if (num_splits > 1 && scratch == nullptr) return ULLM_ERR_BAD_SIZE;
  if (batch == 0) return ULLM_OK;
  float* part_o = scratch;
  float* part_ml = scratch != nullptr ? scratch + (long long)batch * num_q * num_splits * head_dim : nullptr;
  if (head_dim == 64)
    return launch_decode<64>(0, q, q_row_stride, k_cache, v_cache, block_table, max_pages, req_slots, kv_len, out,
                             part_o, part_ml, batch, num_q, num_kv, page_size, window, scale, num_splits, num_pages,
                             status, st, fu);
  return launch_decode<128>(1, q, q_row_stride, k_cache, v_cache, block_table, max_pages, req_slots, kv_len, out, part_o,
                            part_ml, batch, num_q, num_kv, page_size, window, scale, num_splits, num_pages, status, st, fu);
}

extern "C" int ullm_decode_attention(const void* q, long long q_row_stride, const void* k_cache, const void* v_cache,
                                     const int* block_table, int max_pages, const int* req_slots, const int* kv_len,
                                     void* out, float* scratch, int batch, int num_q, int num_kv, int head_dim,
                                     int page_size, int window, float scale, int num_splits, long long num_pages,
                                     int* status, void* stream) {
  DecFuse fu = {};
  return decode_attention_impl(q, q_row_stride, k_cache, v_cache, block_table, max_pages, req_slots, kv_len, out, scratch,
                               batch, num_q, num_kv, head_dim, page_size, window, scale, num_splits, num_pages, status,
                               stream, fu);
}

// The same with q, the new key and the new value taken as the projection left them: the kernel applies the
// per-head RMSNorm (weights may be null) and the rotation itself and writes key and value to their cache slot
// (`slot_mapping` null: nothing is written).  qkv rows: [q heads | k heads | v heads], one row per request.
extern "C" int ullm_decode_attention_fused(const void* qkv, long long q_row_stride, void* k_cache, void* v_cache,
                                           const int* block_table, int max_pages, const int* req_slots,
                                           const int* kv_len, void* out, float* scratch, int batch, int num_q,
                                           int num_kv, int head_dim, int page_size, int window, float scale,
                                           int num_splits, long long num_pages, const float* q_w, const float* k_w,
                                           float eps, const float* cos_t, const float* sin_t, int max_positions,
                                           const int* positions, const int* slot_mapping, int* status, void* stream) {
  if (cos_t == nullptr || sin_t == nullptr || positions == nullptr || max_positions <= 0) return ULLM_ERR_BAD_SIZE;
  DecFuse fu;
  fu.q_w = q_w;
  fu.k_w = k_w;
  fu.cos_t = cos_t;
  fu.sin_t = sin_t;
  fu.positions = positions;
  fu.slot_mapping = slot_mapping;
  fu.k_cache = (__nv_bfloat16*)k_cache;
  fu.v_cache = (__nv_bfloat16*)v_cache;
  fu.num_slots = num_pages * page_size;
  fu.max_positions = max_positions;
  fu.eps = eps;
  return decode_attention_impl(qkv, q_row_stride, k_cache, v_cache, block_table, max_pages, req_slots, kv_len, out,
                               scratch, batch, num_q, num_kv, head_dim, page_size, window, scale, num_splits, num_pages,
                               status, stream, fu);
}

// ---------------------------------------------------------------------------
// The variant for callers that cannot allocate (declared in no_alloc.h).
// ---------------------------------------------------------------------------
#include "no_alloc.h"

// Scratch for the split partials, resident on every device that loads the library.
static __device__ __align__(256) float g_static_scratch[ULLM_STATIC_SCRATCH_FLOATS];

// In host code `g_static_scratch` is only a handle for the symbol; the device
// address comes from cudaGetSymbolAddress, looked up once per device.
#define ULLM_MAX_DEVICES 64
static float* g_static_scratch_addr[ULLM_MAX_DEVICES] = {nullptr};

extern "C" long long ullm_decode_attention_static_capacity(void) { return ULLM_STATIC_SCRATCH_FLOATS; }

extern "C" int ullm_decode_attention_static(const void* q, long long q_row_stride, const void* k_cache,
                                            const void* v_cache, const int* block_table, int max_pages,
                                            const int* req_slots, const int* kv_len, void* out, int batch, int num_q,
                                            int num_kv, int head_dim, int page_size, int window, float scale,
                                            int num_splits, long long num_pages, int* status, void* stream) {
  if (batch < 0 || num_q <= 0 || num_kv <= 0 || head_dim <= 0 || num_splits <= 0) return ULLM_ERR_BAD_SIZE;
  // a single split writes no partials: nothing of the array is touched, so nothing has to fit
  if (num_splits > 1 &&
      ullm_decode_attention_scratch_floats(batch, num_q, head_dim, num_splits) > ULLM_STATIC_SCRATCH_FLOATS)
    return ULLM_ERR_SCRATCH_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= ULLM_MAX_DEVICES) return ULLM_ERR_LAUNCH;
  if (g_static_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_static_scratch) != cudaSuccess || p == nullptr) return ULLM_ERR_LAUNCH;
    g_static_scratch_addr[dev] = p;
  }
  return ullm_decode_attention(q, q_row_stride, k_cache, v_cache, block_table, max_pages, req_slots, kv_len, out,
                               g_static_scratch_addr[dev], batch, num_q, num_kv, head_dim, page_size, window, scale,
                               num_splits, num_pages, status, stream);
}
