// The inner part of the bfloat16 decode attention kernels: one warp runs an online softmax over a range of
// one request's keys for the query heads that share one kv head, with tensor-core products (mma.sync
// m16n8k16, fp32 accumulate); K and V rows are gathered page by page with cp.async into a three-stage ring
// per warp.  Used by the kernel that splits every request's keys evenly (attention_decode.cu) and by the
// one that splits the whole batch's keys evenly over the blocks (attention_decode_balanced.cu).
#pragma once

#include "common.cuh"

#define DEC_WARPS 4
#define DEC_TILE 16   // keys per warp iteration
#define DEC_STAGES 3

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool pred) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3,
                                                  const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// shared memory of one block: per warp a ring of K and V tiles; afterwards reused for the merge
template <int D>
struct DecodeSmem {
  static constexpr int ROW_BYTES = D * 2;
  static constexpr int TILE_BYTES = DEC_TILE * ROW_BYTES;
  static constexpr int WARP_BYTES = DEC_STAGES * 2 * TILE_BYTES;
  static constexpr int RING_BYTES = DEC_WARPS * WARP_BYTES;
  static constexpr int MERGE_BYTES = DEC_WARPS * 16 * (D + 2) * 4;
  static constexpr int BYTES = RING_BYTES > MERGE_BYTES ? RING_BYTES : MERGE_BYTES;
};

// One warp's share: keys [w_begin, w_end) of the request whose block-table row is `bt`, kv head `kh`.
// `q_b`: the request's row of q ([num_q, D] bf16).  `ring`: this warp's DecodeSmem<D>::WARP_BYTES of shared
// memory.  Returns the running maximum m (log2 domain), the sum l (already added over the quad) and the
// unnormalised output o, in the accumulator layout of the tensor instruction: rows lane/4 and lane/4 + 8.
template <int D>
__device__ __forceinline__ void decode_warp_keys(const __nv_bfloat16* __restrict__ q_b, int kh, int group,
                                                 const __nv_bfloat16* __restrict__ k_cache,
                                                 const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ bt,
                                                 long long kv_row, int page_size, long long num_pages, int w_begin,
                                                 int w_end, float scale_log2, unsigned char* ring, int b, int* status,
                                                 float (&m)[2], float (&l)[2], float (&o)[D / 8][4]) {
  constexpr int CHUNKS = D / 8;        // 16-byte chunks per row
  constexpr int KSTEPS = D / 16;       // k-steps of the score product
  constexpr int NT_O = D / 8;          // n-tiles of the output
  using S = DecodeSmem<D>;
  const int lane = threadIdx.x & 31;
  const int tiles = (w_end - w_begin + DEC_TILE - 1) / DEC_TILE;
  // Block-table entries of the range, 32 at a time, one per lane: read here, together with q, so that no
  // load of keys has to wait for a load of its page id inside the loop.
  const int range_last_page = tiles > 0 ? (w_end - 1) / page_size : -1;
  int win_base = tiles > 0 ? w_begin / page_size : 0;
  int win_page = win_base + lane <= range_last_page ? bt[win_base + lane] : -1;
  // ---- Q fragments (A operand), rows >= group are zero -------------------------------
  unsigned qa[KSTEPS][4];
  {
    const int r0 = lane >> 2, r1 = r0 + 8, c = (lane & 3) * 2;
    const __nv_bfloat16* q0 = q_b + (long long)(kh * group + r0) * D;
    const __nv_bfloat16* q1 = q_b + (long long)(kh * group + r1) * D;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      qa[kk][0] = r0 < group ? *reinterpret_cast<const unsigned*>(q0 + kk * 16 + c) : 0u;
      qa[kk][1] = r1 < group ? *reinterpret_cast<const unsigned*>(q1 + kk * 16 + c) : 0u;
      qa[kk][2] = r0 < group ? *reinterpret_cast<const unsigned*>(q0 + kk * 16 + 8 + c) : 0u;
      qa[kk][3] = r1 < group ? *reinterpret_cast<const unsigned*>(q1 + kk * 16 + 8 + c) : 0u;
    }
  }

  auto issue = [&](int tile) {
    unsigned char* kbuf = ring + (tile % DEC_STAGES) * 2 * S::TILE_BYTES;
    unsigned char* vbuf = kbuf + S::TILE_BYTES;
    const int base = w_begin + tile * DEC_TILE;
    // the tile's pages come from the window of 32 block-table entries that the lanes hold; it moves on when
    // the tile reaches beyond it (a tile of 16 keys spans at most 16 pages)
    const int page_last = (min(base + DEC_TILE, w_end) - 1) / page_size;
    if (page_last > win_base + 31) {
      win_base = base / page_size;
      win_page = win_base + lane <= range_last_page ? bt[win_base + lane] : -1;
    }
    // lanes 0..15 look up the slot of row `lane`
    const int key = base + lane;
    const bool valid = lane < DEC_TILE && key < w_end;
    const int page = __shfl_sync(0xffffffffu, win_page, valid ? key / page_size - win_base : 0);
    long long my_slot = -1;
    if (valid) {
      if (page < 0 || page >= num_pages) ullm_report(status, ULLM_STATUS_PAGE, b, page);
      else my_slot = (long long)page * page_size + key % page_size;
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

  m[0] = m[1] = -INFINITY;
  l[0] = l[1] = 0.f;
#pragma unroll
  for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

#pragma unroll
  for (int s = 0; s < DEC_STAGES - 1; ++s) {
    if (s < tiles) issue(s);
    cp_async_commit();
  }
  for (int it = 0; it < tiles; ++it) {
    if (it + DEC_STAGES - 1 < tiles) issue(it + DEC_STAGES - 1);
    cp_async_commit();
    cp_async_wait<DEC_STAGES - 1>();
    __syncwarp();
    const unsigned char* kbuf = ring + (it % DEC_STAGES) * 2 * S::TILE_BYTES;
    const unsigned char* vbuf = kbuf + S::TILE_BYTES;
    // ---- scores: 2 n-tiles of 8 keys ------------------------------------------------
    float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      const int mat = lane >> 3, row = (mat >> 1) * 8 + (lane & 7), ch = 2 * kk + (mat & 1);
      unsigned b0, b1, b2, b3;
      ldmatrix_x4(b0, b1, b2, b3, kbuf + row * S::ROW_BYTES + ((ch ^ (row & 7)) * 16));
      mma_bf16(sc[0], qa[kk], b0, b1);
      mma_bf16(sc[1], qa[kk], b2, b3);
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
      alpha[r] = mx[r] == -INFINITY ? 1.f : exp2f(m[r] - mx[r]);
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
          p[t][e] = m[e >> 1] == -INFINITY ? 0.f : exp2f(sc[t][e] - m[e >> 1]);
          l[e >> 1] += p[t][e];
        }
      pa[0] = pack_bf16(p[0][0], p[0][1]);
      pa[1] = pack_bf16(p[0][2], p[0][3]);
      pa[2] = pack_bf16(p[1][0], p[1][1]);
      pa[3] = pack_bf16(p[1][2], p[1][3]);
    }
    // ---- O = alpha O + P V ------------------------------------------------------------
#pragma unroll
    for (int j = 0; j < NT_O; j += 2) {
      o[j][0] *= alpha[0]; o[j][1] *= alpha[0]; o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
      o[j + 1][0] *= alpha[0]; o[j + 1][1] *= alpha[0]; o[j + 1][2] *= alpha[1]; o[j + 1][3] *= alpha[1];
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

}

// The warps' (m, l, o) into shared memory, [warp][row 16][D + 2] floats (o, then m, then l), behind a barrier
// on both sides: the ring is dead before it is overwritten, and the rows are complete when the call returns.
template <int D>
__device__ __forceinline__ void decode_block_gather(float* mo, const float (&m)[2], const float (&l)[2],
                                                    const float (&o)[D / 8][4]) {
  constexpr int NT_O = D / 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
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
}

// Row r, element d of the block's result from the gathered rows: (max, sum, unnormalised value).
template <int D>
__device__ __forceinline__ void decode_block_combine(const float* mo, int r, int d, float& mm, float& ll, float& acc) {
  mm = -INFINITY;
#pragma unroll
  for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, mo[(w * 16 + r) * (D + 2) + D]);
  ll = 0.f;
  acc = 0.f;
#pragma unroll
  for (int w = 0; w < DEC_WARPS; ++w) {
    const float mw = mo[(w * 16 + r) * (D + 2) + D];
    const float f = mw == -INFINITY ? 0.f : exp2f(mw - mm);
    ll += mo[(w * 16 + r) * (D + 2) + D + 1] * f;
    acc += mo[(w * 16 + r) * (D + 2) + d] * f;
  }
}
