// out[M, N] = x[M, K] . W[N, K]^T for few rows (M <= 64, the decode step's
// matrix products), bfloat16 in, 32-bit accumulate, bfloat16 or float32 out;
// optionally out[M, N/2] = act(gate) * up for a weight that stacks gate rows on
// up rows (the gated feed-forward's first product with its activation fused).
//
// The weight matrix is the big operand and is read exactly once; the kernel is a
// persistent streaming pipeline around the 5th-generation tensor cores:
//
//   * W is the A operand of tcgen05.mma (M = 128 weight rows per tile), x the B
//     operand (N = the batch rows padded to 16/32/48/64): "swap A/B", so that the
//     128-wide side of the instruction is filled by weight rows, not by the batch.
//   * The work is the list of (tile of 128 weight rows, block of 64 k) units in
//     tile-major order, cut into one contiguous, equally long range per block; the
//     grid is one block per SM.  Every SM therefore streams the same number of
//     weight bytes whatever N and K are.  A range may end inside a tile: that
//     tile's partial sums go to a workspace in global memory and the block that
//     arrives last at the tile's counter adds the partials in block order (the
//     result does not depend on who is last) and writes the output.  No block ever
//     waits for another block.
//   * Warp 0 (one thread) issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle)
//     of 128 x 64 weight tiles and Mpad x 64 activation tiles into a ring of
//     shared-memory stages; warp 1 (one thread) issues the MMAs into one of two
//     accumulators [128 lanes x Mpad columns] in tensor memory; warps 2..5 drain a
//     finished accumulator (tcgen05.ld), add bias, apply the activation, write,
//     while the other accumulator fills.  mbarriers carry "stage full" (TMA
//     transaction bytes), "stage free", "accumulator full" (tcgen05.commit) and
//     "accumulator drained".
//   * The weights do not depend on the kernel before this one in the stream: with
//     programmatic dependent launch the first ring of weight tiles is requested
//     before griddepcontrol.wait.
//   * Every load is issued by the block that uses it (no multicast).
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT polls the kernel records
// ULLM_STATUS_TIMEOUT in the status word, stops waiting, still frees its tensor
// memory and returns.  The workspace and the counters belong to one stream: two
// of these products must not run concurrently on different streams.
#include "tcgen05_util.cuh"

#define LIN_BM 128        // weight rows per block (UMMA M)
#define LIN_BK 128        // k elements per stage: two halves of 64 (128 bytes of bf16 = one swizzle row each)
#define LIN_A_HALF (LIN_BM * 128)  // bytes of one half of a weight tile
#define LIN_THREADS 192      // warp 0: loads, warp 1: MMA, warps 2..5: epilogue
#define LIN_MAX_STAGES 12
struct LinParams {
  int M, N, K;          // rows of x, rows of W, shared dimension
  int m_pad;            // M rounded up to 16
  int k_blocks;         // ceil(K / 128)
  int tail_halves;      // halves of 64 k that the last k block holds (1 or 2)
  int n_tiles;          // tiles of weight rows
  int stages;
  int out_f32;          // 1: float32 output, 0: bfloat16
  int act;              // 0: plain product; 1: silu(gate) * up; 2: gelu_tanh(gate) * up
  int n_out;            // columns of out: N, or N / 2 with an activation
  long long units;      // n_tiles * k_blocks
  void* out;            // [M, n_out]
  const void* bias;     // [N] bf16 or null
  float* ws;            // [blocks][2][m_pad][128] partial sums
  int* counters;        // [n_tiles], zero between launches
  int* status;
};

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Weight tile of unit (tile t, k block kb) into the stage at `dst`, one box per half of 64 k.  Plain: rows
// 128 t .. 128 t + 127.  With an activation the map is three-dimensional [2][n_out][K] and a box holds gate
// rows 64 t .. 64 t + 63 above the same rows of up (rows beyond n_out are filled with zeros in both).
__device__ __forceinline__ void lin_load_a(unsigned char* dst, const CUtensorMap* map_w, uint64_t* bar,
                                           const LinParams& p, int t, int kb, int halves) {
  for (int h = 0; h < halves; ++h) {
    if (p.act == 0) tma_load_2d(dst + h * LIN_A_HALF, map_w, bar, kb * LIN_BK + h * 64, t * LIN_BM);
    else tma_load_3d(dst + h * LIN_A_HALF, map_w, bar, kb * LIN_BK + h * 64, t * 64, 0);
  }
}
// The activations' tile of k block kb (all rows of x) behind the stage's two weight halves.
__device__ __forceinline__ void lin_load_b(unsigned char* dst, const CUtensorMap* map_x, uint64_t* bar, int b_bytes,
                                           int kb, int halves) {
  for (int h = 0; h < halves; ++h)
    tma_load_2d(dst + 2 * LIN_A_HALF + h * b_bytes, map_x, bar, kb * LIN_BK + h * 64, 0);
}

// dynamic shared memory: [stages] x (weight halves 2 x 16 KB | activation halves 2 x m_pad*128 B), 1024-byte
// aligned, then [m_pad][64] floats for the gate/up exchange of the fused activation
__global__ void __launch_bounds__(LIN_THREADS, 1)
linear_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      const LinParams p) {
  extern __shared__ unsigned char lin_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[LIN_MAX_STAGES], empty_bar[LIN_MAX_STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int last_flag, wait_flag[2];
  pdl_launch_dependents();
  unsigned char* tiles = (unsigned char*)(((uintptr_t)lin_smem_raw + 1023) & ~(uintptr_t)1023);
  const int b_bytes = p.m_pad * 128;                         // one half of the activations' tile (a multiple of 2 KB)
  const int stage_bytes = 2 * LIN_A_HALF + 2 * b_bytes;
  const int half_tx = LIN_A_HALF + b_bytes;                  // bytes that one half of a unit brings
  float* xchg = reinterpret_cast<float*>(tiles + (size_t)p.stages * stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long G = gridDim.x, blk = blockIdx.x;
  const long long u0 = blk * p.units / G, u1 = (blk + 1) * p.units / G;  // this block's units
  const int my_units = (int)(u1 - u0);
  const uint32_t tmem_cols = p.m_pad <= 16 ? 32 : (p.m_pad <= 32 ? 64 : 128);  // two accumulators

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_full[0], 1);
    mbar_init(&acc_full[1], 1);
    mbar_init(&acc_empty[0], 4);
    mbar_init(&acc_empty[1], 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    // The weights do not depend on the kernel before this one: the first ring of weight tiles is
    // requested at once, before tensor memory is set up and before pdl_wait().
    const int first = min(p.stages, my_units);
    int t = (int)(u0 / p.k_blocks), kb = (int)(u0 % p.k_blocks);
    for (int i = 0; i < first; ++i) {
      const int halves = kb == p.k_blocks - 1 ? p.tail_halves : 2;
      mbar_expect_tx(&full_bar[i], halves * half_tx);
      lin_load_a(tiles + i * stage_bytes, &map_w, &full_bar[i], p, t, kb, halves);
      if (++kb == p.k_blocks) kb = 0, ++t;
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
  pdl_wait();  // from here on the kernel before this one is complete: x may be read, out and ws written

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: TMA loads -------------------------------------------------------------
      const int first = min(p.stages, my_units);
      int t = (int)(u0 / p.k_blocks), kb = (int)(u0 % p.k_blocks);  // unit i's tile and k block, kept by stepping
      for (int i = 0; i < first; ++i) {
        lin_load_b(tiles + i * stage_bytes, &map_x, &full_bar[i], b_bytes, kb, kb == p.k_blocks - 1 ? p.tail_halves : 2);
        if (++kb == p.k_blocks) kb = 0, ++t;
      }
      int s = first == p.stages ? 0 : first;
      uint32_t parity = 0;  // of the stage's "free" barrier: first refill waits for phase 0 to complete
      for (int i = first; i < my_units; ++i) {
        if (!mbar_wait(&empty_bar[s], parity)) {
          ullm_report(p.status, ULLM_STATUS_TIMEOUT, 1, i);
          break;
        }
        unsigned char* a = tiles + s * stage_bytes;
        const int halves = kb == p.k_blocks - 1 ? p.tail_halves : 2;
        mbar_expect_tx(&full_bar[s], halves * half_tx);
        lin_load_a(a, &map_w, &full_bar[s], p, t, kb, halves);
        lin_load_b(a, &map_x, &full_bar[s], b_bytes, kb, halves);
        if (++kb == p.k_blocks) kb = 0, ++t;
        if (++s == p.stages) s = 0, parity ^= 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----------------------------------------------------------------------
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.m_pad >> 3) << 17) |
                             ((uint32_t)(LIN_BM >> 4) << 24);
      // Descriptors step with the stage (address fields count 16 bytes).  The loop is kept short: this one
      // thread's instructions are the pipeline's clock while a prefetched ring drains.
      const uint64_t desc0 = umma_desc(tiles);
      const uint32_t desc_hi = (uint32_t)(desc0 >> 32), lo0 = (uint32_t)desc0;
      const uint32_t stage_step = (uint32_t)stage_bytes >> 4, b_step = (uint32_t)b_bytes >> 4;
      const uint32_t full0 = lin_smem(&full_bar[0]), empty0 = lin_smem(&empty_bar[0]);
      uint32_t a_lo = lo0, full_s = full0, empty_s = empty0;
      bool ok = true;
      int seg = 0, s = 0;
      uint32_t phase = 0;
      int k0 = (int)(u0 % p.k_blocks);
      for (long long u = u0; u < u1 && ok; ++seg) {
        const int n = (int)min((long long)(p.k_blocks - k0), u1 - u);
        const int buf = seg & 1;
        if (!mbar_wait(&acc_empty[buf], ((seg >> 1) & 1) ^ 1)) {  // the epilogue has drained this accumulator
          ullm_report(p.status, ULLM_STATUS_TIMEOUT, 4, seg);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d = tmem_d + (uint32_t)(buf * p.m_pad);
        const int q_tail = k0 + n == p.k_blocks && p.tail_halves == 1 ? n - 1 : n;  // the unit that has one half only
        for (int q = 0; q < n; ++q) {
          if (!mbar_wait_addr(full_s, phase)) {
            ullm_report(p.status, ULLM_STATUS_TIMEOUT, 2, seg);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t b_lo = a_lo + (2 * LIN_A_HALF >> 4);
          // 16 bf16 = 32 bytes further along the swizzled row: +2 in the 16-byte address field
          umma_bf16_lo<-1>(d, a_lo, b_lo, desc_hi, idesc, q > 0 ? 1u : 0u);
          umma_bf16_lo<1>(d, a_lo + 2, b_lo + 2, desc_hi, idesc);
          umma_bf16_lo<1>(d, a_lo + 4, b_lo + 4, desc_hi, idesc);
          umma_bf16_lo<1>(d, a_lo + 6, b_lo + 6, desc_hi, idesc);
          if (q != q_tail) {
            const uint32_t a1 = a_lo + (LIN_A_HALF >> 4), b1 = b_lo + b_step;
            umma_bf16_lo<1>(d, a1, b1, desc_hi, idesc);
            umma_bf16_lo<1>(d, a1 + 2, b1 + 2, desc_hi, idesc);
            umma_bf16_lo<1>(d, a1 + 4, b1 + 4, desc_hi, idesc);
            umma_bf16_lo<1>(d, a1 + 6, b1 + 6, desc_hi, idesc);
          }
          umma_commit_addr(empty_s);  // the stage is free once these MMAs have read it
          a_lo += stage_step, full_s += 8, empty_s += 8;
          if (++s == p.stages) s = 0, phase ^= 1, a_lo = lo0, full_s = full0, empty_s = empty0;
        }
        if (ok) umma_commit(&acc_full[buf]);  // the accumulator is complete once every MMA above is
        u += n;
        k0 = 0;
      }
    }
  } else {
    // ---- epilogue: warps 2..5; a warp reads the accumulator lanes 32 (warp % 4) .. + 31 ----------
    const int quarter = warp & 3;
    const int f = quarter * 32 + lane;  // row of the tile (accumulator lane)
    const int et = threadIdx.x - 64;    // 0..127 among the epilogue threads
    const __nv_bfloat16* bias = (const __nv_bfloat16*)p.bias;
    int seg = 0;
    for (long long u = u0; u < u1; ++seg) {
      const int t = (int)(u / p.k_blocks), k0 = (int)(u % p.k_blocks);
      const int n = (int)min((long long)(p.k_blocks - k0), u1 - u);
      const int buf = seg & 1;
      u += n;
      // One thread waits (bounded) and tells the others, so that all 128 take the same way out.
      if (et == 0) {
        const bool got = mbar_wait(&acc_full[buf], (seg >> 1) & 1);
        if (!got) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 3, seg);
        wait_flag[seg & 1] = got ? 1 : 0;
      }
      epi_bar_sync();
      if (wait_flag[seg & 1] == 0) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float acc[64];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (c * 16 < p.m_pad) {
          float v[16];
          tmem_ld16(tmem_d + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * p.m_pad + c * 16), v);
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c * 16 + j] = v[j];
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);  // the MMA warp may fill this accumulator again

      bool finish = true;  // does this block write the tile's output?
      if (n < p.k_blocks) {
        // part of a tile: park the partial sums, count, and finish the tile if every other part is in
        float* mine = p.ws + ((size_t)(blk * 2 + (seg == 0 ? 0 : 1)) * p.m_pad) * LIN_BM;
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (j < p.m_pad) __stcg(&mine[j * LIN_BM + f], acc[j]);
        __threadfence();
        epi_bar_sync();
        const long long tu0 = (long long)t * p.k_blocks, tu1 = tu0 + p.k_blocks - 1;  // the tile's first, last unit
        const long long b_first = ((tu0 + 1) * G + p.units - 1) / p.units - 1;         // the blocks they belong to
        const long long b_last = ((tu1 + 1) * G + p.units - 1) / p.units - 1;
        if (et == 0) {
          const int parts = (int)(b_last - b_first + 1);
          const int last = atomicAdd(&p.counters[t], 1) == parts - 1;
          if (last) p.counters[t] = 0;  // every part has counted: ready for the next launch
          __threadfence();
          last_flag = last;
        }
        epi_bar_sync();
        finish = last_flag != 0;
        if (finish) {
          // Parts in block order (the same sum whoever is last), four parts' loads in flight at a time.
          const float* base = p.ws + f;
          const size_t part_floats = (size_t)p.m_pad * LIN_BM;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (c * 16 < p.m_pad) {
              float sum[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) sum[j] = 0.f;
              for (long long b0 = b_first; b0 <= b_last; b0 += 4) {
                float v[4][16];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const long long b = b0 + q;
                  const bool on = b <= b_last;
                  // a block's part of this tile is its first (slot 0) iff its range starts inside the tile
                  const int slot = b * p.units >= tu0 * G ? 0 : 1;
                  const float* part = base + (size_t)(b * 2 + slot) * part_floats + (size_t)(c * 16) * LIN_BM;
#pragma unroll
                  for (int j = 0; j < 16; ++j) v[q][j] = on ? __ldcg(&part[j * LIN_BM]) : 0.f;
                }
#pragma unroll
                for (int q = 0; q < 4; ++q)
#pragma unroll
                  for (int j = 0; j < 16; ++j) sum[j] += v[q][j];
              }
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[c * 16 + j] = sum[j];
            }
          }
        }
      }
      if (p.act == 0) {
        const int col = t * LIN_BM + f;
        if (finish && col < p.N) {
          const float bv = bias != nullptr ? __bfloat162float(bias[col]) : 0.f;
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            if (j < p.M) {
              const float v = acc[j] + bv;
              if (p.out_f32) ((float*)p.out)[(long long)j * p.N + col] = v;
              else ((__nv_bfloat16*)p.out)[(long long)j * p.N + col] = __float2bfloat16_rn(v);
            }
          }
        }
      } else if (finish) {  // uniform over the epilogue threads
        // rows 0..63 of the tile are gate features, rows 64..127 the same features of up
        if (f >= 64) {
#pragma unroll
          for (int j = 0; j < 64; ++j)
            if (j < p.m_pad) xchg[j * 64 + (f - 64)] = acc[j];
        }
        epi_bar_sync();
        const int col = t * 64 + f;
        if (f < 64 && col < p.n_out) {
          const float bg = bias != nullptr ? __bfloat162float(bias[col]) : 0.f;
          const float bu = bias != nullptr ? __bfloat162float(bias[p.n_out + col]) : 0.f;
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            if (j < p.M) {
              const float g = acc[j] + bg, up = xchg[j * 64 + f] + bu;
              const float v = (p.act == 1 ? act_silu(g) : act_gelu_tanh(g)) * up;
              if (p.out_f32) ((float*)p.out)[(long long)j * p.n_out + col] = v;
              else ((__nv_bfloat16*)p.out)[(long long)j * p.n_out + col] = __float2bfloat16_rn(v);
            }
          }
        }
        epi_bar_sync();  // xchg is free again
      }
    }
  }
  __syncwarp();  // the lanes of the two single-thread roles wait here for their lane 0
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(tmem_cols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
// Shapes this kernel takes: 1 <= M <= 64, K a multiple of 8 (16-byte rows for TMA), 16-byte aligned bases;
// with an activation N is even (gate rows above up rows).
extern "C" int ullm_linear_tcgen05_supported(int M, int N, int K) {
  return M >= 1 && M <= 64 && N >= 1 && K >= 8 && K % 8 == 0;
}

static int g_lin_attr_set = 0;
static int g_lin_sms = 0;

// Blocks a launch uses (one per SM at most): the workspace holds 2 * m_pad * 128 floats for each.
extern "C" int ullm_linear_tcgen05_blocks() {
  if (g_lin_sms == 0) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      return 0;
    g_lin_sms = sms;
  }
  return g_lin_sms;
}

// act: 0 none, 1 silu(gate) * up, 2 gelu_tanh(gate) * up (out is [M, N / 2]).  ws: float workspace of ws_floats
// floats; counters: n_counters ints, zero at the first launch (the kernel leaves them zero).
extern "C" int ullm_linear_tcgen05(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                                   int out_f32, int act, float* ws, long long ws_floats, int* counters,
                                   int n_counters, int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (!ullm_linear_tcgen05_supported(M, N, K)) return ULLM_ERR_UNSUPPORTED;
  if (act < 0 || act > 2 || (act != 0 && N % 2 != 0)) return ULLM_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return ULLM_ERR_UNSUPPORTED;
  const int sms = ullm_linear_tcgen05_blocks();
  if (sms <= 0) return ULLM_ERR_LAUNCH;
  LinParams p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.m_pad = (M + 15) / 16 * 16;
  p.k_blocks = (K + LIN_BK - 1) / LIN_BK;
  p.tail_halves = K - (p.k_blocks - 1) * LIN_BK > 64 ? 2 : 1;
  p.act = act;
  p.n_out = act != 0 ? N / 2 : N;
  p.n_tiles = act != 0 ? (p.n_out + 63) / 64 : (N + LIN_BM - 1) / LIN_BM;
  p.units = (long long)p.n_tiles * p.k_blocks;
  p.out_f32 = out_f32;
  p.out = out;
  p.bias = bias;
  p.ws = ws;
  p.counters = counters;
  p.status = status;
  const int blocks = (int)(p.units < sms ? p.units : sms);
  if (p.n_tiles > n_counters || (long long)blocks * 2 * p.m_pad * LIN_BM > ws_floats || ws == nullptr ||
      counters == nullptr)
    return ULLM_ERR_UNSUPPORTED;
  const int stage_bytes = 2 * LIN_A_HALF + 2 * p.m_pad * 128;
  const int xchg_bytes = act != 0 ? p.m_pad * 64 * 4 : 0;
  // Stages: the ring is what a block holds in flight, and what it has prefetched while it waits for the kernel
  // before it: all the shared memory a block can have.
  const int ring_kb = 224;
  int stages = (ring_kb * 1024 - 1024 - xchg_bytes) / stage_bytes;
  const long long per_block = (p.units + blocks - 1) / blocks;
  if (stages > per_block) stages = per_block < 2 ? 2 : (int)per_block;
  if (stages > LIN_MAX_STAGES) stages = LIN_MAX_STAGES;
  p.stages = stages;
  const size_t smem = (size_t)stages * stage_bytes + 1024 + xchg_bytes;
  CUtensorMap map_w, map_x;
  if (!get_map(w, N, K, act != 0 ? -64 : LIN_BM, &map_w) || !get_map(x, M, K, p.m_pad, &map_x)) return ULLM_ERR_LAUNCH;
  if (!g_lin_attr_set) {
    if (cudaFuncSetAttribute(linear_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) !=
        cudaSuccess)
      return ULLM_ERR_LAUNCH;
    g_lin_attr_set = 1;
  }
  int rc = ullm_launch_kernel(linear_tcgen05_kernel, dim3(blocks), dim3(LIN_THREADS), smem, st, map_w, map_x, p);
  if (rc != ULLM_OK) return rc;
  return ullm_launch_status();
}
