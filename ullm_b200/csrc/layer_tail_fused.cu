// The second half of a pre-norm decoder layer as ONE kernel, for decode steps (at most 16 rows, bfloat16):
//
//   r   <- residual + attn . Wo^T                       (32-bit sum, rounded once; phase 0)
//   h    = rmsnorm(r) * w                               (applied to the operand on its way into phase 1)
//   a   <- act(h . Wgate^T) * (h . Wup^T)               (phase 1)
//   r   <- r + a . Wdown^T                              (phase 2)
//
// Each product alone is one pass of its weight matrix through the chip and pays a launch, a start-up in which
// memory idles while the first tiles are on their way, and a tail; three products, the norm between them and
// the activation are five launches.  Here one cooperative grid of two blocks per SM streams all three weight
// matrices back to back through the TMA ring of linear_stream.cu:
//
//   * A block's work is a fixed list of items: for each phase, the units (32 output columns; 16 gate + 16 up
//     rows in phase 1) dealt round robin, each with all of K or, where a phase has too few units for the grid
//     (the two products with `hidden` outputs), one of two halves of K.  The producer thread walks that list and
//     keeps the ring full of WEIGHT tiles across phase boundaries: weights depend on nothing.  The batch rows
//     of a phase are what the phase before wrote, so the producer issues those copies only once the grid barrier
//     between the phases has been passed; a stage is complete when both have landed.
//   * Grid barriers are counters in global memory: a block arrives when all its outputs of the phase are written
//     and fenced; producers poll them between copies (never blocking the weight stream), consumers once per
//     phase.  The grid is launched cooperatively, so all blocks are resident.  Every poll loop is bounded: a
//     block that gives up records ULLM_STATUS_TIMEOUT, stops, and lets the others run into their own limits.
//   * The two halves of a split unit meet through a scratch array: each block writes its 32-bit partial sums,
//     takes a ticket for the unit, and the second one adds the two in half order (the same sum whoever comes
//     second), adds the residual, rounds once and stores.  In phase 0 it also leaves the unit's sum of squares
//     per row, from which every block computes the rows' 1/rms after the barrier.
//   * The norm between phases 0 and 1 needs whole rows, but only for one number per row: rmsnorm(r) * w =
//     (1 / rms(r)) * (r * w).  So phase 0's epilogue writes r * w (32-bit product of the unrounded sum, rounded
//     once) as the operand of phase 1, together with the unit's sums of squares, and phase 1 multiplies its
//     32-bit sums by the row's 1 / rms before the activation: one grid barrier between the two, no pass over r.
//     (The separate norm kernel rounds r * w / rms; here r * w is rounded and 1 / rms applied in 32-bit after
//     the product.)
#include <cooperative_groups.h>

#include "linear_stream_core.cuh"

#define LT_POLL_LIMIT (1 << 22)

struct LtPhase {
  int n_units;   // units of 32 output columns
  int k_blocks;  // 256-wide k blocks of all of K
  int ksplit;    // 1 or 2 items per unit
  int kper;      // k blocks per item
  int items;     // n_units * ksplit
  int n_out;     // output columns
};

struct LtMaps {
  CUtensorMap w[3];  // Wo (boxes of 32 rows), Wgate|Wup (boxes of 16 rows), Wdown (boxes of 32 rows)
  CUtensorMap x[3];  // attn, normed, act_out
};

struct LtParams {
  LtPhase ph[3];
  __nv_bfloat16* residual;  // [M, H], updated in place
  __nv_bfloat16* act_out;   // [M, I]
  __nv_bfloat16* normed;    // [M, H]: (residual after phase 0) * norm_w, the operand of phase 1
  const float* norm_w;      // [H]
  float eps;
  int act;                  // 1 silu, 2 gelu_tanh
  int M, H, I;
  int stages;
  float* pair;              // partial sums of split units: [2 halves][units][2][32 lanes][NT][4]
  float* sq;                // phase 0's sums of squares: [units][2][16]
  unsigned* tickets;        // [units] per split phase (phase 0, then phase 2)
  unsigned* bars;           // grid barriers after phases 0 and 1; [2]: blocks that have finished
  int* status;
};

__device__ __forceinline__ unsigned lt_ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 lt_ld_cg_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float lt_ld_cg_f(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ bool lt_mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(lin_smem(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// a position in a block's list of stages: phase, item of the phase, k block of the item
struct LtCursor {
  int ph, j, kb, it;       // phase, item of the phase, k block of the item, stage count
  int slot, round;         // ring slot and how often the ring has been gone round
  int unit, half, kper, kbase;  // of the current item
};

template <int NT>
__global__ void __launch_bounds__(LS_THREADS, 2) layer_tail_fused_kernel(const __grid_constant__ LtMaps maps,
                                                                         const LtParams p) {
  constexpr int XR = 8 * NT;
  constexpr int X_BYTES = 4 * XR * 128;
  constexpr int STAGE_BYTES = LS_W_STAGE_BYTES + X_BYTES;
  constexpr int NP = NT;  // (at most two batch tiles: they meet in one pass)
  extern __shared__ unsigned char lt_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[LS_MAX_STAGES], empty_bar[LS_MAX_STAGES];
  __shared__ float rstd_s[16];
  __shared__ float part_s[16][17];
  __shared__ int abort_flag;
  __shared__ unsigned ticket_s;
  unsigned char* ring = (unsigned char*)(((uintptr_t)lt_smem_raw + 1023) & ~(uintptr_t)1023);
  float* red = reinterpret_cast<float*>(ring + p.stages * STAGE_BYTES);  // [8 warps][32 lanes][NP][4]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = (int)blockIdx.x, G = (int)gridDim.x;
  int n_my[3], total_it = 0;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    n_my[i] = p.ph[i].items > c ? (p.ph[i].items - 1 - c) / G + 1 : 0;
    total_it += n_my[i] * p.ph[i].kper;
  }
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], LS_CONSUMER_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  if (warp == LS_CONSUMER_WARPS) {
    // ---- producer ---------------------------------------------------------------------------------------
    if (lane == 0) {
      // One thread's instruction stream paces the ring, so a position in the block's list of stages is carried
      // along and stepped: nothing is divided per stage (unit and half of an item are worked out once per item).
      auto enter_item = [&](LtCursor& q) {
        while (q.ph < 3 && q.j >= n_my[q.ph]) {
          ++q.ph;
          q.j = 0;
        }
        if (q.ph < 3) {
          const LtPhase& ph = p.ph[q.ph];
          const int item = c + q.j * G;
          q.half = item / ph.n_units;
          q.unit = item - q.half * ph.n_units;
          q.kper = ph.kper;
          q.kbase = q.half * ph.kper;
        }
      };
      auto advance = [&](LtCursor& q) {
        ++q.it;
        if (++q.slot == p.stages) q.slot = 0, ++q.round;
        if (++q.kb == q.kper) {
          q.kb = 0;
          ++q.j;
          enter_item(q);
        }
      };
      LtCursor w = {};
      enter_item(w);
      LtCursor x = w;
      int seen = 0;  // phases whose operand is known to be ready: phase ph > 0 needs grid barrier ph - 1
      int idle = 0;
      while (x.it < total_it) {
        bool progressed = false;
        if (w.it < total_it && (w.round == 0 || lt_mbar_test(&empty_bar[w.slot], (w.round - 1) & 1))) {
          unsigned char* st = ring + w.slot * STAGE_BYTES;
          const int kb = w.kbase + w.kb;
          mbar_expect_tx(&full_bar[w.slot], STAGE_BYTES);
          if (w.ph == 1) {
            tma_load_3d(st, &maps.w[1], &full_bar[w.slot], 0, w.unit * 16, kb * 4);
            tma_load_3d(st + 8192, &maps.w[1], &full_bar[w.slot], 0, p.I + w.unit * 16, kb * 4);
          } else {
            tma_load_3d(st, &maps.w[w.ph], &full_bar[w.slot], 0, w.unit * 32, kb * 4);
          }
          advance(w);
          progressed = true;
        }
        if (x.it < w.it) {
          if (x.ph <= seen) {
            if (x.it == 0) pdl_wait();
            tma_load_3d(ring + x.slot * STAGE_BYTES + LS_W_STAGE_BYTES, &maps.x[x.ph], &full_bar[x.slot], 0, 0,
                        (x.kbase + x.kb) * 4);
            advance(x);
            progressed = true;
          } else if (lt_ld_acquire(&p.bars[seen]) >= (unsigned)G) {
            ++seen;
            asm volatile("fence.proxy.async;" ::: "memory");  // what the others wrote, before the copies that read it
            progressed = true;
          }
        }
        if (progressed) {
          idle = 0;
        } else if (++idle > LT_POLL_LIMIT) {
          ullm_report(p.status, ULLM_STATUS_TIMEOUT, 61, x.it);
          abort_flag = 1;
          break;
        }
      }
    }
  } else {
    // ---- consumers ----------------------------------------------------------------------------------------
    const int mt = warp & 1, kq = warp >> 1;
    const int g = lane >> 2, t = lane & 3;
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int a_chunk = lane >> 4;
    const int b_row = (lane & 7) + (lane >> 4) * 8;
    const int b_chunk = (lane >> 3) & 1;
    bool failed = false;
    int it = 0, s = 0;  // stage count; the ring slot of the next stage and the parity of its use, stepped
    uint32_t parity = 0;
    for (int phi = 0; phi < 3; ++phi) {
      const LtPhase& ph = p.ph[phi];
      if (phi == 1) {
        // ---- the rows' 1 / rms for phase 1's epilogue.  All of phase 0 is done everywhere: ------------------------
        if (threadIdx.x == 0 && !failed) {
          int polls = 0;
          while (lt_ld_acquire(&p.bars[0]) < (unsigned)G) {
            if (++polls > LT_POLL_LIMIT) {
              ullm_report(p.status, ULLM_STATUS_TIMEOUT, 62, 0);
              abort_flag = 1;
              break;
            }
          }
        }
        ls_bar_sync_consumers();
        {
          // the rows' 1/rms: 16 parts of the units' partial sums per row, all loads of a thread in flight together
          const int m = threadIdx.x & 15, part = threadIdx.x >> 4;
          const int total = p.ph[0].n_units * 2;
          const int per = (total + 15) / 16;
          float sum = 0.f;
          for (int q0 = part * per; q0 < (part + 1) * per && q0 < total; q0 += 8) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              v[e] = (q0 + e < (part + 1) * per && q0 + e < total) ? __ldcg(p.sq + (size_t)(q0 + e) * 16 + m) : 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) sum += v[e];
          }
          part_s[part][m] = sum;
        }
        ls_bar_sync_consumers();
        if (threadIdx.x < 16) {
          float sum = 0.f;
          for (int q = 0; q < 16; ++q) sum += part_s[q][threadIdx.x];  // in part order: the same sum in every block
          rstd_s[threadIdx.x] = rsqrtf(sum / (float)p.H + p.eps);
        }
        ls_bar_sync_consumers();
      }
      for (int j = 0; j < n_my[phi]; ++j) {
        const int item = c + j * G, unit = item % ph.n_units, half = item / ph.n_units;
        float acc[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
        for (int kb = 0; kb < ph.kper; ++kb, ++it) {
          if (!failed && !__all_sync(0xffffffffu, mbar_wait(&full_bar[s], parity))) {
            ullm_report(p.status, ULLM_STATUS_TIMEOUT, 63, it);  // (the whole warp gives up together)
            abort_flag = 1;
            failed = true;
          }
          if (!failed) {
            const uint32_t wbox =
                lin_smem(ring + s * STAGE_BYTES + (phi == 1 ? (mt * 4 + kq) * 2048 : kq * 4096 + mt * 2048));
            const uint32_t xbox = lin_smem(ring + s * STAGE_BYTES + LS_W_STAGE_BYTES + kq * (XR * 128));
            uint32_t a[4][4], b[4][NT * 2];
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              ls_ldmatrix4(a[jj], wbox + a_row * 128 + (((jj * 2 + a_chunk) ^ (a_row & 7)) << 4));
              if (NT == 1) {
                const int r = lane & 7, cc = (lane >> 3) & 1;
                ls_ldmatrix2(b[jj][0], b[jj][1], xbox + r * 128 + (((jj * 2 + cc) ^ r) << 4));
              } else {
                uint32_t t4[4];
                ls_ldmatrix4(t4, xbox + b_row * 128 + (((jj * 2 + b_chunk) ^ (b_row & 7)) << 4));
                b[jj][0] = t4[0], b[jj][1] = t4[1], b[jj][2] = t4[2], b[jj][3] = t4[3];
              }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj)
#pragma unroll
              for (int n = 0; n < NT; ++n) ls_mma(acc[n], a[jj], b[jj][n * 2], b[jj][n * 2 + 1]);
          } else {
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
          }
          if (++s == p.stages) s = 0, parity ^= 1;
        }
        // ---- the four k quarters of each half meet; warps 0 and 1 (quarter 0) finish the item ---------------
#pragma unroll
        for (int n = 0; n < NP; ++n)
          *reinterpret_cast<float4*>(red + ((size_t)(warp * 32 + lane) * NP + n) * 4) =
              make_float4(acc[n][0], acc[n][1], acc[n][2], acc[n][3]);
        ls_bar_sync_consumers();
        if (kq == 0) {
          float v[NT][4], up[NT][4];
#pragma unroll
          for (int n = 0; n < NT; ++n) {
#pragma unroll
            for (int i = 0; i < 4; ++i) v[n][i] = 0.f, up[n][i] = 0.f;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 pv = *reinterpret_cast<const float4*>(red + ((size_t)((q * 2 + mt) * 32 + lane) * NP + n) * 4);
              v[n][0] += pv.x, v[n][1] += pv.y, v[n][2] += pv.z, v[n][3] += pv.w;
              if (phi == 1) {
                const float4 pu = *reinterpret_cast<const float4*>(red + ((size_t)((q * 2 + (mt ^ 1)) * 32 + lane) * NP + n) * 4);
                up[n][0] += pu.x, up[n][1] += pu.y, up[n][2] += pu.z, up[n][3] += pu.w;
              }
            }
          }
          if (phi == 1) {
            // ---- act(gate) * up: warp 0 holds the gate sums in v and the up sums in `up` ---------------------
            if (mt == 0 && !failed) {
#pragma unroll
              for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const int col = unit * 16 + g + 8 * (i >> 1), m = n * 8 + 2 * t + (i & 1);
                  if (m < p.M && col < ph.n_out) {
                    const float rs = rstd_s[m], gate = v[n][i] * rs, upv = up[n][i] * rs;
                    p.act_out[(size_t)m * ph.n_out + col] =
                        __float2bfloat16_rn((p.act == 1 ? act_silu(gate) : act_gelu_tanh(gate)) * upv);
                  }
                }
            }
          } else {
            // ---- a product onto the residual; the halves of a split unit meet first ---------------------------
            bool mine = true;  // this block finishes the unit
            if (ph.ksplit == 2) {
              float* slot = p.pair + ((((size_t)half * ph.n_units + unit) * 2 + mt) * 32 + lane) * NT * 4;
#pragma unroll
              for (int n = 0; n < NT; ++n)
                *reinterpret_cast<float4*>(slot + n * 4) = make_float4(v[n][0], v[n][1], v[n][2], v[n][3]);
              __threadfence();
              asm volatile("bar.sync 2, 64;" ::: "memory");
              if (warp == 0 && lane == 0) ticket_s = atomicAdd(p.tickets + (phi == 0 ? 0 : p.ph[0].n_units) + unit, 1u);
              asm volatile("bar.sync 2, 64;" ::: "memory");
              mine = (ticket_s & 1u) != 0;  // the second of the two (tickets only ever grow: their parity tells)
              if (mine) {
                __threadfence();
                const float* other =
                    p.pair + ((((size_t)(half ^ 1) * ph.n_units + unit) * 2 + mt) * 32 + lane) * NT * 4;
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                  const float4 o = lt_ld_cg_f4(other + n * 4);
                  // half 0 + half 1, whoever came second
                  if (half == 1) {
                    v[n][0] = o.x + v[n][0], v[n][1] = o.y + v[n][1], v[n][2] = o.z + v[n][2], v[n][3] = o.w + v[n][3];
                  } else {
                    v[n][0] += o.x, v[n][1] += o.y, v[n][2] += o.z, v[n][3] += o.w;
                  }
                }
              }
            }
            if (mine && !failed) {
              float ss[NT][2];
#pragma unroll
              for (int n = 0; n < NT; ++n) {
                ss[n][0] = ss[n][1] = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const int col = unit * 32 + mt * 16 + g + 8 * (i >> 1), m = n * 8 + 2 * t + (i & 1);
                  if (m < p.M && col < ph.n_out) {
                    const size_t o = (size_t)m * ph.n_out + col;
                    // (read past L1: another block may have written this element in the phase before)
                    const float r = v[n][i] + __bfloat162float(__ushort_as_bfloat16(
                                                  __ldcg(reinterpret_cast<const unsigned short*>(p.residual) + o)));
                    p.residual[o] = __float2bfloat16_rn(r);
                    if (phi == 0) p.normed[o] = __float2bfloat16_rn(r * __ldg(p.norm_w + col));
                    ss[n][i & 1] += r * r;
                  }
                }
              }
              if (phi == 0) {
                // the unit's sums of squares per batch row: over the 8 lanes that share t, then one store each
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                  for (int e = 0; e < 2; ++e) {
                    float s = ss[n][e];
                    s += __shfl_xor_sync(0xffffffffu, s, 4);
                    s += __shfl_xor_sync(0xffffffffu, s, 8);
                    s += __shfl_xor_sync(0xffffffffu, s, 16);
                    if (g == 0) p.sq[((size_t)unit * 2 + mt) * 16 + n * 8 + 2 * t + e] = s;
                  }
                if (NT == 1 && g == 0) {  // rows 8 to 15 do not exist: their sums are zero
                  p.sq[((size_t)unit * 2 + mt) * 16 + 8 + 2 * t] = 0.f;
                  p.sq[((size_t)unit * 2 + mt) * 16 + 8 + 2 * t + 1] = 0.f;
                }
              }
            }
          }
        }
        ls_bar_sync_consumers();  // the partial sums are read: the next item may overwrite them
      }
      // ---- the end of the phase: this block's outputs are written; tell the grid ------------------------------
      __threadfence();
      ls_bar_sync_consumers();
      if (threadIdx.x == 0) {
        asm volatile("fence.proxy.async;" ::: "memory");  // the next phase reads them by TMA
        if (phi < 2) {
          atomicAdd(p.bars + phi, 1u);
        } else if (atomicAdd(p.bars + 2, 1u) == (unsigned)G - 1) {
          // the last block of the launch: nobody looks at the counters any more; the next launch finds zeros
          p.bars[0] = 0;
          p.bars[1] = 0;
          p.bars[2] = 0;
        }
      }
    }
  }
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) {
    // a wait ran out: copies may still be on their way into the ring; wait (bounded) for the last phase of every
    // stage before the block gives its shared memory back
    for (int s = 0; s < p.stages; ++s) {
      int last = -1;
      for (int it = s; it < total_it; it += p.stages) last = it;
      if (last >= 0) mbar_wait(&full_bar[s], (last / p.stages) & 1);
    }
  }
}

static int g_lt_sms = 0;
static int g_lt_attr[2] = {0, 0};
static int g_lt_grid[2] = {0, 0};
static int g_lt_last_grid = 0;
static int g_lt_phase_mask = 7;  // measurements only: phases that run (bit i: phase i); the result is wrong otherwise
extern "C" void ullm_layer_tail_fused_phase_mask(int m) { g_lt_phase_mask = m & 7; }
// The grid of the last launch (tests and measurements read it).
extern "C" int ullm_layer_tail_fused_last_grid(void) { return g_lt_last_grid; }

// Sizes the kernel takes: at most 16 rows; every K a multiple of 256 (whole stages, whole halves); hidden and
// intermediate sizes multiples of 32 and 16.
extern "C" int ullm_layer_tail_fused_supported(int M, int H, int QD, int I) {
  return M >= 1 && M <= 16 && H > 0 && QD > 0 && I > 0 && H % 256 == 0 && QD % 256 == 0 && I % 256 == 0;
}

// Floats of scratch for the halves of split units, and unsigned counters (tickets of both split phases + 4).
extern "C" long long ullm_layer_tail_fused_scratch_floats(int H) {
  const long long units = (H + 31) / 32;
  return 2 * units * 2 * 32 * 2 * 4 + units * 2 * 16;  // pair (two batch tiles at most) + sums of squares
}
extern "C" long long ullm_layer_tail_fused_counters(int H) { return 2LL * ((H + 31) / 32) + 4; }

template <int NT>
static int lt_launch(int which, const LtMaps& maps, LtParams p, cudaStream_t st) {
  constexpr int STAGE_BYTES = LS_W_STAGE_BYTES + 4 * 8 * NT * 128;
  const int red_bytes = LS_CONSUMER_WARPS * 32 * NT * 4 * (int)sizeof(float);
  int stages = (108 * 1024 - 1024 - red_bytes) / STAGE_BYTES;
  if (stages > LS_MAX_STAGES) stages = LS_MAX_STAGES;
  if (stages < 2) return ULLM_ERR_UNSUPPORTED;
  p.stages = stages;
  const size_t smem = (size_t)stages * STAGE_BYTES + red_bytes + 1024;
  if (!g_lt_attr[which]) {
    if (cudaFuncSetAttribute(layer_tail_fused_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024) !=
        cudaSuccess)
      return ULLM_ERR_LAUNCH;
    cudaFuncSetAttribute(layer_tail_fused_kernel<NT>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, layer_tail_fused_kernel<NT>, LS_THREADS, smem) !=
            cudaSuccess ||
        per_sm < 1)
      return ULLM_ERR_LAUNCH;
    g_lt_grid[which] = g_lt_sms * (per_sm > 2 ? 2 : per_sm);  // every block resident: they wait for one another
    g_lt_attr[which] = 1;
  }
  const int grid = g_lt_grid[which];
  g_lt_last_grid = grid;
  // a phase with few units is split in two halves of K when that still fits the grid
  for (int i = 0; i < 3; ++i) {
    LtPhase& ph = p.ph[i];
    ph.ksplit = (i != 1 && ph.n_units * 2 <= grid && ph.k_blocks % 2 == 0 && ph.k_blocks >= 4) ? 2 : 1;
    ph.kper = ph.k_blocks / ph.ksplit;
    ph.items = (g_lt_phase_mask >> i) & 1 ? ph.n_units * ph.ksplit : 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(LS_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, layer_tail_fused_kernel<NT>, maps, p) != cudaSuccess) {
    cudaGetLastError();
    return ULLM_ERR_LAUNCH;
  }
  return ULLM_OK;
}

// attn [M, QD], residual [M, H] (in/out), act_out [M, I] and normed [M, H] (work buffers), w_o [H, QD], w_gate_up [2 I, H],
// w_down [H, I], norm_w [H] float32.  scratch / counters: at least what the two functions above say, the
// counters zero before the first launch (and after a launch that reported a timeout).
extern "C" int ullm_layer_tail_fused(const void* attn, void* residual, void* act_out, void* normed, const void* w_o,
                                     const void* w_gate_up, const void* w_down, const float* norm_w, float eps,
                                     int act, int M, int H, int QD, int I, float* scratch, unsigned* counters,
                                     int* status, void* stream) {
  if (!ullm_layer_tail_fused_supported(M, H, QD, I)) return ULLM_ERR_UNSUPPORTED;
  if (act != 1 && act != 2) return ULLM_ERR_BAD_SIZE;
  if (scratch == nullptr || counters == nullptr || norm_w == nullptr || normed == nullptr) return ULLM_ERR_BAD_SIZE;
  if (g_lt_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&g_lt_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || g_lt_sms <= 0)
      return ULLM_ERR_LAUNCH;
  }
  const int NT = M <= 8 ? 1 : 2;
  LtMaps maps;
  if (!ls_chunked_map(w_o, H, QD, 32, &maps.w[0]) || !ls_chunked_map(w_gate_up, 2LL * I, H, 16, &maps.w[1]) ||
      !ls_chunked_map(w_down, H, I, 32, &maps.w[2]) || !ls_chunked_map(attn, M, QD, 8 * NT, &maps.x[0]) ||
      !ls_chunked_map(normed, M, H, 8 * NT, &maps.x[1]) || !ls_chunked_map(act_out, M, I, 8 * NT, &maps.x[2]))
    return ULLM_ERR_LAUNCH;
  LtParams p = {};
  const int units_h = (H + 31) / 32;
  p.ph[0].n_units = units_h, p.ph[0].k_blocks = QD / LS_BK, p.ph[0].n_out = H;
  p.ph[1].n_units = (I + 15) / 16, p.ph[1].k_blocks = H / LS_BK, p.ph[1].n_out = I;
  p.ph[2].n_units = units_h, p.ph[2].k_blocks = I / LS_BK, p.ph[2].n_out = H;
  p.residual = (__nv_bfloat16*)residual;
  p.act_out = (__nv_bfloat16*)act_out;
  p.normed = (__nv_bfloat16*)normed;
  p.norm_w = norm_w;
  p.eps = eps;
  p.act = act;
  p.M = M, p.H = H, p.I = I;
  p.pair = scratch;
  p.sq = scratch + 2LL * units_h * 2 * 32 * 2 * 4;
  p.tickets = counters;
  p.bars = counters + 2LL * units_h;
  p.status = status;
  if (NT == 1) return lt_launch<1>(0, maps, p, (cudaStream_t)stream);
  return lt_launch<2>(1, maps, p, (cudaStream_t)stream);
}
