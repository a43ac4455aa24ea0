// out[M, N] = x[M, K] . W[N, K]^T for many rows (prompt portions), bfloat16 in, 32-bit accumulate,
// bfloat16 or float32 out; optionally out[M, N/2] = act(gate) * up for a weight that stacks gate rows on up
// rows (the gated feed-forward's first product with its activation in the epilogue: gate and up never reach
// memory).
//
// A persistent kernel, one block per SM, on the 5th-generation tensor cores:
//
//   * An output tile is 128 rows of x by 256 rows of W (with an activation: 128 gate rows and the same 128 rows
//     of up).  tcgen05.mma with M = 128, N = 256, K = 16 runs at the tensor core's full rate; the accumulator
//     [128 lanes x 256 columns] lives in tensor memory, and there are two of them, so that the epilogue of one
//     tile overlaps the products of the next.
//   * Tiles are taken in the order (row tile fastest, then column tile): the blocks that run at the same time
//     share a few panels of W, which stay in L2, and x (a few MB) stays there anyway.
//   * Warp 0 (one thread) issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of 128 x 64 tiles of x and
//     256 x 64 tiles of W into a ring of four stages; warp 1 (one thread) issues the MMAs; warps 2..5 read a
//     finished accumulator (tcgen05.ld: a thread owns one output row), add bias, apply the activation, round
//     and store 32 bytes at a time.  mbarriers carry "stage full", "stage free", "accumulator full",
//     "accumulator drained".
//   * Every load is issued by the block that uses it (no multicast, one CTA per tile).
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT polls the kernel records ULLM_STATUS_TIMEOUT in the
// status word, stops waiting, still frees its tensor memory and returns.
#include "tcgen05_util.cuh"

#define LG_BM 128   // rows of x per tile (UMMA M)
#define LG_BN 256   // rows of W per tile (UMMA N)
#define LG_BK 64    // k per stage: one 128-byte swizzle row
#define LG_STAGES 4
#define LG_THREADS 192
#define LG_A_BYTES (LG_BM * 128)
#define LG_B_BYTES (LG_BN * 128)
#define LG_STAGE_BYTES (LG_A_BYTES + LG_B_BYTES)

struct LgParams {
  int M, N, K;
  int m_tiles, n_tiles, k_blocks;
  int out_f32;   // 1: float32 output, 0: bfloat16
  int act;       // 0: plain product; 1: silu(gate) * up; 2: gelu_tanh(gate) * up
  int n_out;     // columns of out: N, or N / 2 with an activation
  void* out;     // [M, n_out]
  const void* bias;  // [N] bf16 or null
  int* status;
};

__device__ __forceinline__ void lg_epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// 16 accumulator values of one row -> out[row, col0 .. col0 + 15], masked at the right edge
__device__ __forceinline__ void lg_store16(const LgParams& p, int row, int col0, const float (&v)[16]) {
  if (row >= p.M || col0 >= p.n_out) return;
  if (p.out_f32) {
    float* o = reinterpret_cast<float*>(p.out) + (long long)row * p.n_out + col0;
    if (col0 + 16 <= p.n_out && p.n_out % 4 == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(o)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (col0 + i < p.n_out) o[i] = v[i];
    }
  } else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)row * p.n_out + col0;
    if (col0 + 16 <= p.n_out && p.n_out % 8 == 0) {
      uint4 a, b;
      __nv_bfloat162* ha = reinterpret_cast<__nv_bfloat162*>(&a);
      __nv_bfloat162* hb = reinterpret_cast<__nv_bfloat162*>(&b);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        ha[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        hb[i] = __floats2bfloat162_rn(v[8 + 2 * i], v[8 + 2 * i + 1]);
      }
      reinterpret_cast<uint4*>(o)[0] = a;
      reinterpret_cast<uint4*>(o)[1] = b;
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (col0 + i < p.n_out) o[i] = __float2bfloat16_rn(v[i]);
    }
  }
}

__global__ void __launch_bounds__(LG_THREADS, 1)
linear_tcgen05_large_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                            const LgParams p) {
  extern __shared__ unsigned char lg_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[LG_STAGES], empty_bar[LG_STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int wait_flag[2];
  pdl_launch_dependents();
  unsigned char* tiles = (unsigned char*)(((uintptr_t)lg_smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long num_tiles = (long long)p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < LG_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_full[0], 1);
    mbar_init(&acc_full[1], 1);
    mbar_init(&acc_empty[0], 4);
    mbar_init(&acc_empty[1], 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(lin_smem(&tmem_base_slot)),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_base_slot;
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: TMA loads -------------------------------------------------------------
      int s = 0;
      uint32_t parity = 1;  // a fresh barrier passes a wait on parity 1
      for (long long tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int mt = (int)(tile % p.m_tiles), nt = (int)(tile / p.m_tiles);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[s], parity)) {
            ullm_report(p.status, ULLM_STATUS_TIMEOUT, 31, kb);
            tile = num_tiles;
            break;
          }
          unsigned char* a = tiles + s * LG_STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], LG_STAGE_BYTES);
          tma_load_2d(a, &map_x, &full_bar[s], kb * LG_BK, mt * LG_BM);
          if (p.act == 0) tma_load_2d(a + LG_A_BYTES, &map_w, &full_bar[s], kb * LG_BK, nt * LG_BN);
          else tma_load_3d(a + LG_A_BYTES, &map_w, &full_bar[s], kb * LG_BK, nt * (LG_BN / 2), 0);
          if (++s == LG_STAGES) s = 0, parity ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----------------------------------------------------------------------
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(LG_BN >> 3) << 17) |
                             ((uint32_t)(LG_BM >> 4) << 24);
      const uint64_t desc0 = umma_desc(tiles);
      const uint32_t desc_hi = (uint32_t)(desc0 >> 32), lo0 = (uint32_t)desc0;
      const uint32_t full0 = lin_smem(&full_bar[0]), empty0 = lin_smem(&empty_bar[0]);
      uint32_t a_lo = lo0, full_s = full0, empty_s = empty0;
      int s = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int buf = it & 1;
        if (!mbar_wait(&acc_empty[buf], ((it >> 1) & 1) ^ 1)) {  // the epilogue has drained this accumulator
          ullm_report(p.status, ULLM_STATUS_TIMEOUT, 34, it);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d = tmem_d + (uint32_t)(buf * LG_BN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait_addr(full_s, phase)) {
            ullm_report(p.status, ULLM_STATUS_TIMEOUT, 32, kb);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t b_lo = a_lo + (LG_A_BYTES >> 4);
          // 16 bf16 = 32 bytes further along the swizzled row: +2 in the 16-byte address field
          umma_bf16_lo<-1>(d, a_lo, b_lo, desc_hi, idesc, kb > 0 ? 1u : 0u);
          umma_bf16_lo<1>(d, a_lo + 2, b_lo + 2, desc_hi, idesc);
          umma_bf16_lo<1>(d, a_lo + 4, b_lo + 4, desc_hi, idesc);
          umma_bf16_lo<1>(d, a_lo + 6, b_lo + 6, desc_hi, idesc);
          umma_commit_addr(empty_s);  // the stage is free once these MMAs have read it
          a_lo += (LG_STAGE_BYTES >> 4), full_s += 8, empty_s += 8;
          if (++s == LG_STAGES) s = 0, phase ^= 1, a_lo = lo0, full_s = full0, empty_s = empty0;
        }
        if (ok) umma_commit(&acc_full[buf]);  // the accumulator is complete once every MMA above is
      }
    }
  } else {
    // ---- epilogue: warps 2..5; a warp reads the accumulator lanes 32 (warp % 4) .. + 31 ----------
    const int quarter = warp & 3;
    const int et = threadIdx.x - 64;  // 0..127 among the epilogue threads
    const __nv_bfloat16* bias = (const __nv_bfloat16*)p.bias;
    int it = 0;
    for (long long tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int mt = (int)(tile % p.m_tiles), nt = (int)(tile / p.m_tiles);
      const int buf = it & 1;
      // One thread waits (bounded) and tells the others, so that all 128 take the same way out.
      if (et == 0) {
        const bool got = mbar_wait(&acc_full[buf], (it >> 1) & 1);
        if (!got) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 33, it);
        wait_flag[it & 1] = got ? 1 : 0;
      }
      lg_epi_bar_sync();
      if (wait_flag[it & 1] == 0) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = mt * LG_BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_d + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * LG_BN);
      if (p.act == 0) {
#pragma unroll 2
        for (int c = 0; c < LG_BN / 16; ++c) {
          float v[16];
          tmem_ld16(taddr + c * 16, v);
          const int col0 = nt * LG_BN + c * 16;
          if (bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (col0 + i < p.N) v[i] += __bfloat162float(bias[col0 + i]);
          }
          lg_store16(p, row, col0, v);
        }
      } else {
        // columns 0..127 of the accumulator are gate features, columns 128..255 the same features of up
#pragma unroll 2
        for (int c = 0; c < LG_BN / 32; ++c) {
          float g[16], u[16];
          tmem_ld16(taddr + c * 16, g);
          tmem_ld16(taddr + LG_BN / 2 + c * 16, u);
          const int col0 = nt * (LG_BN / 2) + c * 16;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float gv = g[i], uv = u[i];
            if (bias != nullptr && col0 + i < p.n_out) {
              gv += __bfloat162float(bias[col0 + i]);
              uv += __bfloat162float(bias[p.n_out + col0 + i]);
            }
            g[i] = (p.act == 1 ? act_silu(gv) : act_gelu_tanh(gv)) * uv;
          }
          lg_store16(p, row, col0, g);
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);  // the MMA warp may fill this accumulator again
    }
  }
  __syncwarp();  // the lanes of the two single-thread roles wait here for their lane 0
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(512) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// The same product with tiles of 256 rows of x: two 128-row halves share every tile of W in shared memory, so a
// block loads 64 KB for 1,024 tensor-core clocks instead of 48 KB for 512 (two thirds of the traffic from L2,
// which is what bounds the kernel above).  The two halves' accumulators fill all 512 columns of tensor memory:
// there is no spare one, so the epilogue drains half 0, then half 1, while the next tile's products start on
// half 0 as soon as it is drained.  Ring of three 64 KB stages.
// ---------------------------------------------------------------------------------------------
#define LG2_BM 256
#define LG2_STAGES 3
#define LG2_A_BYTES (LG2_BM * 128)
#define LG2_STAGE_BYTES (LG2_A_BYTES + LG_B_BYTES)

__global__ void __launch_bounds__(LG_THREADS, 1)
linear_tcgen05_large2_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                             const LgParams p) {
  extern __shared__ unsigned char lg_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[LG2_STAGES], empty_bar[LG2_STAGES], acc_full, acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int wait_flag[2];
  pdl_launch_dependents();
  unsigned char* tiles = (unsigned char*)(((uintptr_t)lg_smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long num_tiles = (long long)p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < LG2_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_full, 1);
    mbar_init(&acc_empty[0], 4);
    mbar_init(&acc_empty[1], 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(lin_smem(&tmem_base_slot)),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = tmem_base_slot;
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: TMA loads (256 rows of x in one box, 256 rows of W in one box) ------------------
      int s = 0;
      uint32_t parity = 1;  // a fresh barrier passes a wait on parity 1
      for (long long tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int mt = (int)(tile % p.m_tiles), nt = (int)(tile / p.m_tiles);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[s], parity)) {
            ullm_report(p.status, ULLM_STATUS_TIMEOUT, 41, kb);
            tile = num_tiles;
            break;
          }
          unsigned char* a = tiles + s * LG2_STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], LG2_STAGE_BYTES);
          tma_load_2d(a, &map_x, &full_bar[s], kb * LG_BK, mt * LG2_BM);
          if (p.act == 0) tma_load_2d(a + LG2_A_BYTES, &map_w, &full_bar[s], kb * LG_BK, nt * LG_BN);
          else tma_load_3d(a + LG2_A_BYTES, &map_w, &full_bar[s], kb * LG_BK, nt * (LG_BN / 2), 0);
          if (++s == LG2_STAGES) s = 0, parity ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----------------------------------------------------------------------
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(LG_BN >> 3) << 17) |
                             ((uint32_t)(LG_BM >> 4) << 24);
      const uint64_t desc0 = umma_desc(tiles);
      const uint32_t desc_hi = (uint32_t)(desc0 >> 32), lo0 = (uint32_t)desc0;
      const uint32_t full0 = lin_smem(&full_bar[0]), empty0 = lin_smem(&empty_bar[0]);
      uint32_t a_lo = lo0, full_s = full0, empty_s = empty0;
      int s = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const uint32_t drained = (uint32_t)(it & 1) ^ 1;  // parity of "the epilogue of the tile before has drained"
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait_addr(full_s, phase)) {
            ullm_report(p.status, ULLM_STATUS_TIMEOUT, 42, kb);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a1_lo = a_lo + (LG_A_BYTES >> 4), b_lo = a_lo + (LG2_A_BYTES >> 4);
          if (kb == 0) {
            if (!mbar_wait(&acc_empty[0], drained)) {
              ullm_report(p.status, ULLM_STATUS_TIMEOUT, 44, it);
              ok = false;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          }
          // half 0: 16 bf16 = 32 bytes further along the swizzled row is +2 in the 16-byte address field
          umma_bf16_lo<-1>(tmem_d, a_lo, b_lo, desc_hi, idesc, kb > 0 ? 1u : 0u);
          umma_bf16_lo<1>(tmem_d, a_lo + 2, b_lo + 2, desc_hi, idesc);
          umma_bf16_lo<1>(tmem_d, a_lo + 4, b_lo + 4, desc_hi, idesc);
          umma_bf16_lo<1>(tmem_d, a_lo + 6, b_lo + 6, desc_hi, idesc);
          if (kb == 0) {
            if (!mbar_wait(&acc_empty[1], drained)) {
              ullm_report(p.status, ULLM_STATUS_TIMEOUT, 45, it);
              ok = false;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          }
          umma_bf16_lo<-1>(tmem_d + LG_BN, a1_lo, b_lo, desc_hi, idesc, kb > 0 ? 1u : 0u);
          umma_bf16_lo<1>(tmem_d + LG_BN, a1_lo + 2, b_lo + 2, desc_hi, idesc);
          umma_bf16_lo<1>(tmem_d + LG_BN, a1_lo + 4, b_lo + 4, desc_hi, idesc);
          umma_bf16_lo<1>(tmem_d + LG_BN, a1_lo + 6, b_lo + 6, desc_hi, idesc);
          umma_commit_addr(empty_s);  // the stage is free once these MMAs have read it
          a_lo += (LG2_STAGE_BYTES >> 4), full_s += 8, empty_s += 8;
          if (++s == LG2_STAGES) s = 0, phase ^= 1, a_lo = lo0, full_s = full0, empty_s = empty0;
        }
        if (ok) umma_commit(&acc_full);  // both accumulators are complete once every MMA above is
      }
    }
  } else {
    // ---- epilogue: warps 2..5; a warp reads the accumulator lanes 32 (warp % 4) .. + 31, half 0 then half 1 ----
    const int quarter = warp & 3;
    const int et = threadIdx.x - 64;  // 0..127 among the epilogue threads
    const __nv_bfloat16* bias = (const __nv_bfloat16*)p.bias;
    int it = 0;
    for (long long tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int mt = (int)(tile % p.m_tiles), nt = (int)(tile / p.m_tiles);
      // One thread waits (bounded) and tells the others, so that all 128 take the same way out.
      if (et == 0) {
        const bool got = mbar_wait(&acc_full, it & 1);
        if (!got) ullm_report(p.status, ULLM_STATUS_TIMEOUT, 43, it);
        wait_flag[it & 1] = got ? 1 : 0;
      }
      lg_epi_bar_sync();
      if (wait_flag[it & 1] == 0) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      for (int half = 0; half < 2; ++half) {
        const int row = mt * LG2_BM + half * LG_BM + quarter * 32 + lane;
        const uint32_t taddr = tmem_d + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * LG_BN);
        if (p.act == 0) {
#pragma unroll 2
          for (int c = 0; c < LG_BN / 16; ++c) {
            float v[16];
            tmem_ld16(taddr + c * 16, v);
            const int col0 = nt * LG_BN + c * 16;
            if (bias != nullptr) {
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (col0 + i < p.N) v[i] += __bfloat162float(bias[col0 + i]);
            }
            lg_store16(p, row, col0, v);
          }
        } else {
#pragma unroll 2
          for (int c = 0; c < LG_BN / 32; ++c) {
            float g[16], u[16];
            tmem_ld16(taddr + c * 16, g);
            tmem_ld16(taddr + LG_BN / 2 + c * 16, u);
            const int col0 = nt * (LG_BN / 2) + c * 16;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float gv = g[i], uv = u[i];
              if (bias != nullptr && col0 + i < p.n_out) {
                gv += __bfloat162float(bias[col0 + i]);
                uv += __bfloat162float(bias[p.n_out + col0 + i]);
              }
              g[i] = (p.act == 1 ? act_silu(gv) : act_gelu_tanh(gv)) * uv;
            }
            lg_store16(p, row, col0, g);
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[half]);  // the MMA warp may fill this half again
      }
    }
  }
  __syncwarp();  // the lanes of the two single-thread roles wait here for their lane 0
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(512) : "memory");
  }
}

// Shapes this kernel takes: K a multiple of 8 (16-byte rows for TMA), 16-byte aligned bases; with an activation N
// is even.  Any M (made for many rows: a tile holds 128).
extern "C" int ullm_linear_tcgen05_large_supported(int M, int N, int K) {
  return M >= 1 && N >= 1 && K >= 8 && K % 8 == 0;
}

static int g_lg_attr_set = 0;
static int g_lg_sms = 0;

extern "C" int ullm_linear_tcgen05_large(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                                         int out_f32, int act, int variant, int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (!ullm_linear_tcgen05_large_supported(M, N, K)) return ULLM_ERR_UNSUPPORTED;
  if (act < 0 || act > 2 || (act != 0 && N % 2 != 0)) return ULLM_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return ULLM_ERR_UNSUPPORTED;
  if (g_lg_sms == 0) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      return ULLM_ERR_LAUNCH;
    g_lg_sms = sms;
  }
  LgParams p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.act = act;
  p.n_out = act != 0 ? N / 2 : N;
  p.n_tiles = act != 0 ? (p.n_out + LG_BN / 2 - 1) / (LG_BN / 2) : (N + LG_BN - 1) / LG_BN;
  p.k_blocks = (K + LG_BK - 1) / LG_BK;
  p.out_f32 = out_f32;
  p.out = out;
  p.bias = bias;
  p.status = status;
  // Tiles of 128 or of 256 rows of x.  The second form moves two thirds of the bytes per product (measured: 0.885
  // of the time per tile-row where one round of tiles covers the product) but has half as many tiles to spread
  // over the SMs, and its epilogue is not hidden behind the next tile's products, which costs more than the
  // saved traffic where the epilogue is long (the gate activation) or runs many times per block.  So: rounds of
  // tiles x cost of a tile (4 against 7) decides for plain products; with an activation the 128-row form
  // stays.  `variant` forces one (1, 2) or lets that estimate choose (0).
  const long long t1 = (long long)((M + LG_BM - 1) / LG_BM) * p.n_tiles,
                  t2 = (long long)((M + LG2_BM - 1) / LG2_BM) * p.n_tiles;
  const long long c1 = ((t1 + g_lg_sms - 1) / g_lg_sms) * 4, c2 = ((t2 + g_lg_sms - 1) / g_lg_sms) * 7;
  const bool two = variant == 2 || (variant == 0 && act == 0 && M > LG_BM && c2 < c1);
  const int bm = two ? LG2_BM : LG_BM;
  p.m_tiles = (M + bm - 1) / bm;
  const long long tiles = (long long)p.m_tiles * p.n_tiles;
  const int blocks = (int)(tiles < g_lg_sms ? tiles : g_lg_sms);
  CUtensorMap map_x, map_w;
  if (!get_map(x, M, K, bm, &map_x) || !get_map(w, N, K, act != 0 ? -(LG_BN / 2) : LG_BN, &map_w))
    return ULLM_ERR_LAUNCH;
  const size_t smem = (two ? (size_t)LG2_STAGES * LG2_STAGE_BYTES : (size_t)LG_STAGES * LG_STAGE_BYTES) + 1024;
  if (!g_lg_attr_set) {
    if (cudaFuncSetAttribute(linear_tcgen05_large_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)(LG_STAGES * LG_STAGE_BYTES + 1024)) != cudaSuccess ||
        cudaFuncSetAttribute(linear_tcgen05_large2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)(LG2_STAGES * LG2_STAGE_BYTES + 1024)) != cudaSuccess)
      return ULLM_ERR_LAUNCH;
    g_lg_attr_set = 1;
  }
  int rc = two ? ullm_launch_kernel(linear_tcgen05_large2_kernel, dim3(blocks), dim3(LG_THREADS), smem, st, map_x, map_w, p)
               : ullm_launch_kernel(linear_tcgen05_large_kernel, dim3(blocks), dim3(LG_THREADS), smem, st, map_x, map_w, p);
  if (rc != ULLM_OK) return rc;
  return ullm_launch_status();
}
