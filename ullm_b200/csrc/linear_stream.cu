// out[M, N] = x[M, K] . W[N, K]^T for few rows (M <= 32: decode steps), bfloat16 in, 32-bit accumulate,
// bfloat16 or float32 out; optionally out[M, N/2] = act(gate) * up for a weight that stacks gate rows on up
// rows, and optionally out += residual (32-bit sum, rounded once).
//
// With so few rows the product is one pass of the weight matrix through the chip, and what decides its time
// is how early and how evenly the weight bytes are asked for.  This kernel is built around that:
//
//   * A unit is 32 weight rows (16 gate + 16 up rows with an activation) and all of K.  Units are dealt to the
//     blocks round robin; a block streams its units back to back through ONE ring of shared-memory stages, so
//     the ring never drains between units.  A stage holds 32 rows x 256 k of the weight (16 KB) and the same
//     256 k of all batch rows, both brought in by TMA (boxes of 16 rows x 64 k, 128-byte swizzle; rows and
//     columns outside the matrices read as zeros, so any N, any M <= 32 and any K that is a multiple of 8 work).
//   * One producer thread issues the TMA copies (a stage is one copy per matrix when K is a multiple of 64);
//     eight consumer warps multiply: warp w takes the 16-row half w & 1 and the 64-wide k quarter w >> 1 of
//     every stage, reads its fragments (ldmatrix from the swizzled boxes), gives the stage back and only then
//     issues the tensor instructions, with the weight rows on the M side of mma.sync.m16n8k16 and the batch
//     rows on its N side.  The four k quarters of a half meet in shared memory at the end of a unit and are
//     added in a fixed order.
//   * The weights do not depend on the kernel before this one in the stream.  Under programmatic dependent
//     launch the producer fills the whole ring with weight tiles BEFORE griddepcontrol.wait and asks for the
//     batch rows after it, so that this kernel's first megabytes stream while the kernel before it drains.
//     A block needs at most 112 KB of shared memory: its successor's blocks fit beside it on the SM.
//   * A narrow output has too few units to give every SM something to stream.  Then 2, 4 or 8 blocks form a
//     thread-block cluster around one unit, each takes a range of K, and ranks 1.. put their sums into rank 0's
//     shared memory (distributed shared memory, released by an arrival at rank 0's barrier); rank 0 adds them in
//     rank order and writes the result.
//   * Every mbarrier wait is bounded; a wait that runs out records ULLM_STATUS_TIMEOUT, the block stops
//     computing but keeps arriving at its barriers, waits (bounded) for the copies it still has in flight, and
//     returns.
#include "linear_stream_core.cuh"

#define LS_UNIT_ROWS 32

struct LsParams {
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, n_out] or null: out = product (+ bias) + residual
  void* out;                      // [M, n_out]
  int M, N, K;
  int n_out;                      // N, or N / 2 with an activation
  int act;                        // 0 none, 1 silu(gate) * up, 2 gelu_tanh(gate) * up
  int out_f32;
  int num_units;
  int k_blocks;                   // ceil(K / 256)
  int stages;
  int chunked;                    // K is a multiple of 64: a stage comes in by one copy per matrix (3-D boxes)
  int ksplit;                     // 1, 2, 4 or 8: blocks of a cluster that share a unit, each with a range of K
  // An RMSNorm folded around two products (rmsnorm(r) * w = (1 / rms(r)) * (r * w)):
  //   the product in FRONT of the norm (plain, with a residual) also writes r * pre_w, rounded once, as the
  //   next product's operand, and per unit and 16-row half the rows' sums of squares of r;
  const float* pre_w;             // [n_out] norm weight, or null
  __nv_bfloat16* pre_out;         // [M, n_out]
  float* sq_out;                  // [units][2][16]
  //   the product BEHIND it multiplies its 32-bit sums by the rows' 1 / rms before bias and activation.
  const float* sq_in;             // [sq_count][16] partial sums of squares, or null
  int sq_count;
  float sq_inv_cols, sq_eps;      // 1 / (columns of the normed row), the norm's eps
  int* status;
};

// ---- cluster helpers: a block's rank, a peer's shared-memory address, remote stores and barrier arrivals ------
__device__ __forceinline__ uint32_t ls_map_to_rank(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void ls_st_cluster_f4(uint32_t addr, float4 v) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ void ls_arrive_cluster(uint32_t bar_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_addr) : "memory");
}
// bounded wait that also makes the peers' stores (released at cluster scope) visible
__device__ __forceinline__ bool ls_wait_cluster(uint64_t* bar, uint32_t parity) {
  for (int i = 0; i < WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(lin_smem(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void ls_cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// NT: tiles of 8 batch rows (M <= 8 NT).
template <int NT>
__global__ void __launch_bounds__(LS_THREADS, 2) linear_stream_kernel(const __grid_constant__ CUtensorMap w_map,
                                                                   const __grid_constant__ CUtensorMap w32_map,
                                                                   const __grid_constant__ CUtensorMap x_map,
                                                                   const LsParams p) {
  constexpr int XR = 8 * NT;                                    // batch rows of a stage
  constexpr int X_BOX_BYTES = XR * 128;                         // one box: XR rows x 64 k
  constexpr int STAGE_BYTES = LS_W_STAGE_BYTES + 4 * X_BOX_BYTES;
  extern __shared__ unsigned char ls_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[LS_MAX_STAGES], empty_bar[LS_MAX_STAGES];
  __shared__ __align__(8) uint64_t peer_bar;  // rank 0: the peers' partial sums of the current unit have arrived
  __shared__ float rstd_s[16], part_s[16][17];  // the rows' 1 / rms (a norm folded in front of this product)
  __shared__ int abort_flag;
  pdl_launch_dependents();
  unsigned char* ring = (unsigned char*)(((uintptr_t)ls_smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int NP = NT > 1 ? 2 : 1;                            // batch tiles that meet per pass
  float* red = reinterpret_cast<float*>(ring + p.stages * STAGE_BYTES);  // [8 warps][32 lanes][NP][4]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A cluster of `ksplit` blocks (consecutive blockIdx.x) shares its units: rank r takes k blocks
  // [r * kper, (r + 1) * kper) of each, rank 0 gathers the partial sums and writes the result.
  const int rank = (int)blockIdx.x % p.ksplit, cid = (int)blockIdx.x / p.ksplit, ncl = (int)gridDim.x / p.ksplit;
  const int kper = (p.k_blocks + p.ksplit - 1) / p.ksplit;
  const int kb0 = rank * kper;
  const int nkb = p.k_blocks - kb0 < kper ? (p.k_blocks - kb0 > 0 ? p.k_blocks - kb0 : 0) : kper;  // this block's k blocks
  const int my_units = p.num_units > cid ? (p.num_units - 1 - cid) / ncl + 1 : 0;
  const int total_it = my_units * nkb;
  const int half_rows = p.act ? p.N / 2 : 0;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], LS_CONSUMER_WARPS);
    }
    mbar_init(&peer_bar, 64 * (p.ksplit > 1 ? p.ksplit - 1 : 1));  // every lane of the peers' two finishing warps
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  if (p.ksplit > 1) ls_cluster_sync_all();  // the peers' barriers exist before anyone arrives at them

  if (warp == LS_CONSUMER_WARPS) {
    // ---- producer ---------------------------------------------------------------------------------
    // K a multiple of 64: lane 0 brings a stage with one copy per matrix (three-dimensional boxes).  Otherwise
    // lanes 0 to 3 each bring one 64-wide k quarter with two-dimensional boxes, whose ragged last columns read
    // as zeros.  A stage: weight rows of unit u (plain: 32 consecutive rows; with an activation 16 gate rows
    // and the 16 up rows of the same columns), then the batch rows.
    const int lanes = p.chunked ? 1 : 4;
    if (lane < lanes) {
      const int kc = lane;
      // One thread's instruction stream is what paces the ring: no division per stage.  The position in the list
      // of stages (unit, k block) and in the ring (slot, round) is carried along and stepped.
      struct Pos {
        int u, kb, slot, round;
      };
      auto step = [&](Pos& q) {
        if (++q.kb == nkb) q.kb = 0, q.u += ncl;
        if (++q.slot == p.stages) q.slot = 0, ++q.round;
      };
      auto issue_w = [&](const Pos& q) {
        unsigned char* st = ring + q.slot * STAGE_BYTES;
        const int kb = kb0 + q.kb;
        if (lane == 0) mbar_expect_tx(&full_bar[q.slot], STAGE_BYTES);
        if (p.chunked) {
          if (p.act) {
            tma_load_3d(st, &w_map, &full_bar[q.slot], 0, q.u * 16, kb * 4);
            tma_load_3d(st + 8192, &w_map, &full_bar[q.slot], 0, half_rows + q.u * 16, kb * 4);
          } else {
            tma_load_3d(st, &w32_map, &full_bar[q.slot], 0, q.u * 32, kb * 4);
          }
          return;
        }
        __syncwarp(0xf);
        if (p.act) {
          tma_load_2d(st + (0 * 4 + kc) * 2048, &w_map, &full_bar[q.slot], kb * LS_BK + kc * 64, q.u * 16);
          tma_load_2d(st + (1 * 4 + kc) * 2048, &w_map, &full_bar[q.slot], kb * LS_BK + kc * 64, half_rows + q.u * 16);
        } else {
          tma_load_2d(st + kc * 4096, &w32_map, &full_bar[q.slot], kb * LS_BK + kc * 64, q.u * 32);
        }
      };
      auto issue_x = [&](const Pos& q) {
        unsigned char* st = ring + q.slot * STAGE_BYTES + LS_W_STAGE_BYTES;
        const int kb = kb0 + q.kb;
        if (p.chunked)
          tma_load_3d(st, &x_map, &full_bar[q.slot], 0, 0, kb * 4);
        else
          tma_load_2d(st + kc * X_BOX_BYTES, &x_map, &full_bar[q.slot], kb * LS_BK + kc * 64, 0);
      };
      const int first = total_it < p.stages ? total_it : p.stages;
      Pos w = {cid, 0, 0, 0};
      for (int it = 0; it < first; ++it, step(w)) issue_w(w);  // the weights: before the kernel in front has finished
      pdl_wait();
      Pos x = {cid, 0, 0, 0};
      for (int it = 0; it < first; ++it, step(x)) issue_x(x);  // the batch rows: what that kernel wrote
      for (int it = first; it < total_it; ++it, step(w)) {
        if (!mbar_wait(&empty_bar[w.slot], (w.round - 1) & 1)) {
          ullm_report(p.status, ULLM_STATUS_TIMEOUT, 51, it);
          abort_flag = 1;
          break;  // (the four lanes wait on the same barrier: all of them give up or none)
        }
        issue_w(w);
        issue_x(w);
      }
    } else {
      pdl_wait();
    }
  } else {
    // ---- consumers --------------------------------------------------------------------------------
    pdl_wait();
    if (p.sq_in != nullptr) {
      // the rows' 1 / rms from the partial sums of squares that the product in front left (16 parts per row, all
      // loads of a thread in flight together; parts added in a fixed order)
      const int m = threadIdx.x & 15, part = threadIdx.x >> 4;
      const int per = (p.sq_count + 15) / 16;
      float sum = 0.f;
      for (int q0 = part * per; q0 < (part + 1) * per && q0 < p.sq_count; q0 += 8) {
        float v8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e)
          v8[e] = (q0 + e < (part + 1) * per && q0 + e < p.sq_count) ? __ldcg(p.sq_in + (size_t)(q0 + e) * 16 + m) : 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) sum += v8[e];
      }
      part_s[part][m] = sum;
      ls_bar_sync_consumers();
      if (threadIdx.x < 16) {
        float tot = 0.f;
        for (int q = 0; q < 16; ++q) tot += part_s[q][threadIdx.x];
        rstd_s[threadIdx.x] = rsqrtf(tot * p.sq_inv_cols + p.sq_eps);
      }
      ls_bar_sync_consumers();
    }
    const int mt = warp & 1, kq = warp >> 1;
    const int g = lane >> 2, t = lane & 3;
    // ldmatrix row addresses inside a box (rows of 128 bytes, 16-byte chunks XORed with row & 7)
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8;  // matrices 0, 1: rows 0-7, 8-15 (k 0-7); 2, 3: k 8-15
    const int a_chunk = lane >> 4;
    const int b_row = (lane & 7) + (lane >> 4) * 8;        // matrices 0, 1: batch rows 0-7 (k 0-7, 8-15); 2, 3: rows 8-15
    const int b_chunk = (lane >> 3) & 1;
    bool failed = false;
    int s = 0;             // the ring slot of the next stage and the parity of its use, stepped (no division per stage)
    uint32_t parity = 0;
    for (int ui = 0; ui < my_units; ++ui) {
      float acc[NT][4];
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
      // What the end of an output element adds (the residual, the norm weight of a norm folded behind this
      // product) is fetched now by the threads that will finish the unit: its way from L2 then runs beside the
      // k loop, not behind it.
      float res_pre[NT][4], pw_pre[2] = {0.f, 0.f};
      const bool finisher = kq == 0 && rank == 0 && (p.act == 0 || mt == 0);
      if (finisher && (p.residual != nullptr || p.pre_w != nullptr)) {
        const int u2 = cid + ui * ncl;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int col = p.act ? u2 * 16 + g + 8 * i : u2 * 32 + mt * 16 + g + 8 * i;
          if (p.pre_w != nullptr && col < p.n_out) pw_pre[i] = __ldg(p.pre_w + col);
        }
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int col = p.act ? u2 * 16 + g + 8 * (i >> 1) : u2 * 32 + mt * 16 + g + 8 * (i >> 1);
            const int m = n * 8 + 2 * t + (i & 1);
            res_pre[n][i] = (p.residual != nullptr && m < p.M && col < p.n_out)
                                ? __bfloat162float(p.residual[(size_t)m * p.n_out + col]) : 0.f;
          }
      }
      for (int kb = 0; kb < nkb; ++kb) {
        if (!failed && !__all_sync(0xffffffffu, mbar_wait(&full_bar[s], parity))) {
          ullm_report(p.status, ULLM_STATUS_TIMEOUT, 52, ui * nkb + kb);  // (the whole warp gives up together)
          abort_flag = 1;
          failed = true;
        }
        if (!failed) {
          const uint32_t wbox = lin_smem(ring + s * STAGE_BYTES + (p.act ? (mt * 4 + kq) * 2048 : kq * 4096 + mt * 2048));
          const uint32_t xbox = lin_smem(ring + s * STAGE_BYTES + LS_W_STAGE_BYTES + kq * X_BOX_BYTES);
          // the quarter's fragments first, then the tensor instructions: the stage goes back as soon as it is read
          uint32_t a[4][4], b[4][NT * 2];
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // k16 steps of the 64-wide quarter
            ls_ldmatrix4(a[j], wbox + a_row * 128 + (((j * 2 + a_chunk) ^ (a_row & 7)) << 4));
            if (NT == 1) {
              const int r = lane & 7, c = (lane >> 3) & 1;
              ls_ldmatrix2(b[j][0], b[j][1], xbox + r * 128 + (((j * 2 + c) ^ r) << 4));
            } else {
#pragma unroll
              for (int n2 = 0; n2 < NT / 2; ++n2) {
                uint32_t t4[4];
                const int r = b_row + n2 * 16;
                ls_ldmatrix4(t4, xbox + r * 128 + (((j * 2 + b_chunk) ^ (r & 7)) << 4));
                b[j][n2 * 4] = t4[0], b[j][n2 * 4 + 1] = t4[1], b[j][n2 * 4 + 2] = t4[2], b[j][n2 * 4 + 3] = t4[3];
              }
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&empty_bar[s]);
#pragma unroll
          for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int n = 0; n < NT; ++n) ls_mma(acc[n], a[j], b[j][n * 2], b[j][n * 2 + 1]);
        } else {
          __syncwarp();
          if (lane == 0) mbar_arrive(&empty_bar[s]);
        }
        if (++s == p.stages) s = 0, parity ^= 1;
      }
      // ---- the four k quarters of each half meet (two batch tiles per pass); warps 0 and 1 (quarter 0)
      // finish the unit --------------------------------------------------------------------------------
      const int u = cid + ui * ncl;
      // the end of an output element: bias, activation, residual, one rounding, the store
      float ss[NT][2];  // (a norm behind this product) sums of squares of this thread's results, per batch row
#pragma unroll
      for (int n = 0; n < NT; ++n) ss[n][0] = ss[n][1] = 0.f;
      auto finish = [&](int n_tile, const float (&v)[4], const float (&up)[4]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          // accumulator element i: weight row g + 8 (i >> 1), batch row 8 n_tile + 2 t + (i & 1)
          const int row = g + 8 * (i >> 1);
          const int m = n_tile * 8 + 2 * t + (i & 1);
          const int col = p.act ? u * 16 + row : u * 32 + mt * 16 + row;  // column of out
          if (m >= p.M || col >= p.n_out) continue;
          const float rs = p.sq_in != nullptr ? rstd_s[m] : 1.f;
          float r = v[i] * rs;
          if (p.act) {
            float gate = r, upv = up[i] * rs;
            if (p.bias != nullptr) {
              gate += __bfloat162float(p.bias[col]);
              upv += __bfloat162float(p.bias[half_rows + col]);
            }
            r = (p.act == 1 ? act_silu(gate) : act_gelu_tanh(gate)) * upv;
          } else if (p.bias != nullptr) {
            r += __bfloat162float(p.bias[col]);
          }
          const size_t o = (size_t)m * p.n_out + col;
          if (p.residual != nullptr) r += res_pre[n_tile][i];
          if (p.out_f32)
            reinterpret_cast<float*>(p.out)[o] = r;
          else
            reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(r);
          if (p.pre_w != nullptr) {
            p.pre_out[o] = __float2bfloat16_rn(r * pw_pre[i >> 1]);
            ss[n_tile][i & 1] += r * r;
          }
        }
      };
      // the unit's sums of squares per batch row: over the 8 lanes that share t, then one store each
      auto store_sq = [&]() {
        if (p.pre_w == nullptr) return;
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float sv = ss[n][e];
            sv += __shfl_xor_sync(0xffffffffu, sv, 4);
            sv += __shfl_xor_sync(0xffffffffu, sv, 8);
            sv += __shfl_xor_sync(0xffffffffu, sv, 16);
            if (g == 0 && n * 8 + 2 * t + e < 16) p.sq_out[((size_t)u * 2 + mt) * 16 + n * 8 + 2 * t + e] = sv;
          }
        if (NT == 1 && g == 0) {  // rows 8 to 15 do not exist
          p.sq_out[((size_t)u * 2 + mt) * 16 + 8 + 2 * t] = 0.f;
          p.sq_out[((size_t)u * 2 + mt) * 16 + 8 + 2 * t + 1] = 0.f;
        }
      };
      float v_all[NT][4];  // (clusters) this block's sums of the unit, kept until the peers' have arrived
#pragma unroll
      for (int n0 = 0; n0 < NT; n0 += NP) {
#pragma unroll
        for (int n = 0; n < NP; ++n)
          *reinterpret_cast<float4*>(red + ((size_t)(warp * 32 + lane) * NP + n) * 4) =
              make_float4(acc[n0 + n][0], acc[n0 + n][1], acc[n0 + n][2], acc[n0 + n][3]);
        ls_bar_sync_consumers();
        if (kq == 0 && (p.act == 0 || mt == 0)) {
#pragma unroll
          for (int n = 0; n < NP; ++n) {
            float v[4] = {0.f, 0.f, 0.f, 0.f}, up[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int q = 0; q < 4; ++q) {  // in quarter order: the same sum whatever the timing
              const float4 pv = *reinterpret_cast<const float4*>(red + ((size_t)((q * 2 + mt) * 32 + lane) * NP + n) * 4);
              v[0] += pv.x, v[1] += pv.y, v[2] += pv.z, v[3] += pv.w;
              if (p.act) {
                const float4 pu = *reinterpret_cast<const float4*>(red + ((size_t)((q * 2 + 1) * 32 + lane) * NP + n) * 4);
                up[0] += pu.x, up[1] += pu.y, up[2] += pu.z, up[3] += pu.w;
              }
            }
            if (p.ksplit == 1) {
              if (!failed) finish(n0 + n, v, up);
            } else {
#pragma unroll
              for (int i = 0; i < 4; ++i) v_all[n0 + n][i] = v[i];
            }
          }
        }
        ls_bar_sync_consumers();  // the partial sums are read: the next pass may overwrite them
      }
      if (p.ksplit == 1 && kq == 0 && !failed) store_sq();
      if (p.ksplit > 1 && kq == 0) {
        // ---- the blocks of the cluster meet: ranks 1.. put their sums into rank 0's buffer (distributed shared
        // memory) and arrive at its barrier; rank 0 adds them in rank order and finishes the unit.  (The host
        // gives a cluster at most one unit, so the buffer is written once.)
        float* xbuf = red + LS_CONSUMER_WARPS * 32 * NP * 4;  // [ksplit - 1][2 halves][32 lanes][NT][4]
        if (rank > 0) {
          const uint32_t dst = ls_map_to_rank(lin_smem(xbuf + ((size_t)((rank - 1) * 2 + mt) * 32 + lane) * NT * 4), 0);
#pragma unroll
          for (int n = 0; n < NT; ++n)
            ls_st_cluster_f4(dst + n * 16, make_float4(v_all[n][0], v_all[n][1], v_all[n][2], v_all[n][3]));
          ls_arrive_cluster(ls_map_to_rank(lin_smem(&peer_bar), 0));
        } else {
          if (!failed && !__all_sync(0xffffffffu, ls_wait_cluster(&peer_bar, ui & 1))) {
            ullm_report(p.status, ULLM_STATUS_TIMEOUT, 53, ui);
            abort_flag = 1;
            failed = true;
          }
          if (!failed) {
            const float zero[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int n = 0; n < NT; ++n) {
              for (int r = 1; r < p.ksplit; ++r) {
                const float4 pv = *reinterpret_cast<const float4*>(xbuf + (((size_t)((r - 1) * 2 + mt) * 32 + lane) * NT + n) * 4);
                v_all[n][0] += pv.x, v_all[n][1] += pv.y, v_all[n][2] += pv.z, v_all[n][3] += pv.w;
              }
              finish(n, v_all[n], zero);
            }
            store_sq();
          }
        }
      }
    }
  }
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) {
    // a wait ran out: copies may still be on their way into the ring; wait (bounded) for the last phase of
    // every stage before the block gives its shared memory back
    for (int s = 0; s < p.stages; ++s) {
      int last = -1;
      for (int it = s; it < total_it; it += p.stages) last = it;
      if (last >= 0) mbar_wait(&full_bar[s], (last / p.stages) & 1);
    }
  }
  if (p.ksplit > 1) ls_cluster_sync_all();  // no block leaves while a peer may still write to it or arrive at its barrier
}

static int g_ls_sms = 0;
static int g_ls_attr[3] = {0, 0, 0};
static int g_ls_blocks_per_sm = 2;  // blocks the launcher aims for per SM
static int g_ls_smem_kb = 108;      // shared memory a block may take (ring + partial sums): two blocks per SM

extern "C" void ullm_linear_stream_blocks_per_sm(int n) { g_ls_blocks_per_sm = n < 1 ? 1 : (n > 2 ? 2 : n); }
extern "C" void ullm_linear_stream_smem_kb(int kb) { g_ls_smem_kb = kb < 72 ? 72 : (kb > 224 ? 224 : kb); }

extern "C" int ullm_linear_stream_supported(int M, int N, int K) {
  return M >= 1 && M <= 32 && N >= 1 && K >= 8 && K % 8 == 0;
}

static int g_ls_ksplit_max = 8;  // 1 switches the clusters off (measurements compare)
extern "C" void ullm_linear_stream_ksplit_max(int n) { g_ls_ksplit_max = n < 1 ? 1 : (n > 8 ? 8 : n); }

template <int NT>
static int ls_launch(int which, const CUtensorMap& wm, const CUtensorMap& wm32, const CUtensorMap& xm, LsParams p,
                     cudaStream_t st) {
  constexpr int STAGE_BYTES = LS_W_STAGE_BYTES + 4 * 8 * NT * 128;
  const int slots = g_ls_sms * g_ls_blocks_per_sm;
  // Few units (a narrow output): the blocks of a cluster share a unit, each with a range of K, so that every SM
  // has something to stream.  Only plain products (no activation), one unit per cluster, at least two k blocks
  // per block.
  int ksplit = 1;
  if (p.act == 0)
    while (ksplit * 2 <= g_ls_ksplit_max && p.num_units * ksplit * 2 <= slots && p.k_blocks >= ksplit * 4) ksplit *= 2;
  p.ksplit = ksplit;
  const int red_bytes = LS_CONSUMER_WARPS * 32 * (NT > 1 ? 2 : 1) * 4 * (int)sizeof(float);
  const int xbuf_bytes = (ksplit - 1) * 2 * 32 * NT * 4 * (int)sizeof(float);
  int stages = (g_ls_smem_kb * 1024 - 1024 - red_bytes - xbuf_bytes) / STAGE_BYTES;
  if (stages > LS_MAX_STAGES) stages = LS_MAX_STAGES;
  if (stages < 2) return ULLM_ERR_UNSUPPORTED;
  p.stages = stages;
  const size_t smem = (size_t)stages * STAGE_BYTES + red_bytes + xbuf_bytes + 1024;
  if (!g_ls_attr[which]) {
    if (cudaFuncSetAttribute(linear_stream_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024) !=
        cudaSuccess)
      return ULLM_ERR_LAUNCH;
    cudaFuncSetAttribute(linear_stream_kernel<NT>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    g_ls_attr[which] = 1;
  }
  if (ksplit == 1) {
    int grid = slots;
    if (grid > p.num_units) grid = p.num_units;
    return ullm_launch_kernel(linear_stream_kernel<NT>, dim3(grid), dim3(LS_THREADS), smem, st, wm, wm32, xm, p);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.num_units * ksplit);
  cfg.blockDim = dim3(LS_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)ksplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_ullm_pdl ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, linear_stream_kernel<NT>, wm, wm32, xm, p) != cudaSuccess) {
    cudaGetLastError();
    return ULLM_ERR_LAUNCH;
  }
  return ULLM_OK;
}

// Floats of `sq_out` for a product with N output columns: [units][2][16].
extern "C" long long ullm_linear_stream_sq_floats(int N) { return (long long)((N + 31) / 32) * 2 * 16; }

// act: 0 none, 1 silu gate, 2 gelu_tanh gate (weight = [gate rows; up rows], out [M, N / 2]).
// residual: null or [M, n_out] bfloat16, added to the product in 32-bit before the one rounding.
// pre_w / pre_out / sq_out (all or none; plain products of at most 16 rows): also write result * pre_w and the
// units' sums of squares, for an RMSNorm folded behind this product.  sq_in / sq_count / sq_cols / sq_eps: the sums
// of squares that such a product left; this product multiplies its sums by the rows' 1 / rms.
extern "C" int ullm_linear_stream_norm(const void* x, const void* w, const void* bias, const void* residual, void* out,
                                       int M, int N, int K, int out_f32, int act, const float* pre_w, void* pre_out,
                                       float* sq_out, const float* sq_in, int sq_count, int sq_cols, float sq_eps,
                                       int* status, void* stream);

extern "C" int ullm_linear_stream(const void* x, const void* w, const void* bias, const void* residual, void* out,
                                  int M, int N, int K, int out_f32, int act, int* status, void* stream) {
  return ullm_linear_stream_norm(x, w, bias, residual, out, M, N, K, out_f32, act, nullptr, nullptr, nullptr, nullptr, 0,
                                 0, 0.f, status, stream);
}

extern "C" int ullm_linear_stream_norm(const void* x, const void* w, const void* bias, const void* residual, void* out,
                                       int M, int N, int K, int out_f32, int act, const float* pre_w, void* pre_out,
                                       float* sq_out, const float* sq_in, int sq_count, int sq_cols, float sq_eps,
                                       int* status, void* stream) {
  if ((pre_w != nullptr) != (pre_out != nullptr) || (pre_w != nullptr) != (sq_out != nullptr)) return ULLM_ERR_BAD_SIZE;
  if (pre_w != nullptr && (act != 0 || M > 16)) return ULLM_ERR_UNSUPPORTED;
  if (sq_in != nullptr && (sq_count <= 0 || sq_cols <= 0 || M > 16)) return ULLM_ERR_BAD_SIZE;
  if (!ullm_linear_stream_supported(M, N, K)) return ULLM_ERR_UNSUPPORTED;
  if (act < 0 || act > 2 || (act && (N % 2))) return ULLM_ERR_BAD_SIZE;
  if (g_ls_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&g_ls_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || g_ls_sms <= 0)
      return ULLM_ERR_LAUNCH;
  }
  const int NT = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
  CUtensorMap wm, wm32, xm;
  const int chunked = K % 64 == 0;
  // x as a matrix of exactly M rows: boxes of 8 NT rows read zeros past them
  if (chunked) {
    if (!ls_chunked_map(w, N, K, 16, &wm) || !ls_chunked_map(w, N, K, 32, &wm32) ||
        !ls_chunked_map(x, M, K, 8 * NT, &xm))
      return ULLM_ERR_LAUNCH;
  } else if (!get_map(w, N, K, 16, &wm) || !get_map(w, N, K, 32, &wm32) || !get_map(x, M, K, 8 * NT, &xm)) {
    return ULLM_ERR_LAUNCH;
  }
  LsParams p;
  p.bias = (const __nv_bfloat16*)bias;
  p.residual = (const __nv_bfloat16*)residual;
  p.out = out;
  p.M = M, p.N = N, p.K = K;
  p.n_out = act ? N / 2 : N;
  p.act = act;
  p.out_f32 = out_f32;
  p.num_units = act ? (N / 2 + 15) / 16 : (N + 31) / 32;
  p.k_blocks = (K + LS_BK - 1) / LS_BK;
  p.stages = 0;
  p.chunked = chunked;
  p.ksplit = 1;
  p.pre_w = pre_w;
  p.pre_out = (__nv_bfloat16*)pre_out;
  p.sq_out = sq_out;
  p.sq_in = sq_in;
  p.sq_count = sq_count;
  p.sq_inv_cols = sq_cols > 0 ? 1.f / (float)sq_cols : 0.f;
  p.sq_eps = sq_eps;
  p.status = status;
  if (NT == 1) return ls_launch<1>(0, wm, wm32, xm, p, (cudaStream_t)stream);
  if (NT == 2) return ls_launch<2>(1, wm, wm32, xm, p, (cudaStream_t)stream);
  return ls_launch<4>(2, wm, wm32, xm, p, (cudaStream_t)stream);
}
