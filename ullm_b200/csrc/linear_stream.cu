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
//   * One producer thread issues the TMA copies; eight consumer warps multiply: warp w takes the 16-row half
//     w & 1 and the 64-wide k quarter w >> 1 of every stage, with the weight rows on the M side of
//     mma.sync.m16n8k16 and the batch rows on its N side (ldmatrix from the swizzled boxes).  The four k
//     quarters of a half meet in shared memory at the end of a unit and are added in a fixed order.
//   * The weights do not depend on the kernel before this one in the stream.  Under programmatic dependent
//     launch the producer fills the whole ring with weight tiles BEFORE griddepcontrol.wait and asks for the
//     batch rows after it, so that this kernel's first megabytes stream while the kernel before it drains.
//     A block needs at most 112 KB of shared memory: its successor's blocks fit beside it on the SM.
//   * Every mbarrier wait is bounded; a wait that runs out records ULLM_STATUS_TIMEOUT, the block stops
//     computing but keeps arriving at its barriers, waits (bounded) for the copies it still has in flight, and
//     returns.
#include "tcgen05_util.cuh"

#define LS_CONSUMER_WARPS 8
#define LS_THREADS (32 * (LS_CONSUMER_WARPS + 1))
#define LS_UNIT_ROWS 32
#define LS_BK 256                 // k per stage
#define LS_W_STAGE_BYTES 16384    // 32 rows x 256 k x 2 bytes
#define LS_MAX_SMEM (112 * 1024)

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
  int* status;
};

__device__ __forceinline__ void ls_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ls_ldmatrix4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ls_ldmatrix2(uint32_t& r0, uint32_t& r1, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ls_bar_sync_consumers() {
  asm volatile("bar.sync 1, %0;" ::"n"(LS_CONSUMER_WARPS * 32) : "memory");
}

// NT: tiles of 8 batch rows (M <= 8 NT).
template <int NT>
__global__ void __launch_bounds__(LS_THREADS) linear_stream_kernel(const __grid_constant__ CUtensorMap w_map,
                                                                   const __grid_constant__ CUtensorMap x_map,
                                                                   const LsParams p) {
  constexpr int XR = 8 * NT;                                    // batch rows of a stage
  constexpr int X_BOX_BYTES = XR * 128;                         // one box: XR rows x 64 k
  constexpr int STAGE_BYTES = LS_W_STAGE_BYTES + 4 * X_BOX_BYTES;
  extern __shared__ unsigned char ls_smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[8], empty_bar[8];
  __shared__ int abort_flag;
  pdl_launch_dependents();
  unsigned char* ring = (unsigned char*)(((uintptr_t)ls_smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int NP = NT > 1 ? 2 : 1;                            // batch tiles that meet per pass
  float* red = reinterpret_cast<float*>(ring + p.stages * STAGE_BYTES);  // [8 warps][32 lanes][NP][4]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int my_units = p.num_units > (int)blockIdx.x ? (p.num_units - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const int total_it = my_units * p.k_blocks;
  const int half_rows = p.act ? p.N / 2 : 0;

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
    // ---- producer ---------------------------------------------------------------------------------
    if (lane == 0) {
      // weight rows of unit u: plain, 32 consecutive rows; with an activation 16 gate rows and the 16 up rows
      // of the same columns
      auto issue_w = [&](int it) {
        const int s = it % p.stages;
        const int u = (int)blockIdx.x + (it / p.k_blocks) * (int)gridDim.x;
        const int kb = it % p.k_blocks;
        unsigned char* st = ring + s * STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        const int r0 = p.act ? u * 16 : u * 32;
        const int r1 = p.act ? half_rows + u * 16 : u * 32 + 16;
#pragma unroll
        for (int kc = 0; kc < 4; ++kc) {
          tma_load_2d(st + (0 * 4 + kc) * 2048, &w_map, &full_bar[s], kb * LS_BK + kc * 64, r0);
          tma_load_2d(st + (1 * 4 + kc) * 2048, &w_map, &full_bar[s], kb * LS_BK + kc * 64, r1);
        }
      };
      auto issue_x = [&](int it) {
        const int s = it % p.stages;
        const int kb = it % p.k_blocks;
        unsigned char* st = ring + s * STAGE_BYTES + LS_W_STAGE_BYTES;
#pragma unroll
        for (int kc = 0; kc < 4; ++kc) tma_load_2d(st + kc * X_BOX_BYTES, &x_map, &full_bar[s], kb * LS_BK + kc * 64, 0);
      };
      const int first = total_it < p.stages ? total_it : p.stages;
      for (int it = 0; it < first; ++it) issue_w(it);  // the weights: before the kernel in front has finished
      pdl_wait();
      for (int it = 0; it < first; ++it) issue_x(it);  // the batch rows: what that kernel wrote
      bool failed = false;
      for (int it = first; it < total_it && !failed; ++it) {
        const int s = it % p.stages;
        if (!mbar_wait(&empty_bar[s], ((it / p.stages) - 1) & 1)) {
          ullm_report(p.status, ULLM_STATUS_TIMEOUT, 51, it);
          abort_flag = 1;
          failed = true;
          break;
        }
        issue_w(it);
        issue_x(it);
      }
    } else {
      pdl_wait();
    }
  } else {
    // ---- consumers --------------------------------------------------------------------------------
    pdl_wait();
    const int mt = warp & 1, kq = warp >> 1;
    const int g = lane >> 2, t = lane & 3;
    // ldmatrix row addresses inside a box (rows of 128 bytes, 16-byte chunks XORed with row & 7)
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8;  // matrices 0, 1: rows 0-7, 8-15 (k 0-7); 2, 3: k 8-15
    const int a_chunk = lane >> 4;
    const int b_row = (lane & 7) + (lane >> 4) * 8;        // matrices 0, 1: batch rows 0-7 (k 0-7, 8-15); 2, 3: rows 8-15
    const int b_chunk = (lane >> 3) & 1;
    bool failed = false;
    int it = 0;
    for (int ui = 0; ui < my_units; ++ui) {
      float acc[NT][4];
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
      for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
        const int s = it % p.stages;
        if (!failed && !mbar_wait(&full_bar[s], (it / p.stages) & 1)) {
          ullm_report(p.status, ULLM_STATUS_TIMEOUT, 52, it);
          abort_flag = 1;
          failed = true;
        }
        if (!failed) {
          const uint32_t wbox = lin_smem(ring + s * STAGE_BYTES + (mt * 4 + kq) * 2048);
          const uint32_t xbox = lin_smem(ring + s * STAGE_BYTES + LS_W_STAGE_BYTES + kq * X_BOX_BYTES);
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // k16 steps of the 64-wide quarter
            uint32_t a[4];
            ls_ldmatrix4(a, wbox + a_row * 128 + (((j * 2 + a_chunk) ^ (a_row & 7)) << 4));
            if (NT == 1) {
              uint32_t b0, b1;
              const int r = lane & 7, c = (lane >> 3) & 1;
              ls_ldmatrix2(b0, b1, xbox + r * 128 + (((j * 2 + c) ^ r) << 4));
              ls_mma(acc[0], a, b0, b1);
            } else {
#pragma unroll
              for (int n2 = 0; n2 < NT / 2; ++n2) {
                uint32_t b[4];
                const int r = b_row + n2 * 16;
                ls_ldmatrix4(b, xbox + r * 128 + (((j * 2 + b_chunk) ^ (r & 7)) << 4));
                ls_mma(acc[n2 * 2], a, b[0], b[1]);
                ls_mma(acc[n2 * 2 + 1], a, b[2], b[3]);
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[s]);
      }
      // ---- the four k quarters of each half meet (two batch tiles per pass); warps 0 and 1 (quarter 0)
      // finish the unit --------------------------------------------------------------------------------
      const int u = (int)blockIdx.x + ui * (int)gridDim.x;
#pragma unroll
      for (int n0 = 0; n0 < NT; n0 += NP) {
#pragma unroll
        for (int n = 0; n < NP; ++n)
          *reinterpret_cast<float4*>(red + ((size_t)(warp * 32 + lane) * NP + n) * 4) =
              make_float4(acc[n0 + n][0], acc[n0 + n][1], acc[n0 + n][2], acc[n0 + n][3]);
        ls_bar_sync_consumers();
        if (!failed && kq == 0 && (p.act == 0 || mt == 0)) {
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
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              // accumulator element i: weight row g + 8 (i >> 1), batch row 8 (n0 + n) + 2 t + (i & 1)
              const int row = g + 8 * (i >> 1);
              const int m = (n0 + n) * 8 + 2 * t + (i & 1);
              const int col = p.act ? u * 16 + row : u * 32 + mt * 16 + row;  // column of out
              if (m >= p.M || col >= p.n_out) continue;
              float r = v[i];
              if (p.act) {
                float gate = r, upv = up[i];
                if (p.bias != nullptr) {
                  gate += __bfloat162float(p.bias[col]);
                  upv += __bfloat162float(p.bias[half_rows + col]);
                }
                r = (p.act == 1 ? act_silu(gate) : act_gelu_tanh(gate)) * upv;
              } else if (p.bias != nullptr) {
                r += __bfloat162float(p.bias[col]);
              }
              const size_t o = (size_t)m * p.n_out + col;
              if (p.residual != nullptr) r += __bfloat162float(p.residual[o]);
              if (p.out_f32)
                reinterpret_cast<float*>(p.out)[o] = r;
              else
                reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(r);
            }
          }
        }
        ls_bar_sync_consumers();  // the partial sums are read: the next pass may overwrite them
      }
    }
  }
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) {
    // a wait ran out: copies may still be on their way into the ring; wait (bounded) for the last phase of
    // every stage before the block gives its shared memory back
    const int issued = total_it;
    for (int s = 0; s < p.stages; ++s) {
      int last = -1;
      for (int it = s; it < issued; it += p.stages) last = it;
      if (last >= 0) mbar_wait(&full_bar[s], (last / p.stages) & 1);
    }
  }
}

static int g_ls_sms = 0;
static int g_ls_attr[3] = {0, 0, 0};
static int g_ls_blocks_per_sm = 1;  // blocks the launcher aims for per SM (1 leaves room for the next kernel's blocks)

extern "C" void ullm_linear_stream_blocks_per_sm(int n) { g_ls_blocks_per_sm = n < 1 ? 1 : (n > 2 ? 2 : n); }

extern "C" int ullm_linear_stream_supported(int M, int N, int K) {
  return M >= 1 && M <= 32 && N >= 1 && K >= 8 && K % 8 == 0;
}

template <int NT>
static int ls_launch(int which, const CUtensorMap& wm, const CUtensorMap& xm, LsParams p, cudaStream_t st) {
  constexpr int STAGE_BYTES = LS_W_STAGE_BYTES + 4 * 8 * NT * 128;
  const int red_bytes = LS_CONSUMER_WARPS * 32 * (NT > 1 ? 2 : 1) * 4 * (int)sizeof(float);
  int stages = (LS_MAX_SMEM - 1024 - red_bytes) / STAGE_BYTES;
  if (stages > 8) stages = 8;
  if (stages < 2) return ULLM_ERR_UNSUPPORTED;
  p.stages = stages;
  const size_t smem = (size_t)stages * STAGE_BYTES + red_bytes + 1024;
  if (!g_ls_attr[which]) {
    if (cudaFuncSetAttribute(linear_stream_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, LS_MAX_SMEM) !=
        cudaSuccess)
      return ULLM_ERR_LAUNCH;
    cudaFuncSetAttribute(linear_stream_kernel<NT>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    g_ls_attr[which] = 1;
  }
  int grid = g_ls_sms * g_ls_blocks_per_sm;
  if (grid > p.num_units) grid = p.num_units;
  return ullm_launch_kernel(linear_stream_kernel<NT>, dim3(grid), dim3(LS_THREADS), smem, st, wm, xm, p);
}

// act: 0 none, 1 silu gate, 2 gelu_tanh gate (weight = [gate rows; up rows], out [M, N / 2]).
// residual: null or [M, n_out] bfloat16, added to the product in 32-bit before the one rounding.
extern "C" int ullm_linear_stream(const void* x, const void* w, const void* bias, const void* residual, void* out,
                                  int M, int N, int K, int out_f32, int act, int* status, void* stream) {
  if (!ullm_linear_stream_supported(M, N, K)) return ULLM_ERR_UNSUPPORTED;
  if (act < 0 || act > 2 || (act && (N % 2))) return ULLM_ERR_BAD_SIZE;
  if (g_ls_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&g_ls_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || g_ls_sms <= 0)
      return ULLM_ERR_LAUNCH;
  }
  const int NT = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
  CUtensorMap wm, xm;
  // x as a matrix of exactly M rows: boxes of 8 NT rows read zeros past them
  if (!get_map(w, N, K, 16, &wm) || !get_map(x, M, K, 8 * NT, &xm)) return ULLM_ERR_LAUNCH;
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
  p.status = status;
  if (NT == 1) return ls_launch<1>(0, wm, xm, p, (cudaStream_t)stream);
  if (NT == 2) return ls_launch<2>(1, wm, xm, p, (cudaStream_t)stream);
  return ls_launch<4>(2, wm, xm, p, (cudaStream_t)stream);
}
