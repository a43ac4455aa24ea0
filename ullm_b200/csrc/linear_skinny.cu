// out[M, N] = x[M, K] . W[N, K]^T for very few rows (M <= 32: decode steps), bfloat16 in, 32-bit
// accumulate, bfloat16 or float32 out; optionally out[M, N/2] = act(gate) * up for a weight that
// stacks gate rows on up rows.
//
// With so few rows the product is a stream of the weight matrix through the chip: what counts is
// that every SM has enough 16-byte loads in flight from the first cycle on and that nothing is set
// up or torn down around them.  So this kernel uses no shared-memory ring and no tensor memory:
//
//   * A block owns 16 weight rows (16 gate + 16 up rows with an activation) and all of K.  Its 8
//     warps split K into contiguous ranges; a warp's partial sums meet in shared memory and are
//     added in warp order (deterministic), then bias and activation, then the store.
//   * Weight rows are the M side of mma.sync.m16n8k16 (bf16, f32 accumulate), the batch rows its N
//     side.  A thread loads 16 bytes (8 consecutive k) of weight row g and of row g + 8 and 16
//     bytes of batch row g at the same k: the four threads of a quad hold 32 consecutive k, and
//     the tensor instruction is fed the k positions in that (permuted) order for both operands,
//     which leaves the sum unchanged.  No shuffle, no shared-memory staging: global memory to
//     registers to the tensor core.
//   * The weights do not depend on the kernel before this one in the stream: with programmatic
//     dependent launch the first loads of weights are issued before griddepcontrol.wait.
#include "common.cuh"

#define SK_THREADS 256
#define SK_WARPS 8
#define SK_UNROLL 4   // chunks of 32 k in flight per thread and row

__device__ __forceinline__ uint4 sk_ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void sk_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct SkParams {
  const __nv_bfloat16* x;     // [M, K]
  const __nv_bfloat16* w;     // [N, K]
  const __nv_bfloat16* bias;  // [N] or null
  void* out;                  // [M, n_out]
  int M, N, K;
  int n_out;                  // N, or N / 2 with an activation
  int act;                    // 0 none, 1 silu(gate) * up, 2 gelu_tanh(gate) * up
  int out_f32;
};

// NT: tiles of 8 batch rows (M <= 8 NT).  RT: 16-row tiles of the weight per block (1, or 2 = gate + up).
template <int NT, int RT>
__global__ void __launch_bounds__(SK_THREADS) linear_skinny_kernel(const SkParams p) {
  __shared__ float red[SK_WARPS][RT * 16][NT * 8 + 1];
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int chunks = (p.K + 31) / 32;
  const int c_begin = (int)((long long)warp * chunks / SK_WARPS), c_end = (int)((long long)(warp + 1) * chunks / SK_WARPS);
  const int row0 = blockIdx.x * 16;

  // the 2 RT weight rows this thread reads (g and g + 8 of each row tile); rows beyond the matrix read as zero
  const __nv_bfloat16* wrow[RT * 2];
  bool wok[RT * 2];
#pragma unroll
  for (int r = 0; r < RT; ++r) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = row0 + g + 8 * h;
      const bool ok = row < p.n_out;
      const long long abs_row = (long long)(r == 0 ? 0 : p.n_out) + (ok ? row : 0);
      wrow[r * 2 + h] = p.w + abs_row * p.K + t * 8;
      wok[r * 2 + h] = ok;
    }
  }
  const __nv_bfloat16* xrow[NT];
  bool xok[NT];
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int m = n * 8 + g;
    xok[n] = m < p.M;
    xrow[n] = p.x + (long long)(xok[n] ? m : 0) * p.K + t * 8;
  }

  float acc[RT][NT][4];
#pragma unroll
  for (int r = 0; r < RT; ++r)
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[r][n][i] = 0.f;

  // Two sets of weight registers: while the tensor instructions work through one, the loads of the next
  // SK_UNROLL chunks are already in flight into the other.
  uint4 a0[SK_UNROLL][RT * 2], a1[SK_UNROLL][RT * 2];
  auto load_a = [&](uint4 (&a)[SK_UNROLL][RT * 2], int c) {
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u) {
      const int k = (c + u) * 32 + t * 8;
      const bool in = c + u < c_end && k < p.K;
#pragma unroll
      for (int q = 0; q < RT * 2; ++q)
        a[u][q] = in && wok[q] ? sk_ld_stream(wrow[q] + (long long)(c + u) * 32) : make_uint4(0, 0, 0, 0);
    }
  };
  auto consume = [&](const uint4 (&a)[SK_UNROLL][RT * 2], int c) {
    uint4 b[SK_UNROLL][NT];
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u) {
      const int k = (c + u) * 32 + t * 8;
      const bool in = c + u < c_end && k < p.K;
#pragma unroll
      for (int n = 0; n < NT; ++n)
        b[u][n] = in && xok[n] ? __ldg(reinterpret_cast<const uint4*>(xrow[n] + (long long)(c + u) * 32))
                               : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u) {
#pragma unroll
      for (int r = 0; r < RT; ++r) {
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          // the quad's 32 k as two instructions of 16: words x, y feed the first, z, w the second
          sk_mma(acc[r][n], a[u][r * 2].x, a[u][r * 2 + 1].x, a[u][r * 2].y, a[u][r * 2 + 1].y, b[u][n].x, b[u][n].y);
          sk_mma(acc[r][n], a[u][r * 2].z, a[u][r * 2 + 1].z, a[u][r * 2].w, a[u][r * 2 + 1].w, b[u][n].z, b[u][n].w);
        }
      }
    }
  };
  if (c_begin < c_end) load_a(a0, c_begin);
  pdl_wait();  // x is the output of the kernel before this one
  for (int c = c_begin; c < c_end; c += 2 * SK_UNROLL) {
    if (c + SK_UNROLL < c_end) load_a(a1, c + SK_UNROLL);
    consume(a0, c);
    if (c + SK_UNROLL >= c_end) break;
    if (c + 2 * SK_UNROLL < c_end) load_a(a0, c + 2 * SK_UNROLL);
    consume(a1, c + SK_UNROLL);
  }

  // partial sums of the 8 warps meet in shared memory: c0, c1 = [row g][cols 2t, 2t + 1], c2, c3 = [row g + 8][..]
#pragma unroll
  for (int r = 0; r < RT; ++r) {
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      red[warp][r * 16 + g][n * 8 + 2 * t] = acc[r][n][0];
      red[warp][r * 16 + g][n * 8 + 2 * t + 1] = acc[r][n][1];
      red[warp][r * 16 + g + 8][n * 8 + 2 * t] = acc[r][n][2];
      red[warp][r * 16 + g + 8][n * 8 + 2 * t + 1] = acc[r][n][3];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 16 * NT * 8; idx += SK_THREADS) {
    const int row = idx & 15, m = idx >> 4;  // consecutive threads: consecutive output columns
    const int col = row0 + row;
    if (m >= p.M || col >= p.n_out) continue;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < SK_WARPS; ++w) v += red[w][row][m];
    if (p.bias != nullptr) v += __bfloat162float(p.bias[col]);
    if (RT == 2) {
      float up = 0.f;
#pragma unroll
      for (int w = 0; w < SK_WARPS; ++w) up += red[w][16 + row][m];
      if (p.bias != nullptr) up += __bfloat162float(p.bias[p.n_out + col]);
      v = (p.act == 1 ? act_silu(v) : act_gelu_tanh(v)) * up;
    }
    if (p.out_f32) reinterpret_cast<float*>(p.out)[(long long)m * p.n_out + col] = v;
    else reinterpret_cast<__nv_bfloat16*>(p.out)[(long long)m * p.n_out + col] = __float2bfloat16_rn(v);
  }
}

// Shapes this kernel takes: 1 <= M <= 32, K a multiple of 8 (16-byte pieces of a row), 16-byte aligned bases;
// with an activation N is even.
extern "C" int ullm_linear_skinny_supported(int M, int N, int K) {
  return M >= 1 && M <= 32 && N >= 1 && K >= 8 && K % 8 == 0;
}

template <int NT>
static int sk_launch(const SkParams& p, cudaStream_t st) {
  const dim3 grid((p.n_out + 15) / 16), block(SK_THREADS);
  if (p.act != 0) return ullm_launch_kernel(linear_skinny_kernel<NT, 2>, grid, block, 0, st, p);
  return ullm_launch_kernel(linear_skinny_kernel<NT, 1>, grid, block, 0, st, p);
}

extern "C" int ullm_linear_skinny(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                                  int out_f32, int act, void* stream) {
  if (!ullm_linear_skinny_supported(M, N, K)) return ULLM_ERR_UNSUPPORTED;
  if (act < 0 || act > 2 || (act != 0 && N % 2 != 0)) return ULLM_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return ULLM_ERR_UNSUPPORTED;
  SkParams p;
  p.x = (const __nv_bfloat16*)x;
  p.w = (const __nv_bfloat16*)w;
  p.bias = (const __nv_bfloat16*)bias;
  p.out = out;
  p.M = M;
  p.N = N;
  p.K = K;
  p.act = act;
  p.n_out = act != 0 ? N / 2 : N;
  p.out_f32 = out_f32;
  cudaStream_t st = (cudaStream_t)stream;
  int rc;
  if (M <= 8) rc = sk_launch<1>(p, st);
  else if (M <= 16) rc = sk_launch<2>(p, st);
  else if (M <= 24) rc = sk_launch<3>(p, st);
  else rc = sk_launch<4>(p, st);
  if (rc != ULLM_OK) return rc;
  return ullm_launch_status();
}
