// Paged causal attention for bfloat16 batches that hold prompt portions (any
// mix of lengths, single decoded tokens included).  Flash-attention style:
// a block owns 128 rows of one kv head for one request, walks that request's
// keys in tiles of 64, and keeps an online softmax per row.  Products run on
// the tensor cores (mma.sync m16n8k16 bf16, fp32 accumulate); scores, maxima,
// sums and the output accumulator are 32-bit.
//
// Rows are (token, query head of the group) pairs: with G query heads per kv
// head a block covers 128 / G consecutive tokens, so one pass over K and V serves
// all heads that share them.  Row i of a block: token j0 + i / G, head kh * G +
// i % G, position start + j0 + i / G; it sees keys max(0, pos - window + 1) ..
// pos.  K and V tiles are gathered from the pages with cp.async into a two-stage
// ring shared by the block's four warps (16-byte chunks, XOR-swizzled by row);
// each warp owns 32 rows, so a K or V fragment read from shared memory feeds two
// 16-row tiles;
// keys beyond the block's last position are zero-filled, never read.  A warp
// skips a key tile that lies wholly above its rows' diagonal or wholly below
// their window.
#include "common.cuh"

#define PRE_WARPS 4
#define PRE_ROWS_PER_WARP 32
#define PRE_M (PRE_WARPS * PRE_ROWS_PER_WARP)
#define PRE_N 64

__device__ __forceinline__ void pre_cp_async_16(void* smem, const void* gmem, bool pred) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void pre_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void pre_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void pre_ldsm4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(s));
}
__device__ __forceinline__ void pre_ldsm4t(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(s));
}
__device__ __forceinline__ void pre_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x, one MUFU instruction; 2^(-inf) = 0
__device__ __forceinline__ float pre_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pre_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

template <int D>
struct PrefillSmem {
  static constexpr int ROW_BYTES = D * 2;
  static constexpr int Q_BYTES = PRE_M * ROW_BYTES;
  static constexpr int TILE_BYTES = PRE_N * ROW_BYTES;
  static constexpr int SLOT_BYTES = 2 * PRE_N * 8;
  static constexpr int BYTES = Q_BYTES + 2 * 2 * TILE_BYTES + SLOT_BYTES;
};

template <int D>
__global__ void __launch_bounds__(PRE_WARPS * 32, 2)
prefill_attention_kernel(const __nv_bfloat16* __restrict__ q, long long q_row_stride, __nv_bfloat16* __restrict__ out,
                         const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                         const int* __restrict__ block_table, int max_pages, const int* __restrict__ req_slots,
                         const int* __restrict__ cu_q, const int* __restrict__ kv_len, int num_requests, int num_q,
                         int num_kv, int page_size, int window, float scale_log2, long long num_pages, int* status) {
  extern __shared__ __align__(128) unsigned char smem[];
  pdl_launch_dependents();
  pdl_wait();
  constexpr int CHUNKS = D / 8, KSTEPS = D / 16, NT_O = D / 8, NT_S = PRE_N / 8;
  using S = PrefillSmem<D>;
  unsigned char* q_s = smem;
  unsigned char* kv_s = smem + S::Q_BYTES;
  long long* slot_s = reinterpret_cast<long long*>(smem + S::Q_BYTES + 4 * S::TILE_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // A 1-D grid, numbered so that consecutive blocks are the same token tile of all kv heads: the block
  // scheduler then starts the heaviest tiles of EVERY head first (longest work first keeps the SMs level).
  const int kh = (int)(blockIdx.x % num_kv);
  const int G = num_q / num_kv;
  const int tpt = PRE_M / G;  // tokens per block

  // ---- which request and which of its token tiles is this block? --------------------
  // Blocks are numbered from the back: the last tiles of a prompt see the most keys and start first.
  const int tile_id = (int)(gridDim.x / num_kv) - 1 - (int)(blockIdx.x / num_kv);
  int r = -1, first = 0, q_len = 0, q_begin = 0;
  {
    int running = 0;
    for (int i = 0; i < num_requests; ++i) {
      const int b = cu_q[i], n = cu_q[i + 1] - b;
      const int nt = (n + tpt - 1) / tpt;
      if (tile_id < running + nt) {
        r = i;
        first = (tile_id - running) * tpt;
        q_len = n;
        q_begin = b;
        break;
      }
      running += nt;
    }
  }
  if (r < 0) return;
  const int kvl = kv_len[r];
  const int ntok = min(tpt, q_len - first);
  const int rows_valid = ntok * G;
  const int start = kvl - q_len;                     // position of the portion's first token
  const int p0 = start + first, p1 = p0 + ntok - 1;  // positions of this block's tokens
  if (kvl <= 0 || p0 < 0) {                          // padding request: zeros
    for (int i = tid; i < rows_valid * D; i += blockDim.x) {
      const int row = i / D, d = i - row * D;
      out[((long long)(q_begin + first + row / G) * num_q + kh * G + row % G) * D + d] = __float2bfloat16_rn(0.f);
    }
    return;
  }
  const int key0 = window > 0 ? max(0, p0 - window + 1) : 0;
  const int tiles = (p1 - key0 + PRE_N) / PRE_N;
  const int* bt = block_table + (long long)req_slots[r] * max_pages;
  const long long kv_row = (long long)num_kv * D;

  // ---- Q tile -------------------------------------------------------------------------
  for (int c = tid; c < PRE_M * CHUNKS; c += blockDim.x) {
    const int row = c / CHUNKS, ch = c % CHUNKS;
    const bool ok = row < rows_valid;
    const long long off =
        ok ? ((long long)(q_begin + first + row / G) * q_row_stride + (long long)(kh * G + row % G) * D + ch * 8) : 0;
    pre_cp_async_16(q_s + row * S::ROW_BYTES + ((ch ^ (row & 7)) * 16), q + off, ok);
  }
  pre_commit();

  auto issue = [&](int tile) {
    const int st = tile & 1;
    unsigned char* kbuf = kv_s + st * 2 * S::TILE_BYTES;
    unsigned char* vbuf = kbuf + S::TILE_BYTES;
    long long* slots = slot_s + st * PRE_N;
    if (tid < PRE_N) {
      const int key = key0 + tile * PRE_N + tid;
      long long s = -1;
      if (key <= p1) {
        const int page = bt[key / page_size];
        if (page < 0 || page >= num_pages) ullm_report(status, ULLM_STATUS_PAGE, r, page);
        else s = (long long)page * page_size + key % page_size;
      }
      slots[tid] = s;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < PRE_N * CHUNKS / (PRE_WARPS * 32); ++i) {
      const int c = i * PRE_WARPS * 32 + tid;
      const int row = c / CHUNKS, ch = c % CHUNKS;
      const long long s = slots[row];
      const bool ok = s >= 0;
      const long long off = ok ? (s * kv_row + (long long)kh * D + ch * 8) : 0;
      const int sw = row * S::ROW_BYTES + ((ch ^ (row & 7)) * 16);
      pre_cp_async_16(kbuf + sw, k_cache + off, ok);
      pre_cp_async_16(vbuf + sw, v_cache + off, ok);
    }
  };

  // A warp owns 32 rows, two 16-row tiles; a thread's rows in tile mt: base + lane / 4 and + 8.
  // K and V fragments are loaded once per warp and used for both tiles.
  const int wrow = warp * PRE_ROWS_PER_WARP;
  int pos[2][2], lo[2][2];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = wrow + mt * 16 + (lane >> 2) + h * 8;
      pos[mt][h] = row < rows_valid ? p0 + row / G : -1;
      lo[mt][h] = window > 0 ? pos[mt][h] - window + 1 : 0;
    }
  const int w_last = min(rows_valid, wrow + PRE_ROWS_PER_WARP) - 1;
  const bool warp_live = wrow < rows_valid;
  const int wp_max = warp_live ? p0 + w_last / G : -1;
  const int wp_lo = (warp_live && window > 0) ? p0 + wrow / G - window + 1 : 0;
  const int wp_min = p0 + wrow / G;                               // position of the warp's first row
  const bool warp_full = wrow + PRE_ROWS_PER_WARP <= rows_valid;  // no padding rows in this warp

  float m[2][2], l[2][2];
  float o[2][NT_O][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt) {
    m[mt][0] = m[mt][1] = -INFINITY;
    l[mt][0] = l[mt][1] = 0.f;
#pragma unroll
    for (int j = 0; j < NT_O; ++j) o[mt][j][0] = o[mt][j][1] = o[mt][j][2] = o[mt][j][3] = 0.f;
  }

  issue(0);
  pre_commit();
  for (int it = 0; it < tiles; ++it) {
    if (it + 1 < tiles) issue(it + 1);
    pre_commit();
    pre_wait<1>();
    __syncthreads();
    const int kb = key0 + it * PRE_N;
    if (warp_live && kb <= wp_max && kb + PRE_N - 1 >= wp_lo) {
      const unsigned char* kbuf = kv_s + (it & 1) * 2 * S::TILE_BYTES;
      const unsigned char* vbuf = kbuf + S::TILE_BYTES;
      float sc[2][NT_S][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int t = 0; t < NT_S; ++t) sc[mt][t][0] = sc[mt][t][1] = sc[mt][t][2] = sc[mt][t][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        unsigned qa[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          const int mat = lane >> 3, row = wrow + mt * 16 + (mat & 1) * 8 + (lane & 7), ch = 2 * kk + (mat >> 1);
          pre_ldsm4(qa[mt][0], qa[mt][1], qa[mt][2], qa[mt][3], q_s + row * S::ROW_BYTES + ((ch ^ (row & 7)) * 16));
        }
#pragma unroll
        for (int t = 0; t < NT_S; t += 2) {
          const int mat = lane >> 3, row = t * 8 + (mat >> 1) * 8 + (lane & 7), ch = 2 * kk + (mat & 1);
          unsigned b0, b1, b2, b3;
          pre_ldsm4(b0, b1, b2, b3, kbuf + row * S::ROW_BYTES + ((ch ^ (row & 7)) * 16));
          pre_mma(sc[0][t], qa[0], b0, b1);
          pre_mma(sc[0][t + 1], qa[0], b2, b3);
          pre_mma(sc[1][t], qa[1], b0, b1);
          pre_mma(sc[1][t + 1], qa[1], b2, b3);
        }
      }
      // ---- mask and online softmax -----------------------------------------------------
      // Scores stay raw (unscaled) until the exponential: p = 2^(s * scale_log2 - m), one fused
      // multiply-add and one ex2 per element; m is kept in scaled units.  Only tiles that touch the
      // diagonal, a window's edge or padding rows run the mask.
      const bool need_mask = !warp_full || kb + PRE_N - 1 > wp_min || (window > 0 && kb < wp_max - window + 1);
      float alpha[2][2];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        if (need_mask) {
#pragma unroll
          for (int t = 0; t < NT_S; ++t) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int key = kb + t * 8 + (lane & 3) * 2 + (e & 1);
              if (!(key <= pos[mt][e >> 1] && key >= lo[mt][e >> 1])) sc[mt][t][e] = -INFINITY;
            }
          }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int t = 0; t < NT_S; ++t) {
          mx[0] = fmaxf(mx[0], fmaxf(sc[mt][t][0], sc[mt][t][1]));
          mx[1] = fmaxf(mx[1], fmaxf(sc[mt][t][2], sc[mt][t][3]));
        }
        float neg_m[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
          mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
          const float m_new = fmaxf(m[mt][i], mx[i] * scale_log2);
          const float m_use = m_new == -INFINITY ? 0.f : m_new;  // a row that has seen no key yet
          alpha[mt][i] = pre_ex2(m[mt][i] - m_use);
          m[mt][i] = m_new;
          l[mt][i] *= alpha[mt][i];
          neg_m[i] = -m_use;
        }
#pragma unroll
        for (int t = 0; t < NT_S; ++t) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float p = pre_ex2(fmaf(sc[mt][t][e], scale_log2, neg_m[e >> 1]));
            sc[mt][t][e] = p;
            l[mt][e >> 1] += p;
          }
        }
#pragma unroll
        for (int j = 0; j < NT_O; ++j) {
          o[mt][j][0] *= alpha[mt][0];
          o[mt][j][1] *= alpha[mt][0];
          o[mt][j][2] *= alpha[mt][1];
          o[mt][j][3] *= alpha[mt][1];
        }
      }
      // ---- O += P V ---------------------------------------------------------------------
#pragma unroll
      for (int ks = 0; ks < PRE_N / 16; ++ks) {
        unsigned pa[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          pa[mt][0] = pre_pack(sc[mt][2 * ks][0], sc[mt][2 * ks][1]);
          pa[mt][1] = pre_pack(sc[mt][2 * ks][2], sc[mt][2 * ks][3]);
          pa[mt][2] = pre_pack(sc[mt][2 * ks + 1][0], sc[mt][2 * ks + 1][1]);
          pa[mt][3] = pre_pack(sc[mt][2 * ks + 1][2], sc[mt][2 * ks + 1][3]);
        }
#pragma unroll
        for (int j = 0; j < NT_O; j += 2) {
          const int mat = lane >> 3, row = ks * 16 + (mat & 1) * 8 + (lane & 7), ch = j + (mat >> 1);
          unsigned b0, b1, b2, b3;
          pre_ldsm4t(b0, b1, b2, b3, vbuf + row * S::ROW_BYTES + ((ch ^ (row & 7)) * 16));
          pre_mma(o[0][j], pa[0], b0, b1);
          pre_mma(o[0][j + 1], pa[0], b2, b3);
          pre_mma(o[1][j], pa[1], b0, b1);
          pre_mma(o[1][j + 1], pa[1], b2, b3);
        }
      }
    }
    __syncthreads();
  }
  pre_wait<0>();
  const int c = (lane & 3) * 2;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float ls = l[mt][h];
      ls += __shfl_xor_sync(0xffffffffu, ls, 1);
      ls += __shfl_xor_sync(0xffffffffu, ls, 2);
      const float inv = ls > 0.f ? 1.f / ls : 0.f;
      const int row = wrow + mt * 16 + (lane >> 2) + h * 8;
      if (row < rows_valid) {
        __nv_bfloat16* op = out + ((long long)(q_begin + first + row / G) * num_q + kh * G + row % G) * D;
#pragma unroll
        for (int j = 0; j < NT_O; ++j)
          *reinterpret_cast<unsigned*>(op + j * 8 + c) = pre_pack(o[mt][j][2 * h] * inv, o[mt][j][2 * h + 1] * inv);
      }
    }
  }
}

static int g_prefill_attr_set[2] = {0, 0};

template <int D>
static int launch_prefill(int which, const void* q, long long q_row_stride, void* out, const void* k_cache,
                          const void* v_cache, const int* block_table, int max_pages, const int* req_slots,
                          const int* cu_q, const int* kv_len, int tokens, int num_requests, int num_q, int num_kv,
                          int page_size, int window, float scale, long long num_pages, int* status, cudaStream_t st) {
  using S = PrefillSmem<D>;
  if (!g_prefill_attr_set[which]) {
    if (cudaFuncSetAttribute(prefill_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::BYTES) !=
        cudaSuccess)
      return ULLM_ERR_LAUNCH;
    cudaFuncSetAttribute(prefill_attention_kernel<D>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    g_prefill_attr_set[which] = 1;
  }
  const int tpt = PRE_M / (num_q / num_kv);
  // at most ceil(tokens / tpt) + num_requests token tiles exist, however the tokens are spread
  dim3 grid(((tokens + tpt - 1) / tpt + num_requests) * num_kv);
  return ullm_launch_kernel(prefill_attention_kernel<D>, grid, dim3(PRE_WARPS * 32), (size_t)S::BYTES, st,
      (const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_cache,
      (const __nv_bfloat16*)v_cache, block_table, max_pages, req_slots, cu_q, kv_len, num_requests, num_q, num_kv,
      page_size, window, scale * 1.4426950408889634f, num_pages, status);
  return ullm_launch_status();
}

// Sizes this kernel takes: bfloat16, head_dim 64 or 128, at most 32 query heads per kv head.
extern "C" int ullm_prefill_attention_supported(int head_dim, int num_q, int num_kv) {
  if (num_kv <= 0 || num_q % num_kv) return 0;
  return (head_dim == 64 || head_dim == 128) && (num_q / num_kv) <= 32;
}

extern "C" int ullm_prefill_attention(const void* q, long long q_row_stride, void* out, const void* k_cache,
                                      const void* v_cache, const int* block_table, int max_pages, const int* req_slots,
                                      const int* cu_q, const int* kv_len, int tokens, int num_requests, int num_q,
                                      int num_kv, int head_dim, int page_size, int window, float scale,
                                      long long num_pages, int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || num_requests <= 0 || num_q <= 0 || num_kv <= 0 || page_size <= 0 || max_pages <= 0 || window < 0)
    return ULLM_ERR_BAD_SIZE;
  if (!ullm_prefill_attention_supported(head_dim, num_q, num_kv)) return ULLM_ERR_UNSUPPORTED;
  if (tokens == 0) return ULLM_OK;
  if (head_dim == 64)
    return launch_prefill<64>(0, q, q_row_stride, out, k_cache, v_cache, block_table, max_pages, req_slots, cu_q, kv_len,
                              tokens, num_requests, num_q, num_kv, page_size, window, scale, num_pages, status, st);
  return launch_prefill<128>(1, q, q_row_stride, out, k_cache, v_cache, block_table, max_pages, req_slots, cu_q, kv_len,
                             tokens, num_requests, num_q, num_kv, page_size, window, scale, num_pages, status, st);
}
