// Next-token choice from 32-bit logits: argmax, or temperature / top-k /
// top-p / min-p filtering followed by one categorical draw.  One block per row.
//
// Filter semantics are those of ullm/layers/sampler.py:39-52 and :59-107
// (temperature, then top-k, then top-p on what top-k left, then min-p), without
// its full sort of the vocabulary:
//   top-k  keeps values >= the k-th largest (ties at the threshold kept)
//          -> radix select of the k-th largest on order-preserving keys;
//   top-p  drops, in ascending order, every entry whose inclusive running mass
//          is <= 1 - p (equal values stand or fall together)
//          -> radix select on the mass below a key;
//   min-p  drops entries whose probability is below min_p * the largest one
//          -> exp(x - max) < min_p.
// Masses are accumulated as 64-bit fixed point (2^40 per unit of exp(x - max)),
// so every sum is an integer sum: the result does not depend on the order in
// which threads add, and the same row gives the same token in any batch.
// The draw takes the caller's uniform number u in [0, 1) and returns the first
// index whose inclusive running mass exceeds u * total.
// temperature == 0 means argmax (lowest index among equal maxima).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

#define SAMPLE_THREADS 1024
#define FIX_ONE 1099511627776.0f  // 2^40

__device__ __forceinline__ unsigned int order_key(float x) {
  const unsigned int b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned long long mass_of(float x, float mx) {
  return (unsigned long long)(expf(x - mx) * FIX_ONE);
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ ArgMax block_argmax(const float* __restrict__ row, int n, float inv_t, ArgMax* sh) {
  ArgMax best = {-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    ArgMax c = {row[i] * inv_t, i};
    best = better(best, c);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax c = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, c);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = best;
  __syncthreads();
  if (warp == 0) {
    ArgMax c = lane < nw ? sh[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax d = {__shfl_xor_sync(0xffffffffu, c.v, o), __shfl_xor_sync(0xffffffffu, c.i, o)};
      c = better(c, d);
    }
    if (lane == 0) sh[32] = c;
  }
  __syncthreads();
  return sh[32];
}

__device__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  if (warp == 0) {
    unsigned long long t = lane < nw ? sh[lane] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) sh[32] = t;
  }
  __syncthreads();
  return sh[32];
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ uniform, int* __restrict__ out, float* __restrict__ probs_out,
              const int* __restrict__ row_slots, int* __restrict__ last_tokens) {
  __shared__ ArgMax sh_arg[33];
  __shared__ unsigned long long sh_u64[33];
  __shared__ unsigned long long hist_mass[256];
  __shared__ int hist_cnt[256];
  __shared__ unsigned int sh_prefix;
  __shared__ unsigned long long sh_below;
  __shared__ int sh_remaining;
  __shared__ int sh_result;

  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const float* row = logits + (long long)r * row_stride;
  const float temp = temperature != nullptr ? temperature[r] : 0.f;
  float* pout = probs_out != nullptr ? probs_out + (long long)r * vocab : nullptr;

  if (!(temp > 0.f)) {  // greedy
    const ArgMax a = block_argmax(row, vocab, 1.f, sh_arg);
    if (threadIdx.x == 0) {
      out[r] = a.i;
      // the request's newest token stays findable on the device for a step launched before the host reads it
      if (row_slots != nullptr && last_tokens != nullptr && row_slots[r] >= 0) last_tokens[row_slots[r]] = a.i;
    }
    if (pout != nullptr)
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) pout[i] = i == a.i ? 1.f : 0.f;
    return;
  }
  const float inv_t = 1.f / temp;
  const ArgMax top = block_argmax(row, vocab, inv_t, sh_arg);
  const float mx = top.v;

  // ---- top-k: key of the k-th largest value --------------------------------
  int k = top_k != nullptr ? top_k[r] : 0;
  if (k <= 0 || k > vocab) k = vocab;
  unsigned int key_floor = 0u;  // keep keys >= key_floor
  if (k < vocab) {
    if (threadIdx.x == 0) {
      sh_prefix = 0u;
      sh_remaining = k;
    }
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      for (int b = threadIdx.x; b < 256; b += blockDim.x) hist_cnt[b] = 0;
      __syncthreads();
      const unsigned int prefix = sh_prefix;
      const unsigned int mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const unsigned int key = order_key(row[i] * inv_t);
        if ((key & mask) == prefix) atomicAdd(&hist_cnt[(key >> shift) & 255u], 1);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        int remaining = sh_remaining, above = 0, d = 255;
        for (; d > 0; --d) {
          if (above + hist_cnt[d] >= remaining) break;
          above += hist_cnt[d];
        }
        sh_remaining = remaining - above;
        sh_prefix = prefix | ((unsigned int)d << shift);
      }
      __syncthreads();
    }
    key_floor = sh_prefix;
  }

  // ---- top-p: smallest key whose inclusive mass from below exceeds (1-p) Z --
  float p = top_p != nullptr ? top_p[r] : 1.f;
  if (!(p > 0.f)) p = 1.f;
  if (p < 1.f) {
    unsigned long long local = 0ull;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float x = row[i] * inv_t;
      if (order_key(x) >= key_floor) local += mass_of(x, mx);
    }
    const unsigned long long z = block_sum_u64(local, sh_u64);
    const unsigned long long limit = (unsigned long long)((1.0 - (double)p) * (double)z);
    if (threadIdx.x == 0) {
      sh_prefix = 0u;
      sh_below = 0ull;
    }
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      for (int b = threadIdx.x; b < 256; b += blockDim.x) hist_mass[b] = 0ull;
      __syncthreads();
      const unsigned int prefix = sh_prefix;
      const unsigned int mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float x = row[i] * inv_t;
        const unsigned int key = order_key(x);
        if (key >= key_floor && (key & mask) == prefix) atomicAdd(&hist_mass[(key >> shift) & 255u], mass_of(x, mx));
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        unsigned long long below = sh_below;
        int d = 0;
        for (; d < 255; ++d) {
          if (below + hist_mass[d] > limit) break;
          below += hist_mass[d];
        }
        sh_below = below;
        sh_prefix = prefix | ((unsigned int)d << shift);
      }
      __syncthreads();
    }
    key_floor = max(key_floor, sh_prefix);
  }

  // ---- min-p, total mass, draw ----------------------------------------------
  float mp = min_p != nullptr ? min_p[r] : 0.f;
  if (!(mp > 0.f)) mp = 0.f;
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int begin = min(vocab, (int)threadIdx.x * chunk), end = min(vocab, begin + chunk);
  unsigned long long local = 0ull;
  for (int i = begin; i < end; ++i) {
    const float x = row[i] * inv_t;
    if (order_key(x) >= key_floor && expf(x - mx) >= mp) local += mass_of(x, mx);
  }
  // inclusive scan over threads
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned long long incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long nb = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += nb;
  }
  __syncthreads();
  if (lane == 31) sh_u64[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    unsigned long long w = lane < (int)(blockDim.x >> 5) ? sh_u64[lane] : 0ull;
    unsigned long long wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long nb = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += nb;
    }
    sh_u64[lane] = wi - w;  // exclusive offset of each warp
    if (lane == 31) sh_u64[32] = wi;
  }
  __syncthreads();
  const unsigned long long total = sh_u64[32];
  const unsigned long long excl = sh_u64[warp] + incl - local;
  const float u = uniform != nullptr ? uniform[r] : 0.f;
  unsigned long long target = (unsigned long long)((double)u * (double)total);
  if (total > 0ull && target >= total) target = total - 1ull;
  if (threadIdx.x == 0) sh_result = -1;
  __syncthreads();
  if (local > 0ull && target >= excl && target < excl + local) {
    unsigned long long run = excl;
    int pick = begin;
    for (int i = begin; i < end; ++i) {
      const float x = row[i] * inv_t;
      if (order_key(x) >= key_floor && expf(x - mx) >= mp) {
        run += mass_of(x, mx);
        pick = i;
        if (run > target) break;
      }
    }
    sh_result = pick;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int res = sh_result;
    if (res < 0) res = top.i;  // cannot happen: the maximum always has mass 2^40
    out[r] = res;
    if (row_slots != nullptr && last_tokens != nullptr && row_slots[r] >= 0) last_tokens[row_slots[r]] = res;
  }
  if (pout != nullptr) {
    const float inv = total > 0ull ? 1.f / (float)total : 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float x = row[i] * inv_t;
      const bool keep = order_key(x) >= key_floor && expf(x - mx) >= mp;
      pout[i] = keep ? (float)mass_of(x, mx) * inv : 0.f;
    }
  }
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, long long row_stride, int vocab, int* __restrict__ out) {
  __shared__ ArgMax sh_arg[33];
  pdl_launch_dependents();
  pdl_wait();
  const ArgMax a = block_argmax(logits + (long long)blockIdx.x * row_stride, vocab, 1.f, sh_arg);
  if (threadIdx.x == 0) out[blockIdx.x] = a.i;
}

extern "C" int ullm_argmax(const float* logits, long long row_stride, int rows, int vocab, int* out, void* stream) {
  if (rows < 0 || vocab <= 0) return ULLM_ERR_BAD_SIZE;
  if (rows == 0) return ULLM_OK;
  return ullm_launch_kernel(argmax_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, logits, row_stride,
                            vocab, out);
}

// ---------------------------------------------------------------------------------------------
// The same choice with a row spread over a cluster of blocks.
//
// One block per row streams the row's 600 KB (a 150k vocabulary) through a single SM once per pass, and there
// are up to ten passes.  Here a cluster of SC_CLUSTER blocks shares a row: each block loads its slice ONCE into
// shared memory (already divided by the temperature) and every later pass runs over shared memory; what the
// blocks have to agree on (maximum, histogram of a radix digit, sums of mass) is exchanged through distributed
// shared memory, each block reading its peers' small arrays after a cluster barrier.  All sums are integer
// sums, so every block arrives at the same digit and the same token as the one-block kernel above: bit for bit.
// The cluster barrier is the hardware's (barrier.cluster): no block spins on a flag.
// ---------------------------------------------------------------------------------------------
#define SC_THREADS 512
#define SC_WARPS (SC_THREADS / 32)
#define SC_CLUSTER 8
#define SC_UNROLL 5
#define SC_HISTS 8   // private histograms of a block (two warps share one): fewer collisions of the atomics

struct ScShared {
  ArgMax arg_w[SC_WARPS];
  ArgMax arg_cta;                          // read by the peers
  unsigned long long sum_w[SC_WARPS];
  unsigned long long sum_cta[2];           // read by the peers (two uses in a row: total mass, draw)
  int cnt_cta[2][256];                     // this block's digit histogram, by pass parity; read by the peers
  unsigned long long mass_cta[2][256];
  int cnt_tot[256];                        // the cluster's
  unsigned long long mass_tot[256];
  unsigned int prefix;
  int remaining;
  unsigned long long below;
  int result;
};

__device__ __forceinline__ ArgMax sc_block_argmax(ArgMax best, ScShared& sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax c = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, c);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sh.arg_w[warp] = best;
  __syncthreads();
  if (warp == 0) {
    ArgMax c = lane < SC_WARPS ? sh.arg_w[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax d = {__shfl_xor_sync(0xffffffffu, c.v, o), __shfl_xor_sync(0xffffffffu, c.i, o)};
      c = better(c, d);
    }
    if (lane == 0) sh.arg_cta = c;
  }
  __syncthreads();
  return sh.arg_cta;
}

// this block's sum into sh.sum_cta[slot]
__device__ __forceinline__ void sc_block_sum(unsigned long long v, ScShared& sh, int slot) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) sh.sum_w[warp] = v;
  __syncthreads();
  if (warp == 0) {
    unsigned long long t = lane < SC_WARPS ? sh.sum_w[lane] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) sh.sum_cta[slot] = t;
  }
  __syncthreads();
}

// Warp 0 finds, from the top (DESC) or from the bottom, the digit at which the running sum of `tot` first
// reaches (DESC: above + tot[d] >= want) or exceeds (ASC: below + tot[d] > limit) the bound; returns the digit and
// the sum before it.  All lanes of warp 0 take part; the result is valid in every lane of warp 0.
template <bool DESC, typename T>
__device__ __forceinline__ int sc_find_digit(const T* tot, T bound, T start, T* before) {
  const int lane = threadIdx.x & 31;
  // lane l owns the 8 digits of its group: DESC 255 - 8 l - j, ASC 8 l + j  (j = 0..7), in scan order
  T part = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) part += tot[DESC ? 255 - 8 * lane - j : 8 * lane + j];
  T incl = part;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const T nb = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += nb;
  }
  const T excl = start + incl - part;
  // the first lane whose group crosses the bound
  const bool crosses = DESC ? (excl + part >= bound) : (excl + part > bound);
  const unsigned m = __ballot_sync(0xffffffffu, crosses);
  const int owner = m ? __ffs(m) - 1 : 31;
  int digit = DESC ? 0 : 255;
  T bef = excl;
  if (lane == owner) {
    T run = excl;
    int j = 0;
    for (; j < 8; ++j) {
      const int d = DESC ? 255 - 8 * lane - j : 8 * lane + j;
      const T t = tot[d];
      // the scan stops at the last digit (0 from the top, 255 from the bottom) whatever it holds
      if ((DESC ? run + t >= bound : run + t > bound) || d == (DESC ? 0 : 255)) {
        digit = d;
        break;
      }
      run += t;
    }
    if (j == 8) digit = DESC ? 255 - 8 * lane - 7 : 8 * lane + 7, run -= tot[digit];
    bef = run;
  }
  digit = __shfl_sync(0xffffffffu, digit, owner);
  bef = __shfl_sync(0xffffffffu, bef, owner);
  *before = bef;
  return digit;
}

__global__ void __launch_bounds__(SC_THREADS)
sample_cluster_kernel(const float* __restrict__ logits, long long row_stride, int vocab, int slice,
                      const float* __restrict__ temperature, const int* __restrict__ top_k,
                      const float* __restrict__ top_p, const float* __restrict__ min_p,
                      const float* __restrict__ uniform, int* __restrict__ out, float* __restrict__ probs_out,
                      const int* __restrict__ row_slots, int* __restrict__ last_tokens) {
  extern __shared__ __align__(16) unsigned char sc_raw[];
  __shared__ ScShared sh;
  pdl_launch_dependents();
  pdl_wait();
  cg::cluster_group cluster = cg::this_cluster();
  const int C = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  const int r = blockIdx.x / C;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* vals = reinterpret_cast<float*>(sc_raw);                                    // [slice]
  // [SC_HISTS][256] counts, later [SC_HISTS][256] masses in the same memory
  int* cnt_w = reinterpret_cast<int*>(sc_raw + (size_t)slice * 4);
  unsigned long long* mass_w = reinterpret_cast<unsigned long long*>(sc_raw + (size_t)slice * 4);
  const int hist = warp % SC_HISTS;
  const float* row = logits + (long long)r * row_stride;
  const float temp = temperature != nullptr ? temperature[r] : 0.f;
  const bool greedy = !(temp > 0.f);
  const float inv_t = greedy ? 1.f : 1.f / temp;
  float* pout = probs_out != nullptr ? probs_out + (long long)r * vocab : nullptr;
  const int begin = min(vocab, rank * slice), n = min(vocab - begin, slice);

  // ---- the slice, once: scaled values into shared memory (not for a greedy row, which reads them only here),
  // this block's maximum.  SC_UNROLL loads are issued before the first is used.
  ArgMax best = {-INFINITY, 0x7fffffff};
  if ((((uintptr_t)(row + begin)) & 15) == 0) {
    const float4* src = reinterpret_cast<const float4*>(row + begin);
    const int n4 = n / 4;
    for (int i0 = tid; i0 < n4; i0 += SC_UNROLL * SC_THREADS) {
      float4 v[SC_UNROLL];
#pragma unroll
      for (int u = 0; u < SC_UNROLL; ++u) {
        const int i = i0 + u * SC_THREADS;
        v[u] = i < n4 ? __ldg(src + i) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
#pragma unroll
      for (int u = 0; u < SC_UNROLL; ++u) {
        const int i = i0 + u * SC_THREADS;
        if (i >= n4) break;
        v[u].x *= inv_t, v[u].y *= inv_t, v[u].z *= inv_t, v[u].w *= inv_t;
        if (!greedy) *reinterpret_cast<float4*>(vals + 4 * i) = v[u];
        best = better(best, ArgMax{v[u].x, begin + 4 * i});
        best = better(best, ArgMax{v[u].y, begin + 4 * i + 1});
        best = better(best, ArgMax{v[u].z, begin + 4 * i + 2});
        best = better(best, ArgMax{v[u].w, begin + 4 * i + 3});
      }
    }
    for (int i = n4 * 4 + tid; i < n; i += SC_THREADS) {
      const float v = row[begin + i] * inv_t;
      if (!greedy) vals[i] = v;
      best = better(best, ArgMax{v, begin + i});
    }
  } else {
    for (int i0 = tid; i0 < n; i0 += SC_UNROLL * SC_THREADS) {
      float v[SC_UNROLL];
#pragma unroll
      for (int u = 0; u < SC_UNROLL; ++u) {
        const int i = i0 + u * SC_THREADS;
        v[u] = i < n ? __ldg(row + begin + i) : -INFINITY;
      }
#pragma unroll
      for (int u = 0; u < SC_UNROLL; ++u) {
        const int i = i0 + u * SC_THREADS;
        if (i >= n) break;
        v[u] *= inv_t;
        if (!greedy) vals[i] = v[u];
        best = better(best, ArgMax{v[u], begin + i});
      }
    }
  }
  sc_block_argmax(best, sh);
  cluster.sync();
  ArgMax top = {-INFINITY, 0x7fffffff};
  for (int c = 0; c < C; ++c) top = better(top, cluster.map_shared_rank(&sh, c)->arg_cta);
  const float mx = top.v;

  if (greedy) {
    if (rank == 0 && tid == 0) {
      out[r] = top.i;
      // the request's newest token stays findable on the device for a step launched before the host reads it
      if (row_slots != nullptr && last_tokens != nullptr && row_slots[r] >= 0) last_tokens[row_slots[r]] = top.i;
    }
    if (pout != nullptr)
      for (int i = tid; i < n; i += SC_THREADS) pout[begin + i] = begin + i == top.i ? 1.f : 0.f;
    cluster.sync();  // no block leaves while a peer may still read its shared memory
    return;
  }

  int pass_no = 0;  // parity of the published histograms
  // ---- top-k: key of the k-th largest value ---------------------------------------------------------------
  int k = top_k != nullptr ? top_k[r] : 0;
  if (k <= 0 || k > vocab) k = vocab;
  unsigned int key_floor = 0u;  // keep keys >= key_floor
  if (k < vocab) {
    unsigned int prefix = 0u;
    int remaining = k;
    for (int pass = 0; pass < 4; ++pass, ++pass_no) {
      const int shift = 24 - 8 * pass;
      const unsigned int mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int b = tid; b < SC_HISTS * 256; b += SC_THREADS) cnt_w[b] = 0;
      __syncthreads();
      for (int i = tid; i < n; i += SC_THREADS) {
        const unsigned int key = order_key(vals[i]);
        if ((key & mask) == prefix) atomicAdd(&cnt_w[hist * 256 + ((key >> shift) & 255u)], 1);
      }
      __syncthreads();
      if (tid < 256) {
        int t = 0;
#pragma unroll
        for (int w = 0; w < SC_HISTS; ++w) t += cnt_w[w * 256 + tid];
        sh.cnt_cta[pass_no & 1][tid] = t;
      }
      cluster.sync();
      if (tid < 256) {
        int t = 0;
        for (int c = 0; c < C; ++c) t += cluster.map_shared_rank(&sh, c)->cnt_cta[pass_no & 1][tid];
        sh.cnt_tot[tid] = t;
      }
      __syncthreads();
      if (warp == 0) {
        int above;
        const int d = sc_find_digit<true, int>(sh.cnt_tot, remaining, 0, &above);
        if (lane == 0) {
          sh.remaining = remaining - above;
          sh.prefix = prefix | ((unsigned int)d << shift);
        }
      }
      __syncthreads();
      remaining = sh.remaining;
      prefix = sh.prefix;
    }
    key_floor = prefix;
  }

  // ---- top-p: smallest key whose inclusive mass from below exceeds (1-p) Z -----------------------------------
  float p = top_p != nullptr ? top_p[r] : 1.f;
  if (!(p > 0.f)) p = 1.f;
  if (p < 1.f) {
    unsigned long long local = 0ull;
    for (int i = tid; i < n; i += SC_THREADS) {
      const float x = vals[i];
      if (order_key(x) >= key_floor) local += mass_of(x, mx);
    }
    sc_block_sum(local, sh, 0);
    cluster.sync();
    unsigned long long z = 0ull;
    for (int c = 0; c < C; ++c) z += cluster.map_shared_rank(&sh, c)->sum_cta[0];
    const unsigned long long limit = (unsigned long long)((1.0 - (double)p) * (double)z);
    unsigned int prefix = 0u;
    unsigned long long below = 0ull;
    for (int pass = 0; pass < 4; ++pass, ++pass_no) {
      const int shift = 24 - 8 * pass;
      const unsigned int mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int b = tid; b < SC_HISTS * 256; b += SC_THREADS) mass_w[b] = 0ull;
      __syncthreads();
      if (pass == 0 && key_floor == 0u) {  // (after a top-k only its k survivors take part: plain atomics do)
        // every kept element takes part and most fall into a few digits: lanes of a warp with the same digit add
        // once (64-bit atomics on one address are what costs here; for the 32-bit counts above it does not pay).
        // A mass is at most 2^40, so the sums of its low and of its high 20 bits over 32 lanes fit 32 bits.
        for (int i0 = warp * 32; i0 < n; i0 += SC_THREADS) {
          const int i = i0 + lane;
          const float x = i < n ? vals[i] : 0.f;
          const unsigned int key = order_key(x);
          const bool in = i < n && key >= key_floor;
          const unsigned int digit = in ? (key >> 24) : 0xffffffffu;
          const unsigned long long m = in ? mass_of(x, mx) : 0ull;
          const unsigned int same = __match_any_sync(0xffffffffu, digit);
          const unsigned int lo = __reduce_add_sync(same, (unsigned int)(m & 0xfffffull));
          const unsigned int hi = __reduce_add_sync(same, (unsigned int)(m >> 20));
          if (in && lane == __ffs(same) - 1)
            atomicAdd(&mass_w[hist * 256 + digit], ((unsigned long long)hi << 20) + lo);
        }
      } else {
        for (int i = tid; i < n; i += SC_THREADS) {
          const float x = vals[i];
          const unsigned int key = order_key(x);
          if (key >= key_floor && (key & mask) == prefix)
            atomicAdd(&mass_w[hist * 256 + ((key >> shift) & 255u)], mass_of(x, mx));
        }
      }
      __syncthreads();
      if (tid < 256) {
        unsigned long long t = 0ull;
#pragma unroll
        for (int w = 0; w < SC_HISTS; ++w) t += mass_w[w * 256 + tid];
        sh.mass_cta[pass_no & 1][tid] = t;
      }
      cluster.sync();
      if (tid < 256) {
        unsigned long long t = 0ull;
        for (int c = 0; c < C; ++c) t += cluster.map_shared_rank(&sh, c)->mass_cta[pass_no & 1][tid];
        sh.mass_tot[tid] = t;
      }
      __syncthreads();
      if (warp == 0) {
        unsigned long long bef;
        const int d = sc_find_digit<false, unsigned long long>(sh.mass_tot, limit, below, &bef);
        if (lane == 0) {
          sh.below = bef;
          sh.prefix = prefix | ((unsigned int)d << shift);
        }
      }
      __syncthreads();
      below = sh.below;
      prefix = sh.prefix;
    }
    key_floor = max(key_floor, prefix);
  }

  // ---- min-p, total mass, draw ---------------------------------------------------------------------------
  float mp = min_p != nullptr ? min_p[r] : 0.f;
  if (!(mp > 0.f)) mp = 0.f;
  const int chunk = (n + SC_THREADS - 1) / SC_THREADS;
  const int cb = min(n, tid * chunk), ce = min(n, cb + chunk);
  unsigned long long local = 0ull;
  for (int i = cb; i < ce; ++i) {
    const float x = vals[i];
    if (order_key(x) >= key_floor && expf(x - mx) >= mp) local += mass_of(x, mx);
  }
  // inclusive scan over the block's threads, then the blocks in rank order
  unsigned long long incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long nb = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += nb;
  }
  if (lane == 31) sh.sum_w[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    unsigned long long w = lane < SC_WARPS ? sh.sum_w[lane] : 0ull;
    unsigned long long wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long nb = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += nb;
    }
    if (lane < SC_WARPS) sh.sum_w[lane] = wi - w;  // exclusive offset of each warp
    if (lane == 31) sh.sum_cta[1] = wi;            // this block's mass
  }
  if (tid == 0) sh.result = -1;
  cluster.sync();
  unsigned long long total = 0ull, before_block = 0ull;
  for (int c = 0; c < C; ++c) {
    const unsigned long long t = cluster.map_shared_rank(&sh, c)->sum_cta[1];
    if (c < rank) before_block += t;
    total += t;
  }
  const unsigned long long excl = before_block + sh.sum_w[warp] + incl - local;
  const float u = uniform != nullptr ? uniform[r] : 0.f;
  unsigned long long target = (unsigned long long)((double)u * (double)total);
  if (total > 0ull && target >= total) target = total - 1ull;
  if (local > 0ull && target >= excl && target < excl + local) {
    unsigned long long run = excl;
    int pick = cb;
    for (int i = cb; i < ce; ++i) {
      const float x = vals[i];
      if (order_key(x) >= key_floor && expf(x - mx) >= mp) {
        run += mass_of(x, mx);
        pick = i;
        if (run > target) break;
      }
    }
    // exactly one thread of one block of the cluster gets here
    const int res = begin + pick;
    out[r] = res;
    if (row_slots != nullptr && last_tokens != nullptr && row_slots[r] >= 0) last_tokens[row_slots[r]] = res;
  }
  if (total == 0ull && rank == 0 && tid == 0) {  // cannot happen: the maximum always has mass 2^40
    out[r] = top.i;
    if (row_slots != nullptr && last_tokens != nullptr && row_slots[r] >= 0) last_tokens[row_slots[r]] = top.i;
  }
  if (pout != nullptr) {
    const float inv = total > 0ull ? 1.f / (float)total : 0.f;
    for (int i = tid; i < n; i += SC_THREADS) {
      const float x = vals[i];
      const bool keep = order_key(x) >= key_floor && expf(x - mx) >= mp;
      pout[begin + i] = keep ? (float)mass_of(x, mx) * inv : 0.f;
    }
  }
  cluster.sync();  // no block leaves while a peer may still read its shared memory
}

static int g_sc_ready = 0;       // 0 not tried, 1 usable, -1 not usable on this device
static int g_sc_max_smem = 0;
static int g_sample_force_one_block = 0;

// 1: rows always go to the one-block kernel (tests compare the two).
extern "C" void ullm_sample_force_one_block(int on) { g_sample_force_one_block = on ? 1 : 0; }

static size_t sc_smem_bytes(int slice) {
  return (size_t)slice * 4 + (size_t)SC_HISTS * 256 * 8;
}

// Which kernel the last call of ullm_sample launched: 1 the cluster kernel, 0 the one-block kernel.
static int g_sample_last_cluster = 0;
extern "C" int ullm_sample_last_used_cluster(void) { return g_sample_last_cluster; }

extern "C" int ullm_sample(const float* logits, long long row_stride, int rows, int vocab, const float* temperature,
                           const int* top_k, const float* top_p, const float* min_p, const float* uniform, int* out,
                           float* probs_out, const int* row_slots, int* last_tokens, void* stream) {
  if (rows < 0 || vocab <= 0) return ULLM_ERR_BAD_SIZE;
  if (rows == 0) return ULLM_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (g_sc_ready == 0) {
    int dev = 0, max_smem = 0;
    g_sc_ready = -1;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) == cudaSuccess) {
      g_sc_max_smem = max_smem - (int)sizeof(ScShared) - 1024;
      if (g_sc_max_smem > 0 &&
          cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, g_sc_max_smem) == cudaSuccess)
        g_sc_ready = 1;
    }
    cudaGetLastError();
  }
  // a slice is a whole number of 16-byte pieces; the last block's may be shorter or empty
  const int slice = ((vocab + SC_CLUSTER - 1) / SC_CLUSTER + 3) / 4 * 4;
  if (g_sc_ready == 1 && !g_sample_force_one_block && sc_smem_bytes(slice) <= (size_t)g_sc_max_smem) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rows * SC_CLUSTER);
    cfg.blockDim = dim3(SC_THREADS);
    cfg.dynamicSmemBytes = sc_smem_bytes(slice);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = SC_CLUSTER;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_ullm_pdl ? 2 : 1;
    if (cudaLaunchKernelEx(&cfg, sample_cluster_kernel, logits, row_stride, vocab, slice, temperature, top_k, top_p, min_p,
                           uniform, out, probs_out, row_slots, last_tokens) == cudaSuccess) {
      g_sample_last_cluster = 1;
      return ULLM_OK;
    }
    cudaGetLastError();
    g_sc_ready = -1;  // this device does not take the cluster launch: the one-block kernel from now on
  }
  g_sample_last_cluster = 0;
  return ullm_launch_kernel(sample_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, st, logits, row_stride,
                            vocab, temperature, top_k, top_p, min_p, uniform, out, probs_out, row_slots, last_tokens);
}
