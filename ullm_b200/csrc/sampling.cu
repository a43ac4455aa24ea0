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
#include "common.cuh"

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

extern "C" int ullm_sample(const float* logits, long long row_stride, int rows, int vocab, const float* temperature,
                           const int* top_k, const float* top_p, const float* min_p, const float* uniform, int* out,
                           float* probs_out, const int* row_slots, int* last_tokens, void* stream) {
  if (rows < 0 || vocab <= 0) return ULLM_ERR_BAD_SIZE;
  if (rows == 0) return ULLM_OK;
  return ullm_launch_kernel(sample_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, logits, row_stride,
                            vocab, temperature, top_k, top_p, min_p, uniform, out, probs_out, row_slots, last_tokens);
}
