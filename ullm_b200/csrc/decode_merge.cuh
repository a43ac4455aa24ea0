// The second kernel of the decode attention kernels that cut the batch's list of key tiles into equal contiguous
// ranges (one per warp in attention_decode_balanced.cu, one per block in attention_decode_tcgen05.cu): a (request,
// kv head) pair that a range boundary cuts has its parts (max, sum, unnormalised output) in the scratch array,
// and this kernel adds them in range order.
#pragma once

#include "common.cuh"

#define DECB_ROW(D) ((D) + 4)  // floats of a partial row: D outputs, max, sum, padded to 16 bytes

// ranges that work: all ranges of the grid, fewer when the batch holds little (no range shorter than min_tiles)
__host__ __device__ __forceinline__ long long decb_ranges(long long total_tiles, long long ranges, int min_tiles) {
  const long long by_work = total_tiles / min_tiles;
  const long long r = ranges < by_work ? ranges : by_work;
  return r < 1 ? 1 : r;
}

// Pairs that more than one range worked on: out[b, h, :] = sum_i O_i 2^(m_i - M) / sum_i l_i 2^(m_i - M), parts
// in warp order.  A block of 512 threads per (request, kv head): D / 4 threads take four output elements each,
// four such groups share a head (a group takes every fourth part; their sums meet in shared memory), and
// 512 / D heads of the pair are merged at a time.
#define DECB_MERGE_THREADS 512
#define DECB_MERGE_LANES 4
template <int D>
__global__ void __launch_bounds__(DECB_MERGE_THREADS)
decode_balanced_merge_kernel(const float* __restrict__ part, const int* __restrict__ prefix, int* __restrict__ flags,
                             __nv_bfloat16* __restrict__ out, int batch, int num_q, int num_kv, long long warps, int min_tiles) {
  constexpr int PER = D / 4;                                             // threads that hold one row of D
  constexpr int HEADS = DECB_MERGE_THREADS / PER / DECB_MERGE_LANES;     // heads at a time
  __shared__ float s_m[HEADS][DECB_MERGE_LANES], s_l[HEADS][DECB_MERGE_LANES];
  __shared__ float4 s_acc[HEADS][DECB_MERGE_LANES][PER];
  pdl_launch_dependents();
  pdl_wait();
  // Most pairs have nothing to merge (they lay whole inside one warp's range, or the request holds nothing):
  // their blocks leave at once.  The flag is cleared for the next launch.
  if (flags[blockIdx.x] == 0) return;
  __syncthreads();
  if (threadIdx.x == 0) flags[blockIdx.x] = 0;
  const int b = blockIdx.x / num_kv, kh = blockIdx.x % num_kv;
  const int group = num_q / num_kv;
  const int tiles = prefix[b + 1] - prefix[b];
  if (tiles == 0) return;
  const long long W = (long long)num_kv * prefix[batch];
  const long long GW = decb_ranges(W, warps, min_tiles);
  const long long p0 = (long long)num_kv * prefix[b] + (long long)kh * tiles, p1 = p0 + tiles - 1;  // first, last tile
  const long long i_first = ((p0 + 1) * GW + W - 1) / W - 1, i_last = ((p1 + 1) * GW + W - 1) / W - 1;
  if (i_first == i_last) return;
  // Every warp's range holds tiles (decb_ranges), and only the first warp can have begun before the pair: its
  // part is in its slot 1 then; all the others begin inside the pair and left theirs in slot 0.
  const int slot_first = i_first * W / GW >= p0 ? 0 : 1;
  const int t4 = threadIdx.x % PER, sub = threadIdx.x / PER;
  const int lane_g = sub % DECB_MERGE_LANES, hs = sub / DECB_MERGE_LANES;
  for (int r0 = 0; r0 < group; r0 += HEADS) {  // the trip count is the same for every thread
    const int r = r0 + hs;
    float mm = -INFINITY, ll = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < group) {
#pragma unroll 4
      for (long long i = i_first + lane_g; i <= i_last; i += DECB_MERGE_LANES) {
        const float* row = part + ((i * 2 + (i == i_first ? slot_first : 0)) * group + r) * DECB_ROW(D);
        const float mi = row[D], li = row[D + 1];
        const float4 v = *reinterpret_cast<const float4*>(row + t4 * 4);
        const float mn = fmaxf(mm, mi);
        const float f_old = mm == -INFINITY ? 0.f : exp2f(mm - mn), f_new = mi == -INFINITY ? 0.f : exp2f(mi - mn);
        ll = ll * f_old + li * f_new;
        acc.x = acc.x * f_old + v.x * f_new;
        acc.y = acc.y * f_old + v.y * f_new;
        acc.z = acc.z * f_old + v.z * f_new;
        acc.w = acc.w * f_old + v.w * f_new;
        mm = mn;
      }
    }
    if (t4 == 0) {
      s_m[hs][lane_g] = mm;
      s_l[hs][lane_g] = ll;
    }
    s_acc[hs][lane_g][t4] = acc;
    __syncthreads();
    if (lane_g == 0 && r < group) {
      float M = -INFINITY;
#pragma unroll
      for (int g = 0; g < DECB_MERGE_LANES; ++g) M = fmaxf(M, s_m[hs][g]);
      float L = 0.f;
      float4 A = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int g = 0; g < DECB_MERGE_LANES; ++g) {  // in lane order: the same sum in every launch
        const float f = s_m[hs][g] == -INFINITY ? 0.f : exp2f(s_m[hs][g] - M);
        const float4 v = s_acc[hs][g][t4];
        L += s_l[hs][g] * f;
        A.x += v.x * f;
        A.y += v.y * f;
        A.z += v.z * f;
        A.w += v.w * f;
      }
      const float inv = L > 0.f ? 1.f / L : 0.f;
      __nv_bfloat16* o = out + ((long long)b * num_q + kh * group + r) * D + t4 * 4;
      *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(A.x * inv, A.y * inv);
      *reinterpret_cast<__nv_bfloat162*>(o + 2) = __floats2bfloat162_rn(A.z * inv, A.w * inv);
    }
    __syncthreads();
  }
}

