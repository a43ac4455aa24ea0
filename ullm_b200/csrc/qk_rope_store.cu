// Per-head q/k RMSNorm, position rotation, and the write of this step's keys
// and values into the cache pages, fused: one warp per (token, head).
//
//   q head: x <- rope(norm(x))   written back in place (the attention kernel
//                                reads q from the projection buffer)
//   k head: cache[slot] <- rope(norm(x))
//   v head: cache[slot] <- x
//
// Norm, rotation angles (cos/sin read from 32-bit tables) and the rotation
// itself are computed in 32-bit; one rounding at the store.  Rotary layout:
// the first rotary_dim elements of a head are two halves (x1 | x2); o1 = x1 cos
// - x2 sin and o2 = x2 cos + x1 sin stay in place as (o1 | o2).
#include "common.cuh"

#define QK_MAX_HEAD_DIM 512
#define QK_WARPS 4

template <typename T>
__global__ void qk_norm_rope_store_kernel(T* qkv, int tokens, int num_q, int num_kv, int head_dim,
                                          const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                          int rotary_dim, int max_positions, const int* __restrict__ positions,
                                          const int* __restrict__ slot_mapping, T* k_cache, T* v_cache,
                                          long long num_slots, int* status) {
  __shared__ float sh[QK_WARPS][QK_MAX_HEAD_DIM];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = num_q + 2 * num_kv;
  const long long unit = (long long)blockIdx.x * QK_WARPS + warp;
  if (unit >= (long long)tokens * heads) return;
  const int t = (int)(unit / heads);
  const int h = (int)(unit - (long long)t * heads);
  const bool is_q = h < num_q;
  const bool is_k = !is_q && h < num_q + num_kv;
  long long slot = -1;
  if (!is_q) {
    if (slot_mapping == nullptr) return;  // this execution reads another one's cache
    slot = slot_mapping[t];
    if (slot < 0) return;  // padding row
    if (slot >= num_slots) {
      if (lane == 0) ullm_report(status, ULLM_STATUS_SLOT, t, (int)slot);
      return;
    }
  }
  T* src = qkv + (long long)t * heads * head_dim + (long long)h * head_dim;
  float* y = sh[warp];
  if (!is_q && !is_k) {  // value head: plain copy
    const int kvh = h - num_q - num_kv;
    T* dst = v_cache + (slot * num_kv + kvh) * head_dim;
    for (int e = lane; e < head_dim; e += 32) dst[e] = src[e];
    return;
  }
  const float* w = is_q ? q_w : k_w;
  float ss = 0.f;
  for (int e = lane; e < head_dim; e += 32) {
    const float v = to_f32(src[e]);
    y[e] = v;
    ss += v * v;
  }
  if (w != nullptr) {
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)head_dim + eps);
    for (int e = lane; e < head_dim; e += 32) y[e] = y[e] * rstd * w[e];
  }
  __syncwarp();
  T* dst = is_q ? src : k_cache + (slot * num_kv + (h - num_q)) * head_dim;
  const int half = rotary_dim / 2;
  int pos = 0;
  if (rotary_dim > 0) {
    pos = positions[t];
    if (pos < 0 || pos >= max_positions) {
      if (lane == 0) ullm_report(status, ULLM_STATUS_POSITION, t, pos);
      pos = 0;
    }
  }
  const float* cr = cos_t + (long long)pos * half;
  const float* sr = sin_t + (long long)pos * half;
  for (int e = lane; e < head_dim; e += 32) {
    float o;
    if (e < half) {
      o = y[e] * cr[e] - y[e + half] * sr[e];
    } else if (e < rotary_dim) {
      const int j = e - half;
      o = y[e] * cr[j] + y[j] * sr[j];
    } else {
      o = y[e];
    }
    dst[e] = from_f32<T>(o);
  }
}

// bfloat16, head sizes 64 and 128, full rotary: a lane owns D / 32 neighbouring elements (one 4- or 8-byte
// load), the sum of squares is a warp reduction, and the rotation partner (D / 2 further) sits 16 lanes
// away, so no shared memory is needed.  Same arithmetic as the general kernel.
template <int D>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_bf16_kernel(__nv_bfloat16* qkv, int tokens, int num_q, int num_kv, const float* __restrict__ q_w,
                               const float* __restrict__ k_w, float eps, const float* __restrict__ cos_t,
                               const float* __restrict__ sin_t, int max_positions, const int* __restrict__ positions,
                               const int* __restrict__ slot_mapping, __nv_bfloat16* k_cache, __nv_bfloat16* v_cache,
                               long long num_slots, int* status) {
  constexpr int VEC = D / 32;
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = num_q + 2 * num_kv;
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (unit >= (long long)tokens * heads) return;
  const int t = (int)(unit / heads);
  const int h = (int)(unit - (long long)t * heads);
  const bool is_q = h < num_q;
  const bool is_k = !is_q && h < num_q + num_kv;
  long long slot = -1;
  if (!is_q) {
    if (slot_mapping == nullptr) return;
    slot = slot_mapping[t];
    if (slot < 0) return;
    if (slot >= num_slots) {
      if (lane == 0) ullm_report(status, ULLM_STATUS_SLOT, t, (int)slot);
      return;
    }
  }
  __nv_bfloat16* src = qkv + (long long)t * heads * D + (long long)h * D + lane * VEC;
  __nv_bfloat16 raw[VEC];
  if (VEC == 4) *reinterpret_cast<uint2*>(raw) = *reinterpret_cast<const uint2*>(src);
  else *reinterpret_cast<unsigned*>(raw) = *reinterpret_cast<const unsigned*>(src);
  if (!is_q && !is_k) {
    __nv_bfloat16* dst = v_cache + (slot * num_kv + (h - num_q - num_kv)) * D + lane * VEC;
    if (VEC == 4) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(raw);
    else *reinterpret_cast<unsigned*>(dst) = *reinterpret_cast<const unsigned*>(raw);
    return;
  }
  float y[VEC];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    y[i] = __bfloat162float(raw[i]);
    ss += y[i] * y[i];
  }
  const float* w = is_q ? q_w : k_w;
  if (w != nullptr) {
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)D + eps);
#pragma unroll
    for (int i = 0; i < VEC; ++i) y[i] = y[i] * rstd * w[lane * VEC + i];
  }
  int pos = positions[t];
  if (pos < 0 || pos >= max_positions) {
    if (lane == 0) ullm_report(status, ULLM_STATUS_POSITION, t, pos);
    pos = 0;
  }
  const int j0 = (lane & 15) * VEC;  // index into the half-size tables
  const float* cr = cos_t + (long long)pos * (D / 2) + j0;
  const float* sr = sin_t + (long long)pos * (D / 2) + j0;
  __nv_bfloat16 o[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const float partner = __shfl_xor_sync(0xffffffffu, y[i], 16);
    const float c = cr[i], sn = sr[i];
    const float v = lane < 16 ? y[i] * c - partner * sn : y[i] * c + partner * sn;
    o[i] = __float2bfloat16_rn(v);
  }
  __nv_bfloat16* dst = is_q ? src : k_cache + (slot * num_kv + (h - num_q)) * D + lane * VEC;
  if (VEC == 4) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(o);
  else *reinterpret_cast<unsigned*>(dst) = *reinterpret_cast<const unsigned*>(o);
}

extern "C" int ullm_qk_norm_rope_store(int dtype, void* qkv, int tokens, int num_q, int num_kv, int head_dim,
                                       const float* q_w, const float* k_w, float eps, const float* cos_t,
                                       const float* sin_t, int rotary_dim, int max_positions, const int* positions,
                                       const int* slot_mapping, void* k_cache, void* v_cache, long long num_slots,
                                       int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || num_q <= 0 || num_kv <= 0 || head_dim <= 0) return ULLM_ERR_BAD_SIZE;
  if (head_dim > QK_MAX_HEAD_DIM || rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1))
    return ULLM_ERR_UNSUPPORTED;
  if (rotary_dim > 0 && (cos_t == nullptr || sin_t == nullptr || positions == nullptr)) return ULLM_ERR_BAD_SIZE;
  if (tokens == 0) return ULLM_OK;
  const long long units = (long long)tokens * (num_q + 2 * num_kv);
  const long long blocks = (units + QK_WARPS - 1) / QK_WARPS;
  if (blocks > 0x7fffffffLL) return ULLM_ERR_BAD_SIZE;
  if (dtype == ULLM_DTYPE_BF16 && rotary_dim == head_dim && (head_dim == 64 || head_dim == 128) &&
      (uintptr_t)qkv % 8 == 0 && (slot_mapping == nullptr || ((uintptr_t)k_cache % 8 == 0 && (uintptr_t)v_cache % 8 == 0))) {
    const int warps = 8;
    const long long vblocks = (units + warps - 1) / warps;
    if (head_dim == 128)
      return ullm_launch_kernel(qk_norm_rope_store_bf16_kernel<128>, dim3((int)vblocks), dim3(warps * 32), 0, st,
                                (__nv_bfloat16*)qkv, tokens, num_q, num_kv, q_w, k_w, eps, cos_t, sin_t, max_positions,
                                positions, slot_mapping, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, num_slots,
                                status);
    return ullm_launch_kernel(qk_norm_rope_store_bf16_kernel<64>, dim3((int)vblocks), dim3(warps * 32), 0, st,
                              (__nv_bfloat16*)qkv, tokens, num_q, num_kv, q_w, k_w, eps, cos_t, sin_t, max_positions,
                              positions, slot_mapping, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, num_slots,
                              status);
  }
  if (dtype == ULLM_DTYPE_F32)
    return ullm_launch_kernel(qk_norm_rope_store_kernel<float>, dim3((int)blocks), dim3(QK_WARPS * 32), 0, st,
        (float*)qkv, tokens, num_q, num_kv, head_dim, q_w, k_w, eps, cos_t, sin_t, rotary_dim, max_positions,
        positions, slot_mapping, (float*)k_cache, (float*)v_cache, num_slots, status);
  else if (dtype == ULLM_DTYPE_BF16)
    return ullm_launch_kernel(qk_norm_rope_store_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(QK_WARPS * 32), 0, st,
        (__nv_bfloat16*)qkv, tokens, num_q, num_kv, head_dim, q_w, k_w, eps, cos_t, sin_t, rotary_dim, max_positions,
        positions, slot_mapping, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, num_slots, status);
  else
    return ULLM_ERR_BAD_DTYPE;
  return ullm_launch_status();
}
