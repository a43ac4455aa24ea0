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
                                          long long num_slots, int* status, int k_in_place) {
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
  if (!is_q && slot_mapping == nullptr) {
    // nothing is stored (this execution reads another one's cache); with k_in_place the normed and rotated key
    // goes back where it came from, as the query does
    if (!(k_in_place && is_k)) return;
  } else if (!is_q) {
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
  T* dst = (is_q || slot < 0) ? src : k_cache + (slot * num_kv + (h - num_q)) * head_dim;
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

// The same for bfloat16 with head size 64 or 128: D / 8 lanes hold one (token, head) row, each lane FOUR
// neighbouring elements of the row's first half and the four elements D / 2 further (two 8-byte pieces), so an
// element and its rotation partner sit in the same lane and only the sum of squares travels by shuffles.  A warp
// works on 32 / (D / 8) rows side by side and takes QKV_STEPS such sets of one token's heads (6 for many tokens:
// fewer table reads and more bytes in flight per lane; 1 for the few tokens of a decode step, where the shortest
// chain of work per warp counts): the token's position, its rows of the rotation tables and its cache slot are
// read once for all of them, and all the rows are loaded before any arithmetic.  Nothing returns early: lanes
// without work stay in the shuffles.
template <int D, int QKV_STEPS>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_bf16_kernel(__nv_bfloat16* qkv, int tokens, int num_q, int num_kv, const float* __restrict__ q_w,
                               const float* __restrict__ k_w, float eps, const float* __restrict__ cos_t,
                               const float* __restrict__ sin_t, int max_positions, const int* __restrict__ positions,
                               const int* __restrict__ slot_mapping, __nv_bfloat16* k_cache, __nv_bfloat16* v_cache,
                               long long num_slots, int* status) {
  constexpr int LW = D / 8;                  // lanes of a row
  constexpr int ROWS = 32 / LW;              // rows of a warp, side by side
  constexpr int CHUNK = ROWS * QKV_STEPS;    // heads of a token that one warp takes
  constexpr int HALF = D / 2;
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LW, sl = lane % LW;
  const int heads = num_q + 2 * num_kv;
  const int chunks = (heads + CHUNK - 1) / CHUNK;
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  const bool on = unit < (long long)tokens * chunks;  // the same for the whole warp
  const int t = on ? (int)(unit / chunks) : 0;
  const int h0 = on ? (int)(unit - (long long)t * chunks) * CHUNK : heads;

  // what the token's rows share
  long long slot = -1;
  if (on && slot_mapping != nullptr) {
    slot = slot_mapping[t];
    if (slot >= num_slots) {
      if (lane == 0) ullm_report(status, ULLM_STATUS_SLOT, t, (int)slot);
      slot = -1;
    }
  }
  int pos = on ? positions[t] : 0;
  if (pos < 0 || pos >= max_positions) {
    if (lane == 0) ullm_report(status, ULLM_STATUS_POSITION, t, pos);
    pos = 0;
  }
  uint2 raw_lo[QKV_STEPS], raw_hi[QKV_STEPS];
#pragma unroll
  for (int u = 0; u < QKV_STEPS; ++u) {
    const int h = h0 + u * ROWS + sub;
    // key and value rows of a token without a slot (padding, or an execution that reads another one's cache) are skipped
    const bool live = h < heads && (h < num_q || slot >= 0);
    const __nv_bfloat16* row = qkv + ((long long)t * heads + h) * D + sl * 4;
    raw_lo[u] = live ? *reinterpret_cast<const uint2*>(row) : make_uint2(0, 0);
    raw_hi[u] = live ? *reinterpret_cast<const uint2*>(row + HALF) : make_uint2(0, 0);
  }
  const float4 c4 = *reinterpret_cast<const float4*>(cos_t + (long long)pos * HALF + sl * 4);
  const float4 s4 = *reinterpret_cast<const float4*>(sin_t + (long long)pos * HALF + sl * 4);
  const float c[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};

#pragma unroll
  for (int u = 0; u < QKV_STEPS; ++u) {
    const int h = h0 + u * ROWS + sub;
    const bool is_q = h < num_q, is_k = !is_q && h < num_q + num_kv;
    const bool live = h < heads && (is_q || slot >= 0);
    if (live && !is_q && !is_k) {  // value row: plain copy
      __nv_bfloat16* dst = v_cache + (slot * num_kv + (h - num_q - num_kv)) * D + sl * 4;
      *reinterpret_cast<uint2*>(dst) = raw_lo[u];
      *reinterpret_cast<uint2*>(dst + HALF) = raw_hi[u];
    }
    const __nv_bfloat162* pl = reinterpret_cast<const __nv_bfloat162*>(&raw_lo[u]);
    const __nv_bfloat162* ph = reinterpret_cast<const __nv_bfloat162*>(&raw_hi[u]);
    const float2 l01 = __bfloat1622float2(pl[0]), l23 = __bfloat1622float2(pl[1]);
    const float2 h01 = __bfloat1622float2(ph[0]), h23 = __bfloat1622float2(ph[1]);
    float lo[4] = {l01.x, l01.y, l23.x, l23.y}, hi[4] = {h01.x, h01.y, h23.x, h23.y};
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) ss += lo[i] * lo[i] + hi[i] * hi[i];
#pragma unroll
    for (int off = LW / 2; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);  // every lane takes part
    const float* w = is_q ? q_w : k_w;
    if (w != nullptr) {
      const float rstd = rsqrtf(ss / (float)D + eps);
      const float4 w0 = *reinterpret_cast<const float4*>(w + sl * 4), w1 = *reinterpret_cast<const float4*>(w + HALF + sl * 4);
      lo[0] *= rstd * w0.x; lo[1] *= rstd * w0.y; lo[2] *= rstd * w0.z; lo[3] *= rstd * w0.w;
      hi[0] *= rstd * w1.x; hi[1] *= rstd * w1.y; hi[2] *= rstd * w1.z; hi[3] *= rstd * w1.w;
    }
    float ol[4], oh[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ol[i] = lo[i] * c[i] - hi[i] * sn[i];
      oh[i] = hi[i] * c[i] + lo[i] * sn[i];
    }
    if (live && (is_q || is_k)) {
      __nv_bfloat16* dst = is_q ? qkv + ((long long)t * heads + h) * D + sl * 4
                                : k_cache + (slot * num_kv + (h - num_q)) * D + sl * 4;
      uint2 vl, vh;
      __nv_bfloat162* ql = reinterpret_cast<__nv_bfloat162*>(&vl);
      __nv_bfloat162* qh = reinterpret_cast<__nv_bfloat162*>(&vh);
      ql[0] = __floats2bfloat162_rn(ol[0], ol[1]);
      ql[1] = __floats2bfloat162_rn(ol[2], ol[3]);
      qh[0] = __floats2bfloat162_rn(oh[0], oh[1]);
      qh[1] = __floats2bfloat162_rn(oh[2], oh[3]);
      *reinterpret_cast<uint2*>(dst) = vl;
      *reinterpret_cast<uint2*>(dst + HALF) = vh;
    }
  }
}

static int qk_norm_rope_store_impl(int dtype, void* qkv, int tokens, int num_q, int num_kv, int head_dim,
                                   const float* q_w, const float* k_w, float eps, const float* cos_t,
                                   const float* sin_t, int rotary_dim, int max_positions, const int* positions,
                                   const int* slot_mapping, void* k_cache, void* v_cache, long long num_slots,
                                   int* status, void* stream, int k_in_place) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || num_q <= 0 || num_kv <= 0 || head_dim <= 0) return ULLM_ERR_BAD_SIZE;
  if (head_dim > QK_MAX_HEAD_DIM || rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1))
    return ULLM_ERR_UNSUPPORTED;
  if (rotary_dim > 0 && (cos_t == nullptr || sin_t == nullptr || positions == nullptr)) return ULLM_ERR_BAD_SIZE;
  if (tokens == 0) return ULLM_OK;
  const long long units = (long long)tokens * (num_q + 2 * num_kv);
  const long long blocks = (units + QK_WARPS - 1) / QK_WARPS;
  if (blocks > 0x7fffffffLL) return ULLM_ERR_BAD_SIZE;
  if (!k_in_place && dtype == ULLM_DTYPE_BF16 && rotary_dim == head_dim && (head_dim == 64 || head_dim == 128) &&
      (uintptr_t)qkv % 8 == 0 && (slot_mapping == nullptr || ((uintptr_t)k_cache % 8 == 0 && (uintptr_t)v_cache % 8 == 0))) {
    const int warps = 8;
    const int steps = (long long)tokens * (num_q + 2 * num_kv) >= 8192 ? 6 : 1;
    const int chunk = (32 / (head_dim / 8)) * steps;  // heads of a token that one warp takes
    const long long vunits = (long long)tokens * ((num_q + 2 * num_kv + chunk - 1) / chunk);
    const long long vblocks = (vunits + warps - 1) / warps;
#define ULLM_ROPE_LAUNCH(DD, SS)                                                                                   \
  return ullm_launch_kernel(qk_norm_rope_store_bf16_kernel<DD, SS>, dim3((int)vblocks), dim3(warps * 32), 0, st,   \
                            (__nv_bfloat16*)qkv, tokens, num_q, num_kv, q_w, k_w, eps, cos_t, sin_t, max_positions, \
                            positions, slot_mapping, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, num_slots,   \
                            status)
    if (head_dim == 128 && steps == 6) ULLM_ROPE_LAUNCH(128, 6);
    if (head_dim == 128) ULLM_ROPE_LAUNCH(128, 1);
    if (steps == 6) ULLM_ROPE_LAUNCH(64, 6);
    ULLM_ROPE_LAUNCH(64, 1);
#undef ULLM_ROPE_LAUNCH
  }
  if (dtype == ULLM_DTYPE_F32)
    return ullm_launch_kernel(qk_norm_rope_store_kernel<float>, dim3((int)blocks), dim3(QK_WARPS * 32), 0, st,
        (float*)qkv, tokens, num_q, num_kv, head_dim, q_w, k_w, eps, cos_t, sin_t, rotary_dim, max_positions,
        positions, slot_mapping, (float*)k_cache, (float*)v_cache, num_slots, status, k_in_place);
  else if (dtype == ULLM_DTYPE_BF16)
    return ullm_launch_kernel(qk_norm_rope_store_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(QK_WARPS * 32), 0, st,
        (__nv_bfloat16*)qkv, tokens, num_q, num_kv, head_dim, q_w, k_w, eps, cos_t, sin_t, rotary_dim, max_positions,
        positions, slot_mapping, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, num_slots, status, k_in_place);
  else if (dtype == ULLM_DTYPE_F16)
    return ullm_launch_kernel(qk_norm_rope_store_kernel<__half>, dim3((int)blocks), dim3(QK_WARPS * 32), 0, st,
        (__half*)qkv, tokens, num_q, num_kv, head_dim, q_w, k_w, eps, cos_t, sin_t, rotary_dim, max_positions,
        positions, slot_mapping, (__half*)k_cache, (__half*)v_cache, num_slots, status, k_in_place);
  else
    return ULLM_ERR_BAD_DTYPE;
  return ullm_launch_status();
}

extern "C" int ullm_qk_norm_rope_store(int dtype, void* qkv, int tokens, int num_q, int num_kv, int head_dim,
                                       const float* q_w, const float* k_w, float eps, const float* cos_t,
                                       const float* sin_t, int rotary_dim, int max_positions, const int* positions,
                                       const int* slot_mapping, void* k_cache, void* v_cache, long long num_slots,
                                       int* status, void* stream) {
  return qk_norm_rope_store_impl(dtype, qkv, tokens, num_q, num_kv, head_dim, q_w, k_w, eps, cos_t, sin_t, rotary_dim,
                                 max_positions, positions, slot_mapping, k_cache, v_cache, num_slots, status, stream, 0);
}

// Queries AND keys normed (and rotated, if tables are given) where they lie; nothing is stored.  For mixers whose
// position encoding has code of its own: it changes q and k afterwards, and a second call (no weights, no tables,
// a slot mapping) stores the keys and values.
extern "C" int ullm_qk_norm_in_place(int dtype, void* qkv, int tokens, int num_q, int num_kv, int head_dim,
                                     const float* q_w, const float* k_w, float eps, int* status, void* stream) {
  return qk_norm_rope_store_impl(dtype, qkv, tokens, num_q, num_kv, head_dim, q_w, k_w, eps, nullptr, nullptr, 0, 0,
                                 nullptr, nullptr, nullptr, nullptr, 0, status, stream, 1);
}
