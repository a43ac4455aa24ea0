// Embedding gather, row gather, fused residual-add + RMSNorm, gated
// activation, dtype casts.  Every kernel takes any row length; rows that can be
// moved in 16-byte pieces are, others go element by element.
#include "common.cuh"

#include <type_traits>

int g_ullm_pdl = 0;
extern "C" void ullm_set_pdl(int on) { g_ullm_pdl = on ? 1 : 0; }

// ---------------------------------------------------------------------------
// row copies: out[r, :] = src[index[r], :]
// ---------------------------------------------------------------------------
template <typename T>
__global__ void gather_rows_kernel(const int* __restrict__ index, const T* __restrict__ src, T* __restrict__ out,
                                   int rows, int cols, long long src_stride, long long out_stride, int src_rows,
                                   int status_code, int* status, const int* __restrict__ last_tokens,
                                   const int* __restrict__ token_req, const int* __restrict__ req_slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  if (r >= rows) return;
  int s = index[r];
  // An id of -1 stands for "the token this request sampled last": it is still on the device only
  // (last_tokens[request slot]), because the host has launched this step before reading it.
  if (s < 0 && last_tokens != nullptr) {
    const int b = token_req[r];
    s = b >= 0 ? last_tokens[req_slots[b]] : 0;
  }
  if (s < 0 || s >= src_rows) {
    if (threadIdx.x == 0) ullm_report(status, status_code, r, s);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) out[(long long)r * out_stride + c] = from_f32<T>(0.f);
    return;
  }
  const T* sp = src + (long long)s * src_stride;
  T* op = out + (long long)r * out_stride;
  if (rows_are_16B<T>(src, cols, src_stride) && rows_are_16B<T>(out, cols, out_stride)) {
    const int n16 = (int)((cols * sizeof(T)) / 16);
    const uint4* s4 = reinterpret_cast<const uint4*>(sp);
    uint4* o4 = reinterpret_cast<uint4*>(op);
    for (int c = threadIdx.x; c < n16; c += blockDim.x) o4[c] = s4[c];
  } else {
    for (int c = threadIdx.x; c < cols; c += blockDim.x) op[c] = sp[c];
  }
}

template <typename T>
static int gather_rows_launch(const int* index, const void* src, void* out, int rows, int cols, long long src_stride,
                              long long out_stride, int src_rows, int code, int* status, cudaStream_t st,
                              const int* last_tokens = nullptr, const int* token_req = nullptr,
                              const int* req_slots = nullptr) {
  if (rows == 0) return ULLM_OK;
  int threads = 256;
  if (cols * (int)sizeof(T) <= 16 * 64) threads = 64;
  return ullm_launch_kernel(gather_rows_kernel<T>, dim3(rows), dim3(threads), 0, st, index, (const T*)src, (T*)out, rows,
                            cols, src_stride, out_stride, src_rows, code, status, last_tokens, token_req, req_slots);
}

// `last_tokens`, `token_req`, `req_slots` (all three or none): an id of -1 is replaced by
// last_tokens[req_slots[token_req[row]]].
extern "C" int ullm_embedding(int dtype, const int* ids, const void* table, void* out, int tokens, int hidden,
                              int vocab, const int* last_tokens, const int* token_req, const int* req_slots,
                              int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || hidden <= 0 || vocab <= 0) return ULLM_ERR_BAD_SIZE;
  if (last_tokens != nullptr && (token_req == nullptr || req_slots == nullptr)) return ULLM_ERR_BAD_SIZE;
  if (dtype == ULLM_DTYPE_F32)
    return gather_rows_launch<float>(ids, table, out, tokens, hidden, hidden, hidden, vocab, ULLM_STATUS_TOKEN_ID,
                                     status, st, last_tokens, token_req, req_slots);
  if (dtype == ULLM_DTYPE_BF16)
    return gather_rows_launch<__nv_bfloat16>(ids, table, out, tokens, hidden, hidden, hidden, vocab,
                                             ULLM_STATUS_TOKEN_ID, status, st, last_tokens, token_req, req_slots);
  if (dtype == ULLM_DTYPE_F16)
    return gather_rows_launch<__half>(ids, table, out, tokens, hidden, hidden, hidden, vocab, ULLM_STATUS_TOKEN_ID,
                                      status, st, last_tokens, token_req, req_slots);
  return ULLM_ERR_BAD_DTYPE;
}

extern "C" int ullm_gather_rows(int dtype, const int* rows_index, const void* src, void* out, int rows, int cols,
                                int src_rows, int* status, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (rows < 0 || cols <= 0) return ULLM_ERR_BAD_SIZE;
  if (dtype == ULLM_DTYPE_F32)
    return gather_rows_launch<float>(rows_index, src, out, rows, cols, cols, cols, src_rows, ULLM_STATUS_ROW, status,
                                     st);
  if (dtype == ULLM_DTYPE_BF16)
    return gather_rows_launch<__nv_bfloat16>(rows_index, src, out, rows, cols, cols, cols, src_rows, ULLM_STATUS_ROW,
                                             status, st);
  if (dtype == ULLM_DTYPE_F16)
    return gather_rows_launch<__half>(rows_index, src, out, rows, cols, cols, cols, src_rows, ULLM_STATUS_ROW, status,
                                      st);
  return ULLM_ERR_BAD_DTYPE;
}

// ---------------------------------------------------------------------------
// fused residual add + RMSNorm
//   s = x (+ residual)          32-bit
//   residual <- round(s)        (if residual given)
//   out <- round(s * rsqrt(mean(s^2) + eps) * w)
// One block per row; the unrounded sums wait in shared memory between the two
// passes, so the norm sees the 32-bit sum while the stored residual is rounded.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void add_rmsnorm_kernel(const T* x, T* residual, const float* __restrict__ w, T* out, int cols,
                                   float eps) {  // out may be x
  extern __shared__ float row[];  // cols floats, then 33 for the reduction
  pdl_launch_dependents();
  pdl_wait();
  float* scratch = row + cols;
  const long long base = (long long)blockIdx.x * cols;
  float acc = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float s = to_f32(x[base + c]);
    if (residual != nullptr) {
      s += to_f32(residual[base + c]);
      residual[base + c] = from_f32<T>(s);
    }
    row[c] = s;
    acc += s * s;
  }
  const float total = block_sum(acc, scratch);
  const float rstd = rsqrtf(total / (float)cols + eps);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) out[base + c] = from_f32<T>(row[c] * rstd * w[c]);
}

// bfloat16 rows that fit the block's registers (cols <= 16 * threads, a multiple of 8): every thread holds up
// to two groups of 8 elements, all loads are issued before anything else, the row never goes through shared
// memory.  The sum x + residual is formed and squared in 32-bit; the residual is rounded once.
__global__ void __launch_bounds__(512)
add_rmsnorm_bf16x8_reg_kernel(const __nv_bfloat16* x, __nv_bfloat16* residual, const float* __restrict__ w,
                              __nv_bfloat16* out, int cols, float eps) {  // out may be x
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const long long base = (long long)blockIdx.x * cols;
  const int groups = cols / 8;
  const int g0 = threadIdx.x, g1 = threadIdx.x + blockDim.x;
  const bool on0 = g0 < groups, on1 = g1 < groups;
  uint4 xv[2], rv[2];
  xv[0] = on0 ? *reinterpret_cast<const uint4*>(x + base + g0 * 8) : make_uint4(0, 0, 0, 0);
  xv[1] = on1 ? *reinterpret_cast<const uint4*>(x + base + g1 * 8) : make_uint4(0, 0, 0, 0);
  if (residual != nullptr) {
    rv[0] = on0 ? *reinterpret_cast<const uint4*>(residual + base + g0 * 8) : make_uint4(0, 0, 0, 0);
    rv[1] = on1 ? *reinterpret_cast<const uint4*>(residual + base + g1 * 8) : make_uint4(0, 0, 0, 0);
  }
  float s[2][8];
  float acc = 0.f;
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const __nv_bfloat16* xe = reinterpret_cast<const __nv_bfloat16*>(&xv[q]);
    const __nv_bfloat16* re = reinterpret_cast<const __nv_bfloat16*>(&rv[q]);
    uint4 ov;
    __nv_bfloat16* oe = reinterpret_cast<__nv_bfloat16*>(&ov);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      s[q][k] = __bfloat162float(xe[k]);
      if (residual != nullptr) {
        s[q][k] += __bfloat162float(re[k]);
        oe[k] = __float2bfloat16_rn(s[q][k]);
      }
      acc += s[q][k] * s[q][k];
    }
    if (residual != nullptr && (q == 0 ? on0 : on1))
      *reinterpret_cast<uint4*>(residual + base + (q == 0 ? g0 : g1) * 8) = ov;
  }
  const float total = block_sum(acc, scratch);
  const float rstd = rsqrtf(total / (float)cols + eps);
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const int g = q == 0 ? g0 : g1;
    if (g < groups) {
      const float4 w0 = *reinterpret_cast<const float4*>(w + g * 8), w1 = *reinterpret_cast<const float4*>(w + g * 8 + 4);
      const float wk[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      uint4 ov;
      __nv_bfloat16* oe = reinterpret_cast<__nv_bfloat16*>(&ov);
#pragma unroll
      for (int k = 0; k < 8; ++k) oe[k] = __float2bfloat16_rn(s[q][k] * rstd * wk[k]);
      *reinterpret_cast<uint4*>(out + base + g * 8) = ov;
    }
  }
}

// bf16 rows of a multiple of 8 elements on 16-byte boundaries: 8 elements per thread and step.
// Same arithmetic and the same order of additions inside a thread's 8-element groups.
__global__ void add_rmsnorm_bf16x8_kernel(const __nv_bfloat16* x, __nv_bfloat16* residual, const float* __restrict__ w,
                                          __nv_bfloat16* out, int cols, float eps) {  // out may be x
  extern __shared__ float row[];
  float* scratch = row + cols;
  pdl_launch_dependents();
  pdl_wait();
  const long long base = (long long)blockIdx.x * cols;
  const int groups = cols / 8;
  float acc = 0.f;
  for (int g = threadIdx.x; g < groups; g += blockDim.x) {
    const uint4 xv = *reinterpret_cast<const uint4*>(x + base + g * 8);
    const __nv_bfloat16* xe = reinterpret_cast<const __nv_bfloat16*>(&xv);
    float s[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) s[k] = __bfloat162float(xe[k]);
    if (residual != nullptr) {
      const uint4 rv = *reinterpret_cast<const uint4*>(residual + base + g * 8);
      const __nv_bfloat16* re = reinterpret_cast<const __nv_bfloat16*>(&rv);
      uint4 ov;
      __nv_bfloat16* oe = reinterpret_cast<__nv_bfloat16*>(&ov);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        s[k] += __bfloat162float(re[k]);
        oe[k] = __float2bfloat16_rn(s[k]);
      }
      *reinterpret_cast<uint4*>(residual + base + g * 8) = ov;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      row[g * 8 + k] = s[k];
      acc += s[k] * s[k];
    }
  }
  const float total = block_sum(acc, scratch);
  const float rstd = rsqrtf(total / (float)cols + eps);
  for (int g = threadIdx.x; g < groups; g += blockDim.x) {
    uint4 ov;
    __nv_bfloat16* oe = reinterpret_cast<__nv_bfloat16*>(&ov);
#pragma unroll
    for (int k = 0; k < 8; ++k) oe[k] = __float2bfloat16_rn(row[g * 8 + k] * rstd * w[g * 8 + k]);
    *reinterpret_cast<uint4*>(out + base + g * 8) = ov;
  }
}

static int g_rmsnorm_smem_set[4] = {0, 0, 0, 0};

template <typename T>
static int add_rmsnorm_launch(int which, const void* x, void* residual, const float* w, void* out, int rows, int cols,
                              float eps, cudaStream_t st) {
  if (rows == 0) return ULLM_OK;
  const size_t smem = (size_t)(cols + 33) * sizeof(float);
  if (smem > 200 * 1024) return ULLM_ERR_UNSUPPORTED;
  if (smem > 48 * 1024 && !g_rmsnorm_smem_set[which]) {
    if (cudaFuncSetAttribute(add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) !=
        cudaSuccess)
      return ULLM_ERR_LAUNCH;
    g_rmsnorm_smem_set[which] = 1;
  }
  if (std::is_same<T, __nv_bfloat16>::value && cols % 8 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)out % 16 == 0) &&
      (residual == nullptr || (uintptr_t)residual % 16 == 0)) {
    if (smem > 48 * 1024 && !g_rmsnorm_smem_set[2]) {
      if (cudaFuncSetAttribute(add_rmsnorm_bf16x8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) !=
          cudaSuccess)
        return ULLM_ERR_LAUNCH;
      g_rmsnorm_smem_set[2] = 1;
    }
    if (cols <= 16 * 512 && (uintptr_t)w % 16 == 0) {  // the row fits the registers of a block: two groups of 8 per thread
      int threads = 32;
      while (threads < 512 && threads * 16 < cols) threads <<= 1;
      return ullm_launch_kernel(add_rmsnorm_bf16x8_reg_kernel, dim3(rows), dim3(threads), 0, st,
                                (const __nv_bfloat16*)x, (__nv_bfloat16*)residual, w, (__nv_bfloat16*)out, cols, eps);
    }
    int threads = 32;
    while (threads < 512 && threads * 8 < cols) threads <<= 1;
    return ullm_launch_kernel(add_rmsnorm_bf16x8_kernel, dim3(rows), dim3(threads), smem, st,
                              (const __nv_bfloat16*)x, (__nv_bfloat16*)residual, w, (__nv_bfloat16*)out, cols, eps);
  }
  int threads = 32;
  while (threads < 1024 && threads * 4 < cols) threads <<= 1;
  return ullm_launch_kernel(add_rmsnorm_kernel<T>, dim3(rows), dim3(threads), smem, st, (const T*)x, (T*)residual, w,
                            (T*)out, cols, eps);
}

extern "C" int ullm_add_rmsnorm(int dtype, const void* x, void* residual, const float* weight, void* out, int rows,
                                int cols, float eps, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (rows < 0 || cols <= 0) return ULLM_ERR_BAD_SIZE;
  if (dtype == ULLM_DTYPE_F32) return add_rmsnorm_launch<float>(0, x, residual, weight, out, rows, cols, eps, st);
  if (dtype == ULLM_DTYPE_BF16)
    return add_rmsnorm_launch<__nv_bfloat16>(1, x, residual, weight, out, rows, cols, eps, st);
  if (dtype == ULLM_DTYPE_F16) return add_rmsnorm_launch<__half>(3, x, residual, weight, out, rows, cols, eps, st);
  return ULLM_ERR_BAD_DTYPE;
}

// ---------------------------------------------------------------------------
// gated activation: out[t, i] = act(gu[t, i]) * gu[t, I + i], in 32-bit
// ---------------------------------------------------------------------------

template <typename T, int ACT>
__global__ void act_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, long long rows, int inter) {
  pdl_launch_dependents();
  pdl_wait();
  const long long n = rows * inter;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / inter;
    const int c = (int)(i - t * inter);
    const float g = to_f32(gu[t * 2 * inter + c]);
    const float u = to_f32(gu[t * 2 * inter + inter + c]);
    const float a = ACT == 0 ? act_silu(g) : act_gelu_tanh(g);
    out[i] = from_f32<T>(a * u);
  }
}

// bfloat16 in 16-byte pieces: blockIdx.y is the row, a thread takes two pieces of 8 elements and loads gate and
// up of both before anything else (no division per element, four loads in flight per thread).
template <int ACT>
__global__ void __launch_bounds__(256)
act_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, long long rows,
                      int inter) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = inter / 8;
  for (long long t = blockIdx.y; t < rows; t += gridDim.y) {
    const __nv_bfloat16* g_row = gu + t * 2 * inter;
    const int c0 = (blockIdx.x * 2 * blockDim.x + threadIdx.x) * 8, c1 = c0 + blockDim.x * 8;
    const bool on0 = c0 < per_row * 8, on1 = c1 < per_row * 8;
    uint4 gv[2], uv[2];
    gv[0] = on0 ? *reinterpret_cast<const uint4*>(g_row + c0) : make_uint4(0, 0, 0, 0);
    uv[0] = on0 ? *reinterpret_cast<const uint4*>(g_row + inter + c0) : make_uint4(0, 0, 0, 0);
    gv[1] = on1 ? *reinterpret_cast<const uint4*>(g_row + c1) : make_uint4(0, 0, 0, 0);
    uv[1] = on1 ? *reinterpret_cast<const uint4*>(g_row + inter + c1) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(&gv[q]);
      const __nv_bfloat16* u = reinterpret_cast<const __nv_bfloat16*>(&uv[q]);
      uint4 ov;
      __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&ov);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float gf = to_f32(g[k]);
        // (the hardware's exponential and reciprocal: 2 ulp of a 32-bit result that is rounded to bfloat16 next;
        // with expf and a true division this kernel was bound by instructions, not by memory)
        const float a = ACT == 0 ? __fdividef(gf, 1.f + __expf(-gf)) : act_gelu_tanh(gf);
        o[k] = __float2bfloat16_rn(a * to_f32(u[k]));
      }
      if (q == 0 ? on0 : on1) *reinterpret_cast<uint4*>(out + t * inter + (q == 0 ? c0 : c1)) = ov;
    }
  }
}

extern "C" int ullm_act_mul(int dtype, int act, const void* gate_up, void* out, int rows, int inter, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (rows < 0 || inter <= 0) return ULLM_ERR_BAD_SIZE;
  if (act != 0 && act != 1) return ULLM_ERR_UNSUPPORTED;
  if (rows == 0) return ULLM_OK;
  const long long n = (long long)rows * inter;
  const int threads = 256;
  if (dtype == ULLM_DTYPE_BF16 && inter % 8 == 0 && reinterpret_cast<uintptr_t>(gate_up) % 16 == 0 &&
      reinterpret_cast<uintptr_t>(out) % 16 == 0) {
    const dim3 grid((unsigned)((inter / 8 + 2 * threads - 1) / (2 * threads)), (unsigned)(rows < 65535 ? rows : 65535));
    if (act == 0)
      return ullm_launch_kernel(act_mul_bf16x8_kernel<0>, grid, dim3(threads), 0, st, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, (long long)rows, inter);
    else
      return ullm_launch_kernel(act_mul_bf16x8_kernel<1>, grid, dim3(threads), 0, st, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, (long long)rows, inter);
    return ullm_launch_status();
  }
  long long blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == ULLM_DTYPE_F32) {
    if (act == 0)
      return ullm_launch_kernel(act_mul_kernel<float, 0>, dim3((int)blocks), dim3(threads), 0, st, (const float*)gate_up, (float*)out, (long long)rows, inter);
    else
      return ullm_launch_kernel(act_mul_kernel<float, 1>, dim3((int)blocks), dim3(threads), 0, st, (const float*)gate_up, (float*)out, (long long)rows, inter);
  } else if (dtype == ULLM_DTYPE_BF16) {
    if (act == 0)
      return ullm_launch_kernel(act_mul_kernel<__nv_bfloat16, 0>, dim3((int)blocks), dim3(threads), 0, st, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, (long long)rows, inter);
    else
      return ullm_launch_kernel(act_mul_kernel<__nv_bfloat16, 1>, dim3((int)blocks), dim3(threads), 0, st, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, (long long)rows, inter);
  } else if (dtype == ULLM_DTYPE_F16) {
    if (act == 0)
      return ullm_launch_kernel(act_mul_kernel<__half, 0>, dim3((int)blocks), dim3(threads), 0, st, (const __half*)gate_up, (__half*)out, (long long)rows, inter);
    else
      return ullm_launch_kernel(act_mul_kernel<__half, 1>, dim3((int)blocks), dim3(threads), 0, st, (const __half*)gate_up, (__half*)out, (long long)rows, inter);
  } else {
    return ULLM_ERR_BAD_DTYPE;
  }
  return ullm_launch_status();
}

// ---------------------------------------------------------------------------
// bf16 -> f32 cast of a contiguous array (logits for the sampler and the host)
// ---------------------------------------------------------------------------
__global__ void cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, long long n) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = __bfloat162float(in[i]);
}

extern "C" int ullm_cast_bf16_f32(const void* in, float* out, long long n, void* stream) {
  if (n < 0) return ULLM_ERR_BAD_SIZE;
  if (n == 0) return ULLM_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return ullm_launch_kernel(cast_bf16_f32_kernel, dim3((int)blocks), dim3(256), 0, (cudaStream_t)stream,
                            (const __nv_bfloat16*)in, out, n);
}
