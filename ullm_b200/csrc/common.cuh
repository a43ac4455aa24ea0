// Shared device helpers of the sm_100a kernels: element types, 32-bit
// conversion, warp and block reductions, the status word.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define ULLM_DTYPE_F32 0
#define ULLM_DTYPE_BF16 1
#define ULLM_DTYPE_F16 2  // the plain templated kernels only: the tensor-core attention kernels are bfloat16

// Error codes returned by the extern "C" launchers.
#define ULLM_OK 0
#define ULLM_ERR_BAD_DTYPE 1
#define ULLM_ERR_BAD_SIZE 2
#define ULLM_ERR_LAUNCH 3
#define ULLM_ERR_UNSUPPORTED 4

// Codes a kernel writes into the device status word (status[0]; status[1] =
// offending index, status[2] = offending value) instead of reading or writing
// out of range.  The host reads the word when it reads a step's results.
#define ULLM_STATUS_TOKEN_ID 1
#define ULLM_STATUS_POSITION 2
#define ULLM_STATUS_SLOT 3
#define ULLM_STATUS_ROW 4
#define ULLM_STATUS_PAGE 5

__device__ __forceinline__ void ullm_report(int* status, int code, int index, int value) {
  if (status != nullptr && atomicCAS(status, 0, code) == 0) {
    status[1] = index;
    status[2] = value;
  }
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the block, same value in every thread.  `scratch` holds 33 floats.
// The order of additions depends only on blockDim.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Gate activations of a gated feed-forward (codes 0 and 1 of ullm_act_mul), in 32-bit.
__device__ __forceinline__ float act_silu(float g) { return g / (1.f + expf(-g)); }
__device__ __forceinline__ float act_gelu_tanh(float g) {
  const float k = 0.7978845608028654f;
  return 0.5f * g * (1.f + tanhf(k * (g + 0.044715f * g * g * g)));
}

// True when rows of `cols` elements of T starting at `p` can be moved in
// 16-byte pieces.
template <typename T>
__device__ __host__ __forceinline__ bool rows_are_16B(const void* p, long long cols, long long row_stride) {
  return (reinterpret_cast<uintptr_t>(p) % 16 == 0) && ((cols * sizeof(T)) % 16 == 0) &&
         ((row_stride * sizeof(T)) % 16 == 0);
}

// Programmatic dependent launch.  Every kernel of this library starts with
//   pdl_launch_dependents();  the next kernel in the stream may be scheduled as soon as all blocks of
//                             this one are running (its blocks then wait in their own pdl_wait)
//   pdl_wait();               blocks until the previous kernel in the stream has completed and its
//                             writes are visible; nothing that depends on it may be touched before
// so that launch latency and per-block set-up of a kernel overlap with the tail of the one before it.
// A kernel may do work that does not depend on its predecessor (reading weights) before pdl_wait().
// Launches carry the attribute only while ullm_set_pdl(1) is in force; without it both calls are no-ops.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

extern int g_ullm_pdl;

template <typename... KArgs, typename... Args>
static inline int ullm_launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                     Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_ullm_pdl ? 1 : 0;
  if (cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...) != cudaSuccess) {
    cudaGetLastError();
    return ULLM_ERR_LAUNCH;
  }
  return ULLM_OK;
}

static inline int ullm_launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? ULLM_OK : ULLM_ERR_LAUNCH;
}
