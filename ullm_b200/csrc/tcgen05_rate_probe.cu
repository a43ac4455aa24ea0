// A measuring aid, not part of any step: how many clocks one tcgen05.mma (kind::f16, bfloat16 operands,
// cta_group::1, M = 128, K = 16) takes when one thread issues them back to back, for the shapes and operand
// sources the attention and product kernels use.  One block per SM, one issuing thread; the operands are whatever
// shared and tensor memory hold (the values do not matter for the rate).  The wait for the last product is bounded.
#include <cuda.h>

#include "common.cuh"
#include "tcgen05_util.cuh"

#define RP_SMEM (96 * 1024)

// MODE 0: both operands from shared memory, N = 128; 1: N = 256; 2: A from tensor memory, B MN-major, N = 128;
// 3: shared memory, N = 64; 4: eight of mode 0 then eight of mode 2, in turn (what an attention step issues)
template <int MODE>
__global__ void __launch_bounds__(128, 1) tcgen05_rate_kernel(int iters, long long* out, int* status) {
  extern __shared__ __align__(1024) unsigned char rp_smem[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < RP_SMEM / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(rp_smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(lin_smem(&tmem_slot)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_slot;
  if (warp == 0 && lane == 0) {
    // descriptors as their halves: 8-row groups 1024 bytes apart, version 1, 128-byte swizzle
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    const uint32_t a_lo = ((lin_smem(rp_smem) & 0x3FFFF) >> 4) | (1u << 16);
    const uint32_t b_lo = ((lin_smem(rp_smem + 32768) & 0x3FFFF) >> 4) | (1u << 16);
    const uint32_t bv_lo = ((lin_smem(rp_smem + 32768) & 0x3FFFF) >> 4) | ((uint32_t)(16384 >> 4) << 16);
    const uint32_t base = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 4) << 24);
    const uint32_t id64 = base | ((uint32_t)(64 >> 3) << 17), id128 = base | ((uint32_t)(128 >> 3) << 17),
                   id256 = base | ((uint32_t)(256 >> 3) << 17), id128v = id128 | (1u << 16);
    auto ss = [&](uint32_t d, uint32_t a, uint32_t b, uint32_t id) { umma_bf16_lo<1>(d, a, b, hi, id); };
    auto ts = [&](uint32_t d, uint32_t a, uint32_t b, uint32_t id) {
      asm volatile(
          "{\n .reg .b64 db;\n .reg .pred p;\n mov.b64 db, {%2, %3};\n setp.eq.b32 p, 0, 0;\n"
          " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n}\n"
          ::"r"(d), "r"(a), "r"(b), "r"(hi), "r"(id)
          : "memory");
    };
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = (kk >> 2) * 1024 + 2 * (kk & 3);
        if (MODE == 0 || MODE == 4) ss(tmem, a_lo + off, b_lo + off, id128);
        if (MODE == 1) ss(tmem, a_lo + off, b_lo + off, id256);
        if (MODE == 2) ts(tmem + 256, tmem + kk * 8, bv_lo + kk * 128, id128v);
        if (MODE == 3) ss(tmem, a_lo + off, b_lo + off, id64);
      }
      if (MODE == 4) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) ts(tmem + 256, tmem + kk * 8, bv_lo + kk * 128, id128v);
      }
    }
    umma_commit(&bar);
    if (!mbar_wait(&bar, 0)) ullm_report(status, ULLM_STATUS_TIMEOUT, 60, MODE);
    if (blockIdx.x == 0) out[0] = clock64() - t0;
  }
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

// Runs `iters` rounds of 8 (mode 4: 16) products on `blocks` blocks; `out[0]` receives block 0's clocks from the
// first issue to the completion of the last product.  Returns the number of products per block, or -1.
extern "C" int ullm_tcgen05_mma_rate(int mode, int iters, int blocks, long long* out, int* status, void* stream) {
  typedef void (*Kern)(int, long long*, int*);
  static const Kern kernels[5] = {tcgen05_rate_kernel<0>, tcgen05_rate_kernel<1>, tcgen05_rate_kernel<2>,
                                  tcgen05_rate_kernel<3>, tcgen05_rate_kernel<4>};
  if (mode < 0 || mode > 4 || iters <= 0 || iters > (1 << 16) || blocks <= 0) return -1;
  if (cudaFuncSetAttribute(kernels[mode], cudaFuncAttributeMaxDynamicSharedMemorySize, RP_SMEM) != cudaSuccess) return -1;
  kernels[mode]<<<blocks, 128, RP_SMEM, (cudaStream_t)stream>>>(iters, out, status);
  if (cudaGetLastError() != cudaSuccess) return -1;
  return iters * (mode == 4 ? 16 : 8);
}
