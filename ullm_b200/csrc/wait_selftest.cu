// Self-test of the give-up path that every tcgen05 / TMA kernel of this library has.
//
// Those kernels wait on mbarriers (TMA bytes, tcgen05.commit) through mbar_wait_limited(): after a bounded
// number of polls the wait returns false, the kernel records ULLM_STATUS_TIMEOUT with the place it gave up,
// stops waiting, frees its tensor memory and returns, so that the context stays usable and the host raises.
// In a healthy run that path never executes.  This one-block kernel runs it on purpose, without a fault: it
// allocates tensor memory as the product kernels do, initialises a barrier that nothing will ever arrive at,
// waits on it with the poll limit the caller gives (a few thousand), and then does what the real kernels do
// when a wait runs out.  The test checks the status word and that the next ordinary kernel runs.
#include "tcgen05_util.cuh"

#define WAIT_SELFTEST_PLACE 90

__global__ void __launch_bounds__(64) wait_selftest_kernel(int limit, int* status, int* out) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int gave_up;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    gave_up = 0;
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(lin_smem(&tmem_base_slot)),
                 "r"(32)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_slot;
  if (threadIdx.x == 0) {
    // phase 0 of a fresh barrier completes only when someone arrives; nobody does
    if (!mbar_wait_limited(&bar, 0, limit)) {
      ullm_report(status, ULLM_STATUS_TIMEOUT, WAIT_SELFTEST_PLACE, limit);
      gave_up = 1;
    }
  }
  __syncthreads();
  // the way out that the product kernels take: no copy is in flight here, the tensor memory goes back
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(32) : "memory");
  }
  if (threadIdx.x == 0 && out != nullptr) out[0] = gave_up ? 1 : 2;
}

// Launches the self-test with `limit` polls (1 .. 1 << 20).  out[0] becomes 1 when the wait ran out (expected)
// and 2 when it did not.
extern "C" int ullm_wait_selftest(int limit, int* status, int* out, void* stream) {
  if (limit <= 0 || limit > WAIT_LIMIT || status == nullptr) return ULLM_ERR_BAD_SIZE;
  return ullm_launch_kernel(wait_selftest_kernel, dim3(1), dim3(64), 0, (cudaStream_t)stream, limit, status, out);
}
