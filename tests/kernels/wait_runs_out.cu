// A test-only kernel: it waits on an mbarrier at which nobody ever arrives, through the
// package's own bounded wait (csrc/bounded_wait.cuh) with a small limit, while it holds tensor
// memory the way the product kernels do.  The wait runs out, the kernel records its code in the
// error word, frees its tensor memory and returns: nothing traps, nothing hangs, and the
// context stays usable.  The host reads the word and the number of polls.
#include <cuda_runtime.h>
#include <stdint.h>

#define TL_WAIT_LIMIT (1u << 10)
#include "bounded_wait.cuh"

__device__ int test_error_word = 0;

__global__ void wait_runs_out_kernel(int* report) {
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    tl_mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     tl_smem_u32(&tmem_slot)), "r"(32u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_slot;
  bool ok = true;
  if (threadIdx.x == 32) {
    // the role that waits: nobody arrives at `bar`
    ok = tl_mbar_wait(&bar, 0, &abort_flag, 7, &test_error_word);
    report[0] = ok ? 1 : 0;
  }
  __syncthreads();
  if (threadIdx.x == 64) {
    // another role of the block: it finds the flag up and gives up at its first look
    const bool ok2 = tl_mbar_wait(&bar, 0, &abort_flag, 9, &test_error_word);
    report[1] = ok2 ? 1 : 0;
    report[2] = abort_flag;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32u) : "memory");
}

// Runs the kernel once and returns the error word (then cleared); report[0..2] = what the two
// waits returned and the block's flag.  A negative value is a CUDA error, negated.
extern "C" int test_wait_runs_out(int* report_host) {
  int* report = nullptr;
  if (cudaMalloc(&report, 4 * sizeof(int)) != cudaSuccess) return -1;
  cudaMemset(report, 0xff, 4 * sizeof(int));
  wait_runs_out_kernel<<<1, 128>>>(report);
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) { cudaFree(report); return -(int)e; }
  cudaMemcpy(report_host, report, 3 * sizeof(int), cudaMemcpyDeviceToHost);
  cudaFree(report);
  int word = 0, zero = 0;
  cudaMemcpyFromSymbol(&word, test_error_word, sizeof(int));
  cudaMemcpyToSymbol(test_error_word, &zero, sizeof(int));
  return word;
}
