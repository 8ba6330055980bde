// A kernel for tests only: it makes a bounded barrier wait run out on purpose.
//
// The tcgen05 kernels never spin without a limit: a wait on an mbarrier gives up after a number
// of polls, writes kErrWait to the error word, raises the block's abort flag and leaves through
// the common exit.  No correct launch reaches that branch, so this kernel does: one block sets up
// a barrier that nobody arrives at, waits for it with the same mbar_wait and a small limit, and
// reports exactly as the product kernels do.  It ends by itself after `limit` polls; nothing
// hangs and the context stays usable.
#include "tcgen05_utils.cuh"

namespace tk {

__global__ void wait_probe_kernel(unsigned limit, int* err) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  const uint32_t bar_addr = gt_smem_u32(&bar);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(bar_addr, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!mbar_wait(bar_addr, 0, &abort_flag, limit)) {
      set_error(err, kErrWait, (int)blockIdx.x, 0, (int)limit);
      abort_flag = 1;
    }
  }
  __syncthreads();
}

}  // namespace tk

TK_API int tk_wait_probe(unsigned limit, int* err, cudaStream_t stream) {
  if (limit == 0 || limit > (1u << 16)) return (int)cudaErrorInvalidValue;   // a probe stays short
  tk::wait_probe_kernel<<<1, 32, 0, stream>>>(limit, err);
  return (int)cudaGetLastError();
}
