// Self-test of the failure-detection chain: bounded wait -> status word -> host.
// The tensor-core kernels never spin without a limit: a wait that does not complete records
// (kernel id << 8 | site) in the handle's status word and the kernel returns normally, so the
// context stays usable.  This kernel makes such a wait run out on purpose, without any copy or
// MMA in flight: one CTA waits on an mbarrier nobody arrives at, with a limit of 2 ms.
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace etb {
namespace {

__global__ void selftest_wait_timeout_kernel(int* status_word, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  const uint32_t bar_addr = ptx::smem_u32(&bar);
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar_addr, 1);
    abort_flag = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // phase 0 never completes: there is no arrival
    if (!ptx::mbar_wait_ns(bar_addr, 0u, &abort_flag, limit_ns))
      report_timeout(status_word, kKernelSelfTest, 1);
  }
}

}  // namespace

cudaError_t launch_selftest_wait_timeout(int* status_word, cudaStream_t stream) {
  selftest_wait_timeout_kernel<<<1, 32, 0, stream>>>(status_word, 2000000ull);
  return cudaGetLastError();
}

}  // namespace etb
