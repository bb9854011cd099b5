// Self-test entry points: exercise the error-handling paths of the library without provoking a fault.
#include "tcgen05.cuh"

namespace q3 {
namespace tc {

// Two warps wait on an mbarrier that nothing ever arrives at. Warp 0's wait runs out after `limit_ns` and raises the
// CTA-wide abort flag; warp 1 waits with the library's normal (2 s) limit and must leave through that flag, as the
// other roles of a real kernel do. Then the CTA reports and returns like every kernel here: no trap, no hang.
__global__ void wait_timeout_probe_kernel(uint64_t limit_ns, int* status, int* outcome) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_barrier_init();
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5;
  const bool ok = warp == 0 ? mbar_wait(smem_u32(&bar), 0, &abort_flag, limit_ns)
                            : mbar_wait(smem_u32(&bar), 0, &abort_flag);
  __syncthreads();
  if ((threadIdx.x & 31) == 0 && outcome) outcome[warp] = ok ? 1 : 0;   // 0 = this warp's wait gave up
  if (threadIdx.x == 0 && abort_flag) flag_status(status, Q3_STATUS_WAIT_TIMEOUT);
}

}  // namespace tc
}  // namespace q3

using namespace q3;

extern "C" int q3_selftest_wait_timeout(int64_t limit_ns, int* status, int* outcome, q3_stream_t stream) {
  if (!status) return Q3_ERR_ARG;
  if (limit_ns < 1000 || limit_ns > 100000000) return Q3_ERR_SHAPE;   // 1 us .. 100 ms
  tc::wait_timeout_probe_kernel<<<1, 64, 0, (cudaStream_t)stream>>>((uint64_t)limit_ns, status, outcome);
  return launch_status();
}
