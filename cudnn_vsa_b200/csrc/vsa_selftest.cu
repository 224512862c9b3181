// Self-test of the bounded-wait path that every tcgen05 kernel of this library shares: a wait on
// an mbarrier that nothing will ever complete, with a caller-chosen limit.  The kernel must give
// up, record `100 + site` in the status word, let the other threads of the CTA drain, and return
// - leaving the context usable.  Nothing here faults, traps or spins without a bound.
#include "../../include/vsa_b200.h"
#include "vsa_common.cuh"

namespace vsa {
namespace {

constexpr int kSelftestSite = 77;

__global__ void wait_timeout_kernel(int* status, long long limit_cycles) {
  __shared__ uint64_t never;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&never, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  // Thread 0 runs out of time; the others find the abort flag set and return at once.
  if (threadIdx.x == 0) mbar_wait_limit(&never, 0, &abort_flag, status, kSelftestSite, limit_cycles);
  __syncthreads();
  if (threadIdx.x != 0) mbar_wait_limit(&never, 0, &abort_flag, status, kSelftestSite + 1, limit_cycles);
}

}  // namespace
}  // namespace vsa

extern "C" int vsa_selftest_wait_timeout(int32_t* status, int64_t limit_cycles, void* stream) {
  if (status == nullptr || limit_cycles <= 0 || limit_cycles > vsa::kWaitCycles) return vsa::kBadArgument;
  vsa::wait_timeout_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status, limit_cycles);
  return cudaGetLastError() == cudaSuccess ? vsa::kOk : vsa::kCudaError;
}
