// Self-test of the bounded-wait path: a one-warp kernel that waits on an
// mbarrier nothing ever arrives on, with a short iteration cap, and leaves
// through the same route a production kernel takes when its wait runs out (the
// status word is set, the kernel returns, the context stays usable). Nothing
// here hangs or faults: the wait is the ordinary bounded one with a small limit.
#include "common.cuh"
#include "kernels.h"
#include "svodb.h"

namespace svodb {
namespace {

__global__ void __launch_bounds__(32) wait_probe_kernel(uint32_t polls, uint32_t* status, uint32_t* gave_up) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncwarp();
  const bool ok = mbar_wait_for(&bar, 0, status, polls);
  if (threadIdx.x == 0 && gave_up != nullptr) *gave_up = ok ? 0u : 1u;
}

}  // namespace
}  // namespace svodb

extern "C" int svodb_selftest_wait_timeout(uint32_t polls, void* stream) {
  using namespace svodb;
  uint32_t* status = device_status_word();
  if (status == nullptr) {
    set_last_error("selftest_wait_timeout: no status word");
    return SVODB_ERR_LAUNCH;
  }
  if (polls == 0 || polls > (1u << 20)) {
    set_last_error("selftest_wait_timeout: polls must be in 1..2^20 (a short wait)");
    return SVODB_ERR_SHAPE;
  }
  wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(polls, status, nullptr);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("selftest_wait_timeout: %s", cudaGetErrorString(e));
    return SVODB_ERR_LAUNCH;
  }
  return SVODB_OK;
}
