// kb_selftest_wait_timeout: runs the kernels' bounded device-side wait to its limit, on purpose and
// harmlessly, so that the give-up path (status words, abort flag, clean return) can be tested on a GPU.
//
// Every wait of the tcgen05 kernels is sm100::mbar_wait, which polls an mbarrier a bounded number of
// times, then records {KB_ERR_DEVICE_TIMEOUT, wait site, block} in the caller's status words, raises the
// CTA's abort flag and returns false; the roles then leave their loops and the kernel ends normally.  In
// a correct pipeline that path never runs.  This kernel makes it run in the smallest possible setting:
// one CTA whose only mbarrier expects an arrival that nobody makes, no copy in flight, no TMEM held, and
// a limit of 1 024 polls (well under a millisecond) instead of the kernels' 2^22.  Nothing faults and
// nothing hangs: the wait runs out, the second warp sees the abort flag the first one raised, the kernel
// returns and the context stays usable.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace kb {
namespace {

using namespace sm100;

constexpr int kSelftestWaitSite = 900;
constexpr uint32_t kSelftestLimit = 1024;

__global__ void __launch_bounds__(64) wait_timeout_selftest_kernel(int32_t* status, int32_t* seen) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const WaitCtx ctx{&abort_flag, status};
  if (threadIdx.x == 0) {
    // phase 0 of a barrier nobody arrives on: gives up after kSelftestLimit polls
    const bool ok = mbar_wait<0, kSelftestLimit>(&bar, 0, ctx, kSelftestWaitSite);
    seen[0] = ok ? 1 : 0;
  }
  if (threadIdx.x == 32) {
    // a second role waiting on the same barrier with the kernels' own (long) limit: it must leave as soon as
    // the first role has raised the abort flag, not after its own 2^22 polls
    const bool ok = mbar_wait(&bar, 0, ctx, kSelftestWaitSite + 1);
    seen[1] = ok ? 1 : 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) seen[2] = abort_flag;
}

}  // namespace
}  // namespace kb

extern "C" int kb_selftest_wait_timeout(int32_t* status, int32_t* seen, void* stream) {
  if (!status || !seen) return KB_ERR_BAD_ARGUMENT;
  kb::wait_timeout_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status, seen);
  KB_LAUNCH_CHECK("wait_timeout_selftest_kernel");
  return KB_OK;
}
