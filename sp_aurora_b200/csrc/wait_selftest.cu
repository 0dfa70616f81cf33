// Self-test of the bounded device-side wait: one warp waits on an mbarrier that
// nothing ever arrives at. The wait must give up after its cycle budget, record
// {site, block, iteration} in the device status word and let the kernel return
// normally, which spa_check_status() then reports as SPA_ETIMEOUT. Nothing else
// is in flight in this kernel (no TMA, no MMA, no TMEM), so the expiry is exercised
// in isolation; the budget here is about a millisecond instead of the two seconds
// the attention kernels allow.
#define SPA_WAIT_BUDGET_CYCLES (2000000ll)
#include "spa_internal.h"
#include "tc05.cuh"

namespace spa {
namespace {

constexpr int kSelftestSite = 99;
constexpr int kSelftestIter = 7;

__global__ void wait_selftest_kernel(int* status, int* reached_exit) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  WaitCtx wc{status, &abort_flag};
  const bool ok = warp_wait(&bar, 0, wc, kSelftestSite, kSelftestIter);
  if (threadIdx.x == 0) *reached_exit = ok ? 2 : 1;   // 1: the wait gave up and the kernel went on
}

}  // namespace
}  // namespace spa

// Test hook (not part of include/spa.h). `reached_exit` is a device int the kernel sets to
// 1 when the wait expired and control reached the end of the kernel.
extern "C" int spa_internal_wait_selftest(int* reached_exit, void* stream) {
  int* st = spa::device_status_word();
  if (!st || !reached_exit) return SPA_EINVAL;
  spa::wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(st, reached_exit);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    spa::set_error("wait selftest launch: %s", cudaGetErrorString(e));
    return SPA_ECUDA;
  }
  return SPA_OK;
}
