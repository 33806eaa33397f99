// limn_b200_wait_probe: makes one bounded wait run out, on purpose and harmlessly, so that the give-up path
// every tensor-core kernel relies on can be exercised end to end: the status code, later launches standing
// down while the word is set, the work counters left at zero, the word read and cleared by
// limn_b200_device_status, and correct results afterwards.
//
// The probe is one warp. It initialises an mbarrier that expects one arrival, lets nobody arrive, and waits on
// it with the same mbar_wait_for the production kernels use, but with a budget of the caller's choosing (a few
// microseconds in the test) instead of seconds. When the budget runs out the wait returns false, having put
// 0x57410000 | tag into the current device's status word, and the kernel returns normally. Nothing hangs,
// nothing faults, and no production kernel is made to misbehave.
#include "common.h"
#include "sm100_ptx.cuh"

namespace limn_b200 {
namespace {

constexpr unsigned kProbeTag = 0x7e57u;

__global__ void wait_probe_kernel(unsigned* status, long long budget, unsigned* gave_up) {
  __shared__ __align__(8) unsigned long long barrier;
  const uint32_t bar = ptx::smem_addr(&barrier);
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar, 1u);
    ptx::mbar_init_fence();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const bool arrived = ptx::mbar_wait_for(bar, 0u, status, kProbeTag, budget);
    if (gave_up) *gave_up = arrived ? 0u : 1u;
  }
}

}  // namespace
}  // namespace limn_b200

using namespace limn_b200;

extern "C" int limn_b200_wait_probe(long long budget_ticks, unsigned int* gave_up, void* stream) {
  clear_error();
  if (budget_ticks < 0 || budget_ticks > 100000000LL)
    return fail(LIMN_B200_BAD_ARGUMENT, "wait_probe: the budget must be 0..1e8 clock ticks (a fraction of a second), got %lld",
                budget_ticks);
  unsigned int* word = nullptr;
  if (int rc = status_word(&word)) return rc;
  wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(word, budget_ticks, gave_up);
  LIMN_CUDA(cudaGetLastError(), "launching the wait probe");
  note_launches(1);
  return LIMN_B200_OK;
}
