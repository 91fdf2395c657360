// Self-test of the bounded-wait machinery every pipeline kernel of this library relies on.
//
// The GEMM and attention kernels wait on mbarriers with a poll limit; when a wait runs out the
// waiter raises the CTA's abort flag, every role leaves its loop, a bit is OR-ed into the device
// status word, tensor memory is released and the kernel returns -- the context stays usable and
// the host learns of it through oasr_b200_device_status.  In a healthy run none of that code ever
// executes.  This kernel makes it execute on purpose and harmlessly: a consumer waits, with a
// short poll limit, on a barrier that nothing ever arrives on, while a second role waits on a
// barrier that the first one would have signalled.  Nothing faults, traps or spins without bound.
#include "common.cuh"
#include "device_status.cuh"
#include "sm100_ptx.cuh"

namespace ob {
namespace {

__global__ void __launch_bounds__(96) bounded_wait_selftest_kernel(uint32_t poll_limit, uint32_t* status,
                                                                   uint32_t* report) {
  __shared__ __align__(8) uint64_t never_bar;   // no arrival is ever made on this barrier
  __shared__ __align__(8) uint64_t chained_bar; // would be signalled by the role that waits on never_bar
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t abort_word;
  volatile uint32_t* abort_flag = &abort_word;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&never_bar, 1);
    ptx::mbar_init(&chained_bar, 1);
    abort_word = 0;
    ptx::fence_barrier_init();
  }
  if (warp == 1) {               // the same TMEM life cycle as the pipelines: allocate, use nothing, release at the end
    ptx::tmem_alloc(&tmem_slot, 32);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  uint32_t gave_up = 0;
  if (warp == 0 && lane == 0) {
    // role A: its wait runs out after poll_limit polls and raises the abort flag
    if (!ptx::mbar_wait_limited(&never_bar, 0, abort_flag, poll_limit)) gave_up = 1;
    else ptx::mbar_arrive(&chained_bar);
  } else if (warp == 2 && lane == 0) {
    // role B: has the full limit of a production wait, but leaves as soon as it sees role A's abort flag
    if (!ptx::mbar_wait(&chained_bar, 0, abort_flag)) gave_up = 2;
  }
  __syncthreads();
  if (gave_up && status) atomicOr(status, kStatusSelfTest);
  if (gave_up && report) atomicOr(report, gave_up);
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, 32);
  }
}

}  // namespace
}  // namespace ob

extern "C" {

int oasr_b200_selftest_bounded_wait(int64_t poll_limit, uint32_t* report, void* stream) {
  using namespace ob;
  OB_REQUIRE(poll_limit >= 64 && poll_limit <= (int64_t(1) << 20), OASR_ERR_INVALID,
             "selftest_bounded_wait: poll limit must be in [64, 2^20] (got %lld)", (long long)poll_limit);
  bounded_wait_selftest_kernel<<<1, 96, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint32_t>(poll_limit),
                                                                                device_status_ptr(), report);
  return check_launch("bounded-wait self-test launch");
}

}  // extern "C"
