// A bounded wait made to run out on purpose, the harmless way: one thread polls a flag in global memory that nothing
// ever raises, gives up after `limit_ns` (milliseconds in practice), records ERR_TEST_FLAG in the status word exactly as
// the production kernels record their own timeouts, and returns.  The context stays usable, the next launch on the
// stream runs normally, and the host sees the failure through the same status word it polls once per step.  This is
// how the "a peer never answered" path is exercised on a shared GPU: no trap, no failing assert, no endless loop.
#include "ptx_sm100.cuh"

namespace dttt {

__global__ void wait_selftest_kernel(const int* flag, int target, unsigned long long limit_ns, int* status, int* waited_us) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const uint64_t t0 = global_timer_ns();
  bool seen = false;
  // two limits: wall clock (the one that normally ends the wait) and an iteration count that ends it even if the timer
  // did not advance
  for (uint32_t spins = 0; spins < (1u << 24); ++spins) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v - target >= 0) { seen = true; break; }
    if (global_timer_ns() - t0 > limit_ns) break;
    __nanosleep(256);
  }
  if (!seen) atomicCAS(status, 0, ERR_TEST_FLAG);
  if (waited_us) *waited_us = (int)((global_timer_ns() - t0) / 1000ull);
}

}  // namespace dttt

// Wait (at most limit_ns, capped at 50 ms) until *flag >= target; on a timeout the status word becomes ERR_TEST_FLAG.
// waited_us (may be null) receives how long the kernel waited.
extern "C" int dttt_wait_selftest(const int* flag, int target, long long limit_ns, int* status, int* waited_us, cudaStream_t stream) {
  if (!flag || !status) return -2;
  if (limit_ns <= 0 || limit_ns > 50000000ll) limit_ns = 50000000ll;
  dttt::wait_selftest_kernel<<<1, 32, 0, stream>>>(flag, target, (unsigned long long)limit_ns, status, waited_us);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}
