// A check of the bounded waits' give-up path: one thread waits, for a limit of at most ten
// milliseconds, on an mbarrier at which nobody ever arrives.  The wait runs out, the kernel records
// "a wait ran out" in the error record and returns as every kernel of this library does in that
// case: the context stays usable and the next launch works.  Nothing here spins without a bound.
#include "tcgen05_helpers.cuh"

namespace {
__global__ void wait_check_kernel(int* err, unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long bar;
  if (threadIdx.x == 0) {
    mbar_init(s2u(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned long long t0 = global_timer_ns();
    if (!mbar_wait(s2u(&bar), 0, limit_ns))
      dk_report(err, DK_DEV_TIMEOUT, (int)blockIdx.x, 9, (int)((global_timer_ns() - t0) / 1000));   // part 9, microseconds waited
  }
}
}  // namespace

extern "C" int dk_wait_check(int* err, long long limit_ns, cudaStream_t stream) {
  DK_REQUIRE(err != nullptr, "wait_check: no error record");
  DK_REQUIRE(limit_ns > 0 && limit_ns <= 10000000ll, "wait_check: the limit must lie in (0, 10 ms], got %lld ns", limit_ns);
  wait_check_kernel<<<1, 32, 0, stream>>>(err, (unsigned long long)limit_ns);
  return dk_check_launch("wait_check");
}
