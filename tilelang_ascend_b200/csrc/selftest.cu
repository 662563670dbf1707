// Self-test of the bounded-wait path that every tcgen05 kernel of the library relies on.
//
// All in-kernel waits of the library (mbar_wait in ptx.cuh) give up after a cycle budget, record
// kStatusBarrierTimeout in the device status word and let the kernel run to its normal end.  This kernel exercises
// exactly that path without faulting or hanging anything: one thread waits, with a caller-chosen short budget, on an
// mbarrier that nothing ever completes; the wait runs out, the status word is set, the kernel returns.
#include "params.h"
#include "ptx.cuh"

namespace dsa {

__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(int* status, long long budget_cycles, int* gave_up) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_init_fence();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const bool completed = mbar_wait(&bar, 0, status, budget_cycles);  // nobody arrives: the budget ends the wait
    if (gave_up) *gave_up = completed ? 0 : 1;
  }
}

int launch_bounded_wait_selftest(int* status, long long budget_cycles, int* gave_up, cudaStream_t stream) {
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(status, budget_cycles, gave_up);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace dsa
