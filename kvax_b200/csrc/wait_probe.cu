// Self-test of the bounded mbarrier wait that every attention kernel uses: one warp waits on
// a barrier nobody arrives on, gives up after the given budget, records 100 + barrier id in
// the status word and runs to the end of the kernel.  Nothing traps and nothing spins
// without a limit, so the context stays usable; the host then reads the status word.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kvax_b200.h"
#include "ptx.cuh"

namespace {

__global__ void __launch_bounds__(32) wait_probe_kernel(int* status, int* done, unsigned long long budget_ns, int bar_id) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    kvx::mbar_init(&bar, 1);
    abort_flag = 0;
    kvx::mbar_fence_init();
  }
  __syncthreads();
  // Phase 0 of `bar` never completes.  The first lane whose budget runs out raises the abort
  // flag and writes the status; the others leave at their next look at the flag.
  const bool ok = kvx::mbar_wait_budget(&bar, 0, &abort_flag, status, bar_id, budget_ns);
  __syncthreads();
  if (threadIdx.x == 0) *reinterpret_cast<volatile int*>(done) = ok ? 1 : 2;
}

}  // namespace

extern "C" int kvax_b200_wait_probe(int32_t* status, int32_t* done, int64_t budget_ns, int32_t bar_id,
                                    kvax_b200_stream_t stream) {
  if (!status || !done || bar_id < 0) return KVAX_B200_EINVAL;
  if (budget_ns < 1000) budget_ns = 1000;
  if (budget_ns > 100000000ll) budget_ns = 100000000ll;
  wait_probe_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status, done, (unsigned long long)budget_ns, bar_id);
  return cudaGetLastError() == cudaSuccess ? KVAX_B200_OK : KVAX_B200_ELAUNCH;
}
