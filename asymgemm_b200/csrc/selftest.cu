// Self test of the bounded-wait machinery: a one-CTA kernel waits on an mbarrier that nothing ever arrives at.
// The wait must give up after `timeout_ms`, record ST_TIMEOUT_PROBE in the status word and return, leaving the context
// usable. This is how failure detection is exercised on a GPU without faulting, trapping or hanging it.
#include <cuda_runtime.h>

#include "../../include/asymgemm_b200.h"
#include "mgrouped_kernel.cuh"

int agb_fail(int code, const char* message);

namespace agb {

__global__ void wait_limit_probe_kernel(int* status, unsigned long long timeout_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const WaitCtx wc{status, &abort_flag, timeout_ns};
  // every lane polls, as the TMEM-drain warps do; nobody arrives, so all lanes must come back with `false`
  const bool ok = wait_bar(&bar, 0, wc, ST_TIMEOUT_PROBE);
  if (ok) atomicExch(status, 0x7fffff00 | ST_TIMEOUT_PROBE);  // impossible: would mean the wait was satisfied
}

}  // namespace agb

extern "C" int ag_selftest_wait_limit(uint32_t timeout_ms, int32_t* status, void* stream) {
  if (status == nullptr) return agb_fail(AG_E_INVALID, "status must be a device int32");
  if (timeout_ms == 0 || timeout_ms > 2000) return agb_fail(AG_E_INVALID, "timeout_ms must be in 1..2000");
  agb::wait_limit_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, static_cast<unsigned long long>(timeout_ms) * 1000000ull);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return agb_fail(AG_E_CUDA, cudaGetErrorString(e));
  return AG_OK;
}
