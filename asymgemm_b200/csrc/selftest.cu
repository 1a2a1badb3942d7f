// Self test of the bounded-wait machinery: a one-CTA kernel waits on an mbarrier that nothing ever arrives at.
// The wait must give up after `timeout_ms`, record ST_TIMEOUT_PROBE in the status word and return, leaving the context
// usable. This is how failure detection is exercised on a GPU without faulting, trapping or hanging it.
#include <cuda_runtime.h>

#include <vector>

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

// Issue-rate probe. `issuers` threads (warps 2 and 3) each run the issuer's inner sequence of the grouped-GEMM kernels --
// wait for an operand stage, four tcgen05.mma of M128 x N`n_cols` x K16 (bf16), commit to the stage's "empty" barrier --
// against a producer thread of their own that only arrives on the "full" barriers (no loads; the operands are whatever
// shared memory holds). What comes out is how many cycles a step costs when nothing but instruction issue and the tensor
// core itself is in the way: the figure the two-issuer design of the kernels rests on.
__global__ void __launch_bounds__(128, 1) mma_issue_probe_kernel(int steps, int issuers, int n_cols, long long* cycles, int* failed) {
  constexpr int STAGES = 2;   // per issuer
  extern __shared__ uint8_t probe_smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(probe_smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* smem_a = smem;                                   // 2 issuers x 2 stages x 16 KB
  uint8_t* smem_b = smem + 4 * 16384;                       // one 256-row weight stage
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 4 * 16384 + 32768);
  uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(bars + 16);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 12; ++i) mbar_init(&bars[i], 1);
    fence_mbar_init();
  }
  if (warp == 2) {
    tmem_alloc(tmem_base_smem, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_smem;
  auto spin = [&](uint64_t* bar, uint32_t parity) {        // bounded: about a second at the most
    for (uint32_t n = 0; n < (1u << 24); ++n)
      if (mbar_try_wait(bar, parity)) return true;
    atomicExch(failed, 1);
    return false;
  };
  if (lane == 0 && warp < 2 && warp < issuers) {             // producer of issuer `warp`
    uint64_t* full = bars + warp * 4, *empty = full + STAGES;
    bool ok = true;
    for (int g = 0; g < steps && ok; ++g) {
      ok = spin(&empty[g % STAGES], ((g / STAGES) & 1) ^ 1);
      mbar_arrive(&full[g % STAGES]);
    }
  } else if (lane == 0 && warp >= 2 && warp - 2 < issuers) {
    const int t = warp - 2;
    uint64_t* full = bars + t * 4, *empty = full + STAGES, *done = bars + 8 + t;
    const uint32_t idesc = make_idesc(1, 1, static_cast<uint32_t>(n_cols));
    const uint64_t a_desc0 = make_kmajor_sw128_desc(smem_u32(smem_a + t * STAGES * 16384));
    const uint64_t b_desc = make_kmajor_sw128_desc(smem_u32(smem_b));
    const long long t0 = clock64();
    bool ok = true;
    for (int g = 0; g < steps && ok; ++g) {
      const int s = g % STAGES;
      ok = spin(&full[s], (g / STAGES) & 1);
      if (!ok) break;
      tc_fence_after_sync();
      const uint64_t a_desc = a_desc0 + static_cast<uint64_t>((s * 16384) >> 4);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        umma<MmaKind::F16>(tmem_base + t * 256, a_desc + static_cast<uint64_t>(j * 2), b_desc + static_cast<uint64_t>(j * 2), idesc, (g > 0 || j > 0));
      umma_commit(&empty[s]);
    }
    umma_commit(done);
    if (ok) ok = spin(done, 0);
    cycles[blockIdx.x * 2 + t] = ok ? clock64() - t0 : -1;
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 2) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace agb

extern "C" int ag_probe_mma_issue(int32_t issuers, int32_t n_cols, int32_t steps, double* cycles_per_step) {
  if (cycles_per_step == nullptr) return agb_fail(AG_E_INVALID, "cycles_per_step is NULL");
  if (issuers < 1 || issuers > 2 || (n_cols != 128 && n_cols != 256) || steps < 16 || steps > (1 << 20))
    return agb_fail(AG_E_INVALID, "issuers must be 1 or 2, n_cols 128 or 256, steps 16 .. 2^20");
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return agb_fail(AG_E_CUDA, "could not query the device");
  long long* cycles = nullptr;
  int* failed = nullptr;
  const size_t smem_bytes = 4 * 16384 + 32768 + 256 + 1024;
  cudaError_t e = cudaMalloc(&cycles, sizeof(long long) * 2 * sms);
  if (e == cudaSuccess) e = cudaMalloc(&failed, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(cycles, 0, sizeof(long long) * 2 * sms);
  if (e == cudaSuccess) e = cudaMemset(failed, 0, sizeof(int));
  if (e == cudaSuccess) e = cudaFuncSetAttribute(agb::mma_issue_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_bytes));
  std::vector<long long> host(2 * static_cast<size_t>(sms), 0);
  int host_failed = 0;
  if (e == cudaSuccess) {
    agb::mma_issue_probe_kernel<<<sms, 128, smem_bytes>>>(steps, issuers, n_cols, cycles, failed);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(host.data(), cycles, sizeof(long long) * 2 * sms, cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaMemcpy(&host_failed, failed, sizeof(int), cudaMemcpyDeviceToHost);
  cudaFree(cycles);
  cudaFree(failed);
  if (e != cudaSuccess) return agb_fail(AG_E_CUDA, cudaGetErrorString(e));
  long long worst = 0;
  for (long long c : host) {
    if (c < 0) host_failed = 1;
    worst = c > worst ? c : worst;
  }
  if (host_failed) return agb_fail(AG_E_DEVICE, "the issue-rate probe gave up waiting on one of its barriers");
  // every issuer took `steps` steps in `worst` cycles: the CTA finished issuers * steps steps in that time
  *cycles_per_step = static_cast<double>(worst) / (static_cast<double>(steps) * issuers);
  return AG_OK;
}

extern "C" int ag_selftest_wait_limit(uint32_t timeout_ms, int32_t* status, void* stream) {
  if (status == nullptr) return agb_fail(AG_E_INVALID, "status must be a device int32");
  if (timeout_ms == 0 || timeout_ms > 2000) return agb_fail(AG_E_INVALID, "timeout_ms must be in 1..2000");
  agb::wait_limit_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, static_cast<unsigned long long>(timeout_ms) * 1000000ull);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return agb_fail(AG_E_CUDA, cudaGetErrorString(e));
  return AG_OK;
}
