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

// Operand-feed probe: the kernels' producer / issuer rings for 256-column bf16 items -- per 128-byte K atom one 256-row weight
// stage (32 KB) and two 128-row activation stages (16 KB each), two issuers with one row tile each, one producer lane per
// issuer -- with REAL TMA loads from device memory and nothing else (no drain, no item bookkeeping). Groups of six CTAs
// share activation rows and every sixth CTA shares weight rows, as CTAs of the grouped GEMM do through L2.
__global__ void __launch_bounds__(128, 1) operand_feed_probe_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                                                                     int items, int kb_count, int load_a, int load_b, int rows_a, int rows_b,
                                                                     long long* cycles, int* failed) {
  constexpr int SB = 4, PER = 2;   // weight ring; activation stages per issuer
  extern __shared__ uint8_t probe_smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(probe_smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + 2 * PER * 16384;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_b + SB * 32768);
  uint64_t* a_full = bars, *a_empty = bars + 4, *b_full = bars + 8, *b_empty = bars + 12, *done = bars + 16;
  uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(bars + 24);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; ++i) {
      mbar_init(&a_full[i], 1);
      mbar_init(&a_empty[i], 1);
      mbar_init(&b_full[i], 1);
      mbar_init(&b_empty[i], 2);
    }
    mbar_init(&done[0], 1);
    mbar_init(&done[1], 1);
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
  if (warp == 0 && lane == 0) {                               // weight producer
    bool ok = true;
    uint32_t jt = 0;
    for (int it = 0; it < items && ok; ++it) {
      const int b_row = ((it * 7 + static_cast<int>(blockIdx.x) % 6) % (rows_b / 256)) * 256;
      for (int kb = 0; kb < kb_count && ok; ++kb, ++jt) {
        const uint32_t s = jt % SB;
        ok = spin(&b_empty[s], ((jt / SB) & 1) ^ 1);
        if (!ok) break;
        if (load_b) {
          mbar_arrive_expect_tx(&b_full[s], 32768);
          tma_load_2d(smem_b + s * 32768, &tmap_b, &b_full[s], kb * ATOM_BYTES, b_row);
        } else {
          mbar_arrive(&b_full[s]);
        }
      }
    }
  } else if (warp == 1 && lane < 2) {                         // activation producers, one lane per issuer
    const int t = lane;
    bool ok = true;
    uint32_t used = 0;
    for (int it = 0; it < items && ok; ++it) {
      const int a_row = ((it * 25 + static_cast<int>(blockIdx.x) / 6) % (rows_a / 256)) * 256 + t * 128;
      for (int kb = 0; kb < kb_count && ok; ++kb, ++used) {
        const uint32_t s = t * PER + used % PER;
        ok = spin(&a_empty[s], ((used / PER) & 1) ^ 1);
        if (!ok) break;
        if (load_a) {
          mbar_arrive_expect_tx(&a_full[s], 16384);
          tma_load_2d(smem_a + s * 16384, &tmap_a, &a_full[s], kb * ATOM_BYTES, a_row);
        } else {
          mbar_arrive(&a_full[s]);
        }
      }
    }
  } else if ((warp == 2 || warp == 3) && lane == 0) {        // issuers: row tile 0 and row tile 1
    const int t = warp - 2;
    const uint32_t idesc = make_idesc(1, 1, 256);
    const uint64_t a_desc0 = make_kmajor_sw128_desc(smem_u32(smem_a)), b_desc0 = make_kmajor_sw128_desc(smem_u32(smem_b));
    const long long t0 = clock64();
    bool ok = true;
    uint32_t own = 0, jt = 0;
    for (int it = 0; it < items && ok; ++it) {
      for (int kb = 0; kb < kb_count && ok; ++kb, ++jt, ++own) {
        const uint32_t sb = jt % SB, sa = t * PER + own % PER;
        ok = spin(&b_full[sb], (jt / SB) & 1) && spin(&a_full[sa], (own / PER) & 1);
        if (!ok) break;
        tc_fence_after_sync();
        const uint64_t da = a_desc0 + static_cast<uint64_t>((sa * 16384) >> 4), db = b_desc0 + static_cast<uint64_t>((sb * 32768) >> 4);
#pragma unroll
        for (int j = 0; j < 4; ++j) umma<MmaKind::F16>(tmem_base + t * 256, da + static_cast<uint64_t>(j * 2), db + static_cast<uint64_t>(j * 2), idesc, (kb > 0 || j > 0));
        umma_commit(&a_empty[sa]);
        umma_commit(&b_empty[sb]);
      }
    }
    umma_commit(&done[t]);
    if (ok) ok = spin(&done[t], 0);
    cycles[blockIdx.x * 2 + t] = ok ? clock64() - t0 : -1;
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 2) tmem_dealloc(tmem_base, TMEM_COLS);
}

cudaError_t launch_operand_feed_probe(const CUtensorMap& ma, const CUtensorMap& mb, int sms, int items, int kb_count, int load_a, int load_b,
                                      int rows_a, int rows_b, long long* cycles, int* failed) {
  const size_t smem_bytes = 4 * 16384 + 4 * 32768 + 512 + 1024;
  cudaError_t e = cudaFuncSetAttribute(operand_feed_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_bytes));
  if (e != cudaSuccess) return e;
  operand_feed_probe_kernel<<<sms, 128, smem_bytes>>>(ma, mb, items, kb_count, load_a, load_b, rows_a, rows_b, cycles, failed);
  return cudaGetLastError();
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
