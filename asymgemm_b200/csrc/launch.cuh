// Host-side launch interface between the C ABI (capi.cu) and the per-dtype kernel instantiations.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include "mgrouped_kernel.cuh"

namespace agb {

constexpr int kBlockN = 128;   // output columns per item
constexpr int kStagesA = 4;    // activation ring depth (16 KB stages)
constexpr int kStagesB = 8;    // weight ring depth (16 KB stages): 128 KB of host reads in flight per CTA

// One instantiation per dtype lives in its own translation unit (inst_*.cu).
#define AGB_LAUNCH_ARGS int grid, cudaStream_t stream, const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &ms, const GemmParams &p
cudaError_t launch_bf16(AGB_LAUNCH_ARGS);
cudaError_t launch_fp8(AGB_LAUNCH_ARGS);
cudaError_t launch_int8(AGB_LAUNCH_ARGS);

template <Kind KIND>
cudaError_t launch_kind_impl(int grid, cudaStream_t stream, const CUtensorMap& ma, const CUtensorMap& mb,
                             const CUtensorMap& ms, const GemmParams& p) {
  using L = SmemLayout<kBlockN, kStagesA, kStagesB>;
  auto kernel = mgrouped_gemm_kernel<KIND, kBlockN, kStagesA, kStagesB>;
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::dyn_bytes);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  kernel<<<grid, NUM_THREADS, L::dyn_bytes, stream>>>(ma, mb, ms, p);
  return cudaGetLastError();
}

inline cudaError_t launch_mgrouped(int kind, int grid, cudaStream_t stream, const CUtensorMap& ma, const CUtensorMap& mb,
                                   const CUtensorMap& ms, const GemmParams& p) {
  switch (kind) {
    case 0: return launch_bf16(grid, stream, ma, mb, ms, p);
    case 1: return launch_fp8(grid, stream, ma, mb, ms, p);
    case 2: return launch_int8(grid, stream, ma, mb, ms, p);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace agb
