// Copy-only reference for the host link: a persistent kernel that streams a pinned host buffer into shared memory
// with the same TMA access pattern as the grouped GEMM's weight producer (each CTA owns a column of `box_rows` rows
// and walks K in 128-byte swizzled boxes) and discards the data. Its rate is the ceiling for SM-issued reads of
// pinned memory on a given machine, to be read next to the copy-engine rate of ag_measure_host_link.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <cstring>

#include "../../include/asymgemm_b200.h"
#include "mgrouped_kernel.cuh"

int agb_fail(int code, const char* message);

namespace agb {

constexpr int kStreamStages = 8;

__global__ void __launch_bounds__(128) host_stream_kernel(const __grid_constant__ CUtensorMap map, int k_boxes, long long n_tiles,
                                                          int box_rows, int boxes_per_stage, int* status, unsigned long long timeout_ns) {
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t full[kStreamStages];
  __shared__ int abort_flag;
  const uint32_t box_bytes = 128u * box_rows;
  const uint32_t stage_bytes = box_bytes * boxes_per_stage;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStreamStages; ++s) mbar_init(&full[s], 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  const WaitCtx wc{status, &abort_flag, timeout_ns};
  long long issued = 0;
  bool ok = true;
  const int k_groups = (k_boxes + boxes_per_stage - 1) / boxes_per_stage;
  for (long long nt = blockIdx.x; nt < n_tiles && ok; nt += gridDim.x) {
    for (int kg = 0; kg < k_groups && ok; ++kg, ++issued) {
      const int s = static_cast<int>(issued % kStreamStages);
      if (issued >= kStreamStages) ok = wait_bar(&full[s], ((issued / kStreamStages) - 1) & 1, wc, ST_TIMEOUT_B_FULL);
      if (!ok) break;
      mbar_arrive_expect_tx(&full[s], stage_bytes);
      for (int b = 0; b < boxes_per_stage; ++b)
        tma_load_2d(smem + s * stage_bytes + b * box_bytes, &map, &full[s], (kg * boxes_per_stage + b) * 128, static_cast<int>(nt * box_rows));
    }
  }
  const long long first = issued > kStreamStages ? issued - kStreamStages : 0;
  for (long long i = first; i < issued; ++i) wait_bar(&full[i % kStreamStages], (i / kStreamStages) & 1, wc, ST_TIMEOUT_DRAIN, false);
}

}  // namespace agb

extern "C" int ag_measure_host_stream(uint64_t bytes, int64_t row_bytes, int32_t box_rows, int32_t boxes_per_stage, int32_t num_ctas,
                                      int32_t reps, double* gbps_out) {
  if (gbps_out == nullptr || bytes == 0 || row_bytes <= 0 || row_bytes % 128 != 0 || box_rows <= 0 || box_rows > 256 || boxes_per_stage <= 0 ||
      128 * box_rows * boxes_per_stage > 24 * 1024)
    return agb_fail(AG_E_INVALID, "bad arguments (row_bytes % 128 == 0, box_rows <= 256, stage <= 24 KB)");
  void* fn_p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn_p, cudaEnableDefault, &q) != cudaSuccess || fn_p == nullptr)
    return agb_fail(AG_E_CUDA, "cuTensorMapEncodeTiled is not available");
  auto encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn_p);
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = num_ctas > 0 && num_ctas < sms ? num_ctas : sms;
  uint64_t rows = bytes / row_bytes;
  rows -= rows % box_rows;
  if (rows == 0) return agb_fail(AG_E_INVALID, "buffer smaller than one box");
  void* h = nullptr;
  int* status = nullptr;
  if (cudaHostAlloc(&h, rows * row_bytes, cudaHostAllocDefault) != cudaSuccess) return agb_fail(AG_E_CUDA, "cudaHostAlloc failed");
  std::memset(h, 1, rows * row_bytes);
  if (cudaMalloc(&status, sizeof(int)) != cudaSuccess) { cudaFreeHost(h); return agb_fail(AG_E_CUDA, "cudaMalloc failed"); }
  cudaMemset(status, 0, sizeof(int));
  void* hd = nullptr;
  cudaHostGetDevicePointer(&hd, h, 0);
  CUtensorMap map;
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(row_bytes), rows};
  cuuint64_t gstr[1] = {static_cast<cuuint64_t>(row_bytes)};
  cuuint32_t box[2] = {128, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  int rc = AG_OK;
  if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, hd, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
    rc = agb_fail(AG_E_CUDA, "cuTensorMapEncodeTiled failed");
  } else {
    const size_t smem = static_cast<size_t>(128) * box_rows * boxes_per_stage * agb::kStreamStages + 1024;
    cudaFuncSetAttribute(agb::host_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    double best = 0;
    for (int r = 0; r < (reps > 0 ? reps : 3) + 1; ++r) {
      cudaEventRecord(e0, 0);
      agb::host_stream_kernel<<<grid, 128, smem, 0>>>(map, static_cast<int>(row_bytes / 128), static_cast<long long>(rows / box_rows), box_rows,
                                                      boxes_per_stage, status, 2000000000ull);
      cudaEventRecord(e1, 0);
      cudaEventSynchronize(e1);
      float ms = 0;
      cudaEventElapsedTime(&ms, e0, e1);
      if (r > 0 && ms > 0) best = best > rows * row_bytes / (ms * 1e6) ? best : rows * row_bytes / (ms * 1e6);
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    int st = 0;
    cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) rc = agb_fail(AG_E_CUDA, cudaGetErrorString(e));
    else if (st != 0) rc = agb_fail(AG_E_DEVICE, "host stream kernel reported a wait that ran out");
    *gbps_out = best;
  }
  cudaFree(status);
  cudaFreeHost(h);
  return rc;
}
