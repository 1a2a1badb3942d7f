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


// ------------------------------------------------------------------------------------------------- sustained link probe
// A measurement in three steps so that several GPUs (ranks of one job, or threads of one process) can be timed while they
// really stream at the same time: create (allocate and touch the pinned buffer, allocate the device side, build the
// tensor map -- the slow, unevenly long part), then a barrier of the caller's, then run (stream for at least
// `min_seconds`, report the mean), then destroy.
struct ag_link_probe {
  int device = 0;
  int mode = 0;               // 0 = copy engine (cudaMemcpyAsync pinned -> device), 1 = SM-issued TMA reads (host_stream_kernel)
  uint64_t bytes = 0;
  void* host = nullptr;
  void* dev = nullptr;
  int* status = nullptr;
  cudaStream_t stream = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  CUtensorMap map;
  int64_t row_bytes = 0;
  uint64_t rows = 0;
  int grid = 0;
  size_t smem = 0;
};

namespace {
constexpr int kProbeBoxRows = 64, kProbeBoxesPerStage = 2;

cudaError_t probe_pass(ag_link_probe* p) {
  if (p->mode == 0) return cudaMemcpyAsync(p->dev, p->host, p->bytes, cudaMemcpyHostToDevice, p->stream);
  agb::host_stream_kernel<<<p->grid, 128, p->smem, p->stream>>>(p->map, static_cast<int>(p->row_bytes / 128),
                                                               static_cast<long long>(p->rows / kProbeBoxRows), kProbeBoxRows,
                                                               kProbeBoxesPerStage, p->status, 2000000000ull);
  return cudaGetLastError();
}
}  // namespace

extern "C" int ag_link_probe_create(int32_t device, uint64_t bytes, int32_t mode, int64_t row_bytes, ag_link_probe_t** out) {
  if (out == nullptr || bytes < (1u << 20) || (mode != 0 && mode != 1)) return agb_fail(AG_E_INVALID, "bad arguments (bytes >= 1 MiB, mode 0 or 1)");
  if (mode == 1 && (row_bytes <= 0 || row_bytes % 128 != 0)) return agb_fail(AG_E_INVALID, "mode 1 needs row_bytes % 128 == 0");
  *out = nullptr;
  int dev = device;
  if (dev < 0) {
    if (cudaGetDevice(&dev) != cudaSuccess) return agb_fail(AG_E_CUDA, "cudaGetDevice failed");
  } else if (cudaSetDevice(dev) != cudaSuccess) {
    cudaGetLastError();
    return agb_fail(AG_E_CUDA, "cudaSetDevice failed");
  }
  ag_link_probe* p = new ag_link_probe();
  p->device = dev;
  p->mode = mode;
  auto bail = [&](int code, const char* msg) {
    ag_link_probe_destroy(p);
    cudaGetLastError();
    return agb_fail(code, msg);
  };
  if (mode == 1) {
    p->row_bytes = row_bytes;
    p->rows = bytes / row_bytes;
    p->rows -= p->rows % kProbeBoxRows;
    if (p->rows == 0) return bail(AG_E_INVALID, "buffer smaller than one box");
    p->bytes = p->rows * row_bytes;
  } else {
    p->bytes = bytes;
  }
  if (cudaHostAlloc(&p->host, p->bytes, cudaHostAllocPortable) != cudaSuccess) return bail(AG_E_CUDA, "cudaHostAlloc failed");
  std::memset(p->host, 1, p->bytes);
  if (cudaStreamCreateWithFlags(&p->stream, cudaStreamNonBlocking) != cudaSuccess || cudaEventCreate(&p->e0) != cudaSuccess ||
      cudaEventCreate(&p->e1) != cudaSuccess)
    return bail(AG_E_CUDA, "could not create the probe's stream and events");
  if (mode == 0) {
    if (cudaMalloc(&p->dev, p->bytes) != cudaSuccess) return bail(AG_E_CUDA, "cudaMalloc failed");
  } else {
    void* fn_p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn_p, cudaEnableDefault, &q) != cudaSuccess || fn_p == nullptr)
      return bail(AG_E_CUDA, "cuTensorMapEncodeTiled is not available");
    auto encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn_p);
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    p->grid = sms;
    if (cudaMalloc(&p->status, sizeof(int)) != cudaSuccess) return bail(AG_E_CUDA, "cudaMalloc failed");
    cudaMemsetAsync(p->status, 0, sizeof(int), p->stream);
    void* hd = nullptr;
    cudaHostGetDevicePointer(&hd, p->host, 0);
    cuuint64_t gdim[2] = {static_cast<cuuint64_t>(row_bytes), p->rows};
    cuuint64_t gstr[1] = {static_cast<cuuint64_t>(row_bytes)};
    cuuint32_t box[2] = {128, static_cast<cuuint32_t>(kProbeBoxRows)};
    cuuint32_t estr[2] = {1, 1};
    if (encode(&p->map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, hd, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return bail(AG_E_CUDA, "cuTensorMapEncodeTiled failed");
    p->smem = static_cast<size_t>(128) * kProbeBoxRows * kProbeBoxesPerStage * agb::kStreamStages + 1024;
    if (cudaFuncSetAttribute(agb::host_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(p->smem)) != cudaSuccess)
      return bail(AG_E_CUDA, "cudaFuncSetAttribute failed");
  }
  // one untimed pass: first-touch costs of the mapping stay out of the measurement
  if (probe_pass(p) != cudaSuccess || cudaStreamSynchronize(p->stream) != cudaSuccess) return bail(AG_E_CUDA, "the probe's warm-up pass failed");
  *out = p;
  return AG_OK;
}

extern "C" int ag_link_probe_run(ag_link_probe_t* p, double min_seconds, double* gbps_mean) {
  if (p == nullptr || gbps_mean == nullptr || !(min_seconds > 0) || min_seconds > 30) return agb_fail(AG_E_INVALID, "bad arguments (0 < min_seconds <= 30)");
  if (cudaSetDevice(p->device) != cudaSuccess) return agb_fail(AG_E_CUDA, "cudaSetDevice failed");
  // Passes are queued a few at a time and the clock is read in between, so that the stream never runs dry and the run
  // ends soon after `min_seconds`; the mean is all bytes over the time from the first pass's start to the last one's end.
  double total_ms = 0;
  uint64_t passes = 0;
  cudaError_t e = cudaEventRecord(p->e0, p->stream);
  while (e == cudaSuccess && total_ms < min_seconds * 1e3 && passes < 100000) {
    for (int i = 0; i < 2 && e == cudaSuccess; ++i, ++passes) e = probe_pass(p);
    if (e != cudaSuccess) break;
    e = cudaEventRecord(p->e1, p->stream);
    if (e == cudaSuccess) e = cudaEventSynchronize(p->e1);
    float ms = 0;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, p->e0, p->e1);
    total_ms = ms;
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return agb_fail(AG_E_CUDA, cudaGetErrorString(e));
  }
  if (p->mode == 1) {
    int st = 0;
    cudaMemcpyAsync(&st, p->status, sizeof(int), cudaMemcpyDeviceToHost, p->stream);
    cudaStreamSynchronize(p->stream);
    if (st != 0) return agb_fail(AG_E_DEVICE, "host stream kernel reported a wait that ran out");
  }
  *gbps_mean = total_ms > 0 ? static_cast<double>(passes) * static_cast<double>(p->bytes) / (total_ms * 1e6) : 0.0;
  return AG_OK;
}

extern "C" int ag_link_probe_destroy(ag_link_probe_t* p) {
  if (p == nullptr) return AG_OK;
  cudaSetDevice(p->device);
  if (p->stream) cudaStreamSynchronize(p->stream);
  if (p->e0) cudaEventDestroy(p->e0);
  if (p->e1) cudaEventDestroy(p->e1);
  if (p->stream) cudaStreamDestroy(p->stream);
  if (p->dev) cudaFree(p->dev);
  if (p->status) cudaFree(p->status);
  if (p->host) cudaFreeHost(p->host);
  delete p;
  cudaGetLastError();
  return AG_OK;
}
