// ag_m_grouped_fp8_gemm_nt_static_scratch: the FP8 grouped GEMM for callers that must not allocate device memory.
//
// Who needs this. Some hosts of this library run with a device-memory budget that is handed out once at start-up --
// a serving process whose arena owns all of HBM, a plugin loaded into another runtime through FFI that has no CUDA
// allocator of its own, a latency-critical loop where a cudaMalloc (which synchronises the device and may fail when
// memory is nearly full) is not acceptable. Such callers can pass inputs and outputs they already own, but they have
// nowhere to get the scratch buffer that long segments use to replay their weight column (see ag_scratch_bytes).
// This entry point brings its own: a fixed array in the library's device image.
//
// The price: the array (kStaticScratchBytes) is part of the module, so every GPU that loads this library holds it until
// the process exits; problems that need more scratch are rejected; and all calls share the one array, so two calls
// that may run on the GPU at the same time (different streams, or different host threads) race on it. Nothing in the
// array has to be cleared between calls: every byte the kernel reads from it was written earlier in the same launch;
// the array simply keeps whatever the last call left there.
//
// Set-up happens inside the first call on each device (with that device current): the device address of the array is
// looked up once with cudaGetSymbolAddress and remembered. Make that first call outside any stream capture.
// The entry point itself calls no cudaMalloc / cudaFree and no allocating library routine; it requires the caller's
// `status` word because the shared default one is allocated on first use by the other entry points.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "../../include/asymgemm_b200.h"
#include "launch.cuh"

// internal hooks exported by capi.cu
int agb_run_desc(int kind, const ag_gemm_desc_t* desc);
int agb_scratch_need(int kind, const ag_gemm_desc_t* desc, uint64_t* out);
int agb_fail(int code, const char* message);

namespace {

constexpr unsigned long long kStaticScratchBytes = 80ull << 20;  // 80 MiB per GPU that loads the library

// In host code this name is only a handle for cudaGetSymbolAddress; it is never passed to a kernel directly.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_mu;
void* g_scratch_dev[64] = {};

// Device address of the array on the current device, looked up on first use.
int scratch_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) return agb_fail(AG_E_CUDA, "cudaGetDevice failed or device index out of range");
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_scratch_dev[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      char msg[160];
      snprintf(msg, sizeof(msg), "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
      return agb_fail(AG_E_CUDA, msg);
    }
    g_scratch_dev[dev] = ptr;
  }
  *out = g_scratch_dev[dev];
  return AG_OK;
}

}  // namespace

extern "C" {

uint64_t ag_static_scratch_bytes(void) { return kStaticScratchBytes; }

int ag_m_grouped_fp8_gemm_nt_static_scratch(const ag_gemm_desc_t* desc) {
  if (desc == nullptr) return agb_fail(AG_E_INVALID, "desc is NULL");
  if (desc->status == nullptr)
    return agb_fail(AG_E_INVALID, "the static-scratch entry point needs a caller-owned status word (desc->status): "
                                  "it may not allocate the default one");
  if (desc->n <= 0 || desc->k <= 0 || desc->num_groups <= 0 || desc->b == nullptr)
    return agb_fail(AG_E_INVALID, "n, k, num_groups must be positive and b non-NULL");

  void* base = nullptr;
  if (int rc = scratch_address(&base)) return rc;
  // the grouped GEMM wants 1024-byte alignment; the array only promises 256
  const uintptr_t aligned = (reinterpret_cast<uintptr_t>(base) + 1023) & ~static_cast<uintptr_t>(1023);
  const uint64_t usable = kStaticScratchBytes - (aligned - reinterpret_cast<uintptr_t>(base));

  // Scratch this launch would use, from the same arithmetic as the launch itself: one weight column (tile rows x padded K
  // bytes) per CTA when the weights stream from the host (or with no_split); nothing when device-resident weights are
  // cut into one-chunk items, which never replay.
  uint64_t need = 0;
  if (int rc = agb_scratch_need(1, desc, &need)) return rc;
  if (need > usable) {
    char msg[320];
    snprintf(msg, sizeof(msg),
             "this problem needs %llu bytes of scratch (CTAs x tile rows x padded K bytes) but the built-in scratch holds %llu: "
             "lower num_sms, pick a narrower tile_config, or use ag_m_grouped_fp8_gemm_nt with caller-provided scratch",
             static_cast<unsigned long long>(need), static_cast<unsigned long long>(usable));
    return agb_fail(AG_E_INVALID, msg);
  }

  ag_gemm_desc_t g = *desc;
  g.scratch = reinterpret_cast<void*>(aligned);
  g.scratch_bytes = usable;
  g.stage = nullptr;  // staging would create a stream and events on first use: this entry point reads b in the kernel
  g.stage_bytes = 0;
  g.stage_chunk_bytes = 0;
  return agb_run_desc(1, &g);
}

}  // extern "C"
