// Expert-parallel token exchange over peer memory: routing, layout and both exchanges of an MoE layer as a handful of
// kernels that write rows straight into the owner rank's buffers with ordinary stores through peer-mapped pointers
// (NVLink / NVSwitch). Nothing here loads from another GPU's memory, nothing uses TMA or multicast on peer memory, and no
// kernel waits for another GPU: ranks meet at small stream-ordered collectives issued by the caller between the steps.
//
//   histogram (ids -> rows per expert)          caller all-gathers the counts of every rank
//   plan      (count matrix -> where every expert's rows start on its owner, this rank's segment table)
//   dispatch  (every (token, slot) pair's quantised row + scales + a return address -> the owner's padded layout)
//                                                caller: a collective, so that every rank's rows have landed
//   ... the two grouped GEMMs run on the rows where they landed ...
//   return    (every valid result row -> the pair's slot in its source rank's combine buffer)
//                                                caller: a collective, then the weighted top-k sum
//
// The reference's callers do the same steps with torch sort / bincount / index ops and all_gather + reduce_scatter
// (asym_gemm/unified_moe/runtime.py:1422-1476, asym_gemm/training/ep_vanilla.py:173-282).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

#include "../../include/asymgemm_b200.h"

int agb_fail(int code, const char* message);

namespace agb {

constexpr int kMaxRanks = 16;
constexpr int kPlanThreads = 256;

struct PeerTable {
  void* a[kMaxRanks];      // [cap_rows, row_bytes] quantised rows, in the owner's padded contiguous layout
  void* sfa[kMaxRanks];    // [cap_rows, sf_per_row] fp32 scales
  void* meta[kMaxRanks];   // [cap_rows] int64: (source rank << 32) | pair index, or -1 for rows nobody wrote
  void* ret[kMaxRanks];    // [pairs, ret_row_bytes] results, by pair index of the source rank
};

// counts[e] += 1 for every pair routed to expert e. ids is int64 [pairs]; one block-private histogram in shared memory.
__global__ void __launch_bounds__(256) ep_histogram_kernel(const long long* __restrict__ ids, long long pairs, int num_experts,
                                                           int* __restrict__ counts, int* __restrict__ status) {
  extern __shared__ int hist[];
  for (int i = threadIdx.x; i < num_experts; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  for (long long p = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; p < pairs; p += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = ids[p];
    if (e >= 0 && e < num_experts) atomicAdd(&hist[e], 1);
    else atomicCAS(status, 0, AG_EP_BAD_EXPERT);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < num_experts; i += blockDim.x)
    if (hist[i]) atomicAdd(&counts[i], hist[i]);
}

// One block. counts_all [world, E] (row s = rank s's histogram), range_lo [world + 1] (rank r owns experts
// [range_lo[r], range_lo[r+1])). Writes, for this rank `me`:
//   send_base [E]          row in the owner's layout where this rank's rows for expert e start
//   cursors [E]            zeroed (dispatch hands out slots with atomicAdd)
//   offsets [2 * epr_cap]  (start, start + valid rows) of every local expert; experts [epr_cap + 1] = 0 .. epr-1, -1
//   rows_used [2]          rows of the padded layout this rank uses, and its valid rows
//   meta of this rank's padding rows = -1 (peers only ever write valid rows)
__global__ void __launch_bounds__(kPlanThreads) ep_plan_kernel(const int* __restrict__ counts_all, const int* __restrict__ range_lo, int world,
                                                              int me, int num_experts, long long cap_rows, int* __restrict__ send_base,
                                                              int* __restrict__ cursors, int* __restrict__ offsets, int* __restrict__ experts,
                                                              int epr_cap, int* __restrict__ rows_used, long long* __restrict__ my_meta,
                                                              int* __restrict__ status) {
  extern __shared__ int sh[];
  int* total = sh;                    // [E] rows of expert e over all ranks
  int* before = sh + num_experts;     // [E] rows of expert e from ranks below `me`
  int* start = sh + 2 * num_experts;  // [E] first row of expert e in its owner's layout
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    int t = 0, b = 0;
    for (int s = 0; s < world; ++s) {
      const int c = counts_all[s * num_experts + e];
      if (s < me) b += c;
      t += c;
    }
    total[e] = t;
    before[e] = b;
  }
  __syncthreads();
  // every owner's layout: experts in order, each padded to 128 rows (thread r walks rank r's experts)
  for (int r = threadIdx.x; r < world; r += blockDim.x) {
    long long row = 0;
    for (int e = range_lo[r]; e < range_lo[r + 1]; ++e) {
      start[e] = static_cast<int>(row);
      row += (total[e] + 127) / 128 * 128;
    }
    if (row > cap_rows) atomicCAS(status, 0, AG_EP_OVERFLOW);
    if (r == me) {
      int valid = 0;
      for (int e = range_lo[r]; e < range_lo[r + 1]; ++e) valid += total[e];
      rows_used[0] = static_cast<int>(row < cap_rows ? row : cap_rows);
      rows_used[1] = valid;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    send_base[e] = start[e] + before[e];
    cursors[e] = 0;
  }
  const int lo = range_lo[me], epr = range_lo[me + 1] - lo;
  for (int j = threadIdx.x; j <= epr_cap; j += blockDim.x) {
    if (j < epr) {
      offsets[2 * j] = start[lo + j];
      offsets[2 * j + 1] = start[lo + j] + total[lo + j];
      experts[j] = j;
    } else {
      if (j < epr_cap) offsets[2 * j] = offsets[2 * j + 1] = 0;
      experts[j] = -1;
    }
  }
  // padding rows of this rank's layout carry no return address
  for (int j = 0; j < epr; ++j) {
    const int v = start[lo + j] + total[lo + j];
    const int end = start[lo + j] + (total[lo + j] + 127) / 128 * 128;
    for (long long r = v + threadIdx.x; r < end && r < cap_rows; r += blockDim.x) my_meta[r] = -1;
  }
}

// Warp-wide copy of one row of `vecs` 16-byte vectors, four loads in flight per lane before the stores go out: remote
// stores are posted, so the load latency is what has to be covered.
__device__ __forceinline__ void copy_row(const uint4* __restrict__ src, uint4* __restrict__ dst, int vecs, int lane) {
  int i = lane;
  for (; i + 96 < vecs; i += 128) {
    const uint4 v0 = src[i], v1 = src[i + 32], v2 = src[i + 64], v3 = src[i + 96];
    dst[i] = v0;
    dst[i + 32] = v1;
    dst[i + 64] = v2;
    dst[i + 96] = v3;
  }
  for (; i < vecs; i += 32) dst[i] = src[i];
}

__device__ __forceinline__ int owner_of(const int* range_lo, int world, int e) {
  int r = 0;
  while (r + 1 < world && e >= range_lo[r + 1]) ++r;
  return r;
}

// One warp per (token, slot) pair p: the token's quantised row, its scales and the pair's return address go to the next
// free row of its expert on the owner rank. Rows of one expert land in no particular order; every row's result is
// independent of its position, so the layer's output does not depend on that order.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const uint4* __restrict__ x_q, const float* __restrict__ sfx,
                                                          const long long* __restrict__ ids, long long pairs, int top_k, int vec_per_row,
                                                          int sf_per_row, const int* __restrict__ range_lo, int world, int me,
                                                          const int* __restrict__ send_base, int* __restrict__ cursors, long long cap_rows,
                                                          long long* __restrict__ pair_row, PeerTable peers) {
  __shared__ int lo[kMaxRanks + 1];
  if (threadIdx.x <= world) lo[threadIdx.x] = range_lo[threadIdx.x];
  __syncthreads();
  const long long p = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (p >= pairs) return;
  const int e = static_cast<int>(ids[p]);
  const int o = owner_of(lo, world, e);
  int slot = 0;
  if (lane == 0) slot = atomicAdd(&cursors[e], 1);
  slot = __shfl_sync(0xffffffffu, slot, 0);
  const long long dest = static_cast<long long>(send_base[e]) + slot;
  if (pair_row != nullptr && lane == 0) pair_row[p] = dest < cap_rows ? dest : 0;   // one rank: where this pair's result will be
  if (dest >= cap_rows) return;   // the plan kernel has flagged the overflow
  const long long t = p / top_k;
  const uint4* src = x_q + t * vec_per_row;
  uint4* dst = static_cast<uint4*>(peers.a[o]) + dest * vec_per_row;
  copy_row(src, dst, vec_per_row, lane);
  const float* ssrc = sfx + t * sf_per_row;
  float* sdst = static_cast<float*>(peers.sfa[o]) + dest * sf_per_row;
  for (int i = lane; i < sf_per_row; i += 32) sdst[i] = ssrc[i];
  if (lane == 0) static_cast<long long*>(peers.meta[o])[dest] = (static_cast<long long>(me) << 32) | p;
}

// One warp per row of this rank's layout: a valid row's result goes to its pair's slot in the source rank's combine buffer.
__global__ void __launch_bounds__(256) ep_return_kernel(const uint4* __restrict__ out, const long long* __restrict__ meta,
                                                        const int* __restrict__ rows_used, int vec_per_row, PeerTable peers) {
  const long long r = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= rows_used[0]) return;
  const long long m = meta[r];
  if (m < 0) return;
  const int s = static_cast<int>(m >> 32);
  const long long p = m & 0xffffffffLL;
  const uint4* src = out + r * vec_per_row;
  uint4* dst = static_cast<uint4*>(peers.ret[s]) + p * vec_per_row;
  copy_row(src, dst, vec_per_row, lane);
}

}  // namespace agb

namespace {
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
int launch_check() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? AG_OK : agb_fail(AG_E_CUDA, cudaGetErrorString(e));
}
int fill_table(agb::PeerTable* t, const ag_ep_peers_t* peers, int world) {
  if (peers == nullptr || world < 1 || world > agb::kMaxRanks) return agb_fail(AG_E_INVALID, "peers must be given and 1 <= world <= 16");
  std::memset(t, 0, sizeof(*t));
  for (int r = 0; r < world; ++r) {
    t->a[r] = peers->a[r];
    t->sfa[r] = peers->sfa[r];
    t->meta[r] = peers->meta[r];
    t->ret[r] = peers->ret[r];
    if (!t->a[r] || !t->sfa[r] || !t->meta[r] || !t->ret[r] || !aligned16(t->a[r]) || !aligned16(t->ret[r]))
      return agb_fail(AG_E_INVALID, "every rank's a / sfa / meta / ret buffer must be given (a and ret 16-byte aligned)");
  }
  return AG_OK;
}
}  // namespace

extern "C" {

int ag_peer_alloc(uint64_t bytes, void** ptr, unsigned char* handle64) {
  if (ptr == nullptr || handle64 == nullptr || bytes == 0) return agb_fail(AG_E_INVALID, "bad arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) {
    cudaGetLastError();
    return agb_fail(AG_E_CUDA, "cudaMalloc failed for the exchange buffers");
  }
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(p);
    return agb_fail(AG_E_CUDA, "cudaIpcGetMemHandle failed");
  }
  std::memcpy(handle64, &h, 64);
  *ptr = p;
  return AG_OK;
}

int ag_peer_open(const unsigned char* handle64, void** ptr) {
  if (ptr == nullptr || handle64 == nullptr) return agb_fail(AG_E_INVALID, "bad arguments");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return agb_fail(AG_E_CUDA, cudaGetErrorString(e));
  }
  *ptr = p;
  return AG_OK;
}

int ag_peer_close(void* ptr) {
  if (ptr == nullptr) return AG_OK;
  if (cudaIpcCloseMemHandle(ptr) != cudaSuccess) {
    cudaGetLastError();
    return agb_fail(AG_E_CUDA, "cudaIpcCloseMemHandle failed");
  }
  return AG_OK;
}

int ag_peer_free(void* ptr) {
  if (ptr == nullptr) return AG_OK;
  if (cudaFree(ptr) != cudaSuccess) {
    cudaGetLastError();
    return agb_fail(AG_E_CUDA, "cudaFree failed");
  }
  return AG_OK;
}

int ag_ep_histogram(const int64_t* ids, int64_t pairs, int32_t num_experts, int32_t* counts, int32_t* status, void* stream) {
  if (!ids || !counts || !status || pairs < 0 || num_experts <= 0 || num_experts > 8192) return agb_fail(AG_E_INVALID, "bad arguments (1 <= num_experts <= 8192)");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(counts, 0, sizeof(int32_t) * num_experts, st) != cudaSuccess) return agb_fail(AG_E_CUDA, "cudaMemsetAsync failed");
  if (pairs == 0) return AG_OK;
  const long long blocks = (pairs + 255) / 256;
  agb::ep_histogram_kernel<<<static_cast<unsigned>(blocks < 1184 ? blocks : 1184), 256, sizeof(int) * num_experts, st>>>(
      reinterpret_cast<const long long*>(ids), pairs, num_experts, counts, status);
  return launch_check();
}

int ag_ep_plan(const int32_t* counts_all, const int32_t* range_lo, int32_t world, int32_t rank, int32_t num_experts, int64_t cap_rows,
               int32_t* send_base, int32_t* cursors, int32_t* offsets, int32_t* experts, int32_t epr_cap, int32_t* rows_used, int64_t* my_meta,
               int32_t* status, void* stream) {
  if (!counts_all || !range_lo || !send_base || !cursors || !offsets || !experts || !rows_used || !my_meta || !status || world < 1 ||
      world > agb::kMaxRanks || rank < 0 || rank >= world || num_experts <= 0 || num_experts > 4096 || cap_rows <= 0 || epr_cap <= 0)
    return agb_fail(AG_E_INVALID, "bad arguments (1 <= world <= 16, 1 <= num_experts <= 4096)");
  agb::ep_plan_kernel<<<1, agb::kPlanThreads, sizeof(int) * 3 * num_experts, static_cast<cudaStream_t>(stream)>>>(
      counts_all, range_lo, world, rank, num_experts, cap_rows, send_base, cursors, offsets, experts, epr_cap, rows_used,
      reinterpret_cast<long long*>(my_meta), status);
  return launch_check();
}

int ag_ep_dispatch(const void* x_q, const float* sfx, const int64_t* ids, int64_t tokens, int32_t top_k, int64_t row_bytes, int32_t sf_per_row,
                   const int32_t* range_lo, int32_t world, int32_t rank, const int32_t* send_base, int32_t* cursors, int64_t cap_rows,
                   int64_t* pair_row, const ag_ep_peers_t* peers, void* stream) {
  if (!x_q || !sfx || !ids || !range_lo || !send_base || !cursors || tokens < 0 || top_k <= 0 || row_bytes <= 0 || row_bytes % 16 != 0 ||
      sf_per_row <= 0 || !aligned16(x_q) || rank < 0 || rank >= world || cap_rows <= 0)
    return agb_fail(AG_E_INVALID, "bad arguments (rows must be 16-byte multiples and 16-byte aligned)");
  agb::PeerTable t;
  if (int rc = fill_table(&t, peers, world)) return rc;
  const long long pairs = tokens * top_k;
  if (pairs == 0) return AG_OK;
  if (pairs >= (1LL << 32)) return agb_fail(AG_E_INVALID, "more than 2^32 (token, slot) pairs per rank");
  agb::ep_dispatch_kernel<<<static_cast<unsigned>((pairs + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x_q), sfx, reinterpret_cast<const long long*>(ids), pairs, top_k, static_cast<int>(row_bytes / 16), sf_per_row,
      range_lo, world, rank, send_base, cursors, cap_rows, reinterpret_cast<long long*>(pair_row), t);
  return launch_check();
}

int ag_ep_return(const void* out, const int64_t* my_meta, const int32_t* rows_used, int64_t cap_rows, int64_t row_bytes, int32_t world,
                 const ag_ep_peers_t* peers, void* stream) {
  if (!out || !my_meta || !rows_used || cap_rows <= 0 || row_bytes <= 0 || row_bytes % 16 != 0 || !aligned16(out))
    return agb_fail(AG_E_INVALID, "bad arguments (rows must be 16-byte multiples and 16-byte aligned)");
  agb::PeerTable t;
  if (int rc = fill_table(&t, peers, world)) return rc;
  agb::ep_return_kernel<<<static_cast<unsigned>((cap_rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(out), reinterpret_cast<const long long*>(my_meta), rows_used, static_cast<int>(row_bytes / 16), t);
  return launch_check();
}

}  // extern "C"
