// C ABI over the sm_100a grouped-GEMM kernels: argument validation, residency checks for B, tensor-map
// encoding, grid sizing and launch. Mirrors the host-side contract of the reference operator API
// (csrc/apis/gemm.hpp) without torch types; see include/asymgemm_b200.h.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/asymgemm_b200.h"
#include "launch.cuh"

namespace {

thread_local char g_err[512] = "";
std::atomic<int> g_num_sms{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define AG_REQUIRE(cond, ...)                                  \
  do {                                                         \
    if (!(cond)) return fail(AG_E_INVALID, __VA_ARGS__);       \
  } while (0)

#define AG_CUDA(call)                                                                                   \
  do {                                                                                                  \
    cudaError_t e_ = (call);                                                                            \
    if (e_ != cudaSuccess) return fail(AG_E_CUDA, "CUDA error (%s): %s", #call, cudaGetErrorString(e_)); \
  } while (0)

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }();
  return fn;
}

// Byte-typed 2-D map [rows, row_bytes] with a (128 B x box_rows) box and the 128-byte swizzle.
int encode_bytes_2d(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint64_t pitch_bytes,
                    uint32_t box_rows, const char* what) {
  auto fn = encode_fn();
  if (fn == nullptr) return fail(AG_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdim[2] = {row_bytes, rows};
  cuuint64_t gstr[1] = {pitch_bytes};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstr, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(AG_E_CUDA, "cuTensorMapEncodeTiled failed for %s (CUresult %d; base %p, row_bytes %llu, rows %llu)", what,
                static_cast<int>(r), base, static_cast<unsigned long long>(row_bytes), static_cast<unsigned long long>(rows));
  return AG_OK;
}

enum Residency { RES_DEVICE, RES_HOST_MAPPED, RES_UNREACHABLE };

// Where does `p` live, and under which address can the current device read it?
Residency classify(const void* p, const void** dev_alias) {
  cudaPointerAttributes at;
  *dev_alias = p;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
    cudaGetLastError();
    return RES_UNREACHABLE;
  }
  if (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged) return RES_DEVICE;
  if (at.type == cudaMemoryTypeHost) {
    *dev_alias = at.devicePointer != nullptr ? at.devicePointer : p;
    return RES_HOST_MAPPED;
  }
  return RES_UNREACHABLE;  // pageable host memory: an x86 GPU cannot address it
}

int* default_status_word() {
  // One word per device, allocated on first use and kept for the life of the process.
  static std::mutex mu;
  static int* words[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(mu);
  if (words[dev] == nullptr) {
    if (cudaMalloc(&words[dev], sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(words[dev], 0, sizeof(int));
  }
  return words[dev];
}

int device_sm_count(int* out) {
  static int cached[64] = {};
  int dev = 0;
  AG_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && cached[dev] > 0) {
    *out = cached[dev];
    return AG_OK;
  }
  int major = 0, sms = 0;
  AG_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  AG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (major != 10) return fail(AG_E_UNSUPPORTED, "this library is built for sm_100a only (device compute capability major %d)", major);
  if (dev >= 0 && dev < 64) cached[dev] = sms;
  *out = sms;
  return AG_OK;
}

uint64_t k_bytes_of(int kind, int64_t k) {
  switch (kind) {
    case 0: return static_cast<uint64_t>(k) * 2;
    case 3: return static_cast<uint64_t>(k) / 2;   // kind 4 (fp8 with UE8M0 scales): one byte per element, like fp8
    default: return static_cast<uint64_t>(k);
  }
}

// Everything about a launch that follows from the descriptor and from where b lives: tile configuration, grid, whether
// long segments are split into row chunks, and the scratch a replay of long segments would use. run() and the
// scratch-size queries share it, so that they cannot drift apart.
struct LaunchPlan {
  int tile = 0, bn = 0, ka = 0;
  int n_tiles = 0, kb_count = 0;
  int split_rows = 0;        // > 0: device-resident b, segments are cut into chunks of this many rows (no item ever replays)
  int grid = 0;
  int b_box_rows = 0;        // weight rows one TMA load brings (half a tile for the pair kernel)
  uint64_t kpad = 0;         // bytes of one scratch row: K bytes padded to whole weight stages
  uint64_t scratch_need = 0; // 0 = this launch has no use for scratch
};

int plan_launch(int kind, const ag_gemm_desc_t* g, bool host_b, LaunchPlan* out) {
  LaunchPlan pl;
  const bool masked = g->layout == AG_LAYOUT_MASKED;
  const int64_t rows_total = masked ? g->m * g->num_groups : g->m;
  int sms = 0;
  if (int rc = device_sm_count(&sms)) return rc;
  const int cap = g->num_sms > 0 ? g->num_sms : g_num_sms.load();
  const int grid_cap = cap > 0 && cap < sms ? cap : sms;
  pl.tile = g->tile_config > 0 ? g->tile_config - 1 : agb::default_tile(kind, host_b, g->n);
  AG_REQUIRE(pl.tile >= 0 && pl.tile < agb::kNumTileConfigs, "tile_config must be 0 (auto) .. %d", agb::kNumTileConfigs);
  AG_REQUIRE(agb::tile_supported(kind, pl.tile), "tile_config %d does not exist for this operand kind (%s)", pl.tile + 1,
             agb::tile_support_text(kind));
  if (kind == 3 || kind == 4) {
    if (kind == 3) AG_REQUIRE(g->k % 32 == 0, "nvfp4 needs k to be a multiple of 32 (got %lld)", static_cast<long long>(g->k));
    if (masked) AG_REQUIRE(g->m % 128 == 0, "block-scaled masked layout needs M_max to be a multiple of 128 (got %lld)", static_cast<long long>(g->m));
  }
  const bool pair = pl.tile == agb::kTileDevicePair;
  if (pair) {
    AG_REQUIRE(!host_b, "tile_config %d (CTA pairs) is for b resident in device memory", pl.tile + 1);
    AG_REQUIRE(!g->no_split, "tile_config %d (CTA pairs) always splits long segments into row chunks; no_split cannot be combined with it", pl.tile + 1);
    AG_REQUIRE(grid_cap >= 2, "tile_config %d (CTA pairs) needs at least two SMs", pl.tile + 1);
  }
  const agb::TileConfig tc = agb::tile_config_of(kind, pl.tile);
  pl.bn = tc.bn;
  pl.ka = tc.ka;
  pl.n_tiles = static_cast<int>((g->n + pl.bn - 1) / pl.bn);
  pl.kb_count = static_cast<int>((k_bytes_of(kind, g->k) + 127) / 128);
  // Device-resident weights: split long segments into accumulator-sized row chunks so that work spreads evenly.
  // Host-resident weights keep whole segments per item: the weight column must cross the host link only once.
  if (!host_b && !g->no_split) pl.split_rows = 128 * agb::chunk_tiles_of(kind, pl.tile, pl.bn);
  const long long segments = masked ? g->num_groups : g->max_segments;
  const long long seg_items = pl.split_rows > 0 ? rows_total / pl.split_rows + segments : segments;
  const long long items = seg_items * pl.n_tiles;
  AG_REQUIRE(items < (1LL << 31), "the problem has %lld work items; the kernels index them with 32 bits", items);
  if (pair) {   // items are taken by pairs of CTAs
    const long long pairs = items < grid_cap / 2 ? items : grid_cap / 2;
    pl.grid = static_cast<int>(2 * pairs);
    pl.b_box_rows = pl.bn / 2;
  } else {
    pl.grid = static_cast<int>(items < grid_cap ? items : grid_cap);
    pl.b_box_rows = pl.bn;
  }
  if (pl.grid < 0) pl.grid = 0;
  pl.kpad = static_cast<uint64_t>((pl.kb_count + pl.ka - 1) / pl.ka) * pl.ka * 128;
  pl.scratch_need = pl.split_rows > 0 ? 0 : static_cast<uint64_t>(pl.grid) * pl.bn * pl.kpad;
  *out = pl;
  return AG_OK;
}

int run_staged(int kind, const ag_gemm_desc_t* g, uint64_t expert_bytes);

// One launch. `win_n` >= 0: `g->b` holds only the experts [win_lo, win_lo + win_n) (a staged chunk) and the launch
// skips the segments of all others; `g->num_groups` stays the size of the whole weight tensor.
int run(int kind, const ag_gemm_desc_t* g, int win_lo = 0, int win_n = -1) {
  AG_REQUIRE(g != nullptr, "desc is NULL");
  AG_REQUIRE(g->layout == AG_LAYOUT_CONTIGUOUS || g->layout == AG_LAYOUT_MASKED, "unknown layout %d", g->layout);
  AG_REQUIRE(g->d_dtype == AG_D_BF16 || g->d_dtype == AG_D_FP32, "unknown d_dtype %d", g->d_dtype);
  AG_REQUIRE(g->n > 0 && g->k > 0 && g->num_groups > 0, "n, k and num_groups must be positive (n=%lld k=%lld G=%d)",
             static_cast<long long>(g->n), static_cast<long long>(g->k), g->num_groups);
  AG_REQUIRE(g->m >= 0, "m must be non-negative");
  const bool masked = g->layout == AG_LAYOUT_MASKED;
  const int64_t rows_total = masked ? g->m * g->num_groups : g->m;
  if (rows_total == 0) return AG_OK;  // empty problem: nothing to do (csrc/apis/gemm.hpp:114-115)
  if (!masked && g->max_segments <= 0) return AG_OK;
  AG_REQUIRE(g->a != nullptr && g->b != nullptr && g->d != nullptr, "a, b and d must be non-NULL");
  AG_REQUIRE(rows_total < (1LL << 31) && g->n * g->num_groups < (1LL << 31), "row counts must fit in int32");
  AG_REQUIRE(g->n % 8 == 0, "n must be a multiple of 8 (got %lld)", static_cast<long long>(g->n));
  if (masked) AG_REQUIRE(g->masked_m != nullptr, "masked layout needs masked_m");
  else AG_REQUIRE(g->offsets != nullptr && g->experts != nullptr, "contiguous layout needs offsets and experts");
  if (kind >= 1) AG_REQUIRE(g->sfa != nullptr && g->sfb != nullptr, "quantised kinds need sfa and sfb");
  AG_REQUIRE(g->epilogue == AG_EPILOGUE_NONE || g->epilogue == AG_EPILOGUE_SILU_MUL, "unknown epilogue %d", g->epilogue);
  if (g->epilogue == AG_EPILOGUE_SILU_MUL) {
    AG_REQUIRE(kind == 1, "the fused SiLU*mul epilogue exists for fp8 with fp32 scales only");
    AG_REQUIRE(g->n % 256 == 0, "the fused SiLU*mul epilogue needs n to be a multiple of 256 (got %lld)", static_cast<long long>(g->n));
    AG_REQUIRE(g->d_dtype == AG_D_BF16, "the fused SiLU*mul epilogue writes bf16");
  }

  const uint64_t kbytes = k_bytes_of(kind, g->k);
  AG_REQUIRE(kbytes % 16 == 0, "K must make rows a multiple of 16 bytes (row bytes %llu)", static_cast<unsigned long long>(kbytes));
  AG_REQUIRE((reinterpret_cast<uintptr_t>(g->a) & 15) == 0 && (reinterpret_cast<uintptr_t>(g->d) & 15) == 0,
             "a and d must be 16-byte aligned");

  const void* b_dev = nullptr;
  const Residency res = classify(g->b, &b_dev);
  if (res == RES_UNREACHABLE)
    return fail(AG_E_NOT_MAPPED, "b (%p) is neither device memory nor pinned/registered host memory: pin it "
                "(cudaHostAlloc / cudaHostRegister / torch pin_memory) before the call", g->b);
  AG_REQUIRE((reinterpret_cast<uintptr_t>(b_dev) & 15) == 0, "b must be 16-byte aligned");
  if (g->stage != nullptr && win_n < 0 && res == RES_HOST_MAPPED && !(kind == 2 && g->raw_dump != nullptr))
    return run_staged(kind, g, static_cast<uint64_t>(g->n) * kbytes);
  const int b_groups = win_n >= 0 ? win_n : g->num_groups;

  LaunchPlan plan;
  if (int rc = plan_launch(kind, g, res == RES_HOST_MAPPED, &plan)) return rc;
  if (plan.grid <= 0) return AG_OK;
  const int tile = plan.tile, bn = plan.bn, grid = plan.grid;
  const uint64_t kpad = plan.kpad, need = plan.scratch_need;

  agb::GemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.sfa = static_cast<const float*>(g->sfa);
  const void* sfb_dev = g->sfb;
  if (g->sfb != nullptr) {
    const Residency rs = classify(g->sfb, &sfb_dev);
    if (rs == RES_UNREACHABLE) return fail(AG_E_NOT_MAPPED, "sfb (%p) is not addressable by the device", g->sfb);
  }
  p.sfb = static_cast<const float*>(sfb_dev);
  p.d = g->d;
  p.offsets = g->offsets;
  p.experts = g->experts;
  p.masked_m = g->masked_m;
  p.status = g->status != nullptr ? g->status : default_status_word();
  if (p.status == nullptr) return fail(AG_E_CUDA, "could not allocate the status word");
  p.raw_dump = kind == 2 ? g->raw_dump : nullptr;
  p.timeout_ns = static_cast<unsigned long long>(g->timeout_ms ? g->timeout_ms : 4000u) * 1000000ull;
  p.rows_total = rows_total;
  p.layout = masked ? agb::LAYOUT_MASKED : agb::LAYOUT_CONTIGUOUS;
  p.max_segments = masked ? g->num_groups : g->max_segments;
  p.m_max = masked ? static_cast<int>(g->m) : 0;
  p.num_groups = g->num_groups;
  p.expert_lo = win_n >= 0 ? win_lo : 0;
  p.expert_n = b_groups;
  p.n = static_cast<int>(g->n);
  p.n_tiles = plan.n_tiles;
  p.kb_count = plan.kb_count;
  p.sf_k = kind == 3 ? static_cast<int>(agb::fp4_sf_k4_padded_host((g->k + 15) / 16))
           : kind == 4 ? static_cast<int>(agb::fp8_sf_k4_padded_host((g->k + 127) / 128)) : static_cast<int>((g->k + 127) / 128);
  p.sfb_rows = kind == 2 ? static_cast<int>(g->n) : static_cast<int>((g->n + 127) / 128);
  p.d_fp32 = g->d_dtype == AG_D_FP32;
  p.b_streaming = res == RES_HOST_MAPPED;
  p.alpha = g->alpha == 0.f ? 1.f : g->alpha;
  p.split_rows = plan.split_rows;
  p.epilogue = g->epilogue;
  p.d_cols = g->epilogue == AG_EPILOGUE_SILU_MUL ? static_cast<int>(g->n / 2) : static_cast<int>(g->n);
  AG_REQUIRE((g->scatter_meta == nullptr) == (g->scatter_bases == nullptr), "scatter_meta and scatter_bases go together");
  if (g->scatter_meta != nullptr) {
    AG_REQUIRE(!masked, "the result scatter exists for the contiguous layout");
    AG_REQUIRE(kind != 2 || g->raw_dump == nullptr, "raw_dump and the result scatter cannot be combined");
  }
  p.scatter_meta = reinterpret_cast<const long long*>(g->scatter_meta);
  p.scatter_bases = reinterpret_cast<const long long*>(g->scatter_bases);

  // Replay from scratch needs the whole amount; with less (or none) long segments re-read their weight column from b.
  p.use_scratch = (g->scratch != nullptr && need > 0 && g->scratch_bytes >= need) ? 1 : 0;
  if (g->scratch != nullptr)
    AG_REQUIRE((reinterpret_cast<uintptr_t>(g->scratch) & 1023) == 0, "scratch must be 1024-byte aligned");

  CUtensorMap ma, mb, ms;
  if (int rc = encode_bytes_2d(&ma, g->a, kbytes, static_cast<uint64_t>(rows_total), kbytes, 128, "a")) return rc;
  if (int rc = encode_bytes_2d(&mb, b_dev, kbytes, static_cast<uint64_t>(g->n) * b_groups, kbytes, plan.b_box_rows, "b")) return rc;
  if (p.use_scratch) {
    if (int rc = encode_bytes_2d(&ms, g->scratch, kpad, static_cast<uint64_t>(grid) * bn, kpad, bn, "scratch")) return rc;
  } else {
    ms = mb;
  }

  cudaStream_t stream = static_cast<cudaStream_t>(g->stream);
  cudaError_t e = agb::launch_mgrouped(kind, tile, grid, stream, ma, mb, ms, p);
  if (e != cudaSuccess) return fail(AG_E_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
  return AG_OK;
}

// Copy stream and hand-over events of the staged weight path, one set per device, created on first use and kept for
// the life of the process. `free_[j]` is recorded after the GEMM that read half j, `ready[j]` after the copy into it.
constexpr int kMaxStageSlots = 8;

struct StageState {
  cudaStream_t copy = nullptr;
  cudaEvent_t ready[kMaxStageSlots] = {};
  cudaEvent_t free_[kMaxStageSlots] = {};
  cudaEvent_t gate = nullptr;   // "the caller's stream has reached the point of the prefetch call"
  // chunks a prefetch has already put (or is putting) into the halves, for the next staged call on the same operands
  const void* pf_b = nullptr;
  void* pf_stage = nullptr;
  uint64_t pf_expert_bytes = 0;
  uint64_t pf_slot_bytes = 0;
  int pf_slots = 0;
  int pf_count = 0;
};

// The buffer as a ring of equal slots, each holding one chunk of whole experts.
struct StageRing {
  uint64_t slot_bytes;
  int slots;
  int chunk;   // experts per slot
};

int stage_ring(uint64_t stage_bytes, uint64_t chunk_bytes, uint64_t expert_bytes, int num_groups, StageRing* r) {
  uint64_t slot = chunk_bytes > 0 ? chunk_bytes : stage_bytes / 2;
  if (slot > stage_bytes / 2) slot = stage_bytes / 2;
  slot &= ~static_cast<uint64_t>(1023);
  AG_REQUIRE(slot >= expert_bytes, "the staging buffer (%llu bytes, slots of %llu) must hold at least two slots of one %llu-byte expert",
             static_cast<unsigned long long>(stage_bytes), static_cast<unsigned long long>(slot), static_cast<unsigned long long>(expert_bytes));
  const uint64_t n = stage_bytes / slot;
  r->slot_bytes = slot;
  r->slots = static_cast<int>(n < static_cast<uint64_t>(kMaxStageSlots) ? n : kMaxStageSlots);
  r->chunk = static_cast<int>(slot / expert_bytes < static_cast<uint64_t>(num_groups) ? slot / expert_bytes : num_groups);
  return AG_OK;
}
std::mutex g_stage_mu;
StageState g_stage[64];

int stage_state(StageState** out) {
  int dev = 0;
  AG_CUDA(cudaGetDevice(&dev));
  AG_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
  StageState& st = g_stage[dev];
  if (st.copy == nullptr) {
    AG_CUDA(cudaStreamCreateWithFlags(&st.copy, cudaStreamNonBlocking));
    for (int j = 0; j < kMaxStageSlots; ++j) {
      AG_CUDA(cudaEventCreateWithFlags(&st.ready[j], cudaEventDisableTiming));
      AG_CUDA(cudaEventCreateWithFlags(&st.free_[j], cudaEventDisableTiming));
    }
    AG_CUDA(cudaEventCreateWithFlags(&st.gate, cudaEventDisableTiming));
  }
  *out = &st;
  return AG_OK;
}

// Copy of chunk `i` (experts [lo, lo + cnt)) into its slot of the ring, ordered after the GEMM that last read the slot.
int stage_copy(StageState& st, const void* b, void* stage, const StageRing& ring, uint64_t expert_bytes, int i, int lo, int cnt) {
  const int j = i % ring.slots;
  char* dst = static_cast<char*>(stage) + static_cast<uint64_t>(j) * ring.slot_bytes;
  AG_CUDA(cudaStreamWaitEvent(st.copy, st.free_[j], 0));   // an event never recorded yet does not block
  AG_CUDA(cudaMemcpyAsync(dst, static_cast<const char*>(b) + static_cast<uint64_t>(lo) * expert_bytes,
                          static_cast<uint64_t>(cnt) * expert_bytes, cudaMemcpyDefault, st.copy));
  AG_CUDA(cudaEventRecord(st.ready[j], st.copy));
  return AG_OK;
}

// The grouped GEMM as a series of launches over chunks of whole experts that the copy engine brings into `g->stage`.
// The lock is held for the whole series: the events of one device then always belong to one call at a time, and the
// copies of a call wait for the GEMMs of the previous call that read the same half.
int run_staged(int kind, const ag_gemm_desc_t* g, uint64_t expert_bytes) {
  AG_REQUIRE((reinterpret_cast<uintptr_t>(g->stage) & 1023) == 0, "stage must be 1024-byte aligned");
  StageRing ring;
  if (int rc = stage_ring(g->stage_bytes, g->stage_chunk_bytes, expert_bytes, g->num_groups, &ring)) return rc;
  const void* stage_alias = nullptr;
  AG_REQUIRE(classify(g->stage, &stage_alias) == RES_DEVICE, "stage must be device memory");
  std::lock_guard<std::mutex> lk(g_stage_mu);
  StageState* stp = nullptr;
  if (int rc = stage_state(&stp)) return rc;
  StageState& st = *stp;
  cudaStream_t stream = static_cast<cudaStream_t>(g->stream);
  // chunks a matching ag_prefetch_staged_weights has already issued are not copied again
  const bool hit = st.pf_b == g->b && st.pf_stage == g->stage && st.pf_expert_bytes == expert_bytes &&
                   st.pf_slot_bytes == ring.slot_bytes && st.pf_slots == ring.slots;
  const int prefetched = hit ? st.pf_count : 0;
  st.pf_b = nullptr;
  st.pf_count = 0;
  ag_gemm_desc_t c = *g;
  c.stage = nullptr;
  for (int lo = 0, i = 0; lo < g->num_groups; lo += ring.chunk, ++i) {
    const int j = i % ring.slots;
    const int cnt = g->num_groups - lo < ring.chunk ? g->num_groups - lo : ring.chunk;
    if (i >= prefetched)
      if (int rc = stage_copy(st, g->b, g->stage, ring, expert_bytes, i, lo, cnt)) return rc;
    AG_CUDA(cudaStreamWaitEvent(stream, st.ready[j], 0));
    c.b = static_cast<char*>(g->stage) + static_cast<uint64_t>(j) * ring.slot_bytes;
    const int rc = run(kind, &c, lo, cnt);
    AG_CUDA(cudaEventRecord(st.free_[j], stream));   // also after a failed launch: the slot is not in use then
    if (rc != AG_OK) return rc;
  }
  return AG_OK;
}

const char* status_text(int code) {
  switch (code & 0xff) {
    case agb::ST_TIMEOUT_B_EMPTY: return "timed out waiting for a free weight stage";
    case agb::ST_TIMEOUT_A_EMPTY: return "timed out waiting for a free activation stage";
    case agb::ST_TIMEOUT_B_FULL: return "timed out waiting for a weight tile to arrive";
    case agb::ST_TIMEOUT_A_FULL: return "timed out waiting for an activation tile to arrive";
    case agb::ST_TIMEOUT_TM_EMPTY: return "timed out waiting for a free accumulator";
    case agb::ST_TIMEOUT_TM_FULL: return "timed out waiting for an accumulator to complete";
    case agb::ST_TIMEOUT_DRAIN: return "timed out draining copies in flight";
    case agb::ST_BAD_EXPERT: return "an expert id in `experts` is >= num_groups";
    case agb::ST_TIMEOUT_PROBE: return "wait-limit self test expired (expected)";
    case AG_EP_BAD_EXPERT: return "the routing names an expert id outside [0, num_experts)";
    case AG_EP_OVERFLOW: return "a rank's experts received more rows than its exchange buffers hold";
    default: return "unknown status";
  }
}

// Scratch the launch described by `g` would replay long segments from (0: it has no use for any).
int scratch_need(int kind, const ag_gemm_desc_t* g, uint64_t* out) {
  AG_REQUIRE(g != nullptr && out != nullptr, "desc and the output pointer must be non-NULL");
  AG_REQUIRE(kind >= 0 && kind <= 4, "kind must be 0 .. 4");
  AG_REQUIRE(g->layout == AG_LAYOUT_CONTIGUOUS || g->layout == AG_LAYOUT_MASKED, "unknown layout %d", g->layout);
  AG_REQUIRE(g->n > 0 && g->k > 0 && g->num_groups > 0 && g->m >= 0 && g->b != nullptr, "n, k, num_groups must be positive and b non-NULL");
  const void* alias = nullptr;
  const Residency res = classify(g->b, &alias);
  if (res == RES_UNREACHABLE) return fail(AG_E_NOT_MAPPED, "b (%p) is neither device memory nor pinned/registered host memory", g->b);
  LaunchPlan plan;
  if (int rc = plan_launch(kind, g, res == RES_HOST_MAPPED, &plan)) return rc;
  *out = plan.scratch_need;
  return AG_OK;
}

}  // namespace

// Hooks for the other translation units of the library (not part of the public ABI).
int agb_run_desc(int kind, const ag_gemm_desc_t* desc) { return run(kind, desc); }
int agb_scratch_need(int kind, const ag_gemm_desc_t* desc, uint64_t* out) { return scratch_need(kind, desc, out); }
int agb_fail(int code, const char* message) { return fail(code, "%s", message); }

extern "C" {

int ag_m_grouped_bf16_gemm_nt(const ag_gemm_desc_t* desc) { return run(0, desc); }
int ag_m_grouped_fp8_gemm_nt(const ag_gemm_desc_t* desc) { return run(1, desc); }
int ag_m_grouped_int8_gemm_nt(const ag_gemm_desc_t* desc) { return run(2, desc); }
int ag_m_grouped_fp4_gemm_nt(const ag_gemm_desc_t* desc) { return run(3, desc); }
int ag_m_grouped_fp8_ue8m0_gemm_nt(const ag_gemm_desc_t* desc) { return run(4, desc); }

uint64_t ag_fp8_sf_blocked_bytes(int64_t groups, int64_t rows, int64_t kb) {
  return static_cast<uint64_t>(groups) * static_cast<uint64_t>((rows + 127) / 128) * static_cast<uint64_t>(agb::fp8_sf_k4_padded_host(kb)) * 512;
}

int ag_fp8_sf_to_blocked_ue8m0(const float* src, void* dst, int64_t groups, int64_t rows, int64_t kb, int32_t rows_per_scale, void* stream) {
  AG_REQUIRE(src != nullptr && dst != nullptr && groups > 0 && rows > 0 && kb > 0 && (rows_per_scale == 1 || rows_per_scale == 128),
             "bad arguments (rows_per_scale must be 1 or 128)");
  const void* src_dev = src;
  if (classify(src, &src_dev) == RES_UNREACHABLE)
    return fail(AG_E_NOT_MAPPED, "scale tensor (%p) is neither device memory nor pinned/registered host memory", static_cast<const void*>(src));
  cudaError_t e = agb::fp8_sf_to_blocked_ue8m0(static_cast<const float*>(src_dev), dst, groups, rows, kb, rows_per_scale,
                                               static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(AG_E_CUDA, "scale re-layout launch failed: %s", cudaGetErrorString(e));
  return AG_OK;
}

uint64_t ag_scratch_bytes(int32_t kind, int64_t n, int64_t k, int32_t num_sms) {
  (void)n;
  int sms = num_sms;
  if (sms <= 0) {
    if (device_sm_count(&sms) != AG_OK) sms = 148;
  }
  // large enough for every tile configuration: 128 rows per CTA, K padded to 8 atoms
  const uint64_t kpad = (k_bytes_of(kind, k) + 1023) / 1024 * 1024;
  return static_cast<uint64_t>(sms) * 128 * kpad;
}

int ag_scratch_bytes_for(int32_t kind, const ag_gemm_desc_t* desc, uint64_t* bytes_out) { return scratch_need(kind, desc, bytes_out); }

uint64_t ag_gemm_desc_size(void) { return sizeof(ag_gemm_desc_t); }

int ag_read_status(const int32_t* status_dev, void* stream, int32_t* out) {
  const int32_t* src = status_dev != nullptr ? status_dev : default_status_word();
  if (src == nullptr) return fail(AG_E_CUDA, "no status word");
  int32_t v = 0;
  AG_CUDA(cudaMemcpyAsync(&v, src, sizeof(v), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  AG_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  if (out != nullptr) *out = v;
  if (v != 0) return fail(AG_E_DEVICE, "kernel status 0x%x: CTA %d %s", v, v >> 8, status_text(v));
  return AG_OK;
}

void ag_set_num_sms(int32_t num_sms) { g_num_sms.store(num_sms > 0 ? num_sms : 0); }
int32_t ag_get_num_sms(void) {
  int v = g_num_sms.load();
  if (v > 0) return v;
  int sms = 0;
  return device_sm_count(&sms) == AG_OK ? sms : 0;
}
int32_t ag_get_mk_alignment_for_contiguous_layout(void) { return 128; }

uint64_t ag_fp4_sf_blocked_bytes(int64_t groups, int64_t rows, int64_t k16) {
  const uint64_t row_tiles = static_cast<uint64_t>((rows + 127) / 128);
  const uint64_t k4 = static_cast<uint64_t>(agb::fp4_sf_k4_padded_host(k16));
  return static_cast<uint64_t>(groups) * row_tiles * k4 * 512;
}

int ag_fp4_sf_to_blocked(const void* src, void* dst, int64_t groups, int64_t rows, int64_t k16, void* stream) {
  AG_REQUIRE(src != nullptr && dst != nullptr && groups > 0 && rows > 0 && k16 > 0, "bad arguments");
  const void* src_dev = src;
  if (classify(src, &src_dev) == RES_UNREACHABLE)
    return fail(AG_E_NOT_MAPPED, "scale tensor (%p) is neither device memory nor pinned/registered host memory", src);
  AG_REQUIRE((reinterpret_cast<uintptr_t>(dst) & 15) == 0, "dst must be 16-byte aligned");
  cudaError_t e = agb::fp4_sf_to_blocked(src_dev, dst, groups, rows, k16, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(AG_E_CUDA, "scale re-layout launch failed: %s", cudaGetErrorString(e));
  return AG_OK;
}

namespace {
std::mutex g_reg_mu;
void* g_registered[256] = {};   // host ranges registered by ag_prepare_weights, by start address
}  // namespace

int ag_prefetch_staged_weights(const void* b, uint64_t expert_bytes, int32_t num_groups, void* stage, uint64_t stage_bytes,
                               uint64_t stage_chunk_bytes, void* after_stream, int32_t wait_for_stream) {
  AG_REQUIRE(b != nullptr && stage != nullptr && expert_bytes > 0 && num_groups > 0, "bad arguments");
  AG_REQUIRE((reinterpret_cast<uintptr_t>(stage) & 1023) == 0, "stage must be 1024-byte aligned");
  StageRing ring;
  if (int rc = stage_ring(stage_bytes, stage_chunk_bytes, expert_bytes, num_groups, &ring)) return rc;
  const void* alias = nullptr;
  if (classify(b, &alias) != RES_HOST_MAPPED) return AG_OK;   // weights already on the device: nothing to stage
  std::lock_guard<std::mutex> lk(g_stage_mu);
  StageState* stp = nullptr;
  if (int rc = stage_state(&stp)) return rc;
  StageState& st = *stp;
  st.pf_b = nullptr;
  st.pf_count = 0;
  if (wait_for_stream) {
    // the copies start when the work already queued on the caller's stream is done, i.e. when the kernels that read
    // weights over the link themselves have finished and the link would go idle
    AG_CUDA(cudaEventRecord(st.gate, static_cast<cudaStream_t>(after_stream)));
    AG_CUDA(cudaStreamWaitEvent(st.copy, st.gate, 0));
  }
  int i = 0;
  for (int lo = 0; lo < num_groups && i < ring.slots; lo += ring.chunk, ++i) {
    const int cnt = num_groups - lo < ring.chunk ? num_groups - lo : ring.chunk;
    if (int rc = stage_copy(st, b, stage, ring, expert_bytes, i, lo, cnt)) return rc;
  }
  st.pf_b = b;
  st.pf_stage = stage;
  st.pf_expert_bytes = expert_bytes;
  st.pf_slot_bytes = ring.slot_bytes;
  st.pf_slots = ring.slots;
  st.pf_count = i;
  return AG_OK;
}

int ag_prepare_weights(void* ptr, uint64_t bytes, int32_t read_only) {
  AG_REQUIRE(ptr != nullptr && bytes > 0, "ptr must be non-NULL and bytes positive");
  const void* alias = nullptr;
  if (classify(ptr, &alias) != RES_UNREACHABLE) return AG_OK;   // device memory, or already pinned / registered
  std::lock_guard<std::mutex> lk(g_reg_mu);
  int slot = -1;
  for (int i = 0; i < 256 && slot < 0; ++i)
    if (g_registered[i] == nullptr) slot = i;
  AG_REQUIRE(slot >= 0, "too many ranges registered through ag_prepare_weights (256)");
  unsigned flags = cudaHostRegisterPortable | cudaHostRegisterMapped;
  if (read_only) flags |= cudaHostRegisterReadOnly;
  cudaError_t e = cudaHostRegister(ptr, bytes, flags);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(AG_E_CUDA, "cudaHostRegister(%p, %llu bytes%s) failed: %s", ptr, static_cast<unsigned long long>(bytes),
                read_only ? ", read-only" : "", cudaGetErrorString(e));
  }
  g_registered[slot] = ptr;
  return AG_OK;
}

int ag_release_weights(void* ptr) {
  AG_REQUIRE(ptr != nullptr, "ptr must be non-NULL");
  std::lock_guard<std::mutex> lk(g_reg_mu);
  for (int i = 0; i < 256; ++i) {
    if (g_registered[i] != ptr) continue;
    AG_CUDA(cudaHostUnregister(ptr));
    g_registered[i] = nullptr;
    return AG_OK;
  }
  return fail(AG_E_INVALID, "%p was not registered through ag_prepare_weights", ptr);
}

int ag_measure_host_link(uint64_t bytes, int32_t reps, double* gbps_out) {
  AG_REQUIRE(gbps_out != nullptr && bytes > 0, "bad arguments");
  void *h = nullptr, *d = nullptr;
  AG_CUDA(cudaHostAlloc(&h, bytes, cudaHostAllocDefault));
  if (cudaMalloc(&d, bytes) != cudaSuccess) {
    cudaFreeHost(h);
    return fail(AG_E_CUDA, "cudaMalloc(%llu) failed", static_cast<unsigned long long>(bytes));
  }
  std::memset(h, 1, bytes);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  double best = 0;
  for (int r = 0; r < (reps > 0 ? reps : 3); ++r) {
    cudaEventRecord(e0, 0);
    cudaMemcpyAsync(d, h, bytes, cudaMemcpyHostToDevice, 0);
    cudaEventRecord(e1, 0);
    cudaEventSynchronize(e1);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    if (ms > 0) {
      const double g = static_cast<double>(bytes) / (ms * 1e6);
      if (g > best) best = g;
    }
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(d);
  cudaFreeHost(h);
  *gbps_out = best;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(AG_E_CUDA, "CUDA error while measuring the host link: %s", cudaGetErrorString(e));
  return AG_OK;
}

const char* ag_last_error(void) { return g_err; }
const char* ag_version(void) { return "asymgemm_b200 0.1 (sm_100a)"; }

}  // extern "C"

namespace agb {
cudaError_t launch_operand_feed_probe(const CUtensorMap& ma, const CUtensorMap& mb, int sms, int items, int kb_count, int load_a, int load_b,
                                      int rows_a, int rows_b, long long* cycles, int* failed);
}

extern "C" int ag_probe_operand_feed(int32_t load_a, int32_t load_b, double* cycles_per_k_atom) {
  AG_REQUIRE(cycles_per_k_atom != nullptr, "cycles_per_k_atom is NULL");
  int sms = 0;
  if (int rc = device_sm_count(&sms)) return rc;
  constexpr int kRowBytes = 4096, kRowsA = 65536, kRowsB = 128 * 1536, kItems = 12, kAtoms = 32;   // 256 MB + 768 MB
  void *a = nullptr, *b = nullptr;
  long long* cycles = nullptr;
  int* failed = nullptr;
  std::vector<long long> host(2 * static_cast<size_t>(sms), 0);
  int host_failed = 0, rc = AG_OK;
  cudaError_t e = cudaMalloc(&a, static_cast<size_t>(kRowsA) * kRowBytes);
  if (e == cudaSuccess) e = cudaMalloc(&b, static_cast<size_t>(kRowsB) * kRowBytes);
  if (e == cudaSuccess) e = cudaMalloc(&cycles, sizeof(long long) * 2 * sms);
  if (e == cudaSuccess) e = cudaMalloc(&failed, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(a, 0, static_cast<size_t>(kRowsA) * kRowBytes);
  if (e == cudaSuccess) e = cudaMemset(b, 0, static_cast<size_t>(kRowsB) * kRowBytes);
  if (e == cudaSuccess) e = cudaMemset(cycles, 0, sizeof(long long) * 2 * sms);
  if (e == cudaSuccess) e = cudaMemset(failed, 0, sizeof(int));
  if (e == cudaSuccess) {
    CUtensorMap ma, mb;
    rc = encode_bytes_2d(&ma, a, kRowBytes, kRowsA, kRowBytes, 128, "probe a");
    if (rc == AG_OK) rc = encode_bytes_2d(&mb, b, kRowBytes, kRowsB, kRowBytes, 256, "probe b");
    if (rc == AG_OK) {
      for (int rep = 0; rep < 2 && e == cudaSuccess; ++rep) {   // the second pass finds the tensor maps and L2 warm
        e = agb::launch_operand_feed_probe(ma, mb, sms, kItems, kAtoms, load_a != 0, load_b != 0, kRowsA, kRowsB, cycles, failed);
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
      }
      if (e == cudaSuccess) e = cudaMemcpy(host.data(), cycles, sizeof(long long) * 2 * sms, cudaMemcpyDeviceToHost);
      if (e == cudaSuccess) e = cudaMemcpy(&host_failed, failed, sizeof(int), cudaMemcpyDeviceToHost);
    }
  }
  cudaFree(a);
  cudaFree(b);
  cudaFree(cycles);
  cudaFree(failed);
  if (rc != AG_OK) return rc;
  if (e != cudaSuccess) return fail(AG_E_CUDA, "operand-feed probe: %s", cudaGetErrorString(e));
  long long worst = 0;
  for (long long c : host) {
    if (c < 0) host_failed = 1;
    worst = c > worst ? c : worst;
  }
  if (host_failed) return fail(AG_E_DEVICE, "the operand-feed probe gave up waiting on one of its barriers");
  *cycles_per_k_atom = static_cast<double>(worst) / (static_cast<double>(kItems) * kAtoms);
  return AG_OK;
}
