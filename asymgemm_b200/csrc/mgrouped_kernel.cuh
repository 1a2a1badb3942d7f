// m-grouped asymmetric GEMM for sm_100a: D[rows of segment s] = A[rows of s] x B[expert(s)]^T, where the
// weight tensor B [G, N, K] (K-major) may live in pinned, device-mapped host memory and is streamed by
// TMA straight into a shared-memory ring, while A and D live in HBM.
//
// Work decomposition (replaces the reference's one-CTA-per-(n-block, segment) grid and its single B
// slot, asym_gemm/include/asym_gemm/common/asymScheduler.cuh:92-124 and
// asym_gemm/include/asym_gemm/impls/sm100_fp8_asym_gemm_1d1d.cuh:255-330,471):
//   * an item is (segment, n-tile); a persistent CTA takes items c, c+grid, ... with the n-tile index
//     fastest, so CTAs that run together share the same activation rows in L2;
//   * an item's weight column (BN rows x K) is fetched over the host link exactly once. The segment's
//     rows are processed in chunks of CHUNK_TILES 128-row tiles whose fp32/int32 accumulators stay in
//     TMEM across the whole K loop (K outer, M inner inside a chunk). Segments longer than one chunk
//     replay the column from a per-CTA scratch copy in device memory that the first pass writes with a
//     TMA store of the very shared-memory stage the MMA consumes (no second trip over the host link);
//   * no atomics, no partial sums in D: every output element is written once, from fp32;
//   * when B is device-resident there is no link to spare, so long segments are split into accumulator-sized row
//     chunks that become items of their own (fetch_item, split mode) and spread over all CTAs.
//   * which items a CTA takes is worked out once, by all of its threads, into a table in shared memory (build_work_list);
//     the roles read one entry per item instead of walking the segment list.
//
// Tile shape is chosen by where B lives. Streaming from the host, throughput drops once the rows being streamed at
// the same time (CTAs x BN) spread over more than a few thousand 4 KB host pages (measured: 148 CTAs x 128 rows ->
// 44.5 GB/s, 148 x 32 rows -> 51.4 GB/s of a 55.6 GB/s copy-engine peak), so host-resident B uses BN = 64 or 32 with
// KA = several 128-byte K atoms per stage; device-resident B uses BN = 128 or 256 with KA = 1: there the bound is the
// operand traffic from L2 into shared memory, and flops per operand byte grow with the tile.
//
// Four operand kinds share the body: BF16 and NVFP4 accumulate in TMEM in hardware (NVFP4 with its UE4M3 scale
// factors copied into TMEM by tcgen05.cp); FP8 and INT8 produce one raw product per 128-wide K block that the drain warps
// scale in fp32 (block scales are arbitrary fp32 numbers) and add to accumulators kept in TMEM, or in registers (REG_ACC).
//
// Warp roles: warp 0 = B producer (+ scratch spill), warp 1 = A producer (one lane per MMA issuer), warp 2 = TMEM allocator,
// warps 2 and 3 = one tcgen05.mma-issuing thread each (one issuer for block-scaled 64-column tiles), warps 4-7 (and 8-11 where a
// second drain warpgroup pays, see drain_wgs_of) = TMEM drain.
//
// Every mbarrier wait is bounded by a wall-clock limit; on expiry the CTA records a status code, raises a
// shared abort flag that all roles poll, waits for its own copies in flight, frees TMEM and returns.
#pragma once
#include <utility>
#include <cuda_bf16.h>

#include <type_traits>

#include "ptx.cuh"

namespace agb {

enum class Kind : int { BF16 = 0, FP8 = 1, INT8 = 2, NVFP4 = 3, FP8_UE8M0 = 4 };
enum : int { LAYOUT_CONTIGUOUS = 0, LAYOUT_MASKED = 1 };

// status codes written to GemmParams::status (low byte = code, upper bits = CTA index)
enum : int {
  ST_OK = 0,
  ST_TIMEOUT_B_EMPTY = 1,
  ST_TIMEOUT_A_EMPTY = 2,
  ST_TIMEOUT_B_FULL = 3,
  ST_TIMEOUT_A_FULL = 4,
  ST_TIMEOUT_TM_EMPTY = 5,
  ST_TIMEOUT_TM_FULL = 6,
  ST_TIMEOUT_DRAIN = 7,
  ST_BAD_EXPERT = 8,
  ST_TIMEOUT_PROBE = 9,
};

struct GemmParams {
  const float* sfa;        // FP8/INT8: [rows, sf_k] fp32.  NVFP4: blocked UE4M3 bytes (see sf_layout.cuh)
  const float* sfb;        // FP8: [G, ceil(N/128), sf_k]; INT8: [G, N, sf_k]; NVFP4: blocked UE4M3 bytes
  void* d;                 // [rows, N] bf16 or fp32
  const int* offsets;      // contiguous: (start, end) row pairs per segment
  const int* experts;      // contiguous: weight index per segment, list ends at the first negative entry
  const int* masked_m;     // masked: valid rows per group
  int* status;             // one word, 0 = ok
  int* raw_dump;           // INT8 debug hook: int32 block sums [sf_k, rows, N] before scaling, or null
  unsigned long long timeout_ns;
  long long rows_total;    // rows of A / D (contiguous: M, masked: G * m_max)
  int layout;
  int max_segments;        // contiguous: upper bound on segments to visit; masked: G
  int m_max;               // masked: rows per group
  int num_groups;
  int n;
  int n_tiles;             // ceil(N / BN)
  int kb_count;            // ceil(K bytes / 128)
  int sf_k;                // scale blocks along K (FP8/INT8: ceil(K/128); NVFP4: padded count of 64-element blocks)
  int sfb_rows;            // FP8: ceil(N/128); INT8: N; NVFP4: ceil(N/128)
  int d_fp32;
  int use_scratch;         // 1 = replay long segments from the scratch copy, 0 = re-read B from its source
  int b_streaming;         // 1 = B is host memory: mark its lines evict-first in L2
  int split_rows;          // > 0: split segments into chunks of this many rows (one accumulator chunk) per item
  int expert_lo;           // this launch serves the experts [expert_lo, expert_lo + expert_n) only (a staged chunk of the
  int expert_n;            // weights): segments of other experts are skipped, and B holds just these experts' rows
  float alpha;             // NVFP4 global scale (product of the two tensor-level scales), 1.0 otherwise
  int epilogue;            // FP8 only. 1 = the weight rows hold gate and up columns interleaved in groups of 16 (rows 32q..32q+15 =
                           // gate columns 16q.., rows 32q+16..32q+31 = the same up columns) and the drain writes bf16(silu(gate) * up)
                           // into d [rows, n / 2] instead of the raw product
  int d_cols;              // row length of d in elements: n, or n / 2 with the fused activation
  const long long* scatter_meta;    // optional, per row of the product: (buffer index << 32) | row in that buffer, negative = drop
  const long long* scatter_bases;   // optional: addresses of the destination buffers (local or peer memory); both or neither
};

// Where row `grow` of the product goes: d's own row, or -- with a scatter table -- the row its entry names in one of the
// destination buffers (the expert-parallel layer's combine buffers on the ranks the tokens came from). Null = not stored.
__device__ __forceinline__ void* result_row(const GemmParams& p, long long grow, int elem_bytes) {
  if (p.scatter_meta == nullptr) return static_cast<char*>(p.d) + grow * p.d_cols * elem_bytes;
  const long long m = __ldg(p.scatter_meta + grow);
  if (m < 0) return nullptr;
  char* base = reinterpret_cast<char*>(static_cast<uintptr_t>(__ldg(p.scatter_bases + (m >> 32))));
  return base + (m & 0xffffffffLL) * p.d_cols * elem_bytes;
}

struct Item {
  int expert;
  int row0;
  int rows;
  int nt;
};

// ----------------------------------------------------------------------------- work list of a CTA
// Which (segment, row chunk, n-tile) items a CTA works on follows from the segment list in device memory. Every role of the
// CTA needs that sequence, and the roles that matter are single threads whose every instruction is on the critical path of
// the tensor core: walking the segment list there (dependent loads, divisions) cost a quarter of the run time with 128
// segments. So all threads of the CTA build the list once, in shared memory, before the roles start:
//   1. the raw segment entries are copied in (3 ints per segment: contiguous = expert, row begin, row end; masked = rows),
//   2. one warp turns the items per segment into running sums,
//   3. thread i finds item `first + i * stride` by bisection in the sums and writes {expert, row0, rows, n-tile}.
// A role then reads one int4 per item. Lists longer than the table, or segment lists longer than the cache, fall back
// to the walk (fetch_item), which enumerates the items in exactly the same order.
struct SegCache {
  const int* data = nullptr;
  int count = 0;
};

struct WorkList {
  const int4* items = nullptr;   // {expert, row0, rows, n-tile}; rows < 0 ends the list
  int count = 0;                 // entries built; beyond them the roles walk the segment list
  long long first = 0, stride = 1;   // this CTA's i-th item is item `first + i * stride` of the launch
  SegCache segs;
};

// Expert, first row and row count of a segment from its raw entry. `report`: flag an expert index outside B.
__device__ __forceinline__ void decode_segment(const GemmParams& p, int seg, int raw0, int raw1, int raw2, bool report, int& expert, int& row0,
                                               int& rows) {
  if (p.layout == LAYOUT_MASKED) {
    expert = seg;
    row0 = seg * p.m_max;
    rows = raw0 < 0 ? 0 : (raw0 > p.m_max ? p.m_max : raw0);
    if (static_cast<unsigned>(seg - p.expert_lo) >= static_cast<unsigned>(p.expert_n)) rows = 0;  // another launch's expert
  } else {
    expert = raw0;
    int r0 = raw1, r1 = raw2;
    if (r0 < 0) r0 = 0;
    if (r1 > p.rows_total) r1 = static_cast<int>(p.rows_total);
    row0 = r0;
    rows = r1 > r0 ? r1 - r0 : 0;
    if (raw0 >= p.num_groups) {  // would read outside B: flag it and skip
      if (report) atomicCAS(p.status, 0, ST_BAD_EXPERT | (static_cast<int>(blockIdx.x) << 8));
      rows = 0;
    } else if (static_cast<unsigned>(raw0 - p.expert_lo) >= static_cast<unsigned>(p.expert_n)) {
      rows = 0;  // another launch's expert
    }
  }
}

// Items of a segment with `rows` valid rows. Whole-segment mode: one per n-tile. Split mode: its row chunks x n-tiles, in two
// classes that are enumerated one after the other over ALL segments: first every full chunk (class 0), then the shorter
// last chunk of every segment (class 1). Items are dealt to the CTAs in turn, and a full chunk is up to twice the work of
// a tail; with the tails last every CTA gets the same number of full chunks (+-1) and the tails even out what is left
// (in segment order one CTA of the BF16 benchmark case had 832 steps against a mean of 746; tails last: 768).
__device__ __forceinline__ int items_of_segment(const GemmParams& p, int rows, int klass) {
  if (p.split_rows <= 0) return klass == 0 ? p.n_tiles : 0;
  return klass == 0 ? (rows / p.split_rows) * p.n_tiles : ((rows % p.split_rows) ? p.n_tiles : 0);
}

// Called by every thread of the CTA, before the first __syncthreads() that precedes the roles. `seg_data` holds
// 3 * SEG_CAP ints, `seg_first` 2 * SEG_CAP + 2 ints (the last one is scratch), `items` ITEM_CAP entries.
template <int SEG_CAP, int ITEM_CAP>
__device__ __forceinline__ WorkList build_work_list(const GemmParams& p, int* seg_data, int* seg_first, int4* items, long long first,
                                                    long long stride) {
  WorkList wl;
  wl.first = first;
  wl.stride = stride;
  if constexpr (SEG_CAP == 0 || ITEM_CAP == 0) return wl;
  const int cached = min(p.max_segments, SEG_CAP);
  int* list_end = seg_first + 2 * SEG_CAP + 1;       // index of the first negative expert (contiguous layout)
  if (threadIdx.x == 0) *list_end = cached;
  __syncthreads();
  for (int seg = threadIdx.x; seg < cached; seg += blockDim.x) {
    if (p.layout == LAYOUT_MASKED) {
      seg_data[3 * seg] = __ldg(p.masked_m + seg);
    } else {
      const int e = __ldg(p.experts + seg);
      seg_data[3 * seg] = e;
      seg_data[3 * seg + 1] = __ldg(p.offsets + 2 * seg);
      seg_data[3 * seg + 2] = __ldg(p.offsets + 2 * seg + 1);
      if (e < 0) atomicMin(list_end, seg);
    }
  }
  wl.segs.data = seg_data;
  wl.segs.count = cached;
  __syncthreads();
  if (p.max_segments > SEG_CAP) return wl;           // the whole list does not fit: every role walks it
  const int nseg = *list_end;
  const int nvirt = 2 * nseg;                        // entries [0, nseg): class 0 of every segment; [nseg, 2 nseg): class 1
  for (int seg = threadIdx.x; seg < nseg; seg += blockDim.x) {
    int expert, row0, rows;
    decode_segment(p, seg, seg_data[3 * seg], seg_data[3 * seg + 1], seg_data[3 * seg + 2], true, expert, row0, rows);
    seg_first[seg] = items_of_segment(p, rows, 0);
    seg_first[nseg + seg] = items_of_segment(p, rows, 1);
  }
  __syncthreads();
  if (threadIdx.x < 32) {                            // exclusive running sums, 32 entries per step
    int carry = 0;
    for (int base = 0; base < nvirt; base += 32) {
      const int seg = base + static_cast<int>(threadIdx.x);
      const int v = seg < nvirt ? seg_first[seg] : 0;
      int incl = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, d);
        if (static_cast<int>(threadIdx.x) >= d) incl += up;
      }
      if (seg < nvirt) seg_first[seg] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (threadIdx.x == 0) seg_first[nvirt] = carry;
  }
  __syncthreads();
  const long long total = seg_first[nvirt];
  for (int i = threadIdx.x; i < ITEM_CAP; i += blockDim.x) {
    const long long id = first + static_cast<long long>(i) * stride;
    int4 v = make_int4(0, 0, -1, 0);
    if (id < total) {
      int lo = 0, hi = nvirt;                        // the last entry whose first item is <= id
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (seg_first[mid] <= id) lo = mid; else hi = mid;
      }
      const int klass = lo >= nseg ? 1 : 0, seg = lo - klass * nseg;
      int expert, row0, rows;
      decode_segment(p, seg, seg_data[3 * seg], seg_data[3 * seg + 1], seg_data[3 * seg + 2], false, expert, row0, rows);
      const int local = static_cast<int>(id - seg_first[lo]);
      const int within = local / p.n_tiles;          // chunk within the class
      const int chunk = p.split_rows > 0 ? (klass == 0 ? within : rows / p.split_rows) : 0;
      v.x = expert;
      v.w = local - within * p.n_tiles;
      v.y = row0 + chunk * p.split_rows;
      v.z = p.split_rows > 0 ? (klass == 0 ? p.split_rows : rows % p.split_rows) : rows;
    }
    items[i] = v;
  }
  wl.items = items;
  wl.count = ITEM_CAP;
  return wl;                                         // the caller's __syncthreads() publishes the table
}

// Row range and weight index of segment `seg`. Returns 0 past the end of the segment list.
__device__ __forceinline__ int read_segment(const GemmParams& p, const SegCache& sc, int seg, int& expert, int& row0, int& rows) {
  if (seg >= p.max_segments) return 0;
  int raw0, raw1 = 0, raw2 = 0;
  if (seg < sc.count) {
    raw0 = sc.data[3 * seg];
    raw1 = sc.data[3 * seg + 1];
    raw2 = sc.data[3 * seg + 2];
  } else if (p.layout == LAYOUT_MASKED) {
    raw0 = __ldg(p.masked_m + seg);
  } else {
    raw0 = __ldg(p.experts + seg);
    if (raw0 >= 0) {
      raw1 = __ldg(p.offsets + 2 * seg);
      raw2 = __ldg(p.offsets + 2 * seg + 1);
    }
  }
  if (p.layout != LAYOUT_MASKED && raw0 < 0) return 0;
  decode_segment(p, seg, raw0, raw1, raw2, true, expert, row0, rows);
  return 1;
}

// Position of a role's walk through the item list when segments are split into row chunks (p.split_rows > 0).
struct ItemCursor {
  int seg = 0;
  int klass = 0;        // split mode: 0 = walking the full chunks of all segments, 1 = their tails (which come after)
  long long first = 0;  // index of the first item of segment `seg` in class `klass`
  SegCache cache;       // where the first segments' entries can be read from shared memory
  __device__ ItemCursor() {}
  __device__ explicit ItemCursor(const SegCache& c) : cache(c) {}
};

// Maps item index -> work. Returns 0 when the CTA has run out of work, 1 otherwise (rows may still be 0: skip).
// Whole-segment mode (weights streamed from the host): item = (segment, n-tile), the segment's column is fetched once.
// Split mode (weights in device memory, p.split_rows = rows of one accumulator chunk): item = (segment, row chunk, n-tile)
// with the n-tile fastest, so that long segments spread over many CTAs and CTAs running together share A rows in L2.
// Item indices seen by one role only grow, so the cursor advances monotonically: O(segments) reads per CTA in total.
__device__ __forceinline__ int fetch_item(const GemmParams& p, long long item, ItemCursor& cur, Item& it) {
  if (p.split_rows <= 0) {
    const int seg = static_cast<int>(item / p.n_tiles);
    it.nt = static_cast<int>(item - static_cast<long long>(seg) * p.n_tiles);
    return read_segment(p, cur.cache, seg, it.expert, it.row0, it.rows);
  }
  while (true) {
    int expert, row0, rows;
    if (!read_segment(p, cur.cache, cur.seg, expert, row0, rows)) {
      if (cur.klass == 1) return 0;
      cur.klass = 1;      // every full chunk has been handed out: the tails follow, from the first segment again
      cur.seg = 0;
      continue;
    }
    const long long count = items_of_segment(p, rows, cur.klass);
    const long long local = item - cur.first;
    if (local < count) {
      const int within = static_cast<int>(local / p.n_tiles);
      const int chunk = cur.klass == 0 ? within : rows / p.split_rows;
      it.nt = static_cast<int>(local - static_cast<long long>(within) * p.n_tiles);
      it.expert = expert;
      it.row0 = row0 + chunk * p.split_rows;
      it.rows = cur.klass == 0 ? p.split_rows : rows % p.split_rows;
      return 1;
    }
    cur.first += count;
    ++cur.seg;
  }
}

// The i-th item of this CTA: from the table where it reaches, from the walk beyond it.
__device__ __forceinline__ int get_item(const GemmParams& p, const WorkList& wl, int i, ItemCursor& cur, Item& it) {
  if (i < wl.count) {
    const int4 v = wl.items[i];
    if (v.z < 0) return 0;
    it.expert = v.x;
    it.row0 = v.y;
    it.rows = v.z;
    it.nt = v.w;
    return 1;
  }
  return fetch_item(p, wl.first + static_cast<long long>(i) * wl.stride, cur, it);
}

// Position of a user's n-th step in the activation ring. With two MMA issuers the ring is split in halves, one per issuer,
// so that every barrier has ONE consumer who sees each of its phases: a phase test by parity is only valid while the tester
// is less than two phases away from the barrier, and an issuer that has no step for a while (a chunk with a single row
// tile belongs to the other one) would otherwise run ahead of the producer by more than that.
template <int SA, bool DUAL>
struct ARing {
  static constexpr uint32_t PER = DUAL ? SA / 2 : SA;
  static_assert(!DUAL || (SA % 2 == 0 && SA >= 2), "two issuers need an even number of activation stages");
  __device__ static uint32_t stage(uint32_t user, uint32_t n) { return (DUAL ? user * PER : 0u) + n % PER; }
  __device__ static uint32_t phase(uint32_t n) { return (n / PER) & 1u; }
};

template <typename F, int... I>
__device__ __forceinline__ void for_each_index(std::integer_sequence<int, I...>, F&& f) {
  (f(std::integral_constant<int, I>{}), ...);
}

struct WaitCtx {
  int* status;
  volatile int* abort_flag;
  unsigned long long timeout_ns;
};

// Bounded wait. Returns false if the CTA is aborting (either this wait expired or another role's did).
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, const WaitCtx& c, int code, bool honor_abort = true) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t n = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++n & 63u) == 0) {
      if (honor_abort && *c.abort_flag) return false;
      if (global_timer_ns() - t0 > c.timeout_ns) {
        atomicCAS(c.status, 0, code | (static_cast<int>(blockIdx.x) << 8));
        *c.abort_flag = 1;
        return false;
      }
    }
  }
}

template <Kind KIND>
struct KindTraits;
template <>
struct KindTraits<Kind::BF16> {
  static constexpr MmaKind mma = MmaKind::F16;
  static constexpr bool sw_scale = false;
  static constexpr bool block_scaled = false;
  static constexpr uint32_t d_fmt = 1, ab_fmt = 1;
};
template <>
struct KindTraits<Kind::FP8> {
  static constexpr MmaKind mma = MmaKind::F8F6F4;
  static constexpr bool sw_scale = true;
  static constexpr bool block_scaled = false;
  static constexpr uint32_t d_fmt = 1, ab_fmt = 0;
};
template <>
struct KindTraits<Kind::INT8> {
  static constexpr MmaKind mma = MmaKind::I8;
  static constexpr bool sw_scale = true;
  static constexpr bool block_scaled = false;
  static constexpr uint32_t d_fmt = 2, ab_fmt = 1;
};
// NVFP4: the tensor core applies one UE4M3 scale per 16 elements of K to each operand; scales are read from TMEM.
template <>
struct KindTraits<Kind::NVFP4> {
  static constexpr MmaKind mma = MmaKind::F16;  // unused: block-scaled MMAs are issued through umma_nvfp4
  static constexpr bool sw_scale = false;
  static constexpr bool block_scaled = true;
  static constexpr uint32_t d_fmt = 1, ab_fmt = 1;
};
// FP8 with power-of-two block scales applied by the tensor core (what the reference's SM100 FP8 kernel does,
// asym_gemm/include/asym_gemm/impls/sm100_fp8_asym_gemm_1d1d.cuh:433-462): one UE8M0 byte per row and 128-wide K block,
// four K blocks per 32-bit TMEM word, the byte picked by the descriptor's sf-id. No drain-side arithmetic.
template <>
struct KindTraits<Kind::FP8_UE8M0> {
  static constexpr MmaKind mma = MmaKind::F8F6F4;  // unused: issued through umma_mxfp8
  static constexpr bool sw_scale = false;
  static constexpr bool block_scaled = true;
  static constexpr uint32_t d_fmt = 1, ab_fmt = 0;
};

constexpr int BM = 128;            // rows per MMA tile
constexpr int ATOM_BYTES = 128;    // bytes of K per pipeline stage row (one 128-byte swizzle atom)
constexpr int MMA_K_BYTES = 32;    // bytes of K per tcgen05.mma
constexpr int NUM_THREADS = 256;
constexpr int TMEM_COLS = 512;
// NVFP4 scale factors. One tcgen05.mma covers 64 elements of K = 4 scales per row; the scales of 128 rows for one
// MMA form a 512-byte block laid out as byte (r % 32) * 16 + (r / 32) * 4 + c, which tcgen05.cp (32x128b.warpx4)
// turns into 4 TMEM columns. One 128-byte K atom (256 elements) needs 4 such blocks per operand = 2 KB.
constexpr int SF_BLOCK_BYTES = 512;
constexpr int SF_ATOM_BYTES = 4 * SF_BLOCK_BYTES;
constexpr int SF_TMEM_COLS = 64;   // A: 2 x 16 columns, B: 2 x 16 columns (double-buffered)

// Scale-factor bytes staged with every A stage / B stage (0 for kinds without hardware block scaling).
// NVFP4: 2 KB per 128-byte K atom. FP8_UE8M0: one 512-byte block covers four K atoms; it travels with every stage.
template <Kind KIND, int KA>
struct SfStage {
  static constexpr int a = KIND == Kind::NVFP4 ? SF_ATOM_BYTES : (KIND == Kind::FP8_UE8M0 ? SF_BLOCK_BYTES : 0);
  static constexpr int b = KIND == Kind::NVFP4 ? SF_ATOM_BYTES * KA : (KIND == Kind::FP8_UE8M0 ? SF_BLOCK_BYTES : 0);
};

constexpr int work_list_bytes(int segs, int items) { return segs * 12 + (2 * segs + 2) * 4 + 16 + items * 16; }

template <int BN, int KA, int SA, int SB, int SFA_BYTES = 0, int SFB_BYTES = 0>
struct SmemLayout {
  static constexpr int a_stage = BM * ATOM_BYTES;
  static constexpr int b_box = BN * ATOM_BYTES;       // one TMA box: BN rows x 128 bytes of K
  static constexpr int b_stage = b_box * KA;          // KA K-adjacent boxes per stage
  static constexpr int a_off = 0;
  static constexpr int b_off = a_off + SA * a_stage;
  static constexpr int sfa_stage = SFA_BYTES;
  static constexpr int sfb_stage = SFB_BYTES;
  static constexpr int sfa_off = b_off + SB * b_stage;
  static constexpr int sfb2_off = sfa_off + SA * sfa_stage;
  static constexpr int bar_off = sfb2_off + SB * sfb_stage;
  static constexpr int num_bars = 2 * SA + 2 * SB + 32 + 2;
  static constexpr int sfb_off = bar_off + num_bars * 8;          // 4 warps x BN floats (INT8 column scales)
  static constexpr int misc_off = sfb_off + 4 * BN * 4;           // tmem base, abort flag
  // work list (build_work_list): as large as what is left of the 227 KB allows
  static constexpr int work_off = misc_off + 16;
  static constexpr int work_room = 232448 - 1024 - work_off;
  static constexpr int seg_cap = work_room >= work_list_bytes(1024, 512) ? 1024 : (work_room >= work_list_bytes(256, 128) ? 256 : 0);
  static constexpr int item_cap = seg_cap / 2;
  static constexpr int seg_first_off = work_off + seg_cap * 12;
  static constexpr int items_off = (seg_first_off + (2 * seg_cap + 2) * 4 + 15) / 16 * 16;
  static constexpr int total = items_off + item_cap * 16;
  static constexpr int dyn_bytes = total + 1024;                  // slack for manual 1024-byte alignment
};

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Store 32 consecutive output columns of one row. `vals` are fp32 bit patterns.
__device__ __forceinline__ void store_row32(const GemmParams& p, long long grow, int col0, const uint32_t (&vals)[32]) {
  if (p.d_fp32) {
    float* row = static_cast<float*>(result_row(p, grow, 4));
    if (row == nullptr) return;
    float* dst = row + col0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (col0 + j * 4 < p.n) {
        uint4 v = make_uint4(vals[4 * j], vals[4 * j + 1], vals[4 * j + 2], vals[4 * j + 3]);
        *reinterpret_cast<uint4*>(dst + 4 * j) = v;
      }
    }
  } else {
    __nv_bfloat16* row = static_cast<__nv_bfloat16*>(result_row(p, grow, 2));
    if (row == nullptr) return;
    __nv_bfloat16* dst = row + col0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (col0 + j * 8 < p.n) {
        uint4 v;
        v.x = pack_bf16(__uint_as_float(vals[8 * j + 0]), __uint_as_float(vals[8 * j + 1]));
        v.y = pack_bf16(__uint_as_float(vals[8 * j + 2]), __uint_as_float(vals[8 * j + 3]));
        v.z = pack_bf16(__uint_as_float(vals[8 * j + 4]), __uint_as_float(vals[8 * j + 5]));
        v.w = pack_bf16(__uint_as_float(vals[8 * j + 6]), __uint_as_float(vals[8 * j + 7]));
        *reinterpret_cast<uint4*>(dst + 8 * j) = v;
      }
    }
  }
}

// Fused activation of an FP8 gate+up product: `vals` are the fp32 results of 32 consecutive (interleaved) weight rows, 16 gate
// columns followed by the 16 up columns of the same index. Each is rounded to bf16 exactly as the unfused operator would have
// written it, then act = bf16(silu(gate) * up) with silu(g) = g / (1 + exp(-g)) in fp32 -- the arithmetic of the separate
// activation kernel and of the reference's CPU bucket (csrc/cpu/module.cpp:337-347), so fused and unfused agree bit for bit.
// Writes 16 bf16 values at d[grow, col0 / 2 ..].
__device__ __forceinline__ void store_silu_mul16(const GemmParams& p, long long grow, int col0, const uint32_t (&vals)[32]) {
  if (col0 >= p.n) return;
  uint32_t packed[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float act[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(vals[2 * j + h])));
      const float u = __bfloat162float(__float2bfloat16_rn(__uint_as_float(vals[16 + 2 * j + h])));
      const float sg = g / (1.0f + expf(-g));
      act[h] = sg * u;
    }
    packed[j] = pack_bf16(act[0], act[1]);
  }
  __nv_bfloat16* row = static_cast<__nv_bfloat16*>(result_row(p, grow, 2));
  if (row == nullptr) return;
  __nv_bfloat16* dst = row + (col0 >> 1);
  *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  *reinterpret_cast<uint4*>(dst + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
}

// REG_ACC (software-scaled kinds only): the scaled fp32 accumulators of ONE 128-row tile live in the drain warps'
// registers instead of TMEM, all TMEM slots hold raw per-K-block products (a 512/BN-deep MMA pipeline) and the drain
// does one tcgen05.ld + fma per block instead of ld + ld + st. Used when the weights are device-resident, where items are
// one tile tall anyway and the drain, not the host link, sets the pace.
// Drain warpgroups. The software-scaled kinds use two (384 threads) wherever a tile is at least 64 columns wide: warps
// 4-7 own the low half of the tile's columns, warps 8-11 the high half, and the two groups drain a raw slot side by
// side (INT8 with REG_ACC: 272 -> 383 TFLOP/s on the 16-expert case). The exception is FP8 with REG_ACC on 128 columns,
// whose block scale is one scalar per tile: it is bound by operand traffic, not by the drain, and measured slightly
// faster with one. 256-column tiles always use two groups, whatever the kind (128 columns, and for REG_ACC 128
// accumulator registers, per thread).
template <Kind KIND, int BN, bool REG_ACC>
__host__ __device__ constexpr int drain_wgs_of() {
  if (BN == 256) return 2;
  return (KIND != Kind::FP8 && KIND != Kind::INT8) ? 1 : (REG_ACC ? (KIND == Kind::INT8 ? 2 : 1) : (BN >= 64 ? 2 : 1));
}
template <Kind KIND, int BN, bool REG_ACC>
__host__ __device__ constexpr int num_threads_of() { return 128 + 128 * drain_wgs_of<KIND, BN, REG_ACC>(); }
template <Kind KIND, int BN, int KA, int SA, int SB, bool REG_ACC = false>
__global__ void __launch_bounds__(num_threads_of<KIND, BN, REG_ACC>(), 1)
mgrouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_s, const GemmParams p) {
  using T = KindTraits<KIND>;
  using L = SmemLayout<BN, KA, SA, SB, SfStage<KIND, KA>::a, SfStage<KIND, KA>::b>;
  static_assert(KIND != Kind::FP8_UE8M0 || (KA == 1 || KA == 2 || KA == 4), "a UE8M0 scale block spans four K atoms");
  static_assert(BN == 32 || BN == 64 || BN == 128 || BN == 256, "BN must be 32, 64, 128 or 256");
  static_assert(!T::block_scaled || BN <= 128, "block-scaled kinds keep their scale factors in TMEM columns laid out for at most 128 weight rows");
  static_assert(!T::block_scaled || BN >= 64, "block-scaled kinds need BN >= 64");
  // TMEM plan: 512 / BN slots of BN columns. Hardware-accumulated kinds keep one output tile per slot; software-scaled
  // kinds keep scaled fp32 tiles in slots [0, CHUNK_TILES) and double-buffer the raw per-K-block product in the last two.
  constexpr int NUM_SLOTS = (TMEM_COLS - (T::block_scaled ? SF_TMEM_COLS : 0)) / BN;
  static_assert(!REG_ACC || T::sw_scale, "REG_ACC applies to the software-scaled kinds");
  static_assert(!T::sw_scale || REG_ACC || NUM_SLOTS > 2, "software-scaled kinds need TMEM room for two raw slots and at least one accumulator tile");
  constexpr int RAW_SLOTS = REG_ACC ? NUM_SLOTS : 2;                 // raw product slots (software-scaled kinds)
  constexpr int CHUNK_TILES = T::sw_scale ? (REG_ACC ? 1 : NUM_SLOTS - 2) : NUM_SLOTS;
  constexpr int RAW_SLOT0 = REG_ACC ? 0 : CHUNK_TILES;               // first raw slot
  constexpr uint32_t IDESC = KIND == Kind::NVFP4 ? make_idesc_nvfp4(BN) : make_idesc(T::d_fmt, T::ab_fmt, BN);   // FP8_UE8M0: per K atom
  constexpr uint32_t DRAIN_ARRIVALS = 4 * drain_wgs_of<KIND, BN, REG_ACC>();   // one arrival per drain warp
  // two MMA-issuing threads (see the issuer role); the block-scaled kinds need a second set of scale-factor columns in
  // TMEM for the second issuer, which 128-column tiles have room for (3 x 128 accumulator columns + 2 x 64)
  constexpr bool DUAL_ISSUE = !T::block_scaled || BN == 128;
  static_assert(!(T::block_scaled && DUAL_ISSUE) || NUM_SLOTS * BN + 2 * SF_TMEM_COLS <= TMEM_COLS, "no room for the second issuer's scale factors");
  using AR = ARing<SA, DUAL_ISSUE>;
  constexpr uint32_t B_EMPTY_ARRIVALS = (DUAL_ISSUE && !REG_ACC) ? 2 : 1;      // issuers that release a weight stage
  static_assert(!(DUAL_ISSUE && REG_ACC) || KA == 1, "with register accumulators a weight stage serves exactly one step");
  static_assert(!(DUAL_ISSUE && REG_ACC) || (SB % 2 == 0 && RAW_SLOTS % 2 == 0), "alternating issuers must always meet the same stages and slots");
  constexpr uint32_t SF_COL0 = NUM_SLOTS * BN;   // first TMEM column of the scale-factor area
  constexpr int SPILL_DELAY = SB > 2 ? SB - 2 : 1;

  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* smem_a = smem + L::a_off;
  uint8_t* smem_b = smem + L::b_off;
  uint8_t* smem_sfa = smem + L::sfa_off;
  uint8_t* smem_sfb = smem + L::sfb2_off;
  const uint8_t* sfa_blocked = reinterpret_cast<const uint8_t*>(p.sfa);
  const uint8_t* sfb_blocked = reinterpret_cast<const uint8_t*>(p.sfb);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::bar_off);
  uint64_t* a_full = bars;
  uint64_t* a_empty = a_full + SA;
  uint64_t* b_full = a_empty + SA;
  uint64_t* b_empty = b_full + SB;
  uint64_t* tm_full = b_empty + SB;    // [16] hardware-accumulated: per accumulator slot; sw_scale: [0..1] = raw slots
  uint64_t* tm_empty = tm_full + 16;   // [16]
  uint64_t* done_bar = tm_empty + 16;  // [2] an MMA thread drains its own pipeline through its one on abort
  float* sfb_smem = reinterpret_cast<float*>(smem + L::sfb_off);
  uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(smem + L::misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::misc_off + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < SA; ++i) { mbar_init(&a_full[i], 1); mbar_init(&a_empty[i], 1); }
    for (int i = 0; i < SB; ++i) { mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], B_EMPTY_ARRIVALS); }
    for (int i = 0; i < 16; ++i) { mbar_init(&tm_full[i], 1); mbar_init(&tm_empty[i], DRAIN_ARRIVALS); }
    mbar_init(done_bar, 1);
    mbar_init(done_bar + 1, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_s);
  }
  const WorkList work = build_work_list<L::seg_cap, L::item_cap>(p, reinterpret_cast<int*>(smem + L::work_off), reinterpret_cast<int*>(smem + L::seg_first_off),
                                                                reinterpret_cast<int4*>(smem + L::items_off), blockIdx.x, gridDim.x);
  if (warp == 2) {
    tmem_alloc(tmem_base_smem, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_smem;
  const WaitCtx wc{p.status, abort_flag, p.timeout_ns};
  const int kb_count = p.kb_count;                       // 128-byte K atoms
  const int ks_count = (kb_count + KA - 1) / KA;         // B stages along K
  // Tile ownership may alternate between chunks only while the two issuers cannot drift a whole chunk apart: both release
  // every weight stage, so they stay within SB stages of each other, and a chunk must be at least that long. (An issuer that
  // met an accumulator slot's barrier only every other chunk could otherwise be two phases away from it.)
  const bool flip_ok = ks_count >= SB;

  if (warp < 4) {
  if (warp == 0) {
    // ===================================================================== B producer (+ scratch spill)
    if (lane == 0) {
      uint32_t jt = 0;  // stage uses so far
      bool ok = true;
      ItemCursor cursor(work.segs);
      const uint64_t pol_stream = l2_policy_evict_first();
      for (int wi = 0; ok; ++wi) {
        Item it;
        if (!get_item(p, work, wi, cursor, it)) break;
        if (it.rows <= 0) continue;
        const int mtiles = (it.rows + BM - 1) / BM;
        const int chunks = (mtiles + CHUNK_TILES - 1) / CHUNK_TILES;
        const bool spill = p.use_scratch && chunks > 1;
        const int b_row = (it.expert - p.expert_lo) * p.n + it.nt * BN;
        const int s_row = static_cast<int>(blockIdx.x) * BN;
        if (spill) {
          // Loads of the previous item may still be reading this CTA's scratch rows: let them land first.
          const uint32_t first = jt > SB ? jt - SB : 0;
          for (uint32_t q = first; q < jt && ok; ++q) ok = wait_bar(&b_full[q % SB], (q / SB) & 1, wc, ST_TIMEOUT_B_FULL);
        }
        const uint32_t jt_item = jt;
        // Copy stage `q` (K stage index `ks_i` of this item) from shared memory to this CTA's scratch rows.
        auto spill_stage = [&](uint32_t q, int ks_i) -> bool {
          if (!wait_bar(&b_full[q % SB], (q / SB) & 1, wc, ST_TIMEOUT_B_FULL)) return false;
#pragma unroll
          for (int bx = 0; bx < KA; ++bx)
            tma_store_2d(&tmap_s, smem_b + (q % SB) * L::b_stage + bx * L::b_box, (ks_i * KA + bx) * ATOM_BYTES, s_row);
          bulk_commit_group();
          return true;
        };
        for (int chunk = 0; chunk < chunks && ok; ++chunk) {
          const bool from_scratch = spill && chunk > 0;
          if (spill && chunk == 1) bulk_wait_group0();  // the scratch copy is complete and visible
          int next_store = 0;
          for (int ks = 0; ks < ks_count && ok; ++ks, ++jt) {
            const uint32_t s = jt % SB;
            ok = wait_bar(&b_empty[s], ((jt / SB) & 1) ^ 1, wc, ST_TIMEOUT_B_EMPTY);
            if (!ok) break;
            if (spill && chunk == 0) bulk_wait_group_read0();  // earlier spill stores have finished reading their stages
            mbar_arrive_expect_tx(&b_full[s], L::b_stage + L::sfb_stage);
            if constexpr (T::block_scaled) {
              // scales of this stage: KA x 2 KB, contiguous in the blocked layout (the K direction is padded)
              const long long tile128 = static_cast<long long>(it.expert) * p.sfb_rows + ((it.nt * BN) >> 7);
              const long long blk = KIND == Kind::NVFP4 ? static_cast<long long>(ks) * KA * 4 : (static_cast<long long>(ks) * KA) >> 2;
              bulk_load_1d(smem_sfb + s * L::sfb_stage, sfb_blocked + (tile128 * p.sf_k + blk) * SF_BLOCK_BYTES, L::sfb_stage, &b_full[s]);
            }
#pragma unroll
            for (int bx = 0; bx < KA; ++bx) {
              // boxes past the end of K lie wholly outside the tensor and arrive as zeros
              uint8_t* dst = smem_b + s * L::b_stage + bx * L::b_box;
              const int c0 = (ks * KA + bx) * ATOM_BYTES;
              if (from_scratch) tma_load_2d(dst, &tmap_s, &b_full[s], c0, s_row);
              else if (p.b_streaming) tma_load_2d_hint(dst, &tmap_b, &b_full[s], c0, b_row, pol_stream);
              else tma_load_2d(dst, &tmap_b, &b_full[s], c0, b_row);
            }
            if (spill && chunk == 0) {
              while (next_store + SPILL_DELAY <= ks && ok) {
                ok = spill_stage(jt_item + next_store, next_store);
                ++next_store;
              }
            }
          }
          if (spill && chunk == 0) {
            while (next_store < ks_count && ok) {
              ok = spill_stage(jt_item + next_store, next_store);
              ++next_store;
            }
          }
        }
      }
      bulk_wait_group0();
      if (!ok) {  // aborting: let this thread's own loads land before the CTA goes away
        const uint32_t first = jt > SB ? jt - SB : 0;
        for (uint32_t q = first; q < jt; ++q) wait_bar(&b_full[q % SB], (q / SB) & 1, wc, ST_TIMEOUT_DRAIN, false);
      }
    }
  } else if (warp == 1) {
    // ===================================================================== A producer
    // With two issuers, two lanes: each feeds one issuer's half of the ring (the lanes run as divergent threads of the warp,
    // so the issue cost of one lane's barrier test and TMA instruction overlaps with the other's).
    if (lane < (DUAL_ISSUE ? 2 : 1)) {
      const uint32_t me = lane;
      uint32_t it_a = 0, used = 0, chunk_no = 0;   // steps so far: all, and those of this lane's issuer; chunks so far
      bool ok = true;
      ItemCursor cursor(work.segs);
      for (int wi = 0; ok; ++wi) {
        Item it;
        if (!get_item(p, work, wi, cursor, it)) break;
        if (it.rows <= 0) continue;
        const int mtiles = (it.rows + BM - 1) / BM;
        for (int m0 = 0; m0 < mtiles && ok; m0 += CHUNK_TILES, ++chunk_no) {
          const int mc = min(CHUNK_TILES, mtiles - m0);
          const uint32_t flip = flip_ok ? (chunk_no & 1u) : 0u;
          for (int kb = 0; kb < kb_count && ok; ++kb) {
            for (int mt = 0; mt < mc; ++mt, ++it_a) {
              const uint32_t user = DUAL_ISSUE ? ((T::sw_scale ? it_a : static_cast<uint32_t>(mt) + flip) & 1u) : 0u;   // as in the issuer role
              if (user != me) continue;
              const uint32_t s = AR::stage(user, used);
              ok = wait_bar(&a_empty[s], AR::phase(used) ^ 1, wc, ST_TIMEOUT_A_EMPTY);
              if (!ok) break;
              mbar_arrive_expect_tx(&a_full[s], L::a_stage + L::sfa_stage);
              const int a_row = it.row0 + (m0 + mt) * BM;
              if constexpr (T::block_scaled) {
                const long long blk = KIND == Kind::NVFP4 ? static_cast<long long>(kb) * 4 : static_cast<long long>(kb >> 2);
                bulk_load_1d(smem_sfa + s * L::sfa_stage, sfa_blocked + (static_cast<long long>(a_row >> 7) * p.sf_k + blk) * SF_BLOCK_BYTES,
                             L::sfa_stage, &a_full[s]);
              }
              tma_load_2d(smem_a + s * L::a_stage, &tmap_a, &a_full[s], kb * ATOM_BYTES, a_row);
              ++used;
            }
          }
        }
      }
      if (!ok) {
        for (uint32_t q = used > AR::PER ? used - AR::PER : 0; q < used; ++q)
          wait_bar(&a_full[AR::stage(me, q)], AR::phase(q), wc, ST_TIMEOUT_DRAIN, false);
      }
    }
  } else if (warp == 2 || (DUAL_ISSUE && warp == 3)) {
    // ===================================================================== MMA issuer(s)
    // One thread issues what the tensor core does, and every instruction of it (barrier test, MMA, commit, the loop's own
    // arithmetic) costs that thread tens of cycles: a single issuer spends about 950 cycles on a step of four MMAs that
    // the tensor core finishes in 512. So two threads (warps 2 and 3) share the steps: with accumulators in TMEM each row
    // tile belongs to one issuer (the order of the additions into a tile is that thread's program order); with software
    // scaling the steps alternate, each into its own raw slot. Both walk the same sequence and keep the same counters.
    // The block-scaled kinds stay with one issuer: their scale copies into TMEM are ordered with the MMAs by issue order.
    if (lane == 0) {
      const uint32_t issuer = warp - 2;
      uint32_t it_a = 0, own = 0, jt = 0, rt = 0, slot_phase = 0, chunk_no = 0;   // own: steps this issuer has taken
      bool ok = true;
      ItemCursor cursor(work.segs);
      // the operand descriptors are the descriptor of stage 0 plus an offset in its address field
      const uint64_t a_desc0 = make_kmajor_sw128_desc(smem_u32(smem_a));
      const uint64_t b_desc0 = make_kmajor_sw128_desc(smem_u32(smem_b));
      // the barriers of this issuer's NEXT step are tested (non-blocking) before the MMAs of this step are issued, which hides
      // their round trip ("the barrier of the coming step was already complete")
      bool a_seen = false, b_seen = false, r_seen = false;
      const uint32_t sf_base = SF_COL0 + (T::block_scaled && DUAL_ISSUE ? issuer * SF_TMEM_COLS : 0u);   // this issuer's scale columns
      for (int wi = 0; ok; ++wi) {
        Item it;
        if (!get_item(p, work, wi, cursor, it)) break;
        if (it.rows <= 0) continue;
        const int mtiles = (it.rows + BM - 1) / BM;
        for (int m0 = 0; m0 < mtiles && ok; m0 += CHUNK_TILES, ++chunk_no) {
          const int mc = min(CHUNK_TILES, mtiles - m0);
          // With accumulators in TMEM a row tile belongs to one issuer for the whole chunk; which one alternates from chunk to
          // chunk, because tile 0 exists in every chunk and tile 1 only in full ones (fixed ownership left one issuer with
          // up to two thirds of the steps).
          const uint32_t flip = flip_ok ? (chunk_no & 1u) : 0u;
          for (int kb = 0; kb < kb_count && ok; ++kb) {
            const uint32_t sb = jt % SB;
            const int bx = kb % KA;
            // Register accumulators: one step per K atom and stage, so a weight stage has one user and the other issuer
            // leaves it alone. Otherwise both issuers wait for every stage and both release it (b_empty counts two).
            const bool b_mine = !(DUAL_ISSUE && REG_ACC) || (rt & 1u) == issuer;
            if (bx == 0 && b_mine) {
              if (!b_seen) ok = wait_bar(&b_full[sb], (jt / SB) & 1, wc, ST_TIMEOUT_B_FULL);
              b_seen = false;
            }
            if (!ok) break;
            const bool b_last_use = bx == KA - 1 || kb == kb_count - 1;   // the stage is released after this K atom
            const uint64_t b_desc = b_desc0 + static_cast<uint64_t>((sb * L::b_stage + bx * L::b_box) >> 4);
            for (int mt = 0; mt < mc; ++mt, ++it_a) {
              const bool mine = !DUAL_ISSUE || ((T::sw_scale ? rt : static_cast<uint32_t>(mt) + flip) & 1u) == issuer;
              if (mine) {
                const uint32_t sa = AR::stage(issuer, own);
                if (!a_seen) ok = wait_bar(&a_full[sa], AR::phase(own), wc, ST_TIMEOUT_A_FULL);
                if (!ok) break;
                uint32_t d_col;
                if constexpr (T::sw_scale) {
                  const uint32_t rs = rt % RAW_SLOTS;
                  if (!r_seen) ok = wait_bar(&tm_empty[rs], ((rt / RAW_SLOTS) & 1) ^ 1, wc, ST_TIMEOUT_TM_EMPTY);
                  d_col = (RAW_SLOT0 + rs) * BN;
                } else {
                  if (kb == 0) ok = wait_bar(&tm_empty[mt], ((slot_phase >> mt) & 1) ^ 1, wc, ST_TIMEOUT_TM_EMPTY);
                  d_col = mt * BN;
                }
                if (!ok) break;
                a_seen = mbar_test_wait(&a_full[AR::stage(issuer, own + 1)], AR::phase(own + 1));
                if constexpr (!DUAL_ISSUE) {
                  if (mt == mc - 1 && b_last_use) b_seen = mbar_test_wait(&b_full[(jt + 1) % SB], ((jt + 1) / SB) & 1);
                  if constexpr (T::sw_scale) r_seen = mbar_test_wait(&tm_empty[(rt + 1) % RAW_SLOTS], (((rt + 1) / RAW_SLOTS) & 1) ^ 1);
                }
                tc_fence_after_sync();
                const uint64_t a_desc = a_desc0 + static_cast<uint64_t>((sa * L::a_stage) >> 4);
                uint32_t sfa_col = 0, sfb_col = 0;
                if constexpr (T::block_scaled) {
                  // scale factors: shared memory -> TMEM, in issue order ahead of the MMAs that read them
                  constexpr int BLOCKS = KIND == Kind::NVFP4 ? 4 : 1;   // 512-byte blocks per stage and operand
                  sfa_col = sf_base + (own & 1) * 16;
                  sfb_col = sf_base + 32 + (kb & 1) * 16;
                  const uint32_t sfa_addr = smem_u32(smem_sfa + sa * L::sfa_stage);
#pragma unroll
                  for (int j = 0; j < BLOCKS; ++j) tmem_cp_32x128b_warpx4(tmem_base + sfa_col + 4 * j, make_sf_desc(sfa_addr + j * SF_BLOCK_BYTES));
                  if (mt == (DUAL_ISSUE ? static_cast<int>(issuer ^ flip) : 0)) {   // this issuer's first tile of the K atom
                    const uint32_t sfb_addr = smem_u32(smem_sfb + sb * L::sfb_stage + (KIND == Kind::NVFP4 ? bx * SF_ATOM_BYTES : 0));
#pragma unroll
                    for (int j = 0; j < BLOCKS; ++j) tmem_cp_32x128b_warpx4(tmem_base + sfb_col + 4 * j, make_sf_desc(sfb_addr + j * SF_BLOCK_BYTES));
                  }
                  // a 64-row weight tile uses half of its 128-row scale block: words 0-1 or 2-3 of each lane
                  if constexpr (BN == 64) sfb_col += ((it.nt & 1) ? 2 : 0);
                }
#pragma unroll
                for (int j = 0; j < ATOM_BYTES / MMA_K_BYTES; ++j) {
                  const uint64_t da = a_desc + static_cast<uint64_t>(j * (MMA_K_BYTES >> 4));
                  const uint64_t db = b_desc + static_cast<uint64_t>(j * (MMA_K_BYTES >> 4));
                  const uint32_t acc = T::sw_scale ? (j > 0) : (kb > 0 || j > 0);
                  if constexpr (KIND == Kind::NVFP4) {
                    umma_nvfp4(tmem_base + d_col, da, db, IDESC, tmem_base + sfa_col + 4 * j, tmem_base + sfb_col + 4 * j, acc);
                  } else if constexpr (KIND == Kind::FP8_UE8M0) {
                    // all four MMAs of this K atom use the atom's scale byte: byte (kb % 4) of the scale words
                    umma_mxfp8(tmem_base + d_col, da, db, make_idesc_mxfp8(BN, kb & 3), tmem_base + sfa_col, tmem_base + sfb_col, acc);
                  } else {
                    umma<T::mma>(tmem_base + d_col, da, db, IDESC, acc);
                  }
                }
                umma_commit(&a_empty[sa]);
                ++own;
                if constexpr (T::sw_scale) {
                  umma_commit(&tm_full[rt % RAW_SLOTS]);
                } else {
                  if (kb == kb_count - 1) umma_commit(&tm_full[mt]);
                }
              }
              if constexpr (T::sw_scale) ++rt;
            }
            if (ok && b_last_use) {
              if (b_mine) umma_commit(&b_empty[sb]);
              ++jt;
            }
          }
          if constexpr (!T::sw_scale) slot_phase ^= (1u << mc) - 1u;
        }
      }
      if (!ok) {  // aborting: wait until the tensor pipe has retired what this thread issued
        umma_commit(done_bar + issuer);
        wait_bar(done_bar + issuer, 0, wc, ST_TIMEOUT_DRAIN, false);
      }
    }
  }
  } else {
    // ===================================================================== TMEM drain (epilogue)
    const int q = warp & 3;                       // TMEM lane quarter this warp may access
    const int row_in_tile = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    uint32_t rt = 0, slot_phase = 0;
    bool ok = true;
    ItemCursor cursor(work.segs);
    for (int wi = 0; ok; ++wi) {
      Item it;
      if (!get_item(p, work, wi, cursor, it)) break;
      if (it.rows <= 0) continue;
      const int mtiles = (it.rows + BM - 1) / BM;
      const int n0 = it.nt * BN;
      const long long row_end = static_cast<long long>(it.row0) + it.rows;
      for (int m0 = 0; m0 < mtiles && ok; m0 += CHUNK_TILES) {
        const int mc = min(CHUNK_TILES, mtiles - m0);
        if constexpr (T::sw_scale && REG_ACC) {
          // one 128-row tile per chunk; its scaled accumulators stay in registers across the whole K loop
          constexpr int COLS = BN / drain_wgs_of<KIND, BN, REG_ACC>();   // columns owned by this drain warpgroup
          const int col_base = ((warp - 4) >> 2) * COLS;
          const long long grow = static_cast<long long>(it.row0) + m0 * BM + row_in_tile;
          const bool valid = grow < row_end;
          float acc[COLS];
#pragma unroll
          for (int j = 0; j < COLS; ++j) acc[j] = 0.f;
          float* sfb_buf = sfb_smem + (warp - 4) * COLS;     // private to this warp
          // scales of a K block are fetched one block ahead, so that their latency never sits in front of the arithmetic
          const float* sfa_row = p.sfa + grow * p.sf_k;
          // FP8 only: the 128x128 weight block of this warpgroup's columns. With the fused activation the columns are
          // interleaved gate / up rows of the weight, which lie in two different blocks (see GemmParams::epilogue).
          const bool fused = KIND == Kind::FP8 && p.epilogue != 0;
          const int blk_g = min(fused ? (n0 + col_base) >> 8 : (n0 + col_base) >> 7, p.sfb_rows - 1);   // columns past n belong to no block
          const int blk_u = fused ? ((p.n >> 1) + ((n0 + col_base) >> 1)) >> 7 : blk_g;
          const float* sfb_blk = p.sfb + (static_cast<long long>(it.expert) * p.sfb_rows + blk_g) * p.sf_k;
          const float* sfb_blk_u = p.sfb + (static_cast<long long>(it.expert) * p.sfb_rows + blk_u) * p.sf_k;
          float sa_next = valid ? __ldg(sfa_row) : 0.f;
          float sb_next = KIND == Kind::FP8 ? __ldg(sfb_blk) : 0.f;
          float sbu_next = KIND == Kind::FP8 ? __ldg(sfb_blk_u) : 0.f;
          // one 32-column piece of the raw product, scaled and added into the accumulators
          auto accumulate = [&](auto& r, auto c0_tag, float sa, float sb_scalar, float sb_up, int kb) {
            constexpr int W = sizeof(r) / sizeof(r[0]);
            constexpr int c0 = decltype(c0_tag)::value;
            if constexpr (KIND == Kind::INT8) {
              if (p.raw_dump != nullptr && valid) {
                int* dst = p.raw_dump + (static_cast<long long>(kb) * p.rows_total + grow) * p.n + n0 + col_base + c0;
#pragma unroll
                for (int j = 0; j < W; ++j)
                  if (n0 + col_base + c0 + j < p.n) dst[j] = static_cast<int>(r[j]);
              }
            }
            float col_scale[KIND == Kind::INT8 ? W : 1];
            if constexpr (KIND == Kind::INT8) {   // this piece's column scales: 16-byte shared-memory reads (the buffer and c0 are aligned)
#pragma unroll
              for (int q4 = 0; q4 < W / 4; ++q4) {
                const float4 v = reinterpret_cast<const float4*>(sfb_buf + c0)[q4];
                col_scale[4 * q4] = v.x;
                col_scale[4 * q4 + 1] = v.y;
                col_scale[4 * q4 + 2] = v.z;
                col_scale[4 * q4 + 3] = v.w;
              }
            }
#pragma unroll
            for (int j = 0; j < W; ++j) {
              float prod, scale;
              if constexpr (KIND == Kind::INT8) {
                prod = static_cast<float>(static_cast<int>(r[j]));
                scale = sa * col_scale[j];
              } else {
                prod = __uint_as_float(r[j]);
                scale = sa * (((c0 + j) & 16) ? sb_up : sb_scalar);   // columns 16..31 of every 32 are up rows when fused
              }
              acc[c0 + j] = fmaf(prod, scale, acc[c0 + j]);
            }
          };
          // INT8: the per-column weight scales of a K block, one per lane and 32 columns, fetched one block ahead like the others
          float sfc_next[COLS / 32];
          auto fetch_column_scales = [&](int kb) {
#pragma unroll
            for (int j = 0; j < COLS / 32; ++j) {
              const int col = n0 + col_base + j * 32 + lane;
              sfc_next[j] = col < p.n ? __ldg(p.sfb + (static_cast<long long>(it.expert) * p.sfb_rows + col) * p.sf_k + kb) : 0.f;
            }
          };
          if constexpr (KIND == Kind::INT8) fetch_column_scales(0);
          for (int kb = 0; kb < kb_count && ok; ++kb, ++rt) {
            const float sa = sa_next, sb_scalar = sb_next, sb_up = sbu_next;
            if constexpr (KIND == Kind::INT8) {
#pragma unroll
              for (int j = 0; j < COLS / 32; ++j) sfb_buf[j * 32 + lane] = sfc_next[j];
              __syncwarp();
            }
            if (kb + 1 < kb_count) {
              sa_next = valid ? __ldg(sfa_row + kb + 1) : 0.f;
              if constexpr (KIND == Kind::FP8) {
                sb_next = __ldg(sfb_blk + kb + 1);
                sbu_next = __ldg(sfb_blk_u + kb + 1);
              }
              if constexpr (KIND == Kind::INT8) fetch_column_scales(kb + 1);
            }
            const uint32_t rs = rt % RAW_SLOTS;
            ok = wait_bar(&tm_full[rs], (rt / RAW_SLOTS) & 1, wc, ST_TIMEOUT_TM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t raw_addr = lane_addr + (RAW_SLOT0 + rs) * BN + col_base;
            auto release_slot = [&]() {   // this warp has read its part of the raw slot: hand it back before the arithmetic
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&tm_empty[rs]);
            };
            {
              // Two staging buffers, so that the load of the next piece is in flight while this one is scaled and added (one buffer
              // left the warp idle for a TMEM round trip per piece). 128 accumulator registers per thread leave room for two
              // buffers of 8 columns, 64 accumulators for two of 16.
              constexpr int LW = COLS >= 128 ? 8 : 16, NP = COLS / LW;
              uint32_t ra[LW], rb[LW];
              tmem_ld_cols(raw_addr, ra);
              auto step = [&](auto cc_tag) {
                constexpr int cc = decltype(cc_tag)::value;
                auto& cur = (cc & 1) ? rb : ra;
                auto& nxt = (cc & 1) ? ra : rb;
                tmem_wait_ld_into(cur);
                if constexpr (cc + 1 < NP) tmem_ld_cols(raw_addr + (cc + 1) * LW, nxt);
                else release_slot();
                accumulate(cur, std::integral_constant<int, cc * LW>{}, sa, sb_scalar, sb_up, kb);
              };
              for_each_index(std::make_integer_sequence<int, NP>{}, step);
            }
            if constexpr (KIND == Kind::INT8) __syncwarp();  // everyone is done with sfb_buf before the next block refills it
          }
          if (ok && valid) {
#pragma unroll
            for (int cc = 0; cc < COLS / 32; ++cc) {
              uint32_t v[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(acc[cc * 32 + j]);
              if (fused) store_silu_mul16(p, grow, n0 + col_base + cc * 32, v);
              else store_row32(p, grow, n0 + col_base + cc * 32, v);
            }
          }
        } else if constexpr (T::sw_scale) {
          constexpr int COLS = BN / drain_wgs_of<KIND, BN, REG_ACC>();   // columns owned by this drain warpgroup
          const int col_base = ((warp - 4) >> 2) * COLS;
          for (int kb = 0; kb < kb_count && ok; ++kb) {
            // column scales of this K block
            float sb_scalar = 0.f, sb_up = 0.f;
            const bool fused = KIND == Kind::FP8 && p.epilogue != 0;
            if constexpr (KIND == Kind::FP8) {
              const int blk_g = min(fused ? (n0 + col_base) >> 8 : (n0 + col_base) >> 7, p.sfb_rows - 1);   // columns past n belong to no block
              const int blk_u = fused ? ((p.n >> 1) + ((n0 + col_base) >> 1)) >> 7 : blk_g;
              sb_scalar = __ldg(p.sfb + (static_cast<long long>(it.expert) * p.sfb_rows + blk_g) * p.sf_k + kb);
              sb_up = fused ? __ldg(p.sfb + (static_cast<long long>(it.expert) * p.sfb_rows + blk_u) * p.sf_k + kb) : sb_scalar;
            }
            for (int mt = 0; mt < mc && ok; ++mt, ++rt) {
              const long long grow = static_cast<long long>(it.row0) + (m0 + mt) * BM + row_in_tile;
              const bool valid = grow < row_end;
              const float sa = valid ? __ldg(p.sfa + grow * p.sf_k + kb) : 0.f;
              float* sfb_buf = sfb_smem + (warp - 4) * COLS;  // private to this warp: no cross-warp barrier on any path
              if constexpr (KIND == Kind::INT8) {
#pragma unroll
                for (int j = 0; j < COLS / 32; ++j) {
                  const int col = n0 + col_base + j * 32 + lane;
                  sfb_buf[j * 32 + lane] =
                      col < p.n ? __ldg(p.sfb + (static_cast<long long>(it.expert) * p.sfb_rows + col) * p.sf_k + kb) : 0.f;
                }
                __syncwarp();
              }
              const uint32_t rs = rt & 1;
              ok = wait_bar(&tm_full[rs], (rt >> 1) & 1, wc, ST_TIMEOUT_TM_FULL);
              ok = __all_sync(0xffffffffu, ok);
              if (!ok) break;
              tc_fence_after_sync();
              const uint32_t raw_addr = lane_addr + (CHUNK_TILES + rs) * BN + col_base;
              const uint32_t acc_addr = lane_addr + mt * BN + col_base;
              const bool last = kb == kb_count - 1;
#pragma unroll 1
              for (int cc = 0; cc < COLS / 32; ++cc) {
                uint32_t r[32], a[32];
                tmem_ld_32x32b_x32(raw_addr + cc * 32, r);
                if (kb > 0) tmem_ld_32x32b_x32(acc_addr + cc * 32, a);
                tmem_wait_ld();
                if constexpr (KIND == Kind::INT8) {
                  if (p.raw_dump != nullptr && valid) {
                    int* dst = p.raw_dump + (static_cast<long long>(kb) * p.rows_total + grow) * p.n + n0 + col_base + cc * 32;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                      if (n0 + col_base + cc * 32 + j < p.n) dst[j] = static_cast<int>(r[j]);
                  }
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  float prod, scale;
                  if constexpr (KIND == Kind::INT8) {
                    prod = static_cast<float>(static_cast<int>(r[j]));
                    scale = sa * sfb_buf[cc * 32 + j];
                  } else {
                    prod = __uint_as_float(r[j]);
                    scale = sa * ((j & 16) ? sb_up : sb_scalar);
                  }
                  const float prev = kb > 0 ? __uint_as_float(a[j]) : 0.f;
                  a[j] = __float_as_uint(fmaf(prod, scale, prev));
                }
                if (last) {
                  if (valid) {
                    if (fused) store_silu_mul16(p, grow, n0 + col_base + cc * 32, a);
                    else store_row32(p, grow, n0 + col_base + cc * 32, a);
                  }
                } else {
                  tmem_st_32x32b_x32(acc_addr + cc * 32, a);
                }
              }
              if (!last) tmem_wait_st();
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&tm_empty[rs]);
            }
          }
        } else {
          constexpr int COLS = BN / drain_wgs_of<KIND, BN, REG_ACC>();   // columns owned by this drain warpgroup
          const int col_base = ((warp - 4) >> 2) * COLS;
          for (int mt = 0; mt < mc && ok; ++mt) {
            ok = wait_bar(&tm_full[mt], (slot_phase >> mt) & 1, wc, ST_TIMEOUT_TM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            const long long grow = static_cast<long long>(it.row0) + (m0 + mt) * BM + row_in_tile;
            const bool valid = grow < row_end;
            // Read this warp's whole share of the accumulator into registers (at most 128 columns), hand the TMEM slot back,
            // and only then convert and store: the MMA warp can start the next tile on this slot while the stores run.
            uint32_t r[COLS / 32][32];
#pragma unroll
            for (int cc = 0; cc < COLS / 32; ++cc) tmem_ld_32x32b_x32(lane_addr + mt * BN + col_base + cc * 32, r[cc]);
#pragma unroll
            for (int cc = 0; cc < COLS / 32; ++cc) tmem_wait_ld_into(r[cc]);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tm_empty[mt]);
#pragma unroll
            for (int cc = 0; cc < COLS / 32; ++cc) {
              if constexpr (T::block_scaled) {
                if (p.alpha != 1.f) {
#pragma unroll
                  for (int j = 0; j < 32; ++j) r[cc][j] = __float_as_uint(__uint_as_float(r[cc][j]) * p.alpha);
                }
              }
              if (valid) store_row32(p, grow, n0 + col_base + cc * 32, r[cc]);
            }
          }
          slot_phase ^= (1u << mc) - 1u;
        }
      }
    }
  }

  // ===================================================================== common exit: free TMEM on every path
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 2) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace agb
