/*
 * asymgemm_b200.h -- C ABI of the B200 (sm_100a) m-grouped asymmetric MoE GEMM.
 *
 * "Asymmetric": the weight tensor B [G, N, K] (K-major) may stay in pinned / registered host memory and
 * is streamed over the host link by TMA inside the kernel, while activations A and outputs D live in
 * device memory. B may also be device-resident; the same entry points serve both.
 *
 * The entry points below are what a binding of the reference operator API (bytedance-iaas/AsymGEMM,
 * csrc/apis/gemm.hpp, registered in csrc/python_api.cpp) would call for this path. Plain pointers and
 * sizes only; no torch types. All launches are asynchronous on `stream`. Functions return 0 on success
 * and a negative ag_status_t otherwise; ag_last_error() returns a thread-local message for the last
 * failure (the reference raises "Assertion error (file:line): cond", csrc/utils/exception.hpp:14-47).
 */
#ifndef ASYMGEMM_B200_H
#define ASYMGEMM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ag_status {
  AG_OK = 0,
  AG_E_INVALID = -1,     /* malformed descriptor (null pointer, bad shape, misaligned pointer) */
  AG_E_UNSUPPORTED = -2, /* combination not implemented on this device */
  AG_E_CUDA = -3,        /* a CUDA runtime / driver call failed */
  AG_E_NOT_MAPPED = -4,  /* B is host memory that the device cannot address (not pinned / registered) */
  AG_E_DEVICE = -5       /* the kernel reported a status word != 0 (see ag_read_status) */
} ag_status_t;

typedef enum ag_layout {
  AG_LAYOUT_CONTIGUOUS = 0, /* A [M, K], D [M, N]; segments given by (offsets, experts) */
  AG_LAYOUT_MASKED = 1      /* A [G, M_max, K], D [G, M_max, N]; valid rows per group in masked_m */
} ag_layout_t;

typedef enum ag_d_dtype { AG_D_BF16 = 0, AG_D_FP32 = 1 } ag_d_dtype_t;

typedef enum ag_epilogue {
  AG_EPILOGUE_NONE = 0,    /* d = a x b^T */
  AG_EPILOGUE_SILU_MUL = 1 /* fp8 gate+up GEMM of an MoE layer: d [rows, n / 2] = bf16(silu(gate) * up), see ag_gemm_desc_t.epilogue */
} ag_epilogue_t;

/* One grouped-GEMM call. Unused fields must be zero / NULL. */
typedef struct ag_gemm_desc {
  int32_t layout;  /* ag_layout_t */
  int32_t d_dtype; /* ag_d_dtype_t */

  const void* a;   /* device. bf16 [rows, K] | fp8 e4m3 [rows, K] | int8 [rows, K] | packed e2m1 [rows, K/2] */
  const void* sfa; /* device. fp8, int8: fp32 [rows, ceil(K/128)]; nvfp4: ue4m3 [rows, K/16]; bf16: NULL */
  const void* b;   /* device, or pinned/registered host. [G, N, K] in A's element type, K-major */
  const void* sfb; /* device or pinned host. fp8: fp32 [G, ceil(N/128), ceil(K/128)];
                      int8: fp32 [G, N, K/128]; nvfp4: ue4m3 [G, N, K/16]; bf16: NULL */
  void* d;         /* device. [rows, N] bf16 or fp32, row-major, written in place */

  /* contiguous layout: segment i covers rows [offsets[2i], offsets[2i+1]) and uses weight experts[i];
     the list ends at the first negative expert id or after max_segments entries. Both arrays must hold max_segments
     (2 * max_segments) readable entries: the kernels copy the whole list into shared memory with all threads at once. */
  const int32_t* offsets; /* device */
  const int32_t* experts; /* device */
  int32_t max_segments;

  /* masked layout: group g uses rows [g*m, g*m + masked_m[g]) and weight g. */
  const int32_t* masked_m; /* device, [num_groups] */

  int64_t m; /* contiguous: total rows of A and D; masked: M_max (rows per group) */
  int64_t n;
  int64_t k;
  int32_t num_groups; /* G */

  /* Optional device scratch for segments longer than one accumulator chunk (see ag_scratch_bytes).
     NULL: such segments re-read their weight column from `b` once per chunk instead. */
  void* scratch;
  uint64_t scratch_bytes;

  int32_t* status;     /* device int32, optional: 0 = ok, else (cta << 8) | code. Never reset by the call. */
  void* stream;        /* cudaStream_t */
  int32_t num_sms;     /* CTAs to launch at most; 0 = every SM (or the value set by ag_set_num_sms) */
  uint32_t timeout_ms; /* bound on every in-kernel wait; 0 = default (4000 ms) */
  int32_t* raw_dump;   /* int8 only, optional: device int32 [ceil(K/128), rows, N], the exact block sums */
  float alpha;         /* nvfp4 only: product of the two tensor-level scales; 0 is read as 1 */
  int32_t tile_config; /* 0 = choose from where b lives; 1.. = force tile configuration (tuning / tests):
                          1 = 128 columns per item (device-resident b), 2 = 32 columns x 512 B of K per stage
                          (host-resident b), 3 = 32 x 1024 B, 4 = 64 x 256 B, 5 = 128 columns with the scaled accumulators in registers
                          (fp8 / int8 with device-resident b), 6 = 256 columns per item (device-resident b; bf16, fp8, int8),
                          7 = 128 columns with a deep activation ring (device-resident b; bf16 and the hardware-scaled kinds),
                          8 = 256 columns per item on pairs of CTAs that share one 256 x 256 tcgen05.mma.cta_group::2 (device-resident b;
                          bf16, fp8, int8; not with no_split; at least two SMs) */
  int32_t no_split;    /* device-resident b only: 1 = keep one item per (segment, n-tile) instead of splitting long segments into
                          accumulator-sized row chunks across CTAs (tests / tuning); ignored for host-resident b */

  /* Optional copy-engine staging of host-resident b (ignored when b is device memory or raw_dump is set). With a
     non-NULL `stage`, the call does not read b from inside the kernel: it copies as many whole experts as fit in
     one slot of the buffer (cudaMemcpyAsync on a stream of the library's own), runs the grouped GEMM over those experts
     from the buffer while the next ones are copied into the next slot, and so on; same results, every expert of b
     crosses the link whether or not it received rows. The reference stages its streamed weights the same way
     (asym_gemm/unified_moe/runtime.py:110-200). The buffer belongs to the library from the first call that names it
     until the last such call has finished on the GPU; such a call cannot be captured into a CUDA graph. */
  void* stage;          /* device, 1024-byte aligned; NULL = the kernel reads b itself (default) */
  uint64_t stage_bytes; /* at least two slots of one expert (N * K bytes) each */
  uint64_t stage_chunk_bytes; /* bytes of one slot = one chunk of whole experts; 0 = stage_bytes / 2 (a double buffer).
                                 With a smaller value the buffer is a ring of up to 8 slots: the copies then run further
                                 ahead of the GEMMs, which matters when a prefetch (below) fills the ring while other
                                 work keeps the link idle. */

  /* ag_epilogue_t, ag_m_grouped_fp8_gemm_nt only. AG_EPILOGUE_SILU_MUL fuses the activation between the two GEMMs of an MoE
     layer into the gate+up GEMM: b must hold the gate and up rows of every expert INTERLEAVED in groups of 16 -- weight row
     32q + i is gate row 16q + i and weight row 32q + 16 + i is up row 16q + i (i < 16), i.e. row r of the interleaved
     tensor is row (r % 32 / 16) * (n / 2) + r / 32 * 16 + r % 16 of the usual [gate; up] tensor -- while sfb keeps the
     block scales of the usual tensor. d is then bf16 [rows, n / 2] and receives bf16(silu(g) * u), g and u being the bf16
     values the unfused call would have written, silu(g) = g / (1 + exp(-g)) in fp32 (the reference's activation,
     csrc/cpu/module.cpp:337-347): the same bits as the unfused GEMM followed by ag_silu_mul_quant_fp8's activation, without
     the [rows, n] intermediate. n % 256 == 0. */
  int32_t epilogue;

  /* Optional scatter of the result rows (contiguous layout; NULL = rows go to d as usual). With both pointers set, row r of
     the product is not written to d[r] but to row (scatter_meta[r] & 0xffffffff) of the buffer whose address is
     scatter_bases[scatter_meta[r] >> 32]; rows whose entry is negative are not written. scatter_meta: device int64 [m];
     scatter_bases: device array of buffer addresses (as int64), each buffer [*, n] (or [*, n / 2] with the fused epilogue)
     of d's dtype, 16-byte aligned -- memory of this GPU or of a peer GPU mapped into this process (cudaIpcOpenMemHandle /
     peer access): the drain then stores every result row straight into its owner's buffer over NVLink, tile by tile while
     the GEMM runs, and the expert-parallel layer needs no separate return pass (the entries are what ag_ep_dispatch wrote
     into `meta`: (source rank << 32) | pair). Plain stores only: nothing here loads from a peer. The reference's layers
     send results back with a collective after the GEMM (asym_gemm/training/ep_vanilla.py:262-282). */
  const int64_t* scatter_meta;
  const int64_t* scatter_bases;
} ag_gemm_desc_t;

/* BF16 x BF16 -> bf16/fp32. Replaces m_grouped_bf16_asym_gemm_nt_contiguous / _masked
 * (csrc/apis/gemm.hpp:370-418, 420-486; kernel asym_gemm/include/asym_gemm/impls/sm100_bf16_asym_gemm.cuh:98-115). */
int ag_m_grouped_bf16_gemm_nt(const ag_gemm_desc_t* desc);

/* FP8 E4M3 with fp32 scales: A 1x128 per row, B 128x128 per block. Replaces
 * m_grouped_fp8_asym_gemm_nt_contiguous / _masked (csrc/apis/gemm.hpp:81-157, 159-235; kernel
 * asym_gemm/include/asym_gemm/impls/sm100_fp8_asym_gemm_1d1d.cuh:33-40). Scales are applied in fp32 exactly;
 * the reference truncates them to powers of two first (impls/smxx_layout.cuh:96-100), which gives the same
 * result whenever the quantiser produced power-of-two scales. */
int ag_m_grouped_fp8_gemm_nt(const ag_gemm_desc_t* desc);

/* FP8 E4M3 with the block scales applied by the tensor core as UE8M0 (power-of-two) factors: the numerics of the
 * reference's SM100 FP8 kernel (asym_gemm/include/asym_gemm/impls/sm100_fp8_asym_gemm_1d1d.cuh:433-462), which drops the
 * mantissa of every fp32 scale (impls/smxx_layout.cuh:96-100). Exact when the quantiser produced power-of-two scales
 * (use_ue8m0=True); no per-block arithmetic in the drain, so it is the faster path when rows per expert are many.
 * `sfa` and `sfb` are DEVICE buffers in the blocked layout written by ag_fp8_sf_to_blocked_ue8m0 (sfa: groups = 1, rows =
 * all rows of A, rows_per_scale = 1; sfb: groups = G, rows = N, rows_per_scale = 128). Segments must start on multiples
 * of 128 rows; masked M_max % 128 == 0; tile_config 0, 1, 4 or 7. */
int ag_m_grouped_fp8_ue8m0_gemm_nt(const ag_gemm_desc_t* desc);
uint64_t ag_fp8_sf_blocked_bytes(int64_t groups, int64_t rows, int64_t kb);
int ag_fp8_sf_to_blocked_ue8m0(const float* src, void* dst, int64_t groups, int64_t rows, int64_t kb, int32_t rows_per_scale, void* stream);

/* INT8 x INT8 -> exact int32 per 128-wide K block, then fp32 sfa[row,kb] * sfb[col,kb] * sum, summed over
 * K blocks in ascending order. Replaces m_grouped_int8_asym_gemm_nt_contiguous / _masked
 * (csrc/apis/gemm.hpp:569-630; kernel asym_gemm/include/asym_gemm/impls/sm90_int8_asym_gemm_1d1d.cuh:34-41). */
int ag_m_grouped_int8_gemm_nt(const ag_gemm_desc_t* desc);

/* NVFP4: packed E2M1 values, one UE4M3 scale per 16 elements of K. For this entry point `sfa` and `sfb` are DEVICE
 * buffers in the blocked layout produced by ag_fp4_sf_to_blocked (sfa: groups = 1, rows = all rows of A;
 * sfb: groups = G, rows = N); k must be a multiple of 32, every segment must start on a multiple of 128 rows and,
 * in the masked layout, M_max must be a multiple of 128. Replaces
 * m_grouped_fp4_asym_gemm_nt_contiguous / _masked (csrc/apis/gemm.hpp:237-300, 302-365; kernel
 * asym_gemm/include/asym_gemm/impls/sm100_fp4_asym_gemm_1d1d.cuh:44-51). */
int ag_m_grouped_fp4_gemm_nt(const ag_gemm_desc_t* desc);

/* FP8 grouped GEMM (same arguments and results as ag_m_grouped_fp8_gemm_nt) for callers that cannot allocate device
 * memory: processes whose HBM is handed out once at start-up, plugins loaded through FFI with no CUDA allocator of
 * their own, loops that cannot afford a cudaMalloc (it synchronises the device and can fail when memory is nearly
 * full). The scratch that long segments use comes from a fixed 80 MiB array inside the library's device image
 * (ag_static_scratch_bytes); desc->scratch / scratch_bytes are ignored and desc->status MUST be given.
 * Limits: returns AG_E_INVALID with a message when the scratch the launch would use (ag_scratch_bytes_for: CTAs x tile
 * rows x padded K bytes) exceeds the array. With weights on the host, tile_config 0 and all 148 SMs that is K <= 8704
 * (tile_config 2 doubles it, a lower num_sms raises it). With weights in device memory the default launch cuts long
 * segments into one-chunk items that never replay, needs no scratch and has no K limit; only no_split = 1 brings the
 * limit back (K <= 4352 with 128-column items on 148 SMs).
 * every GPU that loads the library holds the array until the process exits; all calls share it, so calls that can
 * overlap on the GPU (other streams or threads) race -- serialise them. The array keeps the last call's contents and
 * needs no clearing. The first call on each device looks up the array's address (cudaGetSymbolAddress): make that
 * call with the device current and outside any stream capture. No cudaMalloc/cudaFree is called on any path.
 * This entry point has no counterpart in the reference. */
int ag_m_grouped_fp8_gemm_nt_static_scratch(const ag_gemm_desc_t* desc);
uint64_t ag_static_scratch_bytes(void);

/* Bytes of scratch that let every long segment replay its weight column from device memory
 * (kind: 0 bf16, 1 fp8, 2 int8, 3 nvfp4). Reference counterpart: none (the reference accumulates bf16
 * partial sums in D instead, impls/sm100_fp8_asym_gemm_1d1d.cuh:648-659). */
uint64_t ag_scratch_bytes(int32_t kind, int64_t n, int64_t k, int32_t num_sms);

/* Exact scratch (bytes) the launch described by `desc` replays long segments from, by the arithmetic of the launch itself
 * (tile configuration from where desc->b lives, grid size, K padded to whole weight stages); 0 when the launch has no use for
 * scratch (device-resident b without no_split). A call whose scratch_bytes is smaller than this runs without replay: long
 * segments then re-read their weight column from b once per accumulator chunk (same results; for host-resident b more
 * trips over the link). kind as above, 4 = fp8 with UE8M0 scales. Only layout, m, n, k, num_groups, max_segments, b,
 * num_sms, tile_config and no_split are read. Reference counterpart: none. */
int ag_scratch_bytes_for(int32_t kind, const ag_gemm_desc_t* desc, uint64_t* bytes_out);

/* Synchronises `stream`, copies the status word to *out and returns AG_OK or AG_E_DEVICE (with a decoded
 * message in ag_last_error). Replaces the reference's device-side trap (asym_gemm/include/asym_gemm/common/utils.cuh:24-40). */
int ag_read_status(const int32_t* status_dev, void* stream, int32_t* out);

/* Process-wide cap on CTAs per launch; 0 restores "all SMs". Replaces set_num_sms / get_num_sms
 * (csrc/apis/runtime.hpp:15-33). */
void ag_set_num_sms(int32_t num_sms);
int32_t ag_get_num_sms(void);

/* Row alignment callers must give every contiguous-layout segment (128). Replaces
 * get_mk_alignment_for_contiguous_layout (csrc/utils/layout.hpp:108-110). */
int32_t ag_get_mk_alignment_for_contiguous_layout(void);

/* Re-lays NVFP4 UE4M3 scales [groups, rows, k16] (row-major bytes; device or pinned host) into the blocked
 * form the kernel copies into TMEM: per group, per 128-row tile, per 4 scale columns one 512-byte block
 * with byte (r % 32) * 16 + (r / 32) * 4 + c. dst is device memory of ag_fp4_sf_blocked_bytes() bytes.
 * Replaces get_mn_major_tma_aligned_packed_byte_sf_tensor (csrc/apis/layout.hpp:14-35). */
uint64_t ag_fp4_sf_blocked_bytes(int64_t groups, int64_t rows, int64_t k16);
int ag_fp4_sf_to_blocked(const void* src, void* dst, int64_t groups, int64_t rows, int64_t k16, void* stream);

/* Starts the copy-engine transfer of the first chunks (as many as the ring has slots) of host-resident weights `b` ([num_groups] experts of
 * `expert_bytes` each) into `stage` ahead of the staged call that will use them -- typically the next layer's weights
 * while this layer's results are still being combined, so that the link does not idle between GEMMs. The next call
 * whose descriptor names the same `b`, `stage`, `stage_bytes` and `stage_chunk_bytes` skips those copies; any other staged call simply
 * overwrites them. The caller must not change the weights between the prefetch and that call. With
 * `wait_for_stream` != 0 the copies start only after the work already queued on `after_stream` (a cudaStream_t) -- for
 * instance a grouped GEMM that is still reading its own weights over the link -- so that they use idle link time instead
 * of competing for it. Returns at once (the copies run on the library's copy stream); a no-op for device-resident `b`. Reference counterpart: the unified runtime
 * issues its staging copies "now", on a side stream, before the work that hides them
 * (asym_gemm/unified_moe/runtime.py:1844-1848). */
int ag_prefetch_staged_weights(const void* b, uint64_t expert_bytes, int32_t num_groups, void* stage, uint64_t stage_bytes,
                               uint64_t stage_chunk_bytes, void* after_stream, int32_t wait_for_stream);

/* Makes an ordinary host allocation (malloc, mmap, a framework's pageable tensor) usable as `b`: page-locks and maps
 * [ptr, ptr + bytes) for the current device's context with cudaHostRegister (portable, mapped; read_only != 0 adds the
 * read-only flag, which file-backed or write-protected mappings need). Memory that is already pinned, registered or
 * device memory is left alone and counts as success. ag_release_weights undoes a registration made here; it refuses a
 * pointer this library did not register. Neither call touches the contents. Reference counterpart: `_pin_on_node`
 * (asym_gemm/unified_moe/runtime.py:236-279), which registers NUMA-placed slabs through libcudart the same way. */
int ag_prepare_weights(void* ptr, uint64_t bytes, int32_t read_only);
int ag_release_weights(void* ptr);

/* Measures pinned-host -> device copy-engine bandwidth (GB/s) with cudaMemcpyAsync over `bytes`, best of
 * `reps`: the denominator for "fraction of host link". Reference counterpart: none (its authors quote
 * ~50 GB/s for the same copy, asym_gemm/unified_moe/runtime.py:115-116). */
int ag_measure_host_link(uint64_t bytes, int32_t reps, double* gbps_out);

/* ---- helper kernels around the two GEMMs of an FP8 MoE layer (all device pointers, asynchronous on `stream`) ----
 * The reference's callers do these steps with separate torch / Triton kernels
 * (asym_gemm/unified_moe/runtime.py:1422-1476,1570,1620-1627; asym_gemm/unified_moe/_triton.py). */

/* x bf16 [rows, cols] -> q e4m3 [rows, cols], sf fp32 [rows, ceil(cols/128)]; sf = max(amax, 1e-4) / 448 per 1x128 block,
 * q = e4m3(x * (1 / sf)): the arithmetic of per_token_cast_to_fp8 (asym_gemm/utils/math.py:24-34). cols % 4 == 0.
 * pow2_scales != 0 rounds every sf up to a power of two first (use_ue8m0=True), for ag_m_grouped_fp8_ue8m0_gemm_nt. */
int ag_quant_rows_fp8(const void* x_bf16, void* q, float* sf, int64_t rows, int64_t cols, int32_t pow2_scales, void* stream);

/* gate_up bf16 [rows, 2*inter] (gate columns first) -> bf16(silu(gate) * up) quantised as above into q [rows, inter],
 * sf [rows, ceil(inter/128)] (activation of csrc/cpu/module.cpp:337-347 followed by the 1x128 quantiser). */
int ag_silu_mul_quant_fp8(const void* gate_up_bf16, void* q, float* sf, int64_t rows, int64_t inter, int32_t pow2_scales, void* stream);

/* dst[dst_rows ? dst_rows[i] : i] = src[src_rows ? src_rows[i] : i], i < rows; rows of row_bytes (multiple of 16) bytes. */
int ag_move_rows(const void* src, void* dst, const int64_t* src_rows, const int64_t* dst_rows, int64_t rows, int64_t row_bytes,
                 void* stream);

/* As ag_quant_rows_fp8 over a buffer of which only the first *rows_used rows hold data (see ag_silu_mul_quant_fp8_upto). */
int ag_quant_rows_fp8_upto(const void* x_bf16, void* q, float* sf, int64_t rows, int64_t cols, int32_t pow2_scales, const int32_t* rows_used,
                           void* stream);

/* As ag_silu_mul_quant_fp8 over a buffer of `rows` rows of which only the first *rows_used (a device int32, read by the
 * kernel) hold data: rows past that count are neither read nor written. For layouts whose size only the device knows
 * (the peer-memory exchange below). rows_used == NULL: all rows. */
int ag_silu_mul_quant_fp8_upto(const void* gate_up_bf16, void* q, float* sf, int64_t rows, int64_t inter, int32_t pow2_scales,
                               const int32_t* rows_used, void* stream);

/* y[t] = sum_j weights[t, j] * rows[pos[t * top_k + j]] accumulated in fp32, rounded once to bf16. cols % 8 == 0.
 * pos == NULL reads rows[t * top_k + j]. */
int ag_combine_topk(const void* rows_bf16, const int64_t* pos, const float* weights, void* y_bf16, int64_t tokens, int32_t top_k,
                    int64_t cols, void* stream);

/* INT8 counterparts for the reference's INT8 MoE layer (asym_gemm/unified_moe/runtime.py:573-583,1558-1627): one scale per
 * row = max(amax * (1/127), 1e-12), written to each of the row's ceil(cols/128) K-block slots so that the tensors can be
 * passed to ag_m_grouped_int8_gemm_nt as they are; q = clamp(rint(x / scale), -127, 127).
 * ag_silu_mul_quant_int8 takes the fp32 gate | up output [rows, 2*inter] and quantises bf16(silu(gate) * up). */
int ag_quant_rows_int8(const void* x_bf16, void* q, float* sf, int64_t rows, int64_t cols, void* stream);
int ag_silu_mul_quant_int8(const void* gate_up_f32, void* q, float* sf, int64_t rows, int64_t inter, void* stream);
/* ag_combine_topk for fp32 rows (cols % 4 == 0); the result is rounded once to bf16. */
int ag_combine_topk_f32(const void* rows_f32, const int64_t* pos, const float* weights, void* y_bf16, int64_t tokens, int32_t top_k,
                        int64_t cols, void* stream);

/* ---- expert-parallel token exchange over peer memory (NVLink / NVSwitch), for the ranks of one node ----
 * The routing, the layout and both exchanges of an MoE layer as kernels that write rows straight into the owner rank's
 * buffers with ordinary stores through peer-mapped pointers; no kernel loads from a peer, none waits for another GPU, and
 * no split size ever reaches the host. The caller issues a small collective on the same stream between the steps
 * (all-gather of the histograms; one after dispatch and one after return, so that every rank's stores have landed before
 * they are read). Every rank allocates the same four buffers with ag_peer_alloc, exchanges the 64-byte handles, and opens
 * the others' with ag_peer_open. The reference's callers do these steps with torch sort / bincount / index kernels and NCCL
 * all_gather + reduce_scatter (asym_gemm/unified_moe/runtime.py:1422-1476, asym_gemm/training/ep_vanilla.py:173-282). */
#define AG_EP_MAX_RANKS 16
#define AG_EP_BAD_EXPERT 64 /* status word: an expert id outside [0, num_experts) in the routing */
#define AG_EP_OVERFLOW 65   /* status word: a rank's experts received more rows than its buffers hold */
typedef struct ag_ep_peers {
  void* a[AG_EP_MAX_RANKS];    /* per rank: [cap_rows, row_bytes] rows in that rank's padded contiguous layout */
  void* sfa[AG_EP_MAX_RANKS];  /* per rank: [cap_rows, sf_per_row] fp32 scales of those rows */
  void* meta[AG_EP_MAX_RANKS]; /* per rank: [cap_rows] int64 return address of each row: (source rank << 32) | pair, -1 = none */
  void* ret[AG_EP_MAX_RANKS];  /* per rank: [tokens * top_k, ret_row_bytes] results by (token, slot) pair of that rank */
} ag_ep_peers_t;

/* Device memory that other processes of the node can map: cudaMalloc + an IPC handle (64 bytes) to send to them;
 * ag_peer_open maps a handle received from another rank (enabling peer access on first use), ag_peer_close unmaps it,
 * ag_peer_free releases one's own. Called once when a layer is built, never per step. */
int ag_peer_alloc(uint64_t bytes, void** ptr, unsigned char* handle64);
int ag_peer_open(const unsigned char* handle64, void** ptr);
int ag_peer_close(void* ptr);
int ag_peer_free(void* ptr);

/* counts[e] = (token, slot) pairs of ids [pairs] (int64) routed to expert e; counts is zeroed first. */
int ag_ep_histogram(const int64_t* ids, int64_t pairs, int32_t num_experts, int32_t* counts, int32_t* status, void* stream);

/* From every rank's histogram counts_all [world, num_experts] and the ownership table range_lo [world + 1] (rank r owns
 * experts [range_lo[r], range_lo[r + 1])): where this rank's rows for each expert start on the owner (send_base [E]), zeroed
 * slot counters (cursors [E]), this rank's own segment table for the grouped GEMM (offsets [2 * epr_cap] = (start, start +
 * valid rows) per local expert, each expert's start a multiple of 128; experts [epr_cap + 1] ending in -1), rows_used [2] =
 * {rows of the padded layout in use, valid rows}, and -1 in my_meta for this rank's padding rows. One small block. */
int ag_ep_plan(const int32_t* counts_all, const int32_t* range_lo, int32_t world, int32_t rank, int32_t num_experts, int64_t cap_rows,
               int32_t* send_base, int32_t* cursors, int32_t* offsets, int32_t* experts, int32_t epr_cap, int32_t* rows_used, int64_t* my_meta,
               int32_t* status, void* stream);

/* Every (token, slot) pair of this rank: the token's row x_q [tokens, row_bytes] and scales sfx [tokens, sf_per_row] are
 * stored into the next free row of the pair's expert on the owner rank, with the pair's return address beside it.
 * pair_row (optional, int64 [tokens * top_k]) receives the row each pair went to: with one rank the results can then be
 * combined straight out of the layout (ag_combine_topk with pos = pair_row) and ag_ep_return is not needed. */
int ag_ep_dispatch(const void* x_q, const float* sfx, const int64_t* ids, int64_t tokens, int32_t top_k, int64_t row_bytes, int32_t sf_per_row,
                   const int32_t* range_lo, int32_t world, int32_t rank, const int32_t* send_base, int32_t* cursors, int64_t cap_rows,
                   int64_t* pair_row, const ag_ep_peers_t* peers, void* stream);

/* Every valid row of this rank's result `out` [cap_rows, row_bytes] is stored into its pair's slot of the source rank's `ret`. */
int ag_ep_return(const void* out, const int64_t* my_meta, const int32_t* rows_used, int64_t cap_rows, int64_t row_bytes, int32_t world,
                 const ag_ep_peers_t* peers, void* stream);

/* Failure-detection self test: launches a one-CTA kernel whose only barrier wait can never be satisfied. After
 * `timeout_ms` (1..2000) the wait gives up, the kernel stores (0 << 8) | 9 ("wait-limit self test expired") in *status
 * and returns; the context stays usable. Replaces nothing in the reference, whose device waits are unbounded
 * (csrc/ep_steal/ep_steal_sync.cu:63-64) and whose device asserts trap (asym_gemm/include/asym_gemm/common/utils.cuh:24-40). */
int ag_selftest_wait_limit(uint32_t timeout_ms, int32_t* status, void* stream);

/* Issue-rate probe of the tensor core, on every SM of the current device: `issuers` (1 or 2) threads per CTA each run the
 * inner sequence of the kernels' MMA role -- wait for an operand stage, four tcgen05.mma of M128 x N`n_cols` (128 or 256) x K16
 * in bf16, commit -- for `steps` steps against producers that only arrive on the barriers (no loads; the operands are
 * whatever shared memory holds, the accumulators are discarded). *cycles_per_step = SM cycles per step of four MMAs, worst
 * CTA; the tensor core's own time for a step is 2 * n_cols cycles. Synchronous (allocates two small device buffers, frees
 * them before it returns); every wait inside is bounded. Reference counterpart: none -- this is the measurement behind the
 * two MMA-issuing threads of the kernels. */
int ag_probe_mma_issue(int32_t issuers, int32_t n_cols, int32_t steps, double* cycles_per_step);

/* Operand-feed probe, on every SM of the current device: the kernels' producer / issuer rings for 256-column bf16 items (per
 * 128-byte K atom one 256-row weight stage and two 128-row activation stages, two issuers) with real TMA loads from device
 * memory (load_a / load_b != 0 switch the loads of the two operands on) and nothing else: no drain, no item bookkeeping.
 * Groups of six CTAs share activation rows and every sixth CTA shares weight rows, as CTAs of the grouped GEMM do through
 * L2. *cycles_per_k_atom = SM cycles per K atom (two steps of four MMAs), worst CTA; the tensor core's own time is 1024.
 * Allocates 1 GB of device memory for the operands and frees it before it returns; synchronous; every wait is bounded.
 * Reference counterpart: none. */
int ag_probe_operand_feed(int32_t load_a, int32_t load_b, double* cycles_per_k_atom);

/* Copy-only ceiling for SM-issued reads of pinned memory: streams a `bytes` pinned buffer laid out as rows of `row_bytes`
 * through shared memory with the weight producer's TMA pattern (each CTA owns columns of `box_rows` rows and walks K in
 * 128-byte boxes, `boxes_per_stage` per stage) on `num_ctas` CTAs (0 = all SMs), best of `reps`. Reference counterpart:
 * none (its authors report ~21.5 GB/s for in-kernel TMA reads, asym_gemm/unified_moe/runtime.py:113-116). */
int ag_measure_host_stream(uint64_t bytes, int64_t row_bytes, int32_t box_rows, int32_t boxes_per_stage, int32_t num_ctas,
                           int32_t reps, double* gbps_out);

/* Sustained host-link measurement in three steps, so that several GPUs can be timed while they really stream at the same
 * time. ag_link_probe_create (slow and unevenly long: allocates and touches `bytes` of pinned memory, the device side and
 * one untimed pass) for `device` (-1 = the current one); then a barrier of the caller's between the ranks or threads that
 * measure together; then ag_link_probe_run streams for at least `min_seconds` and reports the MEAN GB/s over the whole
 * run (not the best pass); ag_link_probe_destroy frees everything. mode 0 = copy engine (cudaMemcpyAsync pinned -> device),
 * mode 1 = SM-issued TMA reads with the weight producer's access pattern (rows of `row_bytes`, a multiple of 128).
 * A probe may be run repeatedly. Reference counterpart: none. */
typedef struct ag_link_probe ag_link_probe_t;
int ag_link_probe_create(int32_t device, uint64_t bytes, int32_t mode, int64_t row_bytes, ag_link_probe_t** out);
int ag_link_probe_run(ag_link_probe_t* probe, double min_seconds, double* gbps_mean);
int ag_link_probe_destroy(ag_link_probe_t* probe);

/* sizeof(ag_gemm_desc_t) as this library was compiled: lets a binding written in another language (ctypes, cgo, JNI)
 * check its mirror of the struct before the first call. */
uint64_t ag_gemm_desc_size(void);

const char* ag_last_error(void);
const char* ag_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ASYMGEMM_B200_H */
