// Host-side launch interface between the C ABI (capi.cu) and the per-dtype kernel instantiations.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include "mgrouped_kernel.cuh"
#include "mgrouped_pair_kernel.cuh"

namespace agb {

// Tile configurations. BN = output columns (= weight rows) per item, KA = 128-byte K atoms per weight stage,
// SB = weight ring depth, SA = activation ring depth (stages of 128 rows x 128 B). The host-streaming configurations keep
// 128 KB of weight reads in flight per CTA; the device-resident ones balance the two rings by what one K step consumes.
constexpr bool kind_is_block_scaled(int kind) { return kind == 3 || kind == 4; }
constexpr bool kind_is_sw_scaled(int kind) { return kind == 1 || kind == 2; }

struct TileConfig {
  int bn, ka, sb, sa;
};
constexpr int kNumTileConfigs = 8;
constexpr TileConfig kTileConfigs[kNumTileConfigs] = {
    {128, 1, 8, 4},  // 0: B resident in device memory, 128-column items
    {32, 4, 8, 4},   // 1: B streamed from host memory, fewest host pages in flight per CTA
    {32, 8, 4, 4},   // 2: as 1 with longer contiguous runs per row
    {64, 2, 8, 4},   // 3: B streamed from host memory (default: 51.0 GB/s of a 55.6 GB/s copy peak on the FP8 7168x4096 case)
    {128, 1, 8, 4},  // 4: FP8 / INT8 with B resident in device memory: scaled accumulators in registers, one tile per item
    {256, 1, 4, 4},  // 5: B resident in device memory, 256-column items: BF16 keeps two 128 x 256 accumulators in TMEM (a weight
                     //    stage serves 256 rows, an activation stage 256 columns: twice the flops per operand byte of 0);
                     //    FP8 / INT8 keep one 128 x 256 tile's scaled accumulators in the registers of two drain warpgroups
    {128, 1, 4, 8},  // 6: B resident in device memory, 128-column items with a deep activation ring: the hardware-scaled kinds
                     //    keep three row tiles per weight stage, so one K step consumes three activation stages
    {256, 1, 6, 6},  // 7: B resident in device memory, 256-column items on PAIRS of CTAs (mgrouped_pair_kernel.cuh): each SM loads
                     //    half of the weight tile and the tensor cores read both halves; BF16, FP8 (fp32 scales) and INT8
};
constexpr int kTileDeviceRegAcc = 4;
constexpr int kTileDeviceWide = 5;
constexpr int kTileDeviceDeepA = 6;
constexpr int kTileDevicePair = 7;
constexpr bool tile_reg_acc(int kind, int tile) { return kind_is_sw_scaled(kind) && (tile == kTileDeviceRegAcc || tile == kTileDeviceWide); }
// rows of one accumulator chunk (what one item covers when long segments are split)
constexpr int chunk_tiles_of(int kind, int tile, int bn) {
  if (tile == kTileDevicePair) return kind_is_sw_scaled(kind) ? 2 : 4;   // 256 rows per pair and accumulator
  return kind_is_block_scaled(kind) ? (512 - 64) / bn : (kind_is_sw_scaled(kind) ? (tile_reg_acc(kind, tile) ? 1 : 512 / bn - 2) : 512 / bn);
}
// NVFP4 also stages 2 KB of scale factors per K atom and operand, so its host-streaming configuration uses
// single-atom stages in a deeper ring to stay inside the 227 KB of shared memory.
constexpr TileConfig kTileFp4Host = {64, 1, 12, 4};
constexpr TileConfig tile_config_of(int kind, int tile) { return (kind == 3 && tile == 3) ? kTileFp4Host : kTileConfigs[tile]; }
constexpr int kTileDevice = 0;
constexpr int kTileHost = 3;
// Which configurations exist for which operand kind (0 bf16, 1 fp8, 2 int8, 3 nvfp4, 4 fp8 with UE8M0 scales).
constexpr bool tile_supported(int kind, int tile) {
  if (tile < 0 || tile >= kNumTileConfigs) return false;
  if (kind_is_block_scaled(kind)) return tile == 0 || tile == 3 || tile == kTileDeviceDeepA;   // 128 or 64 columns per item
  if (kind_is_sw_scaled(kind)) return tile != kTileDeviceDeepA;
  return tile != kTileDeviceRegAcc;   // the pair kernel (8) exists for every kind that is not block-scaled
}
inline const char* tile_support_text(int kind) {
  return kind_is_block_scaled(kind) ? "hardware block-scaled kinds have tile_config 1, 4 and 7"
         : kind_is_sw_scaled(kind) ? "fp8 and int8 have tile_config 1 .. 6 and 8" : "bf16 has tile_config 1 .. 4 and 6 .. 8";
}
// Configuration chosen when the caller does not force one.
// Device-resident weights take 256-column items where the kind has them and N is wide enough to fill one
// (measured on the FP8 7168x4096 and BF16 2048x1536 cases: 1.4x and 1.55x the 128-column items).
constexpr int default_tile(int kind, bool host_b, long long n) {
  if (host_b) return kTileHost;
  if (kind_is_block_scaled(kind)) return kTileDeviceDeepA;   // two issuers, four activation stages each: FP8/UE8M0 1205 against 1140 TFLOP/s
  if (n >= 256 && kind != 2) return kTileDeviceWide;   // INT8 keeps 128-column items: int-to-float conversion and per-column scales on top of the
                                                       // 128 accumulators spill at 256 columns (measured 706 against 344 TFLOP/s)
  return kind_is_sw_scaled(kind) ? kTileDeviceRegAcc : kTileDevice;
}

#define AGB_LAUNCH_ARGS int tile, int grid, cudaStream_t stream, const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &ms, const GemmParams &p
// One instantiation set per dtype lives in its own translation unit (inst_*.cu).
cudaError_t launch_bf16(AGB_LAUNCH_ARGS);
cudaError_t launch_fp8(AGB_LAUNCH_ARGS);
cudaError_t launch_int8(AGB_LAUNCH_ARGS);
cudaError_t launch_fp4(AGB_LAUNCH_ARGS);   // tiles 0, 3 and 6 only
cudaError_t launch_fp8_ue8m0(AGB_LAUNCH_ARGS);   // tiles 0, 3 and 6 only
cudaError_t fp8_sf_to_blocked_ue8m0(const float* src, void* dst, long long groups, long long rows, long long kb, int rows_per_scale,
                                    cudaStream_t stream);
cudaError_t fp4_sf_to_blocked(const void* src, void* dst, long long groups, long long rows, long long k16, cudaStream_t stream);
long long fp4_sf_k4_padded_host(long long k16);
long long fp8_sf_k4_padded_host(long long kb);

template <Kind KIND, int BN, int KA, int SB, bool REG_ACC = false, int SA = 4>
cudaError_t launch_one(int grid, cudaStream_t stream, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& ms,
                       const GemmParams& p) {
  using L = SmemLayout<BN, KA, SA, SB, SfStage<KIND, KA>::a, SfStage<KIND, KA>::b>;
  static_assert(L::dyn_bytes <= 232448, "tile configuration does not fit in shared memory");
  auto kernel = mgrouped_gemm_kernel<KIND, BN, KA, SA, SB, REG_ACC>;
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::dyn_bytes);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  kernel<<<grid, num_threads_of<KIND, BN, REG_ACC>(), L::dyn_bytes, stream>>>(ma, mb, ms, p);
  return cudaGetLastError();
}

// The pair kernel: `grid` counts CTAs and is even; clusters of two are a compile-time attribute of the kernel.
template <Kind KIND>
cudaError_t launch_pair(int grid, cudaStream_t stream, const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p) {
  // BF16: stages of two K atoms (8 MMAs per barrier round trip and commit: the commits that go to both CTAs are what the
  // issuers of a pair spend most on), two per issuer for the activations, two for the weights; FP8 / INT8: single atoms
  constexpr bool sw = KindTraits<KIND>::sw_scale;
  constexpr int SA = sw ? 6 : 4, SB = sw ? 6 : 2, KA = sw ? 1 : 2;
  using L = PairSmem<SA, SB, KA>;
  static_assert(L::dyn_bytes <= 232448, "pair configuration does not fit in shared memory");
  auto kernel = mgrouped_pair_kernel<KIND, SA, SB, KA>;
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::dyn_bytes);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  if (grid < 2 || (grid & 1)) return cudaErrorInvalidValue;
  kernel<<<grid, PAIR_THREADS, L::dyn_bytes, stream>>>(ma, mb, p);
  return cudaGetLastError();
}

template <Kind KIND>
cudaError_t launch_kind_impl(AGB_LAUNCH_ARGS) {
  switch (tile) {
    case 0: return launch_one<KIND, 128, 1, 8>(grid, stream, ma, mb, ms, p);
    case 1: return launch_one<KIND, 32, 4, 8>(grid, stream, ma, mb, ms, p);
    case 2: return launch_one<KIND, 32, 8, 4>(grid, stream, ma, mb, ms, p);
    case 3: return launch_one<KIND, 64, 2, 8>(grid, stream, ma, mb, ms, p);
    case 4:
      if constexpr (KindTraits<KIND>::sw_scale) return launch_one<KIND, 128, 1, 8, true>(grid, stream, ma, mb, ms, p);
      else return cudaErrorInvalidValue;
    case 5: return launch_one<KIND, 256, 1, 4, KindTraits<KIND>::sw_scale, 4>(grid, stream, ma, mb, ms, p);
    case 6:
      if constexpr (!KindTraits<KIND>::sw_scale) return launch_one<KIND, 128, 1, 4, false, 8>(grid, stream, ma, mb, ms, p);
      else return cudaErrorInvalidValue;
    case 7:
      if constexpr (!KindTraits<KIND>::block_scaled) return launch_pair<KIND>(grid, stream, ma, mb, p);
      else return cudaErrorInvalidValue;
    default: return cudaErrorInvalidValue;
  }
}

inline cudaError_t launch_mgrouped(int kind, AGB_LAUNCH_ARGS) {
  switch (kind) {
    case 0: return launch_bf16(tile, grid, stream, ma, mb, ms, p);
    case 1: return launch_fp8(tile, grid, stream, ma, mb, ms, p);
    case 2: return launch_int8(tile, grid, stream, ma, mb, ms, p);
    case 3: return launch_fp4(tile, grid, stream, ma, mb, ms, p);
    case 4: return launch_fp8_ue8m0(tile, grid, stream, ma, mb, ms, p);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace agb
