// Instantiates the grouped-GEMM kernel for FP8 operands with UE8M0 block scales applied by the tensor core.
#include "launch.cuh"

namespace agb {
cudaError_t launch_fp8_ue8m0(AGB_LAUNCH_ARGS) {
  switch (tile) {
    case 0: return launch_one<Kind::FP8_UE8M0, 128, 1, 8>(grid, stream, ma, mb, ms, p);
    case 3: return launch_one<Kind::FP8_UE8M0, 64, 2, 8>(grid, stream, ma, mb, ms, p);
    case 6: return launch_one<Kind::FP8_UE8M0, 128, 1, 4, false, 8>(grid, stream, ma, mb, ms, p);
    default: return cudaErrorInvalidValue;
  }
}
}  // namespace agb
