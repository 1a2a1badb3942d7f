// Instantiates the grouped-GEMM kernel for NVFP4 operands (block-scaled tcgen05.mma), 128- and 64-column items.
#include "launch.cuh"

namespace agb {
cudaError_t launch_fp4(AGB_LAUNCH_ARGS) {
  switch (tile) {
    case 0: return launch_one<Kind::NVFP4, 128, 1, 8>(grid, stream, ma, mb, ms, p);
    case 3: return launch_one<Kind::NVFP4, kTileFp4Host.bn, kTileFp4Host.ka, kTileFp4Host.sb>(grid, stream, ma, mb, ms, p);
    case 6: return launch_one<Kind::NVFP4, 128, 1, 4, false, 8>(grid, stream, ma, mb, ms, p);
    default: return cudaErrorInvalidValue;
  }
}
}  // namespace agb
