// Instantiates the grouped-GEMM kernel for BF16 operands, one kernel per tile configuration.
#include "launch.cuh"

namespace agb {
cudaError_t launch_bf16(AGB_LAUNCH_ARGS) { return launch_kind_impl<Kind::BF16>(tile, grid, stream, ma, mb, ms, p); }
}  // namespace agb
