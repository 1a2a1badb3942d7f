// Instantiates the grouped-GEMM kernel for INT8 operands, one kernel per tile configuration.
#include "launch.cuh"

namespace agb {
cudaError_t launch_int8(AGB_LAUNCH_ARGS) { return launch_kind_impl<Kind::INT8>(tile, grid, stream, ma, mb, ms, p); }
}  // namespace agb
