// The term-table round kernels over F_p^4 for statements of five to eight tables.
#include "round_kernel.cuh"
namespace sc {
cudaError_t launch_round_d4w(int points, int nt, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    return launch_round_wide<4>(points, nt, fold, args, grid, smem, stream);
}
}  // namespace sc
