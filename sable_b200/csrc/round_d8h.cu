// The term-table round kernels over F_p^8 for statements of degree five to eight.
#include "round_kernel.cuh"
namespace sc {
cudaError_t launch_round_d8h(int points, int nt, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    return launch_round_high<8>(points, nt, fold, args, grid, smem, stream);
}
}  // namespace sc
