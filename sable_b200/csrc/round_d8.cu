// The round kernels over F_p^8.
#include "round_kernel.cuh"
namespace sc {
cudaError_t launch_round_d8(int shape, int points, int nt, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    return launch_round_d<8>(shape, points, nt, fold, args, grid, smem, stream);
}
}  // namespace sc
