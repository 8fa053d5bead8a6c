// The round kernels over F_p^4 (every points x tables x fold combination), in a file of their own
// so that the two extension degrees compile side by side.
#include "round_kernel.cuh"
namespace sc {
cudaError_t launch_round_d4(int shape, int points, int nt, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    return launch_round_d<4>(shape, points, nt, fold, args, grid, smem, stream);
}
}  // namespace sc
