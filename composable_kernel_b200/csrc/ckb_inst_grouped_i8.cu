// Instantiates contraction_kernel<MODE_GROUPED, KIND_I8, BN> for BN = 256, 128, 64.
#include "ckb_launch.cuh"

namespace ckb {
cudaError_t launch_grouped_i8(int bn, const KernelParams& p, int grid, cudaStream_t stream)
{
    return launch_bn<MODE_GROUPED, KIND_I8>(bn, p, grid, stream);
}
} // namespace ckb
