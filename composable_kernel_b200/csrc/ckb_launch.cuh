// Launch helpers.  launch_epi<MODE, KIND, EPI> is explicitly instantiated in the generated
// ckb_inst_*.cu files (so that they compile in parallel); find_launch() maps runtime ids to them.
#pragma once
#include "ckb_kernel.cuh"

namespace ckb {

// Tile widths the library instantiates and the pipeline depth that fills shared memory.
//   BN 256 -> 4 stages x 48 KiB, BN 128 -> 6 x 32 KiB, BN 64 -> 8 x 24 KiB  (192 KiB of stages)
template <int BN>
struct StagesFor;
template <>
struct StagesFor<256>
{
    static constexpr int value = 4;
};
template <>
struct StagesFor<128>
{
    static constexpr int value = 6;
};
template <>
struct StagesFor<64>
{
    static constexpr int value = 8;
};

template <int MODE, int KIND, int EPI, int BN>
cudaError_t launch_one(const KernelParams& p, int grid, cudaStream_t stream)
{
    constexpr int STAGES = StagesFor<BN>::value;
    constexpr int SMEM   = SmemLayout<BN, STAGES>::DYN_BYTES;
    auto kern            = contraction_kernel<MODE, KIND, EPI, BN, STAGES>;
    static bool attr_done[64] = {};
    int dev                   = 0;
    cudaError_t err           = cudaGetDevice(&dev);
    if(err != cudaSuccess)
        return err;
    if(dev < 0 || dev >= 64 || !attr_done[dev])
    {
        err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if(err != cudaSuccess)
            return err;
        if(dev >= 0 && dev < 64)
            attr_done[dev] = true;
    }
    kern<<<grid, NUM_THREADS, SMEM, stream>>>(p);
    return cudaGetLastError();
}

template <int MODE, int KIND, int EPI>
cudaError_t launch_epi(int bn, const KernelParams& p, int grid, cudaStream_t stream)
{
    switch(bn)
    {
    case 256: return launch_one<MODE, KIND, EPI, 256>(p, grid, stream);
    case 128: return launch_one<MODE, KIND, EPI, 128>(p, grid, stream);
    case 64: return launch_one<MODE, KIND, EPI, 64>(p, grid, stream);
    default: return cudaErrorInvalidValue;
    }
}

typedef cudaError_t (*LaunchFn)(int, const KernelParams&, int, cudaStream_t);

// nullptr when the (mode, kind, epilogue) combination is not instantiated.
LaunchFn find_launch(int mode, int kind, int epi);

} // namespace ckb
