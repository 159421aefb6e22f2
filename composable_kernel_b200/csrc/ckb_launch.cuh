// Launch helpers.  launch_epi<MODE, KIND, EPI> is explicitly instantiated in the generated
// ckb_inst_*.cu files (so that they compile in parallel); find_launch() maps runtime ids to them.
#pragma once
#include "ckb_kernel.cuh"

namespace ckb {

// Tile widths the library instantiates and the pipeline depth that fills shared memory.
//   one CTA per tile : BN 256 -> 4 stages x 48 KiB, BN 128 -> 6 x 32 KiB, BN 64 -> 8 x 24 KiB
//   CTA pair per tile: BN 256 -> 6 stages x 32 KiB per CTA (256 x 256 tile per pair)
template <int BN, int CG>
struct StagesFor;
template <>
struct StagesFor<256, 1>
{
    static constexpr int value = 4;
};
template <>
struct StagesFor<128, 1>
{
    static constexpr int value = 6;
};
template <>
struct StagesFor<64, 1>
{
    static constexpr int value = 8;
};
template <>
struct StagesFor<256, 2>
{
#ifdef CKB_PAIR_STAGES
    static constexpr int value = CKB_PAIR_STAGES; // build-time override for pipeline-depth experiments (at most 7 fit)
#else
    static constexpr int value = 6;
#endif
};

template <int MODE, int KIND, int EPI, int BN, int CG>
cudaError_t launch_one(const KernelParams& p, int grid, cudaStream_t stream)
{
    constexpr int STAGES = StagesFor<BN, CG>::value;
    constexpr int SMEM   = SmemLayout<BN, STAGES, CG>::DYN_BYTES;
    auto kern            = contraction_kernel<MODE, KIND, EPI, BN, STAGES, CG>;
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
    if constexpr(CG == 1)
    {
        kern<<<grid, NUM_THREADS, SMEM, stream>>>(p);
        return cudaGetLastError();
    }
    else
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim            = dim3(grid, 1, 1); // a multiple of the cluster size
        cfg.blockDim           = dim3(NUM_THREADS, 1, 1);
        cfg.dynamicSmemBytes   = SMEM;
        cfg.stream             = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id               = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = CG;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs                = attr;
        cfg.numAttrs             = 1;
        return cudaLaunchKernelEx(&cfg, kern, p);
    }
}

// cg = CTAs per tile (1 or 2; 2 is instantiated for bn = 256 only).
template <int MODE, int KIND, int EPI>
cudaError_t launch_epi(int bn, int cg, const KernelParams& p, int grid, cudaStream_t stream)
{
    if(cg == 2 && bn == 256)
        return launch_one<MODE, KIND, EPI, 256, 2>(p, grid, stream);
    if(cg != 1)
        return cudaErrorInvalidValue;
    switch(bn)
    {
    case 256: return launch_one<MODE, KIND, EPI, 256, 1>(p, grid, stream);
    case 128: return launch_one<MODE, KIND, EPI, 128, 1>(p, grid, stream);
    case 64: return launch_one<MODE, KIND, EPI, 64, 1>(p, grid, stream);
    default: return cudaErrorInvalidValue;
    }
}

typedef cudaError_t (*LaunchFn)(int, int, const KernelParams&, int, cudaStream_t);

// nullptr when the (mode, kind, epilogue) combination is not instantiated.
LaunchFn find_launch(int mode, int kind, int epi);

} // namespace ckb
