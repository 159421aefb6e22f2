// Launch helpers.  launch_epi<MODE, KIND, EPI> is explicitly instantiated in the generated
// ckb_inst_*.cu files (so that they compile in parallel); find_launch() maps runtime ids to them.
#pragma once
#include <cstdlib>

#include "ckb_kernel.cuh"

namespace ckb {

// Tile widths the library instantiates, the k blocks (128 bytes of K each) one pipeline stage holds and the
// pipeline depth that fills shared memory.  Two k blocks per stage halve the per-block work of the single
// threads that issue the copies and the MMAs (barrier wait, commit, bookkeeping), which is what limits the
// main loop once the tiles are large.
//   one CTA per tile : BN 256 -> 4 stages x 1 x 48 KiB, BN 128 -> 3 x 2 x 32 KiB, BN 64 -> 4 x 2 x 24 KiB
//   CTA pair per tile: BN 256 -> 3 stages x 2 x 32 KiB per CTA (256 x 256 tile per pair)
// The cluster K-split instances use the single-CTA shapes; their raw accumulator tile (BN x 512 bytes) reuses the stages.
// The implicit-GEMM convolution keeps one k block per stage: two were slower with a single-thread producer and no
// faster with the warp-wide one, and six shallow stages ride out the longer latency of the im2col copies.
template <int BN, int CG, int MODE>
struct StagesFor
{
    static constexpr bool conv = MODE == MODE_CONV;
    static constexpr int pair_ksub = conv ? 1 : 2, pair_stages = conv ? 6 : 3;
    static constexpr int ksub  = CG == 2 ? pair_ksub : (BN == 256 || conv) ? 1 : 2;
    static constexpr int value = CG == 2 ? pair_stages : BN == 256 ? 4 : BN == 128 ? (conv ? 6 : 3) : (conv ? 8 : 4);
};

// CKB_NO_PDL=1 turns programmatic dependent launch off (plain stream order).
inline bool programmatic_launch_enabled()
{
    static const bool on = [] {
        const char* s = getenv("CKB_NO_PDL");
        return !(s && atoi(s) != 0);
    }();
    return on;
}

// VARIANT_CLUSTER_K: the cluster K-split instance of the tile shape (a cluster of p.plan.ksplit CTAs per tile);
// VARIANT_BALANCED: the instance with the parking and fix-up loops of the balanced K ranges, for kernel families
// whose plain instance does not carry them.
template <int MODE, int KIND, int EPI, int BN, int CG, int VARIANT = VARIANT_PLAIN>
cudaError_t launch_one(const KernelParams& p, int grid, cudaStream_t stream)
{
    constexpr bool CK    = VARIANT == VARIANT_CLUSTER_K;
    constexpr int STAGES = StagesFor<BN, CG, MODE>::value;
    constexpr int KSUB   = StagesFor<BN, CG, MODE>::ksub;
    constexpr int SMEM   = SmemLayout<BN, STAGES, CG, KSUB>::DYN_BYTES;
    static_assert(SMEM <= 227 * 1024, "pipeline does not fit in shared memory");
    auto kern            = contraction_kernel<MODE, KIND, EPI, BN, STAGES, CG, KSUB, VARIANT>;
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
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim            = dim3(grid, 1, 1); // CG = 2: a multiple of the cluster size
    cfg.blockDim           = dim3(threads_for<MODE>(), 1, 1);
    cfg.dynamicSmemBytes   = SMEM;
    cfg.stream             = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if constexpr(CG == 2 || CK)
    {
        attr[n_attr].id               = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = CK ? p.plan.ksplit : CG;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    if(programmatic_launch_enabled())
    {
        // the start-up of this kernel (barrier set-up, tensor-memory allocation) may overlap the tail of the kernel
        // before it in the stream; the kernel waits (griddepcontrol.wait) before it touches global memory
        attr[n_attr].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    cfg.attrs    = attr;
    cfg.numAttrs = n_attr;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

// cg = CTAs per tile (1 or 2; 2 is instantiated for bn = 256 only).
template <int MODE, int KIND, int EPI>
cudaError_t launch_epi(int bn, int cg, const KernelParams& p, int grid, cudaStream_t stream)
{
    if(p.plan.cluster_k != 0)
    {
        if constexpr(MODE == MODE_GEMM)
        {
            const int ks = p.plan.ksplit;
            if(cg != 1 || !(ks == 2 || ks == 4 || ks == 8) || grid % ks != 0)
                return cudaErrorInvalidValue;
            switch(bn)
            {
            case 256: return launch_one<MODE, KIND, EPI, 256, 1, VARIANT_CLUSTER_K>(p, grid, stream);
            case 128: return launch_one<MODE, KIND, EPI, 128, 1, VARIANT_CLUSTER_K>(p, grid, stream);
            case 64: return launch_one<MODE, KIND, EPI, 64, 1, VARIANT_CLUSTER_K>(p, grid, stream);
            default: return cudaErrorInvalidValue;
            }
        }
        else
            return cudaErrorInvalidValue;
    }
    if(p.plan.stream_k != 0)
    {
        if constexpr(MODE != MODE_GEMM)
            return cudaErrorInvalidValue;
        else if constexpr(!HasKSplit<MODE, KIND, EPI>::value)
        {
            // balanced K ranges for a kernel family whose plain instances do not carry them: 256-wide tiles only
            if(bn != 256 || (cg != 1 && cg != 2))
                return cudaErrorInvalidValue;
            return cg == 2 ? launch_one<MODE, KIND, EPI, 256, 2, VARIANT_BALANCED>(p, grid, stream)
                           : launch_one<MODE, KIND, EPI, 256, 1, VARIANT_BALANCED>(p, grid, stream);
        }
    }
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

// How many clusters of `ks` CTAs of the cluster K-split kernel (256-wide tile; the narrower ones use the same
// shared memory per CTA) the device holds at once: clusters are placed inside one GPC each, so this is less than
// SMs / ks and depends on how many SMs each GPC of the part has.
template <int MODE, int KIND, int EPI>
cudaError_t cluster_capacity(int ks, int* clusters)
{
    constexpr int BN = 256, CG = 1;
    constexpr int STAGES = StagesFor<BN, CG, MODE>::value;
    constexpr int KSUB   = StagesFor<BN, CG, MODE>::ksub;
    constexpr int SMEM   = SmemLayout<BN, STAGES, CG, KSUB>::DYN_BYTES;
    auto kern            = contraction_kernel<MODE, KIND, EPI, BN, STAGES, CG, KSUB, VARIANT_CLUSTER_K>;
    cudaError_t err      = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if(err != cudaSuccess)
        return err;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim            = dim3(ks * 64, 1, 1);
    cfg.blockDim           = dim3(threads_for<MODE>(), 1, 1);
    cfg.dynamicSmemBytes   = SMEM;
    cudaLaunchAttribute attr[1];
    attr[0].id               = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs                = attr;
    cfg.numAttrs             = 1;
    return cudaOccupancyMaxActiveClusters(clusters, kern, &cfg);
}

typedef cudaError_t (*LaunchFn)(int, int, const KernelParams&, int, cudaStream_t);

// nullptr when the (mode, kind, epilogue) combination is not instantiated.
LaunchFn find_launch(int mode, int kind, int epi);

} // namespace ckb
