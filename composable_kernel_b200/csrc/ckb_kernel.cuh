// The persistent, warp-specialised tcgen05 contraction kernel.
//
// One CTA per SM walks tiles  t = blockIdx.x, blockIdx.x + gridDim.x, ...  of the output.
//   warp 0   TMA producer : fills a ring of STAGES shared-memory stages (A tile 128 x 128 B,
//                           B tile BN x 128 B, both K-major, 128-byte swizzle)
//   warp 1   MMA issuer   : one thread issues tcgen05.mma (128 x BN x 16|32) into one of two
//                           TMEM accumulators (2 x BN columns) and commits to mbarriers
//   warps 2-5 epilogue    : tcgen05.ld the finished accumulator (each warp its lane quarter),
//                           apply the fused epilogue, store E with 128-bit stores
// The second accumulator lets the epilogue of tile i overlap the main loop of tile i+1.
//
// Three problem sources share the kernel:
//   MODE_GEMM     one A/B tensor-map pair in the kernel parameters
//   MODE_GROUPED  a device table of per-group tensor maps + tile prefix sums; each role
//                 finds the group of a tile by binary search (the counterpart of
//                 kernel_grouped_gemm_xdl, device/device_grouped_gemm_xdl.hpp:24-87)
//   MODE_CONV     A is read with an im2col tensor map straight from the NHWC image, so the
//                 implicit-GEMM address generation of
//                 device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp:311-369 happens in the TMA unit
//
// Every wait is bounded: after `wait_limit_ns` the waiting thread records a code in the status
// word, raises the CTA's abort flag, and all roles drain and leave through the common exit,
// which frees the tensor memory.
#pragma once
#include "ckb_epilogue.cuh"
#include "ckb_ptx.cuh"

namespace ckb {

enum { MODE_GEMM = 0, MODE_GROUPED = 1, MODE_CONV = 2 };
enum { KIND_F16 = 0, KIND_BF16 = 1, KIND_I8 = 2 };

constexpr int BM          = 128; // rows of an output tile = TMEM lanes
constexpr int BK_BYTES    = 128; // bytes of K per stage row = one swizzle span
constexpr int NUM_THREADS = 192;
constexpr int EPI_WARP0   = 2;

// Device status word (KernelParams::status points at it): 0 = fine; otherwise
// (code << 24) | (block & 0xFFFFFF) of the first wait that gave up.

enum {
    WAIT_EMPTY      = 1, // producer waiting for a free stage
    WAIT_FULL       = 2, // MMA waiting for TMA data
    WAIT_TMEM_EMPTY = 3, // MMA waiting for the epilogue to release an accumulator
    WAIT_TMEM_FULL  = 4, // epilogue waiting for the MMA
    WAIT_DRAIN      = 5  // exit path waiting for copies / MMAs in flight
};

// One group of a grouped GEMM (lives in the caller's device workspace).
struct alignas(128) GroupEntry
{
    CUtensorMap tm_a; // 128 B
    CUtensorMap tm_b; // 128 B
    int32_t M, N, K;
    int32_t tiles_n;
    int32_t tile_start; // first global tile index of this group
    int32_t num_kb;
    int32_t vec_ok;
    int32_t pad_;
    void* e;
    const void* d0;
    const void* d1;
    int64_t lde, ldd0, ldd1;
};

struct ConvGeom
{
    int32_t Ho, Wo, HoWo;
    int32_t Y, X, c_blocks; // c_blocks = ceil(C / channels per stage)
    int32_t stride_h, stride_w, dil_h, dil_w, pad_h, pad_w;
};

struct KernelParams
{
    CUtensorMap tm_a; // GEMM: A (K, M).  CONV: im2col map over the NHWC input
    CUtensorMap tm_b; // GEMM: B^T (K, N). CONV: weights as (C, Y*X, K)
    EpilogueArgs epi; // GROUPED: e/d/ld fields come from the group entry instead
    const GroupEntry* groups;
    int32_t group_count;
    int32_t total_tiles;
    int32_t M, N;     // GEMM / CONV problem (CONV: M = N*Ho*Wo, N = K_out)
    int32_t tiles_n;
    int32_t num_kb;   // k blocks per tile (GEMM / CONV)
    int32_t vec_ok;   // 128-bit epilogue access allowed
    int32_t pad_;
    ConvGeom conv;
    uint64_t wait_limit_ns;
    uint32_t* status; // device status word
};

template <int BN, int STAGES>
struct SmemLayout
{
    static constexpr int A_BYTES     = BM * BK_BYTES;
    static constexpr int B_BYTES     = BN * BK_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFFSET  = STAGES * STAGE_BYTES;
    // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], drain
    static constexpr int NUM_BARS = 2 * STAGES + 5;
    static constexpr int MISC_OFFSET = BAR_OFFSET + NUM_BARS * 8;
    static constexpr int TOTAL       = MISC_OFFSET + 16;
    static constexpr int DYN_BYTES   = TOTAL + 1024; // slack to align the base to 1024 B
};

struct WaitCtx
{
    volatile uint32_t* abort_flag; // shared
    uint64_t limit_ns;
    uint32_t* status;
};

// Bounded mbarrier wait.  Returns false when it gave up (or another role already did).
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, const WaitCtx& w,
                                             uint32_t code)
{
    if(mbar_try_wait(bar, parity))
        return true;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins    = 0;
    while(true)
    {
        if(mbar_try_wait(bar, parity))
            return true;
        if((++spins & 63u) == 0)
        {
            if(*w.abort_flag != 0)
                return false;
            if(global_timer_ns() - t0 > w.limit_ns || spins > (1u << 30))
            {
                atomicCAS(w.status, 0u, (code << 24) | (blockIdx.x & 0xFFFFFFu));
                *w.abort_flag = 1;
                return false;
            }
        }
    }
}

// Finds g with tile_start[g] <= tile < tile_start[g+1].
__device__ __forceinline__ int find_group(const GroupEntry* groups, int group_count, int tile)
{
    int lo = 0, hi = group_count - 1;
    while(lo < hi)
    {
        const int mid = (lo + hi + 1) >> 1;
        if(groups[mid].tile_start <= tile)
            lo = mid;
        else
            hi = mid - 1;
    }
    return lo;
}

template <int EPI, int KIND>
__device__ __forceinline__ void epilogue_rows(uint32_t tmem_acc, int lane_quarter, int lane,
                                              const EpilogueArgs& ea, int64_t m, bool row_ok,
                                              int64_t n_base, int64_t n_limit, int bn,
                                              bool vec_ok)
{
    for(int chunk = 0; chunk < bn / 32; ++chunk)
    {
        const int64_t n0 = n_base + chunk * 32;
        if(n0 >= n_limit)
            break; // uniform over the CTA: the rest of the tile is out of range
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_acc + (static_cast<uint32_t>(lane_quarter * 32) << 16) + chunk * 32, v);
        tmem_ld_wait();
        if(row_ok)
        {
            const int ncols = static_cast<int>(n_limit - n0 < 32 ? n_limit - n0 : 32);
            if constexpr(KIND == KIND_I8)
                epi_store_row_i8<EPI>(v, ea, m, n0, ncols, vec_ok);
            else if constexpr(KIND == KIND_BF16)
                epi_store_row_f<EPI, __nv_bfloat16>(v, ea, m, n0, ncols, vec_ok);
            else
                epi_store_row_f<EPI, __half>(v, ea, m, n0, ncols, vec_ok);
        }
    }
    (void)lane;
}

template <int MODE, int KIND, int BN, int STAGES>
__global__ void __launch_bounds__(NUM_THREADS, 1) contraction_kernel(const __grid_constant__ KernelParams P)
{
    using L = SmemLayout<BN, STAGES>;
    constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;
    constexpr int UMMA_K_BYTES   = 32; // 16 x 16-bit or 32 x 8-bit
    constexpr int K_STEPS        = BK_BYTES / UMMA_K_BYTES;
    constexpr int BK_ELEMS       = (KIND == KIND_I8) ? 128 : 64;
    constexpr uint32_t IDESC =
        (KIND == KIND_I8) ? make_idesc(2u, 1u, BM, BN) : make_idesc(1u, KIND == KIND_BF16 ? 1u : 0u, BM, BN);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr  = smem_u32(smem_raw);
    const uint32_t base_addr = (raw_addr + 1023u) & ~1023u;
    uint8_t* smem            = smem_raw + (base_addr - raw_addr);

    const uint32_t bar_base = base_addr + L::BAR_OFFSET;
    auto full_bar           = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar          = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tmem_full_bar      = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tmem_empty_bar     = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    const uint32_t drain_bar = bar_base + 8u * (2 * STAGES + 4);
    volatile uint32_t* misc  = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFFSET);
    // misc[0] = TMEM base address, misc[1] = abort flag, misc[2] = constant 0

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < STAGES; ++s)
        {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for(int a = 0; a < 2; ++a)
        {
            mbar_init(tmem_full_bar(a), 1);
            mbar_init(tmem_empty_bar(a), 4); // one arrival per epilogue warp
        }
        mbar_init(drain_bar, 1);
        misc[1] = 0;
        misc[2] = 0;
        fence_mbar_init();
    }
    if(warp == 1)
    {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(&misc[0])), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = misc[0];

    WaitCtx wc{&misc[1], P.wait_limit_ns, P.status};

    if(warp == 0)
    {
        // ------------------------------------------------------------------ TMA producer
        if(lane == 0)
        {
            if constexpr(MODE != MODE_GROUPED)
            {
                tma_prefetch_desc(&P.tm_a);
                tma_prefetch_desc(&P.tm_b);
            }
            int stage = 0;
            uint32_t phase = 0;
            uint32_t issued = 0; // bit s set: stage s holds a load this thread has not seen land
            uint32_t last_phase = 0; // bit s: phase of the last load issued into stage s
            bool ok = true;
            for(int tile = blockIdx.x; ok && tile < P.total_tiles; tile += gridDim.x)
            {
                const CUtensorMap* tm_a = &P.tm_a;
                const CUtensorMap* tm_b = &P.tm_b;
                int m_blk, n_blk, num_kb;
                if constexpr(MODE == MODE_GROUPED)
                {
                    const int g         = find_group(P.groups, P.group_count, tile);
                    const GroupEntry* G = P.groups + g;
                    const int local     = tile - G->tile_start;
                    m_blk               = local / G->tiles_n;
                    n_blk               = local % G->tiles_n;
                    num_kb              = G->num_kb;
                    tm_a                = &G->tm_a;
                    tm_b                = &G->tm_b;
                }
                else
                {
                    m_blk  = tile / P.tiles_n;
                    n_blk  = tile % P.tiles_n;
                    num_kb = P.num_kb;
                }
                // CONV: first output pixel of the tile in (n, ho, wo)
                int cv_n = 0, cv_h = 0, cv_w = 0;
                if constexpr(MODE == MODE_CONV)
                {
                    const int m0  = m_blk * BM;
                    cv_n          = m0 / P.conv.HoWo;
                    const int rem = m0 - cv_n * P.conv.HoWo;
                    const int ho  = rem / P.conv.Wo;
                    const int wo  = rem - ho * P.conv.Wo;
                    cv_h          = ho * P.conv.stride_h - P.conv.pad_h;
                    cv_w          = wo * P.conv.stride_w - P.conv.pad_w;
                }
                int cv_y = 0, cv_x = 0, cv_cb = 0;
                for(int kb = 0; kb < num_kb; ++kb)
                {
                    ok = bounded_wait(empty_bar(stage), phase ^ 1u, wc, WAIT_EMPTY);
                    if(!ok)
                        break;
                    const uint32_t a_dst = base_addr + stage * L::STAGE_BYTES;
                    const uint32_t b_dst = a_dst + L::A_BYTES;
                    mbar_arrive_expect_tx(full_bar(stage), L::STAGE_BYTES);
                    if constexpr(MODE == MODE_CONV)
                    {
                        tma_load_im2col_4d(a_dst, tm_a, full_bar(stage), cv_cb * BK_ELEMS, cv_w, cv_h,
                                           cv_n, static_cast<uint16_t>(cv_x * P.conv.dil_w),
                                           static_cast<uint16_t>(cv_y * P.conv.dil_h));
                        tma_load_3d(b_dst, tm_b, full_bar(stage), cv_cb * BK_ELEMS,
                                    cv_y * P.conv.X + cv_x, n_blk * BN);
                        if(++cv_cb == P.conv.c_blocks)
                        {
                            cv_cb = 0;
                            if(++cv_x == P.conv.X)
                            {
                                cv_x = 0;
                                ++cv_y;
                            }
                        }
                    }
                    else
                    {
                        tma_load_2d(a_dst, tm_a, full_bar(stage), kb * BK_ELEMS, m_blk * BM);
                        tma_load_2d(b_dst, tm_b, full_bar(stage), kb * BK_ELEMS, n_blk * BN);
                    }
                    issued |= 1u << stage;
                    last_phase = (last_phase & ~(1u << stage)) | (phase << stage);
                    if(++stage == STAGES)
                    {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            // Do not leave while a bulk copy may still write this CTA's shared memory.
            for(int s = 0; s < STAGES; ++s)
                if(issued & (1u << s))
                {
                    WaitCtx drain{&misc[2], P.wait_limit_ns, P.status}; // misc[2] stays 0: wait regardless of abort
                    bounded_wait(full_bar(s), (last_phase >> s) & 1u, drain, WAIT_DRAIN);
                }
        }
    }
    else if(warp == 1)
    {
        // ------------------------------------------------------------------ MMA issuer
        if(lane == 0)
        {
            int stage = 0;
            uint32_t phase = 0;
            int iter = 0;
            bool ok = true;
            bool issued_any = false;
            for(int tile = blockIdx.x; ok && tile < P.total_tiles; tile += gridDim.x, ++iter)
            {
                int num_kb;
                if constexpr(MODE == MODE_GROUPED)
                    num_kb = P.groups[find_group(P.groups, P.group_count, tile)].num_kb;
                else
                    num_kb = P.num_kb;
                const int acc            = iter & 1;
                const uint32_t acc_phase = (iter >> 1) & 1;
                ok = bounded_wait(tmem_empty_bar(acc), acc_phase ^ 1u, wc, WAIT_TMEM_EMPTY);
                if(!ok)
                    break;
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for(int kb = 0; kb < num_kb; ++kb)
                {
                    ok = bounded_wait(full_bar(stage), phase, wc, WAIT_FULL);
                    if(!ok)
                        break;
                    tc_fence_after_sync();
                    const uint32_t a_addr = base_addr + stage * L::STAGE_BYTES;
                    const uint64_t a_desc = make_smem_desc_k_sw128(a_addr);
                    const uint64_t b_desc = make_smem_desc_k_sw128(a_addr + L::A_BYTES);
#pragma unroll
                    for(int k = 0; k < K_STEPS; ++k)
                    {
                        const uint64_t koff = static_cast<uint64_t>((k * UMMA_K_BYTES) >> 4);
                        if constexpr(KIND == KIND_I8)
                            mma_i8_ss(tmem_d, a_desc + koff, b_desc + koff, IDESC, (kb | k) != 0);
                        else
                            mma_f16_ss(tmem_d, a_desc + koff, b_desc + koff, IDESC, (kb | k) != 0);
                    }
                    issued_any = true;
                    mma_commit(empty_bar(stage)); // stage is free once these MMAs have read it
                    if(++stage == STAGES)
                    {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if(ok)
                    mma_commit(tmem_full_bar(acc)); // accumulator complete
            }
            // Every MMA issued must be finished before the tensor memory is freed.
            if(issued_any)
            {
                mma_commit(drain_bar);
                WaitCtx drain{&misc[2], P.wait_limit_ns, P.status};
                bounded_wait(drain_bar, 0, drain, WAIT_DRAIN);
            }
        }
    }
    else
    {
        // ------------------------------------------------------------------ epilogue warps
        const int quarter = warp & 3; // TMEM lane quarter this warp may read
        int iter          = 0;
        bool ok           = true;
        for(int tile = blockIdx.x; ok && tile < P.total_tiles; tile += gridDim.x, ++iter)
        {
            EpilogueArgs ea = P.epi;
            int m_blk, n_blk, Mdim, Ndim;
            bool vec_ok;
            if constexpr(MODE == MODE_GROUPED)
            {
                const int g         = find_group(P.groups, P.group_count, tile);
                const GroupEntry* G = P.groups + g;
                const int local     = tile - G->tile_start;
                m_blk               = local / G->tiles_n;
                n_blk               = local % G->tiles_n;
                Mdim                = G->M;
                Ndim                = G->N;
                vec_ok              = G->vec_ok != 0;
                ea.e                = G->e;
                ea.d0               = G->d0;
                ea.d1               = G->d1;
                ea.lde              = G->lde;
                ea.ldd0             = G->ldd0;
                ea.ldd1             = G->ldd1;
            }
            else
            {
                m_blk  = tile / P.tiles_n;
                n_blk  = tile % P.tiles_n;
                Mdim   = P.M;
                Ndim   = P.N;
                vec_ok = P.vec_ok != 0;
            }
            const int acc            = iter & 1;
            const uint32_t acc_phase = (iter >> 1) & 1;
            ok = bounded_wait(tmem_full_bar(acc), acc_phase, wc, WAIT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if(!ok)
                break;
            tc_fence_after_sync();
            const uint32_t tmem_acc = tmem_base + acc * BN;
            const int64_t m         = static_cast<int64_t>(m_blk) * BM + quarter * 32 + lane;
            const bool row_ok       = m < Mdim;
            const int64_t n_base    = static_cast<int64_t>(n_blk) * BN;
#define CKB_EPI_CASE(E)                                                                         \
    case E:                                                                                     \
        epilogue_rows<E, KIND>(tmem_acc, quarter, lane, ea, m, row_ok, n_base, Ndim, BN, vec_ok); \
        break;
            if constexpr(KIND == KIND_I8)
            {
                switch(ea.kind)
                {
                    CKB_EPI_CASE(CKB_EPI_PASSTHROUGH)
                    CKB_EPI_CASE(CKB_EPI_RELU)
                    CKB_EPI_CASE(CKB_EPI_REQUANT_RELU_REQUANT)
                    CKB_EPI_CASE(CKB_EPI_REQUANT_RELU_REQUANT_RNE)
                default: break;
                }
            }
            else
            {
                switch(ea.kind)
                {
                    CKB_EPI_CASE(CKB_EPI_PASSTHROUGH)
                    CKB_EPI_CASE(CKB_EPI_RELU)
                    CKB_EPI_CASE(CKB_EPI_SCALE)
                    CKB_EPI_CASE(CKB_EPI_FASTGELU)
                    CKB_EPI_CASE(CKB_EPI_ADD)
                    CKB_EPI_CASE(CKB_EPI_ADD_RELU_F16)
                    CKB_EPI_CASE(CKB_EPI_BILINEAR)
                    CKB_EPI_CASE(CKB_EPI_ADD_ADD_FASTGELU)
                    CKB_EPI_CASE(CKB_EPI_ADD_RELU_ADD)
                    CKB_EPI_CASE(CKB_EPI_ADD_RELU)
                    CKB_EPI_CASE(CKB_EPI_ADD_HARDSWISH)
                default: break;
                }
            }
#undef CKB_EPI_CASE
            // Release the accumulator: all of this warp's tcgen05.ld have completed.
            tc_fence_before_sync();
            __syncwarp();
            if(lane == 0)
                mbar_arrive(tmem_empty_bar(acc));
        }
    }

    // ---------------------------------------------------------------------- common exit
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if(warp == 1)
        tmem_dealloc(tmem_base, TMEM_COLS);
}

} // namespace ckb
