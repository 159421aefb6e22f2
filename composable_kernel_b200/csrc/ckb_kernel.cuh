// The persistent, warp-specialised tcgen05 contraction kernel.
//
// One CTA per SM walks work items  w = blockIdx.x, blockIdx.x + gridDim.x, ...
//   warp 0     TMA producer : fills a ring of STAGES shared-memory stages (A tile 128 x 128 B,
//                             B tile <=BN x 128 B, 128-byte swizzle; K-major, or for the other
//                             GEMM layouts MN-major: boxes of 128 B of M|N positions x the k rows)
//   warp 1     MMA issuer   : one thread issues tcgen05.mma (128 x width x 16|32) into one of two
//                             TMEM accumulators (2 x BN columns) and commits to mbarriers
//   warps 2-9  epilogue     : tcgen05.ld the finished accumulator (two warps per TMEM lane
//                             quarter, each half of the columns), apply the fused epilogue with
//                             the D values prefetched one segment ahead, store E with 128-bit stores
// The second accumulator lets the epilogue of item i overlap the main loop of item i+1.
//
// Work items.  The output is cut into 128 x BN tiles.  With G CTAs, the first floor(T/G)*G tiles
// are whole-tile items; the R = T mod G tiles of the last, partial wave are each cut into
// `split` column slices of BN/split columns (R*split <= G), so that the tail occupies all SMs
// instead of R of them.
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
// CTA pairs (CG = 2).  Large problems run with thread-block clusters of two CTAs on one
// 256 x BN tile: tcgen05.mma.cta_group::2 is issued by the leader CTA (cluster rank 0) and reads
// both CTAs' shared memory; each CTA loads its own 128 rows of A and its own half of the B rows
// (no load has more than one destination CTA), keeps 128 rows of the accumulator in its own
// tensor memory and runs its own epilogue.  All loads post their bytes on the LEADER's "full"
// barrier; the leader's tcgen05.commit fans the "empty" / "accumulator full" arrivals out to both
// CTAs; the epilogue warps of both CTAs release the accumulator on the leader's barrier.
// Compared with CG = 1 a stage holds half the B tile, so the ring is 6 deep instead of 4 and
// every SM pulls a third less operand traffic through L2.
//
// Every wait is bounded: after `wait_limit_ns` the waiting thread records a code in the status
// word, raises the CTA's abort flag, and all roles drain and leave through the common exit,
// which frees the tensor memory.
#pragma once
#include <type_traits>

#include "ckb_epilogue.cuh"
#include "ckb_ptx.cuh"

namespace ckb {

enum { MODE_GEMM = 0, MODE_GROUPED = 1, MODE_CONV = 2 };
enum { KIND_F16 = 0, KIND_BF16 = 1, KIND_I8 = 2 };

constexpr int BM            = 128; // rows of an output tile = TMEM lanes
constexpr int BK_BYTES      = 128; // bytes of K per stage row = one swizzle span
constexpr int NUM_EPI_WARPS = 8;
constexpr int NUM_THREADS   = 64 + 32 * NUM_EPI_WARPS;

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
    CUtensorMap tm_a;       // 128 B
    CUtensorMap tm_b;       // box of BN rows
    CUtensorMap tm_b_split; // box of BN/split rows (tail slices)
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
    CUtensorMap tm_a;       // GEMM: A (K, M).  CONV: im2col map over the NHWC input
    CUtensorMap tm_b;       // GEMM: B^T (K, N). CONV: weights as (C, Y*X, K); box of BN rows
    CUtensorMap tm_b_split; // same tensor, box of BN/split rows
    EpilogueArgs epi;       // GROUPED: e/d/ld fields come from the group entry instead
    const GroupEntry* groups;
    int32_t group_count;
    int32_t total_tiles; // T: 128 x BN tiles over all groups
    int32_t split_start; // first tile index whose tile is cut into column slices (= T if none)
    int32_t split;       // slices per tail tile (1, 2 or 4)
    int32_t total_work;  // split_start + (T - split_start) * split
    int32_t M, N;        // GEMM / CONV problem (CONV: M = N*Ho*Wo, N = K_out)
    int32_t tiles_n;
    int32_t num_kb;      // k blocks per tile (GEMM / CONV)
    int32_t vec_ok;      // 128-bit epilogue access allowed
    int32_t mn_major;    // bit 0: A is M-contiguous (column-major A); bit 1: B is N-contiguous (row-major B)
    ConvGeom conv;
    uint64_t wait_limit_ns;
    uint32_t* status; // device status word
};

template <int BN, int STAGES, int CG>
struct SmemLayout
{
    static constexpr int A_BYTES     = BM * BK_BYTES;
    static constexpr int B_BYTES     = (BN / CG) * BK_BYTES; // a CTA of a pair holds half the B rows
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFFSET  = STAGES * STAGE_BYTES;
    // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], drain
    static constexpr int NUM_BARS    = 2 * STAGES + 5;
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

// What one work item covers.
struct WorkItem
{
    int m_blk;   // row tile
    int n_start; // first output column
    int width;   // columns of this item (BN, or BN/split for a tail slice)
    int num_kb;
    const GroupEntry* group; // MODE_GROUPED only
    bool is_slice;
};

template <int MODE, int BN>
__device__ __forceinline__ WorkItem decode_work(const KernelParams& P, int w)
{
    WorkItem wi;
    int tile, slice = 0;
    wi.width    = BN;
    wi.is_slice = false;
    if(w < P.split_start)
        tile = w;
    else
    {
        const int q = w - P.split_start;
        tile        = P.split_start + q / P.split;
        slice       = q % P.split;
        wi.width    = BN / P.split;
        wi.is_slice = P.split > 1;
    }
    int n_blk;
    if constexpr(MODE == MODE_GROUPED)
    {
        const GroupEntry* G = P.groups + find_group(P.groups, P.group_count, tile);
        const int local     = tile - G->tile_start;
        wi.m_blk            = local / G->tiles_n;
        n_blk               = local % G->tiles_n;
        wi.num_kb           = G->num_kb;
        wi.group            = G;
    }
    else
    {
        wi.m_blk  = tile / P.tiles_n;
        n_blk     = tile % P.tiles_n;
        wi.num_kb = P.num_kb;
        wi.group  = nullptr;
    }
    wi.n_start = n_blk * BN + slice * wi.width;
    return wi;
}

// Epilogue of one warp: rows = its TMEM lane quarter, columns [n_begin, n_end) of row m.
// tmem_addr = lane base | first column of the span inside the accumulator.
template <int EPI, int KIND>
__device__ __forceinline__ void epilogue_span(uint32_t tmem_addr, const EpilogueArgs& ea, int64_t m,
                                              bool row_ok, int64_t n_begin, int64_t n_end, bool vec_ok)
{
    using T          = typename std::conditional<KIND == KIND_BF16, __nv_bfloat16, __half>::type;
    constexpr int ND = (KIND == KIND_I8) ? 0 : epi_num_d(EPI);
    const int nchunks = n_end > n_begin ? static_cast<int>((n_end - n_begin + 31) / 32) : 0;
    DChunk cur, nxt;
    if constexpr(ND > 0)
    {
        if(row_ok && vec_ok && n_end - n_begin >= 32)
            epi_load_d<EPI, T>(cur, ea, m, n_begin);
    }
    for(int c = 0; c < nchunks; ++c)
    {
        const int64_t n0 = n_begin + c * 32;
        const int ncols  = static_cast<int>(n_end - n0 < 32 ? n_end - n0 : 32);
        if constexpr(ND > 0)
        {
            if(row_ok && vec_ok && n_end - (n0 + 32) >= 32)
                epi_load_d<EPI, T>(nxt, ea, m, n0 + 32);
        }
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_addr + c * 32, v);
        tmem_ld_wait();
        if(row_ok)
        {
            if constexpr(KIND == KIND_I8)
                epi_store_row_i8<EPI>(v, ea, m, n0, ncols, vec_ok);
            else
            {
                if(vec_ok && ncols == 32)
                    epi_store_vec_f<EPI, T>(v, cur, ea, m, n0);
                else
                    epi_store_scalar_f<EPI, T>(v, ea, m, n0, ncols);
            }
        }
        if constexpr(ND > 0)
            cur = nxt;
    }
}

// EPI (the fused epilogue functor) is a template parameter: one functor per kernel keeps the
// epilogue warps inside the 168-register budget that ten warps per SM leave.
template <int MODE, int KIND, int EPI, int BN, int STAGES, int CG>
__global__ void __launch_bounds__(NUM_THREADS, 1) contraction_kernel(const __grid_constant__ KernelParams P)
{
    using L = SmemLayout<BN, STAGES, CG>;
    constexpr int TILE_M = BM * CG;
    constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;
    constexpr int UMMA_K_BYTES   = 32; // 16 x 16-bit or 32 x 8-bit
    constexpr int K_STEPS        = BK_BYTES / UMMA_K_BYTES;
    constexpr int BK_ELEMS       = (KIND == KIND_I8) ? 128 : 64;
    constexpr uint32_t C_FMT     = (KIND == KIND_I8) ? 2u : 1u;
    constexpr uint32_t AB_FMT    = (KIND == KIND_F16) ? 0u : 1u; // f16 | bf16 or s8
    // MN-major operands (GEMM layouts other than row-major A x column-major B): one TMA box = one
    // swizzle atom column = BK_ELEMS positions of M|N (128 bytes) x BK_ELEMS rows of k
    constexpr int ATOM_BYTES     = BK_ELEMS * BK_BYTES;
    const bool a_mn              = MODE != MODE_CONV && (P.mn_major & 1) != 0;
    const bool b_mn              = MODE != MODE_CONV && (P.mn_major & 2) != 0;

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
    // CG = 2: rank of this CTA in its pair (0 = leader), work is indexed by pair.
    const uint32_t cta_rank = (CG == 2) ? cluster_ctarank() : 0u;
    const bool is_leader    = cta_rank == 0;
    const int unit          = (CG == 2) ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int num_units     = (CG == 2) ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < STAGES; ++s)
        {
            mbar_init(full_bar(s), 1);  // the (leader's) producer arrival + all bytes of the stage
            mbar_init(empty_bar(s), 1); // one tcgen05.commit arrival
        }
        for(int a = 0; a < 2; ++a)
        {
            mbar_init(tmem_full_bar(a), 1);
            mbar_init(tmem_empty_bar(a), NUM_EPI_WARPS * CG); // one arrival per epilogue warp (of both CTAs)
        }
        mbar_init(drain_bar, 1);
        misc[1] = 0;
        misc[2] = 0;
        fence_mbar_init();
    }
    if(warp == 1)
    {
        if constexpr(CG == 2)
        {
            tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(&misc[0])), TMEM_COLS);
            tmem_relinquish_pair();
        }
        else
        {
            tmem_alloc(smem_u32(const_cast<uint32_t*>(&misc[0])), TMEM_COLS);
            tmem_relinquish();
        }
    }
    tc_fence_before_sync();
    if constexpr(CG == 2)
        cluster_sync_all(); // the peer's barriers must exist before anything is posted on them
    else
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
            int stage           = 0;
            uint32_t phase      = 0;
            uint32_t issued     = 0; // bit s: a load was issued into stage s
            uint32_t last_phase = 0; // bit s: phase of the last load issued into stage s
            bool ok             = true;
            for(int w = unit; ok && w < P.total_work; w += num_units)
            {
                const WorkItem wi       = decode_work<MODE, BN>(P, w);
                const CUtensorMap* tm_a = &P.tm_a;
                const CUtensorMap* tm_b = wi.is_slice ? &P.tm_b_split : &P.tm_b;
                if constexpr(MODE == MODE_GROUPED)
                {
                    tm_a = &wi.group->tm_a;
                    tm_b = wi.is_slice ? &wi.group->tm_b_split : &wi.group->tm_b;
                }
                // bytes of one stage over the whole CTA group (posted on the leader's barrier)
                const uint32_t tx_bytes = CG * L::A_BYTES + wi.width * BK_BYTES;
                const int b_rows        = wi.width / CG;                       // B rows this CTA loads
                const int a_row0        = wi.m_blk * TILE_M + cta_rank * BM;  // first A row of this CTA
                const int b_row0        = wi.n_start + cta_rank * b_rows;
                // CONV: first output pixel of this CTA's rows in (n, ho, wo)
                int cv_n = 0, cv_h = 0, cv_w = 0;
                if constexpr(MODE == MODE_CONV)
                {
                    const int m0  = a_row0;
                    cv_n          = m0 / P.conv.HoWo;
                    const int rem = m0 - cv_n * P.conv.HoWo;
                    const int ho  = rem / P.conv.Wo;
                    const int wo  = rem - ho * P.conv.Wo;
                    cv_h          = ho * P.conv.stride_h - P.conv.pad_h;
                    cv_w          = wo * P.conv.stride_w - P.conv.pad_w;
                }
                int cv_y = 0, cv_x = 0, cv_cb = 0;
                for(int kb = 0; kb < wi.num_kb; ++kb)
                {
                    ok = bounded_wait(empty_bar(stage), phase ^ 1u, wc, WAIT_EMPTY);
                    if(!ok)
                        break;
                    const uint32_t a_dst = base_addr + stage * L::STAGE_BYTES;
                    const uint32_t b_dst = a_dst + L::A_BYTES;
                    if(is_leader)
                        mbar_arrive_expect_tx(full_bar(stage), tx_bytes);
                    if constexpr(CG == 2)
                    {
                        const uint32_t bar = mapa_shared(full_bar(stage), 0); // the leader's barrier
                        if constexpr(MODE == MODE_CONV)
                        {
                            tma_load_im2col_4d_pair(a_dst, tm_a, bar, cv_cb * BK_ELEMS, cv_w, cv_h, cv_n,
                                                    static_cast<uint16_t>(cv_x * P.conv.dil_w),
                                                    static_cast<uint16_t>(cv_y * P.conv.dil_h));
                            tma_load_3d_pair(b_dst, tm_b, bar, cv_cb * BK_ELEMS, cv_y * P.conv.X + cv_x,
                                             b_row0);
                        }
                        else
                        {
                            if(a_mn)
                                for(int j = 0; j < BM / BK_ELEMS; ++j)
                                    tma_load_2d_pair(a_dst + j * ATOM_BYTES, tm_a, bar, a_row0 + j * BK_ELEMS,
                                                     kb * BK_ELEMS);
                            else
                                tma_load_2d_pair(a_dst, tm_a, bar, kb * BK_ELEMS, a_row0);
                            if(b_mn)
                                for(int j = 0; j * BK_ELEMS < b_rows; ++j)
                                    tma_load_2d_pair(b_dst + j * ATOM_BYTES, tm_b, bar, b_row0 + j * BK_ELEMS,
                                                     kb * BK_ELEMS);
                            else
                                tma_load_2d_pair(b_dst, tm_b, bar, kb * BK_ELEMS, b_row0);
                        }
                    }
                    else if constexpr(MODE == MODE_CONV)
                    {
                        tma_load_im2col_4d(a_dst, tm_a, full_bar(stage), cv_cb * BK_ELEMS, cv_w, cv_h,
                                           cv_n, static_cast<uint16_t>(cv_x * P.conv.dil_w),
                                           static_cast<uint16_t>(cv_y * P.conv.dil_h));
                        tma_load_3d(b_dst, tm_b, full_bar(stage), cv_cb * BK_ELEMS,
                                    cv_y * P.conv.X + cv_x, wi.n_start);
                    }
                    else
                    {
                        if(a_mn)
                            for(int j = 0; j < BM / BK_ELEMS; ++j)
                                tma_load_2d(a_dst + j * ATOM_BYTES, tm_a, full_bar(stage), a_row0 + j * BK_ELEMS,
                                            kb * BK_ELEMS);
                        else
                            tma_load_2d(a_dst, tm_a, full_bar(stage), kb * BK_ELEMS, a_row0);
                        if(b_mn)
                            for(int j = 0; j * BK_ELEMS < b_rows; ++j)
                                tma_load_2d(b_dst + j * ATOM_BYTES, tm_b, full_bar(stage), b_row0 + j * BK_ELEMS,
                                            kb * BK_ELEMS);
                        else
                            tma_load_2d(b_dst, tm_b, full_bar(stage), kb * BK_ELEMS, b_row0);
                    }
                    if constexpr(MODE == MODE_CONV)
                    {
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
                    issued |= 1u << stage;
                    last_phase = (last_phase & ~(1u << stage)) | (phase << stage);
                    if(++stage == STAGES)
                    {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            // Do not leave while a bulk copy may still write shared memory.  The leader's barriers
            // count the bytes of both CTAs, and the pair leaves together (cluster sync at the exit).
            for(int s = 0; s < STAGES; ++s)
                if(is_leader && (issued & (1u << s)))
                {
                    WaitCtx drain{&misc[2], P.wait_limit_ns, P.status}; // misc[2] stays 0: wait regardless of abort
                    bounded_wait(full_bar(s), (last_phase >> s) & 1u, drain, WAIT_DRAIN);
                }
        }
    }
    else if(warp == 1)
    {
        // ------------------------------------------------------------------ MMA issuer
        if(lane == 0 && is_leader)
        {
            int stage       = 0;
            uint32_t phase  = 0;
            int iter        = 0;
            bool ok         = true;
            bool issued_any = false;
            for(int w = unit; ok && w < P.total_work; w += num_units, ++iter)
            {
                const WorkItem wi        = decode_work<MODE, BN>(P, w);
                const uint32_t idesc     = make_idesc(C_FMT, AB_FMT, TILE_M, static_cast<uint32_t>(wi.width),
                                                      a_mn ? 1u : 0u, b_mn ? 1u : 0u);
                const int acc            = iter & 1;
                const uint32_t acc_phase = (iter >> 1) & 1;
                ok = bounded_wait(tmem_empty_bar(acc), acc_phase ^ 1u, wc, WAIT_TMEM_EMPTY);
                if(!ok)
                    break;
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for(int kb = 0; kb < wi.num_kb; ++kb)
                {
                    ok = bounded_wait(full_bar(stage), phase, wc, WAIT_FULL);
                    if(!ok)
                        break;
                    tc_fence_after_sync();
                    const uint32_t a_addr = base_addr + stage * L::STAGE_BYTES;
                    const uint64_t a_desc = a_mn ? make_smem_desc_mn_sw128(a_addr, ATOM_BYTES)
                                                 : make_smem_desc_k_sw128(a_addr);
                    const uint64_t b_desc = b_mn ? make_smem_desc_mn_sw128(a_addr + L::A_BYTES, ATOM_BYTES)
                                                 : make_smem_desc_k_sw128(a_addr + L::A_BYTES);
#pragma unroll
                    for(int k = 0; k < K_STEPS; ++k)
                    {
                        // one UMMA K step: 32 bytes along a K-major row, or (BK_ELEMS / K_STEPS) rows of
                        // 128 bytes in an MN-major tile
                        const uint64_t koff_k  = static_cast<uint64_t>((k * UMMA_K_BYTES) >> 4);
                        const uint64_t koff_mn = static_cast<uint64_t>((k * (BK_ELEMS / K_STEPS) * BK_BYTES) >> 4);
                        const uint64_t koff_a  = a_mn ? koff_mn : koff_k;
                        const uint64_t koff_b  = b_mn ? koff_mn : koff_k;
                        if constexpr(CG == 2)
                        {
                            if constexpr(KIND == KIND_I8)
                                mma_i8_ss_pair(tmem_d, a_desc + koff_a, b_desc + koff_b, idesc, (kb | k) != 0);
                            else
                                mma_f16_ss_pair(tmem_d, a_desc + koff_a, b_desc + koff_b, idesc, (kb | k) != 0);
                        }
                        else
                        {
                            if constexpr(KIND == KIND_I8)
                                mma_i8_ss(tmem_d, a_desc + koff_a, b_desc + koff_b, idesc, (kb | k) != 0);
                            else
                                mma_f16_ss(tmem_d, a_desc + koff_a, b_desc + koff_b, idesc, (kb | k) != 0);
                        }
                    }
                    issued_any = true;
                    // the stage is free (in both CTAs) once these MMAs have read it
                    if constexpr(CG == 2)
                        mma_commit_pair_mc(empty_bar(stage), 3);
                    else
                        mma_commit(empty_bar(stage));
                    if(++stage == STAGES)
                    {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if(ok) // accumulator complete (in both CTAs)
                {
                    if constexpr(CG == 2)
                        mma_commit_pair_mc(tmem_full_bar(acc), 3);
                    else
                        mma_commit(tmem_full_bar(acc));
                }
            }
            // Every MMA issued must be finished before the tensor memory is freed.
            if(issued_any)
            {
                if constexpr(CG == 2)
                    mma_commit_pair(drain_bar);
                else
                    mma_commit(drain_bar);
                WaitCtx drain{&misc[2], P.wait_limit_ns, P.status};
                bounded_wait(drain_bar, 0, drain, WAIT_DRAIN);
            }
        }
    }
    else
    {
        // ------------------------------------------------------------------ epilogue warps
        const int quarter = warp & 3;        // TMEM lane quarter this warp may read
        const int half    = (warp - 2) >> 2; // which half of the item's columns
        int iter          = 0;
        bool ok           = true;
        for(int w = unit; ok && w < P.total_work; w += num_units, ++iter)
        {
            const WorkItem wi = decode_work<MODE, BN>(P, w);
            EpilogueArgs ea   = P.epi;
            int Mdim = P.M, Ndim = P.N;
            bool vec_ok = P.vec_ok != 0;
            if constexpr(MODE == MODE_GROUPED)
            {
                const GroupEntry* G = wi.group;
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
            const int span          = wi.width >> 1; // columns per epilogue warp (>= 32)
            const int64_t m =
                static_cast<int64_t>(wi.m_blk) * TILE_M + cta_rank * BM + quarter * 32 + lane;
            const bool row_ok       = m < Mdim;
            const int64_t n_begin   = static_cast<int64_t>(wi.n_start) + half * span;
            const int64_t n_end_raw = n_begin + span;
            const int64_t n_end     = n_end_raw < Ndim ? n_end_raw : Ndim;

            const int acc            = iter & 1;
            const uint32_t acc_phase = (iter >> 1) & 1;
            ok = bounded_wait(tmem_full_bar(acc), acc_phase, wc, WAIT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if(!ok)
                break;
            tc_fence_after_sync();
            const uint32_t tmem_addr =
                tmem_base + acc * BN + half * span + (static_cast<uint32_t>(quarter * 32) << 16);
            epilogue_span<EPI, KIND>(tmem_addr, ea, m, row_ok, n_begin, n_end, vec_ok);
            // Release the accumulator: all of this warp's tcgen05.ld have completed.
            tc_fence_before_sync();
            __syncwarp();
            if(lane == 0)
            {
                if constexpr(CG == 2)
                    mbar_arrive_cluster(mapa_shared(tmem_empty_bar(acc), 0)); // the leader's barrier
                else
                    mbar_arrive(tmem_empty_bar(acc));
            }

            // Ask L2 for the D values of this CTA's next item while its main loop runs.
            if constexpr(KIND != KIND_I8)
            {
                const int wn = w + num_units;
                if(epi_num_d(EPI) > 0 && wn < P.total_work)
                {
                    const WorkItem nx = decode_work<MODE, BN>(P, wn);
                    EpilogueArgs en   = P.epi;
                    int Mn = P.M, Nn = P.N;
                    if constexpr(MODE == MODE_GROUPED)
                    {
                        en.d0   = nx.group->d0;
                        en.d1   = nx.group->d1;
                        en.ldd0 = nx.group->ldd0;
                        en.ldd1 = nx.group->ldd1;
                        Mn      = nx.group->M;
                        Nn      = nx.group->N;
                    }
                    const int spn    = nx.width >> 1;
                    const int64_t mn =
                        static_cast<int64_t>(nx.m_blk) * TILE_M + cta_rank * BM + quarter * 32 + lane;
                    const int64_t nb = static_cast<int64_t>(nx.n_start) + half * spn;
                    if(mn < Mn && nb < Nn)
                    {
                        const int64_t ne = nb + spn < Nn ? nb + spn : Nn;
                        epi_prefetch_d(en, mn, nb, static_cast<int>(ne - nb) * 2, 2);
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------------- common exit
    tc_fence_before_sync();
    if constexpr(CG == 2)
        cluster_sync_all(); // the leader's MMAs read the peer's shared memory until the very end
    else
        __syncthreads();
    tc_fence_after_sync();
    if(warp == 1)
    {
        if constexpr(CG == 2)
            tmem_dealloc_pair(tmem_base, TMEM_COLS);
        else
            tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

} // namespace ckb
