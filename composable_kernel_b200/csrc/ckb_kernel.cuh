// The persistent, warp-specialised tcgen05 contraction kernel.
//
// One CTA per SM walks work items  w = blockIdx.x, blockIdx.x + gridDim.x, ...
//   warp 0     TMA producer : fills a ring of STAGES shared-memory stages, each KSUB k blocks of an
//                             A tile (128 x 128 B) and a B tile (<=BN x 128 B), 128-byte swizzle;
//                             K-major, or for the other GEMM layouts MN-major: boxes of 128 B of
//                             M|N positions x the k rows.  One lane per box, one warp-wide copy.
//   warp 1     MMA issuer   : one thread issues tcgen05.mma (128 x width x 16|32) into one of two
//                             TMEM accumulators (2 x BN columns) and commits to mbarriers
//   warp 10    (convolution only) issues the weight copies, warp 0 then only the im2col copies
//   warps 2-9  epilogue     : tcgen05.ld the finished accumulator (two warps per TMEM lane
//                             quarter, each half of the columns), apply the fused epilogue with
//                             the D values prefetched one segment ahead, write each 32 x 32 segment
//                             of E to a per-warp shared-memory tile and send it off with a TMA store
// The second accumulator lets the epilogue of item i overlap the main loop of item i+1.
//
// Start-up (barrier initialisation, tensor-memory allocation, cluster sync) touches no global memory: the
// kernel then executes griddepcontrol.wait, so that under programmatic dependent launch the start-up
// overlaps the tail of the previous kernel of the stream.
//
// Work items.  The output is cut into 128 x BN tiles.  With G CTAs, the first floor(T/G)*G tiles
// are whole-tile items; the R = T mod G tiles of the last, partial wave are each cut into
// `split` column slices of BN/split columns (R*split <= G), so that the tail occupies all SMs
// instead of R of them.
//
// K-split tail (16-bit MODE_GEMM kernels without D tensors, with a scratch buffer).  Column slices of a tail tile cost almost as much as a whole
// tile, because the MMA role is bound by the number of instructions it issues, not by their width.  When
// KernelParams::ksplit > 1 the R tail tiles are cut along K instead: after its first whole tile every unit runs
// one K slice of a tail tile (full-width MMAs over 1/ksplit of the k blocks) and parks the raw accumulator in the
// scratch buffer; after its next whole tile the unit that ran slice i sums column part i (BN / ksplit columns)
// of that tail tile over all slices, in slice order (deterministic), and applies the epilogue - on the epilogue
// warps only, while the MMA role already works on the next tile.  A per-tile counter in global memory (release /
// acquire, bounded wait) orders slices and reduction.
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
// Compared with CG = 1 a k block holds half the B tile (32 KB instead of 48 KB), and every SM pulls a
// third less operand traffic through L2.
//
// Every wait is bounded: after `wait_limit_ns` the waiting thread records a code in the status
// word, raises the CTA's abort flag, and all roles drain and leave through the common exit,
// which frees the tensor memory.
#pragma once
#include <type_traits>

#include "ckb_epilogue.cuh"
#include "ckb_plan.h"
#include "ckb_ptx.cuh"

// Cycle counters of the three roles, compiled in only with -DCKB_TRACE (a profiling build): per CTA
// sixteen 64-bit words in KernelParams::trace
//   [0] producer: cycles waiting for a free stage     [1] producer: cycles in its loop
//   [2] MMA: cycles waiting for operand data          [3] MMA: cycles waiting for a free accumulator
//   [4] MMA: cycles in its loop                       [5] first epilogue warp: cycles waiting for the MMA
//   [6] first epilogue warp: cycles in its loop       [7] k blocks issued by the MMA role
//   [8] MMA: cycles issuing tcgen05.mma               [9] MMA: cycles issuing tcgen05.commit
//   first epilogue warp, K-split plans: [10] cycles waiting on a tile counter, [11] cycles in fix-up epilogues,
//   [12] cycles parking accumulators
#ifdef CKB_TRACE
#define CKB_TR(...) __VA_ARGS__
#else
#define CKB_TR(...)
#endif

namespace ckb {

enum { KIND_F16 = 0, KIND_BF16 = 1, KIND_I8 = 2 };

constexpr int BK_BYTES      = 128; // bytes of K per stage row = one swizzle span
constexpr int NUM_EPI_WARPS = 8;
constexpr int NUM_THREADS   = 64 + 32 * NUM_EPI_WARPS;
// The convolution runs one warp more: its weight copies are issued by a warp of their own, so that they do not
// queue behind the im2col copy of the same stage in the producer warp (an im2col copy blocks its issuer for about
// 450 cycles; +2.3 % on the N128 C192 71x71 K256 3x3 stride-2 problem, same box, interleaved runs).
template <int MODE>
constexpr int threads_for()
{
    return MODE == MODE_CONV ? NUM_THREADS + 32 : NUM_THREADS;
}

// Device status word (KernelParams::status points at it): 0 = fine; otherwise
// (code << 24) | (block & 0xFFFFFF) of the first wait that gave up.
enum {
    WAIT_EMPTY      = 1, // producer waiting for a free stage
    WAIT_FULL       = 2, // MMA waiting for TMA data
    WAIT_TMEM_EMPTY = 3, // MMA waiting for the epilogue to release an accumulator
    WAIT_TMEM_FULL  = 4, // epilogue waiting for the MMA
    WAIT_DRAIN      = 5, // exit path waiting for copies / MMAs in flight
    WAIT_KSLICES    = 6  // reduction waiting for the K slices of its tail tile
};

// One group of a grouped GEMM (lives in the caller's device workspace).
struct alignas(128) GroupEntry
{
    CUtensorMap tm_a;       // 128 B
    CUtensorMap tm_b;       // box of BN rows
    CUtensorMap tm_b_split; // box of BN/split rows (tail slices)
    CUtensorMap tm_e;       // E as (N, M), 32 x 32 box, for the staged stores of the epilogue
    int32_t M, N, K;
    int32_t tiles_n;
    int32_t tile_start; // first global tile index of this group
    int32_t num_kb;
    int32_t vec_ok;
    int32_t tiles_m;
    int32_t m_fastest;  // tile order inside the group (see tile_position)
    int32_t pad_[3];
    void* e;
    const void* d0;
    const void* d1;
    int64_t lde, ldd0, ldd1;
};

// Division of a 31-bit unsigned number by a run-time constant as multiply-high and shift (host-computed:
// p = 31 + ceil(log2 d), mul = ceil(2^p / d), shr = p - 32; quotient = umulhi(n, mul) >> shr; d = 1 is passed through).
struct FastDiv
{
    uint32_t mul, shr, d, pad_;
};
__device__ __forceinline__ uint32_t fast_div(uint32_t n, const FastDiv& f)
{
    return f.d == 1 ? n : __umulhi(n, f.mul) >> f.shr;
}

struct ConvGeom
{
    int32_t Ho, Wo, HoWo;
    int32_t Y, X, c_blocks; // c_blocks = ceil(C / channels per k block)
    int32_t stride_h, stride_w, dil_h, dil_w, pad_h, pad_w;
    // 3-D convolution (nd3 != 0): depth extents; a 2-D problem has Do = Z = 1
    int32_t nd3, Do, DoHoWo, Z, stride_d, dil_d, pad_d, pad_;
    FastDiv div_wo, div_howo, div_dohowo; // the producer splits a row index into (n, do, ho, wo) once per tile
};

struct KernelParams
{
    CUtensorMap tm_a;       // GEMM: A (K, M[, batch]).  CONV: im2col map over the NHWC input
    CUtensorMap tm_b;       // GEMM: B^T (K, N[, batch]). CONV: weights as (C, Y*X, K); box of BN rows
    CUtensorMap tm_b_split; // same tensor, box of BN/split rows
    CUtensorMap tm_e;       // E as (N, M[, batch]), 32 x 32 box (valid when vec_ok; GROUPED: in the group entry)
    EpilogueArgs epi;       // GROUPED: e/d/ld fields come from the group entry instead
    const GroupEntry* groups;
    PlanParams plan;     // which unit runs which tile / slice in which slot (ckb_plan.h)
    int32_t M, N;        // GEMM / CONV problem (CONV: M = N*Ho*Wo, N = K_out)
    int32_t vec_ok;      // 128-bit epilogue access allowed
    int32_t mn_major;    // bit 0: A is M-contiguous (column-major A); bit 1: B is N-contiguous (row-major B)
    int64_t batch_stride_e, batch_stride_d0, batch_stride_d1; // elements between batches of E / D0 / D1
    uint32_t* ks_partials; // [tail tile][slice][TILE_M rows][BN columns] raw 32-bit accumulators
    uint32_t* ks_counters; // one per tail tile, zero between launches
    uint32_t* ks_flags;    // balanced K ranges: one per (parking slot, CTA of the pair, epilogue warp), set by the
                           // warp that parked its block, cleared by the one warp that reads it back
    uint32_t ks_wait_extra; // test hook: added to the arrival count a reduction waits for, so that the wait runs out
    uint32_t pad_;
    ConvGeom conv;
    uint64_t wait_limit_ns;
    uint32_t* status; // device status word
    unsigned long long* trace; // role cycle counters (profiling builds only, else null)
};

// One stage holds KSUB consecutive k blocks (each 128 bytes of K): A block 0 .. KSUB-1, then B block 0 .. KSUB-1.
template <int BN, int STAGES, int CG, int KSUB>
struct SmemLayout
{
    static constexpr int A_SUB_BYTES = BM * BK_BYTES;
    static constexpr int B_SUB_BYTES = (BN / CG) * BK_BYTES; // a CTA of a pair holds half the B rows
    static constexpr int A_BYTES     = KSUB * A_SUB_BYTES;
    static constexpr int B_BYTES     = KSUB * B_SUB_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // staging tiles of the epilogue's TMA stores: two 2 KiB tiles per epilogue warp
    static constexpr int EPI_OFFSET     = STAGES * STAGE_BYTES;
    static constexpr int EPI_WARP_BYTES = 2 * 2048;
    static constexpr int BAR_OFFSET     = EPI_OFFSET + NUM_EPI_WARPS * EPI_WARP_BYTES;
    // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], drain
    static constexpr int NUM_BARS    = 2 * STAGES + 5;
    static constexpr int MISC_OFFSET = BAR_OFFSET + NUM_BARS * 8;
    static constexpr int TOTAL       = MISC_OFFSET + 16;
    static constexpr int DYN_BYTES   = TOTAL + 1024; // slack to align the base to 1024 B
};

// The exit path waits for copies and MMAs in flight with a limit of its own: the caller's limit may be short (it
// decides how soon a role gives up on another role), but a CTA must not leave while a bulk copy may still write
// its shared memory or an MMA may still write its tensor memory.
constexpr uint64_t kDrainLimitNs = 2000000000ull;

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

// Kernel instances that carry the K-split tail and the whole-problem split through the scratch: 16-bit GEMMs whose
// epilogue reads no D tensor (the host enables them only for those; the reduction holds four parked slices in
// registers next to the epilogue's state, and leaving it out of the others keeps their epilogue inside the register
// budget).
template <int MODE, int KIND, int EPI>
struct HasKSplit
{
    static constexpr bool value = MODE == MODE_GEMM && KIND != KIND_I8 && epi_num_d(EPI) == 0;
};
// Kernel variants (last template argument of the kernel).  The balanced K ranges need parking and a fix-up loop;
// the D-less 16-bit GEMM kernels carry them anyway (they share the parking with the K-split tail), for the other
// plain GEMMs - fused D epilogues, int8 - they are compiled into instances of their own, so that the kernels that
// run the whole-tile plans keep their register budget (with the loops compiled in, the Add + Add + FastGelu kernel
// spilled and lost 2.3 %, the int8 one 0.9 %).
enum { VARIANT_PLAIN = 0, VARIANT_CLUSTER_K = 1, VARIANT_BALANCED = 2 };

// One TMA box of a GEMM operand.  The operand maps of a batched GEMM are 3-D (the third coordinate is the
// batch index); those of a plain GEMM and the per-group maps of MODE_GROUPED are 2-D.
template <int MODE, int CG>
__device__ __forceinline__ void load_matrix_box(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1,
                                                bool batched, int batch)
{
    if(MODE == MODE_GEMM && batched)
    {
        if constexpr(CG == 2)
            tma_load_3d_pair(dst, tm, bar, c0, c1, batch);
        else
            tma_load_3d(dst, tm, bar, c0, c1, batch);
    }
    else
    {
        if constexpr(CG == 2)
            tma_load_2d_pair(dst, tm, bar, c0, c1);
        else
            tma_load_2d(dst, tm, bar, c0, c1);
    }
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Bounded wait until *counter >= target (acquire).  Returns false when it gave up.
__device__ __forceinline__ bool bounded_wait_counter(const uint32_t* counter, uint32_t target, const WaitCtx& w)
{
    if(ld_acquire_gpu(counter) >= target)
        return true;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins    = 0;
    while(true)
    {
        if(ld_acquire_gpu(counter) >= target)
            return true;
        if((++spins & 15u) == 0)
        {
            if(*w.abort_flag != 0)
                return false;
            if(global_timer_ns() - t0 > w.limit_ns || spins > (1u << 28))
            {
                atomicCAS(w.status, 0u, (static_cast<uint32_t>(WAIT_KSLICES) << 24) | (blockIdx.x & 0xFFFFFFu));
                *w.abort_flag = 1;
                return false;
            }
        }
    }
}

// K-split tail.  A parked slice is private to the (CTA, epilogue warp) that will read it back, so it is stored
// in the order that makes every warp-wide access contiguous: per warp a block of 32 rows x `ncols` columns laid
// out as [chunk of 32 columns][quad q of 4 columns][lane] of 16 bytes (lane = row), 512 contiguous bytes per
// instruction, instead of 32 row pieces a row pitch apart.
// Slice side: one warp parks `ncols` (a multiple of 32) raw accumulator columns of its 32 rows.
// With `flag` (balanced K ranges) the block is published to the one warp that will add it back: stores -> fence ->
// flag (a fence per chunk, so that the reader could start on chunk 0 while chunk 1 is parked, was tried: the fences
// made parking three times as slow).
__device__ __forceinline__ void park_span(uint32_t tmem_addr, uint32_t* block, int ncols, int lane, uint32_t* flag = nullptr)
{
    uint4* dst = reinterpret_cast<uint4*>(block) + lane;
    for(int c = 0; c < ncols / 32; ++c)
    {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_addr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for(int q = 0; q < 8; ++q)
            __stcg(dst + (c * 8 + q) * 32, make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
    }
    if(flag)
    {
        __threadfence();
        __syncwarp();
        if(lane == 0)
            atomicExch(flag, 1u);
    }
}

// Reduction side: v = sum over the slices, in slice order, of chunk `c` of this lane's row.  QUADS columns quads
// (of 4 columns) of all slices are in flight together: 2 normally, 1 where the epilogue also holds D values.
template <int KIND, int QUADS>
__device__ __forceinline__ void reduce_chunk(uint32_t (&v)[32], const uint32_t* block, int c, int lane, int ks,
                                             int64_t slice_stride)
{
    auto add = [](uint32_t a, uint32_t b) {
        if constexpr(KIND == KIND_I8)
            return a + b; // int32 accumulators
        else
            return __float_as_uint(__uint_as_float(a) + __uint_as_float(b));
    };
#pragma unroll
    for(int h = 0; h < 8 / QUADS; ++h)
    {
        uint4 acc[QUADS];
#pragma unroll
        for(int base = 0; base < 8; base += 4) // up to 8 slices, four in flight at a time, summed in slice order
        {
            if(base >= ks)
                break;
            uint4 t[4][QUADS];
#pragma unroll
            for(int sl = 0; sl < 4; ++sl)
                if(base + sl < ks)
                {
                    const uint4* src = reinterpret_cast<const uint4*>(block + (base + sl) * slice_stride) + lane;
#pragma unroll
                    for(int q = 0; q < QUADS; ++q)
                        t[sl][q] = __ldcg(src + (c * 8 + h * QUADS + q) * 32);
                }
#pragma unroll
            for(int q = 0; q < QUADS; ++q)
            {
                uint4 a = base == 0 ? t[0][q] : acc[q];
#pragma unroll
                for(int sl = 0; sl < 4; ++sl)
                    if((base > 0 || sl > 0) && base + sl < ks)
                    {
                        a.x = add(a.x, t[sl][q].x);
                        a.y = add(a.y, t[sl][q].y);
                        a.z = add(a.z, t[sl][q].z);
                        a.w = add(a.w, t[sl][q].w);
                    }
                acc[q] = a;
            }
        }
#pragma unroll
        for(int q = 0; q < QUADS; ++q)
        {
            v[(h * QUADS + q) * 4 + 0] = acc[q].x;
            v[(h * QUADS + q) * 4 + 1] = acc[q].y;
            v[(h * QUADS + q) * 4 + 2] = acc[q].z;
            v[(h * QUADS + q) * 4 + 3] = acc[q].w;
        }
    }
}

// Balanced K ranges: waits until the warp with this warp's rows and columns in another unit has parked its block.
// The flag is cleared for the next launch (this warp is its only reader).  Returns false when the wait gave up.
__device__ __forceinline__ bool wait_parked(uint32_t* flag, int lane, const WaitCtx& wc, uint32_t extra)
{
    bool ok = bounded_wait_counter(flag, 1u + extra, wc); // extra: test hook, a value the flag never takes
    ok      = __all_sync(0xffffffffu, ok);
    if(ok && lane == 0)
        __stcg(flag, 0u);
    return ok;
}

// Adds chunk `c` of this lane's row of a parked accumulator (`block`: the block of the warp that parked it) to the
// accumulator values in `v`.
template <int KIND>
__device__ __forceinline__ void fixup_chunk(uint32_t (&v)[32], const uint32_t* block, int c, int lane)
{
    auto add = [](uint32_t a, uint32_t b) {
        if constexpr(KIND == KIND_I8)
            return a + b;
        else
            return __float_as_uint(__uint_as_float(a) + __uint_as_float(b));
    };
    // eight loads of 16 bytes per thread in flight; two chunks at a time would not fit the register budget
    const uint4* src = reinterpret_cast<const uint4*>(block) + lane + c * 8 * 32;
    uint4 t[8];
#pragma unroll
    for(int q = 0; q < 8; ++q)
        t[q] = __ldcg(src + q * 32);
#pragma unroll
    for(int q = 0; q < 8; ++q)
    {
        v[4 * q]     = add(v[4 * q], t[q].x);
        v[4 * q + 1] = add(v[4 * q + 1], t[q].y);
        v[4 * q + 2] = add(v[4 * q + 2], t[q].z);
        v[4 * q + 3] = add(v[4 * q + 3], t[q].w);
    }
}

// Balanced K ranges, tiles in three parts: while the main loop of the head still runs, its epilogue warps copy the
// accumulator that the unit after next parked (the tile's last part, parked early) into the free half of the tensor
// memory, so that the final epilogue reads only one parked accumulator from L2.
__device__ __forceinline__ void prefetch_parked(uint32_t tmem_addr, const uint32_t* block, int ncols, int lane)
{
    for(int c = 0; c < ncols / 32; ++c)
    {
        const uint4* src = reinterpret_cast<const uint4*>(block) + lane + c * 8 * 32;
        uint32_t v[32];
#pragma unroll
        for(int q = 0; q < 8; ++q)
        {
            const uint4 t = __ldcg(src + q * 32);
            v[4 * q] = t.x, v[4 * q + 1] = t.y, v[4 * q + 2] = t.z, v[4 * q + 3] = t.w;
        }
        tmem_st_32x32b_x32(tmem_addr + c * 32, v);
    }
    tmem_st_wait();
}

// Balanced K ranges, the head of a tile: adds the accumulators that other units parked to the one in tensor memory
// at `tmem_addr` and writes the sum back, 32 columns at a time: first the block `parked` of the next unit, then the
// part of the unit after next - prefetched into tensor memory at `tmem_pre` (`has_pre`) or still in L2 (`parked2`).
// In k order whatever the timing, so the result does not depend on it.  The normal epilogue runs afterwards.
template <int KIND>
__device__ __forceinline__ void fixup_span(uint32_t tmem_addr, const uint32_t* parked, const uint32_t* parked2, bool has_pre,
                                           uint32_t tmem_pre, int ncols, int lane)
{
    for(int c = 0; c < ncols / 32; ++c)
    {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_addr + c * 32, v);
        tmem_ld_wait();
        fixup_chunk<KIND>(v, parked, c, lane);
        if(parked2 != nullptr)
            fixup_chunk<KIND>(v, parked2, c, lane);
        else if(has_pre)
        {
            uint32_t w[32];
            tmem_ld_32x32b_x32(tmem_pre + c * 32, w);
            tmem_ld_wait();
#pragma unroll
            for(int i = 0; i < 32; ++i)
                v[i] = (KIND == KIND_I8) ? v[i] + w[i] : __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(w[i]));
        }
        tmem_st_32x32b_x32(tmem_addr + c * 32, v);
    }
    tmem_st_wait();
}

// REDUCE = true: the accumulator comes from the parked K slices (`parked` = this warp's block in slice 0)
// instead of tensor memory.
template <int EPI, int KIND, bool REDUCE = false>
__device__ __forceinline__ void epilogue_span(uint32_t tmem_addr, const EpilogueArgs& ea, StoreStage& st, int lane,
                                              int64_t m, bool row_ok, int64_t n_begin, int64_t n_end, bool vec_ok,
                                              const uint32_t* parked = nullptr, int ks = 0, int64_t slice_stride = 0)
{
    using T          = typename std::conditional<KIND == KIND_BF16, __nv_bfloat16, __half>::type;
    constexpr int ND = (KIND == KIND_I8) ? 0 : epi_num_d(EPI);
    const int nchunks = n_end > n_begin ? static_cast<int>((n_end - n_begin + 31) / 32) : 0;
    // D values of the next chunk are fetched while this one is computed; the reduction path, whose registers hold
    // the parked slices, fetches the chunk's own D values together with them instead.
    constexpr bool PREFETCH_D = ND > 0 && !REDUCE;
    DChunk cur, nxt;
    if constexpr(PREFETCH_D)
    {
        if(row_ok && vec_ok && n_end - n_begin >= 32)
            epi_load_d<EPI, T>(cur, ea, m, n_begin);
    }
    for(int c = 0; c < nchunks; ++c)
    {
        const int64_t n0 = n_begin + c * 32;
        const int ncols  = static_cast<int>(n_end - n0 < 32 ? n_end - n0 : 32);
        if constexpr(PREFETCH_D)
        {
            if(row_ok && vec_ok && n_end - (n0 + 32) >= 32)
                epi_load_d<EPI, T>(nxt, ea, m, n0 + 32);
        }
        else if constexpr(ND > 0)
        {
            if(row_ok && vec_ok && ncols == 32)
                epi_load_d<EPI, T>(cur, ea, m, n0);
        }
        uint32_t v[32];
        if constexpr(REDUCE)
            reduce_chunk<KIND, (ND > 0) ? 1 : 2>(v, parked, c, lane, ks, slice_stride);
        else
        {
            tmem_ld_32x32b_x32(tmem_addr + c * 32, v);
            tmem_ld_wait();
        }
        if(vec_ok && ncols == 32) // warp-uniform: a whole segment leaves through the staged TMA store
        {
            const int row0 = static_cast<int>(m) - lane;
            if constexpr(KIND == KIND_I8)
            {
                uint4 out[2] = {};
                if(row_ok)
                    epi_compute_vec_i8<EPI>(out, v, ea);
                stage_and_store<32>(st, out, lane, static_cast<int>(n0), row0);
            }
            else
            {
                uint4 out[4] = {};
                if(row_ok)
                    epi_compute_vec_f<EPI, T>(out, v, cur, ea, m, n0);
                stage_and_store<64>(st, out, lane, static_cast<int>(n0), row0);
            }
        }
        else if(row_ok)
        {
            if constexpr(KIND == KIND_I8)
                epi_store_scalar_i8<EPI>(v, ea, m, n0, ncols);
            else
                epi_store_scalar_f<EPI, T>(v, ea, m, n0, ncols);
        }
        if constexpr(PREFETCH_D)
            cur = nxt;
    }
}

// ---- cluster K split: accumulators summed over distributed shared memory ------------------------------------------
// CTA r of the cluster sums column part r (BN / KS columns) of the tile.  Two ways of getting the slices there, both
// through the pipeline stages, which are free once every main loop of the cluster is over:
//   push  every CTA sends each quad of 4 columns of its raw accumulator straight to the CTA that owns the quad's part
//         (`st.shared::cluster`, fire and forget), into the slot of its own K slice there: [slice = sending CTA][quad
//         of the part][row] of 16 bytes.  Barrier before (the stages of the peers must be free), barrier after (release
//         / acquire), then each CTA finds all slices of its part in its own shared memory.
//   pull  every CTA keeps its accumulator at home ([quad][row] over all BN columns), one barrier, and CTA r reads its
//         part from every peer with `ld.shared::cluster` (latency bound: 16 reads in flight per thread); a barrier at
//         the exit keeps the shared memory alive until the peers have read it.
// Same box, 128 x 128 x 8192 with 8 CTAs per tile: 10.2 us pull, 9.6 push; 768 x 768 x 4096, 2 x 64-wide: 12.3 / 11.95;
// 1024 x 1024 x 8192, 4 x 256-wide: 19.1 / 20.25 (96 KiB of remote stores per CTA with the whole machine at it).  Push
// is used for clusters of 8 and for 64-wide tiles, pull for 2 and 4 CTAs on 128- and 256-wide tiles.
// In both a warp (32 consecutive rows) moves 512 contiguous bytes per instruction.
__device__ __forceinline__ bool cluster_push(int bn, int ks) { return ks == 8 || bn == 64; }
__device__ __forceinline__ uint32_t part_slot_bytes(int pw) { return static_cast<uint32_t>(pw) * (BM * 4u); }
__device__ __forceinline__ uint32_t partial_offset(int quad, int row) { return static_cast<uint32_t>(quad * BM + row) * 16u; }

// One epilogue warp sends `ncols` (a multiple of 32) accumulator columns of its 32 rows from tensor memory to their
// owners.  `pw_shift` = log2 of the part width in columns (>= 4).
__device__ __forceinline__ void stash_span(uint32_t tmem_addr, uint32_t partial_base, int my_rank, int pw_shift, int row,
                                           int col_begin, int ncols)
{
    const uint32_t slot = partial_base + static_cast<uint32_t>(my_rank) * part_slot_bytes(1 << pw_shift);
    for(int c = 0; c < ncols / 32; ++c)
    {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_addr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for(int q = 0; q < 8; ++q)
        {
            const int col      = col_begin + c * 32 + q * 4;
            const int owner    = col >> pw_shift;
            const int quad     = (col - (owner << pw_shift)) >> 2;
            const uint32_t dst = mapa_shared(slot + partial_offset(quad, row), static_cast<uint32_t>(owner));
            asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v[4 * q]), "r"(v[4 * q + 1]),
                         "r"(v[4 * q + 2]), "r"(v[4 * q + 3])
                         : "memory");
        }
    }
}

// pull: one epilogue warp moves `ncols` (a multiple of 32) accumulator columns of its 32 rows to this CTA's own tile
__device__ __forceinline__ void stash_span_local(uint32_t tmem_addr, uint32_t partial_base, int row, int col_begin, int ncols)
{
    for(int c = 0; c < ncols / 32; ++c)
    {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_addr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for(int q = 0; q < 8; ++q)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(partial_base +
                                                                          partial_offset((col_begin + c * 32) / 4 + q, row)),
                         "r"(v[4 * q]), "r"(v[4 * q + 1]), "r"(v[4 * q + 2]), "r"(v[4 * q + 3])
                         : "memory");
    }
}

__device__ __forceinline__ uint4 ld_cluster_v4(uint32_t cluster_addr)
{
    uint4 v;
    asm volatile("ld.shared::cluster.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(cluster_addr)
                 : "memory");
    return v;
}

__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

// CTA `rank` of a cluster of KS CTAs sums column part `rank` (BN / KS columns) of the tile over the slices that all
// CTAs of the cluster sent it, in slice order (deterministic), applies the epilogue and writes E.  `t` = 0 .. 255
// indexes the epilogue threads; consecutive threads take consecutive rows of one 16-column segment.
template <int EPI, int KIND, int BN, int KS, bool PUSH>
__device__ __forceinline__ void cluster_reduce_epilogue(const KernelParams& P, const WorkItem& wi, uint32_t partial_base,
                                                        int rank, int t)
{
    using T            = typename std::conditional<KIND == KIND_BF16, __nv_bfloat16, __half>::type;
    constexpr int ND   = (KIND == KIND_I8) ? 0 : epi_num_d(EPI);
    constexpr int PW   = BN / KS;           // columns of this CTA's part
    constexpr int SEGS = PW >> 4;           // 16-column segments per row
    constexpr int QG   = KS == 8 ? 2 : 4;   // quads of 4 columns whose slices are fetched together
    static_assert(PW >= 16 && PW % 16 == 0, "column parts are whole 16-column segments");
    const EpilogueArgs& ea = P.epi;
    uint32_t peer[KS];
#pragma unroll
    for(int s = 0; s < KS; ++s)
        peer[s] = PUSH ? 0u : mapa_shared(partial_base, static_cast<uint32_t>(s));
    for(int i = t; i < BM * SEGS; i += 32 * NUM_EPI_WARPS)
    {
        const int seg = i >> 7, row = i & (BM - 1);
        const int col0 = rank * PW + seg * 16; // first column inside the tile
        const int64_t m = static_cast<int64_t>(wi.m_blk) * BM + row, n0 = static_cast<int64_t>(wi.n_start) + col0;
        uint32_t v[16];
#pragma unroll
        for(int g = 0; g < 4 / QG; ++g)
        {
            uint4 part[QG][KS];
#pragma unroll
            for(int q = 0; q < QG; ++q)
#pragma unroll
                for(int s = 0; s < KS; ++s)
                {
                    if constexpr(PUSH)
                        part[q][s] = ld_shared_v4(partial_base + s * part_slot_bytes(PW) + partial_offset(seg * 4 + g * QG + q, row));
                    else
                        part[q][s] = ld_cluster_v4(peer[s] + partial_offset((col0 >> 2) + g * QG + q, row));
                }
#pragma unroll
            for(int q = 0; q < QG; ++q)
            {
                uint4 a = part[q][0];
#pragma unroll
                for(int s = 1; s < KS; ++s)
                {
                    if constexpr(KIND == KIND_I8)
                    {
                        a.x += part[q][s].x, a.y += part[q][s].y, a.z += part[q][s].z, a.w += part[q][s].w;
                    }
                    else
                    {
                        a.x = __float_as_uint(__uint_as_float(a.x) + __uint_as_float(part[q][s].x));
                        a.y = __float_as_uint(__uint_as_float(a.y) + __uint_as_float(part[q][s].y));
                        a.z = __float_as_uint(__uint_as_float(a.z) + __uint_as_float(part[q][s].z));
                        a.w = __float_as_uint(__uint_as_float(a.w) + __uint_as_float(part[q][s].w));
                    }
                }
                const int j = (g * QG + q) * 4;
                v[j] = a.x, v[j + 1] = a.y, v[j + 2] = a.z, v[j + 3] = a.w;
            }
        }
        if(m >= P.M || n0 >= P.N)
            continue;
        const bool full = P.vec_ok != 0 && n0 + 16 <= P.N;
        if constexpr(KIND == KIND_I8)
        {
            int8_t* e_row = static_cast<int8_t*>(ea.e) + m * ea.lde + n0;
            if(full)
            {
                uint32_t w[4];
#pragma unroll
                for(int k = 0; k < 4; ++k)
                {
                    uint32_t packed = 0;
#pragma unroll
                    for(int j = 0; j < 4; ++j)
                        packed |= (static_cast<uint32_t>(epi_apply_i8<EPI>(static_cast<int32_t>(v[4 * k + j]), ea.p)) & 0xFFu)
                                  << (8 * j);
                    w[k] = packed;
                }
                *reinterpret_cast<uint4*>(e_row) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            else
            {
#pragma unroll
                for(int j = 0; j < 16; ++j)
                    if(n0 + j < P.N)
                        e_row[j] = static_cast<int8_t>(epi_apply_i8<EPI>(static_cast<int32_t>(v[j]), ea.p));
            }
        }
        else
        {
            T* e_row        = static_cast<T*>(ea.e) + m * ea.lde + n0;
            const T* d0_row = ND >= 1 ? static_cast<const T*>(ea.d0) + m * ea.ldd0 + n0 : nullptr;
            const T* d1_row = ND >= 2 ? static_cast<const T*>(ea.d1) + m * ea.ldd1 + n0 : nullptr;
            alignas(16) T out[16];
#pragma unroll
            for(int j = 0; j < 16; ++j)
            {
                T a = from_f32<T>(0.0f), b = from_f32<T>(0.0f);
                if(n0 + j < P.N)
                {
                    if constexpr(ND >= 1)
                        a = d0_row[j];
                    if constexpr(ND >= 2)
                        b = d1_row[j];
                }
                out[j] = epi_apply_f<EPI, T>(__uint_as_float(v[j]), a, b, ea.p);
            }
            if(full)
            {
                reinterpret_cast<uint4*>(e_row)[0] = reinterpret_cast<const uint4*>(out)[0];
                reinterpret_cast<uint4*>(e_row)[1] = reinterpret_cast<const uint4*>(out)[1];
            }
            else
            {
#pragma unroll
                for(int j = 0; j < 16; ++j)
                    if(n0 + j < P.N)
                        e_row[j] = out[j];
            }
        }
    }
}

// EPI (the fused epilogue functor) is a template parameter: one functor per kernel keeps the
// epilogue warps inside the 168-register budget that ten warps per SM leave.
// VARIANT_CLUSTER_K: the cluster K split (MODE_GEMM, one CTA per tile): see decode_cluster_k in ckb_plan.h.
// VARIANT_BALANCED: see the enumeration.
template <int MODE, int KIND, int EPI, int BN, int STAGES, int CG, int KSUB, int VARIANT = VARIANT_PLAIN>
__global__ void __launch_bounds__(threads_for<MODE>(), 1) contraction_kernel(const __grid_constant__ KernelParams P)
{
    constexpr bool CK = VARIANT == VARIANT_CLUSTER_K;
    static_assert(!CK || (MODE == MODE_GEMM && CG == 1), "the cluster K split runs plain GEMM tiles on single CTAs");
    static_assert(VARIANT != VARIANT_BALANCED || MODE == MODE_GEMM, "balanced K ranges are a plan of the plain GEMM");
    using L = SmemLayout<BN, STAGES, CG, KSUB>;
    static_assert(!CK || BN * BM * 4 <= STAGES * L::STAGE_BYTES, "the raw accumulator tile must fit in the stages");
    constexpr bool KSPLIT = HasKSplit<MODE, KIND, EPI>::value && !CK;   // K-split tail / whole split through the scratch
    constexpr bool BAL    = MODE == MODE_GEMM && !CK && (HasKSplit<MODE, KIND, EPI>::value || VARIANT == VARIANT_BALANCED);
    constexpr bool PARK   = KSPLIT || BAL;                              // either: accumulators are parked
    constexpr int TILE_M  = BM * CG;
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
    const bool batched           = MODE == MODE_GEMM && P.plan.batch_tiles > 0;

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
    // CK: this CTA's K slice = its rank in the cluster, the cluster's tile = its index
    const int ck_rank = CK ? static_cast<int>(cluster_ctarank()) : 0;
    auto work_item    = [&](int slot) -> WorkItem {
        if constexpr(CK)
            return decode_cluster_k<BN>(P.plan, static_cast<int>(blockIdx.x) / P.plan.ksplit, ck_rank);
        else
            return decode_work<MODE, BN, PARK>(P.plan, P.groups, unit, num_units, slot);
    };

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
    // Everything above (barriers, tensor memory) touched no global memory and may overlap the tail of the previous
    // kernel of the stream; from here on its results (and the K-split scratch it may still use) are needed.
    grid_dependency_wait();
    grid_launch_dependents();

    WaitCtx wc{&misc[1], P.wait_limit_ns, P.status};

    constexpr bool SPLITP = MODE == MODE_CONV; // convolution: warp 0 issues the im2col copies, the last warp the weights
    if(warp == 0 || (SPLITP && warp == 2 + NUM_EPI_WARPS))
    {
        const bool does_b = !SPLITP || warp != 0;
        const bool does_a = !SPLITP || warp == 0;
        // ------------------------------------------------------------------ TMA producer
        // One lane per TMA box of a stage: the lanes compute their destinations and coordinates side by
        // side and the whole stage is issued by one warp-wide copy instruction (two for the convolution,
        // whose A box is an im2col copy), instead of one thread issuing the boxes one after the other.
        //   K-major GEMM operand : 1 box per k block              MN-major: one box per 128 bytes of M|N
        //   lanes [0, n_a) load A boxes, lanes [n_a, n_a + n_b) load B boxes, k block j = box / boxes per block
        if constexpr(MODE != MODE_GROUPED)
        {
            if(lane == 0)
            {
                tma_prefetch_desc(&P.tm_a);
                tma_prefetch_desc(&P.tm_b);
            }
        }
        int stage      = 0;
        uint32_t phase = 0;
        int loads      = 0; // stages filled so far
        bool ok        = true;
        // all bytes of a stage are counted on the leader's barrier
        const uint32_t bar0 = (CG == 2) ? mapa_shared(full_bar(0), 0) : full_bar(0);
        const int a_per_kb  = a_mn ? BM / BK_ELEMS : 1; // A boxes per k block
        CKB_TR(long long tr_wait = 0; const long long tr_start = clock64();)
        for(int slot = 0; ok && slot < P.plan.num_slots; ++slot)
        {
            const WorkItem wi = work_item(slot);
            if(wi.kind != ITEM_TILE && wi.kind != ITEM_KSLICE)
                continue;
            const CUtensorMap* tm_a = &P.tm_a;
            const CUtensorMap* tm_b = wi.is_slice ? &P.tm_b_split : &P.tm_b;
            if constexpr(MODE == MODE_GROUPED)
            {
                tm_a = &P.groups[wi.group].tm_a;
                tm_b = wi.is_slice ? &P.groups[wi.group].tm_b_split : &P.groups[wi.group].tm_b;
            }
            // bytes of one k block over the whole CTA group (posted on the leader's barrier)
            const uint32_t sub_bytes = CG * L::A_SUB_BYTES + wi.width * BK_BYTES;
            const int b_rows         = wi.width / CG;                      // B rows this CTA loads
            const int a_row0         = wi.m_blk * TILE_M + cta_rank * BM; // first A row of this CTA
            const int b_row0         = wi.n_start + cta_rank * b_rows;
            // this lane's box: operand, k block of the stage, offset inside the stage, MN coordinate
            const int b_per_kb = b_mn ? b_rows / BK_ELEMS : 1;
            const int n_a      = a_per_kb * KSUB;
            const bool is_b    = lane >= n_a;
            const int box      = is_b ? lane - n_a : lane;
            const int per_kb   = is_b ? b_per_kb : a_per_kb;
            const int box_j    = box / per_kb; // k block inside the stage
            const int box_i    = box - box_j * per_kb;
            const bool lane_on = lane < n_a + b_per_kb * KSUB;
            const bool box_mn  = is_b ? b_mn : a_mn;
            const uint32_t box_off =
                (is_b ? L::A_BYTES + box_j * L::B_SUB_BYTES : box_j * L::A_SUB_BYTES) + box_i * ATOM_BYTES;
            const int box_row         = (is_b ? b_row0 : a_row0) + box_i * BK_ELEMS;
            const CUtensorMap* box_tm = is_b ? tm_b : tm_a;
            // CONV: first output pixel of this CTA's rows in (n, do, ho, wo), as input coordinates
            int cv_n = 0, cv_d = 0, cv_h = 0, cv_w = 0;
            if constexpr(MODE == MODE_CONV)
            {
                uint32_t rem = static_cast<uint32_t>(a_row0);
                if(P.conv.nd3 != 0)
                {
                    cv_n = fast_div(rem, P.conv.div_dohowo);
                    rem -= cv_n * P.conv.DoHoWo;
                    const uint32_t od = fast_div(rem, P.conv.div_howo);
                    rem -= od * P.conv.HoWo;
                    cv_d = od * P.conv.stride_d - P.conv.pad_d;
                }
                else
                {
                    cv_n = fast_div(rem, P.conv.div_howo);
                    rem -= cv_n * P.conv.HoWo;
                }
                const uint32_t ho = fast_div(rem, P.conv.div_wo);
                const uint32_t wo = rem - ho * P.conv.Wo;
                cv_h              = ho * P.conv.stride_h - P.conv.pad_h;
                cv_w              = wo * P.conv.stride_w - P.conv.pad_w;
            }
            // CONV: running state of this lane's k block: channel coordinate, filter tap index and the tap's
            // offsets (tap position x dilation); stepped by KSUB blocks per stage without multiplications
            int cv_c = 0, cv_cb = 0, cv_x = 0, cv_y = 0, cv_tap = 0;
            uint32_t off_w = 0, off_h = 0, off_d = 0;
            auto conv_step = [&]() {
                cv_c += BK_ELEMS;
                if(++cv_cb == P.conv.c_blocks)
                {
                    cv_cb = 0;
                    cv_c  = 0;
                    ++cv_tap;
                    off_w += P.conv.dil_w;
                    if(++cv_x == P.conv.X)
                    {
                        cv_x  = 0;
                        off_w = 0;
                        off_h += P.conv.dil_h;
                        if(++cv_y == P.conv.Y)
                        {
                            cv_y  = 0;
                            off_h = 0;
                            off_d += P.conv.dil_d;
                        }
                    }
                }
            };
            if constexpr(MODE == MODE_CONV && KSUB > 1)
            {
                for(int i = 0; i < box_j && i < KSUB; ++i) // lanes of the later k blocks of a stage start further on
                    conv_step();
            }
            for(int kb = 0; kb < wi.num_kb; kb += KSUB)
            {
                CKB_TR(const long long tr0 = clock64();)
                ok = bounded_wait(empty_bar(stage), phase ^ 1u, wc, WAIT_EMPTY);
                ok = __all_sync(0xffffffffu, ok);
                CKB_TR(tr_wait += clock64() - tr0;)
                if(!ok)
                    break;
                const int nsub      = (wi.num_kb - kb < KSUB) ? wi.num_kb - kb : KSUB;
                const uint32_t dst  = base_addr + stage * L::STAGE_BYTES + box_off;
                const uint32_t bar  = bar0 + 8u * stage;
                if(is_leader && lane == 0 && does_a) // the bytes of both warps' copies are counted on this barrier
                    mbar_arrive_expect_tx(full_bar(stage), sub_bytes * nsub);
                if(lane_on && box_j < nsub && (is_b ? does_b : does_a))
                {
                    if constexpr(MODE == MODE_CONV)
                    {
                        const uint16_t ow = static_cast<uint16_t>(off_w), oh = static_cast<uint16_t>(off_h);
                        if(!is_b && P.conv.nd3 == 0)
                        {
                            if constexpr(CG == 2)
                                tma_load_im2col_4d_pair(dst, box_tm, bar, cv_c, cv_w, cv_h, cv_n, ow, oh);
                            else
                                tma_load_im2col_4d(dst, box_tm, bar, cv_c, cv_w, cv_h, cv_n, ow, oh);
                        }
                        else if(!is_b)
                        {
                            const uint16_t od = static_cast<uint16_t>(off_d);
                            if constexpr(CG == 2)
                                tma_load_im2col_5d_pair(dst, box_tm, bar, cv_c, cv_w, cv_h, cv_d, cv_n, ow, oh, od);
                            else
                                tma_load_im2col_5d(dst, box_tm, bar, cv_c, cv_w, cv_h, cv_d, cv_n, ow, oh, od);
                        }
                        else
                        {
                            if constexpr(CG == 2)
                                tma_load_3d_pair(dst, box_tm, bar, cv_c, cv_tap, b_row0);
                            else
                                tma_load_3d(dst, box_tm, bar, cv_c, cv_tap, wi.n_start);
                        }
                    }
                    else
                    {
                        const int k0 = (wi.kb_begin + kb + box_j) * BK_ELEMS;
                        load_matrix_box<MODE, CG>(dst, box_tm, bar, box_mn ? box_row : k0, box_mn ? k0 : box_row,
                                                  batched, wi.batch);
                    }
                }
                if constexpr(MODE == MODE_CONV)
                {
#pragma unroll
                    for(int i = 0; i < KSUB; ++i)
                        conv_step();
                }
                ++loads;
                if(++stage == STAGES)
                {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
        CKB_TR(if(P.trace && lane == 0) {
            P.trace[blockIdx.x * 16 + 0] = tr_wait;
            P.trace[blockIdx.x * 16 + 1] = clock64() - tr_start;
        })
        // Do not leave while a bulk copy may still write shared memory: wait for the last fill of every
        // stage used.  The leader's barriers count the bytes of both CTAs, and the pair leaves together
        // (cluster sync at the exit).  Fill number f (0-based) goes to stage f % STAGES with phase
        // (f / STAGES) & 1.
        if(is_leader && lane == 0 && warp == 0)
            for(int s = 0; s < STAGES && s < loads; ++s)
            {
                const int last_fill = ((loads - 1 - s) / STAGES) * STAGES + s;
                WaitCtx drain{&misc[2], kDrainLimitNs, P.status}; // misc[2] stays 0: wait regardless of abort
                bounded_wait(full_bar(s), static_cast<uint32_t>(last_fill / STAGES) & 1u, drain, WAIT_DRAIN);
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
            // Shared-memory descriptors: the high word (swizzle mode, stride / leading offsets) is constant, the
            // low word is the start address >> 4 and is stepped by a register per operand:
            //   K-major : 32 bytes along the 128-byte row per UMMA K step
            //   MN-major: (BK_ELEMS / K_STEPS) rows of 128 bytes per UMMA K step
            // and by `*_jump` from the last K step of one k block to the first of the next block of the stage.
            const uint64_t a_const = (a_mn ? make_smem_desc_mn_sw128(0, ATOM_BYTES) : make_smem_desc_k_sw128(0));
            const uint64_t b_const = (b_mn ? make_smem_desc_mn_sw128(0, ATOM_BYTES) : make_smem_desc_k_sw128(0));
            const uint32_t a_hi = static_cast<uint32_t>(a_const >> 32), b_hi = static_cast<uint32_t>(b_const >> 32);
            const uint32_t a_lo_const = static_cast<uint32_t>(a_const), b_lo_const = static_cast<uint32_t>(b_const);
            const uint32_t a_kstep = a_mn ? ((BK_ELEMS / K_STEPS) * BK_BYTES) >> 4 : UMMA_K_BYTES >> 4;
            const uint32_t b_kstep = b_mn ? ((BK_ELEMS / K_STEPS) * BK_BYTES) >> 4 : UMMA_K_BYTES >> 4;
            const uint32_t a_jump  = (L::A_SUB_BYTES >> 4) - (K_STEPS - 1) * a_kstep;
            const uint32_t b_jump  = (L::B_SUB_BYTES >> 4) - (K_STEPS - 1) * b_kstep;
            const uint32_t idesc_major = (a_mn ? 1u << 15 : 0u) | (b_mn ? 1u << 16 : 0u);
            CKB_TR(long long tr_full = 0, tr_acc = 0, tr_kb = 0, tr_issue = 0, tr_commit = 0;
                   const long long tr_start = clock64();)
            for(int slot = 0; ok && slot < P.plan.num_slots; ++slot)
            {
                const WorkItem wi = work_item(slot);
                if(wi.kind != ITEM_TILE && wi.kind != ITEM_KSLICE)
                    continue;
                const uint32_t idesc     = make_idesc(C_FMT, AB_FMT, TILE_M, static_cast<uint32_t>(wi.width)) | idesc_major;
                const int acc            = iter & 1;
                const uint32_t acc_phase = (iter >> 1) & 1;
                CKB_TR(const long long tr1 = clock64();)
                ok = bounded_wait(tmem_empty_bar(acc), acc_phase ^ 1u, wc, WAIT_TMEM_EMPTY);
                CKB_TR(tr_acc += clock64() - tr1;)
                if(!ok)
                    break;
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + acc * BN;
                uint32_t accumulate   = 0; // the first MMA of the item overwrites the accumulator
                for(int kb = 0; kb < wi.num_kb; kb += KSUB)
                {
                    CKB_TR(const long long tr0 = clock64();)
                    ok = bounded_wait(full_bar(stage), phase, wc, WAIT_FULL);
                    CKB_TR(tr_full += clock64() - tr0; ++tr_kb;)
                    if(!ok)
                        break;
                    const int nsub        = (wi.num_kb - kb < KSUB) ? wi.num_kb - kb : KSUB;
                    const uint32_t a_addr = base_addr + stage * L::STAGE_BYTES;
                    uint32_t a_lo         = a_lo_const | ((a_addr & 0x3FFFFu) >> 4);
                    uint32_t b_lo         = b_lo_const | (((a_addr + L::A_BYTES) & 0x3FFFFu) >> 4);
                    CKB_TR(const long long tr2 = clock64();)
#pragma unroll
                    for(int j = 0; j < KSUB; ++j)
                    {
                        if(KSUB > 1 && j >= nsub)
                            break;
#pragma unroll
                        for(int k = 0; k < K_STEPS; ++k)
                        {
                            if constexpr(CG == 2)
                            {
                                if constexpr(KIND == KIND_I8)
                                    mma_i8_ss_pair_split(tmem_d, a_lo, a_hi, b_lo, b_hi, idesc, accumulate);
                                else
                                    mma_f16_ss_pair_split(tmem_d, a_lo, a_hi, b_lo, b_hi, idesc, accumulate);
                            }
                            else
                            {
                                if constexpr(KIND == KIND_I8)
                                    mma_i8_ss_split(tmem_d, a_lo, a_hi, b_lo, b_hi, idesc, accumulate);
                                else
                                    mma_f16_ss_split(tmem_d, a_lo, a_hi, b_lo, b_hi, idesc, accumulate);
                            }
                            accumulate = 1;
                            a_lo += (k == K_STEPS - 1) ? a_jump : a_kstep;
                            b_lo += (k == K_STEPS - 1) ? b_jump : b_kstep;
                        }
                    }
                    issued_any = true;
                    CKB_TR(const long long tr3 = clock64(); tr_issue += tr3 - tr2;)
                    // the stage is free (in both CTAs) once these MMAs have read it
                    if constexpr(CG == 2)
                        mma_commit_pair_mc(empty_bar(stage), 3);
                    else
                        mma_commit(empty_bar(stage));
                    CKB_TR(tr_commit += clock64() - tr3;)
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
                ++iter;
            }
            CKB_TR(if(P.trace) {
                P.trace[blockIdx.x * 16 + 2] = tr_full;
                P.trace[blockIdx.x * 16 + 3] = tr_acc;
                P.trace[blockIdx.x * 16 + 4] = clock64() - tr_start;
                P.trace[blockIdx.x * 16 + 7] = tr_kb;
                P.trace[blockIdx.x * 16 + 8] = tr_issue;
                P.trace[blockIdx.x * 16 + 9] = tr_commit;
            })
            // Every MMA issued must be finished before the tensor memory is freed.
            if(issued_any)
            {
                if constexpr(CG == 2)
                    mma_commit_pair(drain_bar);
                else
                    mma_commit(drain_bar);
                WaitCtx drain{&misc[2], kDrainLimitNs, P.status};
                bounded_wait(drain_bar, 0, drain, WAIT_DRAIN);
            }
        }
    }
    else if(warp < 2 + NUM_EPI_WARPS)
    {
        // ------------------------------------------------------------------ epilogue warps
        const int quarter = warp & 3;        // TMEM lane quarter this warp may read
        const int half    = (warp - 2) >> 2; // which half of the item's columns
        int iter          = 0;
        bool ok           = true;
        StoreStage st;
        st.buf   = base_addr + L::EPI_OFFSET + (warp - 2) * L::EPI_WARP_BYTES;
        st.count = 0;
        st.tm_e   = &P.tm_e;
        st.batch  = -1;
        if(MODE != MODE_GROUPED && P.vec_ok != 0 && lane == 0)
            tma_prefetch_desc(&P.tm_e);
        CKB_TR(long long tr_wait = 0, tr_ctr = 0, tr_fix = 0, tr_park = 0; const long long tr_start = clock64();)
        for(int slot = 0; ok && slot < P.plan.num_slots; ++slot)
        {
            const WorkItem wi = work_item(slot);
            if(wi.kind == ITEM_NONE)
                continue;
            EpilogueArgs ea   = P.epi;
            int Mdim = P.M, Ndim = P.N;
            bool vec_ok = P.vec_ok != 0;
            if constexpr(MODE == MODE_GROUPED)
            {
                const GroupEntry* G = P.groups + wi.group;
                Mdim                = G->M;
                Ndim                = G->N;
                vec_ok              = G->vec_ok != 0;
                st.tm_e             = &G->tm_e;
                ea.e                = G->e;
                ea.d0               = G->d0;
                ea.d1               = G->d1;
                ea.lde              = G->lde;
                ea.ldd0             = G->ldd0;
                ea.ldd1             = G->ldd1;
            }
            if constexpr(MODE == MODE_GEMM)
            {
                if(P.plan.batch_tiles > 0)
                    st.batch = wi.batch; // batched E map: third coordinate
                if(wi.batch != 0)
                {
                    constexpr int EB = (KIND == KIND_I8) ? 1 : 2;
                    ea.e = static_cast<char*>(ea.e) + wi.batch * P.batch_stride_e * EB;
                    if(ea.d0)
                        ea.d0 = static_cast<const char*>(ea.d0) + wi.batch * P.batch_stride_d0 * EB;
                    if(ea.d1)
                        ea.d1 = static_cast<const char*>(ea.d1) + wi.batch * P.batch_stride_d1 * EB;
                }
            }
            // columns per epilogue warp (>= 32); a 32-column part (reduction of an 8-way K split) is handled by
            // the warps of column half 0 alone, those of half 1 get an empty range
            const int span          = wi.width >= 64 ? wi.width >> 1 : wi.width;
            const int64_t m =
                static_cast<int64_t>(wi.m_blk) * TILE_M + cta_rank * BM + quarter * 32 + lane;
            const bool row_ok       = m < Mdim;
            const int64_t n_begin   = static_cast<int64_t>(wi.n_start) + half * span;
            const int64_t n_end_raw = (wi.width >= 64 || half == 0) ? n_begin + span : n_begin;
            const int64_t n_end     = n_end_raw < Ndim ? n_end_raw : Ndim;

            // K-split tail: this warp's block of the tail tile in slice 0 of the scratch buffer
            // ([tail tile][slice][CTA of the pair][epilogue warp][32 rows x span columns])
            const uint32_t* parked = nullptr;
            uint32_t* fix_flags    = nullptr;
            if constexpr(PARK)
            {
                // (balanced K ranges: [parking slot = unit][CTA of the pair][epilogue warp][...], wi.slice = 0)
                const int per_tail        = P.plan.stream_k != 0 ? 1 : P.plan.ksplit;
                const uint32_t* tail_base = P.ks_partials + static_cast<int64_t>(wi.tail) * per_tail * TILE_M * BN;
                if(wi.kind == ITEM_KSLICE || wi.fix > 0)
                    parked = tail_base + (cta_rank * NUM_EPI_WARPS + half * 4 + quarter) * (32 * (BN / 2));
                if(P.plan.stream_k != 0) // the flag of this warp's block in parking slot wi.tail
                    fix_flags = P.ks_flags + (wi.tail * CG + cta_rank) * NUM_EPI_WARPS + half * 4 + quarter;
                if(KSPLIT && wi.kind == ITEM_REDUCE)
                {
                    // chunks of 32 columns: the tile has BN / 32, each parking warp holds BN / 64 of them
                    const int id0 = (wi.slice * wi.width + half * span) / 32; // first chunk this warp sums
                    const int H   = id0 / (BN / 64);                          // column half of the warp that parked it
                    parked        = tail_base + (cta_rank * NUM_EPI_WARPS + H * 4 + quarter) * (32 * (BN / 2)) +
                             (id0 - H * (BN / 64)) * (8 * 32 * 4);
                }
            }
            if constexpr(KSPLIT)
            {
                if(wi.kind == ITEM_REDUCE)
                {
                    // every slice of this tail tile is parked once all epilogue warps that ran one have arrived
                    uint32_t* counter     = P.ks_counters + wi.ctr;
                    const uint32_t target = static_cast<uint32_t>(P.plan.ksplit) * NUM_EPI_WARPS * CG;
                    ok                    = bounded_wait_counter(counter, target + P.ks_wait_extra, wc);
                    ok                    = __all_sync(0xffffffffu, ok);
                    if(!ok)
                        break;
                    epilogue_span<EPI, KIND, true>(0, ea, st, lane, m, row_ok, n_begin, n_end, vec_ok, parked,
                                                   P.plan.ksplit, static_cast<int64_t>(TILE_M) * BN);
                    // the last of the reducing warps leaves the counter at zero for the next launch
                    __syncwarp();
                    if(lane == 0 && atomicAdd(counter, 1u) + 1u == 2u * target)
                        atomicExch(counter, 0u);
                    continue;
                }
            }
            const int acc            = iter & 1;
            const uint32_t acc_phase = (iter >> 1) & 1;
            ++iter;
            uint32_t tmem_pre       = 0;
            bool has_pre            = false;
            const uint32_t* parked2 = nullptr; // the second parked part, where it cannot be prefetched
            if constexpr(BAL)
            {
                if(wi.fix >= 2)
                {
                    // A tile in three parts.  The part of the unit after next is the tile's last: parked early.  If
                    // this head is the last item of its unit, the other accumulator buffer is free (this warp has
                    // drained its part of it) and takes that part while the head's main loop still runs.
                    CKB_TR(const long long trq0 = clock64();)
                    ok = wait_parked(fix_flags + CG * NUM_EPI_WARPS, lane, wc, P.ks_wait_extra);
                    if(!ok)
                        break;
                    bool last_item = true;
                    for(int later = slot + 1; last_item && later < P.plan.num_slots; ++later)
                        last_item = work_item(later).kind == ITEM_NONE;
                    if(last_item)
                    {
                        has_pre  = true;
                        tmem_pre = tmem_base + (acc ^ 1) * BN + half * span + (static_cast<uint32_t>(quarter * 32) << 16);
                        prefetch_parked(tmem_pre, parked + static_cast<int64_t>(TILE_M) * BN, span, lane);
                    }
                    else
                        parked2 = parked + static_cast<int64_t>(TILE_M) * BN; // whole tiles follow: both buffers are in use
                    CKB_TR(tr_ctr += clock64() - trq0;)
                }
            }
            CKB_TR(const long long tr0 = clock64();)
            ok = bounded_wait(tmem_full_bar(acc), acc_phase, wc, WAIT_TMEM_FULL);
            CKB_TR(tr_wait += clock64() - tr0;)
            ok = __all_sync(0xffffffffu, ok);
            if(!ok)
                break;
            tc_fence_after_sync();
            const uint32_t tmem_addr =
                tmem_base + acc * BN + half * span + (static_cast<uint32_t>(quarter * 32) << 16);
            if constexpr(CK)
            {
                // the accumulator leaves after the cluster barrier below: the pipeline stages it goes to, in this
                // CTA and in its peers, are in use until every main loop of the cluster is over
            }
            else if(PARK && wi.kind == ITEM_KSLICE)
            {
                CKB_TR(const long long trp0 = clock64();)
                park_span(tmem_addr, const_cast<uint32_t*>(parked) + static_cast<int64_t>(wi.slice) * TILE_M * BN, span, lane,
                          fix_flags);
                CKB_TR(tr_park += clock64() - trp0;)
            }
            else if(BAL && wi.fix > 0)
            {
                // the rest of this tile's K range was parked by the next `fix` units as the first item of their runs:
                // the next unit's part is read back from L2 here, the part of the unit after next (if any) is
                // already in tensor memory; the sum goes back into the accumulator and the epilogue runs as usual
                if constexpr(BAL)
                {
                    CKB_TR(const long long trc0 = clock64();)
                    ok = wait_parked(fix_flags, lane, wc, P.ks_wait_extra);
                    CKB_TR(const long long trc1 = clock64(); tr_ctr += trc1 - trc0;)
                    if(ok)
                    {
                        fixup_span<KIND>(tmem_addr, parked, parked2, has_pre, tmem_pre, span, lane);
                        epilogue_span<EPI, KIND>(tmem_addr, ea, st, lane, m, row_ok, n_begin, n_end, vec_ok);
                    }
                    CKB_TR(tr_fix += clock64() - trc1;)
                }
            }
            else
                epilogue_span<EPI, KIND>(tmem_addr, ea, st, lane, m, row_ok, n_begin, n_end, vec_ok);
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

            if constexpr(CK)
                continue; // summed after the cluster barrier below
            if constexpr(PARK)
            {
                if(wi.kind == ITEM_KSLICE && P.plan.stream_k != 0)
                    continue; // published by its flag
                if(KSPLIT && wi.kind == ITEM_KSLICE)
                {
                    // publish the parked slice: stores -> fence -> one arrival per warp
                    __threadfence();
                    __syncwarp();
                    if(lane == 0)
                        atomicAdd(P.ks_counters + wi.ctr, 1u);
                    continue;
                }
            }

            // Ask L2 for the D values of this CTA's next item while its main loop runs.
            if constexpr(KIND != KIND_I8)
            {
                if(epi_num_d(EPI) > 0 && slot + 1 < P.plan.num_slots)
                {
                    const WorkItem nx = work_item(slot + 1);
                    if(nx.kind != ITEM_TILE)
                        continue;
                    EpilogueArgs en   = P.epi;
                    int Mn = P.M, Nn = P.N;
                    if constexpr(MODE == MODE_GROUPED)
                    {
                        en.d0   = P.groups[nx.group].d0;
                        en.d1   = P.groups[nx.group].d1;
                        en.ldd0 = P.groups[nx.group].ldd0;
                        en.ldd1 = P.groups[nx.group].ldd1;
                        Mn      = P.groups[nx.group].M;
                        Nn      = P.groups[nx.group].N;
                    }
                    if constexpr(MODE == MODE_GEMM)
                    {
                        if(nx.batch != 0)
                        {
                            if(en.d0)
                                en.d0 = static_cast<const char*>(en.d0) + nx.batch * P.batch_stride_d0 * 2;
                            if(en.d1)
                                en.d1 = static_cast<const char*>(en.d1) + nx.batch * P.batch_stride_d1 * 2;
                        }
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
        // the staged stores read this CTA's shared memory: they must be done before it goes away
        if(lane == 0)
            bulk_wait_group<0>();
        CKB_TR(if(P.trace && warp == 2 && lane == 0) {
            P.trace[blockIdx.x * 16 + 5] = tr_wait;
            P.trace[blockIdx.x * 16 + 6] = clock64() - tr_start;
            P.trace[blockIdx.x * 16 + 10] = tr_ctr;
            P.trace[blockIdx.x * 16 + 11] = tr_fix;
            P.trace[blockIdx.x * 16 + 12] = tr_park;
        })
    }

    bool ck_pull = false;
    if constexpr(CK)
    {
        // A CTA that gave up on a wait still takes part in every barrier; it hands over nothing, the sums that miss
        // its slice are wrong, and the status word tells the host.
        const bool push = cluster_push(BN, P.plan.ksplit);
        ck_pull         = !push;
        const bool epi  = warp >= 2 && warp < 2 + NUM_EPI_WARPS && misc[1] == 0;
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        constexpr int span = BN / 2;
        const uint32_t tmem_addr = tmem_base + half * span + (static_cast<uint32_t>(quarter * 32) << 16);
        if(push)
        {
            // First barrier: the main loop of every CTA of the cluster is over (the epilogue warps get here only
            // once their accumulator is complete), so the pipeline stages are free everywhere.
            cluster_sync_all();
            if(epi)
            {
                tc_fence_after_sync();
                stash_span(tmem_addr, base_addr, ck_rank, 31 - __clz(BN / P.plan.ksplit), quarter * 32 + lane, half * span, span);
            }
        }
        else if(epi)
            stash_span_local(tmem_addr, base_addr, quarter * 32 + lane, half * span, span);
        cluster_sync_all(); // every slice is where it will be read (release / acquire at cluster scope)
        if(warp >= 2 && warp < 2 + NUM_EPI_WARPS && misc[1] == 0)
        {
            const WorkItem wi = work_item(0);
            const int t       = static_cast<int>(threadIdx.x) - 64;
            if constexpr(BN >= 128)
                if(P.plan.ksplit == 8)
                    cluster_reduce_epilogue<EPI, KIND, BN, 8, true>(P, wi, base_addr, ck_rank, t);
            if(P.plan.ksplit == 4)
                cluster_reduce_epilogue<EPI, KIND, BN, 4, BN == 64>(P, wi, base_addr, ck_rank, t);
            else if(P.plan.ksplit == 2)
                cluster_reduce_epilogue<EPI, KIND, BN, 2, BN == 64>(P, wi, base_addr, ck_rank, t);
        }
    }

    // ---------------------------------------------------------------------- common exit
    tc_fence_before_sync();
    if(CG == 2 || ck_pull)
        cluster_sync_all(); // CG = 2: the leader's MMAs read the peer's shared memory until the very end;
                            // CK, pull: the other CTAs of the cluster read this one's accumulator tile
    else
        __syncthreads();    // (CK, push: nothing touches a peer's shared memory after the second barrier)
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
