// Work decomposition of the contraction kernel: which unit (CTA or CTA pair) runs which tile, column slice or
// K slice in which of its work slots, and the host-side choice of tile shape and tail plan.
//
// Plain C++ with no CUDA types: the same text is compiled into the kernel (decode_work runs in every role), into
// the host side of the library (plan_* run before a launch) and, by g++ alone, into a host-only test that
// enumerates every (unit, slot) of a plan and checks that each output tile, column range and k range is produced
// exactly once - the counterpart of the reference's tile-map tests (test/block_to_ctile_map/
// test_block_to_ctile_map.cpp:205-322) for BlockToCTileMap_M00_N0_M01Adapt (grid/block_to_ctile_map.hpp:112-173).
#pragma once
#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define CKB_HD __host__ __device__ __forceinline__
#else
#define CKB_HD inline
#endif

namespace ckb {

enum { MODE_GEMM = 0, MODE_GROUPED = 1, MODE_CONV = 2 };

constexpr int BM = 128; // rows of an output tile per CTA = TMEM lanes

// The work-enumeration part of the kernel parameters.
struct PlanParams
{
    int32_t total_tiles; // T: (128 * cg) x BN tiles over all groups / batches
    int32_t split_start; // first tile index whose tile is cut into column slices (= T if none)
    int32_t split;       // column slices per tail tile (1, 2 or 4)
    int32_t total_work;  // split_start + (T - split_start) * split
    int32_t tiles_m, tiles_n; // GEMM / CONV: tiles per problem (per batch)
    int32_t num_kb;      // k blocks per tile (GEMM / CONV)
    int32_t batch_tiles; // batched GEMM: tiles per batch (0 = not batched)
    // K-split tail (0 / 1 = off)
    int32_t ksplit;      // K slices per tail tile
    int32_t ks_kb;       // k blocks per slice (a multiple of the k blocks per stage)
    int32_t ks_full;     // tiles that run whole (a multiple of the number of units); tail tiles follow
    int32_t ks_rem;      // tail tiles
    int32_t num_slots;   // work slots per unit
    int32_t m_fastest;   // GEMM / CONV: consecutive tiles walk down a column of tiles instead of along a row
    int32_t group_count; // MODE_GROUPED
    int32_t cluster_k;   // 1: cluster K split - CTA r of cluster t runs K slice r of tile t (see decode_cluster_k)
    int32_t stream_k;    // 1: balanced K ranges - the k blocks of the last ks_rem tiles are dealt out evenly, ks_kb per
                         //    unit, across tile boundaries (ksplit stays 0; see decode_work)
};

// What one work item covers.
enum { ITEM_NONE = 0, ITEM_TILE = 1, ITEM_KSLICE = 2, ITEM_REDUCE = 3 };
struct WorkItem
{
    int kind;    // ITEM_*: TILE runs all roles; KSLICE is a TILE over part of K whose accumulator is parked;
                 // REDUCE is epilogue-only.  A TILE with fix > 0 covers k blocks [0, num_kb) of its tile only and
                 // adds the parked accumulators of the `fix` units that ran the rest before its epilogue
    int m_blk;   // row tile
    int n_start; // first output column
    int width;   // columns of this item (BN, or BN/split for a tail slice)
    int kb_begin, num_kb; // k blocks [kb_begin, kb_begin + num_kb)
    int group;   // MODE_GROUPED: index into the group table
    int batch;   // MODE_GEMM: batch index (0 unless batched)
    int tail;    // KSLICE / REDUCE: index of the tail tile.  Balanced K ranges: the parking slot - of this unit
                 // (KSLICE) or of the first unit whose accumulator is added (TILE with fix > 0)
    int slice;   // KSLICE: which K slice; REDUCE: which column part (of width BN / ksplit)
    int fix;     // TILE: parked accumulators to add (slots tail, tail + 1, ...), in k order
    int ctr;     // index of the counter the item's tile is announced on
    bool is_slice; // a column slice of a tail tile
};

// Finds g with groups[g].tile_start <= tile < groups[g+1].tile_start.
template <class Group>
CKB_HD int find_group(const Group* groups, int group_count, int tile)
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

// Position of tile `local` of a tiles_m x tiles_n problem.  Row order (n fastest) keeps the A row band of
// consecutive tiles in common and walks through all of B once per `units` tiles; column order (m fastest) does the
// opposite.  The operand that is walked through again and again is the one that has to stay in L2, so the host
// picks the order that makes it the smaller one (grouped GEMM: per group).
CKB_HD void tile_position(int local, int tiles_m, int tiles_n, int m_fastest, int* m_blk, int* n_blk)
{
    if(m_fastest)
    {
        *n_blk = local / tiles_m;
        *m_blk = local - *n_blk * tiles_m;
    }
    else
    {
        *m_blk = local / tiles_n;
        *n_blk = local - *m_blk * tiles_n;
    }
}

// Item of `unit` (CTA or CTA pair) in its work slot `slot`.
//   plain / column-slice plan: item w = unit + slot * num_units of the list [whole tiles][slices of the tail tiles]
//   K-split plan             : whole tile, K slice, whole tile, reduction of one column part of the tail tile,
//                              then the remaining whole tiles (parking and reduction both overlap a main loop)
//   balanced K ranges        : the k blocks of the last ks_rem tiles, laid end to end, are dealt out in runs of
//                              ks_kb per unit.  A unit's run starts inside a tile (that part is parked in the
//                              unit's own slot of the scratch: slot 0 of the schedule), may cover whole tiles and
//                              ends with the head [0, n) of a tile, whose other parts the following one or two
//                              units parked long before; the head's epilogue adds them.  The ks_full whole tiles
//                              before that region run between the parked part and the rest of the run.  Nothing
//                              that is waited for ever waits itself: parked parts are always a unit's first item.
// `groups` (MODE_GROUPED) is any array whose elements have tile_start, tiles_m, tiles_n, num_kb and m_fastest.
template <int MODE, int BN, bool KSPLIT, class Group>
CKB_HD WorkItem decode_work(const PlanParams& P, const Group* groups, int unit, int num_units, int slot)
{
    WorkItem wi;
    int tile, slice = 0;
    wi.kind     = ITEM_TILE;
    wi.width    = BN;
    wi.is_slice = false;
    wi.batch    = 0;
    wi.tail     = 0;
    wi.slice    = 0;
    wi.kb_begin = 0;
    wi.group    = 0;
    wi.fix      = 0;
    wi.ctr      = 0;
    int run_kb  = -1; // balanced K ranges: k blocks of this item (else taken from the tile)
    if(KSPLIT && P.stream_k != 0)
    {
        const int dp = P.ks_full / num_units; // whole tiles per unit ahead of the balanced region
        const int j  = slot == 0 ? 0 : slot - dp; // index of the item inside this unit's run (<= 0: a whole tile)
        if(slot != 0 && j <= 0)
            tile = unit + (slot - 1) * num_units;
        else
        {
            const int total = P.ks_rem * P.num_kb;
            const int lo    = unit * P.ks_kb;
            const int hi    = lo + P.ks_kb < total ? lo + P.ks_kb : total;
            const int st    = (lo < total ? lo / P.num_kb : 0) + j; // tile of the balanced region
            const int t_lo  = st * P.num_kb;
            if(lo >= total || t_lo >= hi)
            {
                wi.kind = ITEM_NONE;
                tile    = 0;
            }
            else
            {
                tile          = P.ks_full + st;
                wi.kb_begin   = j == 0 ? lo - t_lo : 0;
                const int end = hi - t_lo < P.num_kb ? hi - t_lo : P.num_kb;
                run_kb        = end - wi.kb_begin;
                wi.ctr        = st;
                if(wi.kb_begin > 0)
                {
                    wi.kind = ITEM_KSLICE;
                    wi.tail = unit;
                }
                else if(end < P.num_kb)
                {
                    wi.fix  = (t_lo + P.num_kb - hi + P.ks_kb - 1) / P.ks_kb;
                    wi.tail = unit + 1;
                }
            }
        }
    }
    else if(KSPLIT && P.ksplit > 1)
    {
        if(slot == 1)
        {
            wi.kind  = unit < P.ks_rem * P.ksplit ? ITEM_KSLICE : ITEM_NONE;
            wi.tail  = unit / P.ksplit;
            wi.slice = unit - wi.tail * P.ksplit;
            wi.ctr   = wi.tail;
            tile     = P.ks_full + wi.tail;
        }
        else if(slot == 3)
        {
            // the unit that ran slice i of a tail tile also sums column part i of it
            wi.kind  = unit < P.ks_rem * P.ksplit ? ITEM_REDUCE : ITEM_NONE;
            wi.tail  = unit / P.ksplit;
            wi.slice = unit - wi.tail * P.ksplit;
            wi.ctr   = wi.tail;
            tile     = P.ks_full + wi.tail;
            slice    = wi.slice;
            wi.width = BN / P.ksplit;
        }
        else
        {
            tile = unit + (slot == 0 ? 0 : slot == 2 ? 1 : slot - 2) * num_units;
            if(tile >= P.ks_full)
                wi.kind = ITEM_NONE;
        }
        if(wi.kind == ITEM_NONE)
            tile = 0;
    }
    else
    {
        const int w = unit + slot * num_units;
        if(w >= P.total_work)
        {
            wi.kind = ITEM_NONE;
            tile    = 0;
        }
        else if(w < P.split_start)
            tile = w;
        else
        {
            const int q = w - P.split_start;
            tile        = P.split_start + q / P.split;
            slice       = q % P.split;
            wi.width    = BN / P.split;
            wi.is_slice = P.split > 1;
        }
    }
    int n_blk;
    if(MODE == MODE_GROUPED)
    {
        wi.group       = find_group(groups, P.group_count, tile);
        const Group& G = groups[wi.group];
        tile_position(tile - G.tile_start, G.tiles_m, G.tiles_n, G.m_fastest, &wi.m_blk, &n_blk);
        wi.num_kb = G.num_kb;
    }
    else
    {
        if(MODE == MODE_GEMM && P.batch_tiles > 0) // batched GEMM: batch-major tile order
        {
            wi.batch = tile / P.batch_tiles;
            tile -= wi.batch * P.batch_tiles;
        }
        tile_position(tile, P.tiles_m, P.tiles_n, P.m_fastest, &wi.m_blk, &n_blk);
        wi.num_kb = P.num_kb;
    }
    if(run_kb >= 0)
        wi.num_kb = run_kb;
    else if(wi.kind == ITEM_KSLICE)
    {
        wi.kb_begin    = wi.slice * P.ks_kb;
        const int rest = P.num_kb - wi.kb_begin;
        wi.num_kb      = rest < P.ks_kb ? rest : P.ks_kb;
    }
    wi.n_start = n_blk * BN + slice * wi.width;
    return wi;
}

// Cluster K split (GEMMs with few tiles and a long K): a thread-block cluster of `ksplit` CTAs works on ONE
// 128 x BN tile, CTA r accumulating K slice r; the slices are summed through distributed shared memory (CTA r
// reads column part r of every CTA's accumulator, in slice order) and CTA r writes that part of E.  Clusters are
// independent of one another: nothing waits across clusters and no global scratch is involved.
// Item of the CTA with cluster rank `rank` in cluster `cluster` (= tile index).
template <int BN>
CKB_HD WorkItem decode_cluster_k(const PlanParams& P, int cluster, int rank)
{
    WorkItem wi;
    wi.kind     = ITEM_KSLICE;
    wi.width    = BN;
    wi.is_slice = false;
    wi.group    = 0;
    wi.batch    = 0;
    wi.fix      = 0;
    wi.ctr      = 0;
    wi.tail     = cluster;
    wi.slice    = rank;
    int tile    = cluster;
    if(P.batch_tiles > 0)
    {
        wi.batch = tile / P.batch_tiles;
        tile -= wi.batch * P.batch_tiles;
    }
    int n_blk;
    tile_position(tile, P.tiles_m, P.tiles_n, P.m_fastest, &wi.m_blk, &n_blk);
    wi.kb_begin    = rank * P.ks_kb;
    const int rest = P.num_kb - wi.kb_begin;
    wi.num_kb      = rest < P.ks_kb ? rest : P.ks_kb;
    wi.n_start     = n_blk * BN;
    return wi;
}

// ---------------------------------------------------------------------------------------------- host side

// A tile shape and tail plan the caller asks for instead of the library's own choice (0 = the library decides).
// This is what distinguishes the instances an instance factory hands out.
struct TileConfig
{
    int bn = 0;        // 64, 128 or 256 accumulator columns
    int cg = 0;        // 1 = one CTA per 128 x bn tile, 2 = a CTA pair per 256 x 256 tile
    int no_ksplit = 0; // 1 = never cut tiles along K
    int kbatch    = 0; // 2, 4 or 8: cut every tile's K loop into that many slices on a cluster (KBatch of the
                       // reference's split-K operation, device_gemm_splitk.hpp:23-42); 0 = the library decides
    int stream_k  = 0; // 1 = balanced K ranges wherever the kernel family has them, whatever the cost model says
};

inline int pick_bn(int64_t M, int64_t N, int sm_count, int min_bn, int forced)
{
    if((forced == 256 || forced == 128 || forced == 64) && forced >= min_bn)
        return forced;
    if(N <= 64 && min_bn <= 64)
        return 64;
    if(N <= 128)
        return 128;
    // Prefer the 256-wide tile (lowest shared-memory traffic per flop) unless it leaves most of the machine idle.
    const int64_t tiles256 = ((M + BM - 1) / BM) * ((N + 255) / 256);
    if(tiles256 < sm_count / 2)
        return 128;
    return 256;
}

// CTAs per tile: pairs (256 x 256 tiles, tcgen05 cta_group::2) once the problem fills the machine with
// 128 x 256 tiles at least once; single CTAs for small problems.
inline int pick_cg(int64_t tiles_128, int bn, int sm_count, int forced)
{
    if(forced == 1 || forced == 2)
        return bn == 256 ? forced : 1;
    return (bn == 256 && tiles_128 >= sm_count) ? 2 : 1;
}

// Column-slice tail: the last, partial wave of tiles is cut into column slices so that it occupies every unit.
struct WorkPlan
{
    int32_t split_start, split, total_work, grid;
};

// `units` = CTAs (one CTA per tile) or CTA pairs (cg = 2) that run concurrently; min_rows = narrowest B slice
// (rows) one CTA loads.
inline WorkPlan plan_work(int64_t total_tiles, int units, int bn, int cg, int min_rows)
{
    WorkPlan w;
    const int64_t G    = units;
    const int64_t full = (total_tiles / G) * G;
    const int64_t rem  = total_tiles - full;
    int split          = 1;
    if(rem > 0)
    {
        // slices of >= 64 columns whose per-CTA share is >= min_rows: K-major 256 -> 4, 128 -> 2, 64 -> 1
        const int min_width = min_rows * cg > 64 ? min_rows * cg : 64;
        const int max_split = bn / min_width;
        while(split * 2 <= max_split && rem * split * 2 <= G)
            split *= 2;
    }
    w.split       = split;
    w.split_start = static_cast<int32_t>(split > 1 ? full : total_tiles);
    w.total_work  = static_cast<int32_t>(split > 1 ? full + rem * split : total_tiles);
    w.grid        = static_cast<int32_t>((w.total_work < G ? w.total_work : G) * cg);
    return w;
}

// Cycle estimates per k block of the MMA role, fitted to timings of 1024 x 1024 x K and 512 x 512 x K with and
// without a K split: 590 for 256 accumulator columns, 340 for 128, 315 for 64 (the narrow ones are bound by the
// issue rate of the single MMA thread, not by the tensor pipe).
inline int kb_cycles(int width) { return width >= 256 ? 590 : width >= 128 ? 340 : 315; }

// Whole-problem K split.  A GEMM with few output tiles and a long K leaves most SMs idle whatever the tile shape;
// cutting every tile's K loop into 2, 4 or 8 slices (the machinery of the K-split tail, with no whole tiles before
// it) puts 2-8 times as many SMs to work on full-width MMAs.  Parking and summing the slices costs about 9100
// cycles (5.5 us), most of it the exposed latency of the reduction's loads.
struct WholeSplit
{
    int bn = 0, cg = 0, ksplit = 0;
    bool cluster = false; // slices summed through distributed shared memory instead of the L2 scratch
};

// Cost model of the K-split plans (SM cycles), fitted to timings on a B200 of 256 x 256 x 16384, 512 x 512 x 8192,
// 768 x 768 x 4096, 1024 x 1024 x 8192, 128 x 4096 x 8192 and 128 x 8192 x 4096 with every slice count pinned:
//   through the L2 scratch (park, counter wait, reload): about 11000 cycles on top of the slice's main loop when
//   most of the machine takes part;
//   inside a cluster: the slice's main loop at 340 cycles per k block for 128-wide tiles and 500 for 256-wide ones
//   (one CTA per tile pulls a 48 KiB stage per k block through L2), plus accumulator -> shared memory, cluster
//   barrier and the hand-over through distributed shared memory: about 1800 cycles for a 64-wide tile, 4500 for a 128-wide
//   one, 10000 for a 256-wide one (the reads are latency bound and grow with the tile).
constexpr int kParkedReduceCycles = 11000;
inline int cluster_kb_cycles(int bn) { return bn >= 256 ? 500 : bn >= 128 ? 340 : 330; }
inline int cluster_reduce_cycles(int bn) { return bn >= 256 ? 10000 : bn >= 128 ? 4500 : 1800; }

// k blocks per slice of a `ks`-way cut (even, so that slices start on a stage boundary); 0 when a slice would be
// empty or shorter than two k blocks.
inline int slice_kb(int num_kb, int ks)
{
    int kb = (num_kb + ks - 1) / ks;
    kb     = (kb + 1) & ~1;
    return (kb >= 2 && static_cast<int64_t>(ks - 1) * kb < num_kb) ? kb : 0;
}

// `parked` / `cluster`: which of the two ways of summing the slices the caller may use (the parked one needs the
// scratch buffer and 16-bit operands with a D-less epilogue; the cluster one works for every kernel).
inline WholeSplit consider_whole_split(int64_t M, int64_t N, int num_kb, int sm_count, int b_min, int64_t est_current,
                                       bool parked, bool cluster, const int* cluster_cap)
{
    WholeSplit best;
    int64_t best_est     = est_current - est_current / 8; // has to beat the plan without it by an eighth
    const int cand[4][2] = {{256, 2}, {256, 1}, {128, 1}, {64, 1}};
    for(const auto& c : cand)
    {
        const int bn = c[0], cg = c[1];
        if(bn / cg < b_min || (cg == 2 && M <= BM)) // a pair tile with one half of its rows empty pays for nothing
            continue;
        if(bn == 64 && !cluster) // 64-wide tiles only as cluster tiles (their reduction is the cheapest)
            continue;
        const int64_t G     = sm_count / cg;
        const int64_t tiles = ((M + BM * cg - 1) / (BM * cg)) * ((N + bn - 1) / bn);
        for(int ks = 8; ks >= 2; ks /= 2)
        {
            if(tiles * ks > G)
                continue;
            const int ks_kb = slice_kb(num_kb, ks);
            if(ks_kb < 4)
                continue;
            for(int way = 0; way < 2; ++way)
            {
                const bool by_cluster = way == 1;
                // parked: column parts of whole 32-column chunks; cluster: one CTA per tile, parts of >= 16 columns,
                // every cluster resident at once (clusters live inside one GPC each, so fewer fit than SMs / ks)
                if(by_cluster ? !(cluster && cg == 1 && bn / ks >= 16 && tiles <= cluster_cap[ks == 2 ? 0 : ks == 4 ? 1 : 2])
                              : !(parked && bn >= 128 && bn / ks >= 32))
                    continue;
                const int64_t est = by_cluster ? static_cast<int64_t>(ks_kb) * cluster_kb_cycles(bn) + cluster_reduce_cycles(bn)
                                               : static_cast<int64_t>(ks_kb) * kb_cycles(bn) + kParkedReduceCycles +
                                                     (ks > 4 ? 1500 : 0);
                if(est < best_est)
                {
                    best_est     = est;
                    best.bn      = bn;
                    best.cg      = cg;
                    best.ksplit  = ks;
                    best.cluster = by_cluster;
                }
            }
        }
    }
    return best;
}

struct GemmPlanInput
{
    int64_t M = 0, N = 0;
    int num_kb    = 0;
    int64_t batch = 0;       // 0 = plain GEMM, else the batch count (batch-major tile order)
    int sm_count  = 0;
    int b_min     = 32;      // narrowest B slice (rows) one CTA loads
    bool ks_pays    = false; // 16-bit operands and an epilogue without D tensors (see the K-split notes)
    bool ks_allowed = false; // scratch may be used (not disabled, not capturing)
    bool bal_ok     = false; // the kernel family has instances with the balanced K ranges for 256-wide tiles (every
                             // plain GEMM; families with ks_pays carry them in all their instances)
    bool cluster_ok = false; // the kernel family has cluster K-split instances (plain GEMM)
    int cluster_cap[3] = {0, 0, 0}; // clusters of 2 / 4 / 8 CTAs the device holds at once
    TileConfig force;
};

struct GemmPlan
{
    int bn = 0, cg = 0;
    int grid = 0;         // CTAs to launch
    int b_split_rows = 0; // rows of the B box of a tail slice, per CTA
    int cluster = 1;      // CTAs per cluster besides the pairing: the slice count of a cluster K split, else 1
    PlanParams pp = {};
    size_t partial_bytes = 0; // parked accumulators of the K split (0 = no scratch needed)
};

constexpr int kMaxTailTiles = 1024; // tail-tile counters at the front of the scratch buffer

// Balanced K ranges (see decode_work): the k blocks of the tiles are laid end to end and dealt out evenly.  The
// library takes the plan by itself only for one partly filled wave of 256-wide tiles, by this cost model in SM
// cycles, fitted to timings of 1280 x 2048 x K (K = 4096 ... 8192; 80 tiles of 128 x 256) on a B200:
//   one CTA per 128 x 256 tile, tiles <= SMs        572 per k block +  5300
//   CTA pairs on 256 x 256 tiles, tiles <= pairs     516 per k block + 10500
//   balanced, one CTA per tile, every SM loading     644 per k block + 19000
//   balanced, CTA pairs                              509 per k block + 24100
// The fixed cost of the balanced plans is the end of the launch: a unit whose whole run is the middle of a tile
// parks its accumulator when everyone else is done (stores, fence, flag: 6000 cycles), and the unit with the head of
// that tile then reads it back (3600) before its epilogue.  The units' K ranges are out of step, so an operand panel
// is fetched once per tile that uses it instead of once per wave: beyond what stays in L2 the plan loses
// (512 x 8192 x 16384 with one CTA per tile: four times the DRAM traffic, 184 us against 104).
constexpr int kBalancedGainPct = 93; // taken when its estimate is at most this share of the plain plan's
inline int64_t est_plain_wave(int num_kb, int cg)
{
    return cg == 2 ? static_cast<int64_t>(num_kb) * 516 + 10500 : static_cast<int64_t>(num_kb) * 572 + 5300;
}
inline int64_t est_balanced(int64_t run_kb, int cg) { return cg == 2 ? run_kb * 509 + 24100 : run_kb * 644 + 19000; }
inline int64_t balanced_operand_limit(int cg) { return cg == 2 ? (128ll << 20) : (64ll << 20); }
inline int64_t balanced_run_kb(int64_t tiles, int num_kb, int64_t units)
{
    const int64_t w = (tiles * num_kb + units - 1) / units;
    return (w + 1) & ~int64_t(1);
}

// CTAs per tile (1 or 2) of the balanced plan the library would take for a problem whose plain plan is one partly
// filled wave of 256-wide tiles with `cg_now` CTAs per tile; 0 = keep the plain plan.
inline int consider_balanced(int64_t M, int64_t N, int num_kb, int sm_count, int b_min, int cg_now, int cg_forced)
{
    const int64_t est_now = est_plain_wave(num_kb, cg_now);
    int best              = 0;
    int64_t best_est      = est_now * kBalancedGainPct / 100;
    for(int cg = 2; cg >= 1; --cg)
    {
        if((cg_forced != 0 && cg_forced != cg) || 256 / cg < b_min || (cg == 2 && M <= BM))
            continue;
        const int64_t G = sm_count / cg, T = ((M + BM * cg - 1) / (BM * cg)) * ((N + 255) / 256);
        if(T >= G || T * 2 <= G || (M + N) * static_cast<int64_t>(num_kb) * 128 > balanced_operand_limit(cg))
            continue;
        const int64_t est = est_balanced(balanced_run_kb(T, num_kb, G), cg);
        if(est <= best_est)
        {
            best_est = est;
            best     = cg;
        }
    }
    return best;
}

// Tile shape, CTA grouping and tail plan of one (batched) GEMM.  Returns false when the tile count does not fit.
inline bool plan_gemm(const GemmPlanInput& in, GemmPlan* out)
{
    GemmPlan g;
    const int64_t nb    = in.batch > 0 ? in.batch : 1;
    const bool may_ks   = in.ks_pays && in.ks_allowed && !in.force.no_ksplit;
    int bn              = pick_bn(in.M, in.N, in.sm_count, in.b_min, in.force.bn);
    int cg              = pick_cg(((in.M + BM - 1) / BM) * ((in.N + bn - 1) / bn) * nb, bn, in.sm_count, in.force.cg);
    const int num_kb    = in.num_kb;
    {
        // One partly filled wave of 128 x 256 tiles over a problem that is narrow in M or N (at most 512): few tiles
        // share each panel of the large operand, so it streams from DRAM nearly once per tile; a CTA pair loads half
        // as much of B per CTA and was 3-12 % faster there (512 x 8192 x 4096: 26.9 against 29.9 us, 512 x 8192 x
        // 16384: 88.6 against 101; square-ish problems of the same tile count lose 4 % with pairs).
        const int64_t tm = (in.M + BM - 1) / BM, t128 = tm * ((in.N + 255) / 256) * nb;
        if(in.force.cg == 0 && bn == 256 && cg == 1 && t128 < in.sm_count && t128 * 2 > in.sm_count && tm % 2 == 0 &&
           (in.M <= 512 || in.N <= 512) && in.b_min <= 128)
            cg = 2;
    }
    int whole_ksplit    = 0;
    bool by_cluster     = false;
    const bool may_cluster = in.cluster_ok && !in.force.no_ksplit && in.batch == 0;
    if((in.force.kbatch == 2 || in.force.kbatch == 4 || in.force.kbatch == 8) && may_cluster && in.force.cg != 2)
    {
        // the caller names the slice count: one CTA per tile, a cluster of kbatch CTAs per tile
        // (several waves of clusters are fine - clusters do not wait for one another - but one must fit)
        const int cap = in.cluster_cap[in.force.kbatch == 2 ? 0 : in.force.kbatch == 4 ? 1 : 2];
        if(slice_kb(num_kb, in.force.kbatch) >= 2 && bn / in.force.kbatch >= 16 && cap >= 1)
        {
            cg           = 1;
            whole_ksplit = in.force.kbatch;
            by_cluster   = true;
        }
    }
    else if((may_ks || may_cluster) && in.batch == 0 && in.force.bn == 0 && in.force.cg == 0)
    {
        // only where the plan without it runs a single, partly filled wave
        const int64_t t0 = ((in.M + BM * cg - 1) / (BM * cg)) * ((in.N + bn - 1) / bn);
        const int64_t G0 = in.sm_count / cg;
        if(t0 * 2 <= G0)
        {
            const WorkPlan w0   = plan_work(t0, static_cast<int>(G0), bn, cg, in.b_min);
            const WholeSplit ws = consider_whole_split(in.M, in.N, num_kb, in.sm_count, in.b_min,
                                                       static_cast<int64_t>(num_kb) * kb_cycles(bn / w0.split), may_ks,
                                                       may_cluster, in.cluster_cap);
            if(ws.ksplit >= 2)
            {
                bn           = ws.bn;
                cg           = ws.cg;
                whole_ksplit = ws.ksplit;
                by_cluster   = ws.cluster;
            }
        }
    }
    const bool may_bal = (in.ks_pays || in.bal_ok) && in.ks_allowed && !in.force.no_ksplit;
    bool balanced      = false;
    if(may_bal && whole_ksplit < 2 && in.batch == 0 && in.force.bn == 0 && bn == 256 && num_kb >= 8)
    {
        const int64_t t_now = ((in.M + BM * cg - 1) / (BM * cg)) * ((in.N + bn - 1) / bn);
        if(t_now < in.sm_count / cg)
        {
            const int cg_bal = consider_balanced(in.M, in.N, num_kb, in.sm_count, in.b_min, cg, in.force.cg);
            if(cg_bal != 0)
            {
                cg       = cg_bal;
                balanced = true;
            }
        }
    }
    if(by_cluster)
    {
        const int64_t tn = (in.N + bn - 1) / bn, tm = (in.M + BM - 1) / BM;
        if(tm * tn * whole_ksplit > 0x3FFFFFFFll)
            return false;
        PlanParams& p = g.pp;
        p.total_tiles = static_cast<int32_t>(tm * tn);
        p.split_start = p.total_tiles;
        p.split       = 1;
        p.total_work  = p.total_tiles;
        p.tiles_m     = static_cast<int32_t>(tm);
        p.tiles_n     = static_cast<int32_t>(tn);
        p.num_kb      = num_kb;
        p.ksplit      = whole_ksplit;
        p.ks_kb       = slice_kb(num_kb, whole_ksplit);
        p.num_slots   = 1;
        p.cluster_k   = 1;
        g.bn           = bn;
        g.cg           = 1;
        g.cluster      = whole_ksplit;
        g.grid         = static_cast<int>(tm * tn * whole_ksplit);
        g.b_split_rows = bn;
        *out           = g;
        return true;
    }
    const int64_t tiles_n   = (in.N + bn - 1) / bn;
    const int64_t tiles_m   = (in.M + BM * cg - 1) / (BM * cg);
    const int64_t all_tiles = tiles_m * tiles_n * nb;
    if(all_tiles > 0x3FFFFFFFll)
        return false;
    const int64_t G   = in.sm_count / cg;
    WorkPlan plan     = plan_work(all_tiles, static_cast<int>(G), bn, cg, in.b_min);
    PlanParams& p     = g.pp;
    const int64_t ful = (all_tiles / G) * G, rem = all_tiles - ful;
    // K-split tail: with whole waves before it and a tail of at most half the units, cut the tail tiles along K.
    // A 256-wide tail tile is cut four ways along K where a quarter of the units suffice; with more tail tiles only
    // two K halves fit, and those beat two 128-column slices only for a long K (parking and reduction cost the same
    // whatever K is, a column slice costs per k block): measured break-even near 78 k blocks.  The four-way cut
    // itself needs a K loop long enough to pay for parking and reduction: taken from 40 k blocks on (48 for the
    // two halves of a 128-wide tile, by the same cost model).
    if(may_ks && rem > 0 && (ful > 0 || whole_ksplit >= 2) && rem * 2 <= G && rem <= kMaxTailTiles)
    {
        int ksplit = whole_ksplit >= 2 ? whole_ksplit
                     : (G / rem >= 4 && bn >= 256) ? (num_kb >= 40 ? 4 : 0)
                     : ((bn == 128 && num_kb >= 48) || (bn >= 256 && num_kb >= 80)) ? 2 : 0;
        int ks_kb  = 0;
        for(; ksplit >= 2; ksplit /= 2)
        {
            ks_kb = (num_kb + ksplit - 1) / ksplit;
            ks_kb = (ks_kb + 1) & ~1; // slices start on a stage boundary (at most two k blocks per stage)
            if(ks_kb >= 4 && static_cast<int64_t>(ksplit - 1) * ks_kb < num_kb)
                break;
        }
        if(ksplit >= 2)
        {
            g.partial_bytes  = static_cast<size_t>(rem) * ksplit * (BM * cg) * bn * sizeof(uint32_t);
            p.ksplit         = ksplit;
            p.ks_kb          = ks_kb;
            p.ks_full        = static_cast<int32_t>(ful);
            p.ks_rem         = static_cast<int32_t>(rem);
            p.num_slots      = static_cast<int32_t>(ful / G + 2 < 4 ? 4 : ful / G + 2);
            plan.split       = 1;
            plan.split_start = static_cast<int32_t>(all_tiles);
            plan.total_work  = static_cast<int32_t>(all_tiles);
            plan.grid        = static_cast<int32_t>(G * cg);
        }
    }
    // Balanced K ranges: by the library's own choice (above) or because the caller asks for them - then also with
    // whole waves before the region, which takes in the last full wave so that every run covers at least a tile.
    if(may_bal && p.ksplit < 2 && whole_ksplit < 2 && in.batch == 0 && (in.ks_pays ? bn >= 128 : bn == 256) && rem > 0 &&
       all_tiles * 2 > G && num_kb >= 8 && (balanced || in.force.stream_k != 0))
    {
        const int64_t D = all_tiles < 2 * G ? 0 : ful - G, R = all_tiles - D;
        const int64_t W = balanced_run_kb(R, num_kb, G);
        if(R <= kMaxTailTiles && W * 2 >= num_kb && R * num_kb < (1ll << 30)) // (unit, k block) positions are 32-bit
        {
            g.partial_bytes  = static_cast<size_t>(G) * (BM * cg) * bn * sizeof(uint32_t); // one parking slot per unit
            p.stream_k       = 1;
            p.ks_kb          = static_cast<int32_t>(W);
            p.ks_full        = static_cast<int32_t>(D);
            p.ks_rem         = static_cast<int32_t>(R);
            p.num_slots      = static_cast<int32_t>(D / G + 1 + (W - 1 + num_kb - 1) / num_kb);
            plan.split       = 1;
            plan.split_start = static_cast<int32_t>(all_tiles);
            plan.total_work  = static_cast<int32_t>(all_tiles);
            plan.grid        = static_cast<int32_t>(G * cg);
        }
    }
    if(p.ksplit < 2 && p.stream_k == 0)
        p.num_slots = static_cast<int32_t>((plan.total_work + G - 1) / G);
    p.total_tiles  = static_cast<int32_t>(all_tiles);
    p.split_start  = plan.split_start;
    p.split        = plan.split;
    p.total_work   = plan.total_work;
    p.tiles_m      = static_cast<int32_t>(tiles_m);
    p.tiles_n      = static_cast<int32_t>(tiles_n);
    p.num_kb       = num_kb;
    p.batch_tiles  = in.batch > 0 ? static_cast<int32_t>(tiles_m * tiles_n) : 0;
    g.bn           = bn;
    g.cg           = cg;
    g.grid         = plan.grid;
    g.b_split_rows = bn / plan.split / cg;
    *out           = g;
    return true;
}

// One group of a grouped GEMM as the planner sees it; the kernel's table entry carries the same fields.
struct GroupTiles
{
    int32_t tile_start, tiles_m, tiles_n, num_kb, m_fastest;
};

struct GroupedPlan
{
    int bn = 0, cg = 0, grid = 0, b_split_rows = 0;
    PlanParams pp = {};
};

// Tile shape and work list of a grouped GEMM: `shapes` holds (M, N, num_kb) per group, `tiles` receives the
// per-group tile counts, prefix sums and tile order.  Within a group the tile order keeps the smaller operand in
// L2: with fewer row tiles than column tiles (M_g < N_g) consecutive tiles walk down a column of tiles, so that A_g
// is the operand every wave reads again while B_g streams through once, and the other way round otherwise.
inline bool plan_grouped(const int64_t (*shapes)[3], int group_count, int sm_count, int b_min, const TileConfig& force,
                         GroupTiles* tiles, GroupedPlan* out)
{
    int64_t max_n = 0, sum_m = 0;
    for(int i = 0; i < group_count; ++i)
    {
        max_n = max_n > shapes[i][1] ? max_n : shapes[i][1];
        sum_m += shapes[i][0];
    }
    const int bn      = pick_bn(sum_m, max_n, sm_count, b_min, force.bn);
    int64_t tiles_128 = 0;
    for(int i = 0; i < group_count; ++i)
        tiles_128 += ((shapes[i][0] + BM - 1) / BM) * ((shapes[i][1] + bn - 1) / bn);
    const int cg      = pick_cg(tiles_128, bn, sm_count, force.cg);
    int64_t all_tiles = 0;
    for(int i = 0; i < group_count; ++i)
    {
        const int64_t tm = (shapes[i][0] + BM * cg - 1) / (BM * cg), tn = (shapes[i][1] + bn - 1) / bn;
        if(all_tiles + tm * tn > 0x3FFFFFFFll)
            return false;
        tiles[i].tile_start = static_cast<int32_t>(all_tiles);
        tiles[i].tiles_m    = static_cast<int32_t>(tm);
        tiles[i].tiles_n    = static_cast<int32_t>(tn);
        tiles[i].num_kb     = static_cast<int32_t>(shapes[i][2]);
        tiles[i].m_fastest  = tm < tn ? 1 : 0;
        all_tiles += tm * tn;
    }
    const WorkPlan plan = plan_work(all_tiles, sm_count / cg, bn, cg, b_min);
    GroupedPlan g;
    g.bn             = bn;
    g.cg             = cg;
    g.grid           = plan.grid;
    g.b_split_rows   = bn / plan.split / cg;
    g.pp.total_tiles = static_cast<int32_t>(all_tiles);
    g.pp.split_start = plan.split_start;
    g.pp.split       = plan.split;
    g.pp.total_work  = plan.total_work;
    g.pp.num_slots   = (plan.total_work + plan.grid / cg - 1) / (plan.grid / cg);
    g.pp.group_count = group_count;
    *out             = g;
    return true;
}

} // namespace ckb
