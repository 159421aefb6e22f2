// Host-only test of the kernel's work decomposition (composable_kernel_b200/csrc/ckb_plan.h): for a sweep of
// problem sizes, SM counts, tile configurations, batch counts and group tables, every (unit, slot) of the plan is
// decoded exactly as the kernel's roles decode it, and the test asserts that
//   - every 32-column chunk of every output tile is written exactly once (by a whole tile, a column slice or a
//     reduction part), with valid tile indices;
//   - under a K split every tail tile's k blocks are covered exactly once by its slices, each slice starts on a
//     stage boundary, the unit that runs slice i reduces column part i, every unit of the launch is needed at the
//     same time only up to the number of units, and the parked partials fit the fixed scratch size;
//   - under balanced K ranges every unit's run is ks_kb k blocks of the region laid end to end, a part that is parked
//     is the first item of its unit and lies in the unit's own parking slot, every tile that is not run whole has
//     exactly one head [0, n) whose `fix` count and first slot name exactly the units that parked the rest, in k
//     order, and all k blocks of the tile are covered once;
//   - the grouped table's prefix sums, per-group tile order and binary search agree.
// It is the counterpart of the reference's tile-map tests (test/block_to_ctile_map/test_block_to_ctile_map.cpp:205-322).
// Build: g++ -std=c++17 -I composable_kernel_b200/csrc tests/cpp/work_plan_test.cpp
#include <array>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <random>
#include <tuple>
#include <vector>

#include "ckb_plan.h"

using namespace ckb;

static long g_checks = 0, g_plans = 0, g_ksplit_plans = 0, g_slice_plans = 0, g_balanced_plans = 0;

#define REQUIRE(cond, ...)                                \
    do                                                    \
    {                                                     \
        ++g_checks;                                       \
        if(!(cond))                                       \
        {                                                 \
            std::printf("FAILED %s:%d: %s\n  ", __FILE__, __LINE__, #cond); \
            std::printf(__VA_ARGS__);                     \
            std::printf("\n");                            \
            std::exit(1);                                 \
        }                                                 \
    } while(0)

struct Coverage
{
    // key: (group or batch, m_blk, first column of a 32-column chunk) -> times written
    std::map<std::tuple<int, int, int>, int> out;
    // key: tail tile -> per k block, times accumulated
    std::map<int, std::vector<int>> tail_k;
    std::map<int, std::vector<int>> tail_slices; // tail -> slice ids seen
    // balanced K ranges: tile of the region -> (first parking slot, count) named by its head; -> units that parked, with
    // the first k block of each part
    std::map<int, std::pair<int, int>> head_fix;
    std::map<int, std::vector<std::pair<int, int>>> parked_by;
    std::map<int, int> unit_kb; // unit -> k blocks of the region it runs
};

template <int MODE, int BN, bool KSPLIT>
static void walk(const PlanParams& P, const GroupTiles* groups, int cg, int grid, Coverage& cov)
{
    const int num_units = grid / cg;
    for(int unit = 0; unit < num_units; ++unit)
        for(int slot = 0; slot < P.num_slots; ++slot)
        {
            const WorkItem wi = decode_work<MODE, BN, KSPLIT>(P, groups, unit, num_units, slot);
            if(wi.kind == ITEM_NONE)
                continue;
            const int scope = MODE == MODE_GROUPED ? wi.group : wi.batch;
            const int tiles_m = MODE == MODE_GROUPED ? groups[wi.group].tiles_m : P.tiles_m;
            const int tiles_n = MODE == MODE_GROUPED ? groups[wi.group].tiles_n : P.tiles_n;
            REQUIRE(wi.m_blk >= 0 && wi.m_blk < tiles_m, "m_blk %d of %d", wi.m_blk, tiles_m);
            REQUIRE(wi.n_start >= 0 && wi.n_start + wi.width <= tiles_n * BN, "columns [%d, %d) of %d", wi.n_start,
                    wi.n_start + wi.width, tiles_n * BN);
            REQUIRE(wi.width >= 32 && wi.width % 32 == 0 && wi.n_start % 32 == 0, "width %d start %d", wi.width, wi.n_start);
            if(wi.kind == ITEM_TILE || wi.kind == ITEM_REDUCE)
                for(int c = wi.n_start; c < wi.n_start + wi.width; c += 32)
                    ++cov.out[{scope, wi.m_blk, c}];
            if(KSPLIT && P.stream_k != 0 && (wi.kind == ITEM_KSLICE || wi.fix > 0 || (slot == 0 || slot > P.ks_full / num_units)))
            {
                // an item of the balanced region
                REQUIRE(wi.kind == ITEM_TILE || wi.kind == ITEM_KSLICE, "kind %d in a balanced run", wi.kind);
                REQUIRE(wi.ctr >= 0 && wi.ctr < P.ks_rem && wi.width == BN && !wi.is_slice, "tile %d of the region", wi.ctr);
                REQUIRE(wi.num_kb >= 1 && wi.kb_begin >= 0 && wi.kb_begin + wi.num_kb <= P.num_kb, "k range [%d, +%d)", wi.kb_begin, wi.num_kb);
                auto& v = cov.tail_k[wi.ctr];
                v.resize(P.num_kb, 0);
                for(int k = wi.kb_begin; k < wi.kb_begin + wi.num_kb; ++k)
                    ++v[k];
                cov.unit_kb[unit] += wi.num_kb;
                if(wi.kind == ITEM_KSLICE)
                {
                    REQUIRE(slot == 0 && wi.tail == unit && wi.kb_begin > 0 && wi.slice == 0 && wi.fix == 0, "a parked part is a unit's first item, in its own slot");
                    cov.parked_by[wi.ctr].push_back({unit, wi.kb_begin});
                }
                else
                {
                    REQUIRE(wi.kb_begin == 0, "a head starts at k block 0");
                    if(wi.num_kb < P.num_kb)
                    {
                        REQUIRE(wi.fix >= 1 && wi.tail == unit + 1, "head of %d k blocks names %d parts from slot %d", wi.num_kb, wi.fix, wi.tail);
                        REQUIRE(cov.head_fix.count(wi.ctr) == 0, "two heads for tile %d", wi.ctr);
                        cov.head_fix[wi.ctr] = {wi.tail, wi.fix};
                    }
                    else
                        REQUIRE(wi.fix == 0, "a whole tile adds nothing");
                }
                continue;
            }
            if(wi.kind == ITEM_TILE)
            {
                const int want_kb = MODE == MODE_GROUPED ? groups[wi.group].num_kb : P.num_kb;
                REQUIRE(wi.fix == 0, "fix-up outside a balanced plan");
                REQUIRE(wi.kb_begin == 0 && wi.num_kb == want_kb, "whole tile covers k blocks [%d, +%d) of %d", wi.kb_begin,
                        wi.num_kb, want_kb);
                if(wi.is_slice)
                    REQUIRE(wi.width == BN / P.split && wi.width >= 64, "slice width %d", wi.width);
            }
            if(wi.kind == ITEM_KSLICE)
            {
                REQUIRE(KSPLIT && slot == 1, "K slice outside slot 1");
                REQUIRE(wi.tail >= 0 && wi.tail < P.ks_rem && wi.slice < P.ksplit, "tail %d slice %d", wi.tail, wi.slice);
                REQUIRE(wi.width == BN && wi.n_start % BN == 0, "a K slice covers the whole tile width");
                REQUIRE(wi.kb_begin % 2 == 0 && wi.num_kb >= 1, "slice [%d, +%d)", wi.kb_begin, wi.num_kb);
                REQUIRE(unit == wi.tail * P.ksplit + wi.slice, "slice owner");
                auto& v = cov.tail_k[wi.tail];
                v.resize(P.num_kb, 0);
                for(int k = wi.kb_begin; k < wi.kb_begin + wi.num_kb; ++k)
                {
                    REQUIRE(k < P.num_kb, "k block %d of %d", k, P.num_kb);
                    ++v[k];
                }
                cov.tail_slices[wi.tail].push_back(wi.slice);
            }
            if(wi.kind == ITEM_REDUCE)
            {
                REQUIRE(KSPLIT && slot == 3, "reduction outside slot 3");
                REQUIRE(unit == wi.tail * P.ksplit + wi.slice, "the unit that ran slice i reduces part i");
                REQUIRE(wi.width == BN / P.ksplit && wi.width >= 32, "reduction part width %d", wi.width);
            }
        }
}

template <int MODE, bool KSPLIT>
static void walk_bn(int bn, const PlanParams& P, const GroupTiles* groups, int cg, int grid, Coverage& cov)
{
    if(bn == 256)
        walk<MODE, 256, KSPLIT>(P, groups, cg, grid, cov);
    else if(bn == 128)
        walk<MODE, 128, KSPLIT>(P, groups, cg, grid, cov);
    else if(bn == 64)
        walk<MODE, 64, KSPLIT>(P, groups, cg, grid, cov);
    else
        REQUIRE(false, "tile width %d", bn);
}

// Cluster K split: cluster c works on tile c, CTA r of the cluster on K slice r; the column parts of the reduction
// (BN / ksplit columns each, one per CTA) are whole 16-column segments.
template <int BN>
static void walk_clusters(const GemmPlanInput& in, const GemmPlan& gp)
{
    const PlanParams& P = gp.pp;
    const int ks = P.ksplit;
    REQUIRE(gp.cg == 1 && gp.cluster == ks && (ks == 2 || ks == 4 || ks == 8), "cluster of %d", gp.cluster);
    REQUIRE(gp.grid == P.total_tiles * ks && P.num_slots == 1 && gp.partial_bytes == 0, "cluster grid");
    REQUIRE(BN / ks >= 16 && (BN / ks) % 16 == 0, "column part of %d columns", BN / ks);
    REQUIRE(P.ks_kb % 2 == 0 && P.ks_kb * (ks - 1) < P.num_kb && P.ks_kb * ks >= P.num_kb, "slice length %d", P.ks_kb);
    if(in.force.kbatch == 0)
        REQUIRE(P.total_tiles <= in.cluster_cap[ks == 2 ? 0 : ks == 4 ? 1 : 2], "%d clusters of %d beyond the capacity",
                P.total_tiles, ks);
    std::map<std::pair<int, int>, int> tiles_seen;
    for(int c = 0; c < P.total_tiles; ++c)
    {
        std::vector<int> k_seen(P.num_kb, 0);
        for(int r = 0; r < ks; ++r)
        {
            const WorkItem wi = decode_cluster_k<BN>(P, c, r);
            REQUIRE(wi.kind == ITEM_KSLICE && wi.slice == r && wi.width == BN, "item of cluster %d rank %d", c, r);
            REQUIRE(wi.m_blk >= 0 && wi.m_blk < P.tiles_m && wi.n_start % BN == 0 && wi.n_start / BN < P.tiles_n, "tile position");
            REQUIRE(wi.num_kb >= 1 && wi.kb_begin % 2 == 0, "slice [%d, +%d)", wi.kb_begin, wi.num_kb);
            for(int k = wi.kb_begin; k < wi.kb_begin + wi.num_kb; ++k)
            {
                REQUIRE(k < P.num_kb, "k block %d", k);
                ++k_seen[k];
            }
            if(r == 0)
                ++tiles_seen[{wi.m_blk, wi.n_start}];
        }
        for(int k = 0; k < P.num_kb; ++k)
            REQUIRE(k_seen[k] == 1, "cluster %d k block %d accumulated %d times", c, k, k_seen[k]);
    }
    REQUIRE(static_cast<int>(tiles_seen.size()) == P.total_tiles, "every tile has one cluster");
}

static long g_cluster_plans = 0;

static void check_gemm_plan(const GemmPlanInput& in)
{
    GemmPlan gp;
    REQUIRE(plan_gemm(in, &gp), "plan_gemm refused M=%lld N=%lld", (long long)in.M, (long long)in.N);
    ++g_plans;
    if(gp.pp.cluster_k)
    {
        ++g_cluster_plans;
        REQUIRE(in.cluster_ok && !in.force.no_ksplit && in.batch == 0, "cluster plan where it is not allowed");
        REQUIRE(gp.pp.tiles_m == (in.M + BM - 1) / BM && gp.pp.tiles_n == (in.N + gp.bn - 1) / gp.bn, "tile counts");
        if(gp.bn == 256)
            walk_clusters<256>(in, gp);
        else if(gp.bn == 128)
            walk_clusters<128>(in, gp);
        else
            walk_clusters<64>(in, gp);
        return;
    }
    const PlanParams& P = gp.pp;
    const int cg = gp.cg, bn = gp.bn, units = in.sm_count / cg;
    REQUIRE(cg == 1 || (cg == 2 && bn == 256), "cg %d bn %d", cg, bn);
    REQUIRE(gp.grid % cg == 0 && gp.grid >= cg && gp.grid <= units * cg, "grid %d", gp.grid);
    REQUIRE(bn / cg >= in.b_min || bn == 64, "B rows per CTA %d below the minimum %d", bn / cg, in.b_min);
    const int64_t nb = in.batch > 0 ? in.batch : 1;
    REQUIRE(P.tiles_m == (in.M + BM * cg - 1) / (BM * cg) && P.tiles_n == (in.N + bn - 1) / bn, "tile counts");
    REQUIRE(P.total_tiles == static_cast<int64_t>(P.tiles_m) * P.tiles_n * nb, "total tiles");
    if(P.stream_k != 0)
    {
        ++g_balanced_plans;
        REQUIRE((in.ks_pays || in.bal_ok) && in.ks_allowed && !in.force.no_ksplit && in.batch == 0 && P.ksplit == 0 && P.split == 1,
                "balanced plan where it is not allowed");
        REQUIRE(gp.grid == units * cg && (in.ks_pays ? bn >= 128 : bn == 256), "a balanced launch uses every unit");
        REQUIRE(P.ks_full % units == 0 && P.ks_full + P.ks_rem == P.total_tiles && P.ks_rem <= kMaxTailTiles, "whole tiles %d + region %d", P.ks_full, P.ks_rem);
        REQUIRE(P.ks_kb % 2 == 0 && static_cast<int64_t>(P.ks_kb) * units >= static_cast<int64_t>(P.ks_rem) * P.num_kb &&
                    static_cast<int64_t>(P.ks_kb - 2) * units < static_cast<int64_t>(P.ks_rem) * P.num_kb, "run length %d", P.ks_kb);
        REQUIRE(gp.partial_bytes == static_cast<size_t>(units) * BM * cg * bn * 4, "one parking slot per unit");
        REQUIRE(gp.partial_bytes <= static_cast<size_t>(in.sm_count) * BM * 256 * 4, "parked bytes beyond the fixed scratch");
    }
    else if(P.ksplit >= 2)
    {
        ++g_ksplit_plans;
        REQUIRE(in.ks_pays && in.ks_allowed && !in.force.no_ksplit, "K split where it is not allowed");
        REQUIRE(gp.grid == units * cg, "a K-split launch uses every unit");
        REQUIRE(P.ks_full % units == 0 && P.ks_full + P.ks_rem == P.total_tiles, "whole tiles %d + tail %d", P.ks_full, P.ks_rem);
        REQUIRE(P.ks_rem * P.ksplit <= units, "slices %d x %d beyond the %d units", P.ks_rem, P.ksplit, units);
        REQUIRE(P.ks_rem <= kMaxTailTiles, "tail tiles beyond the counters");
        REQUIRE(P.ks_kb % 2 == 0 && P.ks_kb * (P.ksplit - 1) < P.num_kb && P.ks_kb * P.ksplit >= P.num_kb, "slice length");
        REQUIRE(bn / P.ksplit >= 32, "reduction part narrower than a chunk");
        REQUIRE(gp.partial_bytes == static_cast<size_t>(P.ks_rem) * P.ksplit * BM * cg * bn * 4, "parked bytes");
        REQUIRE(gp.partial_bytes <= static_cast<size_t>(in.sm_count) * BM * 256 * 4, "parked bytes beyond the fixed scratch");
        REQUIRE(P.num_slots >= 4 && P.num_slots == (P.ks_full / units + 2 < 4 ? 4 : P.ks_full / units + 2), "slots");
    }
    else
    {
        REQUIRE(gp.partial_bytes == 0, "scratch without a K split");
        if(P.split > 1)
        {
            ++g_slice_plans;
            REQUIRE(P.split_start % units == 0 && (P.total_tiles - P.split_start) * P.split <= units, "slice tail");
            REQUIRE(gp.b_split_rows == bn / P.split / cg && gp.b_split_rows * cg >= 64 && gp.b_split_rows >= in.b_min,
                    "rows of a slice's B box: %d", gp.b_split_rows);
        }
        REQUIRE(P.num_slots == (P.total_work + units - 1) / units, "slots");
    }
    Coverage cov;
    if(in.ks_pays || in.bal_ok)
        walk_bn<MODE_GEMM, true>(bn, P, static_cast<const GroupTiles*>(nullptr), cg, gp.grid, cov);
    else
        walk_bn<MODE_GEMM, false>(bn, P, static_cast<const GroupTiles*>(nullptr), cg, gp.grid, cov);
    // every chunk of every tile exactly once
    REQUIRE(static_cast<int64_t>(cov.out.size()) == static_cast<int64_t>(P.total_tiles) * (bn / 32), "chunks written: %zu of %lld",
            cov.out.size(), (long long)P.total_tiles * (bn / 32));
    for(const auto& kv : cov.out)
        REQUIRE(kv.second == 1, "chunk (%d, %d, %d) written %d times", std::get<0>(kv.first), std::get<1>(kv.first),
                std::get<2>(kv.first), kv.second);
    if(P.stream_k != 0)
    {
        REQUIRE(static_cast<int>(cov.tail_k.size()) == P.ks_rem, "tiles of the balanced region");
        for(const auto& kv : cov.tail_k)
            for(int k = 0; k < P.num_kb; ++k)
                REQUIRE(kv.second[k] == 1, "tile %d k block %d accumulated %d times", kv.first, k, kv.second[k]);
        for(const auto& kv : cov.unit_kb)
            REQUIRE(kv.second <= P.ks_kb, "unit %d runs %d k blocks", kv.first, kv.second);
        REQUIRE(cov.parked_by.size() == cov.head_fix.size(), "every tile with parked parts has a head that adds them");
        for(const auto& kv : cov.head_fix)
        {
            const auto& parts = cov.parked_by[kv.first];
            REQUIRE(static_cast<int>(parts.size()) == kv.second.second, "tile %d: %zu parts parked, head adds %d", kv.first, parts.size(), kv.second.second);
            for(size_t i = 0; i < parts.size(); ++i)
            {
                REQUIRE(parts[i].first == kv.second.first + static_cast<int>(i), "tile %d: part %zu parked by unit %d", kv.first, i, parts[i].first);
                if(i > 0)
                    REQUIRE(parts[i].second > parts[i - 1].second, "parts in k order");
            }
        }
    }
    else if(P.ksplit >= 2)
    {
        REQUIRE(static_cast<int>(cov.tail_k.size()) == P.ks_rem, "tail tiles with slices");
        for(const auto& kv : cov.tail_k)
            for(int k = 0; k < P.num_kb; ++k)
                REQUIRE(kv.second[k] == 1, "tail %d k block %d accumulated %d times", kv.first, k, kv.second[k]);
        for(const auto& kv : cov.tail_slices)
            REQUIRE(static_cast<int>(kv.second.size()) == P.ksplit, "tail %d has %zu slices", kv.first, kv.second.size());
    }
}

static void check_grouped_plan(const std::vector<std::array<int64_t, 3>>& shapes, int sm_count, int b_min, TileConfig force)
{
    std::vector<GroupTiles> tiles(shapes.size());
    GroupedPlan gp;
    REQUIRE(plan_grouped(reinterpret_cast<const int64_t(*)[3]>(shapes.data()), static_cast<int>(shapes.size()), sm_count, b_min,
                         force, tiles.data(), &gp),
            "plan_grouped refused");
    ++g_plans;
    const int cg = gp.cg, bn = gp.bn;
    int64_t sum = 0;
    for(size_t i = 0; i < shapes.size(); ++i)
    {
        REQUIRE(tiles[i].tile_start == sum, "prefix sum of group %zu", i);
        REQUIRE(tiles[i].tiles_m == (shapes[i][0] + BM * cg - 1) / (BM * cg) && tiles[i].tiles_n == (shapes[i][1] + bn - 1) / bn,
                "tile counts of group %zu", i);
        REQUIRE(tiles[i].m_fastest == (tiles[i].tiles_m < tiles[i].tiles_n ? 1 : 0), "tile order of group %zu", i);
        sum += static_cast<int64_t>(tiles[i].tiles_m) * tiles[i].tiles_n;
        for(int t = tiles[i].tile_start; t < sum; ++t)
            REQUIRE(find_group(tiles.data(), static_cast<int>(tiles.size()), t) == static_cast<int>(i), "find_group(%d)", t);
    }
    REQUIRE(gp.pp.total_tiles == sum && gp.pp.group_count == static_cast<int>(shapes.size()), "totals");
    Coverage cov;
    walk_bn<MODE_GROUPED, false>(bn, gp.pp, tiles.data(), cg, gp.grid, cov);
    REQUIRE(static_cast<int64_t>(cov.out.size()) == sum * (bn / 32), "chunks written: %zu of %lld", cov.out.size(),
            (long long)sum * (bn / 32));
    for(const auto& kv : cov.out)
        REQUIRE(kv.second == 1, "group %d chunk (%d, %d) written %d times", std::get<0>(kv.first), std::get<1>(kv.first),
                std::get<2>(kv.first), kv.second);
}

int main()
{
    // tile order: both orders enumerate every position once
    for(int tm : {1, 3, 16})
        for(int tn : {1, 2, 16})
            for(int order : {0, 1})
            {
                std::map<std::pair<int, int>, int> seen;
                for(int t = 0; t < tm * tn; ++t)
                {
                    int m, n;
                    tile_position(t, tm, tn, order, &m, &n);
                    REQUIRE(m >= 0 && m < tm && n >= 0 && n < tn, "position");
                    ++seen[{m, n}];
                }
                REQUIRE(static_cast<int>(seen.size()) == tm * tn, "order %d visits every tile", order);
            }

    const int64_t sizes[] = {1, 100, 128, 129, 256, 300, 768, 1000, 2048, 2560, 3328, 3840, 4096, 4864, 8192};
    const int kbs[]       = {1, 3, 4, 16, 27, 32, 40, 47, 48, 64, 80, 128, 256};
    const int sms[]       = {148, 132, 16, 2};
    for(int sm : sms)
        for(int64_t M : sizes)
            for(int64_t N : sizes)
                for(int kb : kbs)
                    for(int pays = 0; pays < 2; ++pays)
                    {
                        GemmPlanInput in;
                        in.M = M, in.N = N, in.num_kb = kb, in.sm_count = sm, in.b_min = 32;
                        in.ks_pays = pays != 0, in.ks_allowed = true;
                        check_gemm_plan(in);
                        if(M <= 1024 && N <= 4096)
                        {
                            // cluster K split: the library's choice under two capacities, and every named K batch
                            GemmPlanInput c = in;
                            c.cluster_ok = true;
                            c.cluster_cap[0] = 70, c.cluster_cap[1] = 33, c.cluster_cap[2] = 13;
                            check_gemm_plan(c);
                            c.cluster_cap[0] = 8, c.cluster_cap[1] = 4, c.cluster_cap[2] = 0;
                            check_gemm_plan(c);
                            for(int kbatch : {2, 4, 8})
                                for(int bn : {0, 64, 128, 256})
                                {
                                    c.force = TileConfig{};
                                    c.force.kbatch = kbatch, c.force.bn = bn;
                                    check_gemm_plan(c);
                                }
                        }
                        if(kb == 40 || kb == 80)
                        {
                            in.ks_allowed = false; // a capturing stream / no scratch
                            check_gemm_plan(in);
                            in.ks_allowed = true;
                            in.b_min      = 64; // N-major B
                            check_gemm_plan(in);
                            for(int bn : {64, 128, 256})
                                for(int cgf : {0, 1, 2})
                                    for(int nks : {0, 1})
                                    {
                                        in.force.bn = bn, in.force.cg = cgf, in.force.no_ksplit = nks;
                                        check_gemm_plan(in);
                                    }
                            in.force = TileConfig{};
                            in.b_min = 32;
                            for(int bn : {0, 128, 256}) // balanced K ranges wherever they apply
                                for(int cgf : {0, 1, 2})
                                {
                                    in.force.bn = bn, in.force.cg = cgf, in.force.stream_k = 1;
                                    check_gemm_plan(in);
                                }
                            in.force = TileConfig{};
                            if(!in.ks_pays) // families with balanced instances only: the library's choice and the pinned plan
                            {
                                in.bal_ok = true;
                                check_gemm_plan(in);
                                for(int cgf : {0, 1, 2})
                                {
                                    in.force.cg = cgf, in.force.stream_k = 1;
                                    check_gemm_plan(in);
                                }
                                in.force  = TileConfig{};
                                in.bal_ok = false;
                            }
                            for(int64_t batch : {2, 3, 40})
                            {
                                in.batch = batch;
                                check_gemm_plan(in);
                            }
                        }
                    }
    // the five benchmark shapes on a B200
    {
        GemmPlanInput in;
        in.sm_count = 148, in.b_min = 32, in.ks_allowed = true;
        in.M = 3840, in.N = 4096, in.num_kb = 64, in.ks_pays = true;
        check_gemm_plan(in);
        GemmPlan gp;
        plan_gemm(in, &gp);
        REQUIRE(gp.bn == 256 && gp.cg == 2 && gp.pp.ksplit == 4 && gp.pp.ks_rem == 18 && gp.pp.ks_full == 222, "fp16 GEMM plan");
        in.num_kb = 32, in.ks_pays = false;
        check_gemm_plan(in);
        plan_gemm(in, &gp);
        REQUIRE(gp.pp.ksplit == 0 && gp.pp.split == 4 && gp.pp.split_start == 222, "int8 GEMM plan");
        in.M = 128 * 36 * 36, in.N = 256, in.num_kb = 27, in.b_min = 64;
        check_gemm_plan(in);
    }
    // one half-filled wave: balanced K ranges on CTA pairs for a long K, the plain plan for a short one or for
    // operands that would not stay in L2
    {
        GemmPlanInput in;
        in.sm_count = 148, in.b_min = 32, in.ks_allowed = true, in.ks_pays = true;
        in.M = 1280, in.N = 2048, in.num_kb = 128;
        GemmPlan gp;
        plan_gemm(in, &gp);
        REQUIRE(gp.pp.stream_k == 1 && gp.cg == 2 && gp.bn == 256 && gp.pp.ks_kb == 70 && gp.pp.ks_full == 0 && gp.pp.ks_rem == 40,
                "1280 x 2048 x 8192: balanced, run %d", gp.pp.ks_kb);
        in.num_kb = 64;
        plan_gemm(in, &gp);
        REQUIRE(gp.pp.stream_k == 0 && gp.cg == 1, "1280 x 2048 x 4096: plain");
        in.M = 512, in.N = 8192, in.num_kb = 256;
        plan_gemm(in, &gp);
        REQUIRE(gp.pp.stream_k == 0, "512 x 8192 x 16384: operands beyond L2, plain");
        in.M = 1280, in.N = 2048, in.num_kb = 128, in.ks_pays = false;
        plan_gemm(in, &gp);
        REQUIRE(gp.pp.stream_k == 0, "no balanced plan for kernels without the scratch path");
        in.bal_ok = true; // fused epilogues, int8: instances of their own
        plan_gemm(in, &gp);
        REQUIRE(gp.pp.stream_k == 1 && gp.cg == 2 && gp.bn == 256 && gp.pp.ks_kb == 70, "balanced instances of the other families");
    }
    // grouped tables
    std::mt19937 rng(1234);
    for(int rep = 0; rep < 300; ++rep)
    {
        std::vector<std::array<int64_t, 3>> shapes(1 + rng() % 24);
        for(auto& s : shapes)
            s = {static_cast<int64_t>(1 + rng() % 4200), static_cast<int64_t>(1 + rng() % 4200), static_cast<int64_t>(1 + rng() % 70)};
        for(int sm : {148, 64})
        {
            check_grouped_plan(shapes, sm, 32, TileConfig{});
            TileConfig f;
            f.bn = 128;
            check_grouped_plan(shapes, sm, 64, f);
        }
    }
    {
        std::vector<std::array<int64_t, 3>> shapes(64);
        for(int g = 0; g < 64; ++g)
            shapes[g] = {256 * (1 + g % 16), 4096, 64};
        check_grouped_plan(shapes, 148, 32, TileConfig{});
    }
    REQUIRE(g_cluster_plans > 1000 && g_ksplit_plans > 1000 && g_slice_plans > 1000 && g_balanced_plans > 1000,
            "the sweep reaches every kind of plan");
    std::printf("work plan checks passed: %ld plans (%ld with a K split through the scratch, %ld with balanced K ranges, %ld "
                "with a cluster K split, %ld with column slices), %ld assertions\n", g_plans, g_ksplit_plans, g_balanced_plans,
                g_cluster_plans, g_slice_plans, g_checks);
    return 0;
}
