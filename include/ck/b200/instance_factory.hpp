// Instance factory with the reference's interface:
//   ck::tensor_operation::device::instance::DeviceOperationInstanceFactory<DeviceOp>::GetInstances()
// (library/include/ck/library/tensor_operation_instance/device_operation_instance_factory.hpp:34-35,
//  gpu/gemm.hpp:233-378, gpu/gemm_add_add_fastgelu.hpp:79+, gpu/grouped_gemm.hpp:76-129).
// The reference returns some two hundred AMD tuning tuples per operation; here each list holds the sm_100a tile
// configurations (see kTileChoices).  Client code that walks the list, asks IsSupportedArgument and keeps the
// fastest instance works unchanged.
#pragma once
#include <memory>
#include <vector>

#include "ck/b200/device_ops.hpp"

namespace ck {
namespace tensor_operation {
namespace device {
namespace instance {

using F64  = double;
using F32  = float;
using F16  = ck::half_t;
using BF16 = ck::bhalf_t;

using EMPTY_TUPLE   = ck::Tuple<>;
using F16_TUPLE     = ck::Tuple<F16>;
using F16_F16_TUPLE = ck::Tuple<F16, F16>;
using F32_TUPLE     = ck::Tuple<F32>;

using Row = ck::tensor_layout::gemm::RowMajor;
using Col = ck::tensor_layout::gemm::ColumnMajor;

using PassThrough    = ck::tensor_operation::element_wise::PassThrough;
using Scale          = ck::tensor_operation::element_wise::Scale;
using Bilinear       = ck::tensor_operation::element_wise::Bilinear;
using AddAddFastGelu = ck::tensor_operation::element_wise::AddAddFastGelu;

template <index_t... Is>
using S = ck::Sequence<Is...>;

template <typename DeviceOp>
struct DeviceOperationInstanceFactory;

// The tile configurations every list holds, in this order.  The first entry leaves the choice to the library (its
// heuristic picks among the others from the problem size); the rest pin one configuration each, so that a client
// that walks the list, asks IsSupportedArgument and times every instance (profiler/include/profile_gemm_impl.hpp:
// 139-249) sees the whole set, as it does with the reference's lists of tuning tuples.
//   M x N of a tile: 256 x 256 on a CTA pair (tcgen05 cta_group::2), 128 x 256, 128 x 128, 128 x 64 on one CTA;
//   the last entry is the pair tile without the K-split tail (no library scratch).
struct TileChoice
{
    int32_t tile_config;
};
inline constexpr TileChoice kTileChoices[] = {
    {0},
    {CKB_TILE_CONFIG(256, 2, 0)},
    {CKB_TILE_CONFIG(256, 1, 0)},
    {CKB_TILE_CONFIG(128, 1, 0)},
    {CKB_TILE_CONFIG(64, 1, 0)},
    {CKB_TILE_CONFIG(256, 2, 1)},
};

// clang-format off
// One operation object per tile configuration.  The reference-style template arguments name the tile that runs:
// BlockSize = the kernel's 320 threads, MPerBlock x NPerBlock = the output tile, KPerBlock = one 128-byte k block.
#define CKB_PUSH_TILE_INSTANCES(OP, ...)                                                                                \
    do                                                                                                                  \
    {                                                                                                                   \
        auto push = [&](auto op, int32_t tc) { op->SetTileConfig(tc); op_ptrs.push_back(std::move(op)); };              \
        push(std::make_unique<OP<__VA_ARGS__, 1, 256, 256, 128, 4 * K1, K1, K1, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, K1, K1, 1, \
                                 S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, K1, K1, 1, 1, 1, S<1, 32, 1, 8>, K1>>(), kTileChoices[0].tile_config); \
        push(std::make_unique<OP<__VA_ARGS__, 1, 320, 256, 256, 8 * K1, K1, K1, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, K1, K1, 1, \
                                 S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, K1, K1, 1, 1, 1, S<1, 32, 1, 8>, K1>>(), kTileChoices[1].tile_config); \
        push(std::make_unique<OP<__VA_ARGS__, 1, 320, 128, 256, 8 * K1, K1, K1, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, K1, K1, 1, \
                                 S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, K1, K1, 1, 1, 1, S<1, 32, 1, 8>, K1>>(), kTileChoices[2].tile_config); \
        push(std::make_unique<OP<__VA_ARGS__, 1, 320, 128, 128, 8 * K1, K1, K1, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, K1, K1, 1, \
                                 S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, K1, K1, 1, 1, 1, S<1, 32, 1, 8>, K1>>(), kTileChoices[3].tile_config); \
        push(std::make_unique<OP<__VA_ARGS__, 1, 320, 128, 64, 8 * K1, K1, K1, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, K1, K1, 1,  \
                                 S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, K1, K1, 1, 1, 1, S<1, 32, 1, 8>, K1>>(), kTileChoices[4].tile_config); \
        push(std::make_unique<OP<__VA_ARGS__, 2, 320, 256, 256, 8 * K1, K1, K1, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, K1, K1, 1, \
                                 S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, K1, K1, 1, 1, 1, S<1, 32, 1, 8>, K1>>(), kTileChoices[5].tile_config); \
    } while(0)

// DeviceGemm<..., PassThrough, PassThrough, PassThrough>
template <typename ALayout, typename BLayout, typename CLayout, typename ADataType, typename BDataType, typename CDataType>
struct DeviceOperationInstanceFactory<DeviceGemm<ALayout, BLayout, CLayout, ADataType, BDataType, CDataType, PassThrough, PassThrough, PassThrough>>
{
    using DeviceOp = DeviceGemm<ALayout, BLayout, CLayout, ADataType, BDataType, CDataType, PassThrough, PassThrough, PassThrough>;
    static auto GetInstances()
    {
        std::vector<std::unique_ptr<DeviceOp>> op_ptrs;
        constexpr index_t K1 = 16 / sizeof(ADataType);
        CKB_PUSH_TILE_INSTANCES(DeviceGemm_Xdl_CShuffle, ALayout, BLayout, CLayout, ADataType, BDataType, CDataType, F32, F32,
                                PassThrough, PassThrough, PassThrough, GemmSpecialization::MNKPadding);
        return op_ptrs;
    }
};

// DeviceGemmMultipleD<..., Tuple<F16, F16>, F16, PassThrough, PassThrough, AddAddFastGelu>
template <typename ALayout, typename BLayout, typename DELayout>
struct DeviceOperationInstanceFactory<DeviceGemmMultipleD<ALayout, BLayout, DELayout, F16, F16, F16_F16_TUPLE, F16, PassThrough, PassThrough, AddAddFastGelu>>
{
    using DeviceOp = DeviceGemmMultipleD<ALayout, BLayout, DELayout, F16, F16, F16_F16_TUPLE, F16, PassThrough, PassThrough, AddAddFastGelu>;
    static auto GetInstances()
    {
        std::vector<std::unique_ptr<DeviceOp>> op_ptrs;
        constexpr index_t K1 = 8;
        CKB_PUSH_TILE_INSTANCES(DeviceGemmMultipleD_Xdl_CShuffle, ALayout, BLayout, DELayout, F16, F16, F32, F32, F16_F16_TUPLE, F16,
                                PassThrough, PassThrough, AddAddFastGelu, GemmSpecialization::MNKPadding);
        return op_ptrs;
    }
};

// DeviceGroupedGemm<..., Tuple<>, F16, PassThrough, PassThrough, PassThrough>
template <typename ALayout, typename BLayout, typename ELayout>
struct DeviceOperationInstanceFactory<DeviceGroupedGemm<ALayout, BLayout, ELayout, F16, F16, EMPTY_TUPLE, F16, PassThrough, PassThrough, PassThrough>>
{
    using DeviceOp = DeviceGroupedGemm<ALayout, BLayout, ELayout, F16, F16, EMPTY_TUPLE, F16, PassThrough, PassThrough, PassThrough>;
    static auto GetInstances()
    {
        std::vector<std::unique_ptr<DeviceOp>> op_ptrs;
        constexpr index_t K1 = 8;
        CKB_PUSH_TILE_INSTANCES(DeviceGroupedGemmXdl, ALayout, BLayout, ELayout, F16, F16, F32, F16, EMPTY_TUPLE, F16,
                                PassThrough, PassThrough, PassThrough, GemmSpecialization::MNKPadding);
        return op_ptrs;
    }
};
#undef CKB_PUSH_TILE_INSTANCES
// clang-format on

} // namespace instance
} // namespace device
} // namespace tensor_operation
} // namespace ck
