// Instance factory with the reference's interface:
//   ck::tensor_operation::device::instance::DeviceOperationInstanceFactory<DeviceOp>::GetInstances()
// (library/include/ck/library/tensor_operation_instance/device_operation_instance_factory.hpp:34-35,
//  gpu/gemm.hpp:233-378, gpu/gemm_add_add_fastgelu.hpp:79+, gpu/grouped_gemm.hpp:76-129).
// The reference returns some two hundred AMD tuning tuples per operation; the sm_100a library chooses its
// tile configuration itself, so each list holds the B200 operation once.  Client code that walks the list,
// asks IsSupportedArgument and keeps the fastest instance works unchanged.
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

// clang-format off
// DeviceGemm<..., PassThrough, PassThrough, PassThrough>
template <typename ALayout, typename BLayout, typename CLayout, typename ADataType, typename BDataType, typename CDataType>
struct DeviceOperationInstanceFactory<DeviceGemm<ALayout, BLayout, CLayout, ADataType, BDataType, CDataType, PassThrough, PassThrough, PassThrough>>
{
    using DeviceOp = DeviceGemm<ALayout, BLayout, CLayout, ADataType, BDataType, CDataType, PassThrough, PassThrough, PassThrough>;
    static auto GetInstances()
    {
        std::vector<std::unique_ptr<DeviceOp>> op_ptrs;
        constexpr index_t K1 = 16 / sizeof(ADataType);
        op_ptrs.push_back(std::make_unique<DeviceGemm_Xdl_CShuffle<
            ALayout, BLayout, CLayout, ADataType, BDataType, CDataType, F32, F32, PassThrough, PassThrough, PassThrough, GemmSpecialization::MNKPadding,
            1, 256, 256, 128, 4 * K1, K1, K1, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, K1, K1, 1,
            S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, K1, K1, 1, 1, 1, S<1, 32, 1, 8>, K1>>());
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
        op_ptrs.push_back(std::make_unique<DeviceGemmMultipleD_Xdl_CShuffle<
            ALayout, BLayout, DELayout, F16, F16, F32, F32, F16_F16_TUPLE, F16, PassThrough, PassThrough, AddAddFastGelu, GemmSpecialization::MNKPadding,
            1, 256, 256, 128, 32, 8, 8, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1,
            S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, 1, 1, S<1, 32, 1, 8>, 8>>());
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
        op_ptrs.push_back(std::make_unique<DeviceGroupedGemmXdl<
            ALayout, BLayout, ELayout, F16, F16, F32, F16, EMPTY_TUPLE, F16, PassThrough, PassThrough, PassThrough, GemmSpecialization::MNKPadding,
            1, 256, 256, 128, 32, 8, 8, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1,
            S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, 1, 1, S<1, 32, 1, 8>, 8>>());
        return op_ptrs;
    }
};
// clang-format on

} // namespace instance
} // namespace device
} // namespace tensor_operation
} // namespace ck
