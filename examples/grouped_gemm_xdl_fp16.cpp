// Grouped fp16 GEMM driver in the style of the reference's example/15_grouped_gemm/grouped_gemm_xdl_fp16.cpp:
// independent GEMMs in one launch, caller-allocated device workspace (GetWorkSpaceSize / SetWorkSpacePointer).
//   usage: grouped_gemm_xdl_fp16 [verify init time [group_count]]
//   group i: M = 256 + 256 i, N = 128 + 128 i, K = 64 + 64 i   (the reference example's shapes)
//   group_count = 64 selects M_g = 256 (1 + g mod 16), N = K = 4096 instead.
#include "example_common.hpp"

#include "ck/library/reference_tensor_operation/cpu/reference_gemm.hpp"
#include "ck/library/utility/check_err.hpp"
#include "ck/tensor_operation/gpu/device/device_grouped_gemm_xdl.hpp"
#include "ck/tensor_operation/gpu/element/element_wise_operation.hpp"

template <ck::index_t... Is>
using S = ck::Sequence<Is...>;
using F16 = ck::half_t;
using F32 = float;
using Row = ck::tensor_layout::gemm::RowMajor;
using Col = ck::tensor_layout::gemm::ColumnMajor;
using PassThrough = ck::tensor_operation::element_wise::PassThrough;

using ADataType = F16;
using BDataType = F16;
using AccDataType = F32;
using CShuffleDataType = F16;
using DsDataType = ck::Tuple<>;
using EDataType = F16;
using ALayout = Row;
using BLayout = Col;
using ELayout = Row;

static constexpr auto GemmDefault = ck::tensor_operation::device::GemmSpecialization::Default;

// clang-format off
using DeviceGemmInstance = ck::tensor_operation::device::DeviceGroupedGemmXdl<
    ALayout, BLayout, ELayout, ADataType, BDataType, AccDataType, CShuffleDataType, DsDataType, EDataType, PassThrough, PassThrough, PassThrough, GemmDefault,
    1, 256, 256, 128, 32, 8, 8, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, 1, 1, S<1, 32, 1, 8>, 8>;
// clang-format on

using ReferenceGemmInstance = ck::tensor_operation::host::ReferenceGemm<ADataType, BDataType, EDataType, AccDataType,
                                                                        PassThrough, PassThrough, PassThrough>;

int main(int argc, char* argv[])
{
    example::RunFlags flags;
    int group_count = 4;
    const int first = example::parse_flags(argc, argv, flags);
    if(argc == 5)
        group_count = std::stoi(argv[first]);
    else if(argc != 1 && argc != 4)
        example::usage_and_exit("arg4: group count");

    std::vector<ck::tensor_operation::device::GemmDesc> gemm_descs;
    for(int i = 0; i < group_count; ++i)
    {
        ck::index_t M = 256 + 256 * i, N = 128 + 128 * i, K = 64 + 64 * i;
        if(group_count == 64)
            M = 256 * (1 + i % 16), N = 4096, K = 4096;
        gemm_descs.push_back({M, N, K, K, K, N, {}});
    }

    std::vector<Tensor<ADataType>> a_tensors;
    std::vector<Tensor<BDataType>> b_tensors;
    std::vector<Tensor<EDataType>> c_host_tensors, c_device_tensors;
    std::vector<std::unique_ptr<DeviceMem>> a_bufs, b_bufs, c_bufs;
    std::vector<const void*> p_a, p_b;
    std::vector<void*> p_c;
    std::vector<std::array<const void*, 0>> p_ds(group_count);
    std::size_t flop = 0, num_btype = 0;

    for(int i = 0; i < group_count; ++i)
    {
        const auto& g = gemm_descs[i];
        a_tensors.emplace_back(example::matrix_descriptor(g.M_, g.K_, g.stride_A_, ALayout{}));
        b_tensors.emplace_back(example::matrix_descriptor(g.K_, g.N_, g.stride_B_, BLayout{}));
        c_host_tensors.emplace_back(example::matrix_descriptor(g.M_, g.N_, g.stride_C_, ELayout{}));
        c_device_tensors.emplace_back(example::matrix_descriptor(g.M_, g.N_, g.stride_C_, ELayout{}));
        std::cout << "gemm[" << i << "] a_m_k: " << a_tensors[i].mDesc << " b_k_n: " << b_tensors[i].mDesc
                  << " c_m_n: " << c_device_tensors[i].mDesc << std::endl;
        flop += std::size_t(2) * g.M_ * g.K_ * g.N_;
        num_btype += sizeof(ADataType) * a_tensors[i].mDesc.GetElementSize() +
                     sizeof(BDataType) * b_tensors[i].mDesc.GetElementSize() +
                     sizeof(EDataType) * c_device_tensors[i].mDesc.GetElementSize();
        if(flags.init_method == 1)
        {
            a_tensors[i].GenerateTensorValue(GeneratorTensor_2<ADataType>{-5, 5});
            b_tensors[i].GenerateTensorValue(GeneratorTensor_2<BDataType>{-5, 5});
        }
        else if(flags.init_method == 2)
        {
            a_tensors[i].GenerateTensorValue(GeneratorTensor_3<ADataType>{0.0, 1.0});
            b_tensors[i].GenerateTensorValue(GeneratorTensor_3<BDataType>{-0.5, 0.5});
        }
        a_bufs.emplace_back(std::make_unique<DeviceMem>(sizeof(ADataType) * a_tensors[i].mDesc.GetElementSpace()));
        b_bufs.emplace_back(std::make_unique<DeviceMem>(sizeof(BDataType) * b_tensors[i].mDesc.GetElementSpace()));
        c_bufs.emplace_back(std::make_unique<DeviceMem>(sizeof(EDataType) * c_device_tensors[i].mDesc.GetElementSpace()));
        a_bufs[i]->ToDevice(a_tensors[i].mData.data());
        b_bufs[i]->ToDevice(b_tensors[i].mData.data());
        p_a.push_back(a_bufs[i]->GetDeviceBuffer());
        p_b.push_back(b_bufs[i]->GetDeviceBuffer());
        p_c.push_back(c_bufs[i]->GetDeviceBuffer());
    }

    auto gemm     = DeviceGemmInstance{};
    auto invoker  = gemm.MakeInvoker();
    auto argument = gemm.MakeArgument(p_a, p_b, p_ds, p_c, gemm_descs, PassThrough{}, PassThrough{}, PassThrough{});

    DeviceMem gemm_desc_workspace(gemm.GetWorkSpaceSize(&argument));
    gemm.SetWorkSpacePointer(&argument, gemm_desc_workspace.GetDeviceBuffer());

    if(!gemm.IsSupportedArgument(argument))
        throw std::runtime_error("wrong! device_gemm with the specified compilation parameters does "
                                 "not support this GEMM problem");

    const float ave_time = invoker.Run(argument, StreamConfig{nullptr, flags.time_kernel});
    if(flags.time_kernel)
        example::print_perf(ave_time, flop, num_btype, gemm.GetTypeString());

    bool pass = true;
    if(flags.do_verification)
    {
        for(int i = 0; i < group_count; ++i)
        {
            c_bufs[i]->FromDevice(c_device_tensors[i].mData.data());
            auto ref_gemm    = ReferenceGemmInstance{};
            auto ref_invoker = ref_gemm.MakeInvoker();
            auto ref_arg     = ref_gemm.MakeArgument(a_tensors[i], b_tensors[i], c_host_tensors[i], PassThrough{},
                                                     PassThrough{}, PassThrough{});
            ref_invoker.Run(ref_arg);
            pass &= ck::utils::check_err(c_device_tensors[i].mData, c_host_tensors[i].mData);
        }
    }
    return pass ? 0 : 1;
}
