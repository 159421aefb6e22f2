// Grouped fp16 GEMM with a bias row per group, E_g = A_g * B_g + D0_g, in the style of the reference's
// example/28_grouped_gemm_bias/grouped_gemm_bias_xdl_fp16.cpp: D0 has stride 0 (one row of N values read by every
// output row), the functor is Add in binary16 (the accumulator reaches it rounded, CShuffleDataType = F16).
//   usage: grouped_gemm_bias_xdl_fp16 [verify init time [group_count]]
//   group i: M = 256 + 256 i, N = 128 + 128 i, K = 64 + 64 i   (the reference example's shapes; it draws the
//   group count with an unseeded rand() % 16 + 1, here it is an argument and defaults to 4)
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
using Add         = ck::tensor_operation::element_wise::Add;

using ADataType = F16;
using BDataType = F16;
using AccDataType = F32;
using CShuffleDataType = F16;
using D0DataType = F16;
using DsDataType = ck::Tuple<D0DataType>;
using CDEElementOp = Add;
using EDataType = F16;
using ALayout = Row;
using BLayout = Col;
using ELayout = Row;

static constexpr auto GemmDefault = ck::tensor_operation::device::GemmSpecialization::Default;

// clang-format off
using DeviceGemmInstance = ck::tensor_operation::device::DeviceGroupedGemmXdl<
    ALayout, BLayout, ELayout, ADataType, BDataType, AccDataType, CShuffleDataType, DsDataType, EDataType, PassThrough, PassThrough, CDEElementOp, GemmDefault,
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
        gemm_descs.push_back({M, N, K, K, K, N, {0}});
    }

    std::vector<Tensor<ADataType>> a_tensors;
    std::vector<Tensor<BDataType>> b_tensors;
    std::vector<Tensor<D0DataType>> d0_tensors;
    std::vector<Tensor<EDataType>> c_host_tensors, c_device_tensors;
    std::vector<std::unique_ptr<DeviceMem>> a_bufs, b_bufs, d0_bufs, c_bufs;
    std::vector<const void*> p_a, p_b;
    std::vector<void*> p_c;
    std::vector<std::array<const void*, 1>> p_ds;
    std::size_t flop = 0, num_btype = 0;

    for(int i = 0; i < group_count; ++i)
    {
        const auto& g = gemm_descs[i];
        a_tensors.emplace_back(example::matrix_descriptor(g.M_, g.K_, g.stride_A_, ALayout{}));
        b_tensors.emplace_back(example::matrix_descriptor(g.K_, g.N_, g.stride_B_, BLayout{}));
        d0_tensors.emplace_back(example::matrix_descriptor(g.M_, g.N_, g.stride_Ds_[0], ELayout{}));
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
            d0_tensors[i].GenerateTensorValue(GeneratorTensor_2<D0DataType>{-5, 5});
        }
        else if(flags.init_method == 2)
        {
            a_tensors[i].GenerateTensorValue(GeneratorTensor_3<ADataType>{0.0, 1.0});
            b_tensors[i].GenerateTensorValue(GeneratorTensor_3<BDataType>{-0.5, 0.5});
            d0_tensors[i].GenerateTensorValue(GeneratorTensor_3<D0DataType>{-0.5, 0.5});
        }
        a_bufs.emplace_back(std::make_unique<DeviceMem>(sizeof(ADataType) * a_tensors[i].mDesc.GetElementSpace()));
        b_bufs.emplace_back(std::make_unique<DeviceMem>(sizeof(BDataType) * b_tensors[i].mDesc.GetElementSpace()));
        d0_bufs.emplace_back(std::make_unique<DeviceMem>(sizeof(D0DataType) * d0_tensors[i].mDesc.GetElementSpace()));
        c_bufs.emplace_back(std::make_unique<DeviceMem>(sizeof(EDataType) * c_device_tensors[i].mDesc.GetElementSpace()));
        a_bufs[i]->ToDevice(a_tensors[i].mData.data());
        b_bufs[i]->ToDevice(b_tensors[i].mData.data());
        d0_bufs[i]->ToDevice(d0_tensors[i].mData.data());
        p_ds.push_back({d0_bufs[i]->GetDeviceBuffer()});
        p_a.push_back(a_bufs[i]->GetDeviceBuffer());
        p_b.push_back(b_bufs[i]->GetDeviceBuffer());
        p_c.push_back(c_bufs[i]->GetDeviceBuffer());
    }

    auto gemm     = DeviceGemmInstance{};
    auto invoker  = gemm.MakeInvoker();
    auto cde_element_op = CDEElementOp{};
    auto argument = gemm.MakeArgument(p_a, p_b, p_ds, p_c, gemm_descs, PassThrough{}, PassThrough{}, cde_element_op);

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
            // the reference example applies the functor to the rounded GEMM result in place
            // (example/28_grouped_gemm_bias/grouped_gemm_bias_xdl_fp16.cpp:263-270)
            for(int m = 0; m < gemm_descs[i].M_; ++m)
                for(int n = 0; n < gemm_descs[i].N_; ++n)
                    cde_element_op(c_host_tensors[i](m, n), c_host_tensors[i](m, n), d0_tensors[i](m, n));
            pass &= ck::utils::check_err(c_device_tensors[i].mData, c_host_tensors[i].mData);
        }
    }
    return pass ? 0 : 1;
}
