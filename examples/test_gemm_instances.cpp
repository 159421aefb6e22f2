// The reference's GEMM unit tests in one program (test/gemm/gemm_fp16.cpp, gemm_bf16.cpp, gemm_int8.cpp with
// test/gemm/gemm_util.hpp:17-233): for every A/B layout the instances of the factory run a 1024^3 problem whose
// operands hold small integers, and the result is compared with the CPU ReferenceGemm on the same tensors.
//   usage: test_gemm_instances [fp16|bf16|int8]       (no argument: all three); exit code 0 = every instance passed
#include <cstring>
#include <iostream>
#include <memory>
#include <string>

#include "ck/ck.hpp"
#include "ck/library/host_tensor/device_memory.hpp"
#include "ck/library/host_tensor/host_tensor.hpp"
#include "ck/library/host_tensor/host_tensor_generator.hpp"
#include "ck/library/reference_tensor_operation/cpu/reference_gemm.hpp"
#include "ck/library/tensor_operation_instance/gpu/gemm.hpp"
#include "ck/library/utility/check_err.hpp"
#include "ck/tensor_operation/gpu/device/device_gemm.hpp"
#include "ck/tensor_operation/gpu/device/tensor_layout.hpp"
#include "ck/tensor_operation/gpu/element/element_wise_operation.hpp"

using Row         = ck::tensor_layout::gemm::RowMajor;
using Col         = ck::tensor_layout::gemm::ColumnMajor;
using PassThrough = ck::tensor_operation::element_wise::PassThrough;

// test/gemm/gemm_util.hpp:17-34
struct GemmParams
{
    ck::index_t M = 1024, N = 1024, K = 1024, StrideA = 1024, StrideB = 1024, StrideC = 1024;
};

template <typename Layout>
HostTensorDescriptor matrix_descriptor(std::size_t row, std::size_t col, std::size_t stride, Layout)
{
    if(std::is_same<Layout, Row>::value)
        return HostTensorDescriptor(std::vector<std::size_t>{row, col}, std::vector<std::size_t>{stride, 1});
    return HostTensorDescriptor(std::vector<std::size_t>{row, col}, std::vector<std::size_t>{1, stride});
}

// One instance against the CPU reference (gemm_util.hpp:120-233: operands from GeneratorTensor_2{-5, 5}).
template <typename ADataType, typename BDataType, typename CDataType, typename AccDataType, typename ALayout,
          typename BLayout, typename CLayout, typename DeviceGemmPtr>
bool test_gemm(DeviceGemmPtr& gemm_ptr)
{
    const GemmParams params;
    Tensor<ADataType> a_m_k(matrix_descriptor(params.M, params.K, params.StrideA, ALayout{}));
    Tensor<BDataType> b_k_n(matrix_descriptor(params.K, params.N, params.StrideB, BLayout{}));
    Tensor<CDataType> c_host(matrix_descriptor(params.M, params.N, params.StrideC, CLayout{}));
    Tensor<CDataType> c_device(matrix_descriptor(params.M, params.N, params.StrideC, CLayout{}));
    a_m_k.GenerateTensorValue(GeneratorTensor_2<ADataType>{-5, 5});
    b_k_n.GenerateTensorValue(GeneratorTensor_2<BDataType>{-5, 5});

    using ReferenceGemmInstance = ck::tensor_operation::host::ReferenceGemm<ADataType, BDataType, CDataType, AccDataType,
                                                                            PassThrough, PassThrough, PassThrough>;
    auto ref_gemm    = ReferenceGemmInstance{};
    auto ref_invoker = ref_gemm.MakeInvoker();
    auto ref_arg     = ref_gemm.MakeArgument(a_m_k, b_k_n, c_host, PassThrough{}, PassThrough{}, PassThrough{});
    ref_invoker.Run(ref_arg);

    DeviceMem a_buf(sizeof(ADataType) * a_m_k.mDesc.GetElementSpace());
    DeviceMem b_buf(sizeof(BDataType) * b_k_n.mDesc.GetElementSpace());
    DeviceMem c_buf(sizeof(CDataType) * c_device.mDesc.GetElementSpace());
    a_buf.ToDevice(a_m_k.mData.data());
    b_buf.ToDevice(b_k_n.mData.data());

    auto invoker_ptr  = gemm_ptr->MakeInvokerPointer();
    auto argument_ptr = gemm_ptr->MakeArgumentPointer(a_buf.GetDeviceBuffer(), b_buf.GetDeviceBuffer(),
                                                      c_buf.GetDeviceBuffer(), params.M, params.N, params.K,
                                                      params.StrideA, params.StrideB, params.StrideC, PassThrough{},
                                                      PassThrough{}, PassThrough{});
    if(!gemm_ptr->IsSupportedArgument(argument_ptr.get()))
    {
        std::cout << gemm_ptr->GetTypeString() << " does not support this GEMM problem" << std::endl;
        return true; // gemm_util.hpp:224-230: an instance that declines is not a failure
    }
    invoker_ptr->Run(argument_ptr.get());
    c_buf.FromDevice(c_device.mData.data());
    const bool ok = ck::utils::check_err(c_device.mData, c_host.mData);
    std::cout << gemm_ptr->GetTypeString() << (ok ? " ..... SUCCESS" : " ..... FAILURE") << std::endl;
    return ok;
}

template <typename T, typename AccDataType>
bool test_all_layouts(const char* name)
{
    auto test = [&](auto a_layout, auto b_layout, auto c_layout) {
        using DeviceOp = ck::tensor_operation::device::DeviceGemm<decltype(a_layout), decltype(b_layout),
                                                                  decltype(c_layout), T, T, T, PassThrough,
                                                                  PassThrough, PassThrough>;
        const auto gemm_ptrs =
            ck::tensor_operation::device::instance::DeviceOperationInstanceFactory<DeviceOp>::GetInstances();
        bool pass = !gemm_ptrs.empty();
        for(auto& gemm_ptr : gemm_ptrs)
            pass &= test_gemm<T, T, T, AccDataType, decltype(a_layout), decltype(b_layout), decltype(c_layout)>(gemm_ptr);
        return pass;
    };
    const bool pass = test(Row{}, Row{}, Row{}) && test(Row{}, Col{}, Row{}) && test(Col{}, Row{}, Row{}) &&
                      test(Col{}, Col{}, Row{});
    std::cout << "TestGemm " << name << " ..... " << (pass ? "SUCCESS" : "FAILURE") << std::endl;
    return pass;
}

int main(int argc, char* argv[])
{
    const std::string which = argc > 1 ? argv[1] : "all";
    bool pass               = true;
    if(which == "all" || which == "fp16")
        pass &= test_all_layouts<ck::half_t, float>("fp16");
    if(which == "all" || which == "bf16")
        pass &= test_all_layouts<ck::bhalf_t, float>("bf16");
    if(which == "all" || which == "int8")
        pass &= test_all_layouts<int8_t, int32_t>("int8");
    return pass ? 0 : 1;
}
