// fp16 GEMM driver in the style of the reference's example/01_gemm/gemm_xdl_fp16.cpp: both instances
// the reference declares (DeviceGemmXdl and DeviceGemm_Xdl_CShuffle) are instantiated with the
// reference's template argument lists; they run on B200 through libckb200.so.
//   usage: gemm_xdl_fp16 [verify init time [M N K StrideA StrideB StrideC]]
#include "example_common.hpp"

#include "ck/library/reference_tensor_operation/cpu/reference_gemm.hpp"
#include "ck/library/utility/check_err.hpp"
#include "ck/tensor_operation/gpu/device/device_gemm_xdl.hpp"
#include "ck/tensor_operation/gpu/device/device_gemm_xdl_cshuffle.hpp"
#include "ck/tensor_operation/gpu/device/gemm_specialization.hpp"
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
using CDataType = F16;
using AccDataType = F32;
using CShuffleDataType = F32;
using ALayout = Row;
using BLayout = Col;
using CLayout = Row;

static constexpr auto GemmDefault = ck::tensor_operation::device::GemmSpecialization::Default;

// clang-format off
using DeviceGemmInstance0 = ck::tensor_operation::device::DeviceGemmXdl<
    ADataType, BDataType, CDataType, AccDataType, ALayout, BLayout, CLayout, PassThrough, PassThrough, PassThrough, GemmDefault,
    256, 256, 128, 4, 8, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true, 7, 1>;
using DeviceGemmInstance1 = ck::tensor_operation::device::DeviceGemm_Xdl_CShuffle<
    ALayout, BLayout, CLayout, ADataType, BDataType, CDataType, AccDataType, CShuffleDataType, PassThrough, PassThrough, PassThrough, GemmDefault,
    1, 256, 256, 128, 32, 8, 8, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, 1, 1, S<1, 32, 1, 8>, 8>;
// clang-format on

using ReferenceGemmInstance = ck::tensor_operation::host::ReferenceGemm<ADataType, BDataType, CDataType, AccDataType,
                                                                        PassThrough, PassThrough, PassThrough>;

template <typename DeviceGemmInstance>
bool run(const example::RunFlags& flags, ck::index_t M, ck::index_t N, ck::index_t K, ck::index_t StrideA,
         ck::index_t StrideB, ck::index_t StrideC)
{
    Tensor<ADataType> a_m_k(example::matrix_descriptor(M, K, StrideA, ALayout{}));
    Tensor<BDataType> b_k_n(example::matrix_descriptor(K, N, StrideB, BLayout{}));
    Tensor<CDataType> c_host(example::matrix_descriptor(M, N, StrideC, CLayout{}));
    Tensor<CDataType> c_device(example::matrix_descriptor(M, N, StrideC, CLayout{}));
    std::cout << "a_m_k: " << a_m_k.mDesc << "\nb_k_n: " << b_k_n.mDesc << "\nc_m_n: " << c_host.mDesc << std::endl;

    if(flags.init_method == 1)
    {
        a_m_k.GenerateTensorValue(GeneratorTensor_2<ADataType>{-5, 5});
        b_k_n.GenerateTensorValue(GeneratorTensor_2<BDataType>{-5, 5});
    }
    else if(flags.init_method == 2)
    {
        a_m_k.GenerateTensorValue(GeneratorTensor_3<ADataType>{0.0, 1.0});
        b_k_n.GenerateTensorValue(GeneratorTensor_3<BDataType>{-0.5, 0.5});
    }

    DeviceMem a_buf(sizeof(ADataType) * a_m_k.mDesc.GetElementSpace());
    DeviceMem b_buf(sizeof(BDataType) * b_k_n.mDesc.GetElementSpace());
    DeviceMem c_buf(sizeof(CDataType) * c_device.mDesc.GetElementSpace());
    a_buf.ToDevice(a_m_k.mData.data());
    b_buf.ToDevice(b_k_n.mData.data());

    auto gemm     = DeviceGemmInstance{};
    auto invoker  = gemm.MakeInvoker();
    auto argument = gemm.MakeArgument(static_cast<ADataType*>(a_buf.GetDeviceBuffer()),
                                      static_cast<BDataType*>(b_buf.GetDeviceBuffer()),
                                      static_cast<CDataType*>(c_buf.GetDeviceBuffer()), M, N, K, StrideA, StrideB,
                                      StrideC, PassThrough{}, PassThrough{}, PassThrough{});
    if(!gemm.IsSupportedArgument(argument))
        throw std::runtime_error("wrong! device_gemm with the specified compilation parameters does "
                                 "not support this GEMM problem");

    const float ave_time = invoker.Run(argument, StreamConfig{nullptr, flags.time_kernel});
    if(flags.time_kernel)
        example::print_perf(ave_time, std::size_t(2) * M * N * K,
                            sizeof(ADataType) * M * K + sizeof(BDataType) * K * N + sizeof(CDataType) * M * N,
                            gemm.GetTypeString());
    c_buf.FromDevice(c_device.mData.data());

    if(flags.do_verification)
    {
        auto ref_gemm    = ReferenceGemmInstance{};
        auto ref_invoker = ref_gemm.MakeInvoker();
        auto ref_arg     = ref_gemm.MakeArgument(a_m_k, b_k_n, c_host, PassThrough{}, PassThrough{}, PassThrough{});
        ref_invoker.Run(ref_arg);
        return ck::utils::check_err(c_device.mData, c_host.mData);
    }
    return true;
}

int main(int argc, char* argv[])
{
    example::RunFlags flags;
    ck::index_t M = 3840, N = 4096, K = 4096, StrideA = 4096, StrideB = 4096, StrideC = 4096;
    const int first = example::parse_flags(argc, argv, flags);
    if(argc == 10)
    {
        M = std::stoi(argv[first]), N = std::stoi(argv[first + 1]), K = std::stoi(argv[first + 2]);
        StrideA = std::stoi(argv[first + 3]), StrideB = std::stoi(argv[first + 4]), StrideC = std::stoi(argv[first + 5]);
    }
    else if(argc != 1 && argc != 4)
        example::usage_and_exit("arg4 to 9: M (256x), N(128x), K(32x), StrideA, StrideB, StrideC");

    const bool ok0 = run<DeviceGemmInstance0>(flags, M, N, K, StrideA, StrideB, StrideC);
    const bool ok1 = run<DeviceGemmInstance1>(flags, M, N, K, StrideA, StrideB, StrideC);
    return ok0 && ok1 ? 0 : 1;
}
