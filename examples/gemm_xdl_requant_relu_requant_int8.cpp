// int8 GEMM + Requant-ReLU-Requant in the style of the reference's
// example/14_gemm_xdl_requant_relu_requant/gemm_xdl_requant_relu_requant_int8.cpp.  The functor of that example is
// provided by the element-wise header under the same name; a fourth optional flag selects the
// round-to-nearest-even variant (scaleRelu 14) instead of the reference's truncating one (scaleRelu 1).
//   usage: gemm_xdl_requant_relu_requant_int8 [verify init time [M N K StrideA StrideB StrideC [rne]]]
#include "example_common.hpp"

#include "ck/library/reference_tensor_operation/cpu/reference_gemm.hpp"
#include "ck/library/utility/check_err.hpp"
#include "ck/tensor_operation/gpu/device/device_gemm_xdl_cshuffle.hpp"
#include "ck/tensor_operation/gpu/element/element_wise_operation.hpp"

template <ck::index_t... Is>
using S = ck::Sequence<Is...>;
using Row = ck::tensor_layout::gemm::RowMajor;
using Col = ck::tensor_layout::gemm::ColumnMajor;
using PassThrough = ck::tensor_operation::element_wise::PassThrough;

using ADataType = int8_t;
using BDataType = int8_t;
using CDataType = int8_t;
using AccDataType = int32_t;
using CShuffleDataType = float;

static constexpr auto GemmDefault = ck::tensor_operation::device::GemmSpecialization::Default;

// clang-format off
template <typename CElementOp>
using DeviceGemmInstance = ck::tensor_operation::device::DeviceGemm_Xdl_CShuffle<
    Row, Col, Row, ADataType, BDataType, CDataType, AccDataType, CShuffleDataType, PassThrough, PassThrough, CElementOp, GemmDefault,
    1, 256, 256, 128, 64, 16, 16, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 16, 16, 1, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 16, 16, 1, 1, 1, S<1, 64, 1, 4>, 16>;
// clang-format on

template <typename CElementOp>
bool run(const example::RunFlags& flags, ck::index_t M, ck::index_t N, ck::index_t K, ck::index_t StrideA,
         ck::index_t StrideB, ck::index_t StrideC, CElementOp c_element_op)
{
    Tensor<ADataType> a_m_k(example::matrix_descriptor(M, K, StrideA, Row{}));
    Tensor<BDataType> b_k_n(example::matrix_descriptor(K, N, StrideB, Col{}));
    Tensor<CDataType> c_host(example::matrix_descriptor(M, N, StrideC, Row{}));
    Tensor<CDataType> c_device(example::matrix_descriptor(M, N, StrideC, Row{}));
    if(flags.init_method != 0)
    {
        // symmetric integers: about half of the outputs end up zero, a tail saturates
        a_m_k.GenerateTensorValue(GeneratorTensor_2<ADataType>{-5, 6});
        b_k_n.GenerateTensorValue(GeneratorTensor_2<BDataType>{-5, 6});
    }
    DeviceMem a_buf(sizeof(ADataType) * a_m_k.mDesc.GetElementSpace());
    DeviceMem b_buf(sizeof(BDataType) * b_k_n.mDesc.GetElementSpace());
    DeviceMem c_buf(sizeof(CDataType) * c_device.mDesc.GetElementSpace());
    a_buf.ToDevice(a_m_k.mData.data());
    b_buf.ToDevice(b_k_n.mData.data());

    auto gemm     = DeviceGemmInstance<CElementOp>{};
    auto invoker  = gemm.MakeInvoker();
    auto argument = gemm.MakeArgument(static_cast<ADataType*>(a_buf.GetDeviceBuffer()),
                                      static_cast<BDataType*>(b_buf.GetDeviceBuffer()),
                                      static_cast<CDataType*>(c_buf.GetDeviceBuffer()), M, N, K, StrideA, StrideB,
                                      StrideC, PassThrough{}, PassThrough{}, c_element_op);
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
        // the reference verifies with a float accumulator (exact below 2^24)
        using ReferenceGemmInstance = ck::tensor_operation::host::ReferenceGemm<ADataType, BDataType, CDataType, float,
                                                                                PassThrough, PassThrough, CElementOp>;
        auto ref_gemm    = ReferenceGemmInstance{};
        auto ref_invoker = ref_gemm.MakeInvoker();
        auto ref_arg     = ref_gemm.MakeArgument(a_m_k, b_k_n, c_host, PassThrough{}, PassThrough{}, c_element_op);
        ref_invoker.Run(ref_arg);
        return ck::utils::check_err(c_device.mData, c_host.mData);
    }
    return true;
}

int main(int argc, char* argv[])
{
    example::RunFlags flags;
    ck::index_t M = 3840, N = 4096, K = 4096, StrideA = 4096, StrideB = 4096, StrideC = 4096;
    bool rne        = false;
    const int first = example::parse_flags(argc, argv, flags);
    if(argc == 10 || argc == 11)
    {
        M = std::stoi(argv[first]), N = std::stoi(argv[first + 1]), K = std::stoi(argv[first + 2]);
        StrideA = std::stoi(argv[first + 3]), StrideB = std::stoi(argv[first + 4]), StrideC = std::stoi(argv[first + 5]);
        rne = argc == 11 && std::stoi(argv[first + 6]) != 0;
    }
    else if(argc != 1 && argc != 4)
        example::usage_and_exit("arg4 to 9: M (256x), N(128x), K(32x), StrideA, StrideB, StrideC; arg10: 1 = rne variant");

    namespace ew = ck::tensor_operation::element_wise;
    const bool ok = rne ? run(flags, M, N, K, StrideA, StrideB, StrideC, ew::RequantReluRequantRne{0.03f, 14.0f})
                        : run(flags, M, N, K, StrideA, StrideB, StrideC, ew::RequantReluRequant{0.03f, 1.0f});
    return ok ? 0 : 1;
}
