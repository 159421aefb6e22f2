// E = FastGelu(A*B + D0 + D1) in the style of the reference's
// example/04_gemm_add_add_fastgelu/gemm_add_add_fastgelu_xdl_fp16.cpp (D0 = bias row with stride 0).
//   usage: gemm_add_add_fastgelu_xdl_fp16 [verify init time [M N K StrideA StrideB StrideD0 StrideD1 StrideE]]
#include "example_common.hpp"

#include "ck/library/reference_tensor_operation/cpu/reference_gemm.hpp"
#include "ck/library/utility/check_err.hpp"
#include "ck/tensor_operation/gpu/device/device_gemm_multiple_d_xdl_cshuffle.hpp"
#include "ck/tensor_operation/gpu/element/element_wise_operation.hpp"

template <ck::index_t... Is>
using S = ck::Sequence<Is...>;
using F16 = ck::half_t;
using F32 = float;
using Row = ck::tensor_layout::gemm::RowMajor;
using Col = ck::tensor_layout::gemm::ColumnMajor;
using PassThrough    = ck::tensor_operation::element_wise::PassThrough;
using AddAddFastGelu = ck::tensor_operation::element_wise::AddAddFastGelu;

using ADataType = F16;
using BDataType = F16;
using AccDataType = F32;
using CShuffleDataType = F32;
using D0DataType = F16;
using D1DataType = F16;
using DsDataType = ck::Tuple<D0DataType, D1DataType>;
using EDataType = F16;
using ALayout = Row;
using BLayout = Col;
using ELayout = Row;
using CDEElementOp = AddAddFastGelu;

static constexpr auto GemmDefault = ck::tensor_operation::device::GemmSpecialization::Default;

// clang-format off
using DeviceOpInstance = ck::tensor_operation::device::DeviceGemmMultipleD_Xdl_CShuffle<
    ALayout, BLayout, ELayout, ADataType, BDataType, AccDataType, CShuffleDataType, DsDataType, EDataType, PassThrough, PassThrough, CDEElementOp, GemmDefault,
    1, 256, 256, 128, 32, 8, 8, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, 1, 1, S<1, 32, 1, 8>, 8>;
// clang-format on

int main(int argc, char* argv[])
{
    example::RunFlags flags;
    ck::index_t M = 3840, N = 4096, K = 4096;
    ck::index_t StrideA = 4096, StrideB = 4096, StrideD0 = 0, StrideD1 = 4096, StrideE = 4096;
    const int first = example::parse_flags(argc, argv, flags);
    if(argc == 12)
    {
        M = std::stoi(argv[first]), N = std::stoi(argv[first + 1]), K = std::stoi(argv[first + 2]);
        StrideA = std::stoi(argv[first + 3]), StrideB = std::stoi(argv[first + 4]);
        StrideD0 = std::stoi(argv[first + 5]), StrideD1 = std::stoi(argv[first + 6]), StrideE = std::stoi(argv[first + 7]);
    }
    else if(argc != 1 && argc != 4)
        example::usage_and_exit("arg4 to 11: M, N, K, StrideA, StrideB, StrideD0, StrideD1, StrideE");

    Tensor<ADataType> a_m_k(example::matrix_descriptor(M, K, StrideA, ALayout{}));
    Tensor<BDataType> b_k_n(example::matrix_descriptor(K, N, StrideB, BLayout{}));
    Tensor<D0DataType> d0_m_n(example::matrix_descriptor(M, N, StrideD0, ELayout{}));
    Tensor<D1DataType> d1_m_n(example::matrix_descriptor(M, N, StrideD1, ELayout{}));
    Tensor<EDataType> e_host(example::matrix_descriptor(M, N, StrideE, ELayout{}));
    Tensor<EDataType> e_device(example::matrix_descriptor(M, N, StrideE, ELayout{}));
    std::cout << "a_m_k: " << a_m_k.mDesc << "\nb_k_n: " << b_k_n.mDesc << "\nd0_m_n: " << d0_m_n.mDesc
              << "\nd1_m_n: " << d1_m_n.mDesc << "\ne_m_n: " << e_host.mDesc << std::endl;

    if(flags.init_method == 1)
    {
        a_m_k.GenerateTensorValue(GeneratorTensor_2<ADataType>{-5, 5});
        b_k_n.GenerateTensorValue(GeneratorTensor_2<BDataType>{-5, 5});
        d0_m_n.GenerateTensorValue(GeneratorTensor_2<D0DataType>{-5, 5});
        d1_m_n.GenerateTensorValue(GeneratorTensor_2<D1DataType>{-5, 5});
    }
    else if(flags.init_method == 2)
    {
        a_m_k.GenerateTensorValue(GeneratorTensor_3<ADataType>{0.0, 1.0});
        b_k_n.GenerateTensorValue(GeneratorTensor_3<BDataType>{-0.5, 0.5});
        d0_m_n.GenerateTensorValue(GeneratorTensor_3<D0DataType>{0.0, 1.0});
        d1_m_n.GenerateTensorValue(GeneratorTensor_3<D1DataType>{0.0, 1.0});
    }

    DeviceMem a_buf(sizeof(ADataType) * a_m_k.mDesc.GetElementSpace());
    DeviceMem b_buf(sizeof(BDataType) * b_k_n.mDesc.GetElementSpace());
    DeviceMem d0_buf(sizeof(D0DataType) * d0_m_n.mDesc.GetElementSpace());
    DeviceMem d1_buf(sizeof(D1DataType) * d1_m_n.mDesc.GetElementSpace());
    DeviceMem e_buf(sizeof(EDataType) * e_device.mDesc.GetElementSpace());
    a_buf.ToDevice(a_m_k.mData.data());
    b_buf.ToDevice(b_k_n.mData.data());
    d0_buf.ToDevice(d0_m_n.mData.data());
    d1_buf.ToDevice(d1_m_n.mData.data());

    auto cde_element_op = CDEElementOp{};
    auto device_op      = DeviceOpInstance{};
    auto invoker        = device_op.MakeInvoker();
    auto argument       = device_op.MakeArgument(
        a_buf.GetDeviceBuffer(), b_buf.GetDeviceBuffer(),
        std::array<const void*, 2>{d0_buf.GetDeviceBuffer(), d1_buf.GetDeviceBuffer()}, e_buf.GetDeviceBuffer(), M, N, K,
        StrideA, StrideB, std::array<ck::index_t, 2>{StrideD0, StrideD1}, StrideE, PassThrough{}, PassThrough{},
        cde_element_op);
    if(!device_op.IsSupportedArgument(argument))
        throw std::runtime_error("wrong! this device_op instance does not support this problem");

    const float ave_time = invoker.Run(argument, StreamConfig{nullptr, flags.time_kernel});
    if(flags.time_kernel)
        example::print_perf(ave_time, std::size_t(2) * M * N * K,
                            sizeof(ADataType) * M * K + sizeof(BDataType) * K * N + sizeof(D0DataType) * N +
                                sizeof(D1DataType) * M * N + sizeof(EDataType) * M * N,
                            device_op.GetTypeString());
    e_buf.FromDevice(e_device.mData.data());

    if(flags.do_verification)
    {
        // C = A*B in fp32 on the host, then the functor element by element (reference: example/04...:215-244)
        Tensor<AccDataType> c_m_n(HostTensorDescriptor(std::vector<std::size_t>{std::size_t(M), std::size_t(N)}));
        using ReferenceGemmInstance = ck::tensor_operation::host::ReferenceGemm<ADataType, BDataType, AccDataType, AccDataType,
                                                                                PassThrough, PassThrough, PassThrough>;
        auto ref_gemm    = ReferenceGemmInstance{};
        auto ref_invoker = ref_gemm.MakeInvoker();
        auto ref_arg     = ref_gemm.MakeArgument(a_m_k, b_k_n, c_m_n, PassThrough{}, PassThrough{}, PassThrough{});
        ref_invoker.Run(ref_arg);
        for(int m = 0; m < M; ++m)
            for(int n = 0; n < N; ++n)
                cde_element_op(e_host(m, n), c_m_n(m, n), d0_m_n(m, n), d1_m_n(m, n));
        return ck::utils::check_err(e_device.mData, e_host.mData) ? 0 : 1;
    }
    return 0;
}
