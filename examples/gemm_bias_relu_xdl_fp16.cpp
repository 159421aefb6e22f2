// E = Relu(A*B + D) with D a bias row of length N (stride 0), in the style of the reference's
// example/03_gemm_bias_relu/gemm_bias_relu_xdl_fp16.cpp.  The functor is local to the example, as there: it adds
// and compares in binary16 (the accumulator reaches it already rounded, CShuffleDataType = F16).  A functor cannot
// cross the C ABI, so the example names the library epilogue that computes it with one EpilogueTraits
// specialisation; the host verification below still calls the functor itself.
//   usage: gemm_bias_relu_xdl_fp16 [verify init time [M N K StrideA StrideB StrideE]]
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
using PassThrough = ck::tensor_operation::element_wise::PassThrough;

// C = A * B;  E = Relu(C + D), all in binary16 (example/03_gemm_bias_relu/gemm_bias_relu_xdl_fp16.cpp:32-43)
struct AddRelu
{
    void operator()(ck::half_t& e, const ck::half_t& c, const ck::half_t& d) const
    {
        const ck::half_t x = c + d;
        e                  = x > 0 ? x : 0;
    }
};

namespace ck {
namespace b200 {
// the library epilogue with this arithmetic: half(acc) + d in binary16, then max(x, 0)
template <>
struct EpilogueTraits<::AddRelu, ctx_gemm_cde>
{
    static constexpr int kind = CKB_EPI_ADD_RELU_F16;
    static void params(const ::AddRelu&, float (&p)[4]) { p[0] = p[1] = p[2] = p[3] = 0; }
};
} // namespace b200
} // namespace ck

using ADataType        = F16;
using BDataType        = F16;
using AccDataType      = F32;
using CShuffleDataType = F16;
using DDataType        = F16;
using DsDataType       = ck::Tuple<DDataType>;
using EDataType        = F16;
using ALayout          = Row;
using BLayout          = Col;
using ELayout          = Row;
using CDEElementOp     = AddRelu;

static constexpr auto GemmSpec = ck::tensor_operation::device::GemmSpecialization::MNKPadding;

// clang-format off
using DeviceOpInstance = ck::tensor_operation::device::DeviceGemmMultipleD_Xdl_CShuffle<
    ALayout, BLayout, ELayout, ADataType, BDataType, AccDataType, CShuffleDataType, DsDataType, EDataType, PassThrough, PassThrough, CDEElementOp, GemmSpec,
    1, 256, 256, 128, 32, 8, 8, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, 1, 1, S<1, 32, 1, 8>, 8>;
// clang-format on

int main(int argc, char* argv[])
{
    example::RunFlags flags;
    ck::index_t M = 3840, N = 4096, K = 4096;
    ck::index_t StrideA = 4096, StrideB = 4096, StrideE = 4096;
    const int first = example::parse_flags(argc, argv, flags);
    if(argc == 10)
    {
        M = std::stoi(argv[first]), N = std::stoi(argv[first + 1]), K = std::stoi(argv[first + 2]);
        StrideA = std::stoi(argv[first + 3]), StrideB = std::stoi(argv[first + 4]), StrideE = std::stoi(argv[first + 5]);
    }
    else if(argc != 1 && argc != 4)
        example::usage_and_exit("arg4 to 9: M, N, K, StrideA, StrideB, StrideE");

    Tensor<ADataType> a_m_k(example::matrix_descriptor(M, K, StrideA, ALayout{}));
    Tensor<BDataType> b_k_n(example::matrix_descriptor(K, N, StrideB, BLayout{}));
    Tensor<DDataType> d_m_n(example::matrix_descriptor(M, N, 0, ELayout{})); // one row, read by every m
    Tensor<EDataType> e_host(example::matrix_descriptor(M, N, StrideE, ELayout{}));
    Tensor<EDataType> e_device(example::matrix_descriptor(M, N, StrideE, ELayout{}));
    std::cout << "a_m_k: " << a_m_k.mDesc << "\nb_k_n: " << b_k_n.mDesc << "\nd_m_n: " << d_m_n.mDesc
              << "\ne_m_n: " << e_host.mDesc << std::endl;

    if(flags.init_method == 1)
    {
        a_m_k.GenerateTensorValue(GeneratorTensor_2<ADataType>{-5, 5});
        b_k_n.GenerateTensorValue(GeneratorTensor_2<BDataType>{-5, 5});
        d_m_n.GenerateTensorValue(GeneratorTensor_2<DDataType>{-5, 5});
    }
    else if(flags.init_method != 0)
    {
        a_m_k.GenerateTensorValue(GeneratorTensor_3<ADataType>{0.0, 1.0});
        b_k_n.GenerateTensorValue(GeneratorTensor_3<BDataType>{-0.5, 0.5});
        d_m_n.GenerateTensorValue(GeneratorTensor_3<DDataType>{0.0, 1.0});
    }

    DeviceMem a_buf(sizeof(ADataType) * a_m_k.mDesc.GetElementSpace());
    DeviceMem b_buf(sizeof(BDataType) * b_k_n.mDesc.GetElementSpace());
    DeviceMem d_buf(sizeof(DDataType) * d_m_n.mDesc.GetElementSpace());
    DeviceMem e_buf(sizeof(EDataType) * e_device.mDesc.GetElementSpace());
    a_buf.ToDevice(a_m_k.mData.data());
    b_buf.ToDevice(b_k_n.mData.data());
    d_buf.ToDevice(d_m_n.mData.data());

    auto cde_element_op = CDEElementOp{};
    auto device_op      = DeviceOpInstance{};
    auto invoker        = device_op.MakeInvoker();
    auto argument       = device_op.MakeArgument(a_buf.GetDeviceBuffer(), b_buf.GetDeviceBuffer(),
                                                 std::array<const void*, 1>{d_buf.GetDeviceBuffer()},
                                                 e_buf.GetDeviceBuffer(), M, N, K, StrideA, StrideB,
                                                 std::array<ck::index_t, 1>{0}, StrideE, PassThrough{}, PassThrough{},
                                                 cde_element_op);
    if(!device_op.IsSupportedArgument(argument))
        throw std::runtime_error("wrong! this device_op instance does not support this problem");

    const float ave_time = invoker.Run(argument, StreamConfig{nullptr, flags.time_kernel});
    if(flags.time_kernel)
        example::print_perf(ave_time, std::size_t(2) * M * N * K,
                            sizeof(ADataType) * M * K + sizeof(BDataType) * K * N + sizeof(EDataType) * M * N +
                                sizeof(EDataType) * N,
                            device_op.GetTypeString());

    if(flags.do_verification)
    {
        // C = A*B rounded to binary16 on the host (the reference rounds the accumulator to CShuffleDataType
        // before the functor sees it), then the functor element by element
        Tensor<CShuffleDataType> c_m_n(HostTensorDescriptor(std::vector<std::size_t>{std::size_t(M), std::size_t(N)}));
        using ReferenceGemmInstance = ck::tensor_operation::host::ReferenceGemm<ADataType, BDataType, CShuffleDataType,
                                                                                AccDataType, PassThrough, PassThrough,
                                                                                PassThrough>;
        auto ref_gemm    = ReferenceGemmInstance{};
        auto ref_invoker = ref_gemm.MakeInvoker();
        auto ref_arg     = ref_gemm.MakeArgument(a_m_k, b_k_n, c_m_n, PassThrough{}, PassThrough{}, PassThrough{});
        ref_invoker.Run(ref_arg);
        for(int m = 0; m < M; ++m)
            for(int n = 0; n < N; ++n)
                cde_element_op(e_host(m, n), c_m_n(m, n), d_m_n(m, n));
        e_buf.FromDevice(e_device.mData.data());
        return ck::utils::check_err(e_device.mData, e_host.mData) ? 0 : 1;
    }
    return 0;
}
