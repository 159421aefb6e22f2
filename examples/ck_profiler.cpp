// ckProfiler-style driver: one binary, one sub-command per operation, positional arguments as in the reference's
// profiler (profiler/src/profiler.cpp:48-148, profile_gemm.cpp:27-58, profile_gemm_add_add_fastgelu.cpp,
// profile_grouped_gemm.cpp, profile_conv_fwd_bias_relu.cpp).  For every instance the factory returns it builds the
// argument, asks IsSupportedArgument, times the kernel, prints a "Perf:" line, verifies against the CPU reference and
// finally prints "Best Perf" (profiler/include/profile_gemm_impl.hpp:139-249).
//
//   ck_profiler gemm                  <dtype 1 fp16|2 bf16|3 int8> <layout 0..3> <verify> <init> <log> <time> M N K StrideA StrideB StrideC
//   ck_profiler gemm_add_add_fastgelu <dtype 1> <layout 1> <verify> <init> <log> <time> M N K StrideA StrideB StrideD0 StrideD1 StrideE
//   ck_profiler grouped_gemm          <dtype 1> <layout 1> <verify> <init> <log> <time> Ms Ns Ks          (comma separated lists)
//   ck_profiler conv_fwd_bias_relu    <dtype 1> <verify> <init> <log> <time> N K C Y X Hi Wi Sy Sx Dy Dx LeftPy LeftPx RightPy RightPx
//   ck_profiler conv_fwd_bias_relu_add  (same arguments; adds a residual tensor after the ReLU)
//   ck_profiler batched_gemm          <dtype 1 fp16|2 bf16|3 int8> <layout 0..3> <verify> <init> <log> <time> M N K StrideA StrideB StrideC
//                                     BatchStrideA BatchStrideB BatchStrideC BatchCount
//   ck_profiler gemm_bilinear         <dtype 1> <layout 0..3> <verify> <init> <log> <time> M N K StrideA StrideB StrideD StrideE alpha beta
//   ck_profiler gemm_splitk           <dtype 1> <layout 0..3> <verify> <init> <log> <time> M N K StrideA StrideB StrideC KBatch
//   ck_profiler conv_fwd              <dtype 1 fp16|2 bf16|3 int8> <layout 1 NHWC> <verify> <init> <log> <time> <nd 1|2|3> N K C
//                                     <filter> <input> <strides> <dilations> <left pads> <right pads>   (nd values each)
// gemm takes the reference's four matrix layouts (0: mk_kn, 1: mk_nk, 2: km_kn, 3: km_nk); the fused and grouped
// sub-commands take layout 1.
#include <cstring>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include "example_common.hpp"

#include "ck/library/reference_tensor_operation/cpu/reference_conv_fwd_bias_activation.hpp"
#include "ck/library/reference_tensor_operation/cpu/reference_gemm.hpp"
#include "ck/library/tensor_operation_instance/gpu/gemm.hpp"
#include "ck/library/tensor_operation_instance/gpu/gemm_add_add_fastgelu.hpp"
#include "ck/library/tensor_operation_instance/gpu/grouped_gemm.hpp"
#include "ck/library/utility/check_err.hpp"
#include "ck/library/utility/conv_util.hpp"
#include "ck/library/reference_tensor_operation/cpu/reference_batched_gemm.hpp"
#include "ck/library/reference_tensor_operation/cpu/reference_conv_fwd.hpp"
#include "ck/tensor_operation/gpu/device/device_batched_gemm_xdl.hpp"
#include "ck/tensor_operation/gpu/device/device_gemm_multiple_d_xdl_cshuffle.hpp"
#include "ck/tensor_operation/gpu/device/device_gemm_xdl_splitk_c_shuffle.hpp"
#include "ck/tensor_operation/gpu/device/device_conv2d_fwd_xdl_c_shuffle_bias_activation_nhwc_kyxc_nhwk.hpp"
#include "ck/tensor_operation/gpu/device/device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp"

namespace inst = ck::tensor_operation::device::instance;
namespace dev  = ck::tensor_operation::device;
using inst::Col;
using inst::PassThrough;
using inst::Row;

struct Best
{
    std::string name;
    float ave_time = 0, tflops = 0, gb_per_sec = 0;
    void offer(const std::string& n, float ms, std::size_t flop, std::size_t bytes)
    {
        const float tf = static_cast<float>(flop) / 1.E9 / ms, gb = bytes / 1.E6 / ms;
        std::cout << "Perf: " << ms << " ms, " << tf << " TFlops, " << gb << " GB/s, " << n << std::endl;
        if(tf > tflops)
            name = n, ave_time = ms, tflops = tf, gb_per_sec = gb;
    }
    void report(const char* what) const
    {
        if(name.empty())
            std::cout << "this device " << what << " instance does not support this problem" << std::endl;
        else
            std::cout << "Best Perf for " << what << ": " << ave_time << " ms, " << tflops << " TFlops, " << gb_per_sec
                      << " GB/s, " << name << std::endl;
    }
};

template <typename T>
void init_tensor(Tensor<T>& t, int init_method, bool is_b)
{
    if(init_method == 1)
        t.GenerateTensorValue(GeneratorTensor_2<T>{-5, 5});
    else if(init_method == 2)
    {
        if(is_b)
            t.GenerateTensorValue(GeneratorTensor_3<T>{-0.5, 0.5});
        else
            t.GenerateTensorValue(GeneratorTensor_3<T>{0.0, 1.0});
    }
}

template <typename T, typename AccT, typename ALayout, typename BLayout>
bool profile_gemm_typed(bool verify, int init, bool time, int M, int N, int K, int sa, int sb, int sc)
{
    using DeviceOp = dev::DeviceGemm<ALayout, BLayout, Row, T, T, T, PassThrough, PassThrough, PassThrough>;
    Tensor<T> a(example::matrix_descriptor(M, K, sa, ALayout{})), b(example::matrix_descriptor(K, N, sb, BLayout{}));
    Tensor<T> c_host(example::matrix_descriptor(M, N, sc, Row{})), c_dev(example::matrix_descriptor(M, N, sc, Row{}));
    init_tensor(a, init, false);
    init_tensor(b, init, true);
    DeviceMem a_buf(sizeof(T) * a.mDesc.GetElementSpace()), b_buf(sizeof(T) * b.mDesc.GetElementSpace()),
        c_buf(sizeof(T) * c_dev.mDesc.GetElementSpace());
    a_buf.ToDevice(a.mData.data());
    b_buf.ToDevice(b.mData.data());
    if(verify)
    {
        using Ref = ck::tensor_operation::host::ReferenceGemm<T, T, T, AccT, PassThrough, PassThrough, PassThrough>;
        auto arg  = Ref::MakeArgument(a, b, c_host, {}, {}, {});
        Ref::MakeInvoker().Run(arg);
    }
    const auto op_ptrs = inst::DeviceOperationInstanceFactory<DeviceOp>::GetInstances();
    std::cout << "found " << op_ptrs.size() << " instances" << std::endl;
    Best best;
    bool pass = true;
    for(auto& op : op_ptrs)
    {
        auto arg = op->MakeArgumentPointer(a_buf.GetDeviceBuffer(), b_buf.GetDeviceBuffer(), c_buf.GetDeviceBuffer(), M, N,
                                           K, sa, sb, sc, {}, {}, {});
        auto inv = op->MakeInvokerPointer();
        if(!op->IsSupportedArgument(arg.get()))
        {
            std::cout << op->GetTypeString() << " does not support this problem" << std::endl;
            continue;
        }
        c_buf.SetZero();
        const float ms = inv->Run(arg.get(), StreamConfig{nullptr, time});
        if(time)
            best.offer(op->GetTypeString() + " [" + op->GetBackendString() + "]", ms, std::size_t(2) * M * N * K, sizeof(T) * (std::size_t(M) * K + std::size_t(K) * N + std::size_t(M) * N));
        else
            best.name = op->GetTypeString() + " [" + op->GetBackendString() + "]";
        if(verify)
        {
            c_buf.FromDevice(c_dev.mData.data());
            pass = pass && ck::utils::check_err(c_dev.mData, c_host.mData);
        }
    }
    best.report("gemm");
    return pass && !best.name.empty();
}

int profile_gemm(int argc, char* argv[])
{
    if(argc != 14)
    {
        std::printf("arg1: tensor operation (gemm: GEMM)\narg2: data type (1: fp16; 2: bf16; 3: int8)\n"
                    "arg3: matrix layout (0: A[m, k] * B[k, n] = C[m, n];\n"
                    "                     1: A[m, k] * B[n, k] = C[m, n];\n"
                    "                     2: A[k, m] * B[k, n] = C[m, n];\n"
                    "                     3: A[k, m] * B[n, k] = C[m, n])\narg4: verification (0: no; 1: yes)\n"
                    "arg5: initialization (0: no init; 1: integer value; 2: decimal value)\n"
                    "arg6: print tensor value (0: no; 1: yes)\narg7: time kernel (0=no, 1=yes)\n"
                    "arg8 to 13: M, N, K, StrideA, StrideB, StrideC\n");
        return 1;
    }
    const int dtype = std::stoi(argv[2]), layout = std::stoi(argv[3]);
    const bool verify = std::stoi(argv[4]), time = std::stoi(argv[7]);
    const int init = std::stoi(argv[5]);
    const int M = std::stoi(argv[8]), N = std::stoi(argv[9]), K = std::stoi(argv[10]);
    const int sa = std::stoi(argv[11]), sb = std::stoi(argv[12]), sc = std::stoi(argv[13]);
    if(layout < 0 || layout > 3 || dtype < 1 || dtype > 3)
    {
        std::cout << "no instance for data type " << dtype << ", matrix layout " << layout << std::endl;
        return 1;
    }
    auto run = [&](auto t, auto acc, auto la, auto lb) {
        return profile_gemm_typed<decltype(t), decltype(acc), decltype(la), decltype(lb)>(verify, init, time, M, N, K, sa,
                                                                                         sb, sc);
    };
    auto by_layout = [&](auto t, auto acc) {
        switch(layout)
        {
        case 0: return run(t, acc, Row{}, Row{}); // MK_KN_MN
        case 1: return run(t, acc, Row{}, Col{}); // MK_NK_MN
        case 2: return run(t, acc, Col{}, Row{}); // KM_KN_MN
        default: return run(t, acc, Col{}, Col{}); // KM_NK_MN
        }
    };
    const bool ok = dtype == 1 ? by_layout(ck::half_t{}, float{})
                               : dtype == 2 ? by_layout(ck::bhalf_t{}, float{}) : by_layout(int8_t{}, int32_t{});
    return ok ? 0 : 1;
}

int profile_gemm_add_add_fastgelu(int argc, char* argv[])
{
    if(argc != 16 || std::stoi(argv[2]) != 1 || std::stoi(argv[3]) != 1)
    {
        std::printf("gemm_add_add_fastgelu 1 1 verify init log time M N K StrideA StrideB StrideD0 StrideD1 StrideE\n");
        return 1;
    }
    using F16      = ck::half_t;
    using DeviceOp = dev::DeviceGemmMultipleD<Row, Col, Row, F16, F16, inst::F16_F16_TUPLE, F16, PassThrough, PassThrough,
                                              inst::AddAddFastGelu>;
    const bool verify = std::stoi(argv[4]), time = std::stoi(argv[7]);
    const int init = std::stoi(argv[5]);
    const int M = std::stoi(argv[8]), N = std::stoi(argv[9]), K = std::stoi(argv[10]);
    const int sa = std::stoi(argv[11]), sb = std::stoi(argv[12]), sd0 = std::stoi(argv[13]), sd1 = std::stoi(argv[14]),
              se = std::stoi(argv[15]);
    Tensor<F16> a(example::matrix_descriptor(M, K, sa, Row{})), b(example::matrix_descriptor(K, N, sb, Col{}));
    Tensor<F16> d0(example::matrix_descriptor(M, N, sd0, Row{})), d1(example::matrix_descriptor(M, N, sd1, Row{}));
    Tensor<F16> e_host(example::matrix_descriptor(M, N, se, Row{})), e_dev(example::matrix_descriptor(M, N, se, Row{}));
    init_tensor(a, init, false);
    init_tensor(b, init, true);
    init_tensor(d0, init, false);
    init_tensor(d1, init, false);
    DeviceMem a_buf(2 * a.mDesc.GetElementSpace()), b_buf(2 * b.mDesc.GetElementSpace()), d0_buf(2 * d0.mDesc.GetElementSpace()),
        d1_buf(2 * d1.mDesc.GetElementSpace()), e_buf(2 * e_dev.mDesc.GetElementSpace());
    a_buf.ToDevice(a.mData.data());
    b_buf.ToDevice(b.mData.data());
    d0_buf.ToDevice(d0.mData.data());
    d1_buf.ToDevice(d1.mData.data());
    const inst::AddAddFastGelu cde_op{};
    if(verify)
    {
        Tensor<float> c(HostTensorDescriptor(std::vector<std::size_t>{std::size_t(M), std::size_t(N)}));
        using Ref = ck::tensor_operation::host::ReferenceGemm<F16, F16, float, float, PassThrough, PassThrough, PassThrough>;
        auto arg  = Ref::MakeArgument(a, b, c, {}, {}, {});
        Ref::MakeInvoker().Run(arg);
        for(int m = 0; m < M; ++m)
            for(int n = 0; n < N; ++n)
                cde_op(e_host(m, n), c(m, n), d0(m, n), d1(m, n));
    }
    Best best;
    bool pass = true;
    for(auto& op : inst::DeviceOperationInstanceFactory<DeviceOp>::GetInstances())
    {
        auto arg = op->MakeArgumentPointer(a_buf.GetDeviceBuffer(), b_buf.GetDeviceBuffer(),
                                           std::array<const void*, 2>{d0_buf.GetDeviceBuffer(), d1_buf.GetDeviceBuffer()},
                                           e_buf.GetDeviceBuffer(), M, N, K, sa, sb, std::array<ck::index_t, 2>{sd0, sd1}, se,
                                           {}, {}, cde_op);
        if(!op->IsSupportedArgument(arg.get()))
        {
            std::cout << op->GetTypeString() << " does not support this problem" << std::endl;
            continue;
        }
        e_buf.SetZero();
        const float ms = op->MakeInvokerPointer()->Run(arg.get(), StreamConfig{nullptr, time});
        if(time)
            best.offer(op->GetTypeString() + " [" + op->GetBackendString() + "]", ms, std::size_t(2) * M * N * K,
                       2 * (std::size_t(M) * K + std::size_t(K) * N + N + 2 * std::size_t(M) * N));
        else
            best.name = op->GetTypeString() + " [" + op->GetBackendString() + "]";
        if(verify)
        {
            e_buf.FromDevice(e_dev.mData.data());
            pass = pass && ck::utils::check_err(e_dev.mData, e_host.mData);
        }
    }
    best.report("gemm_add_add_fastgelu");
    return pass && !best.name.empty() ? 0 : 1;
}

static std::vector<int> parse_list(const char* s)
{
    std::vector<int> v;
    std::stringstream ss(s);
    std::string item;
    while(std::getline(ss, item, ','))
        v.push_back(std::stoi(item));
    return v;
}

// layout: the reference's GemmMatrixLayout (profiler/src/profile_grouped_gemm.cpp:15-25): 0 MK_KN_MN, 1 MK_NK_MN,
// 2 KM_KN_MN, 3 KM_NK_MN; leading dimensions are the packed ones of each layout.
template <typename ALayout, typename BLayout>
int profile_grouped_gemm_layout(char* argv[])
{
    using F16      = ck::half_t;
    using DeviceOp = dev::DeviceGroupedGemm<ALayout, BLayout, Row, F16, F16, inst::EMPTY_TUPLE, F16, PassThrough, PassThrough, PassThrough>;
    constexpr bool a_row = std::is_same<ALayout, Row>::value, b_row = std::is_same<BLayout, Row>::value;
    const bool verify = std::stoi(argv[4]), time = std::stoi(argv[7]);
    const int init = std::stoi(argv[5]);
    const auto Ms = parse_list(argv[8]), Ns = parse_list(argv[9]), Ks = parse_list(argv[10]);
    const std::size_t G = Ms.size();
    if(Ns.size() != G || Ks.size() != G)
        throw std::runtime_error("wrong! inconsistent M/N/Ks, StrideA/B/Cs size");
    std::vector<dev::GemmDesc> descs;
    std::vector<Tensor<F16>> As, Bs, Ch, Cd;
    std::vector<std::unique_ptr<DeviceMem>> a_bufs, b_bufs, c_bufs;
    std::vector<const void*> p_a, p_b;
    std::vector<void*> p_c;
    std::vector<std::array<const void*, 0>> p_ds(G);
    std::size_t flop = 0, bytes = 0;
    for(std::size_t i = 0; i < G; ++i)
    {
        const int lda = a_row ? Ks[i] : Ms[i], ldb = b_row ? Ns[i] : Ks[i];
        descs.push_back({Ms[i], Ns[i], Ks[i], lda, ldb, Ns[i], {}});
        As.emplace_back(example::matrix_descriptor(Ms[i], Ks[i], lda, ALayout{}));
        Bs.emplace_back(example::matrix_descriptor(Ks[i], Ns[i], ldb, BLayout{}));
        Ch.emplace_back(example::matrix_descriptor(Ms[i], Ns[i], Ns[i], Row{}));
        Cd.emplace_back(example::matrix_descriptor(Ms[i], Ns[i], Ns[i], Row{}));
        init_tensor(As[i], init, false);
        init_tensor(Bs[i], init, true);
        a_bufs.emplace_back(std::make_unique<DeviceMem>(2 * As[i].mDesc.GetElementSpace()));
        b_bufs.emplace_back(std::make_unique<DeviceMem>(2 * Bs[i].mDesc.GetElementSpace()));
        c_bufs.emplace_back(std::make_unique<DeviceMem>(2 * Cd[i].mDesc.GetElementSpace()));
        a_bufs[i]->ToDevice(As[i].mData.data());
        b_bufs[i]->ToDevice(Bs[i].mData.data());
        p_a.push_back(a_bufs[i]->GetDeviceBuffer());
        p_b.push_back(b_bufs[i]->GetDeviceBuffer());
        p_c.push_back(c_bufs[i]->GetDeviceBuffer());
        flop += std::size_t(2) * Ms[i] * Ns[i] * Ks[i];
        bytes += 2 * (std::size_t(Ms[i]) * Ks[i] + std::size_t(Ks[i]) * Ns[i] + std::size_t(Ms[i]) * Ns[i]);
    }
    Best best;
    bool pass = true;
    for(auto& op : inst::DeviceOperationInstanceFactory<DeviceOp>::GetInstances())
    {
        auto arg = op->MakeArgumentPointer(p_a, p_b, p_ds, p_c, descs, {}, {}, {});
        DeviceMem workspace(op->GetWorkSpaceSize(arg.get()));
        op->SetWorkSpacePointer(arg.get(), workspace.GetDeviceBuffer());
        if(!op->IsSupportedArgument(arg.get()))
        {
            std::cout << op->GetTypeString() << " does not support this problem" << std::endl;
            continue;
        }
        const float ms = op->MakeInvokerPointer()->Run(arg.get(), StreamConfig{nullptr, time});
        if(time)
            best.offer(op->GetTypeString() + " [" + op->GetBackendString() + "]", ms, flop, bytes);
        else
            best.name = op->GetTypeString() + " [" + op->GetBackendString() + "]";
        if(verify)
            for(std::size_t i = 0; i < G; ++i)
            {
                c_bufs[i]->FromDevice(Cd[i].mData.data());
                using Ref = ck::tensor_operation::host::ReferenceGemm<F16, F16, F16, float, PassThrough, PassThrough, PassThrough>;
                auto rarg = Ref::MakeArgument(As[i], Bs[i], Ch[i], {}, {}, {});
                Ref::MakeInvoker().Run(rarg);
                pass = pass && ck::utils::check_err(Cd[i].mData, Ch[i].mData);
            }
    }
    best.report("grouped_gemm");
    return pass && !best.name.empty() ? 0 : 1;
}

int profile_grouped_gemm(int argc, char* argv[])
{
    const int layout = argc == 11 ? std::stoi(argv[3]) : -1;
    if(argc != 11 || std::stoi(argv[2]) != 1 || layout < 0 || layout > 3)
    {
        std::printf("grouped_gemm 1 <layout 0 MK_KN | 1 MK_NK | 2 KM_KN | 3 KM_NK> verify init log time Ms Ns Ks   "
                    "(comma separated lists, e.g. 256,512 128,256 64,128)\n");
        return 1;
    }
    return layout == 0 ? profile_grouped_gemm_layout<Row, Row>(argv)
                       : layout == 1 ? profile_grouped_gemm_layout<Row, Col>(argv)
                                     : layout == 2 ? profile_grouped_gemm_layout<Col, Row>(argv)
                                                   : profile_grouped_gemm_layout<Col, Col>(argv);
}

int profile_conv_fwd_bias_relu(int argc, char* argv[])
{
    if(argc != 22 || std::stoi(argv[2]) != 1)
    {
        std::printf("conv_fwd_bias_relu 1 verify init log time N K C Y X Hi Wi Sy Sx Dy Dx LeftPy LeftPx RightPy RightPx\n");
        return 1;
    }
    using F16 = ck::half_t;
    const bool verify = std::stoi(argv[3]), time = std::stoi(argv[6]);
    const int init = std::stoi(argv[4]);
    const ck::utils::conv::ConvParams p = ck::utils::conv::parse_conv_params(2, 7, argv);
    const auto out_sp                   = p.GetOutputSpatialLengths();
    using AddRelu = ck::tensor_operation::element_wise::AddRelu;
    // clang-format off
    using Conv = dev::DeviceConv2dFwdXdl_C_Shuffle_Bias_Activation_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<
        F16, F16, F16, float, PassThrough, PassThrough, AddRelu, ck::InMemoryDataOperationEnum::Set, dev::ConvolutionForwardSpecialization::Default,
        256, 128, 256, 4, 8, 32, 32, 2, 4, inst::S<4, 64, 1>, inst::S<1, 0, 2>, inst::S<1, 0, 2>, 2, 8, 8, true,
        inst::S<4, 64, 1>, inst::S<1, 0, 2>, inst::S<1, 0, 2>, 2, 8, 8, true, 1, 1, inst::S<1, 1, 32, 1, 1, 8>, 8>;
    // clang-format on
    const std::size_t N = p.N_, K = p.K_, C = p.C_;
    Tensor<F16> in(ck::utils::conv::get_input_host_tensor_descriptor(
        {N, C, std::size_t(p.input_spatial_lengths_[0]), std::size_t(p.input_spatial_lengths_[1])}));
    Tensor<F16> wei(ck::utils::conv::get_filters_host_tensor_descriptor(
        {K, C, std::size_t(p.filter_spatial_lengths_[0]), std::size_t(p.filter_spatial_lengths_[1])}));
    Tensor<F16> out_h(ck::utils::conv::get_output_host_tensor_descriptor({N, K, std::size_t(out_sp[0]), std::size_t(out_sp[1])}));
    Tensor<F16> out_d(out_h.mDesc), bias(HostTensorDescriptor(std::vector<std::size_t>{K}));
    init_tensor(in, init, false);
    init_tensor(wei, init, true);
    init_tensor(bias, init, false);
    DeviceMem in_buf(2 * in.mDesc.GetElementSpace()), wei_buf(2 * wei.mDesc.GetElementSpace()),
        out_buf(2 * out_d.mDesc.GetElementSpace()), bias_buf(2 * K);
    in_buf.ToDevice(in.mData.data());
    wei_buf.ToDevice(wei.mData.data());
    bias_buf.ToDevice(bias.mData.data());
    std::vector<std::unique_ptr<dev::DeviceConvFwdBiasActivation<PassThrough, PassThrough, AddRelu>>> ops;
    ops.push_back(std::make_unique<Conv>());
    Best best;
    bool pass = true;
    for(auto& op : ops)
    {
        auto arg = op->MakeArgumentPointer(in_buf.GetDeviceBuffer(), wei_buf.GetDeviceBuffer(), out_buf.GetDeviceBuffer(),
                                           bias_buf.GetDeviceBuffer(), p.N_, p.K_, p.C_, p.input_spatial_lengths_,
                                           p.filter_spatial_lengths_, out_sp, p.conv_filter_strides_, p.conv_filter_dilations_,
                                           p.input_left_pads_, p.input_right_pads_, {}, {}, {});
        if(!op->IsSupportedArgument(arg.get()))
        {
            std::cout << op->GetTypeString() << " does not support this problem" << std::endl;
            continue;
        }
        const float ms = op->MakeInvokerPointer()->Run(arg.get(), StreamConfig{nullptr, time});
        if(time)
            best.offer(op->GetTypeString() + " [" + op->GetBackendString() + "]", ms, ck::utils::conv::get_flops(p.N_, p.C_, p.K_, p.filter_spatial_lengths_, out_sp),
                       ck::utils::conv::get_btype<F16, F16, F16>(p.N_, p.C_, p.K_, p.input_spatial_lengths_,
                                                                 p.filter_spatial_lengths_, out_sp) + 2 * K);
        else
            best.name = op->GetTypeString() + " [" + op->GetBackendString() + "]";
        if(verify)
        {
            out_buf.FromDevice(out_d.mData.data());
            using Ref = ck::tensor_operation::host::ReferenceConvFwd_Bias_Activation<F16, F16, F16, PassThrough, PassThrough, AddRelu>;
            auto rarg = Ref::MakeArgument(in, wei, out_h, bias, p.conv_filter_strides_, p.conv_filter_dilations_,
                                          p.input_left_pads_, p.input_right_pads_, {}, {}, {});
            Ref::MakeInvoker().Run(rarg);
            pass = pass && ck::utils::check_err(out_d.mData, out_h.mData);
        }
    }
    best.report("conv_fwd_bias_relu");
    return pass && !best.name.empty() ? 0 : 1;
}

int profile_conv_fwd_bias_relu_add(int argc, char* argv[])
{
    if(argc != 22 || std::stoi(argv[2]) != 1)
    {
        std::printf("conv_fwd_bias_relu_add 1 verify init log time N K C Y X Hi Wi Sy Sx Dy Dx LeftPy LeftPx RightPy RightPx\n");
        return 1;
    }
    using F16 = ck::half_t;
    const bool verify = std::stoi(argv[3]), time = std::stoi(argv[6]);
    const int init = std::stoi(argv[4]);
    const ck::utils::conv::ConvParams p = ck::utils::conv::parse_conv_params(2, 7, argv);
    const auto out_sp                   = p.GetOutputSpatialLengths();
    using AddReluAdd = ck::tensor_operation::element_wise::AddReluAdd;
    // clang-format off
    using Conv = dev::DeviceConv2dFwdXdl_C_Shuffle_Bias_Activation_Add_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<
        F16, F16, F16, float, PassThrough, PassThrough, AddReluAdd, dev::ConvolutionForwardSpecialization::Default,
        256, 128, 256, 4, 8, 32, 32, 2, 4, inst::S<4, 64, 1>, inst::S<1, 0, 2>, inst::S<1, 0, 2>, 2, 8, 8, true,
        inst::S<4, 64, 1>, inst::S<1, 0, 2>, inst::S<1, 0, 2>, 2, 8, 8, true, 1, 1, inst::S<1, 1, 32, 1, 1, 8>, 8>;
    // clang-format on
    const std::size_t N = p.N_, K = p.K_, C = p.C_;
    Tensor<F16> in(ck::utils::conv::get_input_host_tensor_descriptor(
        {N, C, std::size_t(p.input_spatial_lengths_[0]), std::size_t(p.input_spatial_lengths_[1])}));
    Tensor<F16> wei(ck::utils::conv::get_filters_host_tensor_descriptor(
        {K, C, std::size_t(p.filter_spatial_lengths_[0]), std::size_t(p.filter_spatial_lengths_[1])}));
    Tensor<F16> out_h(ck::utils::conv::get_output_host_tensor_descriptor({N, K, std::size_t(out_sp[0]), std::size_t(out_sp[1])}));
    Tensor<F16> out_d(out_h.mDesc), resi(out_h.mDesc), bias(HostTensorDescriptor(std::vector<std::size_t>{K}));
    init_tensor(in, init, false);
    init_tensor(wei, init, true);
    init_tensor(bias, init, false);
    init_tensor(resi, init, false);
    DeviceMem in_buf(2 * in.mDesc.GetElementSpace()), wei_buf(2 * wei.mDesc.GetElementSpace()),
        out_buf(2 * out_d.mDesc.GetElementSpace()), bias_buf(2 * K), resi_buf(2 * resi.mDesc.GetElementSpace());
    in_buf.ToDevice(in.mData.data());
    wei_buf.ToDevice(wei.mData.data());
    bias_buf.ToDevice(bias.mData.data());
    resi_buf.ToDevice(resi.mData.data());
    std::vector<std::unique_ptr<dev::DeviceConvFwdBiasActivationAdd<PassThrough, PassThrough, AddReluAdd>>> ops;
    ops.push_back(std::make_unique<Conv>());
    Best best;
    bool pass = true;
    for(auto& op : ops)
    {
        auto arg = op->MakeArgumentPointer(in_buf.GetDeviceBuffer(), wei_buf.GetDeviceBuffer(), out_buf.GetDeviceBuffer(),
                                           bias_buf.GetDeviceBuffer(), resi_buf.GetDeviceBuffer(), p.N_, p.K_, p.C_, p.input_spatial_lengths_,
                                           p.filter_spatial_lengths_, out_sp, p.conv_filter_strides_, p.conv_filter_dilations_,
                                           p.input_left_pads_, p.input_right_pads_, {}, {}, {});
        if(!op->IsSupportedArgument(arg.get()))
        {
            std::cout << op->GetTypeString() << " does not support this problem" << std::endl;
            continue;
        }
        const float ms = op->MakeInvokerPointer()->Run(arg.get(), StreamConfig{nullptr, time});
        if(time)
            best.offer(op->GetTypeString() + " [" + op->GetBackendString() + "]", ms, ck::utils::conv::get_flops(p.N_, p.C_, p.K_, p.filter_spatial_lengths_, out_sp),
                       ck::utils::conv::get_btype<F16, F16, F16>(p.N_, p.C_, p.K_, p.input_spatial_lengths_,
                                                                 p.filter_spatial_lengths_, out_sp) + 2 * K +
                           2 * resi.mDesc.GetElementSpace());
        else
            best.name = op->GetTypeString() + " [" + op->GetBackendString() + "]";
        if(verify)
        {
            out_buf.FromDevice(out_d.mData.data());
            using Ref = ck::tensor_operation::host::ReferenceConvFwd_Bias_Activation_Add<F16, F16, F16, PassThrough, PassThrough, AddReluAdd>;
            auto rarg = Ref::MakeArgument(in, wei, out_h, bias, resi, p.conv_filter_strides_, p.conv_filter_dilations_,
                                          p.input_left_pads_, p.input_right_pads_, {}, {}, {});
            Ref::MakeInvoker().Run(rarg);
            pass = pass && ck::utils::check_err(out_d.mData, out_h.mData);
        }
    }
    best.report("conv_fwd_bias_relu_add");
    return pass && !best.name.empty() ? 0 : 1;
}

template <typename T, typename ALayout, typename BLayout>
bool profile_batched_gemm_typed(bool verify, int init, bool time, int M, int N, int K, int sa, int sb, int sc, int bsa,
                                int bsb, int bsc, int G)
{
    // clang-format off
    using Op = dev::DeviceBatchedGemmXdl<T, T, T, float, ALayout, BLayout, Row, PassThrough, PassThrough, PassThrough,
        256, 256, 128, 4, 8, 32, 32, 4, 2, inst::S<4, 64, 1>, inst::S<1, 0, 2>, inst::S<1, 0, 2>, 2, 8, 8, true,
        inst::S<4, 64, 1>, inst::S<1, 0, 2>, inst::S<1, 0, 2>, 2, 8, 8, true, 7, 1>;
    // clang-format on
    auto desc3 = [](std::size_t g, std::size_t row, std::size_t col, std::size_t stride, std::size_t bstride, auto layout) {
        const bool row_major = std::is_same<decltype(layout), Row>::value;
        return HostTensorDescriptor(std::vector<std::size_t>{g, row, col},
                                    row_major ? std::vector<std::size_t>{bstride, stride, 1}
                                              : std::vector<std::size_t>{bstride, 1, stride});
    };
    Tensor<T> a(desc3(G, M, K, sa, bsa, ALayout{})), b(desc3(G, K, N, sb, bsb, BLayout{}));
    Tensor<T> c_host(desc3(G, M, N, sc, bsc, Row{})), c_dev(desc3(G, M, N, sc, bsc, Row{}));
    init_tensor(a, init, false);
    init_tensor(b, init, true);
    DeviceMem a_buf(sizeof(T) * a.mDesc.GetElementSpace()), b_buf(sizeof(T) * b.mDesc.GetElementSpace()),
        c_buf(sizeof(T) * c_dev.mDesc.GetElementSpace());
    a_buf.ToDevice(a.mData.data());
    b_buf.ToDevice(b.mData.data());
    c_buf.SetZero();
    Op op;
    auto arg = op.MakeArgumentPointer(a_buf.GetDeviceBuffer(), b_buf.GetDeviceBuffer(), c_buf.GetDeviceBuffer(), M, N, K,
                                      sa, sb, sc, bsa, bsb, bsc, G, {}, {}, {});
    Best best;
    if(!op.IsSupportedArgument(arg.get()))
    {
        best.report("batched_gemm");
        return false;
    }
    const float ms = op.MakeInvokerPointer()->Run(arg.get(), StreamConfig{nullptr, time});
    if(time)
        best.offer(op.GetTypeString(), ms, std::size_t(2) * G * M * N * K,
                   sizeof(T) * G * (std::size_t(M) * K + std::size_t(K) * N + std::size_t(M) * N));
    else
        best.name = op.GetTypeString();
    bool pass = true;
    if(verify)
    {
        using Ref = ck::tensor_operation::host::ReferenceBatchedGemm<T, T, T, PassThrough, PassThrough, PassThrough>;
        auto rarg = Ref::MakeArgument(a, b, c_host, {}, {}, {});
        Ref::MakeInvoker().Run(rarg);
        c_buf.FromDevice(c_dev.mData.data());
        pass = ck::utils::check_err(c_dev.mData, c_host.mData);
    }
    best.report("batched_gemm");
    return pass;
}

int profile_batched_gemm(int argc, char* argv[])
{
    if(argc != 18)
    {
        std::printf("batched_gemm <dtype 1|2|3> <layout 0..3> verify init log time M N K StrideA StrideB StrideC "
                    "BatchStrideA BatchStrideB BatchStrideC BatchCount\n");
        return 1;
    }
    const int dtype = std::stoi(argv[2]), layout = std::stoi(argv[3]);
    const bool verify = std::stoi(argv[4]), time = std::stoi(argv[7]);
    const int init = std::stoi(argv[5]);
    int v[10];
    for(int i = 0; i < 10; ++i)
        v[i] = std::stoi(argv[8 + i]);
    if(layout < 0 || layout > 3 || dtype < 1 || dtype > 3)
        return 1;
    auto run = [&](auto t, auto la, auto lb) {
        return profile_batched_gemm_typed<decltype(t), decltype(la), decltype(lb)>(verify, init, time, v[0], v[1], v[2],
                                                                                   v[3], v[4], v[5], v[6], v[7], v[8], v[9]);
    };
    auto by_layout = [&](auto t) {
        switch(layout)
        {
        case 0: return run(t, Row{}, Row{});
        case 1: return run(t, Row{}, Col{});
        case 2: return run(t, Col{}, Row{});
        default: return run(t, Col{}, Col{});
        }
    };
    const bool ok = dtype == 1 ? by_layout(ck::half_t{}) : dtype == 2 ? by_layout(ck::bhalf_t{}) : by_layout(int8_t{});
    return ok ? 0 : 1;
}

// E = alpha * A * B + beta * D (profiler/src/profile_gemm_bilinear.cpp:29-43) and C = A * B with a KBatch argument
// (profile_gemm_splitk.cpp:29-42); fp16, the four layouts.
template <typename ALayout, typename BLayout>
bool profile_gemm_bilinear_or_splitk(bool bilinear, bool verify, int init, bool time, int M, int N, int K, int sa, int sb,
                                     int sd, int se, float alpha, float beta, int kbatch)
{
    using F16      = ck::half_t;
    using Bilinear = ck::tensor_operation::element_wise::Bilinear;
    // clang-format off
    using BilinearOp = dev::DeviceGemmMultipleD_Xdl_CShuffle<ALayout, BLayout, Row, F16, F16, float, float, ck::Tuple<F16>, F16, PassThrough, PassThrough, Bilinear, dev::GemmSpecialization::MNKPadding,
        1, 256, 256, 128, 32, 8, 8, 32, 32, 4, 2, inst::S<4, 64, 1>, inst::S<1, 0, 2>, inst::S<1, 0, 2>, 2, 8, 8, 1,
        inst::S<4, 64, 1>, inst::S<1, 0, 2>, inst::S<1, 0, 2>, 2, 8, 8, 1, 1, 1, inst::S<1, 32, 1, 8>, 8>;
    using SplitKOp = dev::DeviceGemmXdlSplitKCShuffle<F16, F16, F16, float, ALayout, BLayout, Row, PassThrough, PassThrough, PassThrough, dev::GemmSpecialization::MNKPadding,
        256, 256, 128, 4, 8, 32, 32, 4, 2, inst::S<1, 4, 64, 1>, inst::S<0, 2, 1, 3>, inst::S<0, 2, 1, 3>, 3, 8, 8, true,
        inst::S<1, 4, 64, 1>, inst::S<0, 1, 3, 2>, inst::S<0, 1, 3, 2>, 3, 8, 8, true, 1, 1, inst::S<1, 32, 1, 8>, 8>;
    // clang-format on
    Tensor<F16> a(example::matrix_descriptor(M, K, sa, ALayout{})), b(example::matrix_descriptor(K, N, sb, BLayout{}));
    Tensor<F16> d(example::matrix_descriptor(M, N, sd, Row{}));
    Tensor<F16> e_host(example::matrix_descriptor(M, N, se, Row{})), e_dev(example::matrix_descriptor(M, N, se, Row{}));
    init_tensor(a, init, false);
    init_tensor(b, init, true);
    init_tensor(d, init, false);
    DeviceMem a_buf(2 * a.mDesc.GetElementSpace()), b_buf(2 * b.mDesc.GetElementSpace()),
        d_buf(2 * d.mDesc.GetElementSpace()), e_buf(2 * e_dev.mDesc.GetElementSpace());
    a_buf.ToDevice(a.mData.data());
    b_buf.ToDevice(b.mData.data());
    d_buf.ToDevice(d.mData.data());
    e_buf.SetZero();
    const Bilinear op_fn{alpha, beta};
    std::string name;
    float ms = 0;
    if(bilinear)
    {
        BilinearOp op;
        auto arg = op.MakeArgumentPointer(a_buf.GetDeviceBuffer(), b_buf.GetDeviceBuffer(),
                                          std::array<const void*, 1>{d_buf.GetDeviceBuffer()}, e_buf.GetDeviceBuffer(), M, N,
                                          K, sa, sb, std::array<ck::index_t, 1>{sd}, se, {}, {}, op_fn);
        if(!op.IsSupportedArgument(arg.get()))
            return false;
        ms   = op.MakeInvokerPointer()->Run(arg.get(), StreamConfig{nullptr, time});
        name = op.GetTypeString();
    }
    else
    {
        SplitKOp op;
        auto arg = op.MakeArgumentPointer(a_buf.GetDeviceBuffer(), b_buf.GetDeviceBuffer(), e_buf.GetDeviceBuffer(), M, N, K,
                                          sa, sb, se, {}, {}, {}, kbatch);
        if(!op.IsSupportedArgument(arg.get()))
            return false;
        ms   = op.MakeInvokerPointer()->Run(arg.get(), StreamConfig{nullptr, time});
        name = op.GetTypeString();
    }
    Best best;
    if(time)
        best.offer(name, ms, std::size_t(2) * M * N * K,
                   2 * (std::size_t(M) * K + std::size_t(K) * N + (bilinear ? 2 : 1) * std::size_t(M) * N));
    else
        best.name = name;
    bool pass = true;
    if(verify)
    {
        Tensor<float> c(HostTensorDescriptor(std::vector<std::size_t>{std::size_t(M), std::size_t(N)}));
        using Ref = ck::tensor_operation::host::ReferenceGemm<F16, F16, float, float, PassThrough, PassThrough, PassThrough>;
        auto rarg = Ref::MakeArgument(a, b, c, {}, {}, {});
        Ref::MakeInvoker().Run(rarg);
        for(int m = 0; m < M; ++m)
            for(int n = 0; n < N; ++n)
            {
                if(bilinear)
                    op_fn(e_host(m, n), c(m, n), d(m, n));
                else
                    e_host(m, n) = ck::type_convert<F16>(c(m, n));
            }
        e_buf.FromDevice(e_dev.mData.data());
        pass = ck::utils::check_err(e_dev.mData, e_host.mData);
    }
    best.report(bilinear ? "gemm_bilinear" : "gemm_splitk");
    return pass;
}

int profile_gemm_bilinear_splitk(int argc, char* argv[], bool bilinear)
{
    if(argc != (bilinear ? 17 : 15) || std::stoi(argv[2]) != 1)
    {
        std::printf("gemm_bilinear 1 <layout 0..3> verify init log time M N K StrideA StrideB StrideD StrideE alpha beta\n"
                    "gemm_splitk   1 <layout 0..3> verify init log time M N K StrideA StrideB StrideC KBatch\n");
        return 1;
    }
    const int layout  = std::stoi(argv[3]);
    const bool verify = std::stoi(argv[4]), time = std::stoi(argv[7]);
    const int init = std::stoi(argv[5]);
    const int M = std::stoi(argv[8]), N = std::stoi(argv[9]), K = std::stoi(argv[10]);
    const int sa = std::stoi(argv[11]), sb = std::stoi(argv[12]);
    const int sd = bilinear ? std::stoi(argv[13]) : N, se = std::stoi(argv[bilinear ? 14 : 13]);
    const float alpha = bilinear ? std::stof(argv[15]) : 1.f, beta = bilinear ? std::stof(argv[16]) : 0.f;
    const int kbatch = bilinear ? 1 : std::stoi(argv[14]);
    auto run         = [&](auto la, auto lb) {
        return profile_gemm_bilinear_or_splitk<decltype(la), decltype(lb)>(bilinear, verify, init, time, M, N, K, sa, sb, sd,
                                                                           se, alpha, beta, kbatch);
    };
    const bool ok = layout == 0 ? run(Row{}, Row{}) : layout == 1 ? run(Row{}, Col{}) : layout == 2 ? run(Col{}, Row{})
                                                                                                     : run(Col{}, Col{});
    return ok ? 0 : 1;
}

template <int ND, typename T>
bool profile_convnd_typed(const ck::utils::conv::ConvParams& p, bool verify, int init, bool time)
{
    namespace conv_util = ck::utils::conv;
    // clang-format off
    using Conv = dev::DeviceConvNDFwdXdl_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<
        T, T, T, float, PassThrough, PassThrough, PassThrough, dev::ConvolutionForwardSpecialization::Default, ND,
        256, 128, 256, 4, 8, 32, 32, 2, 4, inst::S<4, 64, 1>, inst::S<1, 0, 2>, inst::S<1, 0, 2>, 2, 8, 8, true,
        inst::S<4, 64, 1>, inst::S<1, 0, 2>, inst::S<1, 0, 2>, 2, 8, 8, true, 7, 1>;
    // clang-format on
    const auto out_sp = p.GetOutputSpatialLengths();
    std::vector<std::size_t> in_dims{std::size_t(p.N_), std::size_t(p.C_)}, wei_dims{std::size_t(p.K_), std::size_t(p.C_)},
        out_dims{std::size_t(p.N_), std::size_t(p.K_)};
    for(int i = 0; i < ND; ++i)
    {
        in_dims.push_back(p.input_spatial_lengths_[i]);
        wei_dims.push_back(p.filter_spatial_lengths_[i]);
        out_dims.push_back(out_sp[i]);
    }
    Tensor<T> in(conv_util::get_input_host_tensor_descriptor(in_dims, ND));
    Tensor<T> wei(conv_util::get_filters_host_tensor_descriptor(wei_dims, ND));
    Tensor<T> out_h(conv_util::get_output_host_tensor_descriptor(out_dims, ND)), out_d(out_h.mDesc);
    init_tensor(in, init, false);
    init_tensor(wei, init, true);
    DeviceMem in_buf(sizeof(T) * in.mDesc.GetElementSpace()), wei_buf(sizeof(T) * wei.mDesc.GetElementSpace()),
        out_buf(sizeof(T) * out_d.mDesc.GetElementSpace());
    in_buf.ToDevice(in.mData.data());
    wei_buf.ToDevice(wei.mData.data());
    std::vector<std::unique_ptr<dev::DeviceConvFwd<PassThrough, PassThrough, PassThrough>>> ops;
    ops.push_back(std::make_unique<Conv>());
    Best best;
    bool pass = true;
    for(auto& op : ops)
    {
        auto arg = op->MakeArgumentPointer(in_buf.GetDeviceBuffer(), wei_buf.GetDeviceBuffer(), out_buf.GetDeviceBuffer(),
                                           p.N_, p.K_, p.C_, p.input_spatial_lengths_, p.filter_spatial_lengths_, out_sp,
                                           p.conv_filter_strides_, p.conv_filter_dilations_, p.input_left_pads_,
                                           p.input_right_pads_, {}, {}, {});
        if(!op->IsSupportedArgument(arg.get()))
        {
            std::cout << op->GetTypeString() << " does not support this problem" << std::endl;
            continue;
        }
        const float ms = op->MakeInvokerPointer()->Run(arg.get(), StreamConfig{nullptr, time});
        if(time)
            best.offer(op->GetTypeString() + " [" + op->GetBackendString() + "]", ms, conv_util::get_flops(p.N_, p.C_, p.K_, p.filter_spatial_lengths_, out_sp),
                       conv_util::get_btype<T, T, T>(p.N_, p.C_, p.K_, p.input_spatial_lengths_,
                                                     p.filter_spatial_lengths_, out_sp));
        else
            best.name = op->GetTypeString() + " [" + op->GetBackendString() + "]";
        if(verify)
        {
            out_buf.FromDevice(out_d.mData.data());
            using Ref = ck::tensor_operation::host::ReferenceConvFwd<T, T, T, PassThrough, PassThrough, PassThrough, ND>;
            auto rarg = Ref::MakeArgument(in, wei, out_h, p.conv_filter_strides_, p.conv_filter_dilations_,
                                          p.input_left_pads_, p.input_right_pads_, {}, {}, {});
            Ref::MakeInvoker().Run(rarg);
            pass = pass && ck::utils::check_err(out_d.mData, out_h.mData);
        }
    }
    best.report("conv_fwd");
    return pass && !best.name.empty();
}

int profile_convnd_fwd(int argc, char* argv[])
{
    const int nd = argc > 8 ? std::stoi(argv[8]) : 0;
    if(nd < 1 || nd > 3 || argc != 9 + 3 + 6 * nd || std::stoi(argv[3]) != 1)
    {
        std::printf("conv_fwd <dtype 1 fp16|2 bf16|3 int8> <layout 1: NHWC> verify init log time <nd 1|2|3> N K C "
                    "<filter> <input> <strides> <dilations> <left pads> <right pads>\n");
        return 1;
    }
    const int dtype = std::stoi(argv[2]);
    const bool verify = std::stoi(argv[4]), time = std::stoi(argv[7]);
    const int init = std::stoi(argv[5]);
    const auto p   = ck::utils::conv::parse_conv_params(nd, 9, argv);
    auto by_type   = [&](auto ndc) {
        constexpr int ND = decltype(ndc)::value;
        return dtype == 1 ? profile_convnd_typed<ND, ck::half_t>(p, verify, init, time)
                          : dtype == 2 ? profile_convnd_typed<ND, ck::bhalf_t>(p, verify, init, time)
                                       : dtype == 3 ? profile_convnd_typed<ND, int8_t>(p, verify, init, time) : false;
    };
    const bool ok = nd == 1 ? by_type(std::integral_constant<int, 1>{})
                            : nd == 2 ? by_type(std::integral_constant<int, 2>{}) : by_type(std::integral_constant<int, 3>{});
    return ok ? 0 : 1;
}

int main(int argc, char* argv[])
{
    if(argc >= 2)
    {
        if(std::strcmp(argv[1], "gemm") == 0)
            return profile_gemm(argc, argv);
        if(std::strcmp(argv[1], "gemm_add_add_fastgelu") == 0)
            return profile_gemm_add_add_fastgelu(argc, argv);
        if(std::strcmp(argv[1], "grouped_gemm") == 0)
            return profile_grouped_gemm(argc, argv);
        if(std::strcmp(argv[1], "conv_fwd_bias_relu") == 0)
            return profile_conv_fwd_bias_relu(argc, argv);
        if(std::strcmp(argv[1], "conv_fwd_bias_relu_add") == 0)
            return profile_conv_fwd_bias_relu_add(argc, argv);
        if(std::strcmp(argv[1], "conv_fwd") == 0)
            return profile_convnd_fwd(argc, argv);
        if(std::strcmp(argv[1], "batched_gemm") == 0)
            return profile_batched_gemm(argc, argv);
        if(std::strcmp(argv[1], "gemm_bilinear") == 0)
            return profile_gemm_bilinear_splitk(argc, argv, true);
        if(std::strcmp(argv[1], "gemm_splitk") == 0)
            return profile_gemm_bilinear_splitk(argc, argv, false);
    }
    std::printf("arg1: tensor operation (gemm: GEMM\n"
                "                        gemm_add_add_fastgelu: GEMM+Add+Add+FastGeLU\n"
                "                        grouped_gemm: Grouped GEMM\n"
                "                        conv_fwd_bias_relu: ForwardConvolution+Bias+ReLU\n"
                "                        conv_fwd_bias_relu_add: ForwardConvolution+Bias+ReLU+Add\n"
                "                        conv_fwd: ForwardConvolution 1-D / 2-D / 3-D\n"
                "                        batched_gemm: Batched GEMM\n"
                "                        gemm_bilinear: GEMM+Bilinear\n"
                "                        gemm_splitk: Split-K GEMM)\n");
    return 0;
}
