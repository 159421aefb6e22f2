// The reference's device test of the N-D forward convolution in its own style
// (test/convnd_fwd/conv{1,2,3}d_fwd.cpp:24-98): a ConvFwdOpInstance describes the problem, OpInstanceRunEngine
// uploads it, computes the expected output with the N-D ReferenceConvFwd and Test()s every device operation of a list.
//   usage: convnd_fwd_instance_engine <nd 1|2|3> [oddc]
// With `oddc` (2-D only) the problem is the reference's odd-channel case (test/convnd_fwd/conv2d_fwd.cpp:110-111, C = 3)
// and the instance one whose operand loads are one element wide, the only width the reference's vector rule accepts there.
#include <functional>
#include <iostream>
#include <string>

#include "ck/ck.hpp"
#include "ck/library/reference_tensor_operation/cpu/reference_conv_fwd.hpp"
#include "ck/library/utility/conv_util.hpp"
#include "ck/library/utility/fill.hpp"
#include "ck/library/utility/op_instance_engine.hpp"
#include "ck/tensor_operation/gpu/device/device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp"

template <ck::index_t... Is>
using S           = ck::Sequence<Is...>;
using PassThrough = ck::tensor_operation::element_wise::PassThrough;
namespace dev     = ck::tensor_operation::device;
namespace ctl     = ck::tensor_layout::convolution;
using namespace ck::utils;

template <int ND, typename T>
void reference_conv(const conv::ConvParams& p, const Tensor<T>& in, const Tensor<T>& wei, Tensor<T>& out)
{
    using Ref = ck::tensor_operation::host::ReferenceConvFwd<T, T, T, PassThrough, PassThrough, PassThrough, ND>;
    auto arg  = Ref::MakeArgument(in, wei, out, p.conv_filter_strides_, p.conv_filter_dilations_, p.input_left_pads_,
                                  p.input_right_pads_, {}, {}, {});
    Ref::MakeInvoker().Run(arg);
}

template <int ND, typename T, typename InL, typename WeiL, typename OutL, ck::index_t LoadWidth = 8>
bool run(const conv::ConvParams& params)
{
    // clang-format off
    using Conv = dev::DeviceConvNDFwdXdl_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<
        T, T, T, float, PassThrough, PassThrough, PassThrough, dev::ConvolutionForwardSpecialization::Default, ND,
        256, 128, 256, 4, 8, 32, 32, 2, 4, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, LoadWidth, LoadWidth, true,
        S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, LoadWidth, LoadWidth, true, 7, 1>;
    // clang-format on
    std::vector<dev::DeviceConvFwdPtr<PassThrough, PassThrough, PassThrough>> conv_ptrs;
    conv_ptrs.push_back(std::make_unique<Conv>());
    conv::ConvFwdOpInstance<T, T, T, InL, WeiL, OutL, PassThrough, PassThrough, PassThrough,
                            FillUniformDistributionIntegerValue<T>, FillUniformDistributionIntegerValue<T>>
        instance(params, true, FillUniformDistributionIntegerValue<T>{}, FillUniformDistributionIntegerValue<T>{});
    using namespace std::placeholders;
    auto reference = std::bind(reference_conv<ND, T>, params, _1, _2, _3);
    OpInstanceRunEngine<T, T, T> engine(instance, reference);
    engine.SetAtol(1e-3);
    engine.SetRtol(1e-3);
    const bool ok   = engine.Test(conv_ptrs);
    const auto best = engine.Profile(conv_ptrs, true, true);
    std::cout << "Best: " << best.best_avg_time << " ms, " << best.best_tflops << " TFlops, " << best.best_op_name << std::endl;
    return ok && !best.best_op_name.empty();
}

int main(int argc, char* argv[])
{
    const int nd = argc > 1 ? std::stoi(argv[1]) : 2;
    bool ok      = false;
    // the default problems of test/convnd_fwd/conv1d_fwd.cpp:73, conv2d_fwd.cpp:104, conv3d_fwd.cpp:76
    if(nd == 2 && argc > 2 && std::string(argv[2]) == "oddc")
        ok = run<2, ck::half_t, ctl::NHWC, ctl::KYXC, ctl::NHWK, 1>(
            conv::ConvParams{2, 4, 256, 3, {3, 3}, {28, 28}, {1, 1}, {1, 1}, {0, 0}, {0, 0}});
    else if(nd == 1)
        ok = run<1, ck::half_t, ctl::NWC, ctl::KXC, ctl::NWK>(conv::ConvParams{1, 4, 256, 64, {3}, {71}, {2}, {2}, {2}, {2}});
    else if(nd == 2)
        ok = run<2, ck::half_t, ctl::NHWC, ctl::KYXC, ctl::NHWK>(
            conv::ConvParams{2, 4, 256, 64, {3, 3}, {36, 36}, {2, 2}, {2, 2}, {2, 2}, {2, 2}});
    else if(nd == 3)
        ok = run<3, ck::half_t, ctl::NDHWC, ctl::KZYXC, ctl::NDHWK>(
            conv::ConvParams{3, 4, 256, 64, {3, 3, 3}, {18, 18, 18}, {1, 1, 1}, {2, 2, 2}, {2, 2, 2}, {2, 2, 2}});
    std::cout << (ok ? "PASSED" : "FAILED") << std::endl;
    return ok ? 0 : 1;
}
