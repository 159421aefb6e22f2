// conv2d forward + bias + ReLU (NHWC / KYXC / NHWK, fp16) in the style of the reference's
// example/06_conv2d_fwd_bias_relu/conv2d_fwd_xdl_bias_relu.cpp; with the first extra flag set to 0 the plain
// convolution of example/09_convnd_fwd (DeviceConvNDFwdXdl..., PassThrough output op); with it set to 2 the
// bias + ReLU + residual add of example/07_conv2d_fwd_bias_relu_add (AddReluAdd output op).
//   usage: conv2d_fwd_xdl_bias_relu [verify init time [mode [N K C Y X Hi Wi Sy Sx Dy Dx LeftPy LeftPx RightPy RightPx]]]
//   default problem: ConvParams{} = N128 K256 C192, 3x3, 71x71, stride 2, dilation 1, pad 1.
#include "example_common.hpp"

#include "ck/library/reference_tensor_operation/cpu/reference_conv_fwd.hpp"
#include "ck/library/reference_tensor_operation/cpu/reference_conv_fwd_bias_activation.hpp"
#include "ck/library/reference_tensor_operation/cpu/reference_conv_fwd_bias_activation_add.hpp"
#include "ck/library/utility/check_err.hpp"
#include "ck/library/utility/conv_util.hpp"
#include "ck/tensor_operation/gpu/device/device_conv2d_fwd_xdl_c_shuffle_bias_activation_nhwc_kyxc_nhwk.hpp"
#include "ck/tensor_operation/gpu/device/device_conv2d_fwd_xdl_c_shuffle_bias_activation_add_nhwc_kyxc_nhwk.hpp"
#include "ck/tensor_operation/gpu/device/device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp"
#include "ck/tensor_operation/gpu/element/element_wise_operation.hpp"

template <ck::index_t... Is>
using S = ck::Sequence<Is...>;

using InDataType  = ck::half_t;
using WeiDataType = ck::half_t;
using OutDataType = ck::half_t;
using AccDataType = float;

using PassThrough = ck::tensor_operation::element_wise::PassThrough;
using AddRelu     = ck::tensor_operation::element_wise::AddRelu;
using AddReluAdd  = ck::tensor_operation::element_wise::AddReluAdd;

static constexpr auto MemorySet      = ck::InMemoryDataOperationEnum::Set;
static constexpr auto ConvFwdDefault = ck::tensor_operation::device::ConvolutionForwardSpecialization::Default;

// clang-format off
using DeviceConvBiasReluInstance = ck::tensor_operation::device::
    DeviceConv2dFwdXdl_C_Shuffle_Bias_Activation_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<
        InDataType, WeiDataType, OutDataType, AccDataType, PassThrough, PassThrough, AddRelu, MemorySet, ConvFwdDefault,
        256, 128, 256, 4, 8, 32, 32, 2, 4, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true,
        S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true, 1, 1, S<1, 1, 32, 1, 1, 8>, 8>;
using DeviceConvBiasReluAddInstance = ck::tensor_operation::device::
    DeviceConv2dFwdXdl_C_Shuffle_Bias_Activation_Add_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<
        InDataType, WeiDataType, OutDataType, AccDataType, PassThrough, PassThrough, AddReluAdd, ConvFwdDefault,
        256, 128, 256, 4, 8, 32, 32, 2, 4, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true,
        S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true, 1, 1, S<1, 1, 32, 1, 1, 8>, 8>;
using DeviceConvInstance = ck::tensor_operation::device::
    DeviceConvNDFwdXdl_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<
        InDataType, WeiDataType, OutDataType, AccDataType, PassThrough, PassThrough, PassThrough, ConvFwdDefault, 2,
        256, 128, 256, 4, 8, 32, 32, 2, 4, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true,
        S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true, 7, 1>;
// clang-format on

int main(int argc, char* argv[])
{
    namespace conv_util = ck::utils::conv;
    example::RunFlags flags;
    int mode = 1; // 0 plain, 1 bias + ReLU, 2 bias + ReLU + residual
    conv_util::ConvParams params;
    const int first = example::parse_flags(argc, argv, flags);
    if(argc >= 5)
        mode = std::stoi(argv[first]);
    const bool with_bias = mode != 0, with_resi = mode == 2;
    if(argc == 20)
        params = conv_util::parse_conv_params(2, first + 1, argv);
    else if(argc != 1 && argc != 4 && argc != 5)
        example::usage_and_exit("arg4: 1 = bias + ReLU, 0 = plain, 2 = bias + ReLU + residual add; arg5 to 19: N, K, C, Y, X, Hi, Wi, Sy, Sx, Dy, Dx, "
                                "LeftPy, LeftPx, RightPy, RightPx");

    const std::vector<ck::index_t> out_sp = params.GetOutputSpatialLengths();
    const std::size_t N = params.N_, K = params.K_, C = params.C_;
    std::vector<std::size_t> in_dims{N, C}, wei_dims{K, C}, out_dims{N, K};
    for(int i = 0; i < 2; ++i)
    {
        in_dims.push_back(params.input_spatial_lengths_[i]);
        wei_dims.push_back(params.filter_spatial_lengths_[i]);
        out_dims.push_back(out_sp[i]);
    }
    // NCHW-ordered lengths with NHWC strides, as the reference's host descriptors
    Tensor<InDataType> input(conv_util::get_input_host_tensor_descriptor(in_dims));
    Tensor<WeiDataType> weights(conv_util::get_filters_host_tensor_descriptor(wei_dims));
    Tensor<OutDataType> host_output(conv_util::get_output_host_tensor_descriptor(out_dims));
    Tensor<OutDataType> device_output(conv_util::get_output_host_tensor_descriptor(out_dims));
    Tensor<OutDataType> bias(HostTensorDescriptor(std::vector<std::size_t>{K}));
    Tensor<OutDataType> resi(conv_util::get_output_host_tensor_descriptor(out_dims)); // residual, laid out like the output
    std::cout << "input: " << input.mDesc << "\nweights: " << weights.mDesc << "\noutput: " << host_output.mDesc
              << "\nbias: " << bias.mDesc << std::endl;

    if(flags.init_method == 1)
    {
        input.GenerateTensorValue(GeneratorTensor_2<InDataType>{-5, 5});
        weights.GenerateTensorValue(GeneratorTensor_2<WeiDataType>{-5, 5});
        bias.GenerateTensorValue(GeneratorTensor_2<OutDataType>{-5, 5});
        resi.GenerateTensorValue(GeneratorTensor_2<OutDataType>{-5, 5});
    }
    else if(flags.init_method == 2)
    {
        input.GenerateTensorValue(GeneratorTensor_3<InDataType>{0.0, 1.0});
        weights.GenerateTensorValue(GeneratorTensor_3<WeiDataType>{-0.5, 0.5});
        bias.GenerateTensorValue(GeneratorTensor_3<OutDataType>{0.0, 1.0});
        resi.GenerateTensorValue(GeneratorTensor_3<OutDataType>{0.0, 1.0});
    }

    DeviceMem in_buf(sizeof(InDataType) * input.mDesc.GetElementSpace());
    DeviceMem wei_buf(sizeof(WeiDataType) * weights.mDesc.GetElementSpace());
    DeviceMem out_buf(sizeof(OutDataType) * device_output.mDesc.GetElementSpace());
    DeviceMem bias_buf(sizeof(OutDataType) * bias.mDesc.GetElementSpace());
    in_buf.ToDevice(input.mData.data());
    wei_buf.ToDevice(weights.mData.data());
    bias_buf.ToDevice(bias.mData.data());
    DeviceMem resi_buf(with_resi ? sizeof(OutDataType) * resi.mDesc.GetElementSpace() : 16);
    if(with_resi)
        resi_buf.ToDevice(resi.mData.data());

    float ave_time = 0;
    std::string type_string;
    if(with_resi)
    {
        auto conv     = DeviceConvBiasReluAddInstance{};
        auto invoker  = conv.MakeInvoker();
        auto argument = conv.MakeArgument(
            static_cast<const InDataType*>(in_buf.GetDeviceBuffer()), static_cast<const WeiDataType*>(wei_buf.GetDeviceBuffer()),
            static_cast<OutDataType*>(out_buf.GetDeviceBuffer()), static_cast<const OutDataType*>(bias_buf.GetDeviceBuffer()),
            static_cast<const OutDataType*>(resi_buf.GetDeviceBuffer()), params.N_, params.K_, params.C_,
            params.input_spatial_lengths_, params.filter_spatial_lengths_, out_sp, params.conv_filter_strides_,
            params.conv_filter_dilations_, params.input_left_pads_, params.input_right_pads_, PassThrough{}, PassThrough{},
            AddReluAdd{});
        if(!conv.IsSupportedArgument(argument))
            throw std::runtime_error("wrong! device operator with the specified compilation parameters does "
                                     "not support this problem");
        ave_time    = invoker.Run(argument, StreamConfig{nullptr, flags.time_kernel});
        type_string = conv.GetTypeString();
    }
    else if(with_bias)
    {
        auto conv     = DeviceConvBiasReluInstance{};
        auto invoker  = conv.MakeInvoker();
        auto argument = conv.MakeArgument(
            static_cast<const InDataType*>(in_buf.GetDeviceBuffer()), static_cast<const WeiDataType*>(wei_buf.GetDeviceBuffer()),
            static_cast<OutDataType*>(out_buf.GetDeviceBuffer()), static_cast<const OutDataType*>(bias_buf.GetDeviceBuffer()),
            params.N_, params.K_, params.C_, params.input_spatial_lengths_, params.filter_spatial_lengths_, out_sp,
            params.conv_filter_strides_, params.conv_filter_dilations_, params.input_left_pads_, params.input_right_pads_,
            PassThrough{}, PassThrough{}, AddRelu{});
        if(!conv.IsSupportedArgument(argument))
            throw std::runtime_error("wrong! device operator with the specified compilation parameters does "
                                     "not support this problem");
        ave_time    = invoker.Run(argument, StreamConfig{nullptr, flags.time_kernel});
        type_string = conv.GetTypeString();
    }
    else
    {
        auto conv     = DeviceConvInstance{};
        auto invoker  = conv.MakeInvoker();
        auto argument = conv.MakeArgument(
            static_cast<const InDataType*>(in_buf.GetDeviceBuffer()), static_cast<const WeiDataType*>(wei_buf.GetDeviceBuffer()),
            static_cast<OutDataType*>(out_buf.GetDeviceBuffer()), params.N_, params.K_, params.C_,
            params.input_spatial_lengths_, params.filter_spatial_lengths_, out_sp, params.conv_filter_strides_,
            params.conv_filter_dilations_, params.input_left_pads_, params.input_right_pads_, PassThrough{}, PassThrough{},
            PassThrough{});
        if(!conv.IsSupportedArgument(argument))
            throw std::runtime_error("wrong! device operator with the specified compilation parameters does "
                                     "not support this problem");
        ave_time    = invoker.Run(argument, StreamConfig{nullptr, flags.time_kernel});
        type_string = conv.GetTypeString();
    }
    if(flags.time_kernel)
    {
        const std::size_t flop = conv_util::get_flops(params.N_, params.C_, params.K_, params.filter_spatial_lengths_, out_sp);
        const std::size_t num_btype =
            conv_util::get_btype<InDataType, WeiDataType, OutDataType>(params.N_, params.C_, params.K_,
                                                                       params.input_spatial_lengths_,
                                                                       params.filter_spatial_lengths_, out_sp) +
            (with_bias ? sizeof(OutDataType) * K : 0) +
            (with_resi ? sizeof(OutDataType) * resi.mDesc.GetElementSize() : 0);
        example::print_perf(ave_time, flop, num_btype, type_string);
    }
    out_buf.FromDevice(device_output.mData.data());

    if(flags.do_verification)
    {
        if(with_resi)
        {
            using Ref = ck::tensor_operation::host::ReferenceConvFwd_Bias_Activation_Add<InDataType, WeiDataType, OutDataType,
                                                                                         PassThrough, PassThrough, AddReluAdd>;
            auto ref_conv = Ref{};
            auto ref_inv  = ref_conv.MakeInvoker();
            auto ref_arg  = ref_conv.MakeArgument(input, weights, host_output, bias, resi, params.conv_filter_strides_,
                                                  params.conv_filter_dilations_, params.input_left_pads_,
                                                  params.input_right_pads_, PassThrough{}, PassThrough{}, AddReluAdd{});
            ref_inv.Run(ref_arg);
        }
        else if(with_bias)
        {
            using Ref = ck::tensor_operation::host::ReferenceConvFwd_Bias_Activation<InDataType, WeiDataType, OutDataType,
                                                                                     PassThrough, PassThrough, AddRelu>;
            auto ref_conv = Ref{};
            auto ref_inv  = ref_conv.MakeInvoker();
            auto ref_arg  = ref_conv.MakeArgument(input, weights, host_output, bias, params.conv_filter_strides_,
                                                  params.conv_filter_dilations_, params.input_left_pads_,
                                                  params.input_right_pads_, PassThrough{}, PassThrough{}, AddRelu{});
            ref_inv.Run(ref_arg);
        }
        else
        {
            using Ref = ck::tensor_operation::host::ReferenceConvFwd<InDataType, WeiDataType, OutDataType, PassThrough,
                                                                     PassThrough, PassThrough, 2>;
            auto ref_conv = Ref{};
            auto ref_inv  = ref_conv.MakeInvoker();
            auto ref_arg  = ref_conv.MakeArgument(input, weights, host_output, params.conv_filter_strides_,
                                                  params.conv_filter_dilations_, params.input_left_pads_,
                                                  params.input_right_pads_, PassThrough{}, PassThrough{}, PassThrough{});
            ref_inv.Run(ref_arg);
        }
        return ck::utils::check_err(device_output.mData, host_output.mData) ? 0 : 1;
    }
    return 0;
}
