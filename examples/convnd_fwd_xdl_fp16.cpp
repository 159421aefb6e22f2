// N-dimensional fp16 forward convolution (NWC / NHWC / NDHWC) in the style of the reference's
// example/09_convnd_fwd/convnd_fwd_xdl_fp16.cpp: the number of spatial dimensions is a run-time argument that picks
// one of three instances of the device operation through a DeviceConvFwdPtr.
//   usage: convnd_fwd_xdl_fp16 [verify init time nd [N K C <filter> <input> <strides> <dilations> <left pads> <right pads>]]
//   (nd values per bracketed group; without a problem the reference's default ConvParams are used)
#include "example_common.hpp"

#include "ck/library/reference_tensor_operation/cpu/reference_conv_fwd.hpp"
#include "ck/library/utility/check_err.hpp"
#include "ck/library/utility/conv_util.hpp"
#include "ck/tensor_operation/gpu/device/device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp"
#include "ck/tensor_operation/gpu/element/element_wise_operation.hpp"

template <ck::index_t... Is>
using S = ck::Sequence<Is...>;
#ifndef CONVND_EXAMPLE_TYPES // convnd_fwd_xdl_int8.cpp defines the four types itself and includes this file
using InDataType  = ck::half_t;
using WeiDataType = ck::half_t;
using OutDataType = ck::half_t;
using AccDataType = float;
#endif
using InElementOp  = ck::tensor_operation::element_wise::PassThrough;
using WeiElementOp = ck::tensor_operation::element_wise::PassThrough;
using OutElementOp = ck::tensor_operation::element_wise::PassThrough;

static constexpr auto ConvFwdDefault = ck::tensor_operation::device::ConvolutionForwardSpecialization::Default;

using DeviceConvFwdBasePtr = ck::tensor_operation::device::DeviceConvFwdPtr<InElementOp, WeiElementOp, OutElementOp>;

// clang-format off
template <ck::index_t NumDimSpatial>
using DeviceConvNDFwdInstance = ck::tensor_operation::device::DeviceConvNDFwdXdl_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<
    InDataType, WeiDataType, OutDataType, AccDataType, InElementOp, WeiElementOp, OutElementOp, ConvFwdDefault, NumDimSpatial,
    256, 128, 256, 4, 8, 32, 32, 2, 4, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true, 7, 1>;
// clang-format on

template <ck::index_t NumDimSpatial>
using ReferenceConvNDFwdInstance =
    ck::tensor_operation::host::ReferenceConvFwd<InDataType, WeiDataType, OutDataType, InElementOp, WeiElementOp,
                                                 OutElementOp, NumDimSpatial>;

DeviceConvFwdBasePtr get_conv_instance(int num_dim_spatial)
{
    switch(num_dim_spatial)
    {
    case 3: return std::make_unique<DeviceConvNDFwdInstance<3>>();
    case 2: return std::make_unique<DeviceConvNDFwdInstance<2>>();
    case 1: return std::make_unique<DeviceConvNDFwdInstance<1>>();
    default: throw std::runtime_error("Unsupported number of spatial dimensions provided!");
    }
}

int main(int argc, char* argv[])
{
    namespace conv_util = ck::utils::conv;
    example::RunFlags flags;
    int num_dim_spatial = 2;
    conv_util::ConvParams params;
    if(argc >= 5)
    {
        example::parse_flags(argc, argv, flags);
        num_dim_spatial = std::stoi(argv[4]);
    }
    if(num_dim_spatial < 1 || num_dim_spatial > 3 || (argc != 1 && argc != 5 && argc != 5 + 3 + 6 * num_dim_spatial))
        example::usage_and_exit("arg4: number of spatial dimensions (1, 2 or 3)\n"
                                "then N, K, C, <filter>, <input>, <strides>, <dilations>, <left pads>, <right pads>");
    if(argc >= 6)
        params = conv_util::parse_conv_params(num_dim_spatial, 5, argv);
    else if(num_dim_spatial != 2)
    {
        // the default ConvParams describe a 2-D problem; keep its extents for the first nd dimensions
        params.num_dim_spatial_ = num_dim_spatial;
        const int nd = num_dim_spatial;
        params.filter_spatial_lengths_.assign(nd, 3);
        params.input_spatial_lengths_.assign(nd, nd == 3 ? 16 : 71);
        params.conv_filter_strides_.assign(nd, 2);
        params.conv_filter_dilations_.assign(nd, 1);
        params.input_left_pads_.assign(nd, 1);
        params.input_right_pads_.assign(nd, 1);
    }

    const std::vector<ck::index_t> out_spatial = params.GetOutputSpatialLengths();
    std::vector<std::size_t> in_dims{std::size_t(params.N_), std::size_t(params.C_)};
    std::vector<std::size_t> wei_dims{std::size_t(params.K_), std::size_t(params.C_)};
    std::vector<std::size_t> out_dims{std::size_t(params.N_), std::size_t(params.K_)};
    in_dims.insert(in_dims.end(), params.input_spatial_lengths_.begin(), params.input_spatial_lengths_.end());
    wei_dims.insert(wei_dims.end(), params.filter_spatial_lengths_.begin(), params.filter_spatial_lengths_.end());
    out_dims.insert(out_dims.end(), out_spatial.begin(), out_spatial.end());

    Tensor<InDataType> input(conv_util::get_input_host_tensor_descriptor(in_dims, num_dim_spatial));
    Tensor<WeiDataType> weights(conv_util::get_filters_host_tensor_descriptor(wei_dims, num_dim_spatial));
    Tensor<OutDataType> host_output(conv_util::get_output_host_tensor_descriptor(out_dims, num_dim_spatial));
    Tensor<OutDataType> device_output(host_output.mDesc);
    std::cout << "input: " << input.mDesc << "\nweights: " << weights.mDesc << "\noutput: " << host_output.mDesc
              << std::endl;

    if(flags.init_method == 1)
    {
        input.GenerateTensorValue(GeneratorTensor_2<InDataType>{-5, 5});
        weights.GenerateTensorValue(GeneratorTensor_2<WeiDataType>{-5, 5});
    }
    else if(flags.init_method != 0)
    {
        input.GenerateTensorValue(GeneratorTensor_3<InDataType>{0.0, 1.0});
        weights.GenerateTensorValue(GeneratorTensor_3<WeiDataType>{-0.5, 0.5});
    }

    DeviceMem in_buf(sizeof(InDataType) * input.mDesc.GetElementSpace());
    DeviceMem wei_buf(sizeof(WeiDataType) * weights.mDesc.GetElementSpace());
    DeviceMem out_buf(sizeof(OutDataType) * device_output.mDesc.GetElementSpace());
    in_buf.ToDevice(input.mData.data());
    wei_buf.ToDevice(weights.mData.data());

    auto conv     = get_conv_instance(num_dim_spatial);
    auto invoker  = conv->MakeInvokerPointer();
    auto argument = conv->MakeArgumentPointer(in_buf.GetDeviceBuffer(), wei_buf.GetDeviceBuffer(), out_buf.GetDeviceBuffer(),
                                              params.N_, params.K_, params.C_, params.input_spatial_lengths_,
                                              params.filter_spatial_lengths_, out_spatial, params.conv_filter_strides_,
                                              params.conv_filter_dilations_, params.input_left_pads_,
                                              params.input_right_pads_, InElementOp{}, WeiElementOp{}, OutElementOp{});
    if(!conv->IsSupportedArgument(argument.get()))
        throw std::runtime_error("wrong! device_conv with the specified compilation parameters does "
                                 "not support this Conv problem");

    const float ave_time = invoker->Run(argument.get(), StreamConfig{nullptr, flags.time_kernel});
    if(flags.time_kernel)
        example::print_perf(ave_time,
                            conv_util::get_flops(params.N_, params.C_, params.K_, params.filter_spatial_lengths_, out_spatial),
                            conv_util::get_btype<InDataType, WeiDataType, OutDataType>(
                                params.N_, params.C_, params.K_, params.input_spatial_lengths_,
                                params.filter_spatial_lengths_, out_spatial),
                            conv->GetTypeString());

    if(flags.do_verification)
    {
        auto verify = [&](auto ref_conv) {
            auto ref_invoker  = ref_conv.MakeInvoker();
            auto ref_argument = ref_conv.MakeArgument(input, weights, host_output, params.conv_filter_strides_,
                                                      params.conv_filter_dilations_, params.input_left_pads_,
                                                      params.input_right_pads_, InElementOp{}, WeiElementOp{},
                                                      OutElementOp{});
            ref_invoker.Run(ref_argument);
            out_buf.FromDevice(device_output.mData.data());
            // Integer-valued inputs give exact sums: the reference example's tight bounds (rtol 1e-5, atol 1e-4)
            // apply.  Decimal inputs are summed in a different order on the device, which can move the single
            // rounding to binary16 by one ulp: there the binary16 defaults of check_err (1e-3) apply.
            if(flags.init_method == 1)
                return ck::utils::check_err(host_output.mData, device_output.mData, "Error: incorrect results!", 1e-5f,
                                            1e-4f) ? 0 : 1;
            return ck::utils::check_err(host_output.mData, device_output.mData) ? 0 : 1;
        };
        switch(num_dim_spatial)
        {
        case 3: return verify(ReferenceConvNDFwdInstance<3>());
        case 2: return verify(ReferenceConvNDFwdInstance<2>());
        default: return verify(ReferenceConvNDFwdInstance<1>());
        }
    }
    return 0;
}
