// Operation-instance run engine with the reference's interface
// (library/include/ck/library/utility/op_instance_engine.hpp:25-246 and the ConvFwdOpInstance of
// library/include/ck/library/utility/conv_util.hpp:399-570): an OpInstance describes one problem (its host tensors,
// how to build the argument of a device operation for it, its flop / byte counts); the engine uploads the inputs
// once, optionally computes a reference output with a caller-supplied functor, and then runs every device operation
// of a list against the problem - Test() verifies, Profile() times and reports the best one.
#pragma once
#include <functional>
#include <iostream>
#include <limits>
#include <memory>
#include <stdexcept>
#include <string>
#include <tuple>
#include <type_traits>
#include <utility>
#include <vector>

#include "ck/b200/device_ops.hpp"
#include "ck/b200/host_tensor.hpp"
#include "ck/b200/host_utility.hpp"

namespace ck {
namespace utils {

struct ProfileBestConfig
{
    std::string best_op_name;
    float best_avg_time   = std::numeric_limits<float>::max();
    float best_tflops     = std::numeric_limits<float>::max();
    float best_gb_per_sec = std::numeric_limits<float>::max();
};

template <typename OutDataType, typename... InArgTypes>
class OpInstance
{
    public:
    template <typename T>
    using TensorPtr      = std::unique_ptr<Tensor<T>>;
    using InTensorsTuple = std::tuple<TensorPtr<InArgTypes>...>;
    using DeviceMemPtr   = std::unique_ptr<DeviceMem>;
    using DeviceBuffers  = std::vector<DeviceMemPtr>;

    virtual ~OpInstance() {}
    virtual InTensorsTuple GetInputTensors() const         = 0;
    virtual TensorPtr<OutDataType> GetOutputTensor() const = 0;
    virtual std::unique_ptr<tensor_operation::device::BaseInvoker>
    MakeInvokerPointer(tensor_operation::device::BaseOperator*) const = 0;
    virtual std::unique_ptr<tensor_operation::device::BaseArgument>
    MakeArgumentPointer(tensor_operation::device::BaseOperator*, const DeviceBuffers&, const DeviceMemPtr&) const = 0;
    virtual std::size_t GetFlops() const = 0;
    virtual std::size_t GetBtype() const = 0;
};

template <typename OutDataType, typename... InArgTypes>
class OpInstanceRunEngine
{
    public:
    using OpInstanceT = OpInstance<InArgTypes..., OutDataType>; // the reference spells the argument order this way
    template <typename T>
    using TensorPtr      = std::unique_ptr<Tensor<T>>;
    using DeviceMemPtr   = std::unique_ptr<DeviceMem>;
    using InTensorsTuple = std::tuple<TensorPtr<InArgTypes>...>;
    using DeviceBuffers  = std::vector<DeviceMemPtr>;

    // reference_op(const Tensor<In>&..., Tensor<Out>&) fills the expected output; without one Test() throws.
    template <typename ReferenceOp = std::function<void()>>
    OpInstanceRunEngine(const OpInstanceT& op_instance, const ReferenceOp& reference_op = ReferenceOp{},
                        bool do_verification = true)
        : op_instance_{op_instance}
    {
        in_tensors_ = op_instance_.GetInputTensors();
        out_tensor_ = op_instance_.GetOutputTensor();
        if constexpr(std::is_invocable_v<ReferenceOp, const Tensor<InArgTypes>&..., Tensor<OutDataType>&>)
        {
            if(do_verification)
            {
                ref_output_ = op_instance_.GetOutputTensor();
                std::apply([&](const auto&... in) { reference_op(*in..., *ref_output_); }, in_tensors_);
            }
        }
        std::apply([&](const auto&... in) { (upload(*in), ...); }, in_tensors_);
        out_device_buffer_ = std::make_unique<DeviceMem>(sizeof(OutDataType) * out_tensor_->mDesc.GetElementSpace());
        out_device_buffer_->SetZero();
    }
    virtual ~OpInstanceRunEngine() {}

    template <typename OpInstancePtr>
    bool Test(const std::vector<OpInstancePtr>& op_ptrs)
    {
        bool res = true;
        for(auto& op_ptr : op_ptrs)
        {
            auto invoker  = op_instance_.MakeInvokerPointer(op_ptr.get());
            auto argument = op_instance_.MakeArgumentPointer(op_ptr.get(), in_device_buffers_, out_device_buffer_);
            if(!op_ptr->IsSupportedArgument(argument.get()))
            {
                std::cout << "Given problem is not supported by instance: \n\t>>>>" << op_ptr->GetTypeString() << std::endl;
                continue;
            }
            std::cout << "Testing instance: " << op_ptr->GetTypeString() << std::endl;
            invoker->Run(argument.get());
            out_device_buffer_->FromDevice(out_tensor_->mData.data());
            if(!ref_output_)
                throw std::runtime_error("OpInstanceRunEngine::Test: Reference value not availabe."
                                         " You have to provide reference function.");
            const bool ok = check(out_tensor_->mData, ref_output_->mData);
            std::cout << (ok ? "SUCCESS" : "FAILURE") << std::endl;
            res = res && ok;
            out_device_buffer_->SetZero();
        }
        return res;
    }

    template <typename OpInstancePtr>
    ProfileBestConfig Profile(const std::vector<OpInstancePtr>& op_ptrs, bool time_kernel = false,
                              bool do_verification = false, bool /*do_log*/ = false)
    {
        ProfileBestConfig best;
        for(auto& op_ptr : op_ptrs)
        {
            auto invoker  = op_instance_.MakeInvokerPointer(op_ptr.get());
            auto argument = op_instance_.MakeArgumentPointer(op_ptr.get(), in_device_buffers_, out_device_buffer_);
            if(!op_ptr->IsSupportedArgument(argument.get()))
                continue;
            const std::string name = op_ptr->GetTypeString();
            const float avg_time   = invoker->Run(argument.get(), StreamConfig{nullptr, time_kernel});
            const float tflops     = static_cast<float>(op_instance_.GetFlops()) / 1.E9 / avg_time;
            const float gb_per_sec = op_instance_.GetBtype() / 1.E6 / avg_time;
            std::cout << "Perf: " << avg_time << " ms, " << tflops << " TFlops, " << gb_per_sec << " GB/s, " << name
                      << std::endl;
            if(avg_time < best.best_avg_time)
            {
                best.best_op_name    = name;
                best.best_tflops     = tflops;
                best.best_gb_per_sec = gb_per_sec;
                best.best_avg_time   = avg_time;
            }
            if(do_verification)
            {
                out_device_buffer_->FromDevice(out_tensor_->mData.data());
                if(!ref_output_)
                    throw std::runtime_error("OpInstanceRunEngine::Profile: Reference value not availabe."
                                             " You have to provide reference function.");
                check(out_tensor_->mData, ref_output_->mData);
            }
            out_device_buffer_->SetZero();
        }
        return best;
    }

    void SetAtol(double a) { atol_ = a; }
    void SetRtol(double r) { rtol_ = r; }

    private:
    template <typename T>
    void upload(const Tensor<T>& t)
    {
        in_device_buffers_.emplace_back(std::make_unique<DeviceMem>(sizeof(T) * t.mDesc.GetElementSpace()))
            ->ToDevice(t.mData.data());
    }
    template <typename T>
    bool check(const std::vector<T>& dev_out, const std::vector<T>& ref_out) const
    {
        return ck::utils::check_err(dev_out, ref_out, "Error: incorrect results!", rtol_, atol_);
    }

    const OpInstanceT& op_instance_;
    double rtol_ = 1e-5, atol_ = 1e-8;
    InTensorsTuple in_tensors_;
    TensorPtr<OutDataType> out_tensor_, ref_output_;
    DeviceBuffers in_device_buffers_;
    DeviceMemPtr out_device_buffer_;
};

namespace conv {

// One forward-convolution problem for the engine (conv_util.hpp:399-570): channels-last host tensors of a
// ConvParams, arguments for any DeviceConvFwd<PassThrough x 3> operation.
template <typename InDataType, typename WeiDataType, typename OutDataType,
          typename InLayout = ck::tensor_layout::convolution::NHWC, typename WeiLayout = ck::tensor_layout::convolution::KYXC,
          typename OutLayout        = ck::tensor_layout::convolution::NHWK,
          typename InElementwiseOp  = ck::tensor_operation::element_wise::PassThrough,
          typename WeiElementwiseOp = ck::tensor_operation::element_wise::PassThrough,
          typename OutElementwiseOp = ck::tensor_operation::element_wise::PassThrough,
          typename InputInitFun = FillUniformDistribution<InDataType>, typename WeightsInitFun = FillUniformDistribution<WeiDataType>>
class ConvFwdOpInstance : public ck::utils::OpInstance<OutDataType, InDataType, WeiDataType>
{
    using DeviceConvFwdOp = tensor_operation::device::DeviceConvFwd<InElementwiseOp, WeiElementwiseOp, OutElementwiseOp>;
    using BaseType        = ck::utils::OpInstance<OutDataType, InDataType, WeiDataType>;
    using DeviceMemPtr    = typename BaseType::DeviceMemPtr;
    using DeviceBuffers   = typename BaseType::DeviceBuffers;
    template <typename T>
    using TensorPtr      = std::unique_ptr<Tensor<T>>;
    using InTensorsTuple = std::tuple<TensorPtr<InDataType>, TensorPtr<WeiDataType>>;

    public:
    ConvFwdOpInstance(const ConvParams& params, bool do_init = true, const InputInitFun& input_init_f = InputInitFun(),
                      const WeightsInitFun& weights_init_f = WeightsInitFun())
        : params_{params}, output_spatial_lengths_{params.GetOutputSpatialLengths()}, do_init_{do_init},
          input_init_f_{input_init_f}, weights_init_f_{weights_init_f}
    {
    }

    InTensorsTuple GetInputTensors() const override
    {
        auto input   = std::make_unique<Tensor<InDataType>>(get_host_tensor_descriptor(dims(params_.N_, params_.C_, params_.input_spatial_lengths_), InLayout{}));
        auto weights = std::make_unique<Tensor<WeiDataType>>(get_host_tensor_descriptor(dims(params_.K_, params_.C_, params_.filter_spatial_lengths_), WeiLayout{}));
        if(do_init_)
        {
            input_init_f_(input->begin(), input->end());
            weights_init_f_(weights->begin(), weights->end());
        }
        return std::make_tuple(std::move(input), std::move(weights));
    }
    TensorPtr<OutDataType> GetOutputTensor() const override
    {
        auto output = std::make_unique<Tensor<OutDataType>>(get_host_tensor_descriptor(dims(params_.N_, params_.K_, output_spatial_lengths_), OutLayout{}));
        if(do_init_)
            std::fill(output->begin(), output->end(), type_convert<OutDataType>(0.f));
        return output;
    }
    std::unique_ptr<tensor_operation::device::BaseInvoker>
    MakeInvokerPointer(tensor_operation::device::BaseOperator* op_ptr) const override
    {
        return cast(op_ptr)->MakeInvokerPointer();
    }
    std::unique_ptr<tensor_operation::device::BaseArgument>
    MakeArgumentPointer(tensor_operation::device::BaseOperator* op_ptr, const DeviceBuffers& in_device_buffers,
                        const DeviceMemPtr& out_device_buffer) const override
    {
        return cast(op_ptr)->MakeArgumentPointer(
            in_device_buffers[0]->GetDeviceBuffer(), in_device_buffers[1]->GetDeviceBuffer(),
            out_device_buffer->GetDeviceBuffer(), params_.N_, params_.K_, params_.C_, params_.input_spatial_lengths_,
            params_.filter_spatial_lengths_, output_spatial_lengths_, params_.conv_filter_strides_,
            params_.conv_filter_dilations_, params_.input_left_pads_, params_.input_right_pads_, InElementwiseOp{},
            WeiElementwiseOp{}, OutElementwiseOp{});
    }
    std::size_t GetFlops() const override
    {
        return get_flops(params_.N_, params_.C_, params_.K_, params_.filter_spatial_lengths_, output_spatial_lengths_);
    }
    std::size_t GetBtype() const override
    {
        return get_btype<InDataType, WeiDataType, OutDataType>(params_.N_, params_.C_, params_.K_,
                                                               params_.input_spatial_lengths_,
                                                               params_.filter_spatial_lengths_, output_spatial_lengths_);
    }

    private:
    static std::vector<std::size_t> dims(index_t a, index_t b, const std::vector<index_t>& spatial)
    {
        std::vector<std::size_t> d{static_cast<std::size_t>(a), static_cast<std::size_t>(b)};
        d.insert(d.end(), spatial.begin(), spatial.end());
        return d;
    }
    static DeviceConvFwdOp* cast(tensor_operation::device::BaseOperator* op_ptr)
    {
        auto conv_ptr = dynamic_cast<DeviceConvFwdOp*>(op_ptr);
        if(!conv_ptr)
            throw std::runtime_error("[ConvFwdOpInstance]: couldn't cast op_ptr to DeviceConvFwdNoOpPtr type!");
        return conv_ptr;
    }
    const ConvParams& params_;
    const std::vector<index_t> output_spatial_lengths_;
    const bool do_init_;
    InputInitFun input_init_f_;
    WeightsInitFun weights_init_f_;
};

} // namespace conv
} // namespace utils
} // namespace ck
