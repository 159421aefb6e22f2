// CPU reference operators with the reference's class names and call sequence, restated for g++:
//   ReferenceGemm                      .../reference_tensor_operation/cpu/reference_gemm.hpp:23-133
//   ReferenceConvFwd (2-D)             .../cpu/reference_conv_fwd.hpp:41-313
//   ReferenceConvFwd_Bias_Activation   .../cpu/reference_conv_fwd_bias_activation.hpp:24-188
// One output element per call of the inner lambda, sequential float (or AccDataType) accumulation,
// element-wise operators applied exactly where the reference applies them, work split over
// std::thread::hardware_concurrency() threads by ParallelTensorFunctor.
#pragma once
#include <thread>

#include "ck/b200/device_ops.hpp"
#include "ck/b200/host_tensor.hpp"

namespace ck {
namespace tensor_operation {
namespace host {

template <typename ADataType, typename BDataType, typename CDataType, typename AccDataType,
          typename AElementwiseOperation, typename BElementwiseOperation, typename CElementwiseOperation>
struct ReferenceGemm : public device::BaseOperator
{
    struct Argument : public device::BaseArgument
    {
        Argument(const Tensor<ADataType>& a_m_k, const Tensor<BDataType>& b_k_n, Tensor<CDataType>& c_m_n,
                 AElementwiseOperation a_element_op, BElementwiseOperation b_element_op,
                 CElementwiseOperation c_element_op)
            : a_m_k_{a_m_k}, b_k_n_{b_k_n}, c_m_n_{c_m_n}, a_element_op_{a_element_op},
              b_element_op_{b_element_op}, c_element_op_{c_element_op}
        {
        }
        const Tensor<ADataType>& a_m_k_;
        const Tensor<BDataType>& b_k_n_;
        Tensor<CDataType>& c_m_n_;
        AElementwiseOperation a_element_op_;
        BElementwiseOperation b_element_op_;
        CElementwiseOperation c_element_op_;
    };

    struct Invoker : public device::BaseInvoker
    {
        float Run(const Argument& arg)
        {
            auto f_mk_kn_mn = [&](auto m, auto n) {
                const int K = static_cast<int>(arg.a_m_k_.mDesc.GetLengths()[1]);
                AccDataType v_acc = 0;
                for(int k = 0; k < K; ++k)
                {
                    ADataType v_a;
                    BDataType v_b;
                    arg.a_element_op_(v_a, arg.a_m_k_(m, k));
                    arg.b_element_op_(v_b, arg.b_k_n_(k, n));
                    v_acc += type_convert<AccDataType>(v_a) * type_convert<AccDataType>(v_b);
                }
                AccDataType v_c;
                arg.c_element_op_(v_c, v_acc);
                arg.c_m_n_(m, n) = type_convert<CDataType>(v_c);
            };
            make_ParallelTensorFunctor(f_mk_kn_mn, arg.c_m_n_.mDesc.GetLengths()[0],
                                       arg.c_m_n_.mDesc.GetLengths()[1])(std::thread::hardware_concurrency());
            return 0;
        }
        float Run(const device::BaseArgument* p_arg, const StreamConfig& = StreamConfig{}) override
        {
            return Run(*dynamic_cast<const Argument*>(p_arg));
        }
    };

    bool IsSupportedArgument(const device::BaseArgument*) override { return true; }
    static auto MakeArgument(const Tensor<ADataType>& a_m_k, const Tensor<BDataType>& b_k_n, Tensor<CDataType>& c_m_n,
                             AElementwiseOperation a_element_op, BElementwiseOperation b_element_op,
                             CElementwiseOperation c_element_op)
    {
        return Argument{a_m_k, b_k_n, c_m_n, a_element_op, b_element_op, c_element_op};
    }
    static auto MakeInvoker() { return Invoker{}; }
    std::string GetTypeString() const override { return "ReferenceGemm"; }
};

// C[g,m,n] = c_op( sum_k a_op(A[g,m,k]) * b_op(B[g,k,n]) ), float accumulation
// (reference_batched_gemm.hpp:21-135); tensors are 3-D with any strides.
template <typename ADataType, typename BDataType, typename CDataType, typename AElementwiseOperation,
          typename BElementwiseOperation, typename CElementwiseOperation>
struct ReferenceBatchedGemm : public device::BaseOperator
{
    struct Argument : public device::BaseArgument
    {
        Argument(const Tensor<ADataType>& a_g_m_k, const Tensor<BDataType>& b_g_k_n, Tensor<CDataType>& c_g_m_n,
                 AElementwiseOperation a_element_op, BElementwiseOperation b_element_op,
                 CElementwiseOperation c_element_op)
            : a_g_m_k_{a_g_m_k}, b_g_k_n_{b_g_k_n}, c_g_m_n_{c_g_m_n}, a_element_op_{a_element_op},
              b_element_op_{b_element_op}, c_element_op_{c_element_op}
        {
        }
        const Tensor<ADataType>& a_g_m_k_;
        const Tensor<BDataType>& b_g_k_n_;
        Tensor<CDataType>& c_g_m_n_;
        AElementwiseOperation a_element_op_;
        BElementwiseOperation b_element_op_;
        CElementwiseOperation c_element_op_;
    };
    struct Invoker : public device::BaseInvoker
    {
        float Run(const Argument& arg)
        {
            auto f = [&](auto g, auto m, auto n) {
                const std::size_t K = arg.a_g_m_k_.mDesc.GetLengths()[2];
                float v_acc         = 0;
                for(std::size_t k = 0; k < K; ++k)
                {
                    ADataType v_a;
                    BDataType v_b;
                    arg.a_element_op_(v_a, arg.a_g_m_k_(g, m, k));
                    arg.b_element_op_(v_b, arg.b_g_k_n_(g, k, n));
                    v_acc += type_convert<float>(v_a) * type_convert<float>(v_b);
                }
                float v_c;
                arg.c_element_op_(v_c, v_acc);
                arg.c_g_m_n_(g, m, n) = type_convert<CDataType>(v_c);
            };
            const auto& l = arg.c_g_m_n_.mDesc.GetLengths();
            make_ParallelTensorFunctor(f, l[0], l[1], l[2])(std::thread::hardware_concurrency());
            return 0;
        }
        float Run(const device::BaseArgument* p_arg, const StreamConfig& = StreamConfig{}) override
        {
            return Run(*dynamic_cast<const Argument*>(p_arg));
        }
    };
    bool IsSupportedArgument(const device::BaseArgument*) override { return true; }
    static auto MakeArgument(const Tensor<ADataType>& a, const Tensor<BDataType>& b, Tensor<CDataType>& c,
                             AElementwiseOperation a_op, BElementwiseOperation b_op, CElementwiseOperation c_op)
    {
        return Argument{a, b, c, a_op, b_op, c_op};
    }
    static auto MakeInvoker() { return Invoker{}; }
    std::string GetTypeString() const override { return "ReferenceBatchedGemm"; }
};

// 1-D, 2-D and 3-D (reference_conv_fwd.hpp:84-254): tensors carry channel-first ordered lengths {N, C, spatial...}
// ({K, C, filter...}, {N, K, out spatial...}) with the strides of any memory layout, see the conv_util host
// descriptors.  Accumulation in float over c, then the filter positions outermost dimension first.
template <typename InDataType, typename WeiDataType, typename OutDataType, typename InElementwiseOperation,
          typename WeiElementwiseOperation, typename OutElementwiseOperation, index_t NumDimSpatial = 2>
struct ReferenceConvFwd : public device::BaseOperator
{
    static_assert(NumDimSpatial >= 1 && NumDimSpatial <= 3, "1-D, 2-D and 3-D convolutions");
    struct Argument : public device::BaseArgument
    {
        Argument(const Tensor<InDataType>& input, const Tensor<WeiDataType>& weight, Tensor<OutDataType>& output,
                 std::vector<index_t> conv_filter_strides, std::vector<index_t> conv_filter_dilations,
                 std::vector<index_t> input_left_pads, std::vector<index_t> input_right_pads,
                 InElementwiseOperation in_element_op, WeiElementwiseOperation wei_element_op,
                 OutElementwiseOperation out_element_op)
            : input_{input}, weight_{weight}, output_{output}, conv_strides_{conv_filter_strides},
              conv_dilations_{conv_filter_dilations}, in_left_pads_{input_left_pads},
              in_right_pads_{input_right_pads}, in_element_op_{in_element_op}, wei_element_op_{wei_element_op},
              out_element_op_{out_element_op}
        {
        }
        const Tensor<InDataType>& input_;
        const Tensor<WeiDataType>& weight_;
        Tensor<OutDataType>& output_;
        std::vector<index_t> conv_strides_, conv_dilations_, in_left_pads_, in_right_pads_;
        InElementwiseOperation in_element_op_;
        WeiElementwiseOperation wei_element_op_;
        OutElementwiseOperation out_element_op_;
    };

    struct Invoker : public device::BaseInvoker
    {
        // input coordinate of output position `o` and filter position `f` along spatial dimension `dim`
        static long_index_t in_pos(const Argument& arg, std::size_t o, std::size_t f, int dim)
        {
            return static_cast<long_index_t>(o * arg.conv_strides_[dim]) +
                   static_cast<long_index_t>(f * arg.conv_dilations_[dim]) -
                   static_cast<long_index_t>(arg.in_left_pads_[dim]);
        }
        static bool inside(long_index_t p, std::size_t len) { return p >= 0 && static_cast<std::size_t>(p) < len; }
        template <typename... Idx>
        static void mac(const Argument& arg, float& v_acc, std::size_t n, std::size_t k, std::size_t c, Idx... sp_and_f)
        {
            // sp_and_f = input positions..., filter positions...
            float v_in, v_wei;
            const std::size_t v[] = {static_cast<std::size_t>(sp_and_f)...};
            if constexpr(NumDimSpatial == 1)
            {
                arg.in_element_op_(v_in, type_convert<float>(arg.input_(n, c, v[0])));
                arg.wei_element_op_(v_wei, type_convert<float>(arg.weight_(k, c, v[1])));
            }
            else if constexpr(NumDimSpatial == 2)
            {
                arg.in_element_op_(v_in, type_convert<float>(arg.input_(n, c, v[0], v[1])));
                arg.wei_element_op_(v_wei, type_convert<float>(arg.weight_(k, c, v[2], v[3])));
            }
            else
            {
                arg.in_element_op_(v_in, type_convert<float>(arg.input_(n, c, v[0], v[1], v[2])));
                arg.wei_element_op_(v_wei, type_convert<float>(arg.weight_(k, c, v[3], v[4], v[5])));
            }
            v_acc += v_in * v_wei;
        }
        template <typename... Out>
        static void store(const Argument& arg, float v_acc, std::size_t n, std::size_t k, Out... o)
        {
            float v_out;
            arg.out_element_op_(v_out, v_acc);
            arg.output_(n, k, o...) = type_convert<OutDataType>(v_out);
        }

        float Run(const Argument& arg)
        {
            const auto& wl = arg.weight_.mDesc.GetLengths(); // K, C, filter...
            const auto& il = arg.input_.mDesc.GetLengths();  // N, C, spatial...
            const auto& ol = arg.output_.mDesc.GetLengths(); // N, K, out spatial...
            const unsigned threads = std::thread::hardware_concurrency();
            if constexpr(NumDimSpatial == 1)
            {
                auto f = [&](auto n, auto k, auto wo) {
                    float v_acc = 0;
                    for(std::size_t c = 0; c < wl[1]; ++c)
                        for(std::size_t x = 0; x < wl[2]; ++x)
                        {
                            const long_index_t wi = in_pos(arg, wo, x, 0);
                            if(inside(wi, il[2]))
                                mac(arg, v_acc, n, k, c, wi, x);
                        }
                    store(arg, v_acc, n, k, wo);
                };
                make_ParallelTensorFunctor(f, ol[0], ol[1], ol[2])(threads);
            }
            else if constexpr(NumDimSpatial == 2)
            {
                auto f = [&](auto n, auto k, auto ho, auto wo) {
                    float v_acc = 0;
                    for(std::size_t c = 0; c < wl[1]; ++c)
                        for(std::size_t y = 0; y < wl[2]; ++y)
                        {
                            const long_index_t hi = in_pos(arg, ho, y, 0);
                            for(std::size_t x = 0; x < wl[3]; ++x)
                            {
                                const long_index_t wi = in_pos(arg, wo, x, 1);
                                if(inside(hi, il[2]) && inside(wi, il[3]))
                                    mac(arg, v_acc, n, k, c, hi, wi, y, x);
                            }
                        }
                    store(arg, v_acc, n, k, ho, wo);
                };
                make_ParallelTensorFunctor(f, ol[0], ol[1], ol[2], ol[3])(threads);
            }
            else
            {
                auto f = [&](auto n, auto k, auto od, auto ho, auto wo) {
                    float v_acc = 0;
                    for(std::size_t c = 0; c < wl[1]; ++c)
                        for(std::size_t z = 0; z < wl[2]; ++z)
                        {
                            const long_index_t di = in_pos(arg, od, z, 0);
                            for(std::size_t y = 0; y < wl[3]; ++y)
                            {
                                const long_index_t hi = in_pos(arg, ho, y, 1);
                                for(std::size_t x = 0; x < wl[4]; ++x)
                                {
                                    const long_index_t wi = in_pos(arg, wo, x, 2);
                                    if(inside(di, il[2]) && inside(hi, il[3]) && inside(wi, il[4]))
                                        mac(arg, v_acc, n, k, c, di, hi, wi, z, y, x);
                                }
                            }
                        }
                    store(arg, v_acc, n, k, od, ho, wo);
                };
                make_ParallelTensorFunctor(f, ol[0], ol[1], ol[2], ol[3], ol[4])(threads);
            }
            return 0;
        }
        float Run(const device::BaseArgument* p_arg, const StreamConfig& = StreamConfig{}) override
        {
            return Run(*dynamic_cast<const Argument*>(p_arg));
        }
    };

    bool IsSupportedArgument(const device::BaseArgument*) override { return true; }
    static auto MakeArgument(const Tensor<InDataType>& input, const Tensor<WeiDataType>& weight,
                             Tensor<OutDataType>& output, std::vector<index_t> conv_filter_strides,
                             std::vector<index_t> conv_filter_dilations, std::vector<index_t> input_left_pads,
                             std::vector<index_t> input_right_pads, InElementwiseOperation in_element_op,
                             WeiElementwiseOperation wei_element_op, OutElementwiseOperation out_element_op)
    {
        return Argument{input, weight, output, conv_filter_strides, conv_filter_dilations, input_left_pads,
                        input_right_pads, in_element_op, wei_element_op, out_element_op};
    }
    static auto MakeInvoker() { return Invoker{}; }
    std::string GetTypeString() const override { return "ReferenceConvFwd"; }
};

namespace detail {
// Float accumulation of one output element of a 2-D convolution over c, y, x (in that order); taps outside the
// image are skipped (reference_conv_fwd_bias_activation.hpp:77-112).  Arg supplies in_n_c_hi_wi_, wei_k_c_y_x_,
// the stride / dilation / left-pad vectors and the input / weight element ops.
template <typename Arg>
float conv2d_accumulate(const Arg& arg, std::size_t n, std::size_t k, std::size_t ho, std::size_t wo)
{
    const auto& wl = arg.wei_k_c_y_x_.mDesc.GetLengths();
    const auto& il = arg.in_n_c_hi_wi_.mDesc.GetLengths();
    float v_acc    = 0;
    for(std::size_t c = 0; c < wl[1]; ++c)
        for(std::size_t y = 0; y < wl[2]; ++y)
        {
            const long_index_t hi = static_cast<long_index_t>(ho * arg.conv_strides_[0]) +
                                    static_cast<long_index_t>(y * arg.conv_dilations_[0]) -
                                    static_cast<long_index_t>(arg.in_left_pads_[0]);
            for(std::size_t x = 0; x < wl[3]; ++x)
            {
                const long_index_t wi = static_cast<long_index_t>(wo * arg.conv_strides_[1]) +
                                        static_cast<long_index_t>(x * arg.conv_dilations_[1]) -
                                        static_cast<long_index_t>(arg.in_left_pads_[1]);
                if(hi >= 0 && static_cast<std::size_t>(hi) < il[2] && wi >= 0 && static_cast<std::size_t>(wi) < il[3])
                {
                    float v_in, v_wei;
                    arg.in_element_op_(v_in, static_cast<const float>(arg.in_n_c_hi_wi_(n, c, hi, wi)));
                    arg.wei_element_op_(v_wei, static_cast<const float>(arg.wei_k_c_y_x_(k, c, y, x)));
                    v_acc += v_in * v_wei;
                }
            }
        }
    return v_acc;
}
} // namespace detail

// out = out_op(acc, float(bias[k])) stored through the implicit float -> OutDataType conversion
template <typename InDataType, typename WeiDataType, typename OutDataType, typename InElementwiseOperation,
          typename WeiElementwiseOperation, typename OutElementwiseOperation>
struct ReferenceConvFwd_Bias_Activation : public device::BaseOperator
{
    struct Argument : public device::BaseArgument
    {
        Argument(const Tensor<InDataType>& in_n_c_hi_wi, const Tensor<WeiDataType>& wei_k_c_y_x,
                 Tensor<OutDataType>& out_n_k_ho_wo, const Tensor<OutDataType>& bias_k,
                 std::vector<index_t> conv_filter_strides, std::vector<index_t> conv_filter_dilations,
                 std::vector<index_t> input_left_pads, std::vector<index_t> input_right_pads,
                 InElementwiseOperation in_element_op, WeiElementwiseOperation wei_element_op,
                 OutElementwiseOperation out_element_op)
            : in_n_c_hi_wi_{in_n_c_hi_wi}, wei_k_c_y_x_{wei_k_c_y_x}, out_n_k_ho_wo_{out_n_k_ho_wo}, bias_k_{bias_k},
              conv_strides_{conv_filter_strides}, conv_dilations_{conv_filter_dilations},
              in_left_pads_{input_left_pads}, in_right_pads_{input_right_pads}, in_element_op_{in_element_op},
              wei_element_op_{wei_element_op}, out_element_op_{out_element_op}
        {
        }
        const Tensor<InDataType>& in_n_c_hi_wi_;
        const Tensor<WeiDataType>& wei_k_c_y_x_;
        Tensor<OutDataType>& out_n_k_ho_wo_;
        const Tensor<OutDataType>& bias_k_;
        std::vector<index_t> conv_strides_, conv_dilations_, in_left_pads_, in_right_pads_;
        InElementwiseOperation in_element_op_;
        WeiElementwiseOperation wei_element_op_;
        OutElementwiseOperation out_element_op_;
    };

    struct Invoker : public device::BaseInvoker
    {
        float Run(const Argument& arg)
        {
            auto f_nchw = [&](auto n, auto k, auto ho, auto wo) {
                const float v_acc = detail::conv2d_accumulate(arg, n, k, ho, wo);
                float v_out;
                arg.out_element_op_(v_out, v_acc, static_cast<float>(arg.bias_k_(k)));
                arg.out_n_k_ho_wo_(n, k, ho, wo) = static_cast<OutDataType>(v_out);
            };
            const auto& ol = arg.out_n_k_ho_wo_.mDesc.GetLengths();
            make_ParallelTensorFunctor(f_nchw, ol[0], ol[1], ol[2], ol[3])(std::thread::hardware_concurrency());
            return 0;
        }
        float Run(const device::BaseArgument* p_arg, const StreamConfig& = StreamConfig{}) override
        {
            return Run(*dynamic_cast<const Argument*>(p_arg));
        }
    };

    bool IsSupportedArgument(const device::BaseArgument*) override { return true; }
    static auto MakeArgument(const Tensor<InDataType>& in_n_c_hi_wi, const Tensor<WeiDataType>& wei_k_c_y_x,
                             Tensor<OutDataType>& out_n_k_ho_wo, const Tensor<OutDataType>& bias_k,
                             std::vector<index_t> conv_filter_strides, std::vector<index_t> conv_filter_dilations,
                             std::vector<index_t> input_left_pads, std::vector<index_t> input_right_pads,
                             InElementwiseOperation in_element_op, WeiElementwiseOperation wei_element_op,
                             OutElementwiseOperation out_element_op)
    {
        return Argument{in_n_c_hi_wi, wei_k_c_y_x, out_n_k_ho_wo, bias_k, conv_filter_strides, conv_filter_dilations,
                        input_left_pads, input_right_pads, in_element_op, wei_element_op, out_element_op};
    }
    static auto MakeInvoker() { return Invoker{}; }
    std::string GetTypeString() const override { return "ReferenceConvFwd_Bias_Activation"; }
};

// out = out_op(acc, float(bias[k]), float(resi[n,k,ho,wo]))
// (reference_conv_fwd_bias_activation_add.hpp:20-185)
template <typename InDataType, typename WeiDataType, typename OutDataType, typename InElementwiseOperation,
          typename WeiElementwiseOperation, typename OutElementwiseOperation>
struct ReferenceConvFwd_Bias_Activation_Add : public device::BaseOperator
{
    struct Argument : public device::BaseArgument
    {
        Argument(const Tensor<InDataType>& in_n_c_hi_wi, const Tensor<WeiDataType>& wei_k_c_y_x,
                 Tensor<OutDataType>& out_n_k_ho_wo, const Tensor<OutDataType>& bias_k,
                 const Tensor<OutDataType>& resi_n_k_ho_wo, std::vector<index_t> conv_filter_strides,
                 std::vector<index_t> conv_filter_dilations, std::vector<index_t> input_left_pads,
                 std::vector<index_t> input_right_pads, InElementwiseOperation in_element_op,
                 WeiElementwiseOperation wei_element_op, OutElementwiseOperation out_element_op)
            : in_n_c_hi_wi_{in_n_c_hi_wi}, wei_k_c_y_x_{wei_k_c_y_x}, out_n_k_ho_wo_{out_n_k_ho_wo}, bias_k_{bias_k},
              resi_n_k_ho_wo_{resi_n_k_ho_wo}, conv_strides_{conv_filter_strides},
              conv_dilations_{conv_filter_dilations}, in_left_pads_{input_left_pads}, in_right_pads_{input_right_pads},
              in_element_op_{in_element_op}, wei_element_op_{wei_element_op}, out_element_op_{out_element_op}
        {
        }
        const Tensor<InDataType>& in_n_c_hi_wi_;
        const Tensor<WeiDataType>& wei_k_c_y_x_;
        Tensor<OutDataType>& out_n_k_ho_wo_;
        const Tensor<OutDataType>& bias_k_;
        const Tensor<OutDataType>& resi_n_k_ho_wo_;
        std::vector<index_t> conv_strides_, conv_dilations_, in_left_pads_, in_right_pads_;
        InElementwiseOperation in_element_op_;
        WeiElementwiseOperation wei_element_op_;
        OutElementwiseOperation out_element_op_;
    };

    struct Invoker : public device::BaseInvoker
    {
        float Run(const Argument& arg)
        {
            auto f_nchw = [&](auto n, auto k, auto ho, auto wo) {
                const float v_acc = detail::conv2d_accumulate(arg, n, k, ho, wo);
                float v_out;
                arg.out_element_op_(v_out, v_acc, static_cast<float>(arg.bias_k_(k)),
                                    static_cast<float>(arg.resi_n_k_ho_wo_(n, k, ho, wo)));
                arg.out_n_k_ho_wo_(n, k, ho, wo) = static_cast<OutDataType>(v_out);
            };
            const auto& ol = arg.out_n_k_ho_wo_.mDesc.GetLengths();
            make_ParallelTensorFunctor(f_nchw, ol[0], ol[1], ol[2], ol[3])(std::thread::hardware_concurrency());
            return 0;
        }
        float Run(const device::BaseArgument* p_arg, const StreamConfig& = StreamConfig{}) override
        {
            return Run(*dynamic_cast<const Argument*>(p_arg));
        }
    };

    bool IsSupportedArgument(const device::BaseArgument*) override { return true; }
    static auto MakeArgument(const Tensor<InDataType>& in_n_c_hi_wi, const Tensor<WeiDataType>& wei_k_c_y_x,
                             Tensor<OutDataType>& out_n_k_ho_wo, const Tensor<OutDataType>& bias_k,
                             const Tensor<OutDataType>& resi_n_k_ho_wo, std::vector<index_t> conv_filter_strides,
                             std::vector<index_t> conv_filter_dilations, std::vector<index_t> input_left_pads,
                             std::vector<index_t> input_right_pads, InElementwiseOperation in_element_op,
                             WeiElementwiseOperation wei_element_op, OutElementwiseOperation out_element_op)
    {
        return Argument{in_n_c_hi_wi, wei_k_c_y_x, out_n_k_ho_wo, bias_k, resi_n_k_ho_wo, conv_filter_strides,
                        conv_filter_dilations, input_left_pads, input_right_pads, in_element_op, wei_element_op,
                        out_element_op};
    }
    static auto MakeInvoker() { return Invoker{}; }
    std::string GetTypeString() const override { return "ReferenceConvFwd_Bias_Activation_Add"; }
};

} // namespace host
} // namespace tensor_operation
} // namespace ck
