// Verification and convolution helpers of the reference's utility library, restated for g++:
//   ck::utils::check_err          library/include/ck/library/utility/check_err.hpp:21-193
//   ck::utils::Fill*              library/include/ck/library/utility/fill.hpp:16-95
//   ck::utils::conv::ConvParams,  library/include/ck/library/utility/conv_util.hpp:86-251,
//     get_flops, get_btype, host tensor descriptors       library/src/utility/conv_util.cpp:22-225
#pragma once
#include <cmath>
#include <iomanip>
#include <iostream>
#include <limits>
#include <random>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

#include "ck/b200/core.hpp"
#include "ck/b200/device_ops.hpp"
#include "ck/b200/host_tensor.hpp"

namespace ck {
namespace utils {

namespace detail {
template <typename T>
struct default_tolerance
{
    static constexpr double rtol = 1e-5, atol = 3e-6; // float / double, check_err.hpp:24-28
};
template <>
struct default_tolerance<half_t>
{
    static constexpr double rtol = 1e-3, atol = 1e-3; // check_err.hpp:109-113
};
template <>
struct default_tolerance<bhalf_t>
{
    static constexpr double rtol = 1e-3, atol = 1e-3; // check_err.hpp:63-69
};
} // namespace detail

// Floating-point types (float, double, half_t, and bhalf_t bit patterns): an element fails when |o - r| > atol + rtol*|r| or either
// value is not finite.  Prints the first few failures and the largest error, like the reference.
template <typename T>
typename std::enable_if<std::is_floating_point<T>::value || std::is_same<T, half_t>::value ||
                            std::is_same<T, bhalf_t>::value,
                        bool>::type
check_err(const std::vector<T>& out, const std::vector<T>& ref, const std::string& msg = "Error: Incorrect results!",
          double rtol = detail::default_tolerance<T>::rtol, double atol = detail::default_tolerance<T>::atol)
{
    if(out.size() != ref.size())
    {
        std::cout << msg << " out.size() != ref.size(), :" << out.size() << " != " << ref.size() << std::endl;
        return false;
    }
    bool res       = true;
    int err_count  = 0;
    double max_err = 0;
    for(std::size_t i = 0; i < ref.size(); ++i)
    {
        const double o   = static_cast<double>(type_convert<float>(out[i]));
        const double r   = static_cast<double>(type_convert<float>(ref[i]));
        const double err = std::abs(o - r);
        if(err > atol + rtol * std::abs(r) || !std::isfinite(o) || !std::isfinite(r))
        {
            max_err = err > max_err ? err : max_err;
            if(++err_count < 5)
                std::cout << msg << std::setw(12) << std::setprecision(7) << " out[" << i << "] != ref[" << i
                          << "]: " << o << " != " << r << std::endl;
            res = false;
        }
    }
    if(!res)
        std::cout << std::setw(12) << std::setprecision(7) << "max err: " << max_err << std::endl;
    return res;
}

// Integers: exact unless atol is given (check_err.hpp:150-193).
template <typename T>
typename std::enable_if<std::is_integral<T>::value && !std::is_same<T, bhalf_t>::value, bool>::type
check_err(const std::vector<T>& out, const std::vector<T>& ref, const std::string& msg = "Error: Incorrect results!",
          double = 0, double atol = 0)
{
    if(out.size() != ref.size())
    {
        std::cout << msg << " out.size() != ref.size(), :" << out.size() << " != " << ref.size() << std::endl;
        return false;
    }
    bool res        = true;
    int err_count   = 0;
    int64_t max_err = 0;
    for(std::size_t i = 0; i < ref.size(); ++i)
    {
        const int64_t err = std::abs(static_cast<int64_t>(out[i]) - static_cast<int64_t>(ref[i]));
        if(err > atol)
        {
            max_err = err > max_err ? err : max_err;
            if(++err_count < 5)
                std::cout << msg << " out[" << i << "] != ref[" << i << "]: " << static_cast<int>(out[i])
                          << " != " << static_cast<int>(ref[i]) << std::endl;
            res = false;
        }
    }
    if(!res)
        std::cout << "max err: " << max_err << std::endl;
    return res;
}

// fill.hpp:16-95
template <typename T>
struct FillUniformDistribution
{
    float a_{-5.f};
    float b_{5.f};
    template <typename ForwardIter>
    void operator()(ForwardIter first, ForwardIter last) const
    {
        std::mt19937 gen(11939);
        std::uniform_real_distribution<float> dis(a_, b_);
        for(; first != last; ++first)
            *first = type_convert<T>(dis(gen));
    }
};
template <typename T>
struct FillUniformDistributionIntegerValue
{
    float a_{-5.f};
    float b_{5.f};
    template <typename ForwardIter>
    void operator()(ForwardIter first, ForwardIter last) const
    {
        std::mt19937 gen(11939);
        std::uniform_real_distribution<float> dis(a_, b_);
        for(; first != last; ++first)
            *first = type_convert<T>(std::round(dis(gen)));
    }
};
template <typename T>
struct FillMonotonicSeq
{
    T init_value_{0};
    T step_{1};
    template <typename ForwardIter>
    void operator()(ForwardIter first, ForwardIter last) const
    {
        T n = init_value_;
        for(; first != last; ++first, n += step_)
            *first = n;
    }
};
template <typename T>
struct FillConstant
{
    T value_{0};
    template <typename ForwardIter>
    void operator()(ForwardIter first, ForwardIter last) const
    {
        for(; first != last; ++first)
            *first = value_;
    }
};

namespace conv {

// 2 * N * K * prod(output) * C * prod(filter)   (conv_util.cpp:22-39)
inline std::size_t get_flops(index_t N, index_t C, index_t K, const std::vector<index_t>& filter_spatial_lengths,
                             const std::vector<index_t>& output_spatial_lengths)
{
    std::size_t f = static_cast<std::size_t>(2) * N * K * C;
    for(index_t v : output_spatial_lengths)
        f *= v;
    for(index_t v : filter_spatial_lengths)
        f *= v;
    return f;
}

// conv_util.hpp:111-136
template <typename InDataType = float, typename WeiDataType = InDataType, typename OutDataType = InDataType>
std::size_t get_btype(index_t N, index_t C, index_t K, const std::vector<index_t>& input_spatial_lengths,
                      const std::vector<index_t>& filter_spatial_lengths,
                      const std::vector<index_t>& output_spatial_lengths)
{
    auto prod = [](const std::vector<index_t>& v) {
        std::size_t p = 1;
        for(index_t x : v)
            p *= x;
        return p;
    };
    return sizeof(InDataType) * (static_cast<std::size_t>(N) * C * prod(input_spatial_lengths)) +
           sizeof(WeiDataType) * (static_cast<std::size_t>(K) * C * prod(filter_spatial_lengths)) +
           sizeof(OutDataType) * (static_cast<std::size_t>(N) * K * prod(output_spatial_lengths));
}

// conv_util.hpp:138-167, conv_util.cpp:41-116
struct ConvParams
{
    // N128 K256 C192, 3x3 filter, 71x71 image, stride 2, dilation 1, pad 1
    ConvParams()
        : num_dim_spatial_(2), N_(128), K_(256), C_(192), filter_spatial_lengths_(2, 3),
          input_spatial_lengths_(2, 71), conv_filter_strides_(2, 2), conv_filter_dilations_(2, 1),
          input_left_pads_(2, 1), input_right_pads_(2, 1)
    {
    }
    ConvParams(index_t n_dim, index_t n_batch, index_t n_out_channels, index_t n_in_channels,
               const std::vector<index_t>& filters_len, const std::vector<index_t>& input_len,
               const std::vector<index_t>& strides, const std::vector<index_t>& dilations,
               const std::vector<index_t>& left_pads, const std::vector<index_t>& right_pads)
        : num_dim_spatial_(n_dim), N_(n_batch), K_(n_out_channels), C_(n_in_channels),
          filter_spatial_lengths_(filters_len), input_spatial_lengths_(input_len), conv_filter_strides_(strides),
          conv_filter_dilations_(dilations), input_left_pads_(left_pads), input_right_pads_(right_pads)
    {
        check_sizes("ConvParams::ConvParams");
    }

    index_t num_dim_spatial_;
    index_t N_, K_, C_;
    std::vector<index_t> filter_spatial_lengths_;
    std::vector<index_t> input_spatial_lengths_;
    std::vector<index_t> conv_filter_strides_;
    std::vector<index_t> conv_filter_dilations_;
    std::vector<index_t> input_left_pads_;
    std::vector<index_t> input_right_pads_;

    // Wo = (Wi + lpad + rpad - ((X - 1) * dilation + 1)) / stride + 1
    std::vector<index_t> GetOutputSpatialLengths() const
    {
        check_sizes("ConvParams::GetOutputSpatialLengths");
        std::vector<index_t> out(num_dim_spatial_, 0);
        for(index_t i = 0; i < num_dim_spatial_; ++i)
        {
            const index_t eff = (filter_spatial_lengths_[i] - 1) * conv_filter_dilations_[i] + 1;
            out[i] = (input_spatial_lengths_[i] + input_left_pads_[i] + input_right_pads_[i] - eff) /
                         conv_filter_strides_[i] +
                     1;
        }
        return out;
    }

    private:
    void check_sizes(const char* who) const
    {
        const std::size_t n = static_cast<std::size_t>(num_dim_spatial_);
        if(filter_spatial_lengths_.size() != n || input_spatial_lengths_.size() != n ||
           conv_filter_strides_.size() != n || conv_filter_dilations_.size() != n || input_left_pads_.size() != n ||
           input_right_pads_.size() != n)
            throw std::runtime_error(std::string(who) +
                                     ": parameter size is different from number of declared dimensions!");
    }
};

// positional: N K C, filter..., input..., strides..., dilations..., left pads..., right pads...  (conv_util.cpp:118-170)
inline ConvParams parse_conv_params(int num_dim_spatial, int arg_idx, char* const argv[])
{
    ConvParams p;
    p.num_dim_spatial_ = num_dim_spatial;
    p.N_               = std::stoi(argv[arg_idx++]);
    p.K_               = std::stoi(argv[arg_idx++]);
    p.C_               = std::stoi(argv[arg_idx++]);
    auto read = [&](std::vector<index_t>& v) {
        v.resize(num_dim_spatial);
        for(int i = 0; i < num_dim_spatial; ++i)
            v[i] = std::stoi(argv[arg_idx++]);
    };
    read(p.filter_spatial_lengths_);
    read(p.input_spatial_lengths_);
    read(p.conv_filter_strides_);
    read(p.conv_filter_dilations_);
    read(p.input_left_pads_);
    read(p.input_right_pads_);
    return p;
}

// Host tensors carry NCHW-ordered LENGTHS with the strides of the memory layout
// (conv_util.hpp:170-251): dims = {N, C, spatial...}.
template <typename TensorLayout>
HostTensorDescriptor get_host_tensor_descriptor(const std::vector<std::size_t>& dims, const TensorLayout&)
{
    namespace L       = ck::tensor_layout::convolution;
    const std::size_t C = dims[1];
    constexpr bool channels_last =
        std::is_same<TensorLayout, L::NWC>::value || std::is_same<TensorLayout, L::KXC>::value ||
        std::is_same<TensorLayout, L::NWK>::value || std::is_same<TensorLayout, L::NHWC>::value ||
        std::is_same<TensorLayout, L::KYXC>::value || std::is_same<TensorLayout, L::NHWK>::value ||
        std::is_same<TensorLayout, L::NDHWC>::value || std::is_same<TensorLayout, L::KZYXC>::value ||
        std::is_same<TensorLayout, L::NDHWK>::value;
    std::vector<std::size_t> strides(dims.size(), 1);
    if(channels_last)
    {
        // memory order: N, spatial..., C
        strides[1]      = 1;
        std::size_t run = C;
        for(std::size_t i = dims.size(); i-- > 2;)
        {
            strides[i] = run;
            run *= dims[i];
        }
        strides[0] = run;
    }
    else
    {
        for(std::size_t i = dims.size(); i-- > 1;)
            strides[i - 1] = strides[i] * dims[i];
    }
    return HostTensorDescriptor(dims, strides);
}

inline HostTensorDescriptor get_input_host_tensor_descriptor(const std::vector<std::size_t>& dims, int = 2)
{
    return get_host_tensor_descriptor(dims, ck::tensor_layout::convolution::NHWC{});
}
inline HostTensorDescriptor get_filters_host_tensor_descriptor(const std::vector<std::size_t>& dims, int = 2)
{
    return get_host_tensor_descriptor(dims, ck::tensor_layout::convolution::KYXC{});
}
inline HostTensorDescriptor get_output_host_tensor_descriptor(const std::vector<std::size_t>& dims, int = 2)
{
    return get_host_tensor_descriptor(dims, ck::tensor_layout::convolution::NHWK{});
}

} // namespace conv
} // namespace utils
} // namespace ck
