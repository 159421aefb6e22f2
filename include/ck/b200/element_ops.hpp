// Element-wise functors of the dense-contraction path, host side.
//
// Same names, namespaces and per-type behaviour as the reference functors
// (include/ck/tensor_operation/gpu/element/*.hpp).  The reference spells the per-type variants
// as member-template specialisations at class scope (a clang extension); they are ordinary
// overloads here.  Each functor also has a twin inside libckb200.so (CKB_EPI_* in ckb200.h):
// ck::b200::EpilogueTraits<Op> names it, and tests pin the two to each other value by value.
//
// Compile host code that uses the binary16 overloads with -fexcess-precision=16 so that half
// arithmetic rounds after every operation.
#pragma once
#include <cmath>

#include "ck/b200/core.hpp"
#include "ckb200.h"

namespace ck {
namespace tensor_operation {
namespace element_wise {

// unary_element_wise_operation.hpp:13-25
struct PassThrough
{
    template <typename T>
    void operator()(T& y, const T& x) const
    {
        y = x;
    }
};

// unary_element_wise_operation.hpp:27-41
struct Scale
{
    Scale(float scale) : scale_(scale) {}
    void operator()(float& y, const float& x) const { y = scale_ * x; }
    float scale_;
};

// unary_element_wise_operation.hpp:98-119
struct Relu
{
    template <typename T>
    void operator()(T& y, const T& x) const
    {
        y = x > 0 ? x : 0;
    }
    void operator()(bhalf_t& y, const bhalf_t& x) const
    {
        const float v = type_convert<float>(x);
        y             = type_convert<bhalf_t>(v > 0 ? v : 0.0f);
    }
};

namespace detail {
// unary_element_wise_operation.hpp:121-135 / element_wise_operation.hpp:127-133
inline float fast_gelu(float x)
{
    const float u   = float(2) * x * (float(0.035677) * x * x + float(0.797885));
    const float emu = static_cast<float>(std::exp(static_cast<double>(-u)));
    const float cdf = float(0.5) + float(0.5) * (float(2) / (float(1) + emu) - float(1));
    return x * cdf;
}
} // namespace detail

struct FastGelu
{
    void operator()(float& y, const float& x) const { y = detail::fast_gelu(x); }
};

// binary_element_wise_operation.hpp:12-54
struct Add
{
    void operator()(float& y, const float& x0, const float& x1) const { y = x0 + x1; }
    void operator()(double& y, const double& x0, const double& x1) const { y = x0 + x1; }
    void operator()(half_t& y, const float& x0, const half_t& x1) const
    {
        y = static_cast<half_t>(type_convert<half_t>(x0) + x1);
    }
    void operator()(half_t& y, const half_t& x0, const half_t& x1) const { y = static_cast<half_t>(x0 + x1); }
};

// binary_element_wise_operation.hpp:93-116
struct Bilinear
{
    Bilinear(float alpha, float beta) : alpha_(alpha), beta_(beta) {}
    void operator()(float& y, const float& x0, const float& x1) const { y = alpha_ * x0 + beta_ * x1; }
    void operator()(half_t& y, const float& x0, const half_t& x1) const
    {
        y = type_convert<half_t>(alpha_ * x0 + beta_ * type_convert<float>(x1));
    }
    float alpha_;
    float beta_;
};

// binary_element_wise_operation.hpp:118-146
struct AddRelu
{
    void operator()(float& y, const float& x0, const float& x1) const
    {
        const float a = x0 + x1;
        y             = a > 0.0f ? a : 0.0f;
    }
    void operator()(double& y, const double& x0, const double& x1) const
    {
        const double a = x0 + x1;
        y              = a > 0.0 ? a : 0.0;
    }
    void operator()(half_t& y, const half_t& x0, const half_t& x1) const
    {
        const half_t a = static_cast<half_t>(x0 + x1);
        y              = a > type_convert<half_t>(0.0f) ? a : type_convert<half_t>(0.0f);
    }
};

// binary_element_wise_operation.hpp:148-181
struct AddHardswish
{
    void operator()(float& y, const float& x0, const float& x1) const
    {
        const float a = x0 + x1;
        const float b = a + float{3};
        y             = (b > 0) * (b > 6.0f ? 6.0f : b) * a * 0.166667f;
    }
};

// element_wise_operation.hpp:46-80
struct AddReluAdd
{
    void operator()(float& y, const float& x0, const float& x1, const float& x2) const
    {
        const float a = x0 + x1;
        const float b = a > 0 ? a : 0;
        y             = b + x2;
    }
    void operator()(half_t& y, const float& x0, const half_t& x1, const half_t& x2) const
    {
        const float a = x0 + type_convert<float>(x1);
        const float b = a > 0 ? a : 0;
        y             = type_convert<half_t>(b + type_convert<float>(x2));
    }
};

// element_wise_operation.hpp:115-140
struct AddAddFastGelu
{
    void operator()(half_t& e, const float& c, const half_t& d0, const half_t& d1) const
    {
        e = type_convert<half_t>(detail::fast_gelu(c + float(d0) + float(d1)));
    }
};

// The user functor of example/14_gemm_xdl_requant_relu_requant/gemm_xdl_requant_relu_requant_int8.cpp:21-39,
// provided here under the same name so that the example needs no trait line of its own.
struct RequantReluRequant
{
    RequantReluRequant(float scaleGemm, float scaleRelu) : scaleGemm_(scaleGemm), scaleRelu_(scaleRelu) {}
    void operator()(float& y, const float& x) const
    {
        const float gemm_requant = scaleGemm_ * x;
        const float relu         = gemm_requant > 0 ? gemm_requant : 0;
        const float relu_requant = scaleRelu_ * relu;
        y = relu_requant > 127 ? 127 : relu_requant < -128 ? -128 : relu_requant;
    }
    float scaleGemm_;
    float scaleRelu_;
};

// sat_int8(rne(s1 * relu(rne(s0 * acc)))): RequantReluRequant with a round-to-nearest-even after
// each scale (no counterpart in the reference).
struct RequantReluRequantRne
{
    RequantReluRequantRne(float scaleGemm, float scaleRelu) : scaleGemm_(scaleGemm), scaleRelu_(scaleRelu) {}
    void operator()(float& y, const float& x) const
    {
        const float q0 = std::nearbyint(scaleGemm_ * x);
        const float r  = q0 > 0 ? q0 : 0;
        const float q1 = std::nearbyint(scaleRelu_ * r);
        y              = q1 > 127 ? 127 : q1 < -128 ? -128 : q1;
    }
    float scaleGemm_;
    float scaleRelu_;
};

} // namespace element_wise
} // namespace tensor_operation

namespace b200 {

namespace ew = ck::tensor_operation::element_wise;

// Maps a functor TYPE to the fused epilogue inside the kernel library.  kind < 0: no device twin,
// IsSupportedArgument() is false.  A driver with its own functor type specialises this trait.
// `Ctx` distinguishes the call sites whose reference semantics differ for one functor name:
//   ctx_gemm_c  : DeviceGemm C op                - functor(float&, float), then type_convert<C>
//   ctx_gemm_cde: DeviceGemmMultipleD / grouped  - functor(E&, float c, D...) with E, D = half
//   ctx_conv    : conv fwd (+bias) out op        - functor(float&, float acc[, float bias]), one rounding
struct ctx_gemm_c;
struct ctx_gemm_cde;
struct ctx_conv;

template <typename Op, typename Ctx = ctx_gemm_c>
struct EpilogueTraits
{
    static constexpr int kind = -1;
    static void params(const Op&, float (&p)[4]) { p[0] = p[1] = p[2] = p[3] = 0; }
};

#define CKB_SIMPLE_TRAIT(OP, CTX, KIND)                                                   \
    template <>                                                                           \
    struct EpilogueTraits<ew::OP, CTX>                                                    \
    {                                                                                     \
        static constexpr int kind = KIND;                                                 \
        static void params(const ew::OP&, float (&p)[4]) { p[0] = p[1] = p[2] = p[3] = 0; } \
    };
CKB_SIMPLE_TRAIT(PassThrough, ctx_gemm_c, CKB_EPI_PASSTHROUGH)
CKB_SIMPLE_TRAIT(PassThrough, ctx_gemm_cde, CKB_EPI_PASSTHROUGH)
CKB_SIMPLE_TRAIT(PassThrough, ctx_conv, CKB_EPI_PASSTHROUGH)
CKB_SIMPLE_TRAIT(Relu, ctx_gemm_c, CKB_EPI_RELU)
CKB_SIMPLE_TRAIT(Relu, ctx_conv, CKB_EPI_RELU)
CKB_SIMPLE_TRAIT(FastGelu, ctx_gemm_c, CKB_EPI_FASTGELU)
CKB_SIMPLE_TRAIT(Add, ctx_gemm_cde, CKB_EPI_ADD)             // half(c) + d0 in binary16
CKB_SIMPLE_TRAIT(AddRelu, ctx_conv, CKB_EPI_ADD_RELU)        // fp32, one rounding
CKB_SIMPLE_TRAIT(AddRelu, ctx_gemm_cde, CKB_EPI_ADD_RELU_F16) // c arrives as half (CShuffleDataType F16)
CKB_SIMPLE_TRAIT(AddHardswish, ctx_conv, CKB_EPI_ADD_HARDSWISH)
CKB_SIMPLE_TRAIT(AddAddFastGelu, ctx_gemm_cde, CKB_EPI_ADD_ADD_FASTGELU)
CKB_SIMPLE_TRAIT(AddReluAdd, ctx_gemm_cde, CKB_EPI_ADD_RELU_ADD)
CKB_SIMPLE_TRAIT(AddReluAdd, ctx_conv, CKB_EPI_ADD_RELU_ADD)
#undef CKB_SIMPLE_TRAIT

template <typename Ctx>
struct EpilogueTraits<ew::Scale, Ctx>
{
    static constexpr int kind = CKB_EPI_SCALE;
    static void params(const ew::Scale& op, float (&p)[4])
    {
        p[0] = op.scale_;
        p[1] = p[2] = p[3] = 0;
    }
};
template <typename Ctx>
struct EpilogueTraits<ew::Bilinear, Ctx>
{
    static constexpr int kind = CKB_EPI_BILINEAR;
    static void params(const ew::Bilinear& op, float (&p)[4])
    {
        p[0] = op.alpha_;
        p[1] = op.beta_;
        p[2] = p[3] = 0;
    }
};
template <typename Ctx>
struct EpilogueTraits<ew::RequantReluRequant, Ctx>
{
    static constexpr int kind = CKB_EPI_REQUANT_RELU_REQUANT;
    static void params(const ew::RequantReluRequant& op, float (&p)[4])
    {
        p[0] = op.scaleGemm_;
        p[1] = op.scaleRelu_;
        p[2] = p[3] = 0;
    }
};
template <typename Ctx>
struct EpilogueTraits<ew::RequantReluRequantRne, Ctx>
{
    static constexpr int kind = CKB_EPI_REQUANT_RELU_REQUANT_RNE;
    static void params(const ew::RequantReluRequantRne& op, float (&p)[4])
    {
        p[0] = op.scaleGemm_;
        p[1] = op.scaleRelu_;
        p[2] = p[3] = 0;
    }
};

template <typename Op>
struct is_passthrough : std::is_same<Op, ew::PassThrough>
{
};

template <typename T>
struct dtype_of;
template <>
struct dtype_of<half_t>
{
    static constexpr int value = CKB_F16;
};
template <>
struct dtype_of<int8_t>
{
    static constexpr int value = CKB_I8;
};
template <>
struct dtype_of<bhalf_t>
{
    static constexpr int value = CKB_BF16;
};
template <>
struct dtype_of<float>
{
    static constexpr int value = -1; // no fp32 kernels in the library
};

} // namespace b200
} // namespace ck
