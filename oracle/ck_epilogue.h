// TEST INFRASTRUCTURE - CPU oracle.  Not part of the shipped library: only tests/,
// __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm may use it.
//
// Host restatement of the Composable Kernel element-wise functors that the dense
// contraction path applies to one accumulator value.  Every function cites the
// reference functor it follows.  half = _Float16 (ck::half_t,
// include/ck/utility/data_type.hpp:11); type_convert is a static_cast
// (data_type.hpp:934-938), i.e. round-to-nearest-even for float->half and
// truncation toward zero for float->int8.
//
// Build with -fexcess-precision=16 -ffp-contract=off so that binary16 arithmetic
// rounds after every operation and no multiply-add is fused.
#pragma once
#include <cmath>
#include <cstdint>

namespace ck_oracle {

using half = _Float16;

enum Epilogue : int {
    EPI_PASSTHROUGH = 0,
    EPI_SCALE = 1,
    EPI_RELU = 2,
    EPI_FASTGELU = 3,
    EPI_ADD = 4,
    EPI_ADD_RELU_F16 = 5,
    EPI_BILINEAR = 6,
    EPI_ADD_ADD_FASTGELU = 7,
    EPI_ADD_RELU_ADD = 8,
    EPI_REQUANT_RELU_REQUANT = 9,
    EPI_REQUANT_RELU_REQUANT_RNE = 10,
    EPI_ADD_RELU = 11,
    EPI_ADD_HARDSWISH = 12,
};

// element/unary_element_wise_operation.hpp:121-135 and element_wise_operation.hpp:127-133.
// The reference calls exp() unqualified on a float; double exp rounded to float is used here
// (differs from expf by at most one float ulp, three orders below the 1e-3 check).
inline float fast_gelu(float x)
{
    const float u   = float(2) * x * (float(0.035677) * x * x + float(0.797885));
    const float emu = static_cast<float>(std::exp(static_cast<double>(-u)));
    const float cdf = float(0.5) + float(0.5) * (float(2) / (float(1) + emu) - float(1));
    return x * cdf;
}

// Round-to-nearest-even to an integer value, kept in float (std::nearbyint in the default
// rounding mode).
inline float rne(float x) { return std::nearbyint(x); }

// Epilogues whose output type is binary16.  c = fp32 accumulator.
inline half apply_f16(int epi, const float* p, float c, half d0, half d1)
{
    switch(epi)
    {
    case EPI_PASSTHROUGH: return static_cast<half>(c); // unary...hpp:13-25 + reference_gemm.hpp:78-80
    case EPI_SCALE: return static_cast<half>(p[0] * c); // unary...hpp:36-39
    case EPI_RELU: return static_cast<half>(c > 0 ? c : 0); // unary...hpp:98-108
    case EPI_FASTGELU: return static_cast<half>(fast_gelu(c));
    case EPI_ADD: { // binary...hpp:31-36: y = type_convert<half_t>(x0) + x1
        half x0 = static_cast<half>(c);
        return static_cast<half>(x0 + d0);
    }
    case EPI_ADD_RELU_F16: { // example/03_gemm_bias_relu/gemm_bias_relu_xdl_fp16.cpp:34-43
        half x = static_cast<half>(static_cast<half>(c) + d0);
        return x > 0 ? x : static_cast<half>(0);
    }
    case EPI_BILINEAR: // binary...hpp:107-112
        return static_cast<half>(p[0] * c + p[1] * static_cast<float>(d0));
    case EPI_ADD_ADD_FASTGELU: // element_wise_operation.hpp:121-139
        return static_cast<half>(fast_gelu(c + static_cast<float>(d0) + static_cast<float>(d1)));
    case EPI_ADD_RELU_ADD: { // element_wise_operation.hpp:71-79
        float a = c + static_cast<float>(d0);
        float b = a > 0 ? a : 0;
        float y = b + static_cast<float>(d1);
        return static_cast<half>(y);
    }
    case EPI_ADD_RELU: { // binary...hpp:123-129 via reference_conv_fwd_bias_activation.hpp:114-118
        float a = c + static_cast<float>(d0);
        return static_cast<half>(a > 0.0f ? a : 0.0f);
    }
    case EPI_ADD_HARDSWISH: { // binary...hpp:153-161
        float a = c + static_cast<float>(d0);
        float b = a + float{3};
        float y = (b > 0) * (b > 6.0f ? 6.0f : b) * a * 0.166667f;
        return static_cast<half>(y);
    }
    default: return static_cast<half>(NAN);
    }
}

// bfloat16 as its bit pattern (ck::bhalf_t = ushort, include/ck/utility/data_type.hpp:10) with the
// reference's conversions (data_type.hpp:940-990): widening is a shift, narrowing rounds to nearest even.
struct bf16
{
    uint16_t bits;
};
inline float bf16_to_float(bf16 x)
{
    const uint32_t u = static_cast<uint32_t>(x.bits) << 16;
    float f;
    __builtin_memcpy(&f, &u, 4);
    return f;
}
inline bf16 float_to_bf16(float x)
{
    uint32_t u;
    __builtin_memcpy(&u, &x, 4);
    if(~u & 0x7f800000u)
        u += 0x7fffu + ((u >> 16) & 1u);
    else if(u & 0xffffu)
        u |= 0x10000u;
    return bf16{static_cast<uint16_t>(u >> 16)};
}

// Epilogues whose output type is bfloat16: the functors that work in float and round once
// (the reference defines no binary16-style arithmetic functors for bhalf_t).
inline bf16 apply_bf16(int epi, const float* p, float c, bf16 d0b, bf16 d1b)
{
    const float d0 = bf16_to_float(d0b), d1 = bf16_to_float(d1b);
    switch(epi)
    {
    case EPI_PASSTHROUGH: return float_to_bf16(c);
    case EPI_SCALE: return float_to_bf16(p[0] * c);
    case EPI_RELU: return float_to_bf16(c > 0 ? c : 0);
    case EPI_FASTGELU: return float_to_bf16(fast_gelu(c));
    case EPI_ADD_RELU: {
        float a = c + d0;
        return float_to_bf16(a > 0.0f ? a : 0.0f);
    }
    case EPI_ADD_HARDSWISH: {
        float a = c + d0;
        float b = a + float{3};
        return float_to_bf16((b > 0) * (b > 6.0f ? 6.0f : b) * a * 0.166667f);
    }
    case EPI_ADD_RELU_ADD: {
        float a = c + d0;
        float b = a > 0 ? a : 0;
        return float_to_bf16(b + d1);
    }
    default: return float_to_bf16(NAN);
    }
}

// Epilogues whose output type is int8.  acc = int32 accumulator.  PassThrough keeps the
// integer path of test/gemm/gemm_int8.cpp:32 (AccDataType = int32_t, static_cast<int8_t>);
// every other functor sees the accumulator as float, as example 14's host reference does
// (AccDataType = float, gemm_xdl_requant_relu_requant_int8.cpp:103-109) - identical while
// |acc| < 2^24.
inline int8_t apply_i8(int epi, const float* p, int32_t acc)
{
    const float c = static_cast<float>(acc);
    switch(epi)
    {
    case EPI_PASSTHROUGH: return static_cast<int8_t>(acc);
    case EPI_REQUANT_RELU_REQUANT: {
        // example/14_gemm_xdl_requant_relu_requant/gemm_xdl_requant_relu_requant_int8.cpp:29-35,
        // then reference_gemm.hpp:80 type_convert<int8_t> = truncation toward zero.
        float gemm_requant = p[0] * c;
        float relu         = gemm_requant > 0 ? gemm_requant : 0;
        float relu_requant = p[1] * relu;
        float y = relu_requant > 127 ? 127 : relu_requant < -128 ? -128 : relu_requant;
        return static_cast<int8_t>(y);
    }
    case EPI_REQUANT_RELU_REQUANT_RNE: {
        // sat_int8(rne(s1 * relu(rne(s0 * acc)))): same functor with a round-to-nearest-even
        // after each scale and a saturating store.
        float q0 = rne(p[0] * c);
        float r  = q0 > 0 ? q0 : 0;
        float q1 = rne(p[1] * r);
        float y  = q1 > 127 ? 127 : q1 < -128 ? -128 : q1;
        return static_cast<int8_t>(y);
    }
    case EPI_RELU: return static_cast<int8_t>(c > 0 ? c : 0);
    default: return 0;
    }
}

} // namespace ck_oracle
