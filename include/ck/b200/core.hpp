// Core vocabulary of the Composable-Kernel-compatible host API on B200.
//
// These headers are HOST-ONLY C++17 (g++): the CUDA kernels live in libckb200.so behind the C ABI
// of ckb200.h, so ck::half_t can stay _Float16 exactly as in the reference
// (include/ck/utility/data_type.hpp:10-11) and keep its conversion rules.
#pragma once
#include <array>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <type_traits>

// The reference marks its functors __host__ __device__; on the host-only side they are plain functions.
#ifndef __host__
#define __host__
#endif
#ifndef __device__
#define __device__
#endif

namespace ck {

using index_t      = int32_t; // include/ck/ck.hpp:176-177
using long_index_t = int64_t;
using half_t       = _Float16; // utility/data_type.hpp:11
using bhalf_t      = unsigned short; // utility/data_type.hpp:10 (bit pattern of a bfloat16)

// include/ck/ck.hpp:153-159
enum struct InMemoryDataOperationEnum
{
    Set,
    AtomicAdd,
    AtomicMax,
    Add
};

// utility/sequence.hpp:38 - compile-time integer list, used only as a template argument here.
template <index_t... Is>
struct Sequence
{
    static constexpr index_t Size() { return sizeof...(Is); }
    static constexpr index_t At(index_t i)
    {
        constexpr index_t v[] = {Is..., 0};
        return v[i];
    }
};

// utility/number.hpp
template <index_t N>
using Number = std::integral_constant<index_t, N>;

// utility/tuple.hpp:103,170 - used as a type list (DsDataType = ck::Tuple<F16, F16>).
template <typename... Ts>
struct Tuple
{
    static constexpr index_t Size() { return sizeof...(Ts); }
};

template <typename T>
struct tuple_size_of;
template <typename... Ts>
struct tuple_size_of<Tuple<Ts...>>
{
    static constexpr index_t value = sizeof...(Ts);
};

template <typename X, typename Y>
using is_same = std::is_same<X, Y>;

// utility/data_type.hpp:934-997: static_cast, except float <-> bhalf_t (bfloat16 bits, RNE).
template <typename Y, typename X>
inline constexpr Y type_convert(X x)
{
    return static_cast<Y>(x);
}
template <>
inline float type_convert<float, bhalf_t>(bhalf_t x)
{
    const uint32_t bits = static_cast<uint32_t>(x) << 16;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}
template <>
inline bhalf_t type_convert<bhalf_t, float>(float x)
{
    uint32_t bits;
    std::memcpy(&bits, &x, 4);
    if(~bits & 0x7f800000u)
        bits += 0x7fffu + ((bits >> 16) & 1u); // zero, normal or subnormal: round to nearest even
    else if(bits & 0xffffu)
        bits |= 0x10000u; // NaN whose payload sits in the low half: keep it a NaN
    return static_cast<bhalf_t>(bits >> 16);
}

namespace math {
template <typename T>
inline constexpr T integer_divide_ceil(T a, T b)
{
    return (a + b - 1) / b;
}
} // namespace math

} // namespace ck

// include/ck/stream_config.hpp:9-13; the stream is a cudaStream_t carried as void* so that host
// code needs no CUDA headers.
struct StreamConfig
{
    void* stream_id_  = nullptr;
    bool time_kernel_ = false;
};
