// Device-side fused epilogues.  Each function is the device twin of a Composable Kernel
// element-wise functor (citations in include/ckb200.h next to the CKB_EPI_* ids) and is
// written operation by operation like the host functor: fp32 arithmetic without fused
// multiply-add (the library is compiled with -fmad=false), binary16 arithmetic through the
// correctly rounded __hadd, one final rounding to the output type.
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/ckb200.h"
#include "ckb_ptx.cuh"

namespace ckb {

struct EpilogueArgs
{
    int32_t kind;   // CKB_EPI_*
    int32_t out_i8; // 1: E is int8 (accumulator is int32), 0: E is 16-bit float
    int32_t bf16;   // 1: 16-bit float type is bfloat16
    int32_t pad_;
    float p[4];
    void* e;
    const void* d0;
    const void* d1;
    int64_t lde, ldd0, ldd1; // row strides in elements (ldd = 0: broadcast row)
};

__host__ __device__ constexpr int epi_num_d(int kind)
{
    return (kind == CKB_EPI_ADD || kind == CKB_EPI_ADD_RELU_F16 || kind == CKB_EPI_BILINEAR ||
            kind == CKB_EPI_ADD_RELU || kind == CKB_EPI_ADD_HARDSWISH)
               ? 1
               : (kind == CKB_EPI_ADD_ADD_FASTGELU || kind == CKB_EPI_ADD_RELU_ADD) ? 2 : 0;
}

// FastGelu with the hardware exponential (ex2.approx) and approximate divide: both are accurate to
// about 2 float ulp, three orders of magnitude inside the 1e-3 check of the binary16 result.
__device__ __forceinline__ float fast_gelu_dev(float x)
{
    const float u   = 2.0f * x * (0.035677f * x * x + 0.797885f);
    const float emu = __expf(-u);
    const float cdf = 0.5f + 0.5f * (__fdividef(2.0f, 1.0f + emu) - 1.0f);
    return x * cdf;
}

// 16-bit float helpers (T = __half or __nv_bfloat16)
template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ __half from_f32<__half>(float x)
{
    return __float2half_rn(x);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x)
{
    return __float2bfloat16_rn(x);
}
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }

// One output element, 16-bit float output.
template <int EPI, typename T>
__device__ __forceinline__ T epi_apply_f(float c, T d0, T d1, const float* p)
{
    if constexpr(EPI == CKB_EPI_PASSTHROUGH)
        return from_f32<T>(c);
    else if constexpr(EPI == CKB_EPI_SCALE)
        return from_f32<T>(p[0] * c);
    else if constexpr(EPI == CKB_EPI_RELU)
        return from_f32<T>(c > 0.0f ? c : 0.0f);
    else if constexpr(EPI == CKB_EPI_FASTGELU)
        return from_f32<T>(fast_gelu_dev(c));
    else if constexpr(EPI == CKB_EPI_ADD)
        return __hadd(from_f32<T>(c), d0);
    else if constexpr(EPI == CKB_EPI_ADD_RELU_F16)
    {
        const T x = __hadd(from_f32<T>(c), d0);
        return to_f32(x) > 0.0f ? x : from_f32<T>(0.0f);
    }
    else if constexpr(EPI == CKB_EPI_BILINEAR)
        return from_f32<T>(p[0] * c + p[1] * to_f32(d0));
    else if constexpr(EPI == CKB_EPI_ADD_ADD_FASTGELU)
        return from_f32<T>(fast_gelu_dev(c + to_f32(d0) + to_f32(d1)));
    else if constexpr(EPI == CKB_EPI_ADD_RELU_ADD)
    {
        const float a = c + to_f32(d0);
        const float b = a > 0.0f ? a : 0.0f;
        return from_f32<T>(b + to_f32(d1));
    }
    else if constexpr(EPI == CKB_EPI_ADD_RELU)
    {
        const float a = c + to_f32(d0);
        return from_f32<T>(a > 0.0f ? a : 0.0f);
    }
    else if constexpr(EPI == CKB_EPI_ADD_HARDSWISH)
    {
        const float a = c + to_f32(d0);
        const float b = a + 3.0f;
        const float y = (b > 0.0f ? 1.0f : 0.0f) * (b > 6.0f ? 6.0f : b) * a * 0.166667f;
        return from_f32<T>(y);
    }
    else
        return from_f32<T>(c);
}

// One output element, int8 output, int32 accumulator.
template <int EPI>
__device__ __forceinline__ int32_t epi_apply_i8(int32_t acc, const float* p)
{
    if constexpr(EPI == CKB_EPI_REQUANT_RELU_REQUANT)
    {
        const float c            = __int2float_rn(acc);
        const float gemm_requant = __fmul_rn(p[0], c);
        const float relu         = gemm_requant > 0.0f ? gemm_requant : 0.0f;
        const float relu_requant = __fmul_rn(p[1], relu);
        const float y =
            relu_requant > 127.0f ? 127.0f : relu_requant < -128.0f ? -128.0f : relu_requant;
        return __float2int_rz(y); // static_cast<int8_t>(float): toward zero
    }
    else if constexpr(EPI == CKB_EPI_REQUANT_RELU_REQUANT_RNE)
    {
        const float c  = __int2float_rn(acc);
        const float q0 = rintf(__fmul_rn(p[0], c)); // round-to-nearest-even
        const float r  = q0 > 0.0f ? q0 : 0.0f;
        const float q1 = rintf(__fmul_rn(p[1], r));
        const float y  = q1 > 127.0f ? 127.0f : q1 < -128.0f ? -128.0f : q1;
        return __float2int_rz(y);
    }
    else if constexpr(EPI == CKB_EPI_RELU)
    {
        const float c = __int2float_rn(acc);
        return __float2int_rz(c > 0.0f ? c : 0.0f);
    }
    else
        return acc; // PassThrough: the store keeps the low 8 bits (static_cast<int8_t>(int32))
}

// D values of one row segment of 32 columns, fetched ahead of the accumulator read so that the
// global-memory latency overlaps the previous segment's arithmetic.  Only the LAST D tensor of the
// functor travels ahead (D1 of a two-D functor, D0 of a one-D functor): the other one is, in the
// fused-bias functors, a broadcast row that stays in L1.
struct DChunk
{
    uint4 d[4];
};

template <int EPI, typename T>
__device__ __forceinline__ void epi_load_d(DChunk& dc, const EpilogueArgs& ea, int64_t m, int64_t n0)
{
    constexpr int ND = epi_num_d(EPI);
    const T* base    = ND >= 2 ? static_cast<const T*>(ea.d1) + m * ea.ldd1 + n0
                               : static_cast<const T*>(ea.d0) + m * ea.ldd0 + n0;
    const uint4* p   = reinterpret_cast<const uint4*>(base);
#pragma unroll
    for(int j = 0; j < 4; ++j)
        dc.d[j] = __ldg(p + j);
}

__device__ __forceinline__ void prefetch_l2(const void* p)
{
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// Asks L2 for the D values of a row segment of `nbytes` bytes that a later tile will read
// (elem_bytes = size of one D element).
__device__ __forceinline__ void epi_prefetch_d(const EpilogueArgs& ea, int64_t m, int64_t n0,
                                               int nbytes, int elem_bytes)
{
    const int nd = epi_num_d(ea.kind);
    if(nd >= 1 && ea.ldd0 != 0)
    {
        const char* p = static_cast<const char*>(ea.d0) + (m * ea.ldd0 + n0) * elem_bytes;
        for(int b = 0; b < nbytes; b += 128)
            prefetch_l2(p + b);
    }
    if(nd >= 2 && ea.ldd1 != 0)
    {
        const char* p = static_cast<const char*>(ea.d1) + (m * ea.ldd1 + n0) * elem_bytes;
        for(int b = 0; b < nbytes; b += 128)
            prefetch_l2(p + b);
    }
}

// Full 32-column segment of one row: the functor applied to 32 accumulators, packed as 4 x 128 bits of E.
// 128-bit D accesses; the last D tensor is already in registers.
template <int EPI, typename T>
__device__ __forceinline__ void epi_compute_vec_f(uint4 (&out)[4], const uint32_t (&v)[32], const DChunk& dc,
                                                  const EpilogueArgs& ea, int64_t m, int64_t n0)
{
    constexpr int ND = epi_num_d(EPI);
    const uint4* d0p = ND >= 2 ? reinterpret_cast<const uint4*>(static_cast<const T*>(ea.d0) + m * ea.ldd0 + n0)
                               : nullptr;
#pragma unroll
    for(int j = 0; j < 4; ++j) // 4 x 8 elements = 4 x 128-bit
    {
        uint4 q0 = dc.d[j], q1 = dc.d[j];
        if constexpr(ND >= 2)
            q0 = __ldg(d0p + j);
        const T* h0 = reinterpret_cast<const T*>(&q0);
        const T* h1 = reinterpret_cast<const T*>(&q1);
        T* ho       = reinterpret_cast<T*>(&out[j]);
#pragma unroll
        for(int i = 0; i < 8; ++i)
            ho[i] = epi_apply_f<EPI, T>(__uint_as_float(v[j * 8 + i]), h0[i], h1[i], ea.p);
    }
}

// Ragged or unaligned segment of `ncols` (<= 32) columns, element by element.
template <int EPI, typename T>
__device__ __forceinline__ void epi_store_scalar_f(const uint32_t (&v)[32], const EpilogueArgs& ea,
                                                   int64_t m, int64_t n0, int ncols)
{
    constexpr int ND = epi_num_d(EPI);
    T* e_row         = static_cast<T*>(ea.e) + m * ea.lde + n0;
    const T* d0_row  = ND >= 1 ? static_cast<const T*>(ea.d0) + m * ea.ldd0 + n0 : nullptr;
    const T* d1_row  = ND >= 2 ? static_cast<const T*>(ea.d1) + m * ea.ldd1 + n0 : nullptr;
#pragma unroll
    for(int i = 0; i < 32; ++i)
    {
        if(i < ncols)
        {
            T a = from_f32<T>(0.0f), b = from_f32<T>(0.0f);
            if constexpr(ND >= 1)
                a = d0_row[i];
            if constexpr(ND >= 2)
                b = d1_row[i];
            e_row[i] = epi_apply_f<EPI, T>(__uint_as_float(v[i]), a, b, ea.p);
        }
    }
}

// int8: full 32-column segment of one row packed as 2 x 128 bits of E.
template <int EPI>
__device__ __forceinline__ void epi_compute_vec_i8(uint4 (&out)[2], const uint32_t (&v)[32], const EpilogueArgs& ea)
{
#pragma unroll
    for(int j = 0; j < 2; ++j) // 2 x 16 elements = 2 x 128-bit
    {
        uint32_t w[4];
#pragma unroll
        for(int k = 0; k < 4; ++k)
        {
            uint32_t packed = 0;
#pragma unroll
            for(int i = 0; i < 4; ++i)
            {
                const int32_t r = epi_apply_i8<EPI>(static_cast<int32_t>(v[j * 16 + k * 4 + i]), ea.p);
                packed |= (static_cast<uint32_t>(r) & 0xFFu) << (8 * i);
            }
            w[k] = packed;
        }
        out[j] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// int8: ragged or unaligned segment, element by element.
template <int EPI>
__device__ __forceinline__ void epi_store_scalar_i8(const uint32_t (&v)[32], const EpilogueArgs& ea, int64_t m,
                                                    int64_t n0, int ncols)
{
    int8_t* e_row = static_cast<int8_t*>(ea.e) + m * ea.lde + n0;
#pragma unroll
    for(int i = 0; i < 32; ++i)
        if(i < ncols)
            e_row[i] = static_cast<int8_t>(epi_apply_i8<EPI>(static_cast<int32_t>(v[i]), ea.p));
}

// ---- staged stores --------------------------------------------------------------------------------
// A full segment (32 rows of one warp x 32 columns) is written to a per-warp shared-memory tile and
// leaves through one TMA store, so that E is written in whole row pieces by the copy unit instead
// of 32 scattered 16-byte pieces per instruction; rows and columns beyond the tensor are clipped by the
// tensor map.  The tile is laid out the way a TMA box with the matching swizzle mode reads it (rows of 64
// bytes with CU_TENSOR_MAP_SWIZZLE_64B: 16-byte chunk index ^= (row >> 1) & 3; rows of 32 bytes with
// SWIZZLE_32B: chunk index ^= (row >> 2) & 1), which also makes the 128-bit shared-memory writes of a warp
// free of bank conflicts.  Two tiles per warp alternate.
struct StoreStage
{
    uint32_t buf;            // shared-memory address of this warp's two tiles (2 x 2 KiB, 1 KiB aligned)
    uint32_t count;          // segments stored so far by this warp
    const CUtensorMap* tm_e; // E as (columns, rows[, batch]) with a 32 x 32 box
    int batch;               // >= 0: third coordinate of a batched E map; < 0: 2-D map
};

template <int ROW_BYTES> // 64: 16-bit E, 32: int8 E
__device__ __forceinline__ void stage_and_store(StoreStage& st, const uint4* out, int lane, int col0, int row0)
{
    constexpr int CHUNKS = ROW_BYTES / 16;
    const uint32_t tile  = st.buf + (st.count & 1u) * 2048u;
    // the store issued two segments ago has to be done reading this tile
    if(lane == 0)
        bulk_wait_group_read<1>();
    __syncwarp();
#pragma unroll
    for(int c = 0; c < CHUNKS; ++c)
    {
        const int sw = ROW_BYTES == 64 ? (c ^ ((lane >> 1) & 3)) : (c ^ ((lane >> 2) & 1));
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tile + lane * ROW_BYTES + sw * 16), "r"(out[c].x),
                     "r"(out[c].y), "r"(out[c].z), "r"(out[c].w)
                     : "memory");
    }
    fence_proxy_async_smem(); // generic-proxy writes -> visible to the copy unit
    __syncwarp();
    if(lane == 0)
    {
        if(st.batch >= 0)
            tma_store_3d(st.tm_e, tile, col0, row0, st.batch);
        else
            tma_store_2d(st.tm_e, tile, col0, row0);
        bulk_commit_group();
    }
    ++st.count;
}

} // namespace ckb
