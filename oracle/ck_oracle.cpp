// TEST INFRASTRUCTURE - CPU oracle.  Not part of the shipped library: only tests/,
// __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm may use it.
//
// CPU restatement ("port") of Composable Kernel's host reference operators for the dense
// contraction path.  The reference headers need clang/hipcc extensions and do not compile
// with g++, so the algorithm is restated here, function by function:
//
//   oracle_gemm            <- ReferenceGemm::Invoker::Run
//                             library/include/ck/library/reference_tensor_operation/cpu/reference_gemm.hpp:57-88
//   oracle_conv2d_fwd      <- ReferenceConvFwd (2-D branch)            .../cpu/reference_conv_fwd.hpp:132-185
//                             ReferenceConvFwd_Bias_Activation         .../cpu/reference_conv_fwd_bias_activation.hpp:74-128
//   thread partition       <- ParallelTensorFunctor                    library/include/ck/library/host_tensor/host_tensor.hpp:142-194
//   oracle_conv_out_len    <- ConvParams::GetOutputSpatialLengths      library/src/utility/conv_util.cpp:84-103
//   oracle_check_err_*     <- ck::utils::check_err                     library/include/ck/library/utility/check_err.hpp:107-193
//
// Parity pins: the conv restatement reproduces the reference's own golden vectors
// (test/reference_conv_fwd/reference_conv_fwd.cpp:94-154) and the output-length table of
// test/conv_util/conv_util.cpp:43-122; see tests/test_oracle_golden.py.  The reference holds no
// golden vectors for ReferenceGemm or for the fused functors; those are pinned by hand-computed
// known-answer cases in the same test file.
//
// This translation unit is the literal ("naive") form: one output element at a time, a
// sequential k loop with a float (or int32) accumulator, no fused multiply-add.
// ck_oracle_fast.cpp holds a blocked form with the same per-output accumulation order.
#include "ck_epilogue.h"

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <thread>
#include <type_traits>
#include <vector>

namespace ck_oracle {

// host_tensor.hpp:174-193: the flattened index space is cut into equal contiguous chunks,
// one std::thread per chunk.
template <typename F>
void parallel_for(int64_t total, int num_thread, F f)
{
    if(num_thread < 1)
        num_thread = 1;
    int64_t work_per_thread = (total + num_thread - 1) / num_thread;
    std::vector<std::thread> threads;
    for(int it = 0; it < num_thread; ++it)
    {
        int64_t begin = it * work_per_thread;
        int64_t end   = std::min<int64_t>((it + 1) * work_per_thread, total);
        if(begin >= end)
            break;
        threads.emplace_back([=] {
            for(int64_t i = begin; i < end; ++i)
                f(i);
        });
    }
    for(auto& t : threads)
        t.join();
}

} // namespace ck_oracle

using namespace ck_oracle;

extern "C" {

int oracle_hardware_concurrency() { return static_cast<int>(std::thread::hardware_concurrency()); }

// E[m,n] = epilogue( sum_k A[m,k]*B[k,n], D0[m,n], D1[m,n] ), any strides (in elements).
// ab_dtype: 0 = binary16 (float accumulate), 1 = int8 (int32 accumulate).
int oracle_gemm_naive(int ab_dtype, int epi, const float* params,
                      const void* a, int64_t a_sm, int64_t a_sk,
                      const void* b, int64_t b_sk, int64_t b_sn,
                      void* e, int64_t e_sm, int64_t e_sn,
                      const void* d0, int64_t d0_sm, int64_t d0_sn,
                      const void* d1, int64_t d1_sm, int64_t d1_sn,
                      int64_t M, int64_t N, int64_t K, int threads)
{
    float p[4] = {0, 0, 0, 0};
    if(params)
        std::memcpy(p, params, sizeof(p));
    if(ab_dtype == 0)
    {
        const half* A  = static_cast<const half*>(a);
        const half* B  = static_cast<const half*>(b);
        const half* D0 = static_cast<const half*>(d0);
        const half* D1 = static_cast<const half*>(d1);
        half* E        = static_cast<half*>(e);
        parallel_for(M * N, threads, [=](int64_t i) {
            const int64_t m = i / N, n = i % N;
            float v_acc = 0; // reference_gemm.hpp:62
            for(int64_t k = 0; k < K; ++k)
            {
                // reference_gemm.hpp:69-73 with PassThrough a/b element ops
                v_acc += static_cast<float>(A[m * a_sm + k * a_sk]) *
                         static_cast<float>(B[k * b_sk + n * b_sn]);
            }
            const half v_d0 = D0 ? D0[m * d0_sm + n * d0_sn] : static_cast<half>(0);
            const half v_d1 = D1 ? D1[m * d1_sm + n * d1_sn] : static_cast<half>(0);
            E[m * e_sm + n * e_sn] = apply_f16(epi, p, v_acc, v_d0, v_d1);
        });
        return 0;
    }
    if(ab_dtype == 1)
    {
        const int8_t* A = static_cast<const int8_t*>(a);
        const int8_t* B = static_cast<const int8_t*>(b);
        int8_t* E       = static_cast<int8_t*>(e);
        parallel_for(M * N, threads, [=](int64_t i) {
            const int64_t m = i / N, n = i % N;
            int32_t v_acc = 0;
            for(int64_t k = 0; k < K; ++k)
                v_acc += static_cast<int32_t>(A[m * a_sm + k * a_sk]) *
                         static_cast<int32_t>(B[k * b_sk + n * b_sn]);
            E[m * e_sm + n * e_sn] = apply_i8(epi, p, v_acc);
        });
        return 0;
    }
    if(ab_dtype == 2) // bfloat16 bit patterns, float accumulate
    {
        const bf16* A  = static_cast<const bf16*>(a);
        const bf16* B  = static_cast<const bf16*>(b);
        const bf16* D0 = static_cast<const bf16*>(d0);
        const bf16* D1 = static_cast<const bf16*>(d1);
        bf16* E        = static_cast<bf16*>(e);
        parallel_for(M * N, threads, [=](int64_t i) {
            const int64_t m = i / N, n = i % N;
            float v_acc = 0;
            for(int64_t k = 0; k < K; ++k)
                v_acc += bf16_to_float(A[m * a_sm + k * a_sk]) * bf16_to_float(B[k * b_sk + n * b_sn]);
            const bf16 v_d0 = D0 ? D0[m * d0_sm + n * d0_sn] : bf16{0};
            const bf16 v_d1 = D1 ? D1[m * d1_sm + n * d1_sn] : bf16{0};
            E[m * e_sm + n * e_sn] = apply_bf16(epi, p, v_acc, v_d0, v_d1);
        });
        return 0;
    }
    return 1;
}

// library/src/utility/conv_util.cpp:84-103 - one spatial dimension.
int oracle_conv_out_len(int in_len, int filter_len, int stride, int dilation, int lpad, int rpad)
{
    const int eff = (filter_len - 1) * dilation + 1;
    return (in_len + lpad + rpad - eff) / stride + 1;
}

// NHWC input, KYXC weights, NHWK output, all packed; float accumulate.
// Loop order c -> y -> x and the skip of out-of-image taps follow reference_conv_fwd.hpp:135-164.
// bias (length K) and resi (N*Ho*Wo*K) may be null; they feed d0 / d1 of the epilogue.
// T = half: any epilogue.  T = float: PassThrough only (the element type of the reference's
// golden-vector test, test/reference_conv_fwd/reference_conv_fwd.cpp:25-33).
} // extern "C"

static inline float elem_to_float(float v) { return v; }
static inline float elem_to_float(half v) { return static_cast<float>(v); }
static inline float elem_to_float(bf16 v) { return bf16_to_float(v); }
static inline float elem_to_float(int8_t v) { return static_cast<float>(v); }

// N-D (1-D, 2-D, 3-D) forward convolution on NDHWC / KZYXC / NDHWK tensors; the 2-D and 1-D cases are the
// 3-D one with depth (and height) 1.  Loop order c -> z -> y -> x as reference_conv_fwd.hpp:132-185 (2-D) and
// :186-254 (3-D); the output is iterated as (n, k, do, ho, wo).
template <typename T>
static int conv3d_fwd_naive_t(int epi, const float* params,
                              const void* in, const void* wei, void* out,
                              const void* bias, const void* resi,
                              int N, int K, int C, int Di, int Hi, int Wi, int Z, int Y, int X,
                              int Do, int Ho, int Wo, int sd, int sh, int sw, int dd, int dh, int dw,
                              int pd, int ph, int pw, int threads)
{
    float p[4] = {0, 0, 0, 0};
    if(params)
        std::memcpy(p, params, sizeof(p));
    const T* In   = static_cast<const T*>(in);
    const T* Wei  = static_cast<const T*>(wei);
    const T* Bias = static_cast<const T*>(bias);
    const T* Resi = static_cast<const T*>(resi);
    T* Out        = static_cast<T*>(out);
    const int64_t total = static_cast<int64_t>(N) * K * Do * Ho * Wo;
    parallel_for(total, threads, [=](int64_t i) {
        const int wo = static_cast<int>(i % Wo);
        const int ho = static_cast<int>((i / Wo) % Ho);
        const int od = static_cast<int>((i / (static_cast<int64_t>(Wo) * Ho)) % Do);
        const int k  = static_cast<int>((i / (static_cast<int64_t>(Wo) * Ho * Do)) % K);
        const int n  = static_cast<int>(i / (static_cast<int64_t>(Wo) * Ho * Do * K));
        float v_acc  = 0;
        for(int c = 0; c < C; ++c)
            for(int z = 0; z < Z; ++z)
            {
                const int64_t di = static_cast<int64_t>(od) * sd + static_cast<int64_t>(z) * dd - pd;
                for(int y = 0; y < Y; ++y)
                {
                    const int64_t hi = static_cast<int64_t>(ho) * sh + static_cast<int64_t>(y) * dh - ph;
                    for(int x = 0; x < X; ++x)
                    {
                        const int64_t wi = static_cast<int64_t>(wo) * sw + static_cast<int64_t>(x) * dw - pw;
                        if(di >= 0 && di < Di && hi >= 0 && hi < Hi && wi >= 0 && wi < Wi)
                        {
                            const float v_in = elem_to_float(
                                In[(((static_cast<int64_t>(n) * Di + di) * Hi + hi) * Wi + wi) * C + c]);
                            const float v_wei = elem_to_float(
                                Wei[(((static_cast<int64_t>(k) * Z + z) * Y + y) * X + x) * C + c]);
                            v_acc += v_in * v_wei;
                        }
                    }
                }
            }
        const int64_t o = (((static_cast<int64_t>(n) * Do + od) * Ho + ho) * Wo + wo) * K + k;
        if constexpr(std::is_same<T, float>::value)
        {
            Out[o] = v_acc; // PassThrough, reference_conv_fwd.hpp:169-172
        }
        else if constexpr(std::is_same<T, int8_t>::value)
        {
            // int8 convolution (example/09_convnd_fwd/convnd_fwd_xdl_int8.cpp:23-26): the reference's float v_acc
            // holds the int32 sum exactly for |sum| < 2^24 (asserted by the tests' value ranges)
            Out[o] = apply_i8(epi, p, static_cast<int32_t>(v_acc));
        }
        else if constexpr(std::is_same<T, bf16>::value)
        {
            const bf16 v_d0 = Bias ? Bias[k] : bf16{0};
            const bf16 v_d1 = Resi ? Resi[o] : bf16{0};
            Out[o]          = apply_bf16(epi, p, v_acc, v_d0, v_d1);
        }
        else
        {
            const half v_d0 = Bias ? Bias[k] : static_cast<half>(0);
            const half v_d1 = Resi ? Resi[o] : static_cast<half>(0);
            Out[o]          = apply_f16(epi, p, v_acc, v_d0, v_d1);
        }
    });
    return 0;
}

template <typename T>
static int conv2d_fwd_naive_t(int epi, const float* params,
                              const void* in, const void* wei, void* out,
                              const void* bias, const void* resi,
                              int N, int K, int C, int Hi, int Wi, int Y, int X, int Ho, int Wo,
                              int sh, int sw, int dh, int dw, int ph, int pw, int threads)
{
    return conv3d_fwd_naive_t<T>(epi, params, in, wei, out, bias, resi, N, K, C, 1, Hi, Wi, 1, Y, X, 1, Ho, Wo, 1,
                                 sh, sw, 1, dh, dw, 0, ph, pw, threads);
}

extern "C" {

int oracle_conv2d_fwd_naive(int epi, const float* params,
                            const void* in, const void* wei, void* out,
                            const void* bias, const void* resi,
                            int N, int K, int C, int Hi, int Wi, int Y, int X, int Ho, int Wo,
                            int sh, int sw, int dh, int dw, int ph, int pw, int threads)
{
    return conv2d_fwd_naive_t<half>(epi, params, in, wei, out, bias, resi, N, K, C, Hi, Wi, Y, X,
                                    Ho, Wo, sh, sw, dh, dw, ph, pw, threads);
}

int oracle_conv2d_fwd_naive_bf16(int epi, const float* params,
                                 const void* in, const void* wei, void* out,
                                 const void* bias, const void* resi,
                                 int N, int K, int C, int Hi, int Wi, int Y, int X, int Ho, int Wo,
                                 int sh, int sw, int dh, int dw, int ph, int pw, int threads)
{
    return conv2d_fwd_naive_t<bf16>(epi, params, in, wei, out, bias, resi, N, K, C, Hi, Wi, Y, X,
                                    Ho, Wo, sh, sw, dh, dw, ph, pw, threads);
}

int oracle_conv2d_fwd_naive_i8(int epi, const float* params,
                               const void* in, const void* wei, void* out,
                               const void* bias, const void* resi,
                               int N, int K, int C, int Hi, int Wi, int Y, int X, int Ho, int Wo,
                               int sh, int sw, int dh, int dw, int ph, int pw, int threads)
{
    return conv2d_fwd_naive_t<int8_t>(epi, params, in, wei, out, bias, resi, N, K, C, Hi, Wi, Y, X,
                                      Ho, Wo, sh, sw, dh, dw, ph, pw, threads);
}

// 3-D forward convolution: dtype 0 = binary16, 1 = int8, 2 = bfloat16 bit patterns, 3 = float (PassThrough only).
int oracle_conv3d_fwd_naive(int dtype, int epi, const float* params,
                            const void* in, const void* wei, void* out, const void* bias, const void* resi,
                            int N, int K, int C, int Di, int Hi, int Wi, int Z, int Y, int X, int Do, int Ho, int Wo,
                            int sd, int sh, int sw, int dd, int dh, int dw, int pd, int ph, int pw, int threads)
{
#define CKO_CONV3D(T)                                                                                             \
    conv3d_fwd_naive_t<T>(epi, params, in, wei, out, bias, resi, N, K, C, Di, Hi, Wi, Z, Y, X, Do, Ho, Wo, sd, sh, \
                          sw, dd, dh, dw, pd, ph, pw, threads)
    switch(dtype)
    {
    case 0: return CKO_CONV3D(half);
    case 1: return CKO_CONV3D(int8_t);
    case 2: return CKO_CONV3D(bf16);
    case 3: return CKO_CONV3D(float);
    default: return 1;
    }
#undef CKO_CONV3D
}

int oracle_conv2d_fwd_naive_f32(const void* in, const void* wei, void* out,
                                int N, int K, int C, int Hi, int Wi, int Y, int X, int Ho, int Wo,
                                int sh, int sw, int dh, int dw, int ph, int pw, int threads)
{
    return conv2d_fwd_naive_t<float>(EPI_PASSTHROUGH, nullptr, in, wei, out, nullptr, nullptr, N, K,
                                     C, Hi, Wi, Y, X, Ho, Wo, sh, sw, dh, dw, ph, pw, threads);
}

// One-element epilogue evaluation, used by the functor known-answer tests and by the test that
// pins the device epilogue to the host functor element by element.
uint16_t oracle_epilogue_f16(int epi, const float* params, float c, uint16_t d0_bits, uint16_t d1_bits)
{
    half d0, d1;
    std::memcpy(&d0, &d0_bits, 2);
    std::memcpy(&d1, &d1_bits, 2);
    half r = apply_f16(epi, params, c, d0, d1);
    uint16_t bits;
    std::memcpy(&bits, &r, 2);
    return bits;
}

int8_t oracle_epilogue_i8(int epi, const float* params, int32_t acc) { return apply_i8(epi, params, acc); }

// check_err.hpp:107-148 (binary16: |o-r| > atol + rtol*|r| or non-finite is an error).
// Returns the number of failing elements; *max_err receives the largest failing error.
int64_t oracle_check_err_f16(const void* out, const void* ref, int64_t count, double rtol,
                             double atol, double* max_err)
{
    const half* O = static_cast<const half*>(out);
    const half* R = static_cast<const half*>(ref);
    int64_t bad   = 0;
    double worst  = 0;
    for(int64_t i = 0; i < count; ++i)
    {
        const double o   = static_cast<float>(O[i]);
        const double r   = static_cast<float>(R[i]);
        const double err = std::abs(o - r);
        if(err > atol + rtol * std::abs(r) || !std::isfinite(o) || !std::isfinite(r))
        {
            worst = std::max(worst, err);
            ++bad;
        }
    }
    if(max_err)
        *max_err = worst;
    return bad;
}

// check_err.hpp:150-193 (integers: exact unless atol given).
int64_t oracle_check_err_i8(const void* out, const void* ref, int64_t count, int64_t atol,
                            int64_t* max_err)
{
    const int8_t* O = static_cast<const int8_t*>(out);
    const int8_t* R = static_cast<const int8_t*>(ref);
    int64_t bad = 0, worst = 0;
    for(int64_t i = 0; i < count; ++i)
    {
        const int64_t err = std::abs(static_cast<int64_t>(O[i]) - static_cast<int64_t>(R[i]));
        if(err > atol)
        {
            worst = std::max(worst, err);
            ++bad;
        }
    }
    if(max_err)
        *max_err = worst;
    return bad;
}

} // extern "C"
