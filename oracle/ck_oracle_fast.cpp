// TEST INFRASTRUCTURE - CPU oracle.  Not part of the shipped library: only tests/,
// __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm may use it.
//
// Blocked form of the oracle in ck_oracle.cpp, used to verify full-size outputs in seconds.
// It keeps the reference's numerical contract: every output element is accumulated in a
// float, over k in increasing order, one product at a time (reference_gemm.hpp:62-74;
// reference_conv_fwd.hpp:135-164 for the c -> y -> x order of the convolution).  Only the
// order in which DIFFERENT outputs are visited changes (register tiles of 6 x 16 outputs).
//
// Fused multiply-add is used in the inner loop.  That is exact here because the product of
// two binary16 (or bfloat16, or int8) values is representable in binary32 without rounding, so
// fma(a,b,acc) == acc + a*b bit for bit.  tests/test_oracle_golden.py asserts fast == naive
// bit-for-bit on small shapes.
//
// Skipped convolution taps are multiplied by an explicit zero instead of being skipped;
// acc + 0.0f == acc for every acc except -0.0f, whose sign no epilogue or checker observes.
#include "ck_epilogue.h"

#include <immintrin.h>

#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

using namespace ck_oracle;

namespace {

constexpr int MR = 6;   // rows of one register tile
constexpr int NR = 16;  // columns of one register tile (two 8-float vectors)
constexpr int KC = 256; // k block kept in cache; blocks are visited in increasing k

// acc[MR][NR] += sum_{k<kc} a[r*lda + k] * bp[k*NR + j], k increasing.
__attribute__((target("avx2,fma"))) void micro_kernel(int kc, const float* a, int64_t lda,
                                                      const float* bp, float* c, int64_t ldc,
                                                      int mr)
{
    __m256 acc[MR][2];
    for(int r = 0; r < MR; ++r)
    {
        if(r < mr)
        {
            acc[r][0] = _mm256_loadu_ps(c + r * ldc);
            acc[r][1] = _mm256_loadu_ps(c + r * ldc + 8);
        }
        else
        {
            acc[r][0] = _mm256_setzero_ps();
            acc[r][1] = _mm256_setzero_ps();
        }
    }
    const float* ar[MR];
    for(int r = 0; r < MR; ++r)
        ar[r] = a + (r < mr ? r : 0) * lda;
    for(int k = 0; k < kc; ++k)
    {
        const __m256 b0 = _mm256_loadu_ps(bp + k * NR);
        const __m256 b1 = _mm256_loadu_ps(bp + k * NR + 8);
        for(int r = 0; r < MR; ++r)
        {
            const __m256 av = _mm256_broadcast_ss(ar[r] + k);
            acc[r][0]       = _mm256_fmadd_ps(av, b0, acc[r][0]);
            acc[r][1]       = _mm256_fmadd_ps(av, b1, acc[r][1]);
        }
    }
    for(int r = 0; r < mr; ++r)
    {
        _mm256_storeu_ps(c + r * ldc, acc[r][0]);
        _mm256_storeu_ps(c + r * ldc + 8, acc[r][1]);
    }
}

template <typename F>
void run_threads(int threads, F f)
{
    if(threads < 1)
        threads = 1;
    std::vector<std::thread> pool;
    for(int t = 0; t < threads; ++t)
        pool.emplace_back([=] { f(t); });
    for(auto& t : pool)
        t.join();
}

// Af: M x K float row-major (ld K).  Bp: packed panels, panel j holds columns [j*NR, j*NR+NR)
// as K x NR floats (zero padded).  Writes Cf (M x Npad, fp32 accumulators).
void gemm_f32_blocked(const float* Af, const float* Bp, float* Cf, int64_t M, int64_t Npad,
                      int64_t K, int threads)
{
    const int64_t n_panels = Npad / NR;
    const int64_t m_blocks = (M + MR - 1) / MR;
    // Work item = a strip of 8 register-tile rows (48 rows) over all of N and K.
    const int64_t strip    = 8;
    const int64_t n_strips = (m_blocks + strip - 1) / strip;
    std::atomic<int64_t> next{0};
    std::atomic<int64_t>* pnext = &next;
    run_threads(threads, [=](int) {
        for(;;)
        {
            const int64_t s = pnext->fetch_add(1);
            if(s >= n_strips)
                break;
            const int64_t mb0 = s * strip, mb1 = std::min(m_blocks, mb0 + strip);
            for(int64_t k0 = 0; k0 < K; k0 += KC) // increasing k: per-output order is preserved
            {
                const int kc = static_cast<int>(std::min<int64_t>(KC, K - k0));
                for(int64_t j = 0; j < n_panels; ++j)
                {
                    const float* bp = Bp + (j * K + k0) * NR;
                    for(int64_t mb = mb0; mb < mb1; ++mb)
                    {
                        const int64_t m0 = mb * MR;
                        const int mr     = static_cast<int>(std::min<int64_t>(MR, M - m0));
                        micro_kernel(kc, Af + m0 * K + k0, K, bp, Cf + m0 * Npad + j * NR, Npad, mr);
                    }
                }
            }
        }
    });
}

template <typename T>
inline float to_f32(T v)
{
    return static_cast<float>(v);
}

} // namespace

extern "C" {

// Same contract as oracle_gemm_naive.  int8 inputs accumulate in float, which equals the int32
// accumulation while every partial sum stays below 2^24; the function returns 2 (and computes
// nothing) when K * max|a| * max|b| could exceed that.
int oracle_gemm_fast(int ab_dtype, int epi, const float* params,
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
    if(ab_dtype != 0 && ab_dtype != 1 && ab_dtype != 2)
        return 1;
    if(M <= 0 || N <= 0)
        return 0;
    const int64_t Npad = (N + NR - 1) / NR * NR;
    std::vector<float> Af(static_cast<size_t>(M) * std::max<int64_t>(K, 1));
    std::vector<float> Bp(static_cast<size_t>(Npad) * std::max<int64_t>(K, 1), 0.0f);
    std::vector<float> Cf(static_cast<size_t>(M) * Npad, 0.0f);
    float* Afp = Af.data();
    float* Bpp = Bp.data();
    float* Cfp = Cf.data();

    if(ab_dtype == 1)
    {
        const int8_t* A = static_cast<const int8_t*>(a);
        const int8_t* B = static_cast<const int8_t*>(b);
        int amax = 0, bmax = 0;
        for(int64_t m = 0; m < M; ++m)
            for(int64_t k = 0; k < K; ++k)
                amax = std::max(amax, std::abs(static_cast<int>(A[m * a_sm + k * a_sk])));
        for(int64_t k = 0; k < K; ++k)
            for(int64_t n = 0; n < N; ++n)
                bmax = std::max(bmax, std::abs(static_cast<int>(B[k * b_sk + n * b_sn])));
        if(static_cast<double>(K) * amax * bmax >= 16777216.0)
            return 2;
    }

    // Convert and pack (parallel over rows / panels).
    std::atomic<int64_t> next_a{0}, next_b{0};
    std::atomic<int64_t>*pa = &next_a, *pb = &next_b;
    run_threads(threads, [=](int) {
        for(;;)
        {
            const int64_t m = pa->fetch_add(1);
            if(m >= M)
                break;
            if(ab_dtype == 0)
            {
                const half* A = static_cast<const half*>(a);
                for(int64_t k = 0; k < K; ++k)
                    Afp[m * K + k] = to_f32(A[m * a_sm + k * a_sk]);
            }
            else if(ab_dtype == 2)
            {
                const bf16* A = static_cast<const bf16*>(a);
                for(int64_t k = 0; k < K; ++k)
                    Afp[m * K + k] = bf16_to_float(A[m * a_sm + k * a_sk]);
            }
            else
            {
                const int8_t* A = static_cast<const int8_t*>(a);
                for(int64_t k = 0; k < K; ++k)
                    Afp[m * K + k] = to_f32(A[m * a_sm + k * a_sk]);
            }
        }
        for(;;)
        {
            const int64_t j = pb->fetch_add(1);
            if(j >= Npad / NR)
                break;
            const int64_t ncols = std::min<int64_t>(NR, N - j * NR);
            for(int64_t k = 0; k < K; ++k)
                for(int64_t c = 0; c < ncols; ++c)
                {
                    const int64_t n = j * NR + c;
                    Bpp[(j * K + k) * NR + c] =
                        ab_dtype == 0   ? to_f32(static_cast<const half*>(b)[k * b_sk + n * b_sn])
                        : ab_dtype == 2 ? bf16_to_float(static_cast<const bf16*>(b)[k * b_sk + n * b_sn])
                                        : to_f32(static_cast<const int8_t*>(b)[k * b_sk + n * b_sn]);
                }
        }
    });

    if(K > 0)
        gemm_f32_blocked(Afp, Bpp, Cfp, M, Npad, K, threads);

    std::atomic<int64_t> next_m{0};
    std::atomic<int64_t>* pm = &next_m;
    run_threads(threads, [=](int) {
        for(;;)
        {
            const int64_t m = pm->fetch_add(1);
            if(m >= M)
                break;
            if(ab_dtype == 2)
            {
                const bf16* D0 = static_cast<const bf16*>(d0);
                const bf16* D1 = static_cast<const bf16*>(d1);
                bf16* E        = static_cast<bf16*>(e);
                for(int64_t n = 0; n < N; ++n)
                {
                    const bf16 v_d0 = D0 ? D0[m * d0_sm + n * d0_sn] : bf16{0};
                    const bf16 v_d1 = D1 ? D1[m * d1_sm + n * d1_sn] : bf16{0};
                    E[m * e_sm + n * e_sn] = apply_bf16(epi, p, Cfp[m * Npad + n], v_d0, v_d1);
                }
            }
            else if(ab_dtype == 0)
            {
                const half* D0 = static_cast<const half*>(d0);
                const half* D1 = static_cast<const half*>(d1);
                half* E        = static_cast<half*>(e);
                for(int64_t n = 0; n < N; ++n)
                {
                    const half v_d0 = D0 ? D0[m * d0_sm + n * d0_sn] : static_cast<half>(0);
                    const half v_d1 = D1 ? D1[m * d1_sm + n * d1_sn] : static_cast<half>(0);
                    E[m * e_sm + n * e_sn] = apply_f16(epi, p, Cfp[m * Npad + n], v_d0, v_d1);
                }
            }
            else
            {
                int8_t* E = static_cast<int8_t*>(e);
                for(int64_t n = 0; n < N; ++n)
                    E[m * e_sm + n * e_sn] =
                        apply_i8(epi, p, static_cast<int32_t>(Cfp[m * Npad + n]));
            }
        }
    });
    return 0;
}

// Same contract as oracle_conv2d_fwd_naive.  The input is expanded row-chunk by row-chunk into
// an explicit (pixels) x (C*Y*X) matrix whose columns are ordered c -> y -> x, so that the
// blocked GEMM above accumulates every output in the reference's order.
int oracle_conv2d_fwd_fast(int epi, const float* params,
                           const void* in, const void* wei, void* out,
                           const void* bias, const void* resi,
                           int N, int K, int C, int Hi, int Wi, int Y, int X, int Ho, int Wo,
                           int sh, int sw, int dh, int dw, int ph, int pw, int threads)
{
    float p[4] = {0, 0, 0, 0};
    if(params)
        std::memcpy(p, params, sizeof(p));
    const half* In   = static_cast<const half*>(in);
    const half* Wei  = static_cast<const half*>(wei);
    const half* Bias = static_cast<const half*>(bias);
    const half* Resi = static_cast<const half*>(resi);
    half* Out        = static_cast<half*>(out);

    const int64_t GK   = static_cast<int64_t>(C) * Y * X;
    const int64_t GM   = static_cast<int64_t>(N) * Ho * Wo;
    const int64_t Npad = (static_cast<int64_t>(K) + NR - 1) / NR * NR;
    if(GM <= 0 || K <= 0)
        return 0;

    // Weights -> packed panels with gemm-k index (c*Y + y)*X + x.
    std::vector<float> Bp(static_cast<size_t>(Npad) * GK, 0.0f);
    for(int64_t k = 0; k < K; ++k)
        for(int c = 0; c < C; ++c)
            for(int y = 0; y < Y; ++y)
                for(int x = 0; x < X; ++x)
                {
                    const int64_t gk = (static_cast<int64_t>(c) * Y + y) * X + x;
                    Bp[((k / NR) * GK + gk) * NR + (k % NR)] =
                        static_cast<float>(Wei[((k * Y + y) * X + x) * C + c]);
                }

    const int64_t chunk = 16384; // output pixels expanded at a time
    std::vector<float> Af(static_cast<size_t>(std::min(chunk, GM)) * GK);
    std::vector<float> Cf(static_cast<size_t>(std::min(chunk, GM)) * Npad);
    float* Afp       = Af.data();
    float* Cfp       = Cf.data();
    const float* Bpp = Bp.data();

    for(int64_t m0 = 0; m0 < GM; m0 += chunk)
    {
        const int64_t mc = std::min(chunk, GM - m0);
        std::fill(Cf.begin(), Cf.begin() + mc * Npad, 0.0f);
        std::atomic<int64_t> next{0};
        std::atomic<int64_t>* pn = &next;
        run_threads(threads, [=](int) {
            for(;;)
            {
                const int64_t r = pn->fetch_add(1);
                if(r >= mc)
                    break;
                const int64_t m = m0 + r;
                const int wo    = static_cast<int>(m % Wo);
                const int ho    = static_cast<int>((m / Wo) % Ho);
                const int n     = static_cast<int>(m / (static_cast<int64_t>(Wo) * Ho));
                float* row      = Afp + r * GK;
                for(int c = 0; c < C; ++c)
                    for(int y = 0; y < Y; ++y)
                    {
                        const int64_t hi = static_cast<int64_t>(ho) * sh + static_cast<int64_t>(y) * dh - ph;
                        for(int x = 0; x < X; ++x)
                        {
                            const int64_t wi =
                                static_cast<int64_t>(wo) * sw + static_cast<int64_t>(x) * dw - pw;
                            float v = 0.0f;
                            if(hi >= 0 && hi < Hi && wi >= 0 && wi < Wi)
                                v = static_cast<float>(
                                    In[((static_cast<int64_t>(n) * Hi + hi) * Wi + wi) * C + c]);
                            row[(static_cast<int64_t>(c) * Y + y) * X + x] = v;
                        }
                    }
            }
        });
        gemm_f32_blocked(Afp, Bpp, Cfp, mc, Npad, GK, threads);
        std::atomic<int64_t> next_o{0};
        std::atomic<int64_t>* po = &next_o;
        run_threads(threads, [=](int) {
            for(;;)
            {
                const int64_t r = po->fetch_add(1);
                if(r >= mc)
                    break;
                const int64_t m = m0 + r;
                for(int k = 0; k < K; ++k)
                {
                    const int64_t o = m * K + k;
                    const half v_d0 = Bias ? Bias[k] : static_cast<half>(0);
                    const half v_d1 = Resi ? Resi[o] : static_cast<half>(0);
                    Out[o]          = apply_f16(epi, p, Cfp[r * Npad + k], v_d0, v_d1);
                }
            }
        });
    }
    return 0;
}

} // extern "C"
