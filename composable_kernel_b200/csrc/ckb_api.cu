// C ABI of the library (include/ckb200.h): argument validation, tensor-map construction and
// kernel launches.  There is no CPU path in this file: every *_run either launches the sm_100a
// kernels or returns an error.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/ckb200.h"
#include "ckb_launch.cuh"

namespace {

using namespace ckb;

thread_local std::string t_last_error;
std::atomic<uint64_t> g_launches{0};

// Device status word read by the kernels through KernelParams::status.
__device__ uint32_t g_status_word;

int fail(int code, const char* fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    t_last_error = buf;
    return code;
}

#define CKB_CUDA(expr)                                                                          \
    do                                                                                          \
    {                                                                                           \
        cudaError_t e__ = (expr);                                                               \
        if(e__ != cudaSuccess)                                                                  \
            return fail(CKB_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));         \
    } while(0)

// ---- driver entry points for tensor-map encoding (no link-time libcuda dependency) -------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                   cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn g_encode_tiled   = nullptr;
EncodeIm2colFn g_encode_im2col = nullptr;
std::once_flag g_entry_once;
int g_driver_version = 0;

void load_entry_points()
{
    std::call_once(g_entry_once, [] {
        void* fn                            = nullptr;
        cudaDriverEntryPointQueryResult qres = cudaDriverEntryPointSymbolNotFound;
        if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) ==
               cudaSuccess &&
           qres == cudaDriverEntryPointSuccess)
            g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
        fn = nullptr;
        if(cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &qres) ==
               cudaSuccess &&
           qres == cudaDriverEntryPointSuccess)
            g_encode_im2col = reinterpret_cast<EncodeIm2colFn>(fn);
        cudaDriverGetVersion(&g_driver_version);
    });
}

// Scratch of the K-split tail (parked accumulator slices + one counter per tail tile), one buffer per stream:
// launches on one stream run one after the other, launches on different streams must not share it.
struct Scratch
{
    void* ptr    = nullptr;
    size_t bytes = 0;
};

struct DeviceInfo
{
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    uint32_t* status = nullptr;
    bool ready       = false;
    std::map<cudaStream_t, Scratch> scratch;
};
DeviceInfo g_dev[64];
std::mutex g_dev_mutex;

int current_device(DeviceInfo** out)
{
    int dev = 0;
    CKB_CUDA(cudaGetDevice(&dev));
    if(dev < 0 || dev >= 64)
        return fail(CKB_ERR_INVALID, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceInfo& d = g_dev[dev];
    if(!d.ready)
    {
        cudaDeviceProp prop;
        CKB_CUDA(cudaGetDeviceProperties(&prop, dev));
        d.sm_count = prop.multiProcessorCount;
        d.cc_major = prop.major;
        d.cc_minor = prop.minor;
        if(prop.major != 10)
            return fail(CKB_ERR_UNSUPPORTED,
                        "device '%s' is compute capability %d.%d; this library holds sm_100a code only",
                        prop.name, prop.major, prop.minor);
        void* sym = nullptr;
        CKB_CUDA(cudaGetSymbolAddress(&sym, g_status_word));
        d.status = static_cast<uint32_t*>(sym);
        CKB_CUDA(cudaMemset(d.status, 0, sizeof(uint32_t)));
        d.ready = true;
    }
    *out = &d;
    return CKB_OK;
}

// True while `stream` records into a CUDA graph (a failed query counts as capturing: nothing is allocated then).
bool stream_is_capturing(cudaStream_t stream)
{
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if(cudaStreamIsCapturing(stream, &st) != cudaSuccess)
    {
        cudaGetLastError();
        return true;
    }
    return st != cudaStreamCaptureStatusNone;
}

constexpr size_t kScratchCounterBytes = 4096; // 1024 tail-tile counters at the front of a scratch buffer

// Grow-only scratch of `stream` with room for `bytes` after the counters; nullptr when the device has no memory
// left for it (the caller then falls back to a plan that needs none).  The counters are zero on return the
// first time and are left at zero by every kernel that uses them.
void* scratch_for(DeviceInfo* dev, cudaStream_t stream, size_t bytes)
{
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    Scratch& sc       = dev->scratch[stream];
    const size_t need = kScratchCounterBytes + bytes;
    // A launch that is being captured into a graph gets no scratch: the graph may be replayed on any stream,
    // next to other launches that use this stream's buffer, and a capture must not see an allocation either.
    // The caller then keeps the plan that needs none.
    if(stream_is_capturing(stream))
        return nullptr;
    if(sc.bytes >= need)
        return sc.ptr;
    if(sc.ptr)
    {
        cudaFree(sc.ptr); // synchronises: no kernel is still using the old buffer
        sc.ptr   = nullptr;
        sc.bytes = 0;
    }
    void* ptr = nullptr;
    if(cudaMalloc(&ptr, need) != cudaSuccess)
    {
        cudaGetLastError();
        return nullptr;
    }
    if(cudaMemset(ptr, 0, kScratchCounterBytes) != cudaSuccess)
    {
        cudaFree(ptr);
        return nullptr;
    }
    sc.ptr   = ptr;
    sc.bytes = need;
    return ptr;
}

uint64_t wait_limit_ns()
{
    static uint64_t v = [] {
        const char* s = getenv("CKB_WAIT_LIMIT_MS");
        double ms     = s ? atof(s) : 2000.0;
        if(ms <= 0)
            ms = 2000.0;
        return static_cast<uint64_t>(ms * 1e6);
    }();
    return v;
}

int forced_bn()
{
    const char* s = getenv("CKB_FORCE_BN");
    return s ? atoi(s) : 0;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int elem_bytes(int dtype) { return dtype == CKB_I8 ? 1 : 2; }

CUtensorMapDataType tm_dtype(int dtype)
{
    return dtype == CKB_I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                           : dtype == CKB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

// K-major matrix [rows][k] with row pitch `ld` elements -> 2-D map, box = 128 bytes x box_rows.
// batch >= 1 adds a third dimension of `batch` matrices `batch_stride` elements apart (box extent 1).
int encode_kmajor_2d(CUtensorMap* tm, int dtype, const void* ptr, int64_t rows, int64_t k,
                     int64_t ld, int box_rows, int64_t batch = 0, int64_t batch_stride = 0)
{
    load_entry_points();
    if(!g_encode_tiled)
        return fail(CKB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    const int eb          = elem_bytes(dtype);
    cuuint64_t dims[3]    = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * eb, static_cast<cuuint64_t>(batch_stride) * eb};
    cuuint32_t box[3]     = {static_cast<cuuint32_t>(BK_BYTES / eb), static_cast<cuuint32_t>(box_rows), 1};
    cuuint32_t estr[3]    = {1, 1, 1};
    CUresult r            = g_encode_tiled(tm, tm_dtype(dtype), batch >= 1 ? 3 : 2, const_cast<void*>(ptr), dims, strides,
                                box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if(r != CUDA_SUCCESS)
        return fail(CKB_ERR_CUDA, "cuTensorMapEncodeTiled failed (CUresult %d) rows=%lld k=%lld ld=%lld",
                    static_cast<int>(r), (long long)rows, (long long)k, (long long)ld);
    return CKB_OK;
}

// MN-major matrix (the M or N index contiguous, pitch `ld` elements between consecutive k) -> 2-D map
// whose box is one swizzle atom column: 128 bytes of MN positions x the k rows of one stage.
int encode_mnmajor_2d(CUtensorMap* tm, int dtype, const void* ptr, int64_t mn, int64_t k, int64_t ld,
                      int64_t batch = 0, int64_t batch_stride = 0)
{
    load_entry_points();
    if(!g_encode_tiled)
        return fail(CKB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    const int eb          = elem_bytes(dtype);
    cuuint64_t dims[3]    = {static_cast<cuuint64_t>(mn), static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(batch)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * eb, static_cast<cuuint64_t>(batch_stride) * eb};
    cuuint32_t box[3]     = {static_cast<cuuint32_t>(BK_BYTES / eb), static_cast<cuuint32_t>(BK_BYTES / eb), 1};
    cuuint32_t estr[3]    = {1, 1, 1};
    CUresult r            = g_encode_tiled(tm, tm_dtype(dtype), batch >= 1 ? 3 : 2, const_cast<void*>(ptr), dims, strides,
                                box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if(r != CUDA_SUCCESS)
        return fail(CKB_ERR_CUDA, "cuTensorMapEncodeTiled failed (CUresult %d) mn=%lld k=%lld ld=%lld",
                    static_cast<int>(r), (long long)mn, (long long)k, (long long)ld);
    return CKB_OK;
}

// E (M x N row-major, pitch `lde` elements) as the (columns, rows[, batch]) map of the epilogue's staged stores:
// 32 x 32 box whose rows are 64 bytes (16-bit E, 64-byte swizzle) or 32 bytes (int8 E, 32-byte swizzle).
// Only encoded when E allows 16-byte accesses (base and pitch multiples of 16 bytes).
int encode_e_map(CUtensorMap* tm, int dtype, const void* ptr, int64_t m, int64_t n, int64_t lde, int64_t batch = 0,
                 int64_t batch_stride = 0)
{
    load_entry_points();
    if(!g_encode_tiled)
        return fail(CKB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    const int eb          = elem_bytes(dtype);
    cuuint64_t dims[3]    = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(m), static_cast<cuuint64_t>(batch)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(lde) * eb, static_cast<cuuint64_t>(batch_stride) * eb};
    cuuint32_t box[3]     = {32, 32, 1};
    cuuint32_t estr[3]    = {1, 1, 1};
    CUresult r = g_encode_tiled(tm, tm_dtype(dtype), batch >= 1 ? 3 : 2, const_cast<void*>(ptr), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE,
                                eb == 1 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B,
                                CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if(r != CUDA_SUCCESS)
        return fail(CKB_ERR_CUDA, "cuTensorMapEncodeTiled (E) failed (CUresult %d) m=%lld n=%lld lde=%lld",
                    static_cast<int>(r), (long long)m, (long long)n, (long long)lde);
    return CKB_OK;
}

// A is M x K: row-major = K-major, column-major = M-major.  B is K x N: column-major = K-major,
// row-major = N-major.
bool a_is_mn_major(const ckb_gemm_desc* d) { return d->a_layout == CKB_COL_MAJOR; }
bool b_is_mn_major(const ckb_gemm_desc* d) { return d->b_layout == CKB_ROW_MAJOR; }

// Tensor map of one operand of a GEMM problem, seen as [mn][k]; box_mn = rows of a K-major box.
int encode_operand(CUtensorMap* tm, int dtype, const void* ptr, int64_t mn, int64_t k, int64_t ld, bool mn_major,
                   int box_mn, int64_t batch = 0, int64_t batch_stride = 0)
{
    return mn_major ? encode_mnmajor_2d(tm, dtype, ptr, mn, k, ld, batch, batch_stride)
                    : encode_kmajor_2d(tm, dtype, ptr, mn, k, ld, box_mn, batch, batch_stride);
}

// Narrowest B slice one CTA loads: 32 rows of a K-major tile (a CTA pair can then cut a 256-wide tail tile into
// four 64-column slices: +1.7 % on the int8 3840 x 4096 x 4096 GEMM against two 128-column slices, which leave
// half of the pairs idle during the tail), one whole swizzle atom (128 bytes of N positions) of an N-major one.
// CKB_MIN_B_ROWS=64 restores the wider minimum for A/B runs.
int min_b_rows(int dtype, bool b_mn)
{
    if(b_mn)
        return BK_BYTES / elem_bytes(dtype);
    const char* s = getenv("CKB_MIN_B_ROWS");
    return (s && atoi(s) == 64) ? 64 : 32;
}

int pick_bn(int64_t M, int64_t N, int sm_count, int min_bn = 64)
{
    const int f = forced_bn();
    if((f == 256 || f == 128 || f == 64) && f >= min_bn)
        return f;
    if(N <= 64 && min_bn <= 64)
        return 64;
    if(N <= 128)
        return 128;
    // Prefer the 256-wide tile (lowest shared-memory traffic per flop) unless it leaves most of
    // the machine idle.
    const int64_t tiles256 = ((M + BM - 1) / BM) * ((N + 255) / 256);
    if(tiles256 < sm_count / 2)
        return 128;
    return 256;
}

// Splits the last, partial wave of tiles into column slices so that it occupies every SM
// (see "Work items" in ckb_kernel.cuh).  Slices are at least 64 columns wide.
struct WorkPlan
{
    int32_t split_start, split, total_work, grid;
};

// `units` = CTAs (one CTA per tile) or CTA pairs (cg = 2) that run concurrently.
WorkPlan plan_work(int64_t total_tiles, int units, int bn, int cg, int min_rows = 64)
{
    WorkPlan w;
    const int64_t G    = units;
    const int64_t full = (total_tiles / G) * G;
    const int64_t rem  = total_tiles - full;
    int split          = 1;
    const char* env    = getenv("CKB_NO_TAIL_SPLIT");
    if(rem > 0 && !(env && atoi(env) != 0))
    {
        // slices of >= 64 columns whose per-CTA share is >= min_rows: K-major 256 -> 4, 128 -> 2, 64 -> 1
        const int min_width = min_rows * cg > 64 ? min_rows * cg : 64;
        const int max_split = bn / min_width;
        while(split * 2 <= max_split && rem * split * 2 <= G)
            split *= 2;
    }
    w.split       = split;
    w.split_start = static_cast<int32_t>(split > 1 ? full : total_tiles);
    w.total_work  = static_cast<int32_t>(split > 1 ? full + rem * split : total_tiles);
    w.grid        = static_cast<int32_t>((w.total_work < G ? w.total_work : G) * cg);
    return w;
}

// CTAs per tile: pairs (256 x 256 tiles, tcgen05 cta_group::2) once the problem fills the machine
// with 128 x 256 tiles at least once; single CTAs for small problems.
int pick_cg(int64_t tiles_128, int bn, int sm_count)
{
    const char* s = getenv("CKB_FORCE_CG");
    if(s && (atoi(s) == 1 || atoi(s) == 2))
        return bn == 256 ? atoi(s) : 1;
    return (bn == 256 && tiles_128 >= sm_count) ? 2 : 1;
}

int kind_of(int dtype) { return dtype == CKB_I8 ? KIND_I8 : dtype == CKB_BF16 ? KIND_BF16 : KIND_F16; }

bool epilogue_valid_for(int epi, int ab_dtype)
{
    if(epi < 0 || epi >= CKB_EPI_COUNT_)
        return false;
    if(ab_dtype == CKB_BF16) // float functors with one rounding; see gen_instances.py for the instantiated sets
        return epi == CKB_EPI_PASSTHROUGH || epi == CKB_EPI_RELU || epi == CKB_EPI_SCALE || epi == CKB_EPI_FASTGELU ||
               epi == CKB_EPI_ADD_RELU || epi == CKB_EPI_ADD_HARDSWISH || epi == CKB_EPI_ADD_RELU_ADD;
    if(ab_dtype == CKB_I8)
        return epi == CKB_EPI_PASSTHROUGH || epi == CKB_EPI_RELU ||
               epi == CKB_EPI_REQUANT_RELU_REQUANT || epi == CKB_EPI_REQUANT_RELU_REQUANT_RNE;
    return epi != CKB_EPI_REQUANT_RELU_REQUANT && epi != CKB_EPI_REQUANT_RELU_REQUANT_RNE;
}

// Shared validation of one GEMM problem.  `why` receives the reason on failure.
int check_gemm(const ckb_gemm_desc* d, bool need_pointers)
{
    if(!d)
        return fail(CKB_ERR_INVALID, "null descriptor");
    if(d->ab_dtype != CKB_F16 && d->ab_dtype != CKB_I8 && d->ab_dtype != CKB_BF16)
        return fail(CKB_ERR_UNSUPPORTED, "A/B dtype %d not supported (f16, bf16 and int8 are)", d->ab_dtype);
    if(d->e_dtype != d->ab_dtype)
        return fail(CKB_ERR_UNSUPPORTED, "E dtype must equal the A/B dtype (f16->f16, bf16->bf16, int8->int8)");
    if((d->a_layout != CKB_ROW_MAJOR && d->a_layout != CKB_COL_MAJOR) ||
       (d->b_layout != CKB_ROW_MAJOR && d->b_layout != CKB_COL_MAJOR))
        return fail(CKB_ERR_INVALID, "unknown A or B layout");
    if(d->e_layout != CKB_ROW_MAJOR)
        return fail(CKB_ERR_UNSUPPORTED, "E (and every D) must be row-major");
    if(!epilogue_valid_for(d->epilogue, d->ab_dtype))
        return fail(CKB_ERR_UNSUPPORTED, "epilogue %d not available for dtype %d", d->epilogue, d->ab_dtype);
    if(d->n_ds != epi_num_d(d->epilogue))
        return fail(CKB_ERR_INVALID, "epilogue %d reads %d D tensors, descriptor gives %d", d->epilogue,
                    epi_num_d(d->epilogue), d->n_ds);
    if(d->M < 1 || d->N < 1 || d->K < 1)
        return fail(CKB_ERR_UNSUPPORTED, "M, N, K must be positive");
    if(d->M > 0x7FFFFF00ll || d->N > 0x7FFFFF00ll || d->K > 0x7FFFFF00ll)
        return fail(CKB_ERR_UNSUPPORTED, "M, N, K must fit in int32");
    const int eb = elem_bytes(d->ab_dtype);
    if(d->lda < (a_is_mn_major(d) ? d->M : d->K) || d->ldb < (b_is_mn_major(d) ? d->N : d->K) || d->lde < d->N)
        return fail(CKB_ERR_INVALID, "leading dimension smaller than the row length");
    if((d->lda * eb) % 16 != 0 || (d->ldb * eb) % 16 != 0)
        return fail(CKB_ERR_UNSUPPORTED, "lda and ldb must be multiples of 16 bytes (TMA row pitch)");
    for(int i = 0; i < d->n_ds; ++i)
        if(d->ldd[i] != 0 && d->ldd[i] < d->N)
            return fail(CKB_ERR_INVALID, "ldd[%d] smaller than N", i);
    if(need_pointers)
    {
        if(!d->p_a || !d->p_b || !d->p_e)
            return fail(CKB_ERR_INVALID, "null tensor pointer");
        if(!aligned16(d->p_a) || !aligned16(d->p_b))
            return fail(CKB_ERR_UNSUPPORTED, "A and B must be 16-byte aligned");
        for(int i = 0; i < d->n_ds; ++i)
            if(!d->p_ds[i])
                return fail(CKB_ERR_INVALID, "null D%d pointer", i);
    }
    return CKB_OK;
}

bool gemm_vec_ok(const ckb_gemm_desc* d)
{
    const int per16 = 16 / elem_bytes(d->ab_dtype);
    bool ok         = aligned16(d->p_e) && d->lde % per16 == 0;
    for(int i = 0; i < d->n_ds; ++i)
        ok = ok && aligned16(d->p_ds[i]) && d->ldd[i] % per16 == 0;
    return ok;
}

void fill_epilogue(EpilogueArgs& ea, const ckb_gemm_desc* d)
{
    ea.kind   = d->epilogue;
    ea.out_i8 = d->ab_dtype == CKB_I8;
    ea.bf16   = d->ab_dtype == CKB_BF16;
    ea.pad_   = 0;
    memcpy(ea.p, d->epi_params, sizeof(ea.p));
    ea.e    = d->p_e;
    ea.d0   = d->n_ds > 0 ? d->p_ds[0] : nullptr;
    ea.d1   = d->n_ds > 1 ? d->p_ds[1] : nullptr;
    ea.lde  = d->lde;
    ea.ldd0 = d->n_ds > 0 ? d->ldd[0] : 0;
    ea.ldd1 = d->n_ds > 1 ? d->ldd[1] : 0;
}

// One launch, or the reference timing protocol (kernel_launch.hpp:12-74): a warm-up launch, then
// n_rep launches between two events.
#ifdef CKB_TRACE
__device__ unsigned long long g_trace[1024 * 16];
#endif

// Profiling builds (-DCKB_TRACE) hand every launch the role cycle counter array; regular builds pass null.
unsigned long long* trace_buffer()
{
#ifdef CKB_TRACE
    void* sym = nullptr;
    return cudaGetSymbolAddress(&sym, g_trace) == cudaSuccess ? static_cast<unsigned long long*>(sym) : nullptr;
#else
    return nullptr;
#endif
}

// CKB_STORE_DIRECT=1 makes every kernel write E with 128-bit global stores instead of the staged TMA stores.
int store_direct_forced()
{
    const char* s = getenv("CKB_STORE_DIRECT");
    return s ? atoi(s) : -1;
}

int run_timed(LaunchFn fn, int bn, int cg, const KernelParams& p_in, int grid, cudaStream_t stream, int n_rep,
              float* avg_ms)
{
    KernelParams p = p_in;
    p.trace        = trace_buffer();
    if(store_direct_forced() >= 0)
        p.store_direct = store_direct_forced();
    if(avg_ms)
        *avg_ms = 0.f;
    if(n_rep <= 0)
    {
        CKB_CUDA(fn(bn, cg, p, grid, stream));
        g_launches.fetch_add(1);
        return CKB_OK;
    }
    CKB_CUDA(fn(bn, cg, p, grid, stream)); // warm-up
    g_launches.fetch_add(1);
    cudaEvent_t start, stop;
    CKB_CUDA(cudaEventCreate(&start));
    CKB_CUDA(cudaEventCreate(&stop));
    CKB_CUDA(cudaDeviceSynchronize());
    CKB_CUDA(cudaEventRecord(start, stream));
    for(int i = 0; i < n_rep; ++i)
    {
        cudaError_t e = fn(bn, cg, p, grid, stream);
        if(e != cudaSuccess)
        {
            cudaEventDestroy(start);
            cudaEventDestroy(stop);
            return fail(CKB_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
        }
    }
    g_launches.fetch_add(n_rep);
    CKB_CUDA(cudaEventRecord(stop, stream));
    CKB_CUDA(cudaEventSynchronize(stop));
    float total = 0.f;
    CKB_CUDA(cudaEventElapsedTime(&total, start, stop));
    cudaEventDestroy(start);
    cudaEventDestroy(stop);
    if(avg_ms)
        *avg_ms = total / n_rep;
    return CKB_OK;
}

} // namespace

namespace ckb {
#define CKB_INST(M, K, E) extern template cudaError_t launch_epi<M, K, E>(int, int, const KernelParams&, int, cudaStream_t);
#include "ckb_instances.def"
#undef CKB_INST

LaunchFn find_launch(int mode, int kind, int epi)
{
#define CKB_INST(M, K, E)                   \
    if(mode == M && kind == K && epi == E)  \
        return &launch_epi<M, K, E>;
#include "ckb_instances.def"
#undef CKB_INST
    return nullptr;
}
} // namespace ckb

namespace ckb {
// Group tables of grouped-GEMM launches that were captured into graphs (see ckb_grouped_gemm_run).
std::mutex g_captured_mutex;
std::map<void*, std::unique_ptr<std::vector<GroupEntry>>> g_captured_tables;
std::vector<std::unique_ptr<std::vector<GroupEntry>>> g_retired_tables;
} // namespace ckb

extern "C" {

int ckb_abi_version(void) { return CKB_ABI_VERSION; }

#ifdef CKB_TRACE
// Profiling builds only: copies the role cycle counters of the last launch (16 words per CTA) to the host.
int ckb_trace_read(unsigned long long* host, int words)
{
    CKB_CUDA(cudaDeviceSynchronize());
    CKB_CUDA(cudaMemcpyFromSymbol(host, g_trace, sizeof(unsigned long long) * words));
    return CKB_OK;
}
#endif

const char* ckb_last_error(void) { return t_last_error.c_str(); }

uint64_t ckb_launch_count(void) { return g_launches.load(); }

int ckb_device_info(char* name, size_t name_bytes, int* sm_count, int* cc_major, int* cc_minor)
{
    int dev = 0;
    CKB_CUDA(cudaGetDevice(&dev));
    cudaDeviceProp prop;
    CKB_CUDA(cudaGetDeviceProperties(&prop, dev));
    if(name && name_bytes)
    {
        strncpy(name, prop.name, name_bytes - 1);
        name[name_bytes - 1] = 0;
    }
    if(sm_count)
        *sm_count = prop.multiProcessorCount;
    if(cc_major)
        *cc_major = prop.major;
    if(cc_minor)
        *cc_minor = prop.minor;
    return CKB_OK;
}

int ckb_device_status(uint32_t* word)
{
    DeviceInfo* dev = nullptr;
    int rc          = current_device(&dev);
    if(rc)
        return rc;
    CKB_CUDA(cudaDeviceSynchronize());
    uint32_t w = 0;
    CKB_CUDA(cudaMemcpy(&w, dev->status, sizeof(w), cudaMemcpyDeviceToHost));
    if(w != 0)
    {
        CKB_CUDA(cudaMemset(dev->status, 0, sizeof(w)));
        // a kernel that gave up may have left tail-tile counters of the K-split scratch half way
        std::lock_guard<std::mutex> lock(g_dev_mutex);
        for(auto& kv : dev->scratch)
            if(kv.second.ptr)
                cudaMemset(kv.second.ptr, 0, kScratchCounterBytes);
    }
    if(word)
        *word = w;
    if(w != 0)
        return fail(CKB_ERR_DEVICE, "kernel wait timed out: code %u in block %u", w >> 24, w & 0xFFFFFFu);
    return CKB_OK;
}

// ---- memory helpers -----------------------------------------------------------------------------
int ckb_malloc(void** dev_ptr, size_t bytes)
{
    if(!dev_ptr)
        return fail(CKB_ERR_INVALID, "null output pointer");
    CKB_CUDA(cudaMalloc(dev_ptr, bytes));
    return CKB_OK;
}
int ckb_free(void* dev_ptr)
{
    CKB_CUDA(cudaFree(dev_ptr));
    return CKB_OK;
}
int ckb_memcpy_h2d(void* dev_dst, const void* host_src, size_t bytes)
{
    CKB_CUDA(cudaMemcpy(dev_dst, host_src, bytes, cudaMemcpyHostToDevice));
    return CKB_OK;
}
int ckb_memcpy_d2h(void* host_dst, const void* dev_src, size_t bytes)
{
    CKB_CUDA(cudaMemcpy(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost));
    return CKB_OK;
}
int ckb_memset(void* dev_ptr, int value, size_t bytes)
{
    CKB_CUDA(cudaMemset(dev_ptr, value, bytes));
    return CKB_OK;
}
int ckb_device_synchronize(void)
{
    CKB_CUDA(cudaDeviceSynchronize());
    return CKB_OK;
}
int ckb_release_scratch(void* stream, int all_streams)
{
    DeviceInfo* dev = nullptr;
    int rc          = current_device(&dev);
    if(rc)
        return rc;
    CKB_CUDA(cudaDeviceSynchronize());
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    for(auto it = dev->scratch.begin(); it != dev->scratch.end();)
    {
        if(all_streams || it->first == static_cast<cudaStream_t>(stream))
        {
            if(it->second.ptr)
                cudaFree(it->second.ptr);
            it = dev->scratch.erase(it);
        }
        else
            ++it;
    }
    if(all_streams)
    {
        std::lock_guard<std::mutex> tables(g_captured_mutex);
        g_captured_tables.clear();
        g_retired_tables.clear();
    }
    return CKB_OK;
}

// ---- GEMM ---------------------------------------------------------------------------------------
int ckb_gemm_supported(const ckb_gemm_desc* desc) { return check_gemm(desc, false); }

// Strides between the matrices of a batch (elements); batch = 0 for a plain GEMM.
struct BatchInfo
{
    int64_t batch, stride_a, stride_b, stride_e, stride_d[2];
    bool vec_ok; // every batch of E / D keeps the 16-byte alignment of the first
};

// Whole-problem K split.  A GEMM with few output tiles and a long K leaves most SMs idle whatever the tile shape;
// cutting every tile's K loop into 2 or 4 slices (the machinery of the K-split tail, with no whole tiles before
// it) puts 2-8 times as many SMs to work on full-width MMAs.  Cycle estimates per k block, fitted to timings of
// 1024 x 1024 x K and 512 x 512 x K with and without the split: 590 for 256 accumulator columns, 340 for 128,
// 315 for 64 (the narrow ones are bound by the issue rate of the single MMA thread, not by the tensor pipe);
// parking and summing the slices costs about 9100 cycles (5.5 us), most of it the exposed latency of the
// reduction's loads.
struct WholeSplit
{
    int bn = 0, cg = 0, ksplit = 0;
};

int kb_cycles(int width) { return width >= 256 ? 590 : width >= 128 ? 340 : 315; }

WholeSplit consider_whole_split(int64_t M, int64_t N, int num_kb, int sm_count, int b_min, int64_t est_current)
{
    WholeSplit best;
    int64_t best_est = est_current - est_current / 8; // has to beat the plan without it by an eighth
    const int cand[3][2] = {{256, 2}, {256, 1}, {128, 1}};
    for(const auto& c : cand)
    {
        const int bn = c[0], cg = c[1];
        if(bn / cg < b_min || (cg == 2 && M <= BM)) // a pair tile with one half of its rows empty pays for nothing
            continue;
        const int64_t G     = sm_count / cg;
        const int64_t tiles = ((M + BM * cg - 1) / (BM * cg)) * ((N + bn - 1) / bn);
        for(int ks = bn / 32; ks >= 2; ks /= 2) // column parts of the reduction are whole 32-column chunks
        {
            if(tiles * ks > G)
                continue;
            int ks_kb = (num_kb + ks - 1) / ks;
            ks_kb     = (ks_kb + 1) & ~1;
            if(ks_kb < 4 || static_cast<int64_t>(ks - 1) * ks_kb >= num_kb)
                continue;
            const int64_t est = static_cast<int64_t>(ks_kb) * kb_cycles(bn) + 9100 + (ks > 4 ? 1500 : 0);
            if(est < best_est)
            {
                best_est    = est;
                best.bn     = bn;
                best.cg     = cg;
                best.ksplit = ks;
            }
        }
    }
    return best;
}

static int gemm_run_impl(const ckb_gemm_desc* d, const BatchInfo& bi, void* stream, int n_rep, float* avg_ms)
{
    int rc = CKB_OK;
    DeviceInfo* dev = nullptr;
    rc              = current_device(&dev);
    if(rc)
        return rc;
    const bool a_mn  = a_is_mn_major(d), b_mn = b_is_mn_major(d);
    const int b_min  = min_b_rows(d->ab_dtype, b_mn);
    int bn           = pick_bn(d->M, d->N, dev->sm_count, b_min);
    const int eb     = elem_bytes(d->ab_dtype);
    KernelParams p;
    memset(&p, 0, sizeof(p));
    rc = encode_operand(&p.tm_a, d->ab_dtype, d->p_a, d->M, d->K, d->lda, a_mn, BM, bi.batch, bi.stride_a);
    if(rc)
        return rc;
    fill_epilogue(p.epi, d);
    const int64_t nb      = bi.batch > 0 ? bi.batch : 1;
    int cg                = pick_cg(((d->M + BM - 1) / BM) * ((d->N + bn - 1) / bn) * nb, bn, dev->sm_count);
    const int bk          = BK_BYTES / eb;
    const int num_kb      = static_cast<int>((d->K + bk - 1) / bk);
    const char* no_ks     = getenv("CKB_NO_SPLITK");
    const bool ks_allowed = !(no_ks && atoi(no_ks) != 0);
    // Measured on 3840 x 4096 x 4096: +5 % for 16-bit operands with a D-less epilogue; a loss for int8 (tiles
    // half as long) and for epilogues that read D tensors (bound by power: parking the partials through L2 costs
    // more energy than the narrow MMAs it removes) - those keep the column slices.
#ifdef CKB_KSPLIT_WITH_D
    const bool ks_pays = d->ab_dtype != CKB_I8;
#else
    const bool ks_pays = d->ab_dtype != CKB_I8 && d->n_ds == 0;
#endif
    int whole_ksplit = 0;
    if(ks_pays && ks_allowed && bi.batch == 0 && forced_bn() == 0 && !getenv("CKB_FORCE_CG") &&
       !stream_is_capturing(static_cast<cudaStream_t>(stream)))
    {
        // only where the plan without it runs a single, partly filled wave
        const int64_t t0 = ((d->M + BM * cg - 1) / (BM * cg)) * ((d->N + bn - 1) / bn);
        const int64_t G0 = dev->sm_count / cg;
        if(t0 * 2 <= G0)
        {
            const WorkPlan w0 = plan_work(t0, static_cast<int>(G0), bn, cg, b_min);
            const WholeSplit ws =
                consider_whole_split(d->M, d->N, num_kb, dev->sm_count, b_min,
                                     static_cast<int64_t>(num_kb) * kb_cycles(bn / w0.split));
            if(ws.ksplit >= 2)
            {
                bn           = ws.bn;
                cg           = ws.cg;
                whole_ksplit = ws.ksplit;
            }
        }
    }
    const int64_t tiles_n = (d->N + bn - 1) / bn;
    const int64_t tiles_m = (d->M + BM * cg - 1) / (BM * cg);
    const int64_t all_tiles = tiles_m * tiles_n * nb;
    if(all_tiles > 0x3FFFFFFFll)
        return fail(CKB_ERR_UNSUPPORTED, "too many tiles");
    WorkPlan plan = plan_work(all_tiles, dev->sm_count / cg, bn, cg, b_min);
    // K-split tail: with whole waves before it and a tail of at most half the units, cut the tail tiles along K
    // (see "K-split tail" in ckb_kernel.cuh); needs scratch, else the column-slice plan above stands.
    const int64_t G   = dev->sm_count / cg;
    const int64_t ful = (all_tiles / G) * G, rem = all_tiles - ful;
    if(ks_pays && ks_allowed && rem > 0 && (ful > 0 || whole_ksplit >= 2) && rem * 2 <= G && rem <= 1024)
    {
        // tail: 4 or 2 slices, reduction in column parts of bn / ksplit >= 64 columns; whole problem: up to 8
        // A 256-wide tail tile is cut four ways along K where a quarter of the units suffice; with more tail tiles only
        // two K halves fit, and those beat two 128-column slices only for a long K (parking and reduction cost the
        // same whatever K is, a column slice costs per k block): measured break-even near 78 k blocks
        // (4096^3: 78.8 us with the K halves, 77.5 us with column slices; 4096 x 4096 x 8192: 160.2 against 165.0 us).
        // The four-way cut itself needs a K loop long enough to pay for parking and reduction: 3840 x 4096 x K
        // with K = 1024 / 2048 / 3072 / 4096 / 6144 took 29.9 / 43.7 / 57.4 / 73.6 / 110.6 us with it and
        // 25.3 / 42.3 / 58.9 / 76.4 / 115.8 us with four column slices: taken from 40 k blocks on (48 for the
        // two halves of a 128-wide tile, by the same cost model).
        int ksplit = whole_ksplit >= 2 ? whole_ksplit
                     : (G / rem >= 4 && bn >= 256) ? (num_kb >= 40 ? 4 : 0)
                     : ((bn == 128 && num_kb >= 48) || (bn >= 256 && num_kb >= 80)) ? 2 : 0;
        int ks_kb  = 0;
        for(; ksplit >= 2; ksplit /= 2)
        {
            ks_kb = (num_kb + ksplit - 1) / ksplit;
            ks_kb = (ks_kb + 1) & ~1; // slices start on a stage boundary (at most two k blocks per stage)
            if(ks_kb >= 4 && static_cast<int64_t>(ksplit - 1) * ks_kb < num_kb)
                break;
        }
        if(ksplit >= 2)
        {
            const size_t part_bytes = static_cast<size_t>(rem) * ksplit * (BM * cg) * bn * sizeof(uint32_t);
            void* sc                = scratch_for(dev, static_cast<cudaStream_t>(stream), part_bytes);
            if(sc)
            {
                p.ksplit      = ksplit;
                p.ks_kb       = ks_kb;
                p.ks_full     = static_cast<int32_t>(ful);
                p.ks_rem      = static_cast<int32_t>(rem);
                p.ks_counters = static_cast<uint32_t*>(sc);
                p.ks_partials = reinterpret_cast<uint32_t*>(static_cast<char*>(sc) + kScratchCounterBytes);
                p.num_slots   = static_cast<int32_t>(ful / G + 2 < 4 ? 4 : ful / G + 2);
                plan.split    = 1;
                plan.split_start = static_cast<int32_t>(all_tiles);
                plan.total_work  = static_cast<int32_t>(all_tiles);
                plan.grid        = static_cast<int32_t>(G * cg);
            }
        }
    }
    if(p.ksplit < 2)
        p.num_slots = static_cast<int32_t>((plan.total_work + G - 1) / G);
    rc = encode_operand(&p.tm_b, d->ab_dtype, d->p_b, d->N, d->K, d->ldb, b_mn, bn / cg, bi.batch, bi.stride_b);
    if(rc)
        return rc;
    rc = encode_operand(&p.tm_b_split, d->ab_dtype, d->p_b, d->N, d->K, d->ldb, b_mn, bn / plan.split / cg, bi.batch,
                        bi.stride_b);
    if(rc)
        return rc;
    p.batch_tiles     = bi.batch > 0 ? static_cast<int32_t>(tiles_m * tiles_n) : 0;
    p.batch_stride_e  = bi.stride_e;
    p.batch_stride_d0 = bi.stride_d[0];
    p.batch_stride_d1 = bi.stride_d[1];
    p.mn_major      = (a_mn ? 1 : 0) | (b_mn ? 2 : 0);
    p.split_start   = plan.split_start;
    p.split         = plan.split;
    p.total_work    = plan.total_work;
    p.total_tiles   = static_cast<int32_t>(all_tiles);
    p.M             = static_cast<int32_t>(d->M);
    p.N             = static_cast<int32_t>(d->N);
    p.tiles_n       = static_cast<int32_t>(tiles_n);
    p.num_kb        = num_kb;
    p.vec_ok        = gemm_vec_ok(d) && bi.vec_ok ? 1 : 0;
    if(p.vec_ok)
    {
        rc = encode_e_map(&p.tm_e, d->e_dtype, d->p_e, d->M, d->N, d->lde, bi.batch, bi.stride_e);
        if(rc)
            return rc;
    }
    p.wait_limit_ns = wait_limit_ns();
    p.status        = dev->status;
    LaunchFn fn     = find_launch(MODE_GEMM, kind_of(d->ab_dtype), d->epilogue);
    if(!fn)
        return fail(CKB_ERR_UNSUPPORTED, "no kernel instance for epilogue %d", d->epilogue);
    return run_timed(fn, bn, cg, p, plan.grid, static_cast<cudaStream_t>(stream), n_rep, avg_ms);
}

int ckb_gemm_run(const ckb_gemm_desc* d, void* stream, int n_rep, float* avg_ms)
{
    int rc = check_gemm(d, true);
    if(rc)
        return rc;
    BatchInfo bi{0, 0, 0, 0, {0, 0}, true}; // batch 0: 2-D operand maps
    return gemm_run_impl(d, bi, stream, n_rep, avg_ms);
}

// ---- batched GEMM -------------------------------------------------------------------------------
static int check_batched(const ckb_batched_gemm_desc* b, bool need_pointers)
{
    if(!b)
        return fail(CKB_ERR_INVALID, "null descriptor");
    int rc = check_gemm(&b->gemm, need_pointers);
    if(rc)
        return rc;
    if(b->batch < 1 || b->batch > 0x7FFFFFFFll)
        return fail(CKB_ERR_UNSUPPORTED, "batch count must be in [1, 2^31)");
    const int eb = elem_bytes(b->gemm.ab_dtype);
    if(b->batch > 1)
    {
        if(b->batch_stride_a < 1 || b->batch_stride_b < 1 || b->batch_stride_e < 0)
            return fail(CKB_ERR_INVALID, "batch strides of A and B must be positive");
        if((b->batch_stride_a * eb) % 16 != 0 || (b->batch_stride_b * eb) % 16 != 0)
            return fail(CKB_ERR_UNSUPPORTED, "batch strides of A and B must be multiples of 16 bytes (TMA pitch)");
    }
    return CKB_OK;
}

int ckb_batched_gemm_supported(const ckb_batched_gemm_desc* desc) { return check_batched(desc, false); }

int ckb_batched_gemm_run(const ckb_batched_gemm_desc* b, void* stream, int n_rep, float* avg_ms)
{
    int rc = check_batched(b, true);
    if(rc)
        return rc;
    const ckb_gemm_desc* d = &b->gemm;
    if(b->batch == 1)
        return ckb_gemm_run(d, stream, n_rep, avg_ms);
    BatchInfo bi{b->batch, b->batch_stride_a, b->batch_stride_b, b->batch_stride_e,
                 {b->batch_stride_d[0], b->batch_stride_d[1]}, true};
    // the 128-bit epilogue path needs every batch of E / D to keep the 16-byte alignment of the first
    const int per16 = 16 / elem_bytes(d->ab_dtype);
    bool strides_vec_ok = bi.stride_e % per16 == 0;
    for(int i = 0; i < d->n_ds; ++i)
        strides_vec_ok = strides_vec_ok && bi.stride_d[i] % per16 == 0;
    bi.vec_ok = strides_vec_ok;
    return gemm_run_impl(d, bi, stream, n_rep, avg_ms);
}

// ---- grouped GEMM -------------------------------------------------------------------------------
static int check_grouped(const ckb_grouped_gemm_desc* g, bool need_pointers)
{
    if(!g || g->group_count < 1 || !g->groups)
        return fail(CKB_ERR_INVALID, "grouped descriptor needs at least one group");
    const ckb_gemm_desc& g0 = g->groups[0];
    for(int i = 0; i < g->group_count; ++i)
    {
        const ckb_gemm_desc& gi = g->groups[i];
        int rc                  = check_gemm(&gi, need_pointers);
        if(rc)
        {
            std::string msg = "group " + std::to_string(i) + ": " + t_last_error;
            t_last_error    = msg;
            return rc;
        }
        if(gi.ab_dtype != g0.ab_dtype || gi.epilogue != g0.epilogue || gi.n_ds != g0.n_ds ||
           gi.a_layout != g0.a_layout || gi.b_layout != g0.b_layout ||
           memcmp(gi.epi_params, g0.epi_params, sizeof(g0.epi_params)) != 0)
            return fail(CKB_ERR_UNSUPPORTED, "group %d: dtype / layout / epilogue differ from group 0", i);
    }
    return CKB_OK;
}

int ckb_grouped_gemm_supported(const ckb_grouped_gemm_desc* desc) { return check_grouped(desc, false); }

int ckb_grouped_gemm_workspace_size(const ckb_grouped_gemm_desc* desc, size_t* bytes)
{
    if(!desc || !bytes || desc->group_count < 1)
        return fail(CKB_ERR_INVALID, "bad arguments");
    *bytes = static_cast<size_t>(desc->group_count) * sizeof(GroupEntry) + 128; // + alignment slack
    return CKB_OK;
}

// Tile shape, CTA grouping and work plan of a grouped problem, and its device table entries.
struct GroupedPlan
{
    int bn, cg, mn_major;
    WorkPlan plan;
    int64_t total_tiles;
};

static int plan_grouped(const ckb_grouped_gemm_desc* g, const DeviceInfo* dev, GroupedPlan* gp)
{
    const int dtype = g->groups[0].ab_dtype;
    const bool a_mn = a_is_mn_major(&g->groups[0]), b_mn = b_is_mn_major(&g->groups[0]);
    const int b_min = min_b_rows(dtype, b_mn);
    int64_t max_n = 0, sum_m = 0;
    for(int i = 0; i < g->group_count; ++i)
    {
        max_n = max_n > g->groups[i].N ? max_n : g->groups[i].N;
        sum_m += g->groups[i].M;
    }
    const int bn      = pick_bn(sum_m, max_n, dev->sm_count, b_min);
    int64_t tiles_128 = 0;
    for(int i = 0; i < g->group_count; ++i)
        tiles_128 += ((g->groups[i].M + BM - 1) / BM) * ((g->groups[i].N + bn - 1) / bn);
    const int cg      = pick_cg(tiles_128, bn, dev->sm_count);
    int64_t all_tiles = 0;
    for(int i = 0; i < g->group_count; ++i)
        all_tiles += ((g->groups[i].M + BM * cg - 1) / (BM * cg)) * ((g->groups[i].N + bn - 1) / bn);
    if(all_tiles > 0x3FFFFFFFll)
        return fail(CKB_ERR_UNSUPPORTED, "too many tiles");
    gp->bn          = bn;
    gp->cg          = cg;
    gp->mn_major    = (a_mn ? 1 : 0) | (b_mn ? 2 : 0);
    gp->plan        = plan_work(all_tiles, dev->sm_count / cg, bn, cg, b_min);
    gp->total_tiles = all_tiles;
    return CKB_OK;
}

static int fill_group_table(const ckb_grouped_gemm_desc* g, const GroupedPlan& gp, GroupEntry* table)
{
    const int dtype = g->groups[0].ab_dtype;
    const int bk    = BK_BYTES / elem_bytes(dtype);
    const bool a_mn = (gp.mn_major & 1) != 0, b_mn = (gp.mn_major & 2) != 0;
    const int bn = gp.bn, cg = gp.cg;
    int64_t tile_start = 0;
    for(int i = 0; i < g->group_count; ++i)
    {
        const ckb_gemm_desc& d = g->groups[i];
        GroupEntry& ge         = table[i];
        memset(&ge, 0, sizeof(ge));
        int rc = encode_operand(&ge.tm_a, dtype, d.p_a, d.M, d.K, d.lda, a_mn, BM);
        if(rc)
            return rc;
        rc = encode_operand(&ge.tm_b, dtype, d.p_b, d.N, d.K, d.ldb, b_mn, bn / cg);
        if(rc)
            return rc;
        rc = encode_operand(&ge.tm_b_split, dtype, d.p_b, d.N, d.K, d.ldb, b_mn, bn / gp.plan.split / cg);
        if(rc)
            return rc;
        const int64_t tm = (d.M + BM * cg - 1) / (BM * cg), tn = (d.N + bn - 1) / bn;
        ge.M          = static_cast<int32_t>(d.M);
        ge.N          = static_cast<int32_t>(d.N);
        ge.K          = static_cast<int32_t>(d.K);
        ge.tiles_n    = static_cast<int32_t>(tn);
        ge.tile_start = static_cast<int32_t>(tile_start);
        ge.num_kb     = static_cast<int32_t>((d.K + bk - 1) / bk);
        ge.vec_ok     = gemm_vec_ok(&d) ? 1 : 0;
        if(ge.vec_ok)
        {
            rc = encode_e_map(&ge.tm_e, dtype, d.p_e, d.M, d.N, d.lde);
            if(rc)
                return rc;
        }
        ge.e          = d.p_e;
        ge.d0         = d.n_ds > 0 ? d.p_ds[0] : nullptr;
        ge.d1         = d.n_ds > 1 ? d.p_ds[1] : nullptr;
        ge.lde        = d.lde;
        ge.ldd0       = d.n_ds > 0 ? d.ldd[0] : 0;
        ge.ldd1       = d.n_ds > 1 ? d.ldd[1] : 0;
        tile_start += tm * tn;
    }
    return CKB_OK;
}

static void fill_grouped_params(KernelParams& p, const ckb_grouped_gemm_desc* g, const GroupedPlan& gp,
                                const GroupEntry* d_table, const DeviceInfo* dev)
{
    memset(&p, 0, sizeof(p));
    fill_epilogue(p.epi, &g->groups[0]);
    p.groups        = d_table;
    p.group_count   = g->group_count;
    p.total_tiles   = static_cast<int32_t>(gp.total_tiles);
    p.split_start   = gp.plan.split_start;
    p.split         = gp.plan.split;
    p.total_work    = gp.plan.total_work;
    p.num_slots     = (gp.plan.total_work + gp.plan.grid / gp.cg - 1) / (gp.plan.grid / gp.cg);
    p.mn_major      = gp.mn_major;
    p.wait_limit_ns = wait_limit_ns();
    p.status        = dev->status;
}

int ckb_grouped_gemm_run(const ckb_grouped_gemm_desc* g, void* workspace, size_t workspace_bytes,
                         void* stream_, int n_rep, float* avg_ms)
{
    int rc = check_grouped(g, true);
    if(rc)
        return rc;
    size_t need = 0;
    ckb_grouped_gemm_workspace_size(g, &need);
    if(!workspace || workspace_bytes < need)
        return fail(CKB_ERR_WORKSPACE, "grouped GEMM needs %zu bytes of device workspace, got %zu", need,
                    workspace ? workspace_bytes : 0);
    DeviceInfo* dev = nullptr;
    rc              = current_device(&dev);
    if(rc)
        return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    GroupedPlan gp;
    rc = plan_grouped(g, dev, &gp);
    if(rc)
        return rc;
    uintptr_t ws_addr = (reinterpret_cast<uintptr_t>(workspace) + 127u) & ~static_cast<uintptr_t>(127u);
    GroupEntry* d_table = reinterpret_cast<GroupEntry*>(ws_addr);
    if(stream_is_capturing(stream))
    {
        // The copy node of a graph reads its host source again at every replay: the table is kept alive in the
        // library, one per workspace, until the next captured launch with the same workspace replaces it.
        std::lock_guard<std::mutex> lock(g_captured_mutex);
        auto held = std::make_unique<std::vector<GroupEntry>>(g->group_count);
        rc        = fill_group_table(g, gp, held->data());
        if(rc)
            return rc;
        CKB_CUDA(cudaMemcpyAsync(d_table, held->data(), held->size() * sizeof(GroupEntry), cudaMemcpyHostToDevice,
                                 stream));
        // a table that an earlier graph captured for this workspace stays readable: it is retired, not freed
        // (ckb_release_scratch with all_streams set drops them all)
        auto& slot = g_captured_tables[workspace];
        if(slot)
            g_retired_tables.push_back(std::move(slot));
        slot = std::move(held);
    }
    else
    {
        std::vector<GroupEntry> table(g->group_count);
        rc = fill_group_table(g, gp, table.data());
        if(rc)
            return rc;
        // Pageable source: the runtime stages the bytes before returning, so `table` may go out of scope.
        CKB_CUDA(cudaMemcpyAsync(d_table, table.data(), table.size() * sizeof(GroupEntry), cudaMemcpyHostToDevice,
                                 stream));
    }

    KernelParams p;
    fill_grouped_params(p, g, gp, d_table, dev);
    LaunchFn fn = find_launch(MODE_GROUPED, kind_of(g->groups[0].ab_dtype), g->groups[0].epilogue);
    if(!fn)
        return fail(CKB_ERR_UNSUPPORTED, "no kernel instance for epilogue %d", g->groups[0].epilogue);
    return run_timed(fn, gp.bn, gp.cg, p, gp.plan.grid, stream, n_rep, avg_ms);
}

// ---- grouped GEMM without allocation ----------------------------------------------------------------
// The per-group table of the grouped kernel, for callers that cannot hand over a workspace.  The
// array lives in the library image on every device.  In HOST code its name is only a handle:
// the device address comes from cudaGetSymbolAddress (looked up once per device, with that device
// current) and that pointer is what the kernel receives.
static __device__ __align__(256) unsigned char g_noalloc_group_table[CKB_NOALLOC_MAX_GROUPS * sizeof(GroupEntry)];
static_assert(sizeof(GroupEntry) == 640, "the documented size of the fixed table assumes 640-byte entries");

static GroupEntry* g_noalloc_dev_ptr[64] = {};
static GroupEntry g_noalloc_host_table[CKB_NOALLOC_MAX_GROUPS]; // host staging, fixed size
static std::mutex g_noalloc_mutex;

int ckb_grouped_gemm_run_noalloc(const ckb_grouped_gemm_desc* g, void* stream_)
{
    int rc = check_grouped(g, true);
    if(rc)
        return rc;
    if(g->group_count > CKB_NOALLOC_MAX_GROUPS)
        return fail(CKB_ERR_LIMIT,
                    "ckb_grouped_gemm_run_noalloc holds at most %d groups in its fixed table, got %d; "
                    "use ckb_grouped_gemm_run with a caller-provided workspace",
                    CKB_NOALLOC_MAX_GROUPS, g->group_count);
    DeviceInfo* dev = nullptr;
    rc              = current_device(&dev);
    if(rc)
        return rc;
    int ordinal = 0;
    CKB_CUDA(cudaGetDevice(&ordinal));
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if(!g_noalloc_dev_ptr[ordinal])
    {
        // once per device, with that device current
        GroupEntry* ptr = nullptr;
        CKB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_group_table));
        if(!ptr)
            return fail(CKB_ERR_CUDA, "cudaGetSymbolAddress returned a null address for the fixed group table");
        g_noalloc_dev_ptr[ordinal] = ptr;
    }
    GroupEntry* d_table = g_noalloc_dev_ptr[ordinal];

    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if(stream_is_capturing(stream))
        return fail(CKB_ERR_UNSUPPORTED, "grouped GEMM copies its group table from host memory at every launch and "
                                         "cannot be captured into a graph");
    GroupedPlan gp;
    rc = plan_grouped(g, dev, &gp);
    if(rc)
        return rc;
    rc = fill_group_table(g, gp, g_noalloc_host_table);
    if(rc)
        return rc;
    // Every entry this launch reads is rewritten here; stale entries beyond group_count are never
    // read.  Pageable source: the runtime stages the bytes before returning, so the host staging
    // table may be reused as soon as the mutex is released.
    CKB_CUDA(cudaMemcpyAsync(d_table, g_noalloc_host_table, static_cast<size_t>(g->group_count) * sizeof(GroupEntry),
                             cudaMemcpyHostToDevice, stream));

    KernelParams p;
    fill_grouped_params(p, g, gp, d_table, dev);
    LaunchFn fn = find_launch(MODE_GROUPED, kind_of(g->groups[0].ab_dtype), g->groups[0].epilogue);
    if(!fn)
        return fail(CKB_ERR_UNSUPPORTED, "no kernel instance for epilogue %d", g->groups[0].epilogue);
    p.trace = trace_buffer();
    CKB_CUDA(fn(gp.bn, gp.cg, p, gp.plan.grid, stream));
    g_launches.fetch_add(1);
    return CKB_OK;
}

// ---- convolution forward (1-D and 2-D through the 2-D entry point, 3-D) ----------------------------
// One description for both entry points: a 2-D problem is a 3-D one with depth 1.
struct ConvProblem
{
    int dtype, epilogue, nd; // nd = 2 (4-D im2col map) or 3 (5-D)
    int N, K, C;
    int Di, Hi, Wi, Z, Y, X, Do, Ho, Wo;
    int sd, sh, sw, dd, dh, dw;
    int pd, ph, pw, pdr, phr, pwr;
    const void *p_in, *p_wei, *p_bias, *p_resi;
    void* p_out;
    float epi_params[4];
};

static ConvProblem problem_of_2d(const ckb_conv2d_fwd_desc* d)
{
    ConvProblem c{};
    c.dtype = d->dtype, c.epilogue = d->epilogue, c.nd = 2;
    c.N = d->N, c.K = d->K, c.C = d->C;
    c.Di = 1, c.Hi = d->Hi, c.Wi = d->Wi, c.Z = 1, c.Y = d->Y, c.X = d->X, c.Do = 1, c.Ho = d->Ho, c.Wo = d->Wo;
    c.sd = 1, c.sh = d->stride_h, c.sw = d->stride_w, c.dd = 1, c.dh = d->dilation_h, c.dw = d->dilation_w;
    c.pd = 0, c.ph = d->pad_h, c.pw = d->pad_w, c.pdr = 0, c.phr = d->pad_h_right, c.pwr = d->pad_w_right;
    c.p_in = d->p_in, c.p_wei = d->p_wei, c.p_bias = d->p_bias, c.p_resi = d->p_resi, c.p_out = d->p_out;
    memcpy(c.epi_params, d->epi_params, sizeof(c.epi_params));
    return c;
}

static ConvProblem problem_of_3d(const ckb_conv3d_fwd_desc* d)
{
    ConvProblem c{};
    c.dtype = d->dtype, c.epilogue = d->epilogue, c.nd = 3;
    c.N = d->N, c.K = d->K, c.C = d->C;
    c.Di = d->Di, c.Hi = d->Hi, c.Wi = d->Wi, c.Z = d->Z, c.Y = d->Y, c.X = d->X;
    c.Do = d->Do, c.Ho = d->Ho, c.Wo = d->Wo;
    c.sd = d->stride_d, c.sh = d->stride_h, c.sw = d->stride_w;
    c.dd = d->dilation_d, c.dh = d->dilation_h, c.dw = d->dilation_w;
    c.pd = d->pad_d, c.ph = d->pad_h, c.pw = d->pad_w;
    c.pdr = d->pad_d_right, c.phr = d->pad_h_right, c.pwr = d->pad_w_right;
    c.p_in = d->p_in, c.p_wei = d->p_wei, c.p_bias = d->p_bias, c.p_resi = d->p_resi, c.p_out = d->p_out;
    memcpy(c.epi_params, d->epi_params, sizeof(c.epi_params));
    return c;
}

// Multiply-high / shift constants of ckb::FastDiv for the divisor d (1 <= d < 2^31).
static FastDiv make_fast_div(uint32_t d)
{
    FastDiv f{0, 0, d, 0};
    if(d > 1)
    {
        uint32_t log2_ceil = 0;
        while((1ull << log2_ceil) < d)
            ++log2_ceil;
        const uint32_t p = 31 + log2_ceil;
        f.mul            = static_cast<uint32_t>(((1ull << p) + d - 1) / d);
        f.shr            = p - 32;
    }
    return f;
}

static int out_len(int in, int pad_l, int pad_r, int filt, int dil, int stride)
{
    return (in + pad_l + pad_r - ((filt - 1) * dil + 1)) / stride + 1;
}

static int check_conv(const ConvProblem& c, bool need_pointers)
{
    if(c.dtype != CKB_F16 && c.dtype != CKB_BF16 && c.dtype != CKB_I8)
        return fail(CKB_ERR_UNSUPPORTED, "convolution forward supports f16, bf16 and int8");
    if(c.dtype == CKB_BF16 && c.epilogue == CKB_EPI_ADD)
        return fail(CKB_ERR_UNSUPPORTED, "the binary16 Add functor has no bfloat16 instance");
    const int e = c.epilogue;
    if(c.dtype == CKB_I8)
    {
        if(!epilogue_valid_for(e, CKB_I8))
            return fail(CKB_ERR_UNSUPPORTED, "epilogue %d not available for int8 convolution forward", e);
    }
    else if(!(e == CKB_EPI_PASSTHROUGH || e == CKB_EPI_RELU || e == CKB_EPI_ADD_RELU ||
              e == CKB_EPI_ADD_HARDSWISH || e == CKB_EPI_ADD_RELU_ADD || e == CKB_EPI_ADD))
        return fail(CKB_ERR_UNSUPPORTED, "epilogue %d not available for convolution forward", e);
    const int eb = elem_bytes(c.dtype);
    if(c.N < 1 || c.K < 1 || c.C < 1 || c.Di < 1 || c.Hi < 1 || c.Wi < 1 || c.Z < 1 || c.Y < 1 || c.X < 1)
        return fail(CKB_ERR_UNSUPPORTED, "all extents must be positive");
    if(c.sd < 1 || c.sh < 1 || c.sw < 1 || c.dd < 1 || c.dh < 1 || c.dw < 1 || c.pd < 0 || c.ph < 0 || c.pw < 0 ||
       c.pdr < 0 || c.phr < 0 || c.pwr < 0)
        return fail(CKB_ERR_INVALID, "strides and dilations must be >= 1, pads >= 0");
    const int dd = out_len(c.Di, c.pd, c.pdr, c.Z, c.dd, c.sd);
    const int ho = out_len(c.Hi, c.ph, c.phr, c.Y, c.dh, c.sh);
    const int wo = out_len(c.Wi, c.pw, c.pwr, c.X, c.dw, c.sw);
    if(dd != c.Do || ho != c.Ho || wo != c.Wo || dd < 1 || ho < 1 || wo < 1)
        return fail(CKB_ERR_INVALID, "Do/Ho/Wo (%d,%d,%d) do not match the convolution geometry (%d,%d,%d)", c.Do,
                    c.Ho, c.Wo, dd, ho, wo);
    if(c.C % (16 / eb) != 0)
        return fail(CKB_ERR_UNSUPPORTED, "C must be a multiple of %d (16-byte pixel pitch for TMA)", 16 / eb);
    // Limits of the im2col tensor map: traversal stride <= 8, box corners within [-128, 127] (4-D maps) or
    // [-16, 15] (5-D maps).
    if(c.sd > 8 || c.sh > 8 || c.sw > 8)
        return fail(CKB_ERR_UNSUPPORTED, "convolution stride > 8 not supported");
    const int lo = c.nd == 3 ? 16 : 128, hi = c.nd == 3 ? 15 : 127;
    const int up_d = c.pdr - (c.Z - 1) * c.dd, up_h = c.phr - (c.Y - 1) * c.dh, up_w = c.pwr - (c.X - 1) * c.dw;
    if(c.pd > lo || c.ph > lo || c.pw > lo || up_d < -lo || up_h < -lo || up_w < -lo || up_d > hi || up_h > hi ||
       up_w > hi)
        return fail(CKB_ERR_UNSUPPORTED, "padding / filter extent beyond the im2col box-corner range");
    const int max_off = c.nd == 3 ? 15 : 255; // im2col offsets share 16 bits: 8 bits each in a 4-D map, 4 bits each in 5-D
    if((c.Z - 1) * c.dd > max_off || (c.Y - 1) * c.dh > max_off || (c.X - 1) * c.dw > max_off)
        return fail(CKB_ERR_UNSUPPORTED, "filter offset beyond the im2col offset range");
    const int64_t gm = static_cast<int64_t>(c.N) * c.Do * c.Ho * c.Wo;
    if(gm > 0x7FFFFF00ll)
        return fail(CKB_ERR_UNSUPPORTED, "N*Do*Ho*Wo must fit in int32");
    // 2 GB per-tensor limit of the reference (device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp:884-892)
    const int64_t two_gb = int64_t(1) << 31;
    if(static_cast<int64_t>(c.N) * c.Di * c.Hi * c.Wi * c.C * eb > two_gb || gm * c.K * eb > two_gb)
        return fail(CKB_ERR_UNSUPPORTED, "tensor larger than 2 GB");
    const int nd = epi_num_d(e);
    if(need_pointers)
    {
        if(!c.p_in || !c.p_wei || !c.p_out)
            return fail(CKB_ERR_INVALID, "null tensor pointer");
        if(!aligned16(c.p_in) || !aligned16(c.p_wei))
            return fail(CKB_ERR_UNSUPPORTED, "input and weights must be 16-byte aligned");
        if(nd >= 1 && !c.p_bias)
            return fail(CKB_ERR_INVALID, "epilogue needs a bias pointer");
        if(nd >= 2 && !c.p_resi)
            return fail(CKB_ERR_INVALID, "epilogue needs a residual pointer");
    }
    return CKB_OK;
}

static int run_conv(const ConvProblem& c, void* stream, int n_rep, float* avg_ms)
{
    int rc = check_conv(c, true);
    if(rc)
        return rc;
    DeviceInfo* dev = nullptr;
    rc              = current_device(&dev);
    if(rc)
        return rc;
    load_entry_points();
    if(!g_encode_im2col || !g_encode_tiled)
        return fail(CKB_ERR_CUDA, "tensor-map entry points not available");
    const int64_t gm = static_cast<int64_t>(c.N) * c.Do * c.Ho * c.Wo;
    const int bn     = pick_bn(gm, c.K, dev->sm_count);
    const int eb     = elem_bytes(c.dtype);
    const int bk     = BK_BYTES / eb; // channels per k block

    KernelParams p;
    memset(&p, 0, sizeof(p));
    {
        // Input as (C, W, H[, D], N); the column of 128 output pixels is walked by the TMA unit.
        const cuuint64_t C = c.C, W = c.Wi, H = c.Hi, D = c.Di;
        cuuint64_t dims[5], strides[4];
        cuuint32_t estr[5];
        int lower[3], upper[3];
        int rank;
        if(c.nd == 3)
        {
            rank    = 5;
            dims[0] = C, dims[1] = W, dims[2] = H, dims[3] = D, dims[4] = c.N;
            strides[0] = C * eb, strides[1] = W * C * eb, strides[2] = H * W * C * eb, strides[3] = D * H * W * C * eb;
            lower[0] = -c.pw, lower[1] = -c.ph, lower[2] = -c.pd;
            upper[0] = c.pwr - (c.X - 1) * c.dw, upper[1] = c.phr - (c.Y - 1) * c.dh, upper[2] = c.pdr - (c.Z - 1) * c.dd;
            estr[0] = 1, estr[1] = c.sw, estr[2] = c.sh, estr[3] = c.sd, estr[4] = 1;
        }
        else
        {
            rank    = 4;
            dims[0] = C, dims[1] = W, dims[2] = H, dims[3] = c.N;
            strides[0] = C * eb, strides[1] = W * C * eb, strides[2] = H * W * C * eb;
            lower[0] = -c.pw, lower[1] = -c.ph;
            upper[0] = c.pwr - (c.X - 1) * c.dw, upper[1] = c.phr - (c.Y - 1) * c.dh;
            estr[0] = 1, estr[1] = c.sw, estr[2] = c.sh, estr[3] = 1;
        }
        CUresult r = g_encode_im2col(&p.tm_a, tm_dtype(c.dtype), rank, const_cast<void*>(c.p_in), dims, strides, lower,
                                     upper, static_cast<cuuint32_t>(bk), static_cast<cuuint32_t>(BM), estr,
                                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if(r != CUDA_SUCCESS)
            return fail(CKB_ERR_CUDA, "cuTensorMapEncodeIm2col failed (CUresult %d)", static_cast<int>(r));
        // Drivers up to CUDA 13.1 mis-encode im2col maps of tensors smaller than 128 KiB; the
        // published remedy (CUTLASS, cute/atom/copy_traits_sm90_im2col.hpp) clears bit 21 of the
        // descriptor's second 64-bit word.
        const int64_t in_bytes = static_cast<int64_t>(c.N) * c.Di * c.Hi * c.Wi * c.C * eb;
        if(g_driver_version <= 13010 && in_bytes < 131072)
            reinterpret_cast<uint64_t*>(&p.tm_a)[1] &= ~(1ull << 21);
    }
    const int64_t tiles_n = (c.K + bn - 1) / bn;
    const int cg          = pick_cg(((gm + BM - 1) / BM) * tiles_n, bn, dev->sm_count);
    const int64_t tiles_m = (gm + BM * cg - 1) / (BM * cg);
    if(tiles_m * tiles_n > 0x3FFFFFFFll)
        return fail(CKB_ERR_UNSUPPORTED, "too many tiles");
    const WorkPlan plan = plan_work(tiles_m * tiles_n, dev->sm_count / cg, bn, cg);
    const int64_t taps  = static_cast<int64_t>(c.Z) * c.Y * c.X;
    for(int which = 0; which < 2; ++which)
    {
        // Weights K[Z]YXC as (C, taps, K): a box never crosses a filter tap, channels beyond C read 0.
        cuuint64_t dims[3]    = {static_cast<cuuint64_t>(c.C), static_cast<cuuint64_t>(taps), static_cast<cuuint64_t>(c.K)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(c.C) * eb, static_cast<cuuint64_t>(taps) * c.C * eb};
        cuuint32_t box[3]     = {static_cast<cuuint32_t>(bk), 1,
                             static_cast<cuuint32_t>((which == 0 ? bn : bn / plan.split) / cg)};
        cuuint32_t estr[3]    = {1, 1, 1};
        CUresult r = g_encode_tiled(which == 0 ? &p.tm_b : &p.tm_b_split, tm_dtype(c.dtype), 3,
                                    const_cast<void*>(c.p_wei), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if(r != CUDA_SUCCESS)
            return fail(CKB_ERR_CUDA, "cuTensorMapEncodeTiled (weights) failed (CUresult %d)", static_cast<int>(r));
    }
    const int nd = epi_num_d(c.epilogue);
    p.epi.kind   = c.epilogue;
    p.epi.out_i8 = c.dtype == CKB_I8;
    p.epi.bf16   = c.dtype == CKB_BF16;
    memcpy(p.epi.p, c.epi_params, sizeof(p.epi.p));
    p.epi.e    = c.p_out;
    p.epi.lde  = c.K;
    p.epi.d0   = nd >= 1 ? c.p_bias : nullptr;
    p.epi.ldd0 = 0;
    p.epi.d1   = nd >= 2 ? c.p_resi : nullptr;
    p.epi.ldd1 = c.K;
    bool vec   = aligned16(c.p_out) && c.K % (16 / eb) == 0;
    if(nd >= 1)
        vec = vec && aligned16(c.p_bias);
    if(nd >= 2)
        vec = vec && aligned16(c.p_resi);
    p.total_tiles   = static_cast<int32_t>(tiles_m * tiles_n);
    p.split_start   = plan.split_start;
    p.split         = plan.split;
    p.total_work    = plan.total_work;
    p.num_slots     = (plan.total_work + plan.grid / cg - 1) / (plan.grid / cg);
    p.M             = static_cast<int32_t>(gm);
    p.N             = c.K;
    p.tiles_n       = static_cast<int32_t>(tiles_n);
    p.conv.nd3      = c.nd == 3 ? 1 : 0;
    p.conv.Do       = c.Do;
    p.conv.Ho       = c.Ho;
    p.conv.Wo       = c.Wo;
    p.conv.HoWo     = c.Ho * c.Wo;
    p.conv.DoHoWo   = c.Do * c.Ho * c.Wo;
    p.conv.div_wo     = make_fast_div(static_cast<uint32_t>(c.Wo));
    p.conv.div_howo   = make_fast_div(static_cast<uint32_t>(c.Ho) * c.Wo);
    p.conv.div_dohowo = make_fast_div(static_cast<uint32_t>(c.Do) * c.Ho * c.Wo);
    p.conv.Z        = c.Z;
    p.conv.Y        = c.Y;
    p.conv.X        = c.X;
    p.conv.c_blocks = (c.C + bk - 1) / bk;
    p.conv.stride_d = c.sd;
    p.conv.stride_h = c.sh;
    p.conv.stride_w = c.sw;
    p.conv.dil_d    = c.dd;
    p.conv.dil_h    = c.dh;
    p.conv.dil_w    = c.dw;
    p.conv.pad_d    = c.pd;
    p.conv.pad_h    = c.ph;
    p.conv.pad_w    = c.pw;
    p.num_kb        = static_cast<int32_t>(taps * p.conv.c_blocks);
    p.vec_ok        = vec ? 1 : 0;
    if(vec)
    {
        rc = encode_e_map(&p.tm_e, c.dtype, c.p_out, gm, c.K, c.K);
        if(rc)
            return rc;
    }
    p.wait_limit_ns = wait_limit_ns();
    p.status        = dev->status;
    LaunchFn fn = find_launch(MODE_CONV, kind_of(c.dtype), c.epilogue);
    if(!fn)
        return fail(CKB_ERR_UNSUPPORTED, "no kernel instance for epilogue %d", c.epilogue);
    return run_timed(fn, bn, cg, p, plan.grid, static_cast<cudaStream_t>(stream), n_rep, avg_ms);
}

int ckb_conv2d_fwd_supported(const ckb_conv2d_fwd_desc* desc)
{
    return desc ? check_conv(problem_of_2d(desc), false) : fail(CKB_ERR_INVALID, "null descriptor");
}

int ckb_conv2d_fwd_run(const ckb_conv2d_fwd_desc* d, void* stream, int n_rep, float* avg_ms)
{
    return d ? run_conv(problem_of_2d(d), stream, n_rep, avg_ms) : fail(CKB_ERR_INVALID, "null descriptor");
}

int ckb_conv3d_fwd_supported(const ckb_conv3d_fwd_desc* desc)
{
    return desc ? check_conv(problem_of_3d(desc), false) : fail(CKB_ERR_INVALID, "null descriptor");
}

int ckb_conv3d_fwd_run(const ckb_conv3d_fwd_desc* d, void* stream, int n_rep, float* avg_ms)
{
    return d ? run_conv(problem_of_3d(d), stream, n_rep, avg_ms) : fail(CKB_ERR_INVALID, "null descriptor");
}

} // extern "C"
