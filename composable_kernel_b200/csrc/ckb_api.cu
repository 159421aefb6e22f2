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
thread_local char t_last_plan[200] = "";
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
    int cluster_cap[3] = {-1, -1, -1}; // clusters of 2 / 4 / 8 CTAs resident at once (-1: not asked yet)
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
        // A process that may use only part of the GPU (an MPS active-thread percentage, a green context) says so
        // with CKB_SM_LIMIT: the K-split plans let units wait for one another, so every unit of a launch has to be
        // resident at the same time, and the runtime reports the whole device whatever the partition is.
        if(const char* lim = getenv("CKB_SM_LIMIT"))
        {
            const int n = atoi(lim) & ~1;
            if(n >= 2 && n < d.sm_count)
                d.sm_count = n;
        }
        d.cc_major = prop.major;
        d.cc_minor = prop.minor;
        if(prop.major != 10)
            return fail(CKB_ERR_UNSUPPORTED,
                        "device '%s' is compute capability %d.%d; this library holds sm_100a code only",
                        prop.name, prop.major, prop.minor);
        void* sym = nullptr;
        CKB_CUDA(cudaGetSymbolAddress(&sym, g_status_word));
        d.status = static_cast<uint32_t*>(sym); // a __device__ variable: zero when the module is loaded
        d.ready  = true;
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

// Front of the scratch buffer: the tail-tile counters, then the flags of the balanced K ranges (one per parking
// slot x CTA x epilogue warp = 8 per SM); 16 KiB hold both for up to 384 SMs.
constexpr size_t kScratchCounterBytes = 16 * 1024;
static_assert(kScratchCounterBytes >= kMaxTailTiles * sizeof(uint32_t) + 384 * 8 * sizeof(uint32_t), "counter area");

// Scratch of `stream` for the K-split plans; nullptr when the device has no memory left for it or the stream is
// capturing (the caller then keeps a plan that needs none).  Every K-split plan parks at most one accumulator tile
// per unit (tail tiles x slices <= units), so the buffer is sized once for that worst case - counters + SMs x 128
// KiB, 19 MB on a B200 - and never grows: no later call frees or allocates.  The counters are zeroed on the stream
// that will use them (ordered before the first kernel that reads them, also on non-blocking streams) and are left
// at zero by every kernel.
void* scratch_for(DeviceInfo* dev, cudaStream_t stream, size_t bytes)
{
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    // A launch that is being captured into a graph gets no scratch: the graph may be replayed on any stream,
    // next to other launches that use this stream's buffer, and a capture must not see an allocation either.
    if(stream_is_capturing(stream))
        return nullptr;
    Scratch& sc            = dev->scratch[stream];
    const size_t worst     = static_cast<size_t>(dev->sm_count) * BM * 256 * sizeof(uint32_t);
    const size_t need      = kScratchCounterBytes + (bytes > worst ? bytes : worst);
    if(sc.bytes >= need)
        return sc.ptr;
    if(sc.ptr) // only reachable if a plan ever parks more than one tile per unit
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
    if(cudaMemsetAsync(ptr, 0, kScratchCounterBytes, stream) != cudaSuccess)
    {
        cudaGetLastError();
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

// Test hook: CKB_TEST_KSLICE_WAIT_EXTRA=n makes the reductions of the K-split plans wait for n arrivals more than
// will ever come, so that the bounded wait runs out (with a short CKB_WAIT_LIMIT_MS) and the give-up path executes.
uint32_t test_kslice_wait_extra()
{
    const char* s = getenv("CKB_TEST_KSLICE_WAIT_EXTRA");
    return s ? static_cast<uint32_t>(atoi(s)) : 0u;
}

// Tile configuration of a call: the descriptor's tile_config field when it is set, else the environment overrides
// CKB_FORCE_BN / CKB_FORCE_CG / CKB_NO_SPLITK (read at every call), else all zero = the library decides.
int check_tile_config(int32_t tc)
{
    const int bn = tc & 0xFFF, cg = (tc >> 12) & 0xF, kbatch = (tc >> 20) & 0xFF, rest = (tc >> 18) & 0x3, top = tc >> 28;
    const int balanced = (tc >> 17) & 1, no_ksplit = (tc >> 16) & 1;
    if(tc < 0 || rest != 0 || top != 0 || !(bn == 0 || bn == 64 || bn == 128 || bn == 256) || cg > 2 ||
       !(kbatch == 0 || kbatch == 1 || kbatch == 2 || kbatch == 4 || kbatch == 8))
        return fail(CKB_ERR_INVALID, "tile_config 0x%x is not a CKB_TILE_CONFIG / CKB_TILE_CONFIG_KBATCH value", tc);
    if(kbatch >= 2 && cg == 2)
        return fail(CKB_ERR_UNSUPPORTED, "a K batch runs on single-CTA tiles (cg = 1)");
    if(balanced && (no_ksplit || kbatch != 0))
        return fail(CKB_ERR_INVALID, "balanced K ranges exclude a K batch and the no-K-split flag");
    if(cg == 2 && bn != 256 && bn != 0)
        return fail(CKB_ERR_UNSUPPORTED, "a CTA pair (cg = 2) works on 256-wide tiles only");
    return CKB_OK;
}

TileConfig tile_config_of(int32_t tc)
{
    TileConfig t;
    if(tc != 0)
    {
        t.bn        = tc & 0xFFF;
        t.cg        = (tc >> 12) & 0xF;
        t.no_ksplit = (tc >> 16) & 1;
        t.stream_k  = (tc >> 17) & 1;
        t.kbatch    = (tc >> 20) & 0xFF;
        if(t.kbatch == 1) // one K batch = no split
        {
            t.kbatch    = 0;
            t.no_ksplit = 1;
        }
        return t;
    }
    const char* s = getenv("CKB_FORCE_BN");
    const int bn  = s ? atoi(s) : 0;
    t.bn          = (bn == 64 || bn == 128 || bn == 256) ? bn : 0;
    s             = getenv("CKB_FORCE_CG");
    const int cg  = s ? atoi(s) : 0;
    t.cg          = (cg == 1 || cg == 2) ? cg : 0;
    s             = getenv("CKB_NO_SPLITK");
    t.no_ksplit   = (s && atoi(s) != 0) ? 1 : 0;
    return t;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int elem_bytes(int dtype) { return dtype == CKB_I8 ? 1 : 2; }

CUtensorMapDataType tm_dtype(int dtype)
{
    return dtype == CKB_I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                           : dtype == CKB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

// cuTensorMapEncodeTiled behind a small per-thread cache.  A tensor map is a pure function of the arguments below,
// and callers launch the same problem again and again (a timing loop, a layer executed every step): a hit copies
// 128 bytes instead of calling into the driver (about a microsecond per map, four maps per GEMM).
struct TiledKey
{
    const void* ptr;
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    int32_t dtype, rank, swizzle, promo;
};
struct TiledEntry
{
    TiledKey key;
    CUtensorMap map;
    bool used;
};
constexpr int kTiledCacheSize = 32;
thread_local TiledEntry t_tiled_cache[kTiledCacheSize];
thread_local int t_tiled_next = 0;

int encode_tiled(CUtensorMap* tm, int dtype, int rank, const void* ptr, const cuuint64_t* dims, const cuuint64_t* strides,
                 const cuuint32_t* box, CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promo, const char* what)
{
    load_entry_points();
    if(!g_encode_tiled)
        return fail(CKB_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    TiledKey key;
    memset(&key, 0, sizeof(key));
    key.ptr = ptr;
    for(int i = 0; i < rank; ++i)
    {
        key.dims[i] = dims[i];
        key.box[i]  = box[i];
        if(i + 1 < rank)
            key.strides[i] = strides[i];
    }
    key.dtype = dtype, key.rank = rank, key.swizzle = swizzle, key.promo = promo;
    for(const TiledEntry& e : t_tiled_cache)
        if(e.used && memcmp(&e.key, &key, sizeof(key)) == 0)
        {
            *tm = e.map;
            return CKB_OK;
        }
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encode_tiled(tm, tm_dtype(dtype), rank, const_cast<void*>(ptr), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if(r != CUDA_SUCCESS)
        return fail(CKB_ERR_CUDA, "cuTensorMapEncodeTiled (%s) failed (CUresult %d): dims %llu x %llu x %llu, pitch %llu B",
                    what, static_cast<int>(r), (unsigned long long)key.dims[0], (unsigned long long)key.dims[1],
                    (unsigned long long)key.dims[2], (unsigned long long)key.strides[0]);
    TiledEntry& slot = t_tiled_cache[t_tiled_next];
    t_tiled_next     = (t_tiled_next + 1) % kTiledCacheSize;
    slot.key         = key;
    slot.map         = *tm;
    slot.used        = true;
    return CKB_OK;
}

// K-major matrix [rows][k] with row pitch `ld` elements -> 2-D map, box = 128 bytes x box_rows.
// batch >= 1 adds a third dimension of `batch` matrices `batch_stride` elements apart (box extent 1).
int encode_kmajor_2d(CUtensorMap* tm, int dtype, const void* ptr, int64_t rows, int64_t k,
                     int64_t ld, int box_rows, int64_t batch = 0, int64_t batch_stride = 0)
{
    const int eb          = elem_bytes(dtype);
    cuuint64_t dims[3]    = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * eb, static_cast<cuuint64_t>(batch_stride) * eb};
    cuuint32_t box[3]     = {static_cast<cuuint32_t>(BK_BYTES / eb), static_cast<cuuint32_t>(box_rows), 1};
    return encode_tiled(tm, dtype, batch >= 1 ? 3 : 2, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "K-major operand");
}

// MN-major matrix (the M or N index contiguous, pitch `ld` elements between consecutive k) -> 2-D map
// whose box is one swizzle atom column: 128 bytes of MN positions x the k rows of one stage.
int encode_mnmajor_2d(CUtensorMap* tm, int dtype, const void* ptr, int64_t mn, int64_t k, int64_t ld,
                      int64_t batch = 0, int64_t batch_stride = 0)
{
    const int eb          = elem_bytes(dtype);
    cuuint64_t dims[3]    = {static_cast<cuuint64_t>(mn), static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(batch)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * eb, static_cast<cuuint64_t>(batch_stride) * eb};
    cuuint32_t box[3]     = {static_cast<cuuint32_t>(BK_BYTES / eb), static_cast<cuuint32_t>(BK_BYTES / eb), 1};
    return encode_tiled(tm, dtype, batch >= 1 ? 3 : 2, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "MN-major operand");
}

// E (M x N row-major, pitch `lde` elements) as the (columns, rows[, batch]) map of the epilogue's staged stores:
// 32 x 32 box whose rows are 64 bytes (16-bit E, 64-byte swizzle) or 32 bytes (int8 E, 32-byte swizzle).
// Only encoded when E allows 16-byte accesses (base and pitch multiples of 16 bytes).
int encode_e_map(CUtensorMap* tm, int dtype, const void* ptr, int64_t m, int64_t n, int64_t lde, int64_t batch = 0,
                 int64_t batch_stride = 0)
{
    const int eb          = elem_bytes(dtype);
    cuuint64_t dims[3]    = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(m), static_cast<cuuint64_t>(batch)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(lde) * eb, static_cast<cuuint64_t>(batch_stride) * eb};
    cuuint32_t box[3]     = {32, 32, 1};
    return encode_tiled(tm, dtype, batch >= 1 ? 3 : 2, ptr, dims, strides, box,
                        eb == 1 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                        "E");
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
int min_b_rows(int dtype, bool b_mn) { return b_mn ? BK_BYTES / elem_bytes(dtype) : 32; }

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

// Shared validation of one GEMM problem.  strict_tma: A and B must be readable by TMA in place (16-byte aligned
// base and pitch) - the rule of the batched and grouped entry points; the plain GEMM copies such operands first.
int check_gemm(const ckb_gemm_desc* d, bool need_pointers, bool strict_tma)
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
    if(strict_tma && ((d->lda * eb) % 16 != 0 || (d->ldb * eb) % 16 != 0))
        return fail(CKB_ERR_UNSUPPORTED, "lda and ldb must be multiples of 16 bytes (TMA row pitch)");
    if(int rc = check_tile_config(d->tile_config))
        return rc;
    for(int i = 0; i < d->n_ds; ++i)
        if(d->ldd[i] != 0 && d->ldd[i] < d->N)
            return fail(CKB_ERR_INVALID, "ldd[%d] smaller than N", i);
    if(need_pointers)
    {
        if(!d->p_a || !d->p_b || !d->p_e)
            return fail(CKB_ERR_INVALID, "null tensor pointer");
        if(strict_tma && (!aligned16(d->p_a) || !aligned16(d->p_b)))
            return fail(CKB_ERR_UNSUPPORTED, "A and B must be 16-byte aligned");
        if((reinterpret_cast<uintptr_t>(d->p_a) | reinterpret_cast<uintptr_t>(d->p_b)) % eb != 0)
            return fail(CKB_ERR_INVALID, "A or B is not aligned to its element size");
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

// Remembers what the calling thread's last launch looked like (ckb_last_plan).
void note_plan(const char* what, int bn, int cg, int grid, const PlanParams& pp, int copies)
{
    snprintf(t_last_plan, sizeof(t_last_plan),
             "%s tile=%dx%d cg=%d grid=%d tiles=%d col_split=%d ksplit=%d cluster_k=%d balanced=%d slots=%d copies=%d", what,
             BM * cg, bn, cg, grid, pp.total_tiles, pp.split, pp.ksplit, pp.cluster_k ? pp.ksplit : 0,
             pp.stream_k ? pp.ks_kb : 0, pp.num_slots, copies);
}

// Work that has to run on the stream before the contraction kernel of the same call: pitch-fixing copies of
// operands that TMA cannot read in place (see repack_pitch_kernel).  Part of every timed repetition.
struct Repack
{
    const void* src;
    void* dst;
    int64_t outer, inner, ld_src, ld_dst;
    int elem_bytes;
};

// Copies an [outer][inner] matrix with pitch ld_src (any alignment) into one with pitch ld_dst (a multiple of 16
// bytes, base 16-byte aligned) and writes zeros into the padding.  One thread per 16 bytes of the destination.
template <typename T>
__global__ void repack_pitch_kernel(const T* __restrict__ src, T* __restrict__ dst, int64_t outer, int64_t inner,
                                    int64_t ld_src, int64_t ld_dst)
{
    constexpr int PER = 16 / sizeof(T);
    const int64_t vec_per_row = ld_dst / PER;
    const int64_t total       = outer * vec_per_row;
    for(int64_t v = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; v < total;
        v += static_cast<int64_t>(gridDim.x) * blockDim.x)
    {
        const int64_t row = v / vec_per_row, col0 = (v - row * vec_per_row) * PER;
        alignas(16) T tmp[PER];
#pragma unroll
        for(int i = 0; i < PER; ++i)
            tmp[i] = col0 + i < inner ? src[row * ld_src + col0 + i] : T(0);
        *reinterpret_cast<uint4*>(dst + row * ld_dst + col0) = *reinterpret_cast<const uint4*>(tmp);
    }
}

cudaError_t launch_repack(const Repack& r, cudaStream_t stream)
{
    const int64_t vecs = r.outer * (r.ld_dst * r.elem_bytes / 16);
    if(vecs <= 0)
        return cudaSuccess;
    const int threads = 256;
    const int64_t want = (vecs + threads - 1) / threads;
    const int blocks   = static_cast<int>(want < 148 * 16 ? want : 148 * 16);
    if(r.elem_bytes == 1)
        repack_pitch_kernel<int8_t><<<blocks, threads, 0, stream>>>(static_cast<const int8_t*>(r.src),
                                                                    static_cast<int8_t*>(r.dst), r.outer, r.inner,
                                                                    r.ld_src, r.ld_dst);
    else
        repack_pitch_kernel<uint16_t><<<blocks, threads, 0, stream>>>(static_cast<const uint16_t*>(r.src),
                                                                      static_cast<uint16_t*>(r.dst), r.outer, r.inner,
                                                                      r.ld_src, r.ld_dst);
    return cudaGetLastError();
}

// One launch, or the reference timing protocol (kernel_launch.hpp:12-74): a warm-up launch, then n_rep launches
// between two events.  `pre` / `n_pre`: copies that belong to the call and run before the kernel every time.
int run_timed(LaunchFn fn, int bn, int cg, const KernelParams& p_in, int grid, cudaStream_t stream, int n_rep,
              float* avg_ms, const Repack* pre = nullptr, int n_pre = 0)
{
    KernelParams p = p_in;
    p.trace        = trace_buffer();
    if(avg_ms)
        *avg_ms = 0.f;
    auto once = [&]() -> cudaError_t {
        for(int i = 0; i < n_pre; ++i)
        {
            cudaError_t e = launch_repack(pre[i], stream);
            if(e != cudaSuccess)
                return e;
        }
        return fn(bn, cg, p, grid, stream);
    };
    if(n_rep <= 0)
    {
        CKB_CUDA(once());
        g_launches.fetch_add(1 + n_pre);
        return CKB_OK;
    }
    CKB_CUDA(once()); // warm-up
    g_launches.fetch_add(1 + n_pre);
    cudaEvent_t start, stop;
    CKB_CUDA(cudaEventCreate(&start));
    CKB_CUDA(cudaEventCreate(&stop));
    CKB_CUDA(cudaDeviceSynchronize());
    CKB_CUDA(cudaEventRecord(start, stream));
    for(int i = 0; i < n_rep; ++i)
    {
        cudaError_t e = once();
        if(e != cudaSuccess)
        {
            cudaEventDestroy(start);
            cudaEventDestroy(stop);
            return fail(CKB_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
        }
    }
    g_launches.fetch_add(static_cast<uint64_t>(n_rep) * (1 + n_pre));
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

// Stream-ordered temporary for repacked operands: allocated and freed on the call's stream (cudaMallocAsync /
// cudaFreeAsync from the device's default pool), so neither end synchronises the device.
struct StreamTemp
{
    void* ptr = nullptr;
    cudaStream_t stream = nullptr;
    ~StreamTemp()
    {
        if(ptr)
            cudaFreeAsync(ptr, stream);
    }
};

bool tma_readable(const void* p, int64_t ld, int eb) { return aligned16(p) && (ld * eb) % 16 == 0; }

} // namespace

namespace ckb {
extern template cudaError_t cluster_capacity<MODE_GEMM, KIND_F16, CKB_EPI_PASSTHROUGH>(int, int*);
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

const char* ckb_last_plan(void) { return t_last_plan; }

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
        {
            std::lock_guard<std::mutex> lock2(g_dev_mutex);
            for(auto& kv : dev->scratch)
                if(kv.second.ptr)
                    cudaMemset(kv.second.ptr, 0, kScratchCounterBytes);
        }
        // the zeroing above runs on the legacy default stream: finish it before the caller launches on any other
        CKB_CUDA(cudaDeviceSynchronize());
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
int ckb_gemm_supported(const ckb_gemm_desc* desc) { return check_gemm(desc, false, false); }

// Strides between the matrices of a batch (elements); batch = 0 for a plain GEMM.
struct BatchInfo
{
    int64_t batch, stride_a, stride_b, stride_e, stride_d[2];
    bool vec_ok; // every batch of E / D keeps the 16-byte alignment of the first
};

static int gemm_run_impl(const ckb_gemm_desc* d_in, const BatchInfo& bi, void* stream_, int n_rep, float* avg_ms)
{
    int rc = CKB_OK;
    DeviceInfo* dev = nullptr;
    rc              = current_device(&dev);
    if(rc)
        return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    ckb_gemm_desc dd    = *d_in;
    const ckb_gemm_desc* d = &dd;
    const bool a_mn  = a_is_mn_major(d), b_mn = b_is_mn_major(d);
    const int eb     = elem_bytes(d->ab_dtype);
    const bool capturing = stream_is_capturing(stream);

    // Operands whose base or pitch is not a multiple of 16 bytes cannot be read by TMA in place: they are copied
    // into a stream-ordered temporary with a padded pitch first (the reference serves such problems with its
    // scalar-load instances, ABlockTransferSrcScalarPerVector = 1).  The copy is part of the call and of its timing.
    Repack pre[2];
    int n_pre = 0;
    StreamTemp temp;
    temp.stream = stream;
    {
        const bool a_bad = !tma_readable(d->p_a, d->lda, eb), b_bad = !tma_readable(d->p_b, d->ldb, eb);
        if(a_bad || b_bad)
        {
            if(bi.batch > 0)
                return fail(CKB_ERR_UNSUPPORTED, "batched GEMM needs 16-byte aligned operands and pitches");
            if(capturing)
                return fail(CKB_ERR_UNSUPPORTED, "operands that need a pitch-fixing copy cannot be captured into a graph");
            const int64_t per16   = 16 / eb;
            const int64_t a_outer = a_mn ? d->K : d->M, a_inner = a_mn ? d->M : d->K;
            const int64_t b_outer = b_mn ? d->K : d->N, b_inner = b_mn ? d->N : d->K;
            const int64_t lda_p = (a_inner + per16 - 1) / per16 * per16, ldb_p = (b_inner + per16 - 1) / per16 * per16;
            const size_t a_bytes = a_bad ? (static_cast<size_t>(a_outer) * lda_p * eb + 255) & ~size_t(255) : 0;
            const size_t b_bytes = b_bad ? (static_cast<size_t>(b_outer) * ldb_p * eb + 255) & ~size_t(255) : 0;
            CKB_CUDA(cudaMallocAsync(&temp.ptr, a_bytes + b_bytes, stream));
            if(a_bad)
            {
                pre[n_pre++] = Repack{d->p_a, temp.ptr, a_outer, a_inner, d->lda, lda_p, eb};
                dd.p_a       = temp.ptr;
                dd.lda       = lda_p;
            }
            if(b_bad)
            {
                void* dst    = static_cast<char*>(temp.ptr) + a_bytes;
                pre[n_pre++] = Repack{d->p_b, dst, b_outer, b_inner, d->ldb, ldb_p, eb};
                dd.p_b       = dst;
                dd.ldb       = ldb_p;
            }
        }
    }

    GemmPlanInput in;
    in.M          = d->M;
    in.N          = d->N;
    in.num_kb     = static_cast<int>((d->K + BK_BYTES / eb - 1) / (BK_BYTES / eb));
    in.batch      = bi.batch;
    in.sm_count   = dev->sm_count;
    in.b_min      = min_b_rows(d->ab_dtype, b_mn);
    in.force      = tile_config_of(d->tile_config);
    // Measured on 3840 x 4096 x 4096: +5 % for 16-bit operands with a D-less epilogue; a loss for int8 (tiles
    // half as long) and for epilogues that read D tensors (bound by power: parking the partials through L2 costs
    // more energy than the narrow MMAs it removes) - those keep the column slices.
    in.ks_pays    = d->ab_dtype != CKB_I8 && d->n_ds == 0;
    in.ks_allowed = !capturing;
    in.bal_ok     = bi.batch == 0; // balanced K ranges: every plain GEMM (instances of their own where ks_pays is false)
    in.cluster_ok = true;
    {
        // asked once per device: how many clusters of 2 / 4 / 8 CTAs fit at the same time
        std::lock_guard<std::mutex> lock(g_dev_mutex);
        for(int i = 0; i < 3; ++i)
        {
            if(dev->cluster_cap[i] < 0)
            {
                int n = 0;
                if(cluster_capacity<MODE_GEMM, KIND_F16, CKB_EPI_PASSTHROUGH>(2 << i, &n) != cudaSuccess)
                {
                    cudaGetLastError();
                    n = 0;
                }
                const int limit    = dev->sm_count / (2 << i); // a CKB_SM_LIMIT partition shrinks it further
                dev->cluster_cap[i] = n < limit ? n : limit;
            }
            in.cluster_cap[i] = dev->cluster_cap[i];
        }
    }
    GemmPlan gp;
    if(!plan_gemm(in, &gp))
        return fail(CKB_ERR_UNSUPPORTED, "too many tiles");
    KernelParams p;
    memset(&p, 0, sizeof(p));
    if(gp.pp.ksplit >= 2 || gp.pp.stream_k != 0)
    {
        // the K split needs scratch; without it the column-slice plan stands
        void* sc = scratch_for(dev, stream, gp.partial_bytes);
        if(sc)
        {
            p.ks_counters   = static_cast<uint32_t*>(sc);
            p.ks_flags      = p.ks_counters + kMaxTailTiles;
            p.ks_partials   = reinterpret_cast<uint32_t*>(static_cast<char*>(sc) + kScratchCounterBytes);
            p.ks_wait_extra = test_kslice_wait_extra();
        }
        else
        {
            in.ks_allowed = false;
            if(!plan_gemm(in, &gp))
                return fail(CKB_ERR_UNSUPPORTED, "too many tiles");
        }
    }
    const int bn = gp.bn, cg = gp.cg;
    rc = encode_operand(&p.tm_a, d->ab_dtype, d->p_a, d->M, d->K, d->lda, a_mn, BM, bi.batch, bi.stride_a);
    if(rc)
        return rc;
    rc = encode_operand(&p.tm_b, d->ab_dtype, d->p_b, d->N, d->K, d->ldb, b_mn, bn / cg, bi.batch, bi.stride_b);
    if(rc)
        return rc;
    rc = encode_operand(&p.tm_b_split, d->ab_dtype, d->p_b, d->N, d->K, d->ldb, b_mn, gp.b_split_rows, bi.batch,
                        bi.stride_b);
    if(rc)
        return rc;
    fill_epilogue(p.epi, d);
    p.plan            = gp.pp;
    p.batch_stride_e  = bi.stride_e;
    p.batch_stride_d0 = bi.stride_d[0];
    p.batch_stride_d1 = bi.stride_d[1];
    p.mn_major      = (a_mn ? 1 : 0) | (b_mn ? 2 : 0);
    p.M             = static_cast<int32_t>(d->M);
    p.N             = static_cast<int32_t>(d->N);
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
    note_plan("gemm", bn, cg, gp.grid, p.plan, n_pre);
    {
        const size_t n = strlen(t_last_plan);
        snprintf(t_last_plan + n, sizeof(t_last_plan) - n, " cluster_cap=%d/%d/%d", in.cluster_cap[0], in.cluster_cap[1],
                 in.cluster_cap[2]);
    }
    return run_timed(fn, bn, cg, p, gp.grid, stream, n_rep, avg_ms, pre, n_pre);
}

int ckb_gemm_run(const ckb_gemm_desc* d, void* stream, int n_rep, float* avg_ms)
{
    int rc = check_gemm(d, true, false);
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
    int rc = check_gemm(&b->gemm, need_pointers, true);
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
    if(int rc = check_tile_config(g->tile_config))
        return rc;
    const ckb_gemm_desc& g0 = g->groups[0];
    for(int i = 0; i < g->group_count; ++i)
    {
        const ckb_gemm_desc& gi = g->groups[i];
        int rc                  = check_gemm(&gi, need_pointers, true);
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

// Tile shape, CTA grouping and work plan of a grouped problem (plan_grouped of ckb_plan.h), and its device table.
struct GroupedLaunch
{
    GroupedPlan plan;
    int mn_major      = 0;
    GroupTiles* tiles = nullptr; // one per group, caller-provided
};

// `shapes` and `tiles`: caller-provided arrays of group_count elements (the allocation-free entry point hands in
// fixed arrays).
static int plan_grouped_call(const ckb_grouped_gemm_desc* g, const DeviceInfo* dev, int64_t (*shapes)[3],
                             GroupTiles* tiles, GroupedLaunch* gl)
{
    const int dtype = g->groups[0].ab_dtype;
    const bool a_mn = a_is_mn_major(&g->groups[0]), b_mn = b_is_mn_major(&g->groups[0]);
    const int bk    = BK_BYTES / elem_bytes(dtype);
    for(int i = 0; i < g->group_count; ++i)
    {
        shapes[i][0] = g->groups[i].M;
        shapes[i][1] = g->groups[i].N;
        shapes[i][2] = (g->groups[i].K + bk - 1) / bk;
    }
    gl->tiles    = tiles;
    gl->mn_major = (a_mn ? 1 : 0) | (b_mn ? 2 : 0);
    if(!plan_grouped(shapes, g->group_count, dev->sm_count, min_b_rows(dtype, b_mn), tile_config_of(g->tile_config),
                     tiles, &gl->plan))
        return fail(CKB_ERR_UNSUPPORTED, "too many tiles");
    return CKB_OK;
}

static int fill_group_table(const ckb_grouped_gemm_desc* g, const GroupedLaunch& gl, GroupEntry* table)
{
    const int dtype = g->groups[0].ab_dtype;
    const bool a_mn = (gl.mn_major & 1) != 0, b_mn = (gl.mn_major & 2) != 0;
    const int bn = gl.plan.bn, cg = gl.plan.cg;
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
        rc = encode_operand(&ge.tm_b_split, dtype, d.p_b, d.N, d.K, d.ldb, b_mn, gl.plan.b_split_rows);
        if(rc)
            return rc;
        ge.M          = static_cast<int32_t>(d.M);
        ge.N          = static_cast<int32_t>(d.N);
        ge.K          = static_cast<int32_t>(d.K);
        ge.tiles_m    = gl.tiles[i].tiles_m;
        ge.tiles_n    = gl.tiles[i].tiles_n;
        ge.tile_start = gl.tiles[i].tile_start;
        ge.num_kb     = gl.tiles[i].num_kb;
        ge.m_fastest  = gl.tiles[i].m_fastest;
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
    }
    return CKB_OK;
}

static void fill_grouped_params(KernelParams& p, const ckb_grouped_gemm_desc* g, const GroupedLaunch& gl,
                                const GroupEntry* d_table, const DeviceInfo* dev)
{
    memset(&p, 0, sizeof(p));
    fill_epilogue(p.epi, &g->groups[0]);
    p.groups        = d_table;
    p.plan          = gl.plan.pp;
    p.mn_major      = gl.mn_major;
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
    GroupedLaunch gp;
    std::vector<int64_t> shapes(static_cast<size_t>(g->group_count) * 3);
    std::vector<GroupTiles> tiles(g->group_count);
    rc = plan_grouped_call(g, dev, reinterpret_cast<int64_t(*)[3]>(shapes.data()), tiles.data(), &gp);
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
    note_plan("grouped", gp.plan.bn, gp.plan.cg, gp.plan.grid, p.plan, 0);
    return run_timed(fn, gp.plan.bn, gp.plan.cg, p, gp.plan.grid, stream, n_rep, avg_ms);
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
static int64_t g_noalloc_shapes[CKB_NOALLOC_MAX_GROUPS][3];      // planner input / output, fixed size
static GroupTiles g_noalloc_tiles[CKB_NOALLOC_MAX_GROUPS];
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
    GroupedLaunch gp;
    rc = plan_grouped_call(g, dev, g_noalloc_shapes, g_noalloc_tiles, &gp);
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
    CKB_CUDA(fn(gp.plan.bn, gp.plan.cg, p, gp.plan.grid, stream));
    g_launches.fetch_add(1);
    return CKB_OK;
}

// ---- convolution forward (1-D and 2-D through the 2-D entry point, 3-D) ----------------------------
// One description for both entry points: a 2-D problem is a 3-D one with depth 1.
struct ConvProblem
{
    int dtype, epilogue, nd; // nd = 2 (4-D im2col map) or 3 (5-D)
    int tile_config;
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
    c.dtype = d->dtype, c.epilogue = d->epilogue, c.nd = 2, c.tile_config = d->tile_config;
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
    c.dtype = d->dtype, c.epilogue = d->epilogue, c.nd = 3, c.tile_config = d->tile_config;
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
    if(int rc = check_tile_config(c.tile_config))
        return rc;
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
        if((reinterpret_cast<uintptr_t>(c.p_in) | reinterpret_cast<uintptr_t>(c.p_wei)) % eb != 0)
            return fail(CKB_ERR_INVALID, "input or weights not aligned to the element size");
        if(nd >= 1 && !c.p_bias)
            return fail(CKB_ERR_INVALID, "epilogue needs a bias pointer");
        if(nd >= 2 && !c.p_resi)
            return fail(CKB_ERR_INVALID, "epilogue needs a residual pointer");
    }
    return CKB_OK;
}

static int run_conv(const ConvProblem& c_in, void* stream_, int n_rep, float* avg_ms)
{
    int rc = check_conv(c_in, true);
    if(rc)
        return rc;
    DeviceInfo* dev = nullptr;
    rc              = current_device(&dev);
    if(rc)
        return rc;
    load_entry_points();
    if(!g_encode_im2col || !g_encode_tiled)
        return fail(CKB_ERR_CUDA, "tensor-map entry points not available");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    ConvProblem c       = c_in;
    const int eb        = elem_bytes(c.dtype);
    const int bk        = BK_BYTES / eb; // channels per k block

    // A channel count whose pixel pitch is not a multiple of 16 bytes (the reference's OddC instances,
    // device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp:921-933, e.g. C = 3) or an unaligned base cannot be read by TMA in
    // place: input and weights are copied into a stream-ordered temporary with the channels zero-padded to the next
    // multiple of 16 bytes, and the problem runs with that channel count (zero channels add nothing to any sum).
    Repack pre[2];
    int n_pre = 0;
    StreamTemp temp;
    temp.stream = stream;
    if(c.C % (16 / eb) != 0 || !aligned16(c.p_in) || !aligned16(c.p_wei))
    {
        if(stream_is_capturing(stream))
            return fail(CKB_ERR_UNSUPPORTED, "tensors that need a channel-padding copy cannot be captured into a graph");
        const int64_t per16 = 16 / eb;
        const int64_t c_pad = (c.C + per16 - 1) / per16 * per16;
        const int64_t pixels = static_cast<int64_t>(c.N) * c.Di * c.Hi * c.Wi;
        const int64_t wrows  = static_cast<int64_t>(c.K) * c.Z * c.Y * c.X;
        const size_t in_bytes  = (static_cast<size_t>(pixels) * c_pad * eb + 255) & ~size_t(255);
        const size_t wei_bytes = (static_cast<size_t>(wrows) * c_pad * eb + 255) & ~size_t(255);
        CKB_CUDA(cudaMallocAsync(&temp.ptr, in_bytes + wei_bytes, stream));
        void* wei_dst = static_cast<char*>(temp.ptr) + in_bytes;
        pre[n_pre++]  = Repack{c.p_in, temp.ptr, pixels, c.C, c.C, c_pad, eb};
        pre[n_pre++]  = Repack{c.p_wei, wei_dst, wrows, c.C, c.C, c_pad, eb};
        c.p_in        = temp.ptr;
        c.p_wei       = wei_dst;
        c.C           = static_cast<int>(c_pad);
    }
    const int64_t gm = static_cast<int64_t>(c.N) * c.Do * c.Ho * c.Wo;
    const int64_t taps = static_cast<int64_t>(c.Z) * c.Y * c.X;
    GemmPlanInput in;
    in.M        = gm;
    in.N        = c.K;
    in.num_kb   = static_cast<int>(taps * ((c.C + bk - 1) / bk));
    in.sm_count = dev->sm_count;
    in.b_min    = 64;
    in.force    = tile_config_of(c.tile_config);
    GemmPlan gp;
    if(!plan_gemm(in, &gp))
        return fail(CKB_ERR_UNSUPPORTED, "too many tiles");
    const int bn = gp.bn, cg = gp.cg;

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
    for(int which = 0; which < 2; ++which)
    {
        // Weights K[Z]YXC as (C, taps, K): a box never crosses a filter tap, channels beyond C read 0.
        cuuint64_t dims[3]    = {static_cast<cuuint64_t>(c.C), static_cast<cuuint64_t>(taps), static_cast<cuuint64_t>(c.K)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(c.C) * eb, static_cast<cuuint64_t>(taps) * c.C * eb};
        cuuint32_t box[3]     = {static_cast<cuuint32_t>(bk), 1,
                             static_cast<cuuint32_t>(which == 0 ? bn / cg : gp.b_split_rows)};
        rc = encode_tiled(which == 0 ? &p.tm_b : &p.tm_b_split, c.dtype, 3, c.p_wei, dims, strides, box,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, "weights");
        if(rc)
            return rc;
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
    p.plan          = gp.pp;
    p.M             = static_cast<int32_t>(gm);
    p.N             = c.K;
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
    note_plan("conv", bn, cg, gp.grid, p.plan, n_pre);
    return run_timed(fn, bn, cg, p, gp.grid, stream, n_rep, avg_ms, pre, n_pre);
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
