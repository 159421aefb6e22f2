/*
 * ckb200.h - C ABI of the B200 (sm_100a) dense-contraction library.
 *
 * Every entry point takes plain pointers and sizes.  The C++ compatibility
 * headers under include/ck/ (the Composable-Kernel-style device-operation
 * classes) and the Python test/bench harness both reach the CUDA kernels only
 * through the functions declared here.
 *
 * Conventions
 *   - return value 0 = success; non-zero = a CKB_ERR_* code, and
 *     ckb_last_error() returns a human-readable message for the calling thread.
 *   - all tensor pointers are DEVICE pointers unless a name says "host".
 *   - strides / leading dimensions are in ELEMENTS, as in the reference API
 *     (include/ck/tensor_operation/gpu/device/device_gemm.hpp:26-38).
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream).
 *   - there is no CPU fallback: every *_run call either launches sm_100a
 *     kernels or fails.
 */
#ifndef CKB200_H
#define CKB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CKB_ABI_VERSION 2

/* ---- error codes ------------------------------------------------------- */
enum {
    CKB_OK              = 0,
    CKB_ERR_UNSUPPORTED = 1, /* IsSupportedArgument would be false                */
    CKB_ERR_INVALID     = 2, /* malformed descriptor (null pointer, bad enum ...) */
    CKB_ERR_CUDA        = 3, /* a CUDA runtime / driver call failed               */
    CKB_ERR_DEVICE      = 4, /* kernel reported a bounded-wait time-out           */
    CKB_ERR_WORKSPACE   = 5, /* workspace missing or too small                    */
    CKB_ERR_LIMIT       = 6  /* size beyond a documented fixed maximum            */
};

/* ---- element types ------------------------------------------------------ */
enum {
    CKB_F16 = 0, /* IEEE binary16  (ck::half_t, utility/data_type.hpp:11)     */
    CKB_I8  = 1, /* int8_t, int32 accumulate                                   */
    CKB_BF16 = 2 /* bfloat16 (ck::bhalf_t, utility/data_type.hpp:10)           */
};

/* ---- matrix layouts (tensor_layout::gemm, device/tensor_layout.hpp:13-25).
 * All four A/B combinations of the reference's GEMM instances run (mk_nk, mk_kn, km_kn, km_nk,
 * library/src/tensor_operation_instance/gpu/gemm/): a K-contiguous operand (row-major A,
 * column-major B) is read as a K-major tile, the other kind as an MN-major tile. */
enum {
    CKB_ROW_MAJOR = 0,
    CKB_COL_MAJOR = 1
};

/*
 * ---- fused epilogues -----------------------------------------------------
 * `c` is the fp32 (or int32->fp32) accumulator value of one output element,
 * d0/d1 the matching elements of the auxiliary tensors, p[] = epi_params.
 * half(x) = round-to-nearest-even conversion to binary16; the output type of
 * the op is E (f16 unless stated).  Each line cites the reference functor.
 */
enum {
    /* e = E(c)                         element/unary_element_wise_operation.hpp:13-25   */
    CKB_EPI_PASSTHROUGH = 0,
    /* e = E(p0*c)                      unary_element_wise_operation.hpp:27-41            */
    CKB_EPI_SCALE = 1,
    /* e = E(c>0?c:0)                   unary_element_wise_operation.hpp:98-119           */
    CKB_EPI_RELU = 2,
    /* e = E(fast_gelu(c))              unary_element_wise_operation.hpp:121-135          */
    CKB_EPI_FASTGELU = 3,
    /* e = half(c) + d0  (binary16 add) binary_element_wise_operation.hpp:31-36           */
    CKB_EPI_ADD = 4,
    /* x = half(c)+d0; e = x>0?x:0      example/03_gemm_bias_relu/gemm_bias_relu_xdl_fp16.cpp:34-43 */
    CKB_EPI_ADD_RELU_F16 = 5,
    /* e = half(p0*c + p1*float(d0))    binary_element_wise_operation.hpp:107-112         */
    CKB_EPI_BILINEAR = 6,
    /* e = half(fast_gelu(c+float(d0)+float(d1)))   element_wise_operation.hpp:115-140    */
    CKB_EPI_ADD_ADD_FASTGELU = 7,
    /* e = half(max(c+float(d0),0)+float(d1))       element_wise_operation.hpp:71-79      */
    CKB_EPI_ADD_RELU_ADD = 8,
    /* y = clamp(p1*max(p0*c,0),-128,127); e = (int8)trunc(y)
     *      example/14_gemm_xdl_requant_relu_requant/gemm_xdl_requant_relu_requant_int8.cpp:21-39,
     *      store cast utility/data_type.hpp:934-938                                          */
    CKB_EPI_REQUANT_RELU_REQUANT = 9,
    /* e = sat_int8(rne(p1*max(rne(p0*c),0)))  (round-to-nearest-even after each scale,
     *      then saturate; no counterpart functor in the reference - this is the
     *      rounding the int8 benchmark configuration specifies)                            */
    CKB_EPI_REQUANT_RELU_REQUANT_RNE = 10,
    /* e = E(max(c+float(d0),0)) in fp32, one rounding
     *      binary_element_wise_operation.hpp:123-129 as used by
     *      reference_conv_fwd_bias_activation.hpp:114-118                                  */
    CKB_EPI_ADD_RELU = 11,
    /* fp32 AddHardswish then one rounding  binary_element_wise_operation.hpp:153-161      */
    CKB_EPI_ADD_HARDSWISH = 12,
    CKB_EPI_COUNT_ = 13
};

#define CKB_MAX_DS 2

/* ---- tile configuration (field `tile_config` of the descriptors) ------------------------
 * 0 = the library chooses the tile shape and the plan for the last, partial wave of tiles from
 * the problem size.  CKB_TILE_CONFIG(bn, cg, no_ksplit) fixes them, which is how an instance
 * factory (library/include/ck/library/tensor_operation_instance/gpu/gemm.hpp:233-378 hands out
 * one device operation per tile configuration) exposes several instances of one operation:
 *   bn        accumulator columns of a tile: 64, 128 or 256 (0 = library's choice)
 *   cg        CTAs per tile: 1 = 128 x bn tiles, 2 = a CTA pair on a 256 x 256 tile
 *             (tcgen05 cta_group::2; bn must be 256 or 0); 0 = library's choice
 *   no_ksplit 1 = never cut tiles along K (keeps a call free of library scratch memory)
 * A configuration that the problem cannot use (bn below the narrowest tile of the B layout) falls
 * back to the library's choice for that field. */
#define CKB_TILE_CONFIG(bn, cg, no_ksplit) ((bn) | ((cg) << 12) | ((no_ksplit) << 16))
/* The same with a K batch: kbatch = 2, 4 or 8 cuts the K loop of every tile into that many slices, each run by one
 * CTA of a thread-block cluster and summed through distributed shared memory in slice order (plain GEMM only; the
 * KBatch of DeviceGemmSplitK, device/device_gemm_splitk.hpp:23-42, with the result written once instead of added
 * atomically).  kbatch = 1 means no split; a count the problem cannot use (slices shorter than two k blocks of
 * 128 bytes, column parts narrower than 16) falls back to the library's choice. */
#define CKB_TILE_CONFIG_KBATCH(bn, cg, kbatch) ((bn) | ((cg) << 12) | ((kbatch) << 20))
/* The same with balanced K ranges: the k blocks of the tiles of the last one or two waves are laid end to end and
 * dealt out evenly over the CTAs (or CTA pairs), across tile boundaries; a CTA whose run ends inside a tile adds
 * the accumulators that the CTAs running the rest of that tile parked in the library's scratch, in k order
 * (plain, non-batched GEMMs: 16-bit GEMMs whose epilogue reads no D tensor on tiles of 128 or 256 columns, int8 and
 * D-reading epilogues on 256-wide tiles; elsewhere the field falls back to the library's choice).  The library also
 * takes this plan by itself where its cost estimate says so. */
#define CKB_TILE_CONFIG_BALANCED(bn, cg) ((bn) | ((cg) << 12) | (1 << 17))

/* ---- GEMM: E = epilogue(A*B, D0, D1) ------------------------------------- */
/* Replaces DeviceGemm::MakeArgumentPointer (device/device_gemm.hpp:26-38) and
 * DeviceGemmMultipleD::MakeArgumentPointer (device/device_gemm_multiple_d.hpp:36-50). */
typedef struct ckb_gemm_desc {
    int32_t ab_dtype;            /* CKB_F16 / CKB_BF16 / CKB_I8 (A and B share it)      */
    int32_t e_dtype;             /* CKB_F16 / CKB_BF16 for float inputs, CKB_I8 for int8 */
    int32_t a_layout;            /* A is M x K: row-major (lda >= K) or column-major (lda >= M) */
    int32_t b_layout;            /* B is K x N: column-major (ldb >= K) or row-major (ldb >= N) */
    int32_t e_layout;            /* E (and every D) is M x N; only CKB_ROW_MAJOR         */
    int32_t epilogue;            /* CKB_EPI_*                                            */
    int32_t n_ds;                /* number of D tensors the epilogue reads (0..2)        */
    int32_t tile_config;         /* 0 or CKB_TILE_CONFIG(...)                            */
    int64_t M, N, K;
    int64_t lda, ldb, lde;       /* leading dimensions in elements                       */
    int64_t ldd[CKB_MAX_DS];     /* row stride of each D; 0 = one row broadcast over M   */
    const void* p_a;
    const void* p_b;
    const void* p_ds[CKB_MAX_DS];
    void* p_e;
    float epi_params[4];
} ckb_gemm_desc;

/* 0 when the problem can run, CKB_ERR_UNSUPPORTED otherwise (never launches).
 * Replaces DeviceGemm_Xdl_CShuffle::IsSupportedArgument
 * (device/device_gemm_xdl_cshuffle.hpp:572-589). */
int ckb_gemm_supported(const ckb_gemm_desc* desc);

/* Launches on `stream`.  n_rep = 0: one asynchronous launch, *avg_ms = 0.
 * n_rep > 0: the reference's timing protocol - one warm-up launch, then n_rep
 * launches between two events, device-synchronised; *avg_ms = mean per launch
 * (include/ck/device_utility/kernel_launch.hpp:12-74 uses n_rep = 10).
 * Replaces DeviceGemm_Xdl_CShuffle::Invoker::Run (device_gemm_xdl_cshuffle.hpp:456-563).
 *
 * Scratch memory: a 16-bit GEMM whose last wave of tiles is partial may cut those tiles along K, which needs
 * device scratch.  The library allocates it once per stream on the first such call, sized for the largest plan it
 * can make (4 KiB + 128 KiB per SM: 19 MB on a B200), so it never grows, and keeps it until ckb_release_scratch.
 * Operands that TMA cannot read in place (A or B whose base or pitch is not a multiple of 16 bytes - the problems
 * the reference serves with its ScalarPerVector = 1 instances) are first copied into a temporary with a padded pitch,
 * allocated and freed on `stream` (cudaMallocAsync / cudaFreeAsync: no device synchronisation); the copy is part of
 * the call and of its timing.  Such a call cannot be captured into a graph.
 * CUDA graphs: with n_rep = 0 the GEMM, batched-GEMM and convolution launches can be captured into a graph (call
 * the library once on the device outside a capture first); a captured launch never uses the scratch, so a graph
 * may be replayed on any stream.  ckb_grouped_gemm_run copies a table from host memory at every launch; when it is
 * captured the library keeps that table alive for the graph's copy node (until ckb_release_scratch with all_streams
 * set).  ckb_grouped_gemm_run_noalloc refuses a capturing stream: its host table is shared by all calls. */
int ckb_gemm_run(const ckb_gemm_desc* desc, void* stream, int n_rep, float* avg_ms);

/* ---- batched GEMM: E[g] = epilogue(A[g]*B[g], D0[g], D1[g]), g = 0..batch-1 -------------- */
/* Replaces DeviceBatchedGemm::MakeArgumentPointer (device/device_batched_gemm.hpp:24-44: one
 * problem shape, pointers of batch 0, BatchStrideA/B/C in elements, Batch) and DeviceBatchedGemmXdl
 * (device/device_batched_gemm_xdl.hpp:119-153).  All batches run in one launch of the persistent
 * kernel; batch strides of A and B must be multiples of 16 bytes. */
typedef struct ckb_batched_gemm_desc {
    ckb_gemm_desc gemm;          /* shape, dtypes, layouts, epilogue; pointers of batch 0   */
    int64_t batch;               /* number of matrices, >= 1                               */
    int64_t batch_stride_a;      /* elements between A[g] and A[g+1]                       */
    int64_t batch_stride_b;
    int64_t batch_stride_e;
    int64_t batch_stride_d[2];   /* 0 = the same D for every batch                         */
} ckb_batched_gemm_desc;

int ckb_batched_gemm_supported(const ckb_batched_gemm_desc* desc);
/* n_rep / avg_ms as ckb_gemm_run. */
int ckb_batched_gemm_run(const ckb_batched_gemm_desc* desc, void* stream, int n_rep, float* avg_ms);

/* ---- grouped GEMM ---------------------------------------------------------- */
/* Replaces DeviceGroupedGemm::MakeArgumentPointer (device/device_grouped_gemm.hpp:33-41);
 * one ckb_gemm_desc per group (GemmDesc, device_grouped_gemm.hpp:11-17).  All groups must
 * share dtypes, layouts and the epilogue. */
typedef struct ckb_grouped_gemm_desc {
    int32_t group_count;
    int32_t tile_config;         /* 0 or CKB_TILE_CONFIG(...); the groups' own fields are ignored */
    const ckb_gemm_desc* groups; /* host array of group_count descriptors */
} ckb_grouped_gemm_desc;

int ckb_grouped_gemm_supported(const ckb_grouped_gemm_desc* desc);

/* Bytes of caller-allocated DEVICE workspace that ckb_grouped_gemm_run needs
 * (DeviceGroupedGemmXdl::GetWorkSpaceSize, device/device_grouped_gemm_xdl.hpp:816-819). */
int ckb_grouped_gemm_workspace_size(const ckb_grouped_gemm_desc* desc, size_t* bytes);

/* Builds the per-group table on the host, copies it into `workspace` on `stream`
 * and launches one persistent kernel over all groups
 * (DeviceGroupedGemmXdl::Invoker::Run, device/device_grouped_gemm_xdl.hpp:648-726). */
int ckb_grouped_gemm_run(const ckb_grouped_gemm_desc* desc, void* workspace,
                         size_t workspace_bytes, void* stream, int n_rep, float* avg_ms);

/* Grouped GEMM for callers that must not allocate.  It has no counterpart in the reference.
 *
 * Who needs it: host code that runs under a fixed device-memory plan - a serving loop whose
 * arena already owns all of HBM, a plug-in called from inside another framework's memory
 * planner, a latency-critical path where cudaMalloc's implicit device synchronisation is not
 * acceptable - cannot provide the workspace that ckb_grouped_gemm_run asks for at call time.
 * This variant keeps the per-group table (the kernel's only scratch memory) in a fixed array
 * that is part of the library image, so the call makes no cudaMalloc / cudaFree and uses no
 * allocating library routine; the caller still passes every input and output buffer.
 *
 * Limits and rules
 *   - at most CKB_NOALLOC_MAX_GROUPS groups; more is rejected with CKB_ERR_LIMIT and a message.
 *     The array costs CKB_NOALLOC_MAX_GROUPS * 640 bytes (160 KiB) of device memory on every
 *     GPU that loads the library, until the process exits.
 *   - the FIRST call on a device looks up the array's device address (cudaGetSymbolAddress with
 *     that device current) and sets the kernel's shared-memory attribute.  Make that first call
 *     during set-up, before any stream capture begins.
 *   - every call on a device shares the one array.  A call rewrites all entries it uses, so
 *     nothing has to be cleared between calls, but two calls whose kernels may overlap on the
 *     GPU (different streams, or host threads racing on one device) would overwrite each
 *     other's table: serialise them on one stream.
 *   - one asynchronous launch on `stream`; there is no timing mode (events would allocate).
 * Results are identical to ckb_grouped_gemm_run on the same descriptors. */
#define CKB_NOALLOC_MAX_GROUPS 256
int ckb_grouped_gemm_run_noalloc(const ckb_grouped_gemm_desc* desc, void* stream);

/* ---- 2-D convolution forward, NHWC / KYXC / NHWK ---------------------------- */
/* Replaces DeviceConvFwd::MakeArgumentPointer (device/device_conv_fwd.hpp:20-36) and
 * DeviceConvFwdBiasActivation::MakeArgumentPointer
 * (device/device_conv_fwd_bias_activation.hpp:21-38).
 * out[n,ho,wo,k] = epilogue( sum_{y,x,c} in[n, ho*sh + y*dh - ph, wo*sw + x*dw - pw, c]
 *                                        * wei[k,y,x,c],  bias[k] )
 * taps outside the image contribute zero.  All three tensors are packed.  A channel count whose pixel pitch is
 * not a multiple of 16 bytes (ConvolutionForwardSpecialization::OddC, e.g. C = 3) runs through a zero-padded
 * stream-ordered copy of input and weights, like the unaligned GEMM operands above. */
typedef struct ckb_conv2d_fwd_desc {
    int32_t dtype;               /* CKB_F16 / CKB_BF16 / CKB_I8 (in, wei, out, bias)     */
    int32_t epilogue;            /* PASSTHROUGH, RELU, ADD_RELU (bias), ADD_HARDSWISH (bias),
                                    ADD_RELU_ADD (bias + residual of the output's shape)   */
    int32_t N, K, C;
    int32_t Hi, Wi;
    int32_t Y, X;
    int32_t Ho, Wo;
    int32_t stride_h, stride_w;
    int32_t dilation_h, dilation_w;
    int32_t pad_h, pad_w;            /* left pads  */
    int32_t pad_h_right, pad_w_right;
    int32_t tile_config;         /* 0 or CKB_TILE_CONFIG(...)                            */
    const void* p_in;
    const void* p_wei;
    void* p_out;
    const void* p_bias;          /* length K, or NULL                                   */
    const void* p_resi;          /* N x Ho x Wo x K residual, or NULL                   */
    float epi_params[4];
} ckb_conv2d_fwd_desc;

int ckb_conv2d_fwd_supported(const ckb_conv2d_fwd_desc* desc);
int ckb_conv2d_fwd_run(const ckb_conv2d_fwd_desc* desc, void* stream, int n_rep, float* avg_ms);

/* ---- 3-D convolution forward, NDHWC / KZYXC / NDHWK -------------------------- */
/* The NumDimSpatial = 3 case of DeviceConvNDFwdXdl_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K
 * (device/device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp:76-1046; 3-D descriptor :372-548).  A 1-D problem
 * (NWC / KXC / NWK) is a 2-D one with Hi = Y = Ho = 1 and goes through ckb_conv2d_fwd_*.
 * out[n,do,ho,wo,k] = epilogue( sum_{z,y,x,c} in[n, do*sd + z*dd - pd, ho*sh + y*dh - ph, wo*sw + x*dw - pw, c]
 *                                            * wei[k,z,y,x,c],  bias[k] )
 * Limits of the 5-D im2col tensor map: pads <= 16, (filter - 1) * dilation <= 15 per dimension. */
typedef struct ckb_conv3d_fwd_desc {
    int32_t dtype;               /* CKB_F16 / CKB_BF16 / CKB_I8                          */
    int32_t epilogue;            /* as ckb_conv2d_fwd_desc                               */
    int32_t N, K, C;
    int32_t Di, Hi, Wi;
    int32_t Z, Y, X;
    int32_t Do, Ho, Wo;
    int32_t stride_d, stride_h, stride_w;
    int32_t dilation_d, dilation_h, dilation_w;
    int32_t pad_d, pad_h, pad_w;     /* left pads */
    int32_t pad_d_right, pad_h_right, pad_w_right;
    int32_t tile_config;         /* 0 or CKB_TILE_CONFIG(...)                            */
    const void* p_in;
    const void* p_wei;
    void* p_out;
    const void* p_bias;          /* length K, or NULL                                   */
    const void* p_resi;          /* N x Do x Ho x Wo x K residual, or NULL              */
    float epi_params[4];
} ckb_conv3d_fwd_desc;

int ckb_conv3d_fwd_supported(const ckb_conv3d_fwd_desc* desc);
int ckb_conv3d_fwd_run(const ckb_conv3d_fwd_desc* desc, void* stream, int n_rep, float* avg_ms);

/* ---- device memory helpers (DeviceMem, library/src/host_tensor/device_memory.cpp:7-28) */
int ckb_malloc(void** dev_ptr, size_t bytes);
int ckb_free(void* dev_ptr);
int ckb_memcpy_h2d(void* dev_dst, const void* host_src, size_t bytes);
int ckb_memcpy_d2h(void* host_dst, const void* dev_src, size_t bytes);
int ckb_memset(void* dev_ptr, int value, size_t bytes);
int ckb_device_synchronize(void);
/* Frees the scratch memory this library holds for `stream` on the current device (all streams of the device when
 * `all_streams` is non-zero; that also drops the host tables kept for captured grouped-GEMM launches, whose graphs
 * must not be replayed afterwards).  Synchronises the device first.  For callers that create and destroy streams. */
int ckb_release_scratch(void* stream, int all_streams);

/* ---- diagnostics ------------------------------------------------------------- */
/* Message of the last failing call made by this thread ("" if none). */
const char* ckb_last_error(void);
/* One line describing the launch plan of the calling thread's last *_run call: tile shape, CTAs per tile, grid,
 * column slices or K slices of the last wave, cluster K split, pitch-fixing copies and, for a GEMM, how many
 * clusters of 2 / 4 / 8 CTAs the device holds at once ("" before the first call). */
const char* ckb_last_plan(void);
/* Device name / SM count of the current device (device_utility/device_prop.hpp:12-52). */
int ckb_device_info(char* name, size_t name_bytes, int* sm_count, int* cc_major, int* cc_minor);
/* Number of kernel launches issued by this library in this process. */
uint64_t ckb_launch_count(void);
/* Reads (and clears) the device-side status word: 0 = no kernel reported a
 * bounded-wait time-out since the last call.  Synchronises the device. */
int ckb_device_status(uint32_t* word);
int ckb_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* CKB200_H */
