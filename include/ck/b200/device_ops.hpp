// Device operations of the dense-contraction path with the reference's names, template parameter
// lists and member functions, realised on B200 through the C ABI of ckb200.h.
//
// Every class template below accepts, positionally, exactly what example / instance code of the
// reference writes.  The AMD tuning parameters (everything from BlockSize on: tile sizes, XDL
// shapes, transfer cluster lengths, vector widths) are accepted, shown by GetTypeString() and
// otherwise ignored: the sm_100a kernels choose their own tiles.  Layout tags, data types and
// element-wise operators are honoured; combinations without a kernel make IsSupportedArgument()
// return false, and Invoker::Run() on such an argument throws like the reference does.
#pragma once
#include <array>
#include <cassert>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "ck/b200/core.hpp"
#include "ck/b200/element_ops.hpp"
#include "ckb200.h"

namespace ck {

// device/tensor_layout.hpp:13-129
namespace tensor_layout {
struct BaseTensorLayout
{
};
namespace gemm {
struct RowMajor : BaseTensorLayout
{
    static constexpr const char* name = "RowMajor";
};
struct ColumnMajor : BaseTensorLayout
{
    static constexpr const char* name = "ColumnMajor";
};
} // namespace gemm
namespace convolution {
#define CKB_CONV_TAG(T)                        \
    struct T : BaseTensorLayout                \
    {                                          \
        static constexpr const char* name = #T; \
    };
CKB_CONV_TAG(NWC) CKB_CONV_TAG(NHWC) CKB_CONV_TAG(NDHWC) CKB_CONV_TAG(NCW) CKB_CONV_TAG(NCHW) CKB_CONV_TAG(NCDHW)
CKB_CONV_TAG(KXC) CKB_CONV_TAG(KYXC) CKB_CONV_TAG(KZYXC) CKB_CONV_TAG(KCX) CKB_CONV_TAG(KCYX) CKB_CONV_TAG(KCZYX)
CKB_CONV_TAG(NWK) CKB_CONV_TAG(NHWK) CKB_CONV_TAG(NDHWK) CKB_CONV_TAG(NKW) CKB_CONV_TAG(NKHW) CKB_CONV_TAG(NKDHW)
#undef CKB_CONV_TAG
} // namespace convolution
} // namespace tensor_layout

enum struct LoopScheduler
{
    Default,
    Interwave
};
constexpr LoopScheduler make_default_loop_scheduler() { return LoopScheduler::Default; }

namespace tensor_operation {
namespace device {

// device/gemm_specialization.hpp:10-36.  Ragged M / N / K are always handled here (TMA zero fill,
// masked stores), so every value behaves like MNKPadding.
enum struct GemmSpecialization
{
    Default,
    MPadding,
    NPadding,
    KPadding,
    MNPadding,
    MKPadding,
    NKPadding,
    MNKPadding
};
inline std::string getGemmSpecializationString(const GemmSpecialization& s)
{
    static const char* names[] = {"Default",   "MPadding",  "NPadding",  "KPadding",
                                  "MNPadding", "MKPadding", "NKPadding", "MNKPadding"};
    return names[static_cast<int>(s)];
}

// device/convolution_forward_specialization.hpp:13-31
enum struct ConvolutionForwardSpecialization
{
    Default,
    Filter1x1Pad0,
    Filter1x1Stride1Pad0,
    OddC
};
inline std::string getConvForwardSpecializationString(const ConvolutionForwardSpecialization& s)
{
    static const char* names[] = {"Default", "Filter1x1Pad0", "Filter1x1Stride1Pad0", "OddC"};
    return names[static_cast<int>(s)];
}

// ---- polymorphic roots (device/device_base.hpp:14-57) ---------------------------------------------
struct BaseArgument
{
    BaseArgument()                    = default;
    BaseArgument(const BaseArgument&) = default;
    BaseArgument& operator=(const BaseArgument&) = default;
    virtual ~BaseArgument() {}
    void* p_workspace_ = nullptr;
};

struct BaseInvoker
{
    virtual float Run(const BaseArgument*, const StreamConfig& = StreamConfig{}) { return 0.f; }
    virtual ~BaseInvoker() {}
};

struct BaseOperator
{
    virtual bool IsSupportedArgument(const BaseArgument*) { return false; }
    virtual std::string GetTypeString() const { return ""; }
    // What runs behind the reference-style type string on this backend (not part of the reference interface).
    virtual std::string GetBackendString() const
    {
        if(tile_config_ == 0)
            return "B200 tcgen05 + TMA, tile shape chosen by the library";
        const int bn = tile_config_ & 0xFFF, cg = (tile_config_ >> 12) & 0xF;
        return "B200 tcgen05 + TMA, " + std::to_string(cg == 2 ? 256 : 128) + " x " + std::to_string(bn) + " tile" +
               (cg == 2 ? " per CTA pair" : "") + (((tile_config_ >> 16) & 1) ? ", no K split" : "");
    }
    // Tile configuration this instance asks the library for: 0 = the library's own choice, else a
    // CKB_TILE_CONFIG(bn, cg, no_ksplit) value (ckb200.h).  MakeArgumentPointer writes it into the argument; an
    // instance factory hands out one operation object per configuration.
    void SetTileConfig(int32_t tile_config) { tile_config_ = tile_config; }
    int32_t GetTileConfig() const { return tile_config_; }
    virtual size_t GetWorkSpaceSize(const BaseArgument*) const { return 0; }
    virtual void SetWorkSpacePointer(BaseArgument* p_arg, void* p_workspace) const
    {
        assert(p_arg);
        p_arg->p_workspace_ = p_workspace;
    }
    virtual ~BaseOperator() {}

    protected:
    int32_t tile_config_ = 0;
};

// ---- abstract operations -----------------------------------------------------------------------
// device_gemm.hpp:24-40
template <typename ALayout, typename BLayout, typename CLayout, typename ADataType, typename BDataType,
          typename CDataType, typename AElementwiseOperation, typename BElementwiseOperation,
          typename CElementwiseOperation>
struct DeviceGemm : public BaseOperator
{
    virtual std::unique_ptr<BaseArgument>
    MakeArgumentPointer(const void* p_a, const void* p_b, void* p_c, index_t M, index_t N, index_t K,
                        index_t StrideA, index_t StrideB, index_t StrideC, AElementwiseOperation a_element_op,
                        BElementwiseOperation b_element_op, CElementwiseOperation c_element_op) = 0;
    virtual std::unique_ptr<BaseInvoker> MakeInvokerPointer()                                  = 0;
};
template <typename... Ts>
using DeviceGemmPtr = std::unique_ptr<DeviceGemm<Ts...>>;

// device_gemm_multiple_d.hpp:32-53
template <typename ALayout, typename BLayout, typename DELayout, typename ADataType, typename BDataType,
          typename DsDataType, typename EDataType, typename AElementwiseOperation,
          typename BElementwiseOperation, typename CDEElementwiseOperation>
struct DeviceGemmMultipleD : public BaseOperator
{
    static constexpr index_t NumDTensor = DsDataType::Size();
    virtual std::unique_ptr<BaseArgument>
    MakeArgumentPointer(const void* p_a, const void* p_b, std::array<const void*, NumDTensor> p_ds, void* p_e,
                        index_t M, index_t N, index_t K, index_t StrideA, index_t StrideB,
                        std::array<index_t, NumDTensor> StrideDs, index_t StrideE,
                        AElementwiseOperation a_element_op, BElementwiseOperation b_element_op,
                        CDEElementwiseOperation cde_element_op) = 0;
    virtual std::unique_ptr<BaseInvoker> MakeInvokerPointer() = 0;
};
template <typename... Ts>
using DeviceGemmMultipleDPtr = std::unique_ptr<DeviceGemmMultipleD<Ts...>>;

// device_gemm_splitk.hpp:15-42
template <typename ALayout, typename BLayout, typename CLayout, typename ADataType, typename BDataType,
          typename CDataType, typename AElementwiseOperation, typename BElementwiseOperation,
          typename CElementwiseOperation>
struct DeviceGemmSplitK : public BaseOperator
{
    virtual std::unique_ptr<BaseArgument>
    MakeArgumentPointer(const void* p_a, const void* p_b, void* p_c, index_t M, index_t N, index_t K, index_t StrideA,
                        index_t StrideB, index_t StrideC, AElementwiseOperation a_element_op,
                        BElementwiseOperation b_element_op, CElementwiseOperation c_element_op, index_t KBatch) = 0;
    virtual std::unique_ptr<BaseInvoker> MakeInvokerPointer()                                                   = 0;
};
template <typename... Ts>
using DeviceGemmSplitKPtr = std::unique_ptr<DeviceGemmSplitK<Ts...>>;

// device_batched_gemm.hpp:15-52
template <typename ALayout, typename BLayout, typename CLayout, typename ADataType, typename BDataType,
          typename CDataType, typename AElementwiseOperation, typename BElementwiseOperation,
          typename CElementwiseOperation>
struct DeviceBatchedGemm : public BaseOperator
{
    virtual std::unique_ptr<BaseArgument>
    MakeArgumentPointer(const void* p_a, const void* p_b, void* p_c, index_t M, index_t N, index_t K, index_t StrideA,
                        index_t StrideB, index_t StrideC, index_t BatchStrideA, index_t BatchStrideB,
                        index_t BatchStrideC, index_t Batch, AElementwiseOperation a_element_op,
                        BElementwiseOperation b_element_op, CElementwiseOperation c_element_op) = 0;
    virtual std::unique_ptr<BaseInvoker> MakeInvokerPointer()                                    = 0;
};
template <typename... Ts>
using DeviceBatchedGemmPtr = std::unique_ptr<DeviceBatchedGemm<Ts...>>;

// device_grouped_gemm.hpp:11-44
struct GemmDesc
{
    index_t M_, N_, K_;
    index_t stride_A_, stride_B_, stride_C_;
    std::vector<index_t> stride_Ds_;
};
template <typename ALayout, typename BLayout, typename DELayout, typename ADataType, typename BDataType,
          typename DsDataType, typename EDataType, typename AElementwiseOperation,
          typename BElementwiseOperation, typename CElementwiseOperation>
struct DeviceGroupedGemm : public BaseOperator
{
    static constexpr index_t NumDTensor = DsDataType::Size();
    virtual std::unique_ptr<BaseArgument>
    MakeArgumentPointer(std::vector<const void*>& p_a, std::vector<const void*>& p_b,
                        std::vector<std::array<const void*, NumDTensor>>& p_ds, std::vector<void*>& p_e,
                        std::vector<GemmDesc>& gemm_desc, AElementwiseOperation a_element_op,
                        BElementwiseOperation b_element_op, CElementwiseOperation c_element_op) = 0;
    virtual std::unique_ptr<BaseInvoker> MakeInvokerPointer()                                   = 0;
};
template <typename... Ts>
using DeviceGroupedGemmPtr = std::unique_ptr<DeviceGroupedGemm<Ts...>>;

// device_conv_fwd.hpp:18-39
template <typename InElementwiseOperation, typename WeiElementwiseOperation, typename OutElementwiseOperation>
struct DeviceConvFwd : public BaseOperator
{
    virtual std::unique_ptr<BaseArgument>
    MakeArgumentPointer(const void* p_in, const void* p_wei, void* p_out, index_t N, index_t K, index_t C,
                        std::vector<index_t> input_spatial_lengths, std::vector<index_t> filter_spatial_lengths,
                        std::vector<index_t> output_spatial_lengths, std::vector<index_t> conv_filter_strides,
                        std::vector<index_t> conv_filter_dilations, std::vector<index_t> input_left_pads,
                        std::vector<index_t> input_right_pads, InElementwiseOperation in_element_op,
                        WeiElementwiseOperation wei_element_op, OutElementwiseOperation out_element_op) = 0;
    virtual std::unique_ptr<BaseInvoker> MakeInvokerPointer()                                          = 0;
};
template <typename I, typename W, typename O>
using DeviceConvFwdPtr = std::unique_ptr<DeviceConvFwd<I, W, O>>;

// device_conv_fwd_bias_activation.hpp:19-41
template <typename InElementwiseOperation, typename WeiElementwiseOperation, typename OutElementwiseOperation>
struct DeviceConvFwdBiasActivation : public BaseOperator
{
    virtual std::unique_ptr<BaseArgument>
    MakeArgumentPointer(const void* p_in, const void* p_wei, void* p_out, const void* p_bias, index_t N, index_t K,
                        index_t C, std::vector<index_t> input_spatial_lengths,
                        std::vector<index_t> filter_spatial_lengths, std::vector<index_t> output_spatial_lengths,
                        std::vector<index_t> conv_filter_strides, std::vector<index_t> conv_filter_dilations,
                        std::vector<index_t> input_left_pads, std::vector<index_t> input_right_pads,
                        InElementwiseOperation in_element_op, WeiElementwiseOperation wei_element_op,
                        OutElementwiseOperation out_element_op) = 0;
    virtual std::unique_ptr<BaseInvoker> MakeInvokerPointer()  = 0;
};
template <typename I, typename W, typename O>
using DeviceConvFwdBiasActivationPtr = std::unique_ptr<DeviceConvFwdBiasActivation<I, W, O>>;

// device_conv_fwd_bias_activation_add.hpp:15-45
template <typename InElementwiseOperation, typename WeiElementwiseOperation, typename OutElementwiseOperation>
struct DeviceConvFwdBiasActivationAdd : public BaseOperator
{
    virtual std::unique_ptr<BaseArgument>
    MakeArgumentPointer(const void* p_in, const void* p_wei, void* p_out, const void* p_bias, const void* p_resi,
                        index_t N, index_t K, index_t C, std::vector<index_t> input_spatial_lengths,
                        std::vector<index_t> filter_spatial_lengths, std::vector<index_t> output_spatial_lengths,
                        std::vector<index_t> conv_filter_strides, std::vector<index_t> conv_filter_dilations,
                        std::vector<index_t> input_left_pads, std::vector<index_t> input_right_pads,
                        InElementwiseOperation in_element_op, WeiElementwiseOperation wei_element_op,
                        OutElementwiseOperation out_element_op) = 0;
    virtual std::unique_ptr<BaseInvoker> MakeInvokerPointer()  = 0;
};
template <typename I, typename W, typename O>
using DeviceConvFwdBiasActivationAddPtr = std::unique_ptr<DeviceConvFwdBiasActivationAdd<I, W, O>>;

} // namespace device
} // namespace tensor_operation

// ---- shared machinery behind the concrete operations ------------------------------------------------
namespace b200 {

namespace dev = ck::tensor_operation::device;

template <typename Layout>
struct layout_of;
template <>
struct layout_of<tensor_layout::gemm::RowMajor>
{
    static constexpr int value = CKB_ROW_MAJOR;
};
template <>
struct layout_of<tensor_layout::gemm::ColumnMajor>
{
    static constexpr int value = CKB_COL_MAJOR;
};

inline constexpr int kTimedRepeats = 10; // device_utility/kernel_launch.hpp:32

[[noreturn]] inline void throw_invalid_setting()
{
    // device_gemm_xdl_cshuffle.hpp:475-481
    throw std::runtime_error(std::string("wrong! GridwiseGemm has invalid setting: ") + ckb_last_error());
}
inline void check_runtime(int rc)
{
    // device_utility/hip_check_error.hpp:8-17: runtime failures are std::runtime_error
    if(rc != CKB_OK)
        throw std::runtime_error(std::string("ckb200: ") + ckb_last_error());
}

template <typename Derived, typename Base>
const Derived& argument_cast(const Base* p)
{
    const Derived* d = dynamic_cast<const Derived*>(p);
    if(!d)
        throw std::runtime_error("wrong! argument object belongs to a different device operation");
    return *d;
}

// What a GemmSpecialization means for IsSupportedArgument.  The reference pads the dimensions a specialisation
// names up to the block tile (device_gemm_xdl_cshuffle.hpp:84-346) and then demands M % MPerBlock == 0 &&
// N % NPerBlock == 0 && K % KPerBlock == 0 of the padded problem (gridwise_gemm_xdl_cshuffle_v1.hpp:222-226): an
// instance therefore rejects a ragged dimension its specialisation does not pad.  The kernel behind these headers
// handles ragged edges by itself (TMA zero fill, predicated stores), so this rule is kept only so that an instance
// answers as the reference's instance would; define CK_B200_RELAXED_GEMM_SPECIALIZATION to accept every shape.
constexpr bool pads_m(dev::GemmSpecialization s)
{
    return s == dev::GemmSpecialization::MPadding || s == dev::GemmSpecialization::MNPadding ||
           s == dev::GemmSpecialization::MKPadding || s == dev::GemmSpecialization::MNKPadding;
}
constexpr bool pads_n(dev::GemmSpecialization s)
{
    return s == dev::GemmSpecialization::NPadding || s == dev::GemmSpecialization::MNPadding ||
           s == dev::GemmSpecialization::NKPadding || s == dev::GemmSpecialization::MNKPadding;
}
constexpr bool pads_k(dev::GemmSpecialization s)
{
    return s == dev::GemmSpecialization::KPadding || s == dev::GemmSpecialization::MKPadding ||
           s == dev::GemmSpecialization::NKPadding || s == dev::GemmSpecialization::MNKPadding;
}
template <dev::GemmSpecialization Spec, index_t MPerBlock, index_t NPerBlock, index_t KPerBlock>
inline bool specialization_accepts(index_t M, index_t N, index_t K)
{
#ifdef CK_B200_RELAXED_GEMM_SPECIALIZATION
    (void)M, (void)N, (void)K;
    return true;
#else
    return (pads_m(Spec) || M % MPerBlock == 0) && (pads_n(Spec) || N % NPerBlock == 0) &&
           (pads_k(Spec) || K % KPerBlock == 0);
#endif
}

// -------- GEMM (single C op or multiple D) --------
struct GemmArgument : dev::BaseArgument
{
    ckb_gemm_desc desc{};
    bool host_ok = true; // A/B ops are PassThrough and the epilogue functor has a device twin
    void set_tile_config(int32_t tc) { desc.tile_config = tc; }
};

struct GemmInvoker : dev::BaseInvoker
{
    float Run(const GemmArgument& arg, const StreamConfig& stream_config = StreamConfig{})
    {
        if(!arg.host_ok || ckb_gemm_supported(&arg.desc) != CKB_OK)
            throw_invalid_setting();
        float ms = 0.f;
        check_runtime(ckb_gemm_run(&arg.desc, stream_config.stream_id_,
                                   stream_config.time_kernel_ ? kTimedRepeats : 0, &ms));
        return ms;
    }
    float Run(const dev::BaseArgument* p_arg, const StreamConfig& stream_config = StreamConfig{}) override
    {
        return Run(argument_cast<GemmArgument>(p_arg), stream_config);
    }
};

// -------- batched GEMM --------
struct BatchedGemmArgument : dev::BaseArgument
{
    ckb_batched_gemm_desc desc{};
    bool host_ok = true;
    void set_tile_config(int32_t tc) { desc.gemm.tile_config = tc; }
};

struct BatchedGemmInvoker : dev::BaseInvoker
{
    float Run(const BatchedGemmArgument& arg, const StreamConfig& stream_config = StreamConfig{})
    {
        if(!arg.host_ok || ckb_batched_gemm_supported(&arg.desc) != CKB_OK)
            throw_invalid_setting();
        float ms = 0.f;
        check_runtime(ckb_batched_gemm_run(&arg.desc, stream_config.stream_id_,
                                           stream_config.time_kernel_ ? kTimedRepeats : 0, &ms));
        return ms;
    }
    float Run(const dev::BaseArgument* p_arg, const StreamConfig& stream_config = StreamConfig{}) override
    {
        return Run(argument_cast<BatchedGemmArgument>(p_arg), stream_config);
    }
};

template <typename ALayout, typename BLayout, typename ELayout, typename ADataType, typename BDataType,
          typename EDataType, typename AOp, typename BOp, typename EpiOp, typename Ctx, std::size_t NumD>
GemmArgument make_gemm_argument(const void* p_a, const void* p_b, const std::array<const void*, NumD>& p_ds,
                                void* p_e, index_t M, index_t N, index_t K, index_t StrideA, index_t StrideB,
                                const std::array<index_t, NumD>& StrideDs, index_t StrideE, const EpiOp& op)
{
    static_assert(NumD <= CKB_MAX_DS, "at most two D tensors");
    GemmArgument a;
    ckb_gemm_desc& d = a.desc;
    d.ab_dtype       = dtype_of<ADataType>::value;
    d.e_dtype        = dtype_of<EDataType>::value;
    d.a_layout       = layout_of<ALayout>::value;
    d.b_layout       = layout_of<BLayout>::value;
    d.e_layout       = layout_of<ELayout>::value;
    d.epilogue       = EpilogueTraits<EpiOp, Ctx>::kind;
    EpilogueTraits<EpiOp, Ctx>::params(op, d.epi_params);
    d.n_ds = static_cast<int32_t>(NumD);
    d.M    = M;
    d.N    = N;
    d.K    = K;
    d.lda  = StrideA;
    d.ldb  = StrideB;
    d.lde  = StrideE;
    for(std::size_t i = 0; i < NumD; ++i)
    {
        d.p_ds[i] = p_ds[i];
        d.ldd[i]  = StrideDs[i];
    }
    d.p_a     = p_a;
    d.p_b     = p_b;
    d.p_e     = p_e;
    a.host_ok = is_passthrough<AOp>::value && is_passthrough<BOp>::value && std::is_same<ADataType, BDataType>::value &&
                EpilogueTraits<EpiOp, Ctx>::kind >= 0;
    return a;
}

inline bool gemm_supported(const GemmArgument& a) { return a.host_ok && ckb_gemm_supported(&a.desc) == CKB_OK; }

// -------- grouped GEMM --------
struct GroupedGemmArgument : dev::BaseArgument
{
    std::vector<ckb_gemm_desc> groups;
    bool host_ok        = true;
    int32_t tile_config = 0;
    void set_tile_config(int32_t tc) { tile_config = tc; }
    ckb_grouped_gemm_desc view() const
    {
        ckb_grouped_gemm_desc g{};
        g.tile_config = tile_config;
        g.group_count = static_cast<int32_t>(groups.size());
        g.groups      = groups.data();
        return g;
    }
    size_t workspace_bytes() const
    {
        const ckb_grouped_gemm_desc g = view();
        size_t n                      = 0;
        ckb_grouped_gemm_workspace_size(&g, &n);
        return n;
    }
};

struct GroupedGemmInvoker : dev::BaseInvoker
{
    float Run(const GroupedGemmArgument& arg, const StreamConfig& stream_config = StreamConfig{})
    {
        const ckb_grouped_gemm_desc g = arg.view();
        if(!arg.host_ok || ckb_grouped_gemm_supported(&g) != CKB_OK)
            throw_invalid_setting();
        float ms = 0.f;
        check_runtime(ckb_grouped_gemm_run(&g, arg.p_workspace_, arg.p_workspace_ ? arg.workspace_bytes() : 0,
                                           stream_config.stream_id_,
                                           stream_config.time_kernel_ ? kTimedRepeats : 0, &ms));
        return ms;
    }
    float Run(const dev::BaseArgument* p_arg, const StreamConfig& stream_config = StreamConfig{}) override
    {
        return Run(argument_cast<GroupedGemmArgument>(p_arg), stream_config);
    }
};

// -------- convolution forward (1-D, 2-D, 3-D) --------
struct ConvArgument : dev::BaseArgument
{
    ckb_conv2d_fwd_desc desc{};  // 1-D (as a 2-D problem of height 1) and 2-D
    ckb_conv3d_fwd_desc desc3{}; // 3-D
    bool is_3d   = false;
    bool host_ok = true;
    void set_tile_config(int32_t tc) { desc.tile_config = desc3.tile_config = tc; }
};

inline bool conv_supported(const ConvArgument& a);

struct ConvInvoker : dev::BaseInvoker
{
    float Run(const ConvArgument& arg, const StreamConfig& stream_config = StreamConfig{})
    {
        if(!conv_supported(arg))
            throw_invalid_setting();
        float ms      = 0.f;
        const int rep = stream_config.time_kernel_ ? kTimedRepeats : 0;
        check_runtime(arg.is_3d ? ckb_conv3d_fwd_run(&arg.desc3, stream_config.stream_id_, rep, &ms)
                                : ckb_conv2d_fwd_run(&arg.desc, stream_config.stream_id_, rep, &ms));
        return ms;
    }
    float Run(const dev::BaseArgument* p_arg, const StreamConfig& stream_config = StreamConfig{}) override
    {
        return Run(argument_cast<ConvArgument>(p_arg), stream_config);
    }
};

// The spatial vectors decide the dimensionality (the reference's NumDimSpatial); a 1-D problem is passed on as a
// 2-D one of height 1.
template <typename InDataType, typename InOp, typename WeiOp, typename OutOp>
ConvArgument make_conv_argument(const void* p_in, const void* p_wei, void* p_out, const void* p_bias,
                                const void* p_resi, index_t N, index_t K, index_t C,
                                const std::vector<index_t>& in_sp, const std::vector<index_t>& filt_sp,
                                const std::vector<index_t>& out_sp, const std::vector<index_t>& strides,
                                const std::vector<index_t>& dilations, const std::vector<index_t>& lpads,
                                const std::vector<index_t>& rpads, const OutOp& op)
{
    ConvArgument a;
    const std::size_t nd = in_sp.size();
    const bool same_nd   = filt_sp.size() == nd && out_sp.size() == nd && strides.size() == nd &&
                         dilations.size() == nd && lpads.size() == nd && rpads.size() == nd;
    a.host_ok = same_nd && nd >= 1 && nd <= 3 && is_passthrough<InOp>::value && is_passthrough<WeiOp>::value &&
                EpilogueTraits<OutOp, ctx_conv>::kind >= 0;
    a.is_3d = nd == 3;
    auto fill_common = [&](auto& d) {
        d.dtype    = dtype_of<InDataType>::value;
        d.epilogue = EpilogueTraits<OutOp, ctx_conv>::kind;
        EpilogueTraits<OutOp, ctx_conv>::params(op, d.epi_params);
        d.N      = N;
        d.K      = K;
        d.C      = C;
        d.p_in   = p_in;
        d.p_wei  = p_wei;
        d.p_out  = p_out;
        d.p_bias = p_bias;
        d.p_resi = p_resi;
    };
    fill_common(a.desc);
    fill_common(a.desc3);
    if(!same_nd)
        return a;
    if(nd == 3)
    {
        ckb_conv3d_fwd_desc& d = a.desc3;
        d.Di = in_sp[0], d.Hi = in_sp[1], d.Wi = in_sp[2];
        d.Z = filt_sp[0], d.Y = filt_sp[1], d.X = filt_sp[2];
        d.Do = out_sp[0], d.Ho = out_sp[1], d.Wo = out_sp[2];
        d.stride_d = strides[0], d.stride_h = strides[1], d.stride_w = strides[2];
        d.dilation_d = dilations[0], d.dilation_h = dilations[1], d.dilation_w = dilations[2];
        d.pad_d = lpads[0], d.pad_h = lpads[1], d.pad_w = lpads[2];
        d.pad_d_right = rpads[0], d.pad_h_right = rpads[1], d.pad_w_right = rpads[2];
    }
    else if(nd == 2 || nd == 1)
    {
        ckb_conv2d_fwd_desc& d = a.desc;
        const std::size_t w    = nd - 1; // index of the innermost (width) dimension
        d.Hi = nd == 2 ? in_sp[0] : 1, d.Wi = in_sp[w];
        d.Y = nd == 2 ? filt_sp[0] : 1, d.X = filt_sp[w];
        d.Ho = nd == 2 ? out_sp[0] : 1, d.Wo = out_sp[w];
        d.stride_h = nd == 2 ? strides[0] : 1, d.stride_w = strides[w];
        d.dilation_h = nd == 2 ? dilations[0] : 1, d.dilation_w = dilations[w];
        d.pad_h = nd == 2 ? lpads[0] : 0, d.pad_w = lpads[w];
        d.pad_h_right = nd == 2 ? rpads[0] : 0, d.pad_w_right = rpads[w];
    }
    return a;
}

// device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp:921-933.  The kernel behind these headers has no such limit (a channel
// count that TMA cannot read in place goes through a padded copy); the rule is kept so that an instance answers as
// the reference's instance would, and CK_B200_RELAXED_GEMM_SPECIALIZATION lifts it together with the GEMM rule.
inline bool vector_widths_accept(index_t C, index_t K, index_t a_vec, index_t b_vec, index_t c_vec)
{
#ifdef CK_B200_RELAXED_GEMM_SPECIALIZATION
    (void)C, (void)K, (void)a_vec, (void)b_vec, (void)c_vec;
    return true;
#else
    return a_vec > 0 && b_vec > 0 && c_vec > 0 && C % a_vec == 0 && C % b_vec == 0 && K % c_vec == 0;
#endif
}

// device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp:894-919: an instance built for a 1x1 filter specialisation rejects every
// other geometry (Default and OddC accept all).
template <dev::ConvolutionForwardSpecialization Spec>
inline bool conv_specialization_accepts(const std::vector<index_t>& filt_sp, const std::vector<index_t>& strides,
                                        const std::vector<index_t>& lpads, const std::vector<index_t>& rpads)
{
    constexpr bool one_by_one = Spec == dev::ConvolutionForwardSpecialization::Filter1x1Pad0 ||
                                Spec == dev::ConvolutionForwardSpecialization::Filter1x1Stride1Pad0;
    if(!one_by_one)
        return true;
    if(strides.size() != filt_sp.size() || lpads.size() != filt_sp.size() || rpads.size() != filt_sp.size())
        return false;
    for(std::size_t i = 0; i < filt_sp.size(); ++i)
    {
        if(!(filt_sp[i] == 1 && lpads[i] == 0 && rpads[i] == 0))
            return false;
        if(Spec == dev::ConvolutionForwardSpecialization::Filter1x1Stride1Pad0 && strides[i] != 1)
            return false;
    }
    return true;
}

inline bool conv_supported(const ConvArgument& a)
{
    return a.host_ok &&
           (a.is_3d ? ckb_conv3d_fwd_supported(&a.desc3) : ckb_conv2d_fwd_supported(&a.desc)) == CKB_OK;
}

} // namespace b200

// ---- concrete operations (reference names and template parameter lists) ---------------------------
namespace tensor_operation {
namespace device {

// The seven block-transfer parameters the reference repeats for A and for B.
#define CKB_XFER(P)                                                                                         \
    typename P##ThreadClusterLengths, typename P##ThreadClusterArrangeOrder, typename P##SrcAccessOrder,    \
        index_t P##SrcVectorDim, index_t P##SrcScalarPerVector, index_t P##DstScalarPerVector, index_t P##LdsExtra

// device_gemm_xdl_cshuffle.hpp:26-67
template <typename ALayout, typename BLayout, typename CLayout, typename ADataType, typename BDataType,
          typename CDataType, typename GemmAccDataType, typename CShuffleDataType, typename AElementwiseOperation,
          typename BElementwiseOperation, typename CElementwiseOperation, GemmSpecialization GemmSpec,
          index_t NumGemmKPrefetchStage, index_t BlockSize, index_t MPerBlock, index_t NPerBlock, index_t KPerBlock,
          index_t AK1, index_t BK1, index_t MPerXDL, index_t NPerXDL, index_t MXdlPerWave, index_t NXdlPerWave,
          CKB_XFER(ABlockTransfer), CKB_XFER(BBlockTransfer), index_t CShuffleMXdlPerWavePerShuffle,
          index_t CShuffleNXdlPerWavePerShuffle, typename CShuffleBlockTransferClusterLengths,
          index_t CShuffleBlockTransferScalarPerVector, LoopScheduler LoopSched = make_default_loop_scheduler()>
struct DeviceGemm_Xdl_CShuffle : public DeviceGemm<ALayout, BLayout, CLayout, ADataType, BDataType, CDataType,
                                                   AElementwiseOperation, BElementwiseOperation, CElementwiseOperation>
{
    using Argument = b200::GemmArgument;
    using Invoker  = b200::GemmInvoker;

    static auto MakeArgument(const ADataType* p_a, const BDataType* p_b, CDataType* p_c, index_t M, index_t N,
                             index_t K, index_t StrideA, index_t StrideB, index_t StrideC, AElementwiseOperation,
                             BElementwiseOperation, CElementwiseOperation c_element_op)
    {
        auto arg = b200::make_gemm_argument<ALayout, BLayout, CLayout, ADataType, BDataType, CDataType,
                                            AElementwiseOperation, BElementwiseOperation, CElementwiseOperation,
                                            b200::ctx_gemm_c, 0>(p_a, p_b, {}, p_c, M, N, K, StrideA, StrideB, {},
                                                                 StrideC, c_element_op);
        arg.host_ok = arg.host_ok && b200::specialization_accepts<GemmSpec, MPerBlock, NPerBlock, KPerBlock>(M, N, K);
        return arg;
    }
    static auto MakeInvoker() { return Invoker{}; }
    static bool IsSupportedArgument(const Argument& arg) { return b200::gemm_supported(arg); }
    bool IsSupportedArgument(const BaseArgument* p_arg) override
    {
        return IsSupportedArgument(b200::argument_cast<Argument>(p_arg));
    }
    std::unique_ptr<BaseArgument> MakeArgumentPointer(const void* p_a, const void* p_b, void* p_c, index_t M, index_t N,
                                                      index_t K, index_t StrideA, index_t StrideB, index_t StrideC,
                                                      AElementwiseOperation a_op, BElementwiseOperation b_op,
                                                      CElementwiseOperation c_op) override
    {
        auto arg = std::make_unique<Argument>(MakeArgument(static_cast<const ADataType*>(p_a),
                                                       static_cast<const BDataType*>(p_b), static_cast<CDataType*>(p_c),
                                                       M, N, K, StrideA, StrideB, StrideC, a_op, b_op, c_op));
        arg->set_tile_config(this->tile_config_);
        return arg;
    }
    std::unique_ptr<BaseInvoker> MakeInvokerPointer() override { return std::make_unique<Invoker>(); }
    std::string GetTypeString() const override
    {
        std::ostringstream s; // device_gemm_xdl_cshuffle.hpp:655-672
        s << "DeviceGemm_Xdl_CShuffle<" << BlockSize << ", " << MPerBlock << ", " << NPerBlock << ", " << KPerBlock
          << ", " << AK1 << ", " << BK1 << ">";
        return s.str();
    }
};

// device_gemm_xdl.hpp:22-59 (the instance example/01_gemm/gemm_xdl_fp16.cpp activates)
template <typename ADataType, typename BDataType, typename CDataType, typename AccDataType, typename ALayout,
          typename BLayout, typename CLayout, typename AElementwiseOperation, typename BElementwiseOperation,
          typename CElementwiseOperation, GemmSpecialization GemmSpec, index_t BlockSize, index_t MPerBlock,
          index_t NPerBlock, index_t K0PerBlock, index_t K1, index_t MPerXDL, index_t NPerXDL, index_t MXdlPerWave,
          index_t NXdlPerWave, CKB_XFER(ABlockTransfer), CKB_XFER(BBlockTransfer), index_t CThreadTransferSrcDstVectorDim,
          index_t CThreadTransferDstScalarPerVector, index_t NumPrefetch = 1>
struct DeviceGemmXdl : public DeviceGemm<ALayout, BLayout, CLayout, ADataType, BDataType, CDataType,
                                         AElementwiseOperation, BElementwiseOperation, CElementwiseOperation>
{
    using Argument = b200::GemmArgument;
    using Invoker  = b200::GemmInvoker;

    static auto MakeArgument(const ADataType* p_a, const BDataType* p_b, CDataType* p_c, index_t M, index_t N,
                             index_t K, index_t StrideA, index_t StrideB, index_t StrideC, AElementwiseOperation,
                             BElementwiseOperation, CElementwiseOperation c_element_op)
    {
        auto arg = b200::make_gemm_argument<ALayout, BLayout, CLayout, ADataType, BDataType, CDataType,
                                            AElementwiseOperation, BElementwiseOperation, CElementwiseOperation,
                                            b200::ctx_gemm_c, 0>(p_a, p_b, {}, p_c, M, N, K, StrideA, StrideB, {},
                                                                 StrideC, c_element_op);
        arg.host_ok = arg.host_ok && b200::specialization_accepts<GemmSpec, MPerBlock, NPerBlock, K0PerBlock * K1>(M, N, K);
        return arg;
    }
    static auto MakeInvoker() { return Invoker{}; }
    static bool IsSupportedArgument(const Argument& arg) { return b200::gemm_supported(arg); }
    bool IsSupportedArgument(const BaseArgument* p_arg) override
    {
        return IsSupportedArgument(b200::argument_cast<Argument>(p_arg));
    }
    std::unique_ptr<BaseArgument> MakeArgumentPointer(const void* p_a, const void* p_b, void* p_c, index_t M, index_t N,
                                                      index_t K, index_t StrideA, index_t StrideB, index_t StrideC,
                                                      AElementwiseOperation a_op, BElementwiseOperation b_op,
                                                      CElementwiseOperation c_op) override
    {
        auto arg = std::make_unique<Argument>(MakeArgument(static_cast<const ADataType*>(p_a),
                                                       static_cast<const BDataType*>(p_b), static_cast<CDataType*>(p_c),
                                                       M, N, K, StrideA, StrideB, StrideC, a_op, b_op, c_op));
        arg->set_tile_config(this->tile_config_);
        return arg;
    }
    std::unique_ptr<BaseInvoker> MakeInvokerPointer() override { return std::make_unique<Invoker>(); }
    std::string GetTypeString() const override
    {
        std::ostringstream s; // device_gemm_xdl.hpp:522-541
        s << "DeviceGemmXdl<" << BlockSize << ", " << MPerBlock << ", " << NPerBlock << ", " << K0PerBlock << ", " << K1
          << ", " << MPerXDL << ", " << NPerXDL << ", " << MXdlPerWave << ", " << NXdlPerWave
          << ">";
        return s.str();
    }
};

// device_gemm_xdl_splitk_c_shuffle.hpp:23-60.  KBatch is the reference's tuning knob for how many ways the K loop
// is cut (partial sums added atomically into a zero-initialised C); here KBatch = 2, 4 or 8 becomes the slice count
// of the cluster K split and the result is written once, in a fixed summation order.
template <typename ADataType, typename BDataType, typename CDataType, typename AccDataType, typename ALayout,
          typename BLayout, typename CLayout, typename AElementwiseOperation, typename BElementwiseOperation,
          typename CElementwiseOperation, GemmSpecialization GemmSpec, index_t BlockSize, index_t MPerBlock,
          index_t NPerBlock, index_t K0PerBlock, index_t K1, index_t MPerXDL, index_t NPerXDL, index_t MXdlPerWave,
          index_t NXdlPerWave, CKB_XFER(ABlockTransfer), CKB_XFER(BBlockTransfer), index_t CShuffleMRepeatPerShuffle,
          index_t CShuffleNRepeatPerShuffle, typename CBlockTransferClusterLengths,
          index_t CBlockTransferScalarPerVector>
struct DeviceGemmXdlSplitKCShuffle : public DeviceGemmSplitK<ALayout, BLayout, CLayout, ADataType, BDataType, CDataType,
                                                             AElementwiseOperation, BElementwiseOperation,
                                                             CElementwiseOperation>
{
    using Argument = b200::GemmArgument;
    using Invoker  = b200::GemmInvoker;

    static auto MakeArgument(const ADataType* p_a, const BDataType* p_b, CDataType* p_c, index_t M, index_t N,
                             index_t K, index_t StrideA, index_t StrideB, index_t StrideC, AElementwiseOperation,
                             BElementwiseOperation, CElementwiseOperation c_element_op, index_t KBatch)
    {
        auto arg = b200::make_gemm_argument<ALayout, BLayout, CLayout, ADataType, BDataType, CDataType,
                                            AElementwiseOperation, BElementwiseOperation, CElementwiseOperation,
                                            b200::ctx_gemm_c, 0>(p_a, p_b, {}, p_c, M, N, K, StrideA, StrideB, {},
                                                                 StrideC, c_element_op);
        // device_gemm_xdl_splitk_c_shuffle.hpp pads K to a multiple of KBatch * K0PerBlock * K1 whatever the
        // specialisation; M and N follow the usual rule
        arg.host_ok = arg.host_ok && KBatch >= 1 && b200::specialization_accepts<GemmSpec, MPerBlock, NPerBlock, 1>(M, N, K);
        // KBatch = 1: no split; 2, 4 or 8: that many K slices on a thread-block cluster, summed in slice order and
        // written once (the reference adds the slices atomically into a zero-initialised C); any other count leaves
        // the choice to the library
        if(KBatch == 1 || KBatch == 2 || KBatch == 4 || KBatch == 8)
            arg.desc.tile_config = CKB_TILE_CONFIG_KBATCH(0, 0, static_cast<int32_t>(KBatch));
        return arg;
    }
    static auto MakeInvoker() { return Invoker{}; }
    static bool IsSupportedArgument(const Argument& arg) { return b200::gemm_supported(arg); }
    bool IsSupportedArgument(const BaseArgument* p_arg) override
    {
        return IsSupportedArgument(b200::argument_cast<Argument>(p_arg));
    }
    std::unique_ptr<BaseArgument> MakeArgumentPointer(const void* p_a, const void* p_b, void* p_c, index_t M, index_t N,
                                                      index_t K, index_t StrideA, index_t StrideB, index_t StrideC,
                                                      AElementwiseOperation a_op, BElementwiseOperation b_op,
                                                      CElementwiseOperation c_op, index_t KBatch) override
    {
        auto arg = std::make_unique<Argument>(MakeArgument(static_cast<const ADataType*>(p_a),
                                                       static_cast<const BDataType*>(p_b), static_cast<CDataType*>(p_c),
                                                       M, N, K, StrideA, StrideB, StrideC, a_op, b_op, c_op, KBatch));
        if(this->tile_config_ != 0)
            arg->set_tile_config(this->tile_config_);
        return arg;
    }
    std::unique_ptr<BaseInvoker> MakeInvokerPointer() override { return std::make_unique<Invoker>(); }
    std::string GetTypeString() const override
    {
        std::ostringstream s;
        s << "DeviceGemmXdlSplitKCShuffle<" << BlockSize << ", " << MPerBlock << ", " << NPerBlock << ", " << K0PerBlock
          << ">";
        return s.str();
    }
};

// device_batched_gemm_xdl.hpp:119-153
template <typename ADataType, typename BDataType, typename CDataType, typename AccDataType, typename ALayout,
          typename BLayout, typename CLayout, typename AElementwiseOperation, typename BElementwiseOperation,
          typename CElementwiseOperation, index_t BlockSize, index_t MPerBlock, index_t NPerBlock, index_t K0PerBlock,
          index_t K1, index_t MPerXDL, index_t NPerXDL, index_t MXdlPerWave, index_t NXdlPerWave,
          CKB_XFER(ABlockTransfer), CKB_XFER(BBlockTransfer), index_t CThreadTransferSrcDstVectorDim,
          index_t CThreadTransferDstScalarPerVector>
struct DeviceBatchedGemmXdl : public DeviceBatchedGemm<ALayout, BLayout, CLayout, ADataType, BDataType, CDataType,
                                                       AElementwiseOperation, BElementwiseOperation, CElementwiseOperation>
{
    using Argument = b200::BatchedGemmArgument;
    using Invoker  = b200::BatchedGemmInvoker;

    static auto MakeArgument(const ADataType* p_a, const BDataType* p_b, CDataType* p_c, index_t M, index_t N,
                             index_t K, index_t StrideA, index_t StrideB, index_t StrideC, index_t BatchStrideA,
                             index_t BatchStrideB, index_t BatchStrideC, index_t Batch, AElementwiseOperation,
                             BElementwiseOperation, CElementwiseOperation c_element_op)
    {
        const auto one = b200::make_gemm_argument<ALayout, BLayout, CLayout, ADataType, BDataType, CDataType,
                                                  AElementwiseOperation, BElementwiseOperation, CElementwiseOperation,
                                                  b200::ctx_gemm_c, 0>(p_a, p_b, {}, p_c, M, N, K, StrideA, StrideB, {},
                                                                       StrideC, c_element_op);
        Argument arg;
        arg.host_ok             = one.host_ok;
        arg.desc.gemm           = one.desc;
        arg.desc.batch          = Batch;
        arg.desc.batch_stride_a = BatchStrideA;
        arg.desc.batch_stride_b = BatchStrideB;
        arg.desc.batch_stride_e = BatchStrideC;
        return arg;
    }
    static auto MakeInvoker() { return Invoker{}; }
    static bool IsSupportedArgument(const Argument& arg)
    {
        return arg.host_ok && ckb_batched_gemm_supported(&arg.desc) == CKB_OK;
    }
    bool IsSupportedArgument(const BaseArgument* p_arg) override
    {
        return IsSupportedArgument(b200::argument_cast<Argument>(p_arg));
    }
    std::unique_ptr<BaseArgument>
    MakeArgumentPointer(const void* p_a, const void* p_b, void* p_c, index_t M, index_t N, index_t K, index_t StrideA,
                        index_t StrideB, index_t StrideC, index_t BatchStrideA, index_t BatchStrideB,
                        index_t BatchStrideC, index_t Batch, AElementwiseOperation a_op, BElementwiseOperation b_op,
                        CElementwiseOperation c_op) override
    {
        auto arg = std::make_unique<Argument>(MakeArgument(
            static_cast<const ADataType*>(p_a), static_cast<const BDataType*>(p_b), static_cast<CDataType*>(p_c), M, N, K,
            StrideA, StrideB, StrideC, BatchStrideA, BatchStrideB, BatchStrideC, Batch, a_op, b_op, c_op));
        arg->set_tile_config(this->tile_config_);
        return arg;
    }
    std::unique_ptr<BaseInvoker> MakeInvokerPointer() override { return std::make_unique<Invoker>(); }
    std::string GetTypeString() const override
    {
        std::ostringstream s; // device_batched_gemm_xdl.hpp:625-644
        s << "DeviceBatchedGemmXdl<" << BlockSize << ", " << MPerBlock << ", " << NPerBlock << ", " << K0PerBlock
          << ">";
        return s.str();
    }
};

// device_gemm_multiple_d_xdl_cshuffle.hpp:100-142
template <typename ALayout, typename BLayout, typename DELayout, typename ADataType, typename BDataType,
          typename GemmAccDataType, typename CShuffleDataType, typename DsDataType, typename EDataType,
          typename AElementwiseOperation, typename BElementwiseOperation, typename CDEElementwiseOperation,
          GemmSpecialization GemmSpec, index_t NumGemmKPrefetchStage, index_t BlockSize, index_t MPerBlock,
          index_t NPerBlock, index_t KPerBlock, index_t AK1, index_t BK1, index_t MPerXDL, index_t NPerXDL,
          index_t MXdlPerWave, index_t NXdlPerWave, CKB_XFER(ABlockTransfer), CKB_XFER(BBlockTransfer),
          index_t CShuffleMXdlPerWavePerShuffle, index_t CShuffleNXdlPerWavePerShuffle,
          typename CDEBlockTransferClusterLengths, index_t CDEBlockTransferScalarPerVector,
          LoopScheduler LoopSched = make_default_loop_scheduler()>
struct DeviceGemmMultipleD_Xdl_CShuffle
    : public DeviceGemmMultipleD<ALayout, BLayout, DELayout, ADataType, BDataType, DsDataType, EDataType,
                                 AElementwiseOperation, BElementwiseOperation, CDEElementwiseOperation>
{
    static constexpr index_t NumDTensor = DsDataType::Size();
    using Argument                      = b200::GemmArgument;
    using Invoker                       = b200::GemmInvoker;

    static auto MakeArgument(const void* p_a, const void* p_b, std::array<const void*, NumDTensor> p_ds, void* p_e,
                             index_t M, index_t N, index_t K, index_t StrideA, index_t StrideB,
                             std::array<index_t, NumDTensor> StrideDs, index_t StrideE, AElementwiseOperation,
                             BElementwiseOperation, CDEElementwiseOperation cde_element_op)
    {
        auto arg = b200::make_gemm_argument<ALayout, BLayout, DELayout, ADataType, BDataType, EDataType,
                                            AElementwiseOperation, BElementwiseOperation, CDEElementwiseOperation,
                                            b200::ctx_gemm_cde, NumDTensor>(p_a, p_b, p_ds, p_e, M, N, K, StrideA,
                                                                            StrideB, StrideDs, StrideE, cde_element_op);
        arg.host_ok = arg.host_ok && b200::specialization_accepts<GemmSpec, MPerBlock, NPerBlock, KPerBlock>(M, N, K);
        return arg;
    }
    static auto MakeInvoker() { return Invoker{}; }
    static bool IsSupportedArgument(const Argument& arg) { return b200::gemm_supported(arg); }
    bool IsSupportedArgument(const BaseArgument* p_arg) override
    {
        return IsSupportedArgument(b200::argument_cast<Argument>(p_arg));
    }
    std::unique_ptr<BaseArgument>
    MakeArgumentPointer(const void* p_a, const void* p_b, std::array<const void*, NumDTensor> p_ds, void* p_e, index_t M,
                        index_t N, index_t K, index_t StrideA, index_t StrideB, std::array<index_t, NumDTensor> StrideDs,
                        index_t StrideE, AElementwiseOperation a_op, BElementwiseOperation b_op,
                        CDEElementwiseOperation cde_op) override
    {
        auto arg = std::make_unique<Argument>(
            MakeArgument(p_a, p_b, p_ds, p_e, M, N, K, StrideA, StrideB, StrideDs, StrideE, a_op, b_op, cde_op));
        arg->set_tile_config(this->tile_config_);
        return arg;
    }
    std::unique_ptr<BaseInvoker> MakeInvokerPointer() override { return std::make_unique<Invoker>(); }
    std::string GetTypeString() const override
    {
        std::ostringstream s; // device_gemm_multiple_d_xdl_cshuffle.hpp:735-753
        s << "DeviceGemmMultipleD_Xdl_CShuffle<" << BlockSize << ", " << MPerBlock << ", " << NPerBlock << ", "
          << KPerBlock << ", " << AK1 << ", " << BK1 << ", " << getGemmSpecializationString(GemmSpec)
          << ">";
        return s.str();
    }
};

// device_grouped_gemm_xdl.hpp:89-131
template <typename ALayout, typename BLayout, typename DELayout, typename ADataType, typename BDataType,
          typename GemmAccDataType, typename CShuffleDataType, typename DsDataType, typename EDataType,
          typename AElementwiseOperation, typename BElementwiseOperation, typename CDEElementwiseOperation,
          GemmSpecialization GemmSpec, index_t NumPrefetch, index_t BlockSize, index_t MPerBlock, index_t NPerBlock,
          index_t KPerBlock, index_t AK1, index_t BK1, index_t MPerXDL, index_t NPerXDL, index_t MXdlPerWave,
          index_t NXdlPerWave, CKB_XFER(ABlockTransfer), CKB_XFER(BBlockTransfer), index_t CShuffleMXdlPerWavePerShuffle,
          index_t CShuffleNXdlPerWavePerShuffle, typename CDEBlockTransferClusterLengths,
          index_t CDEBlockTransferScalarPerVector, LoopScheduler LoopSched = make_default_loop_scheduler()>
struct DeviceGroupedGemmXdl
    : public DeviceGroupedGemm<ALayout, BLayout, DELayout, ADataType, BDataType, DsDataType, EDataType,
                               AElementwiseOperation, BElementwiseOperation, CDEElementwiseOperation>
{
    static constexpr index_t NumDTensor = DsDataType::Size();
    using Argument                      = b200::GroupedGemmArgument;
    using Invoker                       = b200::GroupedGemmInvoker;

    static auto MakeArgument(std::vector<const void*>& p_a, std::vector<const void*>& p_b,
                             std::vector<std::array<const void*, NumDTensor>>& p_ds, std::vector<void*>& p_e,
                             std::vector<GemmDesc>& gemm_descs, AElementwiseOperation, BElementwiseOperation,
                             CDEElementwiseOperation c_element_op)
    {
        const std::size_t n = gemm_descs.size();
        // device_grouped_gemm_xdl.hpp:547-552
        if(!(n == p_a.size() && n == p_b.size() && n == p_e.size()) || (NumDTensor > 0 && n != p_ds.size()))
            throw std::runtime_error("wrong! group_count_ != P_a/b/c.size");
        Argument arg;
        arg.groups.reserve(n);
        for(std::size_t i = 0; i < n; ++i)
        {
            std::array<const void*, NumDTensor> ds{};
            std::array<index_t, NumDTensor> sds{};
            for(index_t j = 0; j < NumDTensor; ++j)
            {
                ds[j]  = p_ds[i][j];
                sds[j] = gemm_descs[i].stride_Ds_.size() > static_cast<std::size_t>(j) ? gemm_descs[i].stride_Ds_[j] : 0;
            }
            auto one = b200::make_gemm_argument<ALayout, BLayout, DELayout, ADataType, BDataType, EDataType,
                                                AElementwiseOperation, BElementwiseOperation, CDEElementwiseOperation,
                                                b200::ctx_gemm_cde, NumDTensor>(
                p_a[i], p_b[i], ds, p_e[i], gemm_descs[i].M_, gemm_descs[i].N_, gemm_descs[i].K_, gemm_descs[i].stride_A_,
                gemm_descs[i].stride_B_, sds, gemm_descs[i].stride_C_, c_element_op);
            // device_grouped_gemm_xdl.hpp:586-628: a group the instance cannot run makes the argument unsupported
            arg.host_ok = arg.host_ok && one.host_ok &&
                          b200::specialization_accepts<GemmSpec, MPerBlock, NPerBlock, KPerBlock>(
                              gemm_descs[i].M_, gemm_descs[i].N_, gemm_descs[i].K_);
            arg.groups.push_back(one.desc);
        }
        return arg;
    }
    static auto MakeInvoker() { return Invoker{}; }
    static bool IsSupportedArgument(const Argument& arg)
    {
        const ckb_grouped_gemm_desc g = arg.view();
        return arg.host_ok && ckb_grouped_gemm_supported(&g) == CKB_OK;
    }
    bool IsSupportedArgument(const BaseArgument* p_arg) override
    {
        return IsSupportedArgument(b200::argument_cast<Argument>(p_arg));
    }
    std::unique_ptr<BaseArgument>
    MakeArgumentPointer(std::vector<const void*>& p_a, std::vector<const void*>& p_b,
                        std::vector<std::array<const void*, NumDTensor>>& p_ds, std::vector<void*>& p_e,
                        std::vector<GemmDesc>& gemm_descs, AElementwiseOperation a_op, BElementwiseOperation b_op,
                        CDEElementwiseOperation c_op) override
    {
        auto arg = std::make_unique<Argument>(MakeArgument(p_a, p_b, p_ds, p_e, gemm_descs, a_op, b_op, c_op));
        arg->set_tile_config(this->tile_config_);
        return arg;
    }
    std::unique_ptr<BaseInvoker> MakeInvokerPointer() override { return std::make_unique<Invoker>(); }
    // device_grouped_gemm_xdl.hpp:816-819: caller-allocated device memory
    size_t GetWorkSpaceSize(const BaseArgument* p_arg) const override
    {
        return b200::argument_cast<Argument>(p_arg).workspace_bytes();
    }
    std::string GetTypeString() const override
    {
        std::ostringstream s; // device_grouped_gemm_xdl.hpp:793-814
        s << "DeviceGroupedGemmXdl<" << BlockSize << ", " << MPerBlock << ", " << NPerBlock << ", " << KPerBlock << ", "
          << AK1 << ", " << BK1 << ", " << MPerXDL << ", " << NPerXDL << ", " << MXdlPerWave << ", " << NXdlPerWave
          << ">";
        return s.str();
    }
};

// device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp:42-75 (NumDimSpatial = 1, 2 or 3: NWC, NHWC, NDHWC tensors)
template <typename InDataType, typename WeiDataType, typename OutDataType, typename AccDataType,
          typename InElementwiseOperation, typename WeiElementwiseOperation, typename OutElementwiseOperation,
          ConvolutionForwardSpecialization ConvForwardSpecialization, index_t NumDimSpatial, index_t BlockSize,
          index_t MPerBlock, index_t NPerBlock, index_t K0PerBlock, index_t K1, index_t MPerXDL, index_t NPerXDL,
          index_t MXdlPerWave, index_t NXdlPerWave, CKB_XFER(ABlockTransfer), CKB_XFER(BBlockTransfer),
          index_t CThreadTransferSrcDstVectorDim, index_t CThreadTransferDstScalarPerVector>
struct DeviceConvNDFwdXdl_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K
    : public DeviceConvFwd<InElementwiseOperation, WeiElementwiseOperation, OutElementwiseOperation>
{
    using Argument = b200::ConvArgument;
    using Invoker  = b200::ConvInvoker;

    static auto MakeArgument(const InDataType* p_in, const WeiDataType* p_wei, OutDataType* p_out, index_t N, index_t K,
                             index_t C, std::vector<index_t> input_spatial_lengths,
                             std::vector<index_t> filter_spatial_lengths, std::vector<index_t> output_spatial_lengths,
                             std::vector<index_t> conv_filter_strides, std::vector<index_t> conv_filter_dilations,
                             std::vector<index_t> input_left_pads, std::vector<index_t> input_right_pads,
                             InElementwiseOperation, WeiElementwiseOperation, OutElementwiseOperation out_element_op)
    {
        auto arg = b200::make_conv_argument<InDataType, InElementwiseOperation, WeiElementwiseOperation,
                                            OutElementwiseOperation>(
            p_in, p_wei, p_out, nullptr, nullptr, N, K, C, input_spatial_lengths, filter_spatial_lengths,
            output_spatial_lengths, conv_filter_strides, conv_filter_dilations, input_left_pads, input_right_pads,
            out_element_op);
        arg.host_ok = arg.host_ok && static_cast<std::size_t>(NumDimSpatial) == input_spatial_lengths.size() &&
                      std::is_same<InDataType, WeiDataType>::value && std::is_same<InDataType, OutDataType>::value &&
                      b200::conv_specialization_accepts<ConvForwardSpecialization>(
                          filter_spatial_lengths, conv_filter_strides, input_left_pads, input_right_pads) &&
                      // device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp:921-933: the instance's vector widths must divide
                      // C and K - a channel count like C = 3 needs the ScalarPerVector = 1 (OddC) instances
                      b200::vector_widths_accept(C, K, ABlockTransferSrcScalarPerVector, BBlockTransferSrcScalarPerVector,
                                                 CThreadTransferDstScalarPerVector);
        return arg;
    }
    static auto MakeInvoker() { return Invoker{}; }
    static bool IsSupportedArgument(const Argument& arg) { return b200::conv_supported(arg); }
    bool IsSupportedArgument(const BaseArgument* p_arg) override
    {
        return IsSupportedArgument(b200::argument_cast<Argument>(p_arg));
    }
    std::unique_ptr<BaseArgument>
    MakeArgumentPointer(const void* p_in, const void* p_wei, void* p_out, index_t N, index_t K, index_t C,
                        std::vector<index_t> in_sp, std::vector<index_t> filt_sp, std::vector<index_t> out_sp,
                        std::vector<index_t> strides, std::vector<index_t> dilations, std::vector<index_t> lpads,
                        std::vector<index_t> rpads, InElementwiseOperation in_op, WeiElementwiseOperation wei_op,
                        OutElementwiseOperation out_op) override
    {
        auto arg = std::make_unique<Argument>(MakeArgument(static_cast<const InDataType*>(p_in),
                                                       static_cast<const WeiDataType*>(p_wei),
                                                       static_cast<OutDataType*>(p_out), N, K, C, in_sp, filt_sp, out_sp,
                                                       strides, dilations, lpads, rpads, in_op, wei_op, out_op));
        arg->set_tile_config(this->tile_config_);
        return arg;
    }
    std::unique_ptr<BaseInvoker> MakeInvokerPointer() override { return std::make_unique<Invoker>(); }
    std::string GetTypeString() const override
    {
        std::ostringstream s;
        s << "DeviceConvNDFwdXdl_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<" << BlockSize
          << ", " << MPerBlock << ", " << NPerBlock << ", " << K0PerBlock << ", "
          << getConvForwardSpecializationString(ConvForwardSpecialization)
          << ">";
        return s.str();
    }
};

// device_conv2d_fwd_xdl_c_shuffle_bias_activation_nhwc_kyxc_nhwk.hpp:26-62
template <typename InDataType, typename WeiDataType, typename OutDataType, typename AccDataType,
          typename InElementwiseOperation, typename WeiElementwiseOperation, typename OutElementwiseOperation,
          InMemoryDataOperationEnum OutGlobalMemoryDataOperation, ConvolutionForwardSpecialization ConvForwardSpecialization,
          index_t BlockSize, index_t MPerBlock, index_t NPerBlock, index_t K0PerBlock, index_t K1, index_t MPerXDL,
          index_t NPerXDL, index_t MXdlPerWave, index_t NXdlPerWave, CKB_XFER(ABlockTransfer), CKB_XFER(BBlockTransfer),
          index_t CShuffleMXdlPerWavePerShuffle, index_t CShuffleNXdlPerWavePerShuffle,
          typename CBlockTransferClusterLengths, index_t CBlockTransferScalarPerVector>
struct DeviceConv2dFwdXdl_C_Shuffle_Bias_Activation_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K
    : public DeviceConvFwdBiasActivation<InElementwiseOperation, WeiElementwiseOperation, OutElementwiseOperation>
{
    using Argument = b200::ConvArgument;
    using Invoker  = b200::ConvInvoker;

    // bias pointer in 4th position (device_conv2d_fwd_xdl_c_shuffle_bias_activation_nhwc_kyxc_nhwk.hpp:820-857)
    static auto MakeArgument(const InDataType* p_in, const WeiDataType* p_wei, OutDataType* p_out,
                             const OutDataType* p_bias, index_t N, index_t K, index_t C,
                             std::vector<index_t> input_spatial_lengths, std::vector<index_t> filter_spatial_lengths,
                             std::vector<index_t> output_spatial_lengths, std::vector<index_t> conv_filter_strides,
                             std::vector<index_t> conv_filter_dilations, std::vector<index_t> input_left_pads,
                             std::vector<index_t> input_right_pads, InElementwiseOperation, WeiElementwiseOperation,
                             OutElementwiseOperation out_element_op)
    {
        auto arg = b200::make_conv_argument<InDataType, InElementwiseOperation, WeiElementwiseOperation,
                                            OutElementwiseOperation>(
            p_in, p_wei, p_out, p_bias, nullptr, N, K, C, input_spatial_lengths, filter_spatial_lengths,
            output_spatial_lengths, conv_filter_strides, conv_filter_dilations, input_left_pads, input_right_pads,
            out_element_op);
        arg.host_ok = arg.host_ok && OutGlobalMemoryDataOperation == InMemoryDataOperationEnum::Set &&
                      std::is_same<InDataType, WeiDataType>::value && std::is_same<InDataType, OutDataType>::value &&
                      b200::conv_specialization_accepts<ConvForwardSpecialization>(
                          filter_spatial_lengths, conv_filter_strides, input_left_pads, input_right_pads) &&
                      // device_conv2d_fwd_xdl_c_shuffle_bias_activation_nhwc_kyxc_nhwk.hpp:793-806
                      b200::vector_widths_accept(C, K, ABlockTransferSrcScalarPerVector, BBlockTransferSrcScalarPerVector,
                                                 CBlockTransferScalarPerVector);
        return arg;
    }
    static auto MakeInvoker() { return Invoker{}; }
    static bool IsSupportedArgument(const Argument& arg) { return b200::conv_supported(arg); }
    bool IsSupportedArgument(const BaseArgument* p_arg) override
    {
        return IsSupportedArgument(b200::argument_cast<Argument>(p_arg));
    }
    std::unique_ptr<BaseArgument>
    MakeArgumentPointer(const void* p_in, const void* p_wei, void* p_out, const void* p_bias, index_t N, index_t K,
                        index_t C, std::vector<index_t> in_sp, std::vector<index_t> filt_sp, std::vector<index_t> out_sp,
                        std::vector<index_t> strides, std::vector<index_t> dilations, std::vector<index_t> lpads,
                        std::vector<index_t> rpads, InElementwiseOperation in_op, WeiElementwiseOperation wei_op,
                        OutElementwiseOperation out_op) override
    {
        auto arg = std::make_unique<Argument>(
            MakeArgument(static_cast<const InDataType*>(p_in), static_cast<const WeiDataType*>(p_wei),
                         static_cast<OutDataType*>(p_out), static_cast<const OutDataType*>(p_bias), N, K, C, in_sp,
                         filt_sp, out_sp, strides, dilations, lpads, rpads, in_op, wei_op, out_op));
        arg->set_tile_config(this->tile_config_);
        return arg;
    }
    std::unique_ptr<BaseInvoker> MakeInvokerPointer() override { return std::make_unique<Invoker>(); }
    std::string GetTypeString() const override
    {
        std::ostringstream s;
        s << "DeviceConv2dFwdXdl_C_Shuffle_Bias_Activation_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<" << BlockSize
          << ", " << MPerBlock << ", " << NPerBlock << ", " << K0PerBlock
          << ">";
        return s.str();
    }
};

// device_conv2d_fwd_xdl_c_shuffle_bias_activation_add_nhwc_kyxc_nhwk.hpp:25-66: out = out_op(conv, bias[k], resi)
// with the residual tensor laid out like the output (NHWK).
template <typename InDataType, typename WeiDataType, typename OutDataType, typename AccDataType,
          typename InElementwiseOperation, typename WeiElementwiseOperation, typename OutElementwiseOperation,
          ConvolutionForwardSpecialization ConvForwardSpecialization, index_t BlockSize, index_t MPerBlock,
          index_t NPerBlock, index_t K0PerBlock, index_t K1, index_t MPerXDL, index_t NPerXDL, index_t MXdlPerWave,
          index_t NXdlPerWave, CKB_XFER(ABlockTransfer), CKB_XFER(BBlockTransfer), index_t CShuffleMXdlPerWavePerShuffle,
          index_t CShuffleNXdlPerWavePerShuffle, typename CBlockTransferClusterLengths,
          index_t CBlockTransferScalarPerVector>
struct DeviceConv2dFwdXdl_C_Shuffle_Bias_Activation_Add_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K
    : public DeviceConvFwdBiasActivationAdd<InElementwiseOperation, WeiElementwiseOperation, OutElementwiseOperation>
{
    using Argument = b200::ConvArgument;
    using Invoker  = b200::ConvInvoker;

    static auto MakeArgument(const InDataType* p_in, const WeiDataType* p_wei, OutDataType* p_out,
                             const OutDataType* p_bias, const OutDataType* p_resi, index_t N, index_t K, index_t C,
                             std::vector<index_t> input_spatial_lengths, std::vector<index_t> filter_spatial_lengths,
                             std::vector<index_t> output_spatial_lengths, std::vector<index_t> conv_filter_strides,
                             std::vector<index_t> conv_filter_dilations, std::vector<index_t> input_left_pads,
                             std::vector<index_t> input_right_pads, InElementwiseOperation, WeiElementwiseOperation,
                             OutElementwiseOperation out_element_op)
    {
        auto arg = b200::make_conv_argument<InDataType, InElementwiseOperation, WeiElementwiseOperation,
                                            OutElementwiseOperation>(
            p_in, p_wei, p_out, p_bias, p_resi, N, K, C, input_spatial_lengths, filter_spatial_lengths,
            output_spatial_lengths, conv_filter_strides, conv_filter_dilations, input_left_pads, input_right_pads,
            out_element_op);
        arg.host_ok = arg.host_ok && std::is_same<InDataType, WeiDataType>::value &&
                      std::is_same<InDataType, OutDataType>::value &&
                      b200::conv_specialization_accepts<ConvForwardSpecialization>(
                          filter_spatial_lengths, conv_filter_strides, input_left_pads, input_right_pads) &&
                      b200::vector_widths_accept(C, K, ABlockTransferSrcScalarPerVector, BBlockTransferSrcScalarPerVector,
                                                 CBlockTransferScalarPerVector);
        return arg;
    }
    static auto MakeInvoker() { return Invoker{}; }
    static bool IsSupportedArgument(const Argument& arg) { return b200::conv_supported(arg); }
    bool IsSupportedArgument(const BaseArgument* p_arg) override
    {
        return IsSupportedArgument(b200::argument_cast<Argument>(p_arg));
    }
    std::unique_ptr<BaseArgument>
    MakeArgumentPointer(const void* p_in, const void* p_wei, void* p_out, const void* p_bias, const void* p_resi,
                        index_t N, index_t K, index_t C, std::vector<index_t> in_sp, std::vector<index_t> filt_sp,
                        std::vector<index_t> out_sp, std::vector<index_t> strides, std::vector<index_t> dilations,
                        std::vector<index_t> lpads, std::vector<index_t> rpads, InElementwiseOperation in_op,
                        WeiElementwiseOperation wei_op, OutElementwiseOperation out_op) override
    {
        auto arg = std::make_unique<Argument>(
            MakeArgument(static_cast<const InDataType*>(p_in), static_cast<const WeiDataType*>(p_wei),
                         static_cast<OutDataType*>(p_out), static_cast<const OutDataType*>(p_bias),
                         static_cast<const OutDataType*>(p_resi), N, K, C, in_sp, filt_sp, out_sp, strides, dilations,
                         lpads, rpads, in_op, wei_op, out_op));
        arg->set_tile_config(this->tile_config_);
        return arg;
    }
    std::unique_ptr<BaseInvoker> MakeInvokerPointer() override { return std::make_unique<Invoker>(); }
    std::string GetTypeString() const override
    {
        std::ostringstream s;
        s << "DeviceConv2dFwdXdl_C_Shuffle_Bias_Activation_Add_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<"
          << BlockSize << ", " << MPerBlock << ", " << NPerBlock << ", " << K0PerBlock
          << ">";
        return s.str();
    }
};

#undef CKB_XFER

} // namespace device
} // namespace tensor_operation
} // namespace ck
