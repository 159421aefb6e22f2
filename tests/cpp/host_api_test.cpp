// Host-only checks of the Composable-Kernel-compatible C++ headers (no GPU call is made):
// descriptors, ConvParams, check_err, the CPU reference operators against the reference's golden
// vectors, functor semantics, epilogue-trait mapping, IsSupportedArgument and type strings.
#include <cmath>
#include <cstdio>
#include <iostream>
#include <string>
#include <vector>

#include "ck/ck.hpp"
#include "ck/library/host_tensor/host_tensor.hpp"
#include "ck/library/host_tensor/host_tensor_generator.hpp"
#include "ck/library/reference_tensor_operation/cpu/reference_conv_fwd.hpp"
#include "ck/library/reference_tensor_operation/cpu/reference_conv_fwd_bias_activation.hpp"
#include "ck/library/reference_tensor_operation/cpu/reference_gemm.hpp"
#include "ck/library/tensor_operation_instance/gpu/gemm.hpp"
#include "ck/library/tensor_operation_instance/gpu/gemm_add_add_fastgelu.hpp"
#include "ck/library/tensor_operation_instance/gpu/grouped_gemm.hpp"
#include "ck/library/utility/check_err.hpp"
#include "ck/library/utility/conv_util.hpp"
#include "ck/library/utility/fill.hpp"
#include "ck/tensor_operation/gpu/device/device_conv2d_fwd_xdl_c_shuffle_bias_activation_nhwc_kyxc_nhwk.hpp"
#include "ck/tensor_operation/gpu/device/device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp"
#include "ck/tensor_operation/gpu/device/device_batched_gemm_xdl.hpp"
#include "ck/tensor_operation/gpu/device/device_gemm_multiple_d_xdl_cshuffle.hpp"
#include "ck/tensor_operation/gpu/device/device_gemm_xdl_cshuffle.hpp"
#include "ck/tensor_operation/gpu/device/device_gemm_xdl_splitk_c_shuffle.hpp"
#include "ck/tensor_operation/gpu/device/device_grouped_gemm_xdl.hpp"
#include "ck/tensor_operation/gpu/element/element_wise_operation.hpp"

static int g_failed = 0;
#define EXPECT(cond)                                                          \
    do                                                                        \
    {                                                                         \
        if(!(cond))                                                           \
        {                                                                     \
            std::printf("FAILED %s:%d  %s\n", __FILE__, __LINE__, #cond);     \
            ++g_failed;                                                       \
        }                                                                     \
    } while(0)

template <ck::index_t... Is>
using S = ck::Sequence<Is...>;
using F16 = ck::half_t;
using Row = ck::tensor_layout::gemm::RowMajor;
using Col = ck::tensor_layout::gemm::ColumnMajor;
namespace ew  = ck::tensor_operation::element_wise;
namespace dev = ck::tensor_operation::device;

static constexpr auto GemmDefault = dev::GemmSpecialization::Default;
// clang-format off
template <typename AL, typename BL, typename T, typename COp>
using Gemm = dev::DeviceGemm_Xdl_CShuffle<AL, BL, Row, T, T, T, float, float, ew::PassThrough, ew::PassThrough, COp, GemmDefault,
    1, 256, 256, 128, 32, 8, 8, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, 1, 1, S<1, 32, 1, 8>, 8>;
template <dev::GemmSpecialization Spec>
using GemmSpec = dev::DeviceGemm_Xdl_CShuffle<Row, Col, Row, F16, F16, F16, float, float, ew::PassThrough, ew::PassThrough, ew::PassThrough, Spec,
    1, 256, 256, 128, 32, 8, 8, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, 1, 1, S<1, 32, 1, 8>, 8>;
template <typename CDEOp, typename Ds>
using GemmMultiD = dev::DeviceGemmMultipleD_Xdl_CShuffle<Row, Col, Row, F16, F16, float, float, Ds, F16, ew::PassThrough, ew::PassThrough, CDEOp, GemmDefault,
    1, 256, 256, 128, 32, 8, 8, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, 1, 1, S<1, 32, 1, 8>, 8>;
// clang-format on

struct LocalFunctor // a driver's own functor without a trait: must be reported as unsupported
{
    void operator()(float& y, const float& x) const { y = 3 * x; }
};

static void test_descriptors()
{
    HostTensorDescriptor packed(std::vector<std::size_t>{2, 3, 4});
    EXPECT(packed.GetStrides() == (std::vector<std::size_t>{12, 4, 1}));
    EXPECT(packed.GetElementSize() == 24 && packed.GetElementSpace() == 24);
    HostTensorDescriptor colmajor(std::vector<std::size_t>{3, 5}, std::vector<std::size_t>{1, 8});
    EXPECT(colmajor.GetElementSpace() == 1 + 2 * 1 + 4 * 8); // host_tensor.cpp:26-35
    EXPECT(colmajor.GetOffsetFromMultiIndex(2, 3) == 26);
    Tensor<float> t(std::vector<std::size_t>{3, 5}, std::vector<std::size_t>{1, 8});
    t.GenerateTensorValue(GeneratorTensor_Sequential<1>{}, 2);
    EXPECT(t(2, 3) == 3.0f && t.mData[26] == 3.0f);
    // NCHW-ordered lengths with NHWC strides (conv_util.hpp:209-215)
    auto d = ck::utils::conv::get_input_host_tensor_descriptor(std::vector<std::size_t>{2, 3, 4, 5});
    EXPECT(d.GetStrides() == (std::vector<std::size_t>{60, 1, 15, 3}));
}

static void test_conv_params()
{
    ck::utils::conv::ConvParams p; // test/conv_util/conv_util.cpp:43-79
    EXPECT(p.GetOutputSpatialLengths() == (std::vector<ck::index_t>{36, 36}));
    p.conv_filter_strides_ = {1, 1};
    EXPECT(p.GetOutputSpatialLengths() == (std::vector<ck::index_t>{71, 71}));
    p.conv_filter_strides_ = {2, 2};
    p.input_left_pads_ = p.input_right_pads_ = {2, 2};
    EXPECT(p.GetOutputSpatialLengths() == (std::vector<ck::index_t>{37, 37}));
    p.conv_filter_dilations_ = {2, 2};
    EXPECT(p.GetOutputSpatialLengths() == (std::vector<ck::index_t>{36, 36}));
    p.conv_filter_strides_ = {3, 3};
    p.input_left_pads_ = p.input_right_pads_ = {1, 1};
    EXPECT(p.GetOutputSpatialLengths() == (std::vector<ck::index_t>{23, 23}));
    ck::utils::conv::ConvParams q;
    EXPECT(ck::utils::conv::get_flops(q.N_, q.C_, q.K_, q.filter_spatial_lengths_, {36, 36}) == 146767085568ull);
    EXPECT((ck::utils::conv::get_btype<F16, F16, F16>(q.N_, q.C_, q.K_, q.input_spatial_lengths_,
                                                      q.filter_spatial_lengths_, {36, 36}) == 333594624ull));
}

static void test_check_err()
{
    std::vector<F16> ref{F16(1.0f), F16(100.0f), F16(0.0f)};
    std::vector<F16> ok{F16(1.001f), F16(100.06f), F16(0.0009f)};
    EXPECT(ck::utils::check_err(ok, ref));
    std::vector<F16> bad{F16(1.01f), F16(100.0f), F16(0.0f)};
    EXPECT(!ck::utils::check_err(bad, ref, "expected failure:"));
    EXPECT(ck::utils::check_err(std::vector<int8_t>{1, 2}, std::vector<int8_t>{1, 2}));
    EXPECT(!ck::utils::check_err(std::vector<int8_t>{1, 2}, std::vector<int8_t>{1, 3}, "expected failure:"));
}

// test/reference_conv_fwd/reference_conv_fwd.cpp:94-154: monotonic input, weights 0.5
static void test_reference_conv_golden()
{
    using Ref = ck::tensor_operation::host::ReferenceConvFwd<float, float, float, ew::PassThrough, ew::PassThrough,
                                                             ew::PassThrough, 2>;
    {
        Tensor<float> in(ck::utils::conv::get_input_host_tensor_descriptor(std::vector<std::size_t>{1, 2, 6, 6}));
        Tensor<float> wei(ck::utils::conv::get_filters_host_tensor_descriptor(std::vector<std::size_t>{1, 2, 3, 3}));
        Tensor<float> out(ck::utils::conv::get_output_host_tensor_descriptor(std::vector<std::size_t>{1, 1, 4, 4}));
        ck::utils::FillMonotonicSeq<float>{}(in.begin(), in.end());
        ck::utils::FillConstant<float>{0.5f}(wei.begin(), wei.end());
        auto arg = Ref::MakeArgument(in, wei, out, {1, 1}, {1, 1}, {0, 0}, {0, 0}, {}, {}, {});
        Ref::MakeInvoker().Run(arg);
        std::vector<float> want{130.5, 148.5, 166.5, 184.5, 238.5, 256.5, 274.5, 292.5,
                                346.5, 364.5, 382.5, 400.5, 454.5, 472.5, 490.5, 508.5};
        EXPECT(ck::utils::check_err(out.mData, want));
    }
    {
        Tensor<float> in(ck::utils::conv::get_input_host_tensor_descriptor(std::vector<std::size_t>{1, 2, 12, 12}));
        Tensor<float> wei(ck::utils::conv::get_filters_host_tensor_descriptor(std::vector<std::size_t>{2, 2, 3, 3}));
        Tensor<float> out(ck::utils::conv::get_output_host_tensor_descriptor(std::vector<std::size_t>{1, 2, 5, 5}));
        ck::utils::FillMonotonicSeq<float>{}(in.begin(), in.end());
        ck::utils::FillConstant<float>{0.5f}(wei.begin(), wei.end());
        auto arg = Ref::MakeArgument(in, wei, out, {2, 2}, {2, 2}, {1, 1}, {1, 1}, {}, {}, {});
        Ref::MakeInvoker().Run(arg);
        EXPECT(out.mData.size() == 50);
        EXPECT(out.mData[0] == 210.f && out.mData[1] == 210.f && out.mData[2] == 327.f && out.mData[12] == 706.5f &&
               out.mData[48] == 2110.5f && out.mData[49] == 2110.5f);
    }
}

static void test_reference_gemm_and_functors()
{
    // integer GEMM: exact
    Tensor<F16> a(std::vector<std::size_t>{3, 4}), c(std::vector<std::size_t>{3, 2});
    Tensor<F16> b(std::vector<std::size_t>{4, 2}, std::vector<std::size_t>{1, 4}); // column-major
    // generators are called with one index per dimension (variadic, like the reference's GeneratorTensor_*)
    a.GenerateTensorValue([](auto... is) {
        const std::size_t i[] = {static_cast<std::size_t>(is)...};
        return F16(float(i[0] + 1) * float(i[1] % 2 ? -1 : 1));
    });
    b.GenerateTensorValue([](auto... is) {
        const std::size_t i[] = {static_cast<std::size_t>(is)...};
        return F16(float(i[0] + i[1]));
    });
    using Ref = ck::tensor_operation::host::ReferenceGemm<F16, F16, F16, float, ew::PassThrough, ew::PassThrough,
                                                          ew::PassThrough>;
    auto arg = Ref::MakeArgument(a, b, c, {}, {}, {});
    Ref::MakeInvoker().Run(arg);
    for(int m = 0; m < 3; ++m)
        for(int n = 0; n < 2; ++n)
        {
            float want = 0;
            for(int k = 0; k < 4; ++k)
                want += float(m + 1) * (k % 2 ? -1.f : 1.f) * float(k + n);
            EXPECT(float(c(m, n)) == want);
        }
    // functor semantics
    F16 y;
    ew::Add{}(y, 2049.0f, F16(1.0f)); // half(2049)=2048; 2048+1 ties to even -> 2048
    EXPECT(float(y) == 2048.0f);
    float f;
    ew::AddRelu{}(f, -3.0f, 1.0f);
    EXPECT(f == 0.0f);
    ew::RequantReluRequant{0.03f, 1.0f}(f, 50.0f);
    EXPECT(static_cast<int8_t>(f) == 1); // 1.5 truncates
    ew::RequantReluRequantRne{0.03f, 14.0f}(f, 50.0f);
    EXPECT(f == 28.0f); // rne(1.5) = 2
    ew::AddAddFastGelu{}(y, 10.0f, F16(0.5f), F16(0.25f));
    EXPECT(float(y) == 10.75f);
}

static void test_traits_and_support()
{
    using namespace ck::b200;
    static_assert(EpilogueTraits<ew::PassThrough, ctx_gemm_c>::kind == CKB_EPI_PASSTHROUGH, "");
    static_assert(EpilogueTraits<ew::AddAddFastGelu, ctx_gemm_cde>::kind == CKB_EPI_ADD_ADD_FASTGELU, "");
    static_assert(EpilogueTraits<ew::AddRelu, ctx_conv>::kind == CKB_EPI_ADD_RELU, "");
    static_assert(EpilogueTraits<ew::AddRelu, ctx_gemm_cde>::kind == CKB_EPI_ADD_RELU_F16, "");
    static_assert(EpilogueTraits<ew::RequantReluRequant, ctx_gemm_c>::kind == CKB_EPI_REQUANT_RELU_REQUANT, "");
    static_assert(EpilogueTraits<LocalFunctor, ctx_gemm_c>::kind == -1, "");

    F16* pa = reinterpret_cast<F16*>(0x1000);
    F16* pb = reinterpret_cast<F16*>(0x2000);
    F16* pc = reinterpret_cast<F16*>(0x3000);
    using G = Gemm<Row, Col, F16, ew::PassThrough>;
    G gemm;
    auto ok = gemm.MakeArgument(pa, pb, pc, 3840, 4096, 4096, 4096, 4096, 4096, {}, {}, {});
    EXPECT(gemm.IsSupportedArgument(ok));
    EXPECT(gemm.IsSupportedArgument(&ok)); // polymorphic overload
    // A dimension the specialisation does not pad must divide the instance's block tile (256 x 128 x 32 here),
    // as in gridwise_gemm_xdl_cshuffle_v1.hpp:222-226 over the descriptors of device_gemm_xdl_cshuffle.hpp:84-346.
    auto ragged_default = gemm.MakeArgument(pa, pb, pc, 100, 40, 72, 72, 72, 40, {}, {}, {});
    EXPECT(!gemm.IsSupportedArgument(ragged_default));
    GemmSpec<dev::GemmSpecialization::MNKPadding> padded;
    auto ragged = padded.MakeArgument(pa, pb, pc, 100, 40, 72, 72, 72, 40, {}, {}, {});
    EXPECT(padded.IsSupportedArgument(ragged));
    GemmSpec<dev::GemmSpecialization::MNPadding> mn_padded;
    EXPECT(!mn_padded.IsSupportedArgument(mn_padded.MakeArgument(pa, pb, pc, 100, 40, 72, 72, 72, 40, {}, {}, {})));
    EXPECT(mn_padded.IsSupportedArgument(mn_padded.MakeArgument(pa, pb, pc, 100, 40, 96, 96, 96, 40, {}, {}, {})));
    GemmSpec<dev::GemmSpecialization::KPadding> k_padded;
    EXPECT(k_padded.IsSupportedArgument(k_padded.MakeArgument(pa, pb, pc, 512, 256, 72, 72, 72, 256, {}, {}, {})));
    EXPECT(!k_padded.IsSupportedArgument(k_padded.MakeArgument(pa, pb, pc, 500, 256, 72, 72, 72, 256, {}, {}, {})));
    // a pitch that TMA cannot address in place is served through a padded copy (the reference's ScalarPerVector = 1 case)
    auto odd = padded.MakeArgument(pa, pb, pc, 100, 40, 70, 70, 70, 40, {}, {}, {});
    EXPECT(padded.IsSupportedArgument(odd));
    // a leading dimension shorter than the row is refused whatever the specialisation
    auto bad = padded.MakeArgument(pa, pb, pc, 100, 40, 72, 64, 72, 40, {}, {}, {});
    EXPECT(!padded.IsSupportedArgument(bad));
    bool threw = false;
    try
    {
        padded.MakeInvoker().Run(bad);
    }
    catch(const std::runtime_error& e)
    {
        threw = std::string(e.what()).find("GridwiseGemm has invalid setting") != std::string::npos;
    }
    EXPECT(threw); // device_gemm_xdl_cshuffle.hpp:475-481
    EXPECT(gemm.GetTypeString() == "DeviceGemm_Xdl_CShuffle<256, 256, 128, 32, 8, 8>"); // device_gemm_xdl_cshuffle.hpp:655-672
    EXPECT(gemm.GetBackendString().find("B200") == 0);

    Gemm<Col, Col, F16, ew::PassThrough> gemm_km; // A column-major (km_nk): lda counts M
    auto km = gemm_km.MakeArgument(pa, pb, pc, 256, 256, 128, 256, 128, 256, {}, {}, {});
    EXPECT(gemm_km.IsSupportedArgument(km));
    auto km_bad = gemm_km.MakeArgument(pa, pb, pc, 256, 256, 128, 128, 128, 256, {}, {}, {});
    EXPECT(!gemm_km.IsSupportedArgument(km_bad));
    Gemm<Row, Row, F16, ew::PassThrough> gemm_kn; // B row-major (mk_kn): ldb counts N
    auto kn = gemm_kn.MakeArgument(pa, pb, pc, 256, 512, 128, 128, 512, 512, {}, {}, {});
    EXPECT(gemm_kn.IsSupportedArgument(kn));
    Gemm<Row, Col, F16, LocalFunctor> gemm_local;
    auto loc = gemm_local.MakeArgument(pa, pb, pc, 256, 256, 256, 256, 256, 256, {}, {}, LocalFunctor{});
    EXPECT(!gemm_local.IsSupportedArgument(loc));
    Gemm<Row, Col, int8_t, ew::RequantReluRequant> gemm_i8;
    auto i8 = gemm_i8.MakeArgument(reinterpret_cast<int8_t*>(pa), reinterpret_cast<int8_t*>(pb),
                                   reinterpret_cast<int8_t*>(pc), 3840, 4096, 4096, 4096, 4096, 4096, {}, {},
                                   ew::RequantReluRequant{0.03f, 1.0f});
    EXPECT(gemm_i8.IsSupportedArgument(i8));

    GemmMultiD<ew::AddAddFastGelu, ck::Tuple<F16, F16>> md;
    auto mda = md.MakeArgument(pa, pb, std::array<const void*, 2>{pa, pb}, pc, 3840, 4096, 4096, 4096, 4096,
                               std::array<ck::index_t, 2>{0, 4096}, 4096, {}, {}, {});
    EXPECT(md.IsSupportedArgument(mda));
    std::unique_ptr<dev::BaseArgument> base =
        md.MakeArgumentPointer(pa, pb, std::array<const void*, 2>{pa, pb}, pc, 3840, 4096, 4096, 4096, 4096,
                               std::array<ck::index_t, 2>{0, 4096}, 4096, {}, {}, {});
    EXPECT(md.IsSupportedArgument(base.get()));
    EXPECT(md.GetTypeString().find("DeviceGemmMultipleD_Xdl_CShuffle<256, 256, 128, 32, 8, 8, Default>") == 0);

    // grouped: size mismatch throws (device_grouped_gemm_xdl.hpp:547-552); workspace size reported
    // clang-format off
    using Grouped = dev::DeviceGroupedGemmXdl<Row, Col, Row, F16, F16, float, F16, ck::Tuple<>, F16, ew::PassThrough, ew::PassThrough, ew::PassThrough, GemmDefault,
        1, 256, 256, 128, 32, 8, 8, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, 1, 1, 1, S<1, 32, 1, 8>, 8>;
    // clang-format on
    Grouped gg;
    std::vector<const void*> va{pa, pa}, vb{pb, pb};
    std::vector<void*> vc{pc, pc};
    std::vector<std::array<const void*, 0>> vds(2);
    std::vector<dev::GemmDesc> descs{{256, 128, 64, 64, 64, 128, {}}, {512, 256, 128, 128, 128, 256, {}}};
    auto ga = gg.MakeArgument(va, vb, vds, vc, descs, {}, {}, {});
    EXPECT(gg.IsSupportedArgument(ga));
    EXPECT(gg.GetWorkSpaceSize(&ga) >= 2 * 512);
    std::vector<const void*> short_a{pa};
    threw = false;
    try
    {
        gg.MakeArgument(short_a, vb, vds, vc, descs, {}, {}, {});
    }
    catch(const std::runtime_error&)
    {
        threw = true;
    }
    EXPECT(threw);

    // conv: default ConvParams is supported, inconsistent output size is not
    // clang-format off
    using Conv = dev::DeviceConv2dFwdXdl_C_Shuffle_Bias_Activation_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<
        F16, F16, F16, float, ew::PassThrough, ew::PassThrough, ew::AddRelu, ck::InMemoryDataOperationEnum::Set,
        dev::ConvolutionForwardSpecialization::Default, 256, 128, 256, 4, 8, 32, 32, 2, 4, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true,
        S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true, 1, 1, S<1, 1, 32, 1, 1, 8>, 8>;
    // clang-format on
    Conv conv;
    ck::utils::conv::ConvParams p;
    auto ca = conv.MakeArgument(pa, pb, pc, pa, p.N_, p.K_, p.C_, p.input_spatial_lengths_, p.filter_spatial_lengths_,
                                p.GetOutputSpatialLengths(), p.conv_filter_strides_, p.conv_filter_dilations_,
                                p.input_left_pads_, p.input_right_pads_, {}, {}, {});
    EXPECT(conv.IsSupportedArgument(ca));
    auto cb = conv.MakeArgument(pa, pb, pc, pa, p.N_, p.K_, p.C_, p.input_spatial_lengths_, p.filter_spatial_lengths_,
                                {35, 36}, p.conv_filter_strides_, p.conv_filter_dilations_, p.input_left_pads_,
                                p.input_right_pads_, {}, {}, {});
    EXPECT(!conv.IsSupportedArgument(cb));

    // an instance specialised for 1x1 filters refuses every other geometry
    // (device_conv2d_fwd_xdl_c_shuffle_bias_activation_nhwc_kyxc_nhwk.hpp IsSupportedArgument, same rule as
    // device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp:894-919)
    // clang-format off
    using Conv1x1 = dev::DeviceConv2dFwdXdl_C_Shuffle_Bias_Activation_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<
        F16, F16, F16, float, ew::PassThrough, ew::PassThrough, ew::AddRelu, ck::InMemoryDataOperationEnum::Set,
        dev::ConvolutionForwardSpecialization::Filter1x1Stride1Pad0, 256, 128, 256, 4, 8, 32, 32, 2, 4, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true,
        S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true, 1, 1, S<1, 1, 32, 1, 1, 8>, 8>;
    // clang-format on
    Conv1x1 conv1x1;
    EXPECT(!conv1x1.IsSupportedArgument(conv1x1.MakeArgument(
        pa, pb, pc, pa, p.N_, p.K_, p.C_, p.input_spatial_lengths_, p.filter_spatial_lengths_, p.GetOutputSpatialLengths(),
        p.conv_filter_strides_, p.conv_filter_dilations_, p.input_left_pads_, p.input_right_pads_, {}, {}, {})));
    EXPECT(conv1x1.IsSupportedArgument(conv1x1.MakeArgument(pa, pb, pc, pa, 4, 64, 64, {20, 20}, {1, 1}, {20, 20}, {1, 1},
                                                            {1, 1}, {0, 0}, {0, 0}, {}, {}, {})));
    EXPECT(!conv1x1.IsSupportedArgument(conv1x1.MakeArgument(pa, pb, pc, pa, 4, 64, 64, {20, 20}, {1, 1}, {10, 10}, {2, 2},
                                                             {1, 1}, {0, 0}, {0, 0}, {}, {}, {})));
}

// The instance lists a profiler-style client walks: non-empty for the kernels that exist, each instance
// answering IsSupportedArgument through the abstract interface; float GEMM has an instance that refuses.
static void test_instance_factory()
{
    namespace inst = dev::instance;
    using inst::Col;
    using inst::Row;
    using PT = inst::PassThrough;
    const void* pa = reinterpret_cast<const void*>(0x1000);
    void* pc       = reinterpret_cast<void*>(0x3000);
    {
        using Op = dev::DeviceGemm<Row, Col, Row, ck::half_t, ck::half_t, ck::half_t, PT, PT, PT>;
        auto ops = inst::DeviceOperationInstanceFactory<Op>::GetInstances();
        EXPECT(ops.size() == 6); // the library's own choice + five pinned tile configurations
        EXPECT(ops[0]->GetTileConfig() == 0 && ops[1]->GetTileConfig() == CKB_TILE_CONFIG(256, 2, 0));
        EXPECT(ops[1]->GetTypeString() == "DeviceGemm_Xdl_CShuffle<320, 256, 256, 64, 8, 8>");
        EXPECT(ops[4]->GetTypeString() == "DeviceGemm_Xdl_CShuffle<320, 128, 64, 64, 8, 8>");
        EXPECT(ops[5]->GetBackendString().find("no K split") != std::string::npos);
        for(auto& op : ops)
        {
            auto a = op->MakeArgumentPointer(pa, pa, pc, 256, 256, 64, 64, 64, 256, {}, {}, {});
            EXPECT(op->IsSupportedArgument(a.get()));
            EXPECT(dynamic_cast<ck::b200::GemmArgument*>(a.get())->desc.tile_config == op->GetTileConfig());
        }
        auto arg = ops[0]->MakeArgumentPointer(pa, pa, pc, 256, 256, 64, 64, 64, 256, {}, {}, {});
        EXPECT(ops[0]->IsSupportedArgument(arg.get()));
        EXPECT(ops[0]->GetTypeString().find("DeviceGemm_Xdl_CShuffle") != std::string::npos);
        auto bad = ops[0]->MakeArgumentPointer(pa, pa, pc, 256, 256, 64, 60, 64, 256, {}, {}, {});
        EXPECT(!ops[0]->IsSupportedArgument(bad.get())); // StrideA < K
    }
    {
        using Op = dev::DeviceGemm<Row, Col, Row, ck::bhalf_t, ck::bhalf_t, ck::bhalf_t, PT, PT, PT>;
        auto ops = inst::DeviceOperationInstanceFactory<Op>::GetInstances();
        auto arg = ops[0]->MakeArgumentPointer(pa, pa, pc, 256, 256, 64, 64, 64, 256, {}, {}, {});
        EXPECT(ops[0]->IsSupportedArgument(arg.get()));
    }
    {
        using Op = dev::DeviceGemm<Row, Col, Row, int8_t, int8_t, int8_t, PT, PT, PT>;
        auto ops = inst::DeviceOperationInstanceFactory<Op>::GetInstances();
        auto arg = ops[0]->MakeArgumentPointer(pa, pa, pc, 256, 256, 64, 64, 64, 256, {}, {}, {});
        EXPECT(ops[0]->IsSupportedArgument(arg.get()));
    }
    {
        using Op = dev::DeviceGemm<Row, Col, Row, float, float, float, PT, PT, PT>;
        auto ops = inst::DeviceOperationInstanceFactory<Op>::GetInstances();
        auto arg = ops[0]->MakeArgumentPointer(pa, pa, pc, 256, 256, 64, 64, 64, 256, {}, {}, {});
        EXPECT(!ops[0]->IsSupportedArgument(arg.get())); // no fp32 kernels
    }
    {
        using Op = dev::DeviceGemmMultipleD<Row, Col, Row, ck::half_t, ck::half_t, inst::F16_F16_TUPLE, ck::half_t, PT, PT,
                                            inst::AddAddFastGelu>;
        auto ops = inst::DeviceOperationInstanceFactory<Op>::GetInstances();
        EXPECT(ops.size() == 6);
        auto arg = ops[0]->MakeArgumentPointer(pa, pa, std::array<const void*, 2>{pa, pa}, pc, 256, 256, 64, 64, 64,
                                               std::array<ck::index_t, 2>{0, 256}, 256, {}, {}, {});
        EXPECT(ops[0]->IsSupportedArgument(arg.get()));
    }
    {
        using Op = dev::DeviceGroupedGemm<Row, Col, Row, ck::half_t, ck::half_t, inst::EMPTY_TUPLE, ck::half_t, PT, PT, PT>;
        auto ops = inst::DeviceOperationInstanceFactory<Op>::GetInstances();
        EXPECT(ops.size() == 6);
        std::vector<const void*> as{pa, pa}, bs{pa, pa};
        std::vector<void*> cs{pc, pc};
        std::vector<std::array<const void*, 0>> ds(2);
        std::vector<dev::GemmDesc> descs{{256, 128, 64, 64, 64, 128, {}}, {512, 256, 128, 128, 128, 256, {}}};
        auto arg = ops[0]->MakeArgumentPointer(as, bs, ds, cs, descs, {}, {}, {});
        EXPECT(ops[0]->GetWorkSpaceSize(arg.get()) > 0);
        auto arg3 = ops[3]->MakeArgumentPointer(as, bs, ds, cs, descs, {}, {}, {});
        EXPECT(ops[3]->IsSupportedArgument(arg3.get()));
        EXPECT(dynamic_cast<ck::b200::GroupedGemmArgument*>(arg3.get())->view().tile_config == CKB_TILE_CONFIG(128, 1, 0));
    }
}

// DeviceBatchedGemmXdl with the reference's positional template list (example/../batched_gemm test instances)
static void test_batched_gemm_host_side()
{
    // clang-format off
    using Batched = dev::DeviceBatchedGemmXdl<F16, F16, F16, float, Row, Col, Row, ew::PassThrough, ew::PassThrough, ew::PassThrough,
        256, 256, 128, 4, 8, 32, 32, 4, 2, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true,
        S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true, 7, 1>;
    // clang-format on
    const F16* pa = reinterpret_cast<const F16*>(0x1000);
    F16* pc       = reinterpret_cast<F16*>(0x3000);
    Batched op;
    auto arg = op.MakeArgument(pa, pa, pc, 256, 256, 64, 64, 64, 256, 256 * 64, 256 * 64, 256 * 256, 8, {}, {}, {});
    EXPECT(op.IsSupportedArgument(arg));
    auto none = op.MakeArgument(pa, pa, pc, 256, 256, 64, 64, 64, 256, 256 * 64, 256 * 64, 256 * 256, 0, {}, {}, {});
    EXPECT(!op.IsSupportedArgument(none));
    EXPECT(op.GetTypeString().find("DeviceBatchedGemmXdl<256, 256, 128, 4>") == 0);
    // clang-format off
    using SplitK = dev::DeviceGemmXdlSplitKCShuffle<F16, F16, F16, float, Row, Col, Row, ew::PassThrough, ew::PassThrough, ew::PassThrough, GemmDefault,
        256, 256, 128, 4, 8, 32, 32, 4, 2, S<1, 4, 64, 1>, S<0, 2, 1, 3>, S<0, 2, 1, 3>, 3, 8, 8, true,
        S<1, 4, 64, 1>, S<0, 1, 3, 2>, S<0, 1, 3, 2>, 3, 8, 8, true, 1, 1, S<1, 32, 1, 8>, 8>;
    // clang-format on
    SplitK sk;
    dev::DeviceGemmSplitK<Row, Col, Row, F16, F16, F16, ew::PassThrough, ew::PassThrough, ew::PassThrough>* sk_base = &sk;
    auto sk_arg = sk_base->MakeArgumentPointer(pa, pa, pc, 256, 256, 512, 512, 512, 256, {}, {}, {}, 4);
    EXPECT(sk_base->IsSupportedArgument(sk_arg.get()));
    auto sk_bad = sk_base->MakeArgumentPointer(pa, pa, pc, 256, 256, 512, 512, 512, 256, {}, {}, {}, 0);
    EXPECT(!sk_base->IsSupportedArgument(sk_bad.get()));
    dev::DeviceBatchedGemm<Row, Col, Row, F16, F16, F16, ew::PassThrough, ew::PassThrough, ew::PassThrough>* base = &op;
    auto parg = base->MakeArgumentPointer(pa, pa, pc, 256, 256, 64, 64, 64, 256, 256 * 64, 256 * 64, 256 * 256, 8, {}, {}, {});
    EXPECT(base->IsSupportedArgument(parg.get()));
}

// 1-D and 3-D: the reference's golden vectors for its CPU operator (test/reference_conv_fwd/reference_conv_fwd.cpp:
// Conv1DNWC, Conv1DNWCStridesDilationsPadding, Conv3DNCDHW) and the NumDimSpatial = 1 / 3 device operations.
static void test_convnd_host_side()
{
    namespace host = ck::tensor_operation::host;
    {
        using Ref = host::ReferenceConvFwd<float, float, float, ew::PassThrough, ew::PassThrough, ew::PassThrough, 1>;
        Tensor<float> in(ck::utils::conv::get_input_host_tensor_descriptor(std::vector<std::size_t>{1, 2, 6}));
        Tensor<float> wei(ck::utils::conv::get_filters_host_tensor_descriptor(std::vector<std::size_t>{1, 2, 3}));
        Tensor<float> out(ck::utils::conv::get_output_host_tensor_descriptor(std::vector<std::size_t>{1, 1, 4}));
        ck::utils::FillMonotonicSeq<float>{}(in.begin(), in.end());
        ck::utils::FillConstant<float>{0.5f}(wei.begin(), wei.end());
        auto arg = Ref::MakeArgument(in, wei, out, {1}, {1}, {0}, {0}, {}, {}, {});
        Ref::MakeInvoker().Run(arg);
        EXPECT(ck::utils::check_err(out.mData, std::vector<float>{7.5, 13.5, 19.5, 25.5}));
    }
    {
        using Ref = host::ReferenceConvFwd<float, float, float, ew::PassThrough, ew::PassThrough, ew::PassThrough, 1>;
        Tensor<float> in(ck::utils::conv::get_input_host_tensor_descriptor(std::vector<std::size_t>{1, 2, 12}));
        Tensor<float> wei(ck::utils::conv::get_filters_host_tensor_descriptor(std::vector<std::size_t>{2, 2, 3}));
        Tensor<float> out(ck::utils::conv::get_output_host_tensor_descriptor(std::vector<std::size_t>{1, 2, 5}));
        ck::utils::FillMonotonicSeq<float>{}(in.begin(), in.end());
        ck::utils::FillConstant<float>{0.5f}(wei.begin(), wei.end());
        auto arg = Ref::MakeArgument(in, wei, out, {2}, {2}, {1}, {1}, {}, {}, {});
        Ref::MakeInvoker().Run(arg);
        EXPECT(ck::utils::check_err(out.mData, std::vector<float>{9., 9., 19.5, 19.5, 31.5, 31.5, 43.5, 43.5, 55.5, 55.5}));
    }
    {
        // NCDHW in memory (packed channel-first descriptor), output NKDHW, input 0, 0.1, 0.2, ...
        using Ref = host::ReferenceConvFwd<float, float, float, ew::PassThrough, ew::PassThrough, ew::PassThrough, 3>;
        Tensor<float> in(HostTensorDescriptor(std::vector<std::size_t>{1, 2, 6, 6, 6}));
        Tensor<float> wei(HostTensorDescriptor(std::vector<std::size_t>{1, 2, 3, 3, 3}));
        Tensor<float> out(HostTensorDescriptor(std::vector<std::size_t>{1, 1, 4, 4, 4}));
        ck::utils::FillMonotonicSeq<float>{0.f, 0.1f}(in.begin(), in.end());
        ck::utils::FillConstant<float>{0.5f}(wei.begin(), wei.end());
        auto arg = Ref::MakeArgument(in, wei, out, {1, 1, 1}, {1, 1, 1}, {0, 0, 0}, {0, 0, 0}, {}, {}, {});
        Ref::MakeInvoker().Run(arg);
        EXPECT(out.mData.size() == 64);
        EXPECT(std::abs(out.mData[0] - 407.7f) < 1e-2f && std::abs(out.mData[1] - 410.4f) < 1e-2f &&
               std::abs(out.mData[16] - 504.9f) < 1e-2f && std::abs(out.mData[63] - 756.f) < 1e-2f);
    }
    // clang-format off
    using Conv1d = dev::DeviceConvNDFwdXdl_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<
        F16, F16, F16, float, ew::PassThrough, ew::PassThrough, ew::PassThrough, dev::ConvolutionForwardSpecialization::Default, 1,
        256, 128, 256, 4, 8, 32, 32, 2, 4, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true,
        S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true, 7, 1>;
    using Conv3d = dev::DeviceConvNDFwdXdl_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<
        F16, F16, F16, float, ew::PassThrough, ew::PassThrough, ew::PassThrough, dev::ConvolutionForwardSpecialization::Default, 3,
        256, 128, 256, 4, 8, 32, 32, 2, 4, S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true,
        S<4, 64, 1>, S<1, 0, 2>, S<1, 0, 2>, 2, 8, 8, true, 7, 1>;
    // clang-format on
    const F16* pa = reinterpret_cast<const F16*>(0x1000);
    F16* pc       = reinterpret_cast<F16*>(0x3000);
    // test/convnd_fwd/conv1d_fwd.cpp:73-74 and conv3d_fwd.cpp:76-77
    auto a1 = Conv1d::MakeArgument(pa, pa, pc, 4, 256, 64, {71}, {3}, {36}, {2}, {2}, {2}, {2}, {}, {}, {});
    EXPECT(Conv1d::IsSupportedArgument(a1));
    auto a3 = Conv3d::MakeArgument(pa, pa, pc, 4, 256, 64, {28, 28, 28}, {3, 3, 3}, {14, 14, 14}, {2, 2, 2}, {2, 2, 2},
                                   {2, 2, 2}, {2, 2, 2}, {}, {}, {});
    EXPECT(Conv3d::IsSupportedArgument(a3));
    auto mismatch = Conv3d::MakeArgument(pa, pa, pc, 4, 256, 64, {28, 28}, {3, 3}, {14, 14}, {2, 2}, {2, 2}, {2, 2},
                                         {2, 2}, {}, {}, {});
    EXPECT(!Conv3d::IsSupportedArgument(mismatch)); // a 2-D problem handed to the 3-D instance
    EXPECT(Conv3d{}.GetTypeString().find("DeviceConvNDFwdXdl_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<") == 0);
    // device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp:921-933: C = 3 needs an instance whose vector widths divide it
    auto c3 = Conv1d::MakeArgument(pa, pa, pc, 4, 256, 3, {71}, {3}, {36}, {2}, {2}, {2}, {2}, {}, {}, {});
    EXPECT(!Conv1d::IsSupportedArgument(c3));
}

int main()
{
    test_convnd_host_side();
    test_batched_gemm_host_side();
    test_instance_factory();
    test_descriptors();
    test_conv_params();
    test_check_err();
    test_reference_conv_golden();
    test_reference_gemm_and_functors();
    test_traits_and_support();
    std::printf(g_failed ? "%d checks FAILED\n" : "all host API checks passed\n", g_failed);
    return g_failed ? 1 : 0;
}
