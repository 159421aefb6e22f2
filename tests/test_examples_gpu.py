"""GPU tests: the reference-style C++ example drivers run on the device and verify themselves against
the CPU reference operators of the compat headers (exit code 0 = check_err passed, as in the reference)."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "examples", "bin")


@pytest.fixture(scope="module")
def examples_built(cuda_device):
    res = subprocess.run(["make", "-C", os.path.join(ROOT, "examples"), "-j4"], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    return BIN


def run_example(name, *args, timeout=900):
    res = subprocess.run([os.path.join(BIN, name)] + [str(a) for a in args], capture_output=True, text=True,
                         timeout=timeout)
    assert res.returncode == 0, f"{name} {args}: rc={res.returncode}\n{res.stdout[-2000:]}\n{res.stderr[-2000:]}"
    return res.stdout


def test_gemm_fp16_example(examples_built):
    # verify=1, integer init, timed; both reference instances (DeviceGemmXdl, DeviceGemm_Xdl_CShuffle)
    out = run_example("gemm_xdl_fp16", 1, 1, 1, 512, 768, 256, 256, 256, 768)
    assert out.count("Perf:") == 2 and "TFlops" in out
    run_example("gemm_xdl_fp16", 1, 2, 0, 768, 384, 160, 160, 160, 384)  # decimal init
    # The example's instances use GemmSpecialization::Default: a shape that does not divide the 256 x 128 x 32 block
    # tile is refused, as by the reference (gridwise_gemm_xdl_cshuffle_v1.hpp:222-226); the MNKPadding instances of
    # the factory take it (test_profiler_driver).
    res = subprocess.run([os.path.join(BIN, "gemm_xdl_fp16"), "1", "2", "0", "300", "200", "136", "136", "136", "200"],
                         capture_output=True, text=True, timeout=300)
    assert res.returncode != 0 and "does not support" in res.stdout + res.stderr


def test_gemm_add_add_fastgelu_example(examples_built):
    out = run_example("gemm_add_add_fastgelu_xdl_fp16", 1, 2, 1, 512, 512, 256, 256, 256, 0, 512, 512)
    assert "DeviceGemmMultipleD_Xdl_CShuffle" in out


def test_gemm_bilinear_example(examples_built):
    # example-local AlphaBetaAdd functor mapped to the library's bilinear epilogue by one trait specialisation
    # M N K StrideA StrideB StrideD StrideE alpha beta
    out = run_example("gemm_bilinear_xdl_fp16", 1, 1, 1, 512, 768, 256, 256, 256, 768, 768, 2.0, 0.5)
    assert "DeviceGemmMultipleD_Xdl_CShuffle" in out
    run_example("gemm_bilinear_xdl_fp16", 1, 2, 0, 256, 384, 192, 192, 192, 400, 392, 0.75, -1.25)  # padded D and E


def test_gemm_bias_relu_example(examples_built):
    # example-local binary16 AddRelu functor, bias row with stride 0, MNKPadding instance: ragged sizes are accepted
    out = run_example("gemm_bias_relu_xdl_fp16", 1, 1, 1, 512, 768, 256, 256, 256, 768)
    assert "DeviceGemmMultipleD_Xdl_CShuffle" in out
    # Integer init throughout: the functor adds in binary16 after the accumulator has been rounded to binary16, so
    # with decimal inputs a last-bit difference of the fp32 sum (summation order) can grow to two binary16 spacings
    # of the result, beyond check_err's 1e-3 bounds; integer inputs give exact sums.
    run_example("gemm_bias_relu_xdl_fp16", 1, 1, 0, 300, 200, 136, 136, 136, 200)


def test_grouped_gemm_bias_example(examples_built):
    out = run_example("grouped_gemm_bias_xdl_fp16", 1, 1, 1)
    assert "DeviceGroupedGemmXdl" in out
    run_example("grouped_gemm_bias_xdl_fp16", 1, 1, 0, 7)  # integer init: binary16 functor, see the bias + ReLU test


def test_convnd_fwd_example(examples_built):
    # verify init time nd N K C <filter> <input> <strides> <dilations> <left pads> <right pads>
    out = run_example("convnd_fwd_xdl_fp16", 1, 1, 1, 1, 4, 64, 32, 3, 71, 2, 1, 1, 1)
    assert "Perf:" in out and "DeviceConvNDFwdXdl" in out
    run_example("convnd_fwd_xdl_fp16", 1, 2, 0, 2, 4, 64, 64, 3, 3, 17, 19, 2, 1, 1, 2, 1, 2, 1, 2)
    run_example("convnd_fwd_xdl_fp16", 1, 1, 0, 3, 2, 32, 16, 3, 3, 3, 9, 10, 11, 1, 2, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1)
    # the int8 instance list of the same example (int32 accumulation, bit-exact)
    run_example("convnd_fwd_xdl_int8", 1, 1, 0, 2, 4, 64, 64, 3, 3, 17, 19, 2, 1, 1, 2, 1, 2, 1, 2)
    run_example("convnd_fwd_xdl_int8", 1, 1, 0, 1, 4, 64, 32, 3, 71, 2, 1, 1, 1)


def test_client_examples_walk_the_instance_factory(examples_built):
    """Client-style programs: device-operation interface + instance list only, best instance re-run at the end."""
    out = run_example("client_gemm", 512, 768, 256, 256, 256, 768)
    assert "found 6 instances" in out and "Best Perf:" in out and out.rstrip().endswith("Done")
    out = run_example("client_gemm_add_add_fastgelu", 512, 768, 256, 256, 256, 0, 768, 768)
    assert "Best Perf:" in out and "DeviceGemmMultipleD_Xdl_CShuffle" in out and out.rstrip().endswith("Done")


def test_reference_style_gemm_instance_tests(examples_built):
    """The reference's test/gemm programs: every factory instance, four layouts, fp16 / bf16 / int8, 1024^3."""
    out = run_example("test_gemm_instances")
    for name in ("fp16", "bf16", "int8"):
        assert f"TestGemm {name} ..... SUCCESS" in out
    assert "FAILURE" not in out


def test_grouped_gemm_random_groups_four_layouts(examples_built):
    """The reference's test/grouped_gemm/grouped_gemm_fp16.cpp: 1-10 groups with M, N in 256..2560 and K in
    128..1280 (multiples of 256 / 128), all four A/B layouts, verified against the CPU reference (seeded here)."""
    import random
    rnd = random.Random(11939)
    for layout in (0, 1, 2, 3):
        g = rnd.randrange(10) + 1
        ms = ",".join(str(256 + 256 * rnd.randrange(10)) for _ in range(g))
        ns = ",".join(str(256 + 256 * rnd.randrange(10)) for _ in range(g))
        ks = ",".join(str(128 + 128 * rnd.randrange(10)) for _ in range(g))
        out = run_example("ck_profiler", "grouped_gemm", 1, layout, 1, 1, 0, 1, ms, ns, ks)
        assert "Best Perf for grouped_gemm" in out


def test_int8_requant_example_both_roundings(examples_built):
    run_example("gemm_xdl_requant_relu_requant_int8", 1, 1, 0, 512, 512, 1024, 1024, 1024, 512)
    run_example("gemm_xdl_requant_relu_requant_int8", 1, 1, 0, 512, 512, 1024, 1024, 1024, 512, 1)


def test_grouped_gemm_example(examples_built):
    out = run_example("grouped_gemm_xdl_fp16", 1, 1, 1)  # the reference example's four groups
    assert "DeviceGroupedGemmXdl" in out


def test_conv_examples(examples_built):
    # N K C Y X Hi Wi Sy Sx Dy Dx LeftPy LeftPx RightPy RightPx
    geom = (4, 64, 64, 3, 3, 17, 17, 2, 2, 1, 1, 1, 1, 1, 1)
    out = run_example("conv2d_fwd_xdl_bias_relu", 1, 2, 1, 1, *geom)
    assert "DeviceConv2dFwdXdl_C_Shuffle_Bias_Activation_Input_N_Hi_Wi_C_Weight_K_Y_X_C_Output_N_Ho_Wo_K<" in out
    run_example("conv2d_fwd_xdl_bias_relu", 1, 1, 0, 0, *geom)  # plain convolution, integer init
    out = run_example("conv2d_fwd_xdl_bias_relu", 1, 2, 1, 2, *geom)  # bias + ReLU + residual add (example 07)
    assert "Bias_Activation_Add" in out


def test_default_shapes_timing_only(examples_built):
    """The headline shapes through the C++ drivers (verification is covered by the Python parity tests)."""
    out = run_example("gemm_xdl_fp16", 0, 1, 1)
    assert out.count("Perf:") == 2
    out = run_example("conv2d_fwd_xdl_bias_relu", 0, 2, 1)
    assert "Perf:" in out


def test_profiler_driver_walks_instance_lists(examples_built):
    """ckProfiler-style sub-commands: instances come from DeviceOperationInstanceFactory, every one is
    verified against the CPU reference operator and the best one is reported."""
    # gemm <dtype> <layout> verify init log time M N K StrideA StrideB StrideC
    for dtype in (1, 2, 3):  # fp16, bf16, int8
        out = run_example("ck_profiler", "gemm", dtype, 1, 1, 1, 0, 1, 512, 768, 256, 256, 256, 768)
        assert "Best Perf for gemm" in out and "DeviceGemm_Xdl_CShuffle" in out
    out = run_example("ck_profiler", "gemm", 1, 1, 1, 2, 0, 1, 300, 200, 136, 136, 136, 200)  # ragged: MNKPadding instances
    assert "Best Perf for gemm" in out
    # the other three matrix layouts of profile_gemm.cpp (0: mk_kn, 2: km_kn, 3: km_nk); M N K = 512 768 256
    for layout, sa, sb in ((0, 256, 768), (2, 512, 768), (3, 512, 256)):
        out = run_example("ck_profiler", "gemm", 1, layout, 1, 1, 0, 1, 512, 768, 256, sa, sb, 768)
        assert "Best Perf for gemm" in out
    out = run_example("ck_profiler", "gemm_add_add_fastgelu", 1, 1, 1, 2, 0, 1, 384, 512, 256, 256, 256, 0, 512, 512)
    assert "Best Perf for gemm_add_add_fastgelu" in out
    out = run_example("ck_profiler", "grouped_gemm", 1, 1, 1, 1, 0, 1, "256,512,768", "128,256,384", "64,128,192")
    assert "Best Perf for grouped_gemm" in out
    out = run_example("ck_profiler", "conv_fwd_bias_relu", 1, 1, 2, 0, 1, 4, 64, 64, 3, 3, 17, 17, 2, 2, 1, 1, 1, 1, 1, 1)
    assert "Best Perf for conv_fwd_bias_relu" in out
    # profile_conv_fwd_bias_relu_add.cpp: the same problem with a residual tensor added after the ReLU
    out = run_example("ck_profiler", "conv_fwd_bias_relu_add", 1, 1, 2, 0, 1, 4, 64, 64, 3, 3, 17, 17, 2, 2, 1, 1, 1, 1,
                      1, 1)
    assert "Best Perf for conv_fwd_bias_relu_add" in out


def test_profiler_driver_convnd(examples_built):
    """conv_fwd sub-command (profiler/src/profile_convnd_fwd.cpp:60-115): 1-D, 2-D and 3-D channels-last problems of
    the reference's device tests, verified against the N-D ReferenceConvFwd of the compat headers."""
    # conv_fwd dtype layout verify init log time nd N K C <filter> <input> <strides> <dilations> <lpads> <rpads>
    out = run_example("ck_profiler", "conv_fwd", 1, 1, 1, 1, 0, 1, 1, 4, 256, 64, 3, 71, 2, 2, 2, 2)
    assert "Best Perf for conv_fwd" in out and "DeviceConvNDFwdXdl" in out
    out = run_example("ck_profiler", "conv_fwd", 3, 1, 1, 1, 0, 1, 2, 4, 64, 64, 3, 3, 17, 17, 2, 2, 1, 1, 1, 1, 1, 1)
    assert "DeviceConvNDFwdXdl" in out
    out = run_example("ck_profiler", "conv_fwd", 1, 1, 1, 1, 0, 1, 3, 2, 64, 32, 3, 3, 3, 10, 10, 10, 1, 1, 1, 2, 2, 2,
                      2, 2, 2, 2, 2, 2)
    assert "Best Perf for conv_fwd" in out and "DeviceConvNDFwdXdl" in out


def test_profiler_driver_batched_gemm(examples_built):
    """batched_gemm sub-command (profiler/src/profile_batched_gemm.cpp:27-60), verified against ReferenceBatchedGemm."""
    # dtype layout verify init log time M N K StrideA StrideB StrideC BatchStrideA BatchStrideB BatchStrideC BatchCount
    out = run_example("ck_profiler", "batched_gemm", 1, 1, 1, 1, 0, 1, 256, 384, 128, 128, 128, 384,
                      256 * 128, 384 * 128, 256 * 384, 8)
    assert "Best Perf for batched_gemm" in out and "DeviceBatchedGemmXdl" in out
    out = run_example("ck_profiler", "batched_gemm", 3, 2, 1, 1, 0, 0, 256, 384, 128, 256, 384, 384,
                      256 * 128, 384 * 128, 256 * 384, 3)  # int8, A[g,k,m] * B[g,k,n]
    assert "Best Perf for batched_gemm" in out


@pytest.mark.parametrize("nd", [1, 2, 3])
def test_op_instance_run_engine_conv(examples_built, nd):
    """ConvFwdOpInstance + OpInstanceRunEngine (library/include/ck/library/utility/op_instance_engine.hpp:72-246,
    conv_util.hpp:399-570) in the style of test/convnd_fwd/conv{1,2,3}d_fwd.cpp: Test() then Profile()."""
    out = run_example("convnd_fwd_instance_engine", nd)
    assert "SUCCESS" in out and "PASSED" in out and "Perf:" in out


def test_odd_channel_conv_and_odd_pitch_gemm_through_the_device_ops(examples_built):
    """The reference's odd-channel problem (test/convnd_fwd/conv2d_fwd.cpp:110-111: C = 3) through an instance whose
    operand loads are one element wide, and a K = 1001, lda = ldb = 1001 GEMM through the MNKPadding instances of the
    factory: both verified by the example's CPU reference operator."""
    out = run_example("convnd_fwd_instance_engine", 2, "oddc")
    assert "SUCCESS" in out and "PASSED" in out and "Perf:" in out
    out = run_example("ck_profiler", "gemm", 1, 1, 1, 1, 0, 1, 515, 333, 1001, 1001, 1001, 333)
    assert "Best Perf for gemm" in out


def test_profiler_driver_bilinear_and_splitk(examples_built):
    """gemm_bilinear (profile_gemm_bilinear.cpp:29-43) and gemm_splitk (profile_gemm_splitk.cpp:29-42)."""
    out = run_example("ck_profiler", "gemm_bilinear", 1, 1, 1, 2, 0, 1, 384, 512, 256, 256, 256, 512, 512, 0.5, 1.5)
    assert "Best Perf for gemm_bilinear" in out
    out = run_example("ck_profiler", "gemm_bilinear", 1, 2, 1, 1, 0, 0, 384, 512, 256, 384, 512, 512, 512, 2.0, -1.0)
    out = run_example("ck_profiler", "gemm_splitk", 1, 1, 1, 1, 0, 1, 256, 256, 2048, 2048, 2048, 256, 4)
    assert "Best Perf for gemm_splitk" in out and "DeviceGemmXdlSplitKCShuffle" in out
