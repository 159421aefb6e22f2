"""GPU parity tests of the implicit-GEMM conv2d forward path (TMA im2col producer) vs the oracle."""
import json
import os

import numpy as np
import pytest
import torch

import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from oracle import ck_oracle as oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu


def run_conv(inp, wei, stride, dilation, pad, op=None, bias=None, resi=None, time_kernel=False):
    op = op or ck.PassThrough()
    N, Hi, Wi, C = inp.shape
    K, Y, X, _ = wei.shape
    Ho = oracle.conv_out_len(Hi, Y, stride[0], dilation[0], pad[0], pad[0])
    Wo = oracle.conv_out_len(Wi, X, stride[1], dilation[1], pad[1], pad[1])
    di, dw = H.to_dev(inp), H.to_dev(wei)
    db = H.to_dev(bias) if bias is not None else None
    dr = H.to_dev(resi) if resi is not None else None
    out = torch.full((N, Ho, Wo, K), float("nan"), dtype=torch.float16, device="cuda")
    conv = ck.DeviceConvFwd()
    arg = conv.MakeArgument(di.data_ptr(), dw.data_ptr(), out.data_ptr(), N, K, C, (Hi, Wi), (Y, X), (Ho, Wo),
                            stride, dilation, pad, pad, None, None, op,
                            p_bias=db.data_ptr() if db is not None else None,
                            p_resi=dr.data_ptr() if dr is not None else None)
    assert conv.IsSupportedArgument(arg), capi.last_error()
    ms = conv.MakeInvoker().Run(arg, ck.StreamConfig(None, time_kernel))
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    return out.cpu().numpy(), ms


# N, C, Hi, Wi, K, Y, X, stride, dilation, pad
CASES = [
    (4, 64, 36, 36, 256, 3, 3, (2, 2), (2, 2), (2, 2)),   # test/convnd_fwd/conv2d_fwd.cpp:104 default
    (4, 64, 28, 28, 256, 1, 1, (1, 1), (1, 1), (0, 0)),   # :106 filter 1x1 stride 1 pad 0
    (4, 64, 28, 28, 256, 1, 1, (2, 2), (1, 1), (0, 0)),   # :108 filter 1x1 stride 2 pad 0
    (2, 192, 15, 15, 256, 3, 3, (2, 2), (1, 1), (1, 1)),  # the headline geometry, small image (odd Hi)
    (3, 8, 11, 7, 24, 3, 2, (1, 1), (1, 1), (1, 1)),      # C below one stage, K not a multiple of 8
    (2, 72, 9, 12, 40, 2, 3, (1, 2), (2, 1), (1, 2)),     # anisotropic stride / dilation / pad, C tail
    (1, 16, 5, 5, 16, 5, 5, (1, 1), (1, 1), (2, 2)),      # filter as large as the image
    (5, 32, 10, 10, 64, 3, 3, (3, 3), (2, 2), (1, 1)),    # test/conv_util geometry s3 p1 d2
]


@pytest.mark.parametrize("case", CASES)
def test_conv2d_fwd_bias_relu(cuda_device, case):
    N, C, Hi, Wi, K, Y, X, s, d, p = case
    rng = np.random.default_rng(N * 100 + C)
    inp, wei, bias = H.rand_f16(rng, (N, Hi, Wi, C)), H.rand_f16(rng, (K, Y, X, C)), H.rand_f16(rng, (K,))
    out, _ = run_conv(inp, wei, s, d, p, ck.AddRelu(), bias)
    ref = oracle.conv2d_fwd(inp, wei, s, d, p, epilogue=oracle.EPI_ADD_RELU, bias=bias)
    H.assert_close(out, ref)


@pytest.mark.parametrize("case", CASES[:4])
def test_conv2d_fwd_plain_integer_inputs_bit_exact(cuda_device, case):
    """DeviceConvNDFwd with PassThrough; FillUniformDistributionIntegerValue-style inputs
    (fill.hpp:50-63) make the result independent of the accumulation order."""
    N, C, Hi, Wi, K, Y, X, s, d, p = case
    rng = np.random.default_rng(11939)
    inp = rng.integers(-5, 6, (N, Hi, Wi, C)).astype(np.float16)
    wei = rng.integers(-5, 6, (K, Y, X, C)).astype(np.float16)
    out, _ = run_conv(inp, wei, s, d, p)
    ref = oracle.conv2d_fwd(inp, wei, s, d, p)
    np.testing.assert_array_equal(out.view(np.uint16), ref.view(np.uint16))


def test_conv2d_fwd_bias_relu_add_and_other_epilogues(cuda_device):
    N, C, Hi, Wi, K, Y, X, s, d, p = CASES[3]
    rng = np.random.default_rng(17)
    inp, wei, bias = H.rand_f16(rng, (N, Hi, Wi, C)), H.rand_f16(rng, (K, Y, X, C)), H.rand_f16(rng, (K,))
    ref0 = oracle.conv2d_fwd(inp, wei, s, d, p)
    resi = H.rand_f16(rng, ref0.shape)
    out, _ = run_conv(inp, wei, s, d, p, ck.AddReluAdd(), bias, resi)
    H.assert_close(out, oracle.conv2d_fwd(inp, wei, s, d, p, epilogue=oracle.EPI_ADD_RELU_ADD, bias=bias, resi=resi))
    out, _ = run_conv(inp, wei, s, d, p, ck.AddHardswish(), bias)
    H.assert_close(out, oracle.conv2d_fwd(inp, wei, s, d, p, epilogue=oracle.EPI_ADD_HARDSWISH, bias=bias))
    out, _ = run_conv(inp, wei, s, d, p, ck.Relu())
    H.assert_close(out, oracle.conv2d_fwd(inp, wei, s, d, p, epilogue=oracle.EPI_RELU))


def test_reference_golden_vectors_on_device(cuda_device):
    """The reference's golden cases (test/reference_conv_fwd/reference_conv_fwd.cpp:94-154) have
    C = 2; they run on the device with the channels zero-padded to 8 (zeros add nothing)."""
    golden = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_conv_fwd_2d.json")))
    for case in golden["conv_cases"]:
        g = case["geometry"]
        seq = np.arange(g["N"] * g["Hi"] * g["Wi"] * g["C"], dtype=np.float32).reshape(g["N"], g["Hi"], g["Wi"], g["C"])
        inp = np.zeros((g["N"], g["Hi"], g["Wi"], 8), np.float16)
        inp[..., :g["C"]] = seq
        Kp = 8
        wei = np.zeros((Kp, g["Y"], g["X"], 8), np.float16)
        wei[:g["K"], :, :, :g["C"]] = 0.5
        out, _ = run_conv(inp, wei, (g["s"],) * 2, (g["d"],) * 2, (g["p"],) * 2)
        want = np.array(case["expected"], np.float32).reshape(case["output_shape_nhwk"]).astype(np.float16)
        np.testing.assert_array_equal(out[..., :g["K"]], want)
        assert (out[..., g["K"]:] == 0).all()


def test_full_size_conv_bias_relu(cuda_device):
    """N128 C192 71x71 K256 3x3 s2 p1 (ConvParams default, conv_util.cpp:41-53): every output checked."""
    rng = np.random.default_rng(11939 + 4000)
    N, C, Hi, Wi, K = 128, 192, 71, 71, 256
    inp, wei, bias = H.rand_f16(rng, (N, Hi, Wi, C)), H.rand_f16(rng, (K, 3, 3, C)), H.rand_f16(rng, (K,))
    out, ms = run_conv(inp, wei, (2, 2), (1, 1), (1, 1), ck.AddRelu(), bias, time_kernel=True)
    assert out.shape == (128, 36, 36, 256) and ms > 0
    ref = oracle.conv2d_fwd(inp, wei, (2, 2), (1, 1), (1, 1), epilogue=oracle.EPI_ADD_RELU, bias=bias)
    H.assert_close(out, ref)


def test_batch_shards_compose(cuda_device):
    """Sharding the batch (the multi-GPU split) gives the same bytes as the whole batch."""
    rng = np.random.default_rng(31)
    inp, wei, bias = H.rand_f16(rng, (8, 15, 15, 64)), H.rand_f16(rng, (64, 3, 3, 64)), H.rand_f16(rng, (64,))
    whole, _ = run_conv(inp, wei, (2, 2), (1, 1), (1, 1), ck.AddRelu(), bias)
    parts = [run_conv(inp[i:i + 2], wei, (2, 2), (1, 1), (1, 1), ck.AddRelu(), bias)[0] for i in range(0, 8, 2)]
    np.testing.assert_array_equal(np.concatenate(parts).view(np.uint16), whole.view(np.uint16))


# int8 convolution (example/09_convnd_fwd/convnd_fwd_xdl_int8.cpp:23-26: int8 in / weights / out, int32 accumulate).
# N, C, Hi, Wi, K, Y, X, stride, dilation, pad — C is a multiple of 16 (16-byte pixel pitch)
CASES_I8 = [
    (4, 64, 36, 36, 256, 3, 3, (2, 2), (2, 2), (2, 2)),
    (2, 192, 15, 15, 256, 3, 3, (2, 2), (1, 1), (1, 1)),
    (3, 16, 11, 7, 48, 3, 2, (1, 1), (1, 1), (1, 1)),     # C far below one k block of 128 channels
    (2, 144, 9, 12, 40, 2, 3, (1, 2), (2, 1), (1, 2)),    # channel tail (144 = 128 + 16), K not a multiple of 16
]


def run_conv_i8(inp, wei, stride, dilation, pad, op):
    N, Hi, Wi, C = inp.shape
    K, Y, X, _ = wei.shape
    Ho = oracle.conv_out_len(Hi, Y, stride[0], dilation[0], pad[0], pad[0])
    Wo = oracle.conv_out_len(Wi, X, stride[1], dilation[1], pad[1], pad[1])
    di, dw = H.to_dev(inp), H.to_dev(wei)
    out = torch.full((N, Ho, Wo, K), -77, dtype=torch.int8, device="cuda")
    conv = ck.DeviceConvFwd(capi.CKB_I8)
    arg = conv.MakeArgument(di.data_ptr(), dw.data_ptr(), out.data_ptr(), N, K, C, (Hi, Wi), (Y, X), (Ho, Wo),
                            stride, dilation, pad, pad, None, None, op)
    assert conv.IsSupportedArgument(arg), capi.last_error()
    conv.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    return out.cpu().numpy()


@pytest.mark.parametrize("case", CASES_I8)
def test_conv2d_fwd_int8_bit_exact(cuda_device, case):
    N, C, Hi, Wi, K, Y, X, s, d, p = case
    rng = np.random.default_rng(N * 31 + C)
    inp = rng.integers(-5, 6, (N, Hi, Wi, C)).astype(np.int8)
    wei = rng.integers(-5, 6, (K, Y, X, C)).astype(np.int8)
    for op in (ck.RequantReluRequant(0.03, 1.0), ck.RequantReluRequantRne(0.03, 14.0), ck.Relu(), ck.PassThrough()):
        out = run_conv_i8(inp, wei, s, d, p, op)
        ref = oracle.conv2d_fwd(inp, wei, s, d, p, epilogue=op.kind, params=op.params)
        np.testing.assert_array_equal(out, ref)


def test_conv2d_fwd_int8_odd_channel_pitch_runs_through_the_padded_copy(cuda_device):
    """24 int8 channels are a 24-byte pixel pitch, which TMA cannot read in place."""
    rng = np.random.default_rng(77)
    inp = rng.integers(-5, 6, (2, 8, 8, 24)).astype(np.int8)
    wei = rng.integers(-5, 6, (32, 3, 3, 24)).astype(np.int8)
    out = run_conv_i8(inp, wei, (1, 1), (1, 1), (1, 1), ck.PassThrough())
    np.testing.assert_array_equal(out, oracle.conv2d_fwd(inp, wei, (1, 1), (1, 1), (1, 1)))
