"""GPU parity tests of the problems TMA cannot read in place: GEMM operands whose pitch or base address is not a
multiple of 16 bytes (the reference serves them with its ScalarPerVector = 1 instances) and convolutions whose
channel count gives such a pixel pitch (ConvolutionForwardSpecialization::OddC,
device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp:921-933; the reference's test case is test/convnd_fwd/conv2d_fwd.cpp:110-111).
The library copies such operands into a padded, stream-ordered temporary and runs the same kernel; results must
match the oracle exactly as for aligned operands."""
import numpy as np
import pytest
import torch

import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from oracle import ck_oracle as oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu
ROW, COL = capi.CKB_ROW_MAJOR, capi.CKB_COL_MAJOR


def _gemm(a, b, a_layout, b_layout, dtype=capi.CKB_F16, offset_a=0, offset_b=0, time_kernel=False):
    """a: (M, K), b: (K, N) logical matrices; physical images packed in the given layouts, optionally starting
    `offset` elements into their buffers (a base address that is not 16-byte aligned)."""
    M, K = a.shape
    N = b.shape[1]
    a_img = np.ascontiguousarray(a.T if a_layout == COL else a)
    b_img = np.ascontiguousarray(b.T if b_layout == COL else b)

    def place(img, off):
        buf = torch.zeros(img.size + off + 16, dtype=torch.int8 if dtype == capi.CKB_I8 else torch.float16, device="cuda")
        buf[off:off + img.size] = torch.from_numpy(img.reshape(-1)).cuda()
        return buf, buf.data_ptr() + off * buf.element_size()
    abuf, pa = place(a_img, offset_a)
    bbuf, pb = place(b_img, offset_b)
    e = torch.full((M, N), -77 if dtype == capi.CKB_I8 else float("nan"),
                   dtype=torch.int8 if dtype == capi.CKB_I8 else torch.float16, device="cuda")
    g = ck.DeviceGemm(dtype, a_layout, b_layout)
    arg = g.MakeArgument(pa, pb, e.data_ptr(), M, N, K, a_img.shape[1], b_img.shape[1], N)
    assert g.IsSupportedArgument(arg), capi.last_error()
    ms = g.MakeInvoker().Run(arg, ck.StreamConfig(None, time_kernel))
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    return e.cpu().numpy(), ms


@pytest.mark.parametrize("layouts", [(ROW, COL), (ROW, ROW), (COL, ROW), (COL, COL)], ids=["mk_nk", "mk_kn", "km_kn", "km_nk"])
def test_gemm_with_odd_pitches_bit_exact(cuda_device, layouts):
    """K = 1001 with lda = ldb = 1001 for the K-contiguous operands; M = 515 / N = 333 as the pitch of the others."""
    rng = np.random.default_rng(1001)
    M, N, K = 515, 333, 1001
    a = rng.integers(-5, 6, (M, K)).astype(np.float16)
    b = rng.integers(-5, 6, (K, N)).astype(np.float16)
    out, _ = _gemm(a, b, *layouts)
    np.testing.assert_array_equal(out.view(np.uint16), oracle.gemm(a, b).view(np.uint16))


def test_gemm_odd_pitch_real_inputs_timed_and_int8(cuda_device):
    rng = np.random.default_rng(5)
    M, N, K = 1000, 1200, 1001
    a = rng.uniform(-1, 1, (M, K)).astype(np.float16)
    b = rng.uniform(-1, 1, (K, N)).astype(np.float16)
    out, ms = _gemm(a, b, ROW, COL, time_kernel=True)  # the copy runs in every timed repetition
    assert ms > 0
    H.assert_close(out, oracle.gemm(a, b))
    a8 = rng.integers(-5, 6, (300, 1001)).astype(np.int8)
    b8 = rng.integers(-5, 6, (1001, 200)).astype(np.int8)
    out8, _ = _gemm(a8, b8, ROW, COL, dtype=capi.CKB_I8)
    np.testing.assert_array_equal(out8, oracle.gemm(a8, b8))


def test_gemm_with_unaligned_base_addresses(cuda_device):
    """Aligned pitches, but A starts 2 and B 6 bytes off a 16-byte boundary."""
    rng = np.random.default_rng(9)
    M, N, K = 256, 384, 512
    a = rng.integers(-5, 6, (M, K)).astype(np.float16)
    b = rng.integers(-5, 6, (K, N)).astype(np.float16)
    out, _ = _gemm(a, b, ROW, COL, offset_a=1, offset_b=3)
    np.testing.assert_array_equal(out.view(np.uint16), oracle.gemm(a, b).view(np.uint16))


def _conv(inp, wei, stride, dilation, pad, op=None, bias=None):
    op = op or ck.PassThrough()
    N, Hi, Wi, C = inp.shape
    K, Y, X, _ = wei.shape
    Ho = oracle.conv_out_len(Hi, Y, stride[0], dilation[0], pad[0], pad[0])
    Wo = oracle.conv_out_len(Wi, X, stride[1], dilation[1], pad[1], pad[1])
    di, dw = H.to_dev(inp), H.to_dev(wei)
    db = H.to_dev(bias) if bias is not None else None
    out = torch.full((N, Ho, Wo, K), float("nan"), dtype=torch.float16, device="cuda")
    conv = ck.DeviceConvFwd()
    arg = conv.MakeArgument(di.data_ptr(), dw.data_ptr(), out.data_ptr(), N, K, C, (Hi, Wi), (Y, X), (Ho, Wo),
                            stride, dilation, pad, pad, None, None, op, p_bias=db.data_ptr() if db is not None else None)
    assert conv.IsSupportedArgument(arg), capi.last_error()
    conv.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    return out.cpu().numpy()


def test_reference_odd_c_case(cuda_device):
    """params_oddC_ of test/convnd_fwd/conv2d_fwd.cpp:110-111: N 4, K 256, C 3, 3x3 filter, 28x28 image, stride 1,
    dilation 1, no padding - with the integer values the reference's test uses (bit exact) and with real values."""
    rng = np.random.default_rng(3)
    inp = rng.integers(-5, 6, (4, 28, 28, 3)).astype(np.float16)
    wei = rng.integers(-5, 6, (256, 3, 3, 3)).astype(np.float16)
    out = _conv(inp, wei, (1, 1), (1, 1), (0, 0))
    np.testing.assert_array_equal(out.view(np.uint16), oracle.conv2d_fwd(inp, wei, (1, 1), (1, 1), (0, 0)).view(np.uint16))
    inp, wei, bias = H.rand_f16(rng, (4, 28, 28, 3)), H.rand_f16(rng, (256, 3, 3, 3)), H.rand_f16(rng, (256,))
    out = _conv(inp, wei, (1, 1), (1, 1), (0, 0), ck.AddRelu(), bias)
    H.assert_close(out, oracle.conv2d_fwd(inp, wei, (1, 1), (1, 1), (0, 0), epilogue=oracle.EPI_ADD_RELU, bias=bias))


@pytest.mark.parametrize("C", [1, 5, 12, 67, 100])
def test_conv_channel_counts_that_are_not_multiples_of_eight(cuda_device, C):
    rng = np.random.default_rng(C)
    inp = rng.integers(-3, 4, (3, 13, 10, C)).astype(np.float16)
    wei = rng.integers(-3, 4, (40, 3, 2, C)).astype(np.float16)
    out = _conv(inp, wei, (2, 1), (1, 2), (1, 1))
    np.testing.assert_array_equal(out.view(np.uint16), oracle.conv2d_fwd(inp, wei, (2, 1), (1, 2), (1, 1)).view(np.uint16))
