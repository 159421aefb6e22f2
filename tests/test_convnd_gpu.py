"""GPU parity tests of the 1-D and 3-D forward convolution (the NumDimSpatial = 1 / 3 cases of
DeviceConvNDFwdXdl..., device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp:76) against the oracle.

Geometries are those of the reference's device tests (test/convnd_fwd/conv1d_fwd.cpp:73-94,
conv3d_fwd.cpp:76-98: ConvParams{nd, N, K, C, filter, input, strides, dilations, left pads, right pads}) with
FillUniformDistributionIntegerValue-style inputs, which make the result independent of the summation order, so the
comparison is bit for bit; the reference's golden vectors for its CPU operator run through the device as well."""
import json
import os

import numpy as np
import pytest
import torch

import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from oracle import ck_oracle as oracle

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x.view(np.int16) if x.dtype == np.uint16 else x)).cuda()


def run_convnd(inp, wei, stride, dilation, pad, op=None, bias=None, dtype=capi.CKB_F16):
    """inp (N, *spatial, C), wei (K, *filter, C) channels-last; returns (N, *out_spatial, K)."""
    op = op or ck.PassThrough()
    nd = inp.ndim - 2
    N, C, K = inp.shape[0], inp.shape[-1], wei.shape[0]
    in_sp, filt = inp.shape[1:-1], wei.shape[1:-1]
    out_sp = [oracle.conv_out_len(i, f, s, d, p, p) for i, f, s, d, p in zip(in_sp, filt, stride, dilation, pad)]
    di, dw = dev(inp), dev(wei)
    db = dev(bias) if bias is not None else None
    tdt = {capi.CKB_F16: torch.float16, capi.CKB_BF16: torch.int16, capi.CKB_I8: torch.int8}[dtype]
    out = torch.zeros((N, *out_sp, K), dtype=tdt, device="cuda")
    conv = ck.DeviceConvFwd(dtype)
    arg = conv.MakeArgument(di.data_ptr(), dw.data_ptr(), out.data_ptr(), N, K, C, in_sp, filt, out_sp, stride, dilation,
                            pad, pad, None, None, op, p_bias=db.data_ptr() if db is not None else None)
    assert conv.IsSupportedArgument(arg), capi.last_error()
    conv.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    res = out.cpu().numpy()
    assert len(nd * [0]) == nd
    return res.view(np.uint16) if dtype == capi.CKB_BF16 else res


def ints(rng, shape, dtype=np.float16):
    return rng.integers(-5, 6, shape).astype(dtype)


# N, K, C, filter, input, stride, dilation, pad
CASES_1D = [
    (4, 256, 64, (3,), (71,), (2,), (2,), (2,)),
    (4, 256, 64, (1,), (28,), (1,), (1,), (0,)),
    (4, 256, 64, (1,), (28,), (2,), (1,), (0,)),
    (4, 256, 64, (3,), (36,), (1,), (2,), (2,)),
    (3, 40, 24, (5,), (50,), (3,), (1,), (1,)),   # ragged K and C
]
CASES_3D = [
    (4, 256, 64, (3, 3, 3), (28, 28, 28), (2, 2, 2), (2, 2, 2), (2, 2, 2)),
    (4, 256, 64, (1, 1, 1), (28, 28, 28), (1, 1, 1), (1, 1, 1), (0, 0, 0)),
    (4, 256, 64, (1, 1, 1), (28, 28, 28), (2, 2, 2), (1, 1, 1), (0, 0, 0)),
    (4, 256, 64, (3, 3, 3), (18, 18, 18), (1, 1, 1), (2, 2, 2), (2, 2, 2)),
    (2, 40, 24, (2, 3, 1), (7, 9, 11), (1, 2, 3), (3, 1, 2), (1, 2, 0)),   # anisotropic everything, ragged K and C
]


@pytest.mark.parametrize("case", CASES_1D)
def test_conv1d_fwd_bit_exact(cuda_device, case):
    N, K, C, filt, in_sp, s, d, p = case
    rng = np.random.default_rng(sum(in_sp) + C)
    inp, wei = ints(rng, (N, *in_sp, C)), ints(rng, (K, *filt, C))
    out = run_convnd(inp, wei, s, d, p)
    ref = oracle.conv1d_fwd(inp, wei, s[0], d[0], p[0])
    np.testing.assert_array_equal(out.view(np.uint16), ref.view(np.uint16))


@pytest.mark.parametrize("case", CASES_3D)
def test_conv3d_fwd_bit_exact(cuda_device, case):
    N, K, C, filt, in_sp, s, d, p = case
    rng = np.random.default_rng(sum(in_sp) + C)
    inp, wei = ints(rng, (N, *in_sp, C)), ints(rng, (K, *filt, C))
    out = run_convnd(inp, wei, s, d, p)
    ref = oracle.conv3d_fwd(inp, wei, s, d, p)
    np.testing.assert_array_equal(out.view(np.uint16), ref.view(np.uint16))


def test_conv3d_fwd_bias_relu_real_inputs_and_other_types(cuda_device):
    N, K, C, filt, in_sp, s, d, p = CASES_3D[3]
    rng = np.random.default_rng(5)
    inp = rng.uniform(-1, 1, (N, *in_sp, C)).astype(np.float16)
    wei = rng.uniform(-1, 1, (K, *filt, C)).astype(np.float16)
    bias = rng.uniform(-1, 1, (K,)).astype(np.float16)
    out = run_convnd(inp, wei, s, d, p, ck.AddRelu(), bias)
    ref = oracle.conv3d_fwd(inp, wei, s, d, p, epilogue=oracle.EPI_ADD_RELU, bias=bias)
    bad, max_err = oracle.check_err(out, ref, 1e-3, 1e-3)
    assert bad == 0, (bad, max_err)
    # int8 (channel pitch 16 bytes) and bfloat16, integer inputs, bit for bit
    i8_in, i8_w = ints(rng, (2, 6, 7, 8, 32), np.int8), ints(rng, (48, 3, 2, 3, 32), np.int8)
    op = ck.RequantReluRequant(0.03, 1.0)
    out = run_convnd(i8_in, i8_w, (1, 1, 2), (1, 2, 1), (1, 1, 1), op, dtype=capi.CKB_I8)
    np.testing.assert_array_equal(out, oracle.conv3d_fwd(i8_in, i8_w, (1, 1, 2), (1, 2, 1), (1, 1, 1), epilogue=op.kind,
                                                         params=op.params))
    bf_in = oracle.to_bf16(ints(rng, (2, 6, 7, 8, 16), np.float32))
    bf_w = oracle.to_bf16(ints(rng, (24, 3, 3, 3, 16), np.float32))
    out = run_convnd(bf_in, bf_w, (1, 1, 1), (1, 1, 1), (1, 1, 1), dtype=capi.CKB_BF16)
    np.testing.assert_array_equal(out, oracle.conv3d_fwd(bf_in, bf_w, (1, 1, 1), (1, 1, 1), (1, 1, 1)))


def test_reference_golden_vectors_1d_3d_on_the_device(cuda_device):
    """The reference's golden vectors (2 input channels) with the channels zero-padded to 8 for the 16-byte pitch;
    the 3-D case with the 0.1-step input is compared within check_err's binary16 tolerance."""
    fx = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_conv_fwd_1d_3d.json")))
    for case in fx["cases"]:
        g = case["geometry"]
        nd, N, K, C, sp = g["nd"], g["N"], g["K"], g["C"], g["in_sp"]
        seq = np.arange(N * C * int(np.prod(sp)), dtype=np.float64) * case["input_step"]
        if nd == 1:
            logical = seq.reshape(N, sp[0], C)
        else:
            logical = seq.reshape(N, C, *sp).transpose(0, 2, 3, 4, 1)
        inp = np.zeros((*logical.shape[:-1], 8), dtype=np.float16)
        inp[..., :C] = logical.astype(np.float16)
        wei = np.zeros((K, *g["filt"], 8), dtype=np.float16)
        wei[..., :C] = 0.5
        out = run_convnd(inp, wei, g["stride"], g["dil"], g["pad"])
        order = (0, nd + 1, *range(1, nd + 1)) if case["output_order"].startswith("N,K") else tuple(range(nd + 2))
        got = out.transpose(order).ravel().astype(np.float64)
        # expected from the same binary16-rounded inputs (the fixture's values come from unrounded float inputs)
        exact = np.array(case["derived"])
        if np.array_equal(logical.astype(np.float16).astype(np.float64), logical):
            np.testing.assert_allclose(got, exact.astype(np.float16).astype(np.float64), rtol=0, atol=0)
        else:
            ref = oracle.conv3d_fwd(inp.reshape(N, *([1] * (3 - nd)), *sp, 8), wei.reshape(K, *([1] * (3 - nd)), *g["filt"], 8),
                                    tuple([1] * (3 - nd) + g["stride"]), tuple([1] * (3 - nd) + g["dil"]),
                                    tuple([0] * (3 - nd) + g["pad"]))
            np.testing.assert_array_equal(out.ravel().view(np.uint16), ref.ravel().view(np.uint16))
            np.testing.assert_allclose(got, exact, rtol=2e-3, atol=2e-3)


def test_convnd_limits_are_reported(cuda_device):
    conv = ck.DeviceConvFwd()
    # 5-D im2col maps take (filter - 1) * dilation <= 15
    arg = conv.MakeArgument(0x1000, 0x2000, 0x3000, 1, 8, 8, (40, 40, 40), (3, 3, 3), (22, 22, 22), (1, 1, 1), (9, 9, 9),
                            (0, 0, 0), (0, 0, 0))
    assert not conv.IsSupportedArgument(arg)
    assert "im2col" in capi.last_error()
    # inconsistent vector lengths
    arg = conv.MakeArgument(0x1000, 0x2000, 0x3000, 1, 8, 8, (40, 40), (3, 3, 3), (38, 38), (1, 1), (1, 1), (0, 0), (0, 0))
    assert not conv.IsSupportedArgument(arg)
