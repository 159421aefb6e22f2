"""CPU tests that pin the oracle (oracle/) to the reference's golden vectors and to
hand-derived known answers.  No GPU needed."""
import json
import os

import numpy as np
import pytest

from oracle import ck_oracle as oracle

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_conv_fwd_2d.json")


def _golden():
    with open(GOLDEN) as f:
        return json.load(f)


@pytest.mark.parametrize("idx", [0, 1])
def test_conv_matches_reference_golden_vectors(idx):
    """test/reference_conv_fwd/reference_conv_fwd.cpp:94-154 (float tensors, exact compare)."""
    case = _golden()["conv_cases"][idx]
    g = case["geometry"]
    inp = np.arange(g["N"] * g["Hi"] * g["Wi"] * g["C"], dtype=np.float32).reshape(g["N"], g["Hi"], g["Wi"], g["C"])
    wei = np.full((g["K"], g["Y"], g["X"], g["C"]), 0.5, dtype=np.float32)
    out = oracle.conv2d_fwd_f32(inp, wei, (g["s"],) * 2, (g["d"],) * 2, (g["p"],) * 2)
    assert list(out.shape) == case["output_shape_nhwk"]
    np.testing.assert_array_equal(out.ravel(), np.array(case["expected"], dtype=np.float32))


def test_conv_f16_paths_match_golden_case1():
    """Case 1 fits binary16 exactly (max 508.5), so the f16 naive and blocked forms must hit it too."""
    case = _golden()["conv_cases"][0]
    g = case["geometry"]
    inp = np.arange(72, dtype=np.float32).reshape(1, 6, 6, 2).astype(np.float16)
    wei = np.full((1, 3, 3, 2), 0.5, dtype=np.float16)
    for fast in (False, True):
        out = oracle.conv2d_fwd(inp, wei, fast=fast)
        np.testing.assert_array_equal(out.astype(np.float32).ravel(), np.array(case["expected"], np.float32))


def test_conv_output_length_table():
    """test/conv_util/conv_util.cpp:43-79."""
    for c in _golden()["output_length_cases"]:
        assert oracle.conv_out_len(*c["args"]) == c["expected"]


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (7, 5, 3), (65, 33, 130), (130, 70, 257)])
def test_gemm_integer_inputs_exact(M, N, K):
    """Integer-valued f16 inputs: every product and partial sum is an integer below 2^24, so the
    float accumulation equals exact integer arithmetic (independent numpy int64 matmul)."""
    rng = np.random.default_rng(M * 1000 + N)
    a = rng.integers(-5, 6, (M, K))
    bt = rng.integers(-5, 6, (N, K))
    expect = (a.astype(np.int64) @ bt.T.astype(np.int64)).astype(np.float16)
    for fast in (False, True):
        e = oracle.gemm(a.astype(np.float16), bt.astype(np.float16).T, fast=fast)
        np.testing.assert_array_equal(e, expect)
    e8 = oracle.gemm(a.astype(np.int8), bt.astype(np.int8).T, fast=True)
    np.testing.assert_array_equal(e8, (a @ bt.T).astype(np.int8))


@pytest.mark.parametrize("seed", range(4))
def test_blocked_form_is_bit_identical_to_naive(seed):
    rng = np.random.default_rng(seed)
    M, N, K = rng.integers(1, 90), rng.integers(1, 70), rng.integers(1, 600)
    a = rng.uniform(-1, 1, (M, K)).astype(np.float16)
    bt = rng.uniform(-1, 1, (N, K)).astype(np.float16)
    d0 = np.broadcast_to(rng.uniform(-1, 1, (N,)).astype(np.float16), (M, N))
    d1 = rng.uniform(-1, 1, (M, N)).astype(np.float16)
    for epi, dd0, dd1 in [(oracle.EPI_PASSTHROUGH, None, None), (oracle.EPI_ADD_ADD_FASTGELU, d0, d1),
                          (oracle.EPI_ADD, d0, None)]:
        e1 = oracle.gemm(a, bt.T, epi, None, dd0, dd1, fast=False)
        e2 = oracle.gemm(a, bt.T, epi, None, dd0, dd1, fast=True)
        np.testing.assert_array_equal(e1.view(np.uint16), e2.view(np.uint16))
    # convolution with stride / dilation / padding
    N_, C, Hi, Wi, Kc = 2, 8, 9, 7, 5
    inp = rng.uniform(-1, 1, (N_, Hi, Wi, C)).astype(np.float16)
    wei = rng.uniform(-1, 1, (Kc, 3, 2, C)).astype(np.float16)
    bias = rng.uniform(-1, 1, (Kc,)).astype(np.float16)
    kw = dict(stride=(2, 1), dilation=(1, 2), pad=(1, 2), epilogue=oracle.EPI_ADD_RELU, bias=bias)
    o1 = oracle.conv2d_fwd(inp, wei, fast=False, **kw)
    o2 = oracle.conv2d_fwd(inp, wei, fast=True, **kw)
    np.testing.assert_array_equal(o1.view(np.uint16), o2.view(np.uint16))


def test_requant_functors_known_answers():
    """example/14...int8.cpp:29-35 + truncating store; and the round-to-nearest-even variant."""
    p = (0.03, 1.0)
    f32 = np.float32
    for acc, want in [(100, 3), (50, 1), (-40, 0), (5000, 127), (33, 0), (34, 1)]:
        y = f32(p[1]) * max(f32(p[0]) * f32(acc), f32(0))
        assert oracle.epilogue_i8(oracle.EPI_REQUANT_RELU_REQUANT, p, acc) == int(np.trunc(min(max(y, -128), 127)))
        assert oracle.epilogue_i8(oracle.EPI_REQUANT_RELU_REQUANT, p, acc) == want
    p = (0.03, 14.0)
    # rne(0.03*50=1.5)=2 -> 28 ; rne(0.03*83=2.49)=2 -> 28 ; rne(0.03*84=2.52)=3 -> 42 ; ties to even: 0.03*... ;
    for acc, want in [(50, 28), (83, 28), (84, 42), (-50, 0), (1000, 127), (0, 0), (16, 0), (17, 14)]:
        assert oracle.epilogue_i8(oracle.EPI_REQUANT_RELU_REQUANT_RNE, p, acc) == want
    # PassThrough keeps the low 8 bits of the int32 accumulator (static_cast<int8_t>)
    assert oracle.epilogue_i8(oracle.EPI_PASSTHROUGH, None, 300) == 44
    assert oracle.epilogue_i8(oracle.EPI_PASSTHROUGH, None, -3) == -3


def test_f16_functors_known_answers():
    h = np.float16
    # Add<half,float,half>: half(c) + d0 in binary16 (binary_element_wise_operation.hpp:31-36):
    # 2049.0f -> 2048h; 2048h + 1h = 2049 -> ties-to-even 2048h.  (A float add would give 2050.)
    assert oracle.epilogue_f16(oracle.EPI_ADD, None, 2049.0, 1.0) == h(2048)
    assert oracle.epilogue_f16(oracle.EPI_ADD_RELU_F16, None, -3.0, 1.0) == h(0)
    assert oracle.epilogue_f16(oracle.EPI_ADD_RELU_F16, None, 3.0, 1.0) == h(4)
    # fp32 AddRelu with a single rounding: 2049 + 1 = 2050 exactly representable
    assert oracle.epilogue_f16(oracle.EPI_ADD_RELU, None, 2049.0, 1.0) == h(2050)
    assert oracle.epilogue_f16(oracle.EPI_BILINEAR, (0.5, 2.0), 3.0, 1.5) == h(4.5)
    assert oracle.epilogue_f16(oracle.EPI_ADD_RELU_ADD, None, -2.0, 1.0, 0.25) == h(0.25)
    assert oracle.epilogue_f16(oracle.EPI_SCALE, (0.25,), 10.0) == h(2.5)
    assert oracle.epilogue_f16(oracle.EPI_RELU, None, -1.0) == h(0)
    # FastGelu / AddAddFastGelu against the formula in float64 (element_wise_operation.hpp:127-133)
    for x in (-3.0, -0.5, 0.0, 0.7, 2.0, 6.0):
        u = 2 * x * (0.035677 * x * x + 0.797885)
        ref = x * (0.5 + 0.5 * (2 / (1 + np.exp(-u)) - 1))
        got = float(oracle.epilogue_f16(oracle.EPI_FASTGELU, None, x))
        assert abs(got - ref) <= 1e-3 * abs(ref) + 1e-3
        got2 = float(oracle.epilogue_f16(oracle.EPI_ADD_ADD_FASTGELU, None, x - 0.75, 0.5, 0.25))
        assert abs(got2 - ref) <= 1e-3 * abs(ref) + 1e-3
    # AddHardswish: a = 1+1 = 2, b = 5 -> 5*2*0.166667
    got = float(oracle.epilogue_f16(oracle.EPI_ADD_HARDSWISH, None, 1.0, 1.0))
    assert abs(got - 5 * 2 * 0.166667) < 2e-3


def test_check_err_rule():
    """check_err.hpp:107-148: an element fails when |o-r| > atol + rtol*|r| or is not finite."""
    ref = np.array([1.0, 100.0, 0.0, 5.0], dtype=np.float16)
    ok = np.array([1.001, 100.06, 0.0009, 5.0], dtype=np.float16)
    assert oracle.check_err(ok, ref)[0] == 0
    bad = np.array([1.01, 100.0, 0.0, np.inf], dtype=np.float16)
    assert oracle.check_err(bad, ref)[0] == 2
    assert oracle.check_err(np.array([1, 2], np.int8), np.array([1, 3], np.int8)) == (1, 1)


def test_conv_bias_relu_against_direct_numpy():
    """ReferenceConvFwd_Bias_Activation (reference_conv_fwd_bias_activation.hpp:74-128) against an
    independent numpy evaluation in float64 (tolerance of the f16 check rule)."""
    rng = np.random.default_rng(5)
    N, C, Hi, Wi, K, Y, X, s, p = 2, 8, 7, 7, 6, 3, 3, 2, 1
    inp = rng.uniform(-1, 1, (N, Hi, Wi, C)).astype(np.float16)
    wei = rng.uniform(-1, 1, (K, Y, X, C)).astype(np.float16)
    bias = rng.uniform(-1, 1, (K,)).astype(np.float16)
    out = oracle.conv2d_fwd(inp, wei, (s, s), (1, 1), (p, p), epilogue=oracle.EPI_ADD_RELU, bias=bias)
    Ho = Wo = (Hi + 2 * p - Y) // s + 1
    pad = np.zeros((N, Hi + 2 * p, Wi + 2 * p, C))
    pad[:, p:p + Hi, p:p + Wi] = inp
    ref = np.zeros((N, Ho, Wo, K))
    for ho in range(Ho):
        for wo in range(Wo):
            win = pad[:, ho * s:ho * s + Y, wo * s:wo * s + X, :]
            ref[:, ho, wo, :] = np.einsum("nyxc,kyxc->nk", win, wei.astype(np.float64))
    ref = np.maximum(ref + bias.astype(np.float64), 0)
    assert np.all(np.abs(out.astype(np.float64) - ref) <= 1e-3 + 1e-3 * np.abs(ref))


def test_bf16_conversion_known_answers():
    """type_convert<bhalf_t>(float), include/ck/utility/data_type.hpp:953-990: round to nearest even."""
    f = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.140625, 0.0], dtype=np.float32)
    b = oracle.to_bf16(f)
    # 1.00390625 = 1 + 2^-8 is a tie between 1.0 (even mantissa) and 1.0078125 -> 1.0;
    # 1.01171875 = 1 + 3*2^-8 is a tie between 1.0078125 (odd) and 1.015625 (even) -> 1.015625
    np.testing.assert_array_equal(oracle.from_bf16(b), np.array([1.0, 1.0, 1.015625, -2.5, 3.140625, 0.0], np.float32))
    assert b[0] == 0x3F80 and b[3] == 0xC020


def test_bf16_gemm_blocked_equals_naive_and_integer_exact():
    rng = np.random.default_rng(12)
    M, N, K = 37, 29, 150
    a = rng.integers(-5, 6, (M, K)).astype(np.float32)
    bt = rng.integers(-5, 6, (N, K)).astype(np.float32)
    e1 = oracle.gemm(oracle.to_bf16(a), oracle.to_bf16(bt).T, fast=False)
    e2 = oracle.gemm(oracle.to_bf16(a), oracle.to_bf16(bt).T, fast=True)
    np.testing.assert_array_equal(e1, e2)
    np.testing.assert_array_equal(e1, oracle.to_bf16((a @ bt.T).astype(np.float32)))
    ar = oracle.to_bf16(rng.uniform(-1, 1, (M, K)).astype(np.float32))
    br = oracle.to_bf16(rng.uniform(-1, 1, (N, K)).astype(np.float32))
    d0 = np.broadcast_to(oracle.to_bf16(rng.uniform(-1, 1, (N,)).astype(np.float32)), (M, N))
    for epi, d in [(oracle.EPI_FASTGELU, None), (oracle.EPI_ADD_RELU, d0)]:
        np.testing.assert_array_equal(oracle.gemm(ar, br.T, epi, None, d, fast=False),
                                      oracle.gemm(ar, br.T, epi, None, d, fast=True))


def test_int8_conv_matches_exact_integer_arithmetic():
    """int8 convolution of the oracle (int32-exact sum, static_cast<int8_t> store) against numpy int64 arithmetic."""
    rng = np.random.default_rng(0)
    inp = rng.integers(-5, 6, (2, 5, 6, 16)).astype(np.int8)
    wei = rng.integers(-5, 6, (8, 3, 3, 16)).astype(np.int8)
    out = oracle.conv2d_fwd(inp, wei, (1, 1), (1, 1), (1, 1), epilogue=oracle.EPI_PASSTHROUGH)
    padded = np.zeros((2, 7, 8, 16), dtype=np.int64)
    padded[:, 1:6, 1:7, :] = inp
    ref = np.zeros((2, 5, 6, 8), dtype=np.int64)
    for y in range(3):
        for x in range(3):
            ref += np.einsum("nhwc,kc->nhwk", padded[:, y:y + 5, x:x + 6, :], wei[:, y, x, :].astype(np.int64))
    np.testing.assert_array_equal(out, ref.astype(np.int8))  # low 8 bits, as static_cast<int8_t>(int32)
    relu = oracle.conv2d_fwd(inp, wei, (1, 1), (1, 1), (1, 1), epilogue=oracle.EPI_REQUANT_RELU_REQUANT,
                             params=[0.03, 1.0])
    expect = np.clip(np.trunc(np.float32(1.0) * np.maximum(np.float32(0.03) * ref.astype(np.float32), 0)), -128, 127)
    np.testing.assert_array_equal(relu, expect.astype(np.int8))


def test_reference_conv_1d_3d_golden_vectors():
    """The reference's own golden vectors for its 1-D and 3-D CPU convolution
    (tests/golden/reference_conv_fwd_1d_3d.json, made by tests/golden/make_convnd_golden.py)."""
    import json
    import os
    fx = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_conv_fwd_1d_3d.json")))
    assert len(fx["cases"]) == 4
    for case in fx["cases"]:
        g = case["geometry"]
        nd, N, K, C = g["nd"], g["N"], g["K"], g["C"]
        sp = g["in_sp"]
        step = np.float32(case["input_step"])
        count = N * C * int(np.prod(sp))
        seq = (np.arange(count, dtype=np.float32) * step).astype(np.float32)
        if nd == 1:  # NWC in memory
            inp = seq.reshape(N, sp[0], C)
            wei = np.full((K, g["filt"][0], C), 0.5, np.float32)
            out = oracle.conv1d_fwd(inp, wei, g["stride"][0], g["dil"][0], g["pad"][0])
            got = out.ravel()  # N, W, K order
        else:        # NCDHW in memory -> the oracle's NDHWC
            inp = np.ascontiguousarray(seq.reshape(N, C, *sp).transpose(0, 2, 3, 4, 1))
            wei = np.full((K, *g["filt"], C), 0.5, np.float32)
            out = oracle.conv3d_fwd(inp, wei, tuple(g["stride"]), tuple(g["dil"]), tuple(g["pad"]))
            got = out.transpose(0, 4, 1, 2, 3).ravel()  # N, K, D, H, W order
        assert list(out.shape[1:1 + nd]) == case["output_spatial"]
        np.testing.assert_allclose(got, np.array(case["expected"], np.float32), rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(got, np.array(case["derived"]), rtol=1e-5, atol=1e-6)
