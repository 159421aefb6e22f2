"""Seeded random GEMM problems against the oracle: shapes, layouts, operand types and epilogues drawn at random, so that
tile widths, CTA pairs, both tail plans, ragged edges and the staged / element-wise store paths meet in combinations the
hand-written cases do not list.  Integer-valued inputs: bit-exact for PassThrough / Relu / int8 functors; FastGelu and
Scale within the reference's check_err tolerance."""
import numpy as np
import pytest
import torch

import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from oracle import ck_oracle as oracle

pytestmark = pytest.mark.gpu

ROW, COL = capi.CKB_ROW_MAJOR, capi.CKB_COL_MAJOR


def draw_case(rng, big):
    dtype = [capi.CKB_F16, capi.CKB_BF16, capi.CKB_I8][rng.integers(0, 3)]
    per16 = 16 if dtype == capi.CKB_I8 else 8
    if big:
        M, N = int(rng.integers(1500, 4200)), int(rng.integers(1500, 4200))
        K = int(rng.integers(4, 40)) * 16
    else:
        M, N = int(rng.integers(1, 700)), int(rng.integers(1, 700))
        K = int(rng.integers(1, 40)) * 16
    a_layout, b_layout = [ROW, COL][rng.integers(0, 2)], [ROW, COL][rng.integers(0, 2)]
    # leading dimensions: the contiguous extent rounded up to 16 bytes, sometimes padded further
    def ld(extent):
        return (extent + per16 - 1) // per16 * per16 + per16 * int(rng.integers(0, 3))
    lda = ld(K if a_layout == ROW else M)
    ldb = ld(K if b_layout == COL else N)
    lde = N if rng.integers(0, 2) else ld(N)  # N itself may be unaligned: element-wise stores
    if dtype == capi.CKB_I8:
        op = [ck.PassThrough(), ck.Relu(), ck.RequantReluRequant(0.03, 1.0), ck.RequantReluRequantRne(0.03, 14.0)][
            rng.integers(0, 4)]
    else:
        op = [ck.PassThrough(), ck.Relu(), ck.Scale(0.5), ck.FastGelu()][rng.integers(0, 4)]
    return dtype, M, N, K, a_layout, b_layout, lda, ldb, lde, op


def run_case(rng, case):
    dtype, M, N, K, a_layout, b_layout, lda, ldb, lde, op = case
    if dtype == capi.CKB_I8:
        a, b = rng.integers(-5, 6, (M, K)).astype(np.int8), rng.integers(-5, 6, (K, N)).astype(np.int8)
    else:
        a, b = rng.integers(-5, 6, (M, K)).astype(np.float32), rng.integers(-5, 6, (K, N)).astype(np.float32)
        if dtype == capi.CKB_BF16:
            a, b = oracle.to_bf16(a), oracle.to_bf16(b)
        else:
            a, b = a.astype(np.float16), b.astype(np.float16)

    def image(x, col_major, ldim):
        src = x.T if col_major else x
        buf = np.zeros((src.shape[0], ldim), dtype=x.dtype)
        buf[:, :src.shape[1]] = src
        return torch.from_numpy(buf.view(np.int16) if buf.dtype == np.uint16 else buf).cuda()

    da, db = image(a, a_layout == COL, lda), image(b, b_layout == COL, ldb)
    tdt = {capi.CKB_I8: torch.int8, capi.CKB_F16: torch.float16, capi.CKB_BF16: torch.int16}[dtype]
    e = torch.zeros((M, lde), dtype=tdt, device="cuda")
    gemm = ck.DeviceGemm(dtype, a_layout, b_layout)
    arg = gemm.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), M, N, K, lda, ldb, lde, None, None, op)
    assert gemm.IsSupportedArgument(arg), capi.last_error()
    gemm.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    out = e.cpu().numpy()[:, :N]
    out = out.view(np.uint16) if dtype == capi.CKB_BF16 else out
    ref = oracle.gemm(a, b, op.kind, op.params)
    exact = dtype == capi.CKB_I8 or op.kind in (capi.CKB_EPI_PASSTHROUGH, capi.CKB_EPI_RELU)
    if exact:
        np.testing.assert_array_equal(out, ref, err_msg=str(case[:9]))
    elif dtype == capi.CKB_BF16:
        o, r = oracle.from_bf16(out), oracle.from_bf16(ref)
        assert np.all(np.abs(o - r) <= np.abs(r) * 2.0 ** -7 + 1e-3), case[:9]
    else:
        bad, max_err = oracle.check_err(np.ascontiguousarray(out), ref, 1e-3, 1e-3)
        assert bad == 0, (case[:9], bad, max_err)


@pytest.mark.parametrize("seed", range(60))
def test_random_small_gemm(cuda_device, seed):
    rng = np.random.default_rng(1000 + seed)
    run_case(rng, draw_case(rng, big=False))


@pytest.mark.parametrize("seed", range(12))
def test_random_large_gemm(cuda_device, seed):
    rng = np.random.default_rng(5000 + seed)
    run_case(rng, draw_case(rng, big=True))


@pytest.mark.parametrize("seed", range(30))
def test_random_convolution(cuda_device, seed):
    """Random 1-D / 2-D / 3-D channels-last convolutions (f16 / bf16 / int8), PassThrough, integer inputs: bit exact."""
    rng = np.random.default_rng(9000 + seed)
    nd = int(rng.integers(1, 4))
    dtype = [capi.CKB_F16, capi.CKB_BF16, capi.CKB_I8][rng.integers(0, 3)]
    cmul = 16 if dtype == capi.CKB_I8 else 8
    N, C, K = int(rng.integers(1, 5)), cmul * int(rng.integers(1, 14)), int(rng.integers(1, 70))
    filt = [int(rng.integers(1, 4)) for _ in range(nd)]
    dil = [int(rng.integers(1, 4)) for _ in range(nd)]
    stride = [int(rng.integers(1, 4)) for _ in range(nd)]
    pad = [int(rng.integers(0, 3)) for _ in range(nd)]
    in_sp = [int(rng.integers((f - 1) * d + 1, (f - 1) * d + 1 + (14 if nd < 3 else 8))) for f, d in zip(filt, dil)]
    out_sp = [oracle.conv_out_len(i, f, s, d, p, p) for i, f, s, d, p in zip(in_sp, filt, stride, dil, pad)]
    np_dt = np.int8 if dtype == capi.CKB_I8 else np.float32
    inp = rng.integers(-4, 5, (N, *in_sp, C)).astype(np_dt)
    wei = rng.integers(-4, 5, (K, *filt, C)).astype(np_dt)
    if dtype == capi.CKB_BF16:
        inp, wei = oracle.to_bf16(inp), oracle.to_bf16(wei)
    elif dtype == capi.CKB_F16:
        inp, wei = inp.astype(np.float16), wei.astype(np.float16)
    view = (lambda x: x.view(np.int16)) if dtype == capi.CKB_BF16 else (lambda x: x)
    di, dw = torch.from_numpy(view(inp)).cuda(), torch.from_numpy(view(wei)).cuda()
    tdt = {capi.CKB_I8: torch.int8, capi.CKB_F16: torch.float16, capi.CKB_BF16: torch.int16}[dtype]
    out = torch.zeros((N, *out_sp, K), dtype=tdt, device="cuda")
    conv = ck.DeviceConvFwd(dtype)
    arg = conv.MakeArgument(di.data_ptr(), dw.data_ptr(), out.data_ptr(), N, K, C, in_sp, filt, out_sp, stride, dil, pad,
                            pad)
    assert conv.IsSupportedArgument(arg), capi.last_error()
    conv.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    res = out.cpu().numpy()
    res = res.view(np.uint16) if dtype == capi.CKB_BF16 else res
    lead = [1] * (3 - nd)
    ref = oracle.conv3d_fwd(inp.reshape(N, *lead, *in_sp, C), wei.reshape(K, *lead, *filt, C), tuple(lead + stride),
                            tuple(lead + dil), tuple([0] * (3 - nd) + pad))
    np.testing.assert_array_equal(res.reshape(ref.shape), ref, err_msg=str((nd, dtype, N, C, K, filt, in_sp, stride, dil, pad)))
