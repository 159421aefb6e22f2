"""GPU parity tests of the four A/B layout combinations of the reference's GEMM instances
(mk_nk, mk_kn, km_kn, km_nk: library/src/tensor_operation_instance/gpu/gemm/device_gemm_xdl_*_instance.cpp and
test/gemm/gemm_util.hpp:106-225, which runs every test type over Row/Col operands).

The logical problem is the same for every layout (A is M x K, B is K x N); only the memory order of the operands
changes, so each case is checked against the same oracle call.  Integer-valued inputs make the comparison bit-exact
for f16, bf16 and int8."""
import os

import numpy as np
import pytest
import torch

import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from oracle import ck_oracle as oracle

pytestmark = pytest.mark.gpu

ROW, COL = capi.CKB_ROW_MAJOR, capi.CKB_COL_MAJOR
LAYOUTS = [(ROW, COL), (ROW, ROW), (COL, ROW), (COL, COL)]  # mk_nk, mk_kn, km_kn, km_nk
NAMES = {(ROW, COL): "mk_nk", (ROW, ROW): "mk_kn", (COL, ROW): "km_kn", (COL, COL): "km_nk"}


def make_inputs(rng, dtype, M, N, K, kind="int"):
    """Logical A (M,K), B (K,N) in the numpy dtype the oracle expects."""
    if dtype == capi.CKB_I8:
        return rng.integers(-5, 6, (M, K)).astype(np.int8), rng.integers(-5, 6, (K, N)).astype(np.int8)
    if kind == "int":
        a, b = rng.integers(-5, 6, (M, K)).astype(np.float32), rng.integers(-5, 6, (K, N)).astype(np.float32)
    else:
        a, b = rng.uniform(-1, 1, (M, K)).astype(np.float32), rng.uniform(-1, 1, (K, N)).astype(np.float32)
    if dtype == capi.CKB_BF16:
        return oracle.to_bf16(a), oracle.to_bf16(b)
    return a.astype(np.float16), b.astype(np.float16)


def physical(x, col_major, pad):
    """Memory image of the logical matrix x (rows, cols) in the given order, with `pad` extra elements of
    pitch.  Returns (array whose buffer is the image, leading dimension)."""
    src = x.T if col_major else x
    buf = np.zeros((src.shape[0], src.shape[1] + pad), dtype=x.dtype)
    buf[:, :src.shape[1]] = src
    return buf, buf.shape[1]


def dev(x):
    if x.dtype == np.uint16:
        x = x.view(np.int16)
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def run_layout(dtype, a_layout, b_layout, a, b, pad_a=0, pad_b=0, op=None):
    M, K = a.shape
    N = b.shape[1]
    a_img, lda = physical(a, a_layout == COL, pad_a)
    b_img, ldb = physical(b, b_layout == COL, pad_b)
    da, db = dev(a_img), dev(b_img)
    tdt = {capi.CKB_I8: torch.int8, capi.CKB_F16: torch.float16, capi.CKB_BF16: torch.int16}[dtype]
    e = torch.zeros((M, N), dtype=tdt, device="cuda")
    gemm = ck.DeviceGemmMultipleD(dtype, a_layout, b_layout)
    arg = gemm.MakeArgument(da.data_ptr(), db.data_ptr(), [], e.data_ptr(), M, N, K, lda, ldb, [], N, None, None,
                            op or ck.PassThrough())
    assert gemm.IsSupportedArgument(arg), capi.last_error()
    gemm.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    out = e.cpu().numpy()
    return out.view(np.uint16) if dtype == capi.CKB_BF16 else out


@pytest.mark.parametrize("dtype", [capi.CKB_F16, capi.CKB_BF16, capi.CKB_I8], ids=["f16", "bf16", "i8"])
@pytest.mark.parametrize("layouts", LAYOUTS, ids=[NAMES[l] for l in LAYOUTS])
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (208, 144, 80), (400, 336, 272), (128, 64, 48)])
def test_gemm_layouts_small_bit_exact(cuda_device, dtype, layouts, M, N, K):
    """One CTA per tile, all three tile widths, ragged M, N and K (the leading dimensions stay multiples of
    16 bytes, as TMA requires)."""
    rng = np.random.default_rng(M * 7 + N * 3 + K + dtype)
    a, b = make_inputs(rng, dtype, M, N, K)
    out = run_layout(dtype, layouts[0], layouts[1], a, b, pad_a=16, pad_b=32)
    np.testing.assert_array_equal(out, oracle.gemm(a, b))


@pytest.mark.parametrize("dtype", [capi.CKB_F16, capi.CKB_I8], ids=["f16", "i8"])
@pytest.mark.parametrize("layouts", LAYOUTS, ids=[NAMES[l] for l in LAYOUTS])
def test_gemm_layouts_cta_pairs_with_tail(cuda_device, dtype, layouts):
    """Large enough for CTA pairs (256 x 256 tiles) with a partial last wave that is cut into column slices."""
    M, N, K = 2048, 2560, 512
    rng = np.random.default_rng(99 + dtype)
    a, b = make_inputs(rng, dtype, M, N, K)
    out = run_layout(dtype, layouts[0], layouts[1], a, b)
    np.testing.assert_array_equal(out, oracle.gemm(a, b))


@pytest.mark.parametrize("layouts", LAYOUTS, ids=[NAMES[l] for l in LAYOUTS])
def test_gemm_layouts_single_cta_wide_tile_with_tail(cuda_device, layouts):
    """The 128 x 256 single-CTA kernel (forced) with a split tail wave."""
    M, N, K = 1920, 2560, 256  # 15 x 10 = 150 tiles on 148 SMs: 2 tail tiles
    rng = np.random.default_rng(5)
    a, b = make_inputs(rng, capi.CKB_F16, M, N, K)
    os.environ["CKB_FORCE_CG"] = "1"
    try:
        out = run_layout(capi.CKB_F16, layouts[0], layouts[1], a, b)
    finally:
        del os.environ["CKB_FORCE_CG"]
    np.testing.assert_array_equal(out, oracle.gemm(a, b))


@pytest.mark.parametrize("layouts", LAYOUTS[1:], ids=[NAMES[l] for l in LAYOUTS[1:]])
def test_gemm_layouts_real_inputs_with_epilogue(cuda_device, layouts):
    M, N, K = 512, 384, 320
    rng = np.random.default_rng(17)
    a, b = make_inputs(rng, capi.CKB_F16, M, N, K, kind="real")
    op = ck.FastGelu()
    out = run_layout(capi.CKB_F16, layouts[0], layouts[1], a, b, op=op)
    ref = oracle.gemm(a, b, op.kind, op.params)
    bad, max_err = oracle.check_err(out, ref, 1e-3, 1e-3)
    assert bad == 0, (bad, max_err)


def test_leading_dimension_rules_follow_the_layout(cuda_device):
    gemm = ck.DeviceGemmMultipleD(capi.CKB_F16, COL, ROW)
    ok = gemm.MakeArgument(0x1000, 0x2000, [], 0x4000, 256, 512, 128, 256, 512, [], 512, None, None, ck.PassThrough())
    assert gemm.IsSupportedArgument(ok), capi.last_error()
    # column-major A needs lda >= M, row-major B needs ldb >= N
    bad = gemm.MakeArgument(0x1000, 0x2000, [], 0x4000, 256, 512, 128, 128, 512, [], 512, None, None, ck.PassThrough())
    assert not gemm.IsSupportedArgument(bad)
    bad = gemm.MakeArgument(0x1000, 0x2000, [], 0x4000, 256, 512, 128, 256, 128, [], 512, None, None, ck.PassThrough())
    assert not gemm.IsSupportedArgument(bad)


@pytest.mark.parametrize("layouts", LAYOUTS[1:], ids=[NAMES[l] for l in LAYOUTS[1:]])
def test_grouped_gemm_layouts(cuda_device, layouts):
    rng = np.random.default_rng(23)
    shapes = [(256, 128, 64), (200, 264, 136), (512, 384, 256)]
    keep, p_a, p_b, p_e, descs, refs, outs = [], [], [], [], [], [], []
    for M, N, K in shapes:
        a, b = make_inputs(rng, capi.CKB_F16, M, N, K)
        a_img, lda = physical(a, layouts[0] == COL, 8)
        b_img, ldb = physical(b, layouts[1] == COL, 8)
        da, db = dev(a_img), dev(b_img)
        e = torch.zeros((M, N), dtype=torch.float16, device="cuda")
        keep += [da, db]
        outs.append(e)
        p_a.append(da.data_ptr())
        p_b.append(db.data_ptr())
        p_e.append(e.data_ptr())
        descs.append(ck.GemmDescHost(M, N, K, lda, ldb, N, []))
        refs.append(oracle.gemm(a, b))
    op = ck.DeviceGroupedGemm(capi.CKB_F16, layouts[0], layouts[1])
    arg = op.MakeArgument(p_a, p_b, [[] for _ in shapes], p_e, descs, None, None, ck.PassThrough())
    ws = torch.empty(op.GetWorkSpaceSize(arg), dtype=torch.uint8, device="cuda")
    op.SetWorkSpacePointer(arg, ws.data_ptr())
    assert op.IsSupportedArgument(arg), capi.last_error()
    op.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    for e, ref in zip(outs, refs):
        np.testing.assert_array_equal(e.cpu().numpy(), ref)
