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


def draw_case(rng, big, wide=False):
    """wide: also draw what the plain cases leave at their defaults - any K, leading dimensions that are not multiples
    of 16 bytes (the padded-copy path), a pinned tile configuration or a named K batch, and long K with few tiles."""
    dtype = [capi.CKB_F16, capi.CKB_BF16, capi.CKB_I8][rng.integers(0, 3)]
    per16 = 16 if dtype == capi.CKB_I8 else 8
    if big:
        M, N = int(rng.integers(1500, 4200)), int(rng.integers(1500, 4200))
        K = int(rng.integers(4, 40)) * 16
    else:
        M, N = int(rng.integers(1, 700)), int(rng.integers(1, 700))
        K = int(rng.integers(1, 40)) * 16
    if wide:
        K = int(rng.integers(1, 3000)) if rng.integers(0, 2) else int(rng.integers(64, 160)) * 64
        if K > 3000:
            M, N = int(rng.integers(1, 600)), int(rng.integers(1, 600))
    a_layout, b_layout = [ROW, COL][rng.integers(0, 2)], [ROW, COL][rng.integers(0, 2)]
    # leading dimensions: the contiguous extent rounded up to 16 bytes, sometimes padded further
    def ld(extent):
        if wide and rng.integers(0, 2):
            return extent + int(rng.integers(0, 2 * per16))  # any pitch
        return (extent + per16 - 1) // per16 * per16 + per16 * int(rng.integers(0, 3))
    lda = ld(K if a_layout == ROW else M)
    ldb = ld(K if b_layout == COL else N)
    lde = N if rng.integers(0, 2) else ld(N)  # N itself may be unaligned: element-wise stores
    if dtype == capi.CKB_I8:
        op = [ck.PassThrough(), ck.Relu(), ck.RequantReluRequant(0.03, 1.0), ck.RequantReluRequantRne(0.03, 14.0)][
            rng.integers(0, 4)]
    else:
        op = [ck.PassThrough(), ck.Relu(), ck.Scale(0.5), ck.FastGelu()][rng.integers(0, 4)]
    tile = 0
    if wide:
        tile = [0, capi.tile_config(256, 2), capi.tile_config(256, 1), capi.tile_config(128, 1), capi.tile_config(64, 1),
                capi.tile_config(256, 2, 1), capi.tile_config(kbatch=2), capi.tile_config(kbatch=4), capi.tile_config(kbatch=8),
                capi.tile_config(128, 1, kbatch=4), capi.tile_config(64, 1, kbatch=2)][rng.integers(0, 11)]
    return dtype, M, N, K, a_layout, b_layout, lda, ldb, lde, op, tile


def run_case(rng, case):
    dtype, M, N, K, a_layout, b_layout, lda, ldb, lde, op, tile = case
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
    gemm = ck.DeviceGemm(dtype, a_layout, b_layout, tile_config=tile)
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
        np.testing.assert_array_equal(out, ref, err_msg=str(case[:9]) + " " + capi.last_plan())
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


@pytest.mark.parametrize("seed", range(24))
def test_random_gemm_around_one_wave_of_tiles(cuda_device, seed):
    """Half a wave to two waves of 128 x 256 / 256 x 256 tiles, where the plan for the partial wave matters: the
    library's choice, balanced K ranges on single CTAs and on pairs, pinned tiles, no K split - bit for bit."""
    rng = np.random.default_rng(9000 + seed)
    M = int(rng.choice([640, 768, 1024, 1280, 1408, 1536, 1792, 2048, 2304])) - int(rng.choice([0, 0, 1, 17, 100]))
    N = int(rng.choice([1024, 1536, 2048, 2560, 3072, 4096])) - int(rng.choice([0, 0, 8, 24, 200]))
    K = int(rng.choice([1024, 2048, 2368, 4096])) - int(rng.choice([0, 0, 8, 64]))
    tile = [0, capi.tile_config(256, 1, balanced=1), capi.tile_config(256, 2, balanced=1), capi.tile_config(128, 1, balanced=1),
            capi.tile_config(256, 2), capi.tile_config(256, 1), capi.tile_config(no_ksplit=1), 0][rng.integers(0, 8)]
    dtype = [capi.CKB_F16, capi.CKB_BF16][rng.integers(0, 2)]
    op = [ck.PassThrough(), ck.Relu()][rng.integers(0, 2)]
    per16 = 8
    ld = lambda extent: (extent + per16 - 1) // per16 * per16
    run_case(rng, (dtype, M, N, K, ROW, COL, ld(K), ld(K), ld(N), op, tile))


@pytest.mark.parametrize("seed", range(80))
def test_random_gemm_any_pitch_tile_configuration_and_k_batch(cuda_device, seed):
    rng = np.random.default_rng(7000 + seed)
    run_case(rng, draw_case(rng, big=seed % 8 == 0, wide=True))


@pytest.mark.parametrize("seed", range(45))
def test_random_convolution(cuda_device, seed):
    """Random 1-D / 2-D / 3-D channels-last convolutions (f16 / bf16 / int8), PassThrough, integer inputs: bit exact."""
    rng = np.random.default_rng(9000 + seed)
    nd = int(rng.integers(1, 4))
    dtype = [capi.CKB_F16, capi.CKB_BF16, capi.CKB_I8][rng.integers(0, 3)]
    cmul = 16 if dtype == capi.CKB_I8 else 8
    N, C, K = int(rng.integers(1, 5)), cmul * int(rng.integers(1, 14)), int(rng.integers(1, 70))
    if seed % 3 == 0:
        C = int(rng.integers(1, 100))  # any channel count: the zero-padded copy of input and weights
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


def _typed(x, dtype):
    """Integer-valued float array -> the numpy form the oracle takes for `dtype`."""
    if dtype == capi.CKB_I8:
        return x.astype(np.int8)
    if dtype == capi.CKB_BF16:
        return oracle.to_bf16(x.astype(np.float32))
    return x.astype(np.float16)


def _dev_image(x, col_major, ldim):
    src = x.T if col_major else x
    buf = np.zeros((src.shape[0], ldim), dtype=x.dtype)
    buf[:, :src.shape[1]] = src
    return torch.from_numpy(buf.view(np.int16) if buf.dtype == np.uint16 else buf).cuda()


_TORCH = {capi.CKB_I8: torch.int8, capi.CKB_F16: torch.float16, capi.CKB_BF16: torch.int16}


@pytest.mark.parametrize("seed", range(24))
def test_random_multi_d_gemm(cuda_device, seed):
    """Epilogues that read D tensors (DeviceGemmMultipleD): random functor, layout, shape and D strides (0 = one row
    broadcast over M, N, or a padded pitch).  Integer inputs: the functors without a transcendental are bit exact."""
    rng = np.random.default_rng(20000 + seed)
    dtype = [capi.CKB_F16, capi.CKB_BF16][rng.integers(0, 2)]
    ops = [ck.Add(), ck.AddRelu(), ck.AddHardswish(), ck.Bilinear(0.5, 2.0), ck.AddAddFastGelu(), ck.AddReluAdd()]
    if dtype == capi.CKB_BF16:
        ops = [ck.AddRelu(), ck.AddHardswish(), ck.AddReluAdd()]
    op = ops[rng.integers(0, len(ops))]
    big = seed % 4 == 0
    M, N = (int(rng.integers(1500, 4000)), int(rng.integers(1500, 4000))) if big else (
        int(rng.integers(1, 600)), int(rng.integers(1, 600)))
    K = int(rng.integers(1, 24)) * 16
    a_layout, b_layout = [ROW, COL][rng.integers(0, 2)], [ROW, COL][rng.integers(0, 2)]
    a, b = _typed(rng.integers(-5, 6, (M, K)), dtype), _typed(rng.integers(-5, 6, (K, N)), dtype)
    lda = ((K if a_layout == ROW else M) + 7) // 8 * 8
    ldb = ((K if b_layout == COL else N) + 7) // 8 * 8
    da, db = _dev_image(a, a_layout == COL, lda), _dev_image(b, b_layout == COL, ldb)
    n_d = capi.EPI_NUM_D[op.kind]
    d_np, d_dev, ldds = [], [], []
    for i in range(n_d):
        mode = int(rng.integers(0, 3))  # 0: broadcast row, 1: packed, 2: padded pitch
        if mode == 0:
            row = _typed(rng.integers(-5, 6, (N,)), dtype)
            d_np.append(np.broadcast_to(row, (M, N)))
            d_dev.append(torch.from_numpy(row.view(np.int16) if row.dtype == np.uint16 else row).cuda())
            ldds.append(0)
        else:
            full = _typed(rng.integers(-5, 6, (M, N)), dtype)
            ldd = N if mode == 1 else N + 8 * int(rng.integers(1, 3))
            d_np.append(full)
            d_dev.append(_dev_image(full, False, ldd))
            ldds.append(ldd)
    e = torch.zeros((M, N), dtype=_TORCH[dtype], device="cuda")
    gemm = ck.DeviceGemmMultipleD(dtype, a_layout, b_layout)
    arg = gemm.MakeArgument(da.data_ptr(), db.data_ptr(), [t.data_ptr() for t in d_dev], e.data_ptr(), M, N, K, lda, ldb,
                            ldds, N, None, None, op)
    assert gemm.IsSupportedArgument(arg), capi.last_error()
    gemm.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    out = e.cpu().numpy()
    out = out.view(np.uint16) if dtype == capi.CKB_BF16 else out
    ref = oracle.gemm(a, b, op.kind, op.params, d_np[0] if n_d > 0 else None, d_np[1] if n_d > 1 else None)
    what = (seed, dtype, op.kind, M, N, K, a_layout, b_layout, ldds)
    if op.kind in (capi.CKB_EPI_ADD_ADD_FASTGELU, capi.CKB_EPI_ADD_HARDSWISH):
        if dtype == capi.CKB_BF16:
            o, r = oracle.from_bf16(out), oracle.from_bf16(ref)
            assert np.all(np.abs(o - r) <= np.abs(r) * 2.0 ** -7 + 1e-3), what
        else:
            bad, max_err = oracle.check_err(np.ascontiguousarray(out), ref, 1e-3, 1e-3)
            assert bad == 0, (what, bad, max_err)
    else:
        np.testing.assert_array_equal(out, ref, err_msg=str(what))


@pytest.mark.parametrize("seed", range(10))
def test_random_grouped_gemm(cuda_device, seed):
    """Grouped GEMM (DeviceGroupedGemm): 1 to 12 groups of unrelated shapes in one launch, random layout and type."""
    rng = np.random.default_rng(30000 + seed)
    dtype = [capi.CKB_F16, capi.CKB_BF16, capi.CKB_I8][rng.integers(0, 3)]
    per16 = 16 if dtype == capi.CKB_I8 else 8
    a_layout, b_layout = [ROW, COL][rng.integers(0, 2)], [ROW, COL][rng.integers(0, 2)]
    groups = int(rng.integers(1, 13))
    keep, p_a, p_b, p_e, descs, refs, outs = [], [], [], [], [], [], []
    for g in range(groups):
        M, N = int(rng.integers(1, 900)), int(rng.integers(1, 900))
        K = int(rng.integers(1, 20)) * 16
        a, b = _typed(rng.integers(-5, 6, (M, K)), dtype), _typed(rng.integers(-5, 6, (K, N)), dtype)
        lda = ((K if a_layout == ROW else M) + per16 - 1) // per16 * per16
        ldb = ((K if b_layout == COL else N) + per16 - 1) // per16 * per16
        lde = (N + per16 - 1) // per16 * per16
        da, db = _dev_image(a, a_layout == COL, lda), _dev_image(b, b_layout == COL, ldb)
        e = torch.zeros((M, lde), dtype=_TORCH[dtype], device="cuda")
        keep += [da, db]
        outs.append((e, N))
        p_a.append(da.data_ptr())
        p_b.append(db.data_ptr())
        p_e.append(e.data_ptr())
        descs.append(ck.GemmDescHost(M, N, K, lda, ldb, lde, []))
        refs.append(oracle.gemm(a, b))
    op = ck.DeviceGroupedGemm(dtype, a_layout, b_layout)
    arg = op.MakeArgument(p_a, p_b, [[] for _ in range(groups)], p_e, descs, None, None, ck.PassThrough())
    ws = torch.empty(max(op.GetWorkSpaceSize(arg), 1), dtype=torch.uint8, device="cuda")
    op.SetWorkSpacePointer(arg, ws.data_ptr())
    assert op.IsSupportedArgument(arg), capi.last_error()
    op.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    for g, ((e, N), ref) in enumerate(zip(outs, refs)):
        out = e.cpu().numpy()[:, :N]
        out = out.view(np.uint16) if dtype == capi.CKB_BF16 else out
        np.testing.assert_array_equal(out, ref, err_msg=str((seed, g, dtype, a_layout, b_layout, ref.shape)))


@pytest.mark.parametrize("seed", range(10))
def test_random_batched_gemm(cuda_device, seed):
    """Batched GEMM (DeviceBatchedGemm): random batch count, shape, layout, type and batch-stride padding."""
    from tests.test_batched_gpu import inputs, oracle_batched, run_batched

    rng = np.random.default_rng(40000 + seed)
    dtype = [capi.CKB_F16, capi.CKB_BF16, capi.CKB_I8][rng.integers(0, 3)]
    per16 = 16 if dtype == capi.CKB_I8 else 8
    G = int(rng.integers(1, 20))
    # run_batched packs the matrices (leading dimension = contiguous extent): keep those TMA-addressable
    M, N = per16 * int(rng.integers(1, 40)), per16 * int(rng.integers(1, 40))
    K = per16 * int(rng.integers(1, 24))
    layouts = ([ROW, COL][rng.integers(0, 2)], [ROW, COL][rng.integers(0, 2)])
    pad = per16 * int(rng.integers(0, 4))
    a, b = inputs(rng, dtype, G, M, N, K)
    out = run_batched(dtype, layouts[0], layouts[1], a, b, pad)
    np.testing.assert_array_equal(out, oracle_batched(a, b), err_msg=str((seed, dtype, G, M, N, K, layouts, pad)))
