"""GPU parity tests of the balanced K ranges: where the last wave of tiles is neither full nor small, the k blocks of
the last one or two waves' tiles are laid end to end and dealt out evenly over the CTAs (or CTA pairs), across tile
boundaries.  A CTA whose run starts inside a tile parks that part as a raw accumulator; the CTA whose run ends with the
head of the tile adds the parked parts in k order before the epilogue.  Integer-valued inputs make every partial sum
exact, so the comparison with the oracle is bit for bit; real-valued inputs are held to the reference's tolerance;
repeated launches check that the per-tile counters are left at zero."""
import re

import numpy as np
import pytest
import torch

import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from oracle import ck_oracle as oracle

pytestmark = pytest.mark.gpu


def run(a, bt, tile_config=0, op=None, dtype=capi.CKB_F16, reps=1):
    M, K = a.shape
    N = bt.shape[0]
    as_dev = lambda x: torch.from_numpy(x.view(np.int16) if x.dtype == np.uint16 else x).cuda()
    da, db = as_dev(a), as_dev(bt)
    e = torch.full((M, N), -3, dtype=torch.int16 if dtype == capi.CKB_BF16 else torch.float16, device="cuda")
    g = ck.DeviceGemm(dtype, tile_config=tile_config)
    arg = g.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), M, N, K, K, K, N, None, None, op or ck.PassThrough())
    assert g.IsSupportedArgument(arg), capi.last_error()
    torch.cuda.synchronize()
    for _ in range(reps):
        g.MakeInvoker().Run(arg)
    plan = capi.last_plan()
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    res = e.cpu().numpy()
    return (res.view(np.uint16) if dtype == capi.CKB_BF16 else res), plan


def balanced_run_length(plan):
    return int(re.search(r"balanced=(\d+)", plan).group(1))


def ints(rng, shape):
    return rng.integers(-5, 6, shape).astype(np.float16)


@pytest.mark.parametrize("M,N,K,bn,cg", [
    (1280, 2048, 4096, 256, 1),   # 80 tiles on 148 CTAs: runs of 36 k blocks, tiles shared by two or three CTAs
    (1280, 2048, 4096, 256, 2),   # 40 pair tiles on 74 pairs
    (1280, 1536, 4096, 128, 1),   # 120 tiles of 128 x 128
    (768, 8192, 2048, 256, 2),    # 96 pair tiles on 74 pairs: whole tiles inside the runs
    (512, 8192, 2368, 256, 1),    # 37 k blocks per tile: parts start on odd k blocks
    (1000, 2500, 2600, 256, 2),   # ragged M, N (scalar stores) and K
    (4096, 4864, 1024, 256, 2),   # 304 pair tiles: three whole waves, then 82 tiles balanced
    (3840, 4096, 1024, 256, 1),   # 480 tiles: two whole waves, then 184 tiles balanced
])
def test_balanced_k_ranges_bit_exact(cuda_device, M, N, K, bn, cg):
    rng = np.random.default_rng(M + N + K + bn + cg)
    a, bt = ints(rng, (M, K)), ints(rng, (N, K))
    out, plan = run(a, bt, capi.tile_config(bn, cg, balanced=1), reps=3)
    assert balanced_run_length(plan) > 0, plan
    np.testing.assert_array_equal(out, oracle.gemm(a, bt.T))


def test_library_takes_the_balanced_plan_for_a_half_filled_wave_with_a_long_k(cuda_device):
    """80 tiles of 128 x 256 on 148 SMs leave 68 SMs idle for the whole launch.  With K = 8192 (operands of 54 MB, which
    stay in L2) the library balances the K ranges by itself; with K = 4096 the shorter main loop does not pay for the
    fix-up and the plain plan stands."""
    rng = np.random.default_rng(3)
    M, N, K = 1280, 2048, 8192
    a, bt = ints(rng, (M, K)), ints(rng, (N, K))
    out, plan = run(a, bt, reps=2)
    assert balanced_run_length(plan) == 70, plan
    np.testing.assert_array_equal(out, oracle.gemm(a, bt.T))
    # pinned off: the plain plan, same bits (integer inputs)
    out2, plan2 = run(a, bt, capi.tile_config(no_ksplit=1))
    assert balanced_run_length(plan2) == 0, plan2
    np.testing.assert_array_equal(out2, out)
    _, plan3 = run(a[:, :4096].copy(), bt[:, :4096].copy())
    assert balanced_run_length(plan3) == 0, plan3


def test_balanced_real_inputs_relu_and_bf16(cuda_device):
    rng = np.random.default_rng(5)
    M, N, K = 1280, 2048, 2048
    a = rng.uniform(-1, 1, (M, K)).astype(np.float16)
    bt = rng.uniform(-1, 1, (N, K)).astype(np.float16)
    op = ck.Relu()
    out, plan = run(a, bt, capi.tile_config(256, 1, balanced=1), op)
    assert balanced_run_length(plan) > 0, plan
    bad, max_err = oracle.check_err(out, oracle.gemm(a, bt.T, op.kind, op.params), 1e-3, 1e-3)
    assert bad == 0, (bad, max_err)
    a16 = oracle.to_bf16(rng.integers(-5, 6, (M, K)).astype(np.float32))
    b16 = oracle.to_bf16(rng.integers(-5, 6, (N, K)).astype(np.float32))
    out, plan = run(a16, b16, capi.tile_config(256, 2, balanced=1), dtype=capi.CKB_BF16)
    assert balanced_run_length(plan) > 0, plan
    np.testing.assert_array_equal(out, oracle.gemm(a16, b16.T))


@pytest.mark.parametrize("cg", [1, 2])
def test_balanced_int8_requantisation_bit_exact(cuda_device, cg):
    """int8 GEMMs run the balanced plan in kernel instances of their own (256-wide tiles)."""
    rng = np.random.default_rng(9 + cg)
    M, N, K = 1280, 2048, 4096
    a = rng.integers(-5, 6, (M, K)).astype(np.int8)
    bt = rng.integers(-5, 6, (N, K)).astype(np.int8)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    e = torch.zeros((M, N), dtype=torch.int8, device="cuda")
    fn = ck.RequantReluRequantRne(0.03, 14.0)
    g = ck.DeviceGemm(capi.CKB_I8, tile_config=capi.tile_config(256, cg, balanced=1))
    arg = g.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), M, N, K, K, K, N, None, None, fn)
    assert g.IsSupportedArgument(arg), capi.last_error()
    for _ in range(2):
        g.MakeInvoker().Run(arg)
    plan = capi.last_plan()
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    assert balanced_run_length(plan) > 0, plan
    np.testing.assert_array_equal(e.cpu().numpy(), oracle.gemm(a, bt.T, fn.kind, fn.params))


@pytest.mark.parametrize("cg", [1, 2])
def test_balanced_with_fused_d_epilogue(cuda_device, cg):
    """Add + Add + FastGelu (a bias row and a residual) on top of balanced K ranges: the parked parts are summed into
    the accumulator in tensor memory, then the usual epilogue reads D0 and D1."""
    rng = np.random.default_rng(21 + cg)
    M, N, K = 1280 - 3, 2048, 2048
    a = rng.uniform(-1, 1, (M, K)).astype(np.float16)
    bt = rng.uniform(-1, 1, (N, K)).astype(np.float16)
    d0 = rng.uniform(-1, 1, (N,)).astype(np.float16)
    d1 = rng.uniform(-1, 1, (M, N)).astype(np.float16)
    da, db, dd0, dd1 = (torch.from_numpy(x).cuda() for x in (a, bt, d0, d1))
    e = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    op = ck.DeviceGemmMultipleD(tile_config=capi.tile_config(256, cg, balanced=1))
    arg = op.MakeArgument(da.data_ptr(), db.data_ptr(), [dd0.data_ptr(), dd1.data_ptr()], e.data_ptr(), M, N, K,
                          K, K, [0, N], N, None, None, ck.AddAddFastGelu())
    assert op.IsSupportedArgument(arg), capi.last_error()
    for _ in range(2):
        op.MakeInvoker().Run(arg)
    plan = capi.last_plan()
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    assert balanced_run_length(plan) > 0, plan
    ref = oracle.gemm(a, bt.T, oracle.EPI_ADD_ADD_FASTGELU, None, np.broadcast_to(d0, (M, N)), d1)
    bad, err = oracle.check_err(e.cpu().numpy(), ref)
    assert bad == 0, (bad, err)


def test_balanced_flag_falls_back_on_narrow_tiles_of_the_other_families(cuda_device):
    """The balanced instances of int8 and D-reading kernels exist for 256-wide tiles; a pinned 128-wide tile keeps
    its plan and the flag is not an error."""
    rng = np.random.default_rng(9)
    a = rng.integers(-5, 6, (1280, 1024)).astype(np.int8)
    bt = rng.integers(-5, 6, (1536, 1024)).astype(np.int8)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    e = torch.zeros((1280, 1536), dtype=torch.int8, device="cuda")
    g = ck.DeviceGemm(capi.CKB_I8, tile_config=capi.tile_config(128, 1, balanced=1))
    arg = g.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), 1280, 1536, 1024, 1024, 1024, 1536)
    assert g.IsSupportedArgument(arg), capi.last_error()
    g.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert balanced_run_length(capi.last_plan()) == 0
    np.testing.assert_array_equal(e.cpu().numpy(), oracle.gemm(a, bt.T))
