"""GPU parity tests of the cluster K split: a thread-block cluster of 2, 4 or 8 CTAs works on one output tile, every
CTA accumulates one K slice, and the slices are summed through distributed shared memory in slice order.  The slice
count is named through the descriptor's tile configuration (the KBatch of the reference's split-K operation,
device/device_gemm_splitk.hpp:23-42) or chosen by the library for GEMMs with few tiles and a long K.  Integer-valued
inputs make every partial sum exact, so results are compared with the oracle bit for bit."""
import numpy as np
import pytest
import torch

import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from oracle import ck_oracle as oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu
ROW, COL = capi.CKB_ROW_MAJOR, capi.CKB_COL_MAJOR


def run(a, bt, tile_config=0, op=None, dtype=capi.CKB_F16, d0=None, d1=None, reps=1):
    M, K = a.shape
    N = bt.shape[0]
    to = lambda x: torch.from_numpy(x.view(np.int16) if x.dtype == np.uint16 else x).cuda()
    da, db = to(a), to(bt)
    tdt = {capi.CKB_I8: torch.int8, capi.CKB_F16: torch.float16, capi.CKB_BF16: torch.int16}[dtype]
    e = torch.zeros((M, N), dtype=tdt, device="cuda")
    ds, lds, keep = [], [], []
    for d in (d0, d1):
        if d is not None:
            t = to(d)
            keep.append(t)
            ds.append(t.data_ptr())
            lds.append(0 if d.ndim == 1 else d.shape[1])
    g = ck.DeviceGemmMultipleD(dtype, tile_config=tile_config)
    arg = g.MakeArgument(da.data_ptr(), db.data_ptr(), ds, e.data_ptr(), M, N, K, K, K, lds, N, None, None,
                         op or ck.PassThrough())
    assert g.IsSupportedArgument(arg), capi.last_error()
    for _ in range(reps):
        g.MakeInvoker().Run(arg)
    plan = capi.last_plan()
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    out = e.cpu().numpy()
    return (out.view(np.uint16) if dtype == capi.CKB_BF16 else out), plan


def ints(rng, shape, dtype=np.float16):
    return rng.integers(-5, 6, shape).astype(dtype)


@pytest.mark.parametrize("bn", [256, 128, 64])
@pytest.mark.parametrize("kbatch", [2, 4, 8])
def test_named_k_batch_bit_exact(cuda_device, bn, kbatch):
    if bn // kbatch < 16:
        pytest.skip("column parts narrower than 16 columns fall back to the library's choice")
    rng = np.random.default_rng(bn + kbatch)
    M, N, K = 300, 520, 4096  # ragged rows and columns; 64 k blocks
    a, bt = ints(rng, (M, K)), ints(rng, (N, K))
    out, plan = run(a, bt, capi.tile_config(bn, 1, kbatch=kbatch), reps=2)
    assert f"cluster_k={kbatch}" in plan and f"tile=128x{bn}" in plan, plan
    np.testing.assert_array_equal(out, oracle.gemm(a, bt.T))


def test_ragged_k_and_last_slice_shorter(cuda_device):
    rng = np.random.default_rng(1)
    M, N, K = 256, 256, 4104  # 65 k blocks: four slices of 18, 18, 18 and 11, the last k block holds 8 of 64 columns
    a, bt = ints(rng, (M, K)), ints(rng, (N, K))
    out, plan = run(a, bt, capi.tile_config(256, 1, kbatch=4))
    assert "cluster_k=4" in plan, plan
    np.testing.assert_array_equal(out, oracle.gemm(a, bt.T))
    # eight slices do not fit 65 k blocks (the last would be empty): the library's own choice runs instead
    out, plan = run(a, bt, capi.tile_config(256, 1, kbatch=8))
    assert "cluster_k=8" not in plan, plan
    np.testing.assert_array_equal(out, oracle.gemm(a, bt.T))


def test_k_batch_with_fused_epilogues_int8_and_bf16(cuda_device):
    rng = np.random.default_rng(2)
    M, N, K = 384, 640, 2048
    a = rng.uniform(-1, 1, (M, K)).astype(np.float16)
    bt = rng.uniform(-1, 1, (N, K)).astype(np.float16)
    d0 = rng.uniform(-1, 1, (N,)).astype(np.float16)
    d1 = rng.uniform(-1, 1, (M, N)).astype(np.float16)
    op = ck.AddAddFastGelu()
    out, plan = run(a, bt, capi.tile_config(256, 1, kbatch=4), op, d0=d0, d1=d1)
    assert "cluster_k=4" in plan, plan
    H.assert_close(out, oracle.gemm(a, bt.T, op.kind, op.params, np.broadcast_to(d0, (M, N)), d1))
    a8, b8 = ints(rng, (M, K), np.int8), ints(rng, (N, K), np.int8)
    op8 = ck.RequantReluRequantRne(0.03, 14.0)
    out8, plan = run(a8, b8, capi.tile_config(128, 1, kbatch=8), op8, dtype=capi.CKB_I8)
    assert "cluster_k=8" in plan, plan
    np.testing.assert_array_equal(out8, oracle.gemm(a8, b8.T, op8.kind, op8.params))
    ab = oracle.to_bf16(rng.integers(-5, 6, (M, K)).astype(np.float32))
    bb = oracle.to_bf16(rng.integers(-5, 6, (N, K)).astype(np.float32))
    outb, plan = run(ab, bb, capi.tile_config(256, 1, kbatch=2), dtype=capi.CKB_BF16)
    assert "cluster_k=2" in plan, plan
    np.testing.assert_array_equal(outb, oracle.gemm(ab, bb.T))


@pytest.mark.parametrize("M,N,K", [(256, 256, 16384), (768, 768, 4096), (128, 4096, 8192), (512, 512, 8192),
                                   (100, 200, 12288)])
def test_library_chooses_the_cluster_split_for_few_tiles_and_long_k(cuda_device, M, N, K):
    rng = np.random.default_rng(M + N + K)
    a, bt = ints(rng, (M, K)), ints(rng, (N, K))
    out, plan = run(a, bt, reps=2)
    assert "ksplit=" in plan and "ksplit=0" not in plan, plan  # every tile cut along K, one way or the other
    np.testing.assert_array_equal(out, oracle.gemm(a, bt.T))
    # real-valued inputs: within the reference's check_err rule of the oracle
    ar = rng.uniform(-1, 1, (M, K)).astype(np.float16)
    br = rng.uniform(-1, 1, (N, K)).astype(np.float16)
    outr, _ = run(ar, br, op=ck.Relu())
    H.assert_close(outr, oracle.gemm(ar, br.T, oracle.EPI_RELU))


def test_more_clusters_than_the_machine_holds_at_once(cuda_device):
    """Clusters are independent of one another: 80 tiles x 8 slices = 640 CTAs run in several waves."""
    rng = np.random.default_rng(5)
    M, N, K = 1280, 2048, 2048
    a, bt = ints(rng, (M, K)), ints(rng, (N, K))
    out, plan = run(a, bt, capi.tile_config(256, 1, kbatch=8))
    assert "cluster_k=8" in plan and "grid=640" in plan, plan
    np.testing.assert_array_equal(out, oracle.gemm(a, bt.T))
