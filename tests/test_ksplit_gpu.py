"""GPU parity tests of the K-split tail wave: when a GEMM has whole waves of tiles plus a small remainder, the
remaining tiles are cut along K, parked as raw accumulators and summed in slice order before the epilogue.
Integer-valued inputs make every partial sum exact, so the comparison with the oracle is bit for bit; a
real-valued case checks the reference's tolerance, repeated launches check that the per-tile counters are left
at zero, and two streams check that concurrent launches do not share scratch."""
import os

import numpy as np
import pytest
import torch

import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from oracle import ck_oracle as oracle

pytestmark = pytest.mark.gpu


def run(a, bt, op=None, dtype=capi.CKB_F16, stream=None, reps=1, out=None):
    M, K = a.shape
    N = bt.shape[0]
    as_dev = lambda x: torch.from_numpy(x.view(np.int16) if x.dtype == np.uint16 else x).cuda()
    da, db = as_dev(a), as_dev(bt)
    e = out if out is not None else torch.zeros((M, N), dtype=torch.int16 if dtype == capi.CKB_BF16 else torch.float16,
                                                device="cuda")
    g = ck.DeviceGemm(dtype)
    arg = g.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), M, N, K, K, K, N, None, None, op or ck.PassThrough())
    assert g.IsSupportedArgument(arg), capi.last_error()
    torch.cuda.synchronize()  # inputs and the zeroed output are in place before a launch on another stream
    for _ in range(reps):
        g.MakeInvoker().Run(arg, ck.StreamConfig(stream, False))
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    res = e.cpu().numpy()
    return res.view(np.uint16) if dtype == capi.CKB_BF16 else res


def ints(rng, shape):
    return rng.integers(-5, 6, shape).astype(np.float16)


@pytest.mark.parametrize("M,N,K,env", [
    (2048, 2560, 2560, {}),                       # 80 pair tiles on 74 pairs: 6 tail tiles, 4 slices (40 k blocks)
    (2048, 2560, 1024, {}),                       # same tiles, 16 k blocks: too short for the K split, column slices
    (2048, 3328, 5120, {}),                       # 104 pair tiles: 30 tail tiles, 2 K halves (80 k blocks)
    (2048, 3328, 512, {}),                        # same tiles, short K: the tail stays with column slices
    (2000, 2500, 2600, {}),                       # ragged M, N (scalar stores) and K
    (2048, 2560, 2560, {"CKB_FORCE_CG": "1"}),    # 160 single-CTA tiles on 148 SMs
    (2048, 2560, 3072, {"CKB_FORCE_BN": "128"}),  # 128-wide tiles: 2 slices (48 k blocks)
    (4096, 4864, 2560, {}),                       # several whole waves before the tail
])
def test_ksplit_tail_bit_exact(cuda_device, M, N, K, env):
    rng = np.random.default_rng(M + N + K)
    a, bt = ints(rng, (M, K)), ints(rng, (N, K))
    os.environ.update(env)
    try:
        out = run(a, bt, reps=2)  # twice: the second launch finds the counters as the first left them
    finally:
        for k in env:
            del os.environ[k]
    np.testing.assert_array_equal(out, oracle.gemm(a, bt.T))


def test_ksplit_matches_column_slices_and_oracle_on_real_inputs(cuda_device):
    rng = np.random.default_rng(7)
    M, N, K = 2048, 2560, 2560
    a = rng.uniform(-1, 1, (M, K)).astype(np.float16)
    bt = rng.uniform(-1, 1, (N, K)).astype(np.float16)
    op = ck.Relu()
    out = run(a, bt, op)
    ref = oracle.gemm(a, bt.T, op.kind, op.params)
    bad, max_err = oracle.check_err(out, ref, 1e-3, 1e-3)
    assert bad == 0, (bad, max_err)
    os.environ["CKB_NO_SPLITK"] = "1"
    try:
        cols = run(a, bt, op)
    finally:
        del os.environ["CKB_NO_SPLITK"]
    bad, max_err = oracle.check_err(out, cols, 1e-3, 1e-3)
    assert bad == 0, (bad, max_err)
    # the split changes the summation order only inside the 6 tail tiles
    assert (out != cols).mean() < 0.08


def test_ksplit_bf16(cuda_device):
    rng = np.random.default_rng(11)
    M, N, K = 2048, 2560, 2560
    a = oracle.to_bf16(rng.integers(-5, 6, (M, K)).astype(np.float32))
    bt = oracle.to_bf16(rng.integers(-5, 6, (N, K)).astype(np.float32))
    out = run(a, bt, dtype=capi.CKB_BF16)
    np.testing.assert_array_equal(out, oracle.gemm(a, bt.T))


def test_first_ksplit_launch_of_a_fresh_scratch_on_a_side_stream(cuda_device):
    """The scratch of a stream is allocated, and its counters zeroed, by the first K-split launch on that stream; the
    zeroing has to be ordered before that launch on the stream itself - a torch side stream is non-blocking, so work on
    the legacy default stream is not."""
    capi.check(capi.lib().ckb_release_scratch(None, 1))  # every stream starts without scratch
    rng = np.random.default_rng(19)
    M, N, K = 2048, 2560, 2560
    a, bt = ints(rng, (M, K)), ints(rng, (N, K))
    ref = oracle.gemm(a, bt.T)
    for _ in range(3):
        st = torch.cuda.Stream()
        out = run(a, bt, stream=st.cuda_stream, reps=2)
        np.testing.assert_array_equal(out, ref)
        capi.check(capi.lib().ckb_release_scratch(st.cuda_stream, 0))


@pytest.mark.parametrize("cfg", [(256, 2, 0), (256, 1, 0), (128, 1, 0), (64, 1, 0), (256, 2, 1), (0, 0, 1)])
def test_pinned_tile_configurations_bit_exact(cuda_device, cfg):
    """The tile configurations an instance factory hands out (CKB_TILE_CONFIG): same results from every one."""
    rng = np.random.default_rng(23)
    M, N, K = 2048, 2560, 2560
    a, bt = ints(rng, (M, K)), ints(rng, (N, K))
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    e = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    g = ck.DeviceGemm(capi.CKB_F16, tile_config=capi.tile_config(*cfg))
    arg = g.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), M, N, K, K, K, N)
    assert g.IsSupportedArgument(arg), capi.last_error()
    g.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    np.testing.assert_array_equal(e.cpu().numpy(), oracle.gemm(a, bt.T))


def test_ksplit_on_two_streams_at_once(cuda_device):
    """Each stream has its own scratch: interleaved launches of two different problems stay correct."""
    rng = np.random.default_rng(13)
    shapes = [(2048, 2560, 2560), (2048, 3328, 5120)]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    ins = [(ints(rng, (M, K)), ints(rng, (N, K))) for M, N, K in shapes]
    keep, outs, args = [], [], []
    g = ck.DeviceGemm(capi.CKB_F16)
    for (a, bt), (M, N, K) in zip(ins, shapes):
        da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
        e = torch.zeros((M, N), dtype=torch.float16, device="cuda")
        keep += [da, db]
        outs.append(e)
        args.append(g.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), M, N, K, K, K, N))
    torch.cuda.synchronize()
    for _ in range(4):
        for st, arg in zip(streams, args):
            g.MakeInvoker().Run(arg, ck.StreamConfig(st.cuda_stream, False))
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    for e, (a, bt) in zip(outs, ins):
        np.testing.assert_array_equal(e.cpu().numpy(), oracle.gemm(a, bt.T))


def test_ksplit_tail_of_a_batched_gemm_spans_batches(cuda_device):
    """Batched GEMM whose tail tiles belong to different batches: 40 batches of 512 x 512 x 2560 are 160 pair tiles on
    74 pairs (148 whole, 12 tail tiles cut in four along K: 40 k blocks, the shortest K loop that takes the split)."""
    rng = np.random.default_rng(17)
    G, M, N, K = 40, 512, 512, 2560
    a, bt = ints(rng, (G, M, K)), ints(rng, (G, N, K))
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    e = torch.zeros((G, M, N), dtype=torch.float16, device="cuda")
    op = ck.DeviceBatchedGemm(capi.CKB_F16)
    arg = op.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), M, N, K, K, K, N, M * K, N * K, M * N, G)
    assert op.IsSupportedArgument(arg), capi.last_error()
    op.MakeInvoker().Run(arg)
    op.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    out = e.cpu().numpy()
    for g in range(G):
        np.testing.assert_array_equal(out[g], oracle.gemm(a[g], bt[g].T))


@pytest.mark.parametrize("M,N,K", [
    (512, 512, 8192),     # 4 pair tiles x 4 slices
    (1024, 1024, 4096),   # 16 pair tiles x 4 slices
    (256, 256, 16384),    # one pair tile, 4 slices of 64 k blocks
    (128, 384, 6144),     # a single row of tiles: M fills half a pair tile
    (1000, 700, 5000),    # ragged M, N (scalar stores) and K (last slice shorter than the others)
    (1536, 2048, 2048),   # 2 slices only: 48 pair tiles on 74 pairs would not take 4
    (192, 128, 3072),     # narrow N: the 128-wide tile, 2 slices
])
def test_whole_problem_k_split_bit_exact(cuda_device, M, N, K):
    """Few output tiles and a long K: every tile's K loop is cut (no whole tiles before the slices)."""
    rng = np.random.default_rng(M * 3 + N * 5 + K)
    a, bt = ints(rng, (M, K)), ints(rng, (N, K))
    out = run(a, bt, reps=2)
    np.testing.assert_array_equal(out, oracle.gemm(a, bt.T))


def test_whole_problem_k_split_bf16_layouts_and_functor(cuda_device):
    from tests.test_layouts_gpu import COL, ROW, make_inputs, run_layout

    rng = np.random.default_rng(4321)
    M, N, K = 640, 768, 6144
    for dtype in (capi.CKB_F16, capi.CKB_BF16):
        a, b = make_inputs(rng, dtype, M, N, K)
        ref = oracle.gemm(a, b)
        for layouts in ((ROW, COL), (ROW, ROW), (COL, ROW), (COL, COL)):
            np.testing.assert_array_equal(run_layout(dtype, layouts[0], layouts[1], a, b), ref, err_msg=str((dtype, layouts)))
    a, b = make_inputs(rng, capi.CKB_F16, M, N, K, kind="real")
    op = ck.FastGelu()
    out = run_layout(capi.CKB_F16, ROW, COL, a, b, op=op)
    bad, max_err = oracle.check_err(out, oracle.gemm(a, b, op.kind, op.params), 1e-3, 1e-3)
    assert bad == 0, (bad, max_err)


def test_whole_problem_k_split_matches_the_unsplit_plan(cuda_device):
    """Same problem with the K split switched off: the column-slice plan.  Integer inputs: identical bits."""
    rng = np.random.default_rng(99)
    a, bt = ints(rng, (768, 8192)), ints(rng, (512, 8192))
    split = run(a, bt)
    os.environ["CKB_NO_SPLITK"] = "1"
    try:
        plain = run(a, bt)
    finally:
        del os.environ["CKB_NO_SPLITK"]
    np.testing.assert_array_equal(split, plain)
    np.testing.assert_array_equal(split, oracle.gemm(a, bt.T))
