"""GPU tests of the library under CUDA graph capture and of the scratch-memory entry point.

A captured launch must not allocate, free or synchronise, and its result must not depend on state that another stream
can touch while the graph replays: GEMM, batched GEMM and convolution launches are captured with n_rep = 0 and replayed
with fresh inputs; the grouped GEMM copies a host table at every launch, which the library keeps alive for a captured
launch, while the entry point with the fixed table must refuse a capturing stream without breaking the capture."""
import ctypes

import numpy as np
import pytest
import torch

import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from oracle import ck_oracle as oracle

pytestmark = pytest.mark.gpu


def _ints(rng, shape, dtype=np.float16):
    return rng.integers(-5, 6, shape).astype(dtype)


def test_gemm_and_conv_replay_from_a_graph(cuda_device):
    rng = np.random.default_rng(77)
    M, N, K = 3840, 4096, 1024  # partial last wave: the eager plan cuts its tiles along K and owns scratch
    a, bt = _ints(rng, (M, K)), _ints(rng, (N, K))
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    e = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    gemm = ck.DeviceGemm(capi.CKB_F16)
    garg = gemm.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), M, N, K, K, K, N, None, None, ck.PassThrough())
    assert gemm.IsSupportedArgument(garg), capi.last_error()

    Nb, C, Kc, H = 8, 64, 96, 19
    inp, wei = _ints(rng, (Nb, H, H, C)), _ints(rng, (Kc, 3, 3, C))
    di, dw = torch.from_numpy(inp).cuda(), torch.from_numpy(wei).cuda()
    Ho = oracle.conv_out_len(H, 3, 2, 1, 1, 1)
    out = torch.zeros((Nb, Ho, Ho, Kc), dtype=torch.float16, device="cuda")
    conv = ck.DeviceConvFwd(capi.CKB_F16)
    carg = conv.MakeArgument(di.data_ptr(), dw.data_ptr(), out.data_ptr(), Nb, Kc, C, [H, H], [3, 3], [Ho, Ho], [2, 2],
                             [1, 1], [1, 1], [1, 1])
    assert conv.IsSupportedArgument(carg), capi.last_error()

    # eager warm-up on the side stream the capture will use (first-use initialisation happens here)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        gemm.MakeInvoker().Run(garg, ck.StreamConfig(side.cuda_stream, False))
        conv.MakeInvoker().Run(carg, ck.StreamConfig(side.cuda_stream, False))
    side.synchronize()
    np.testing.assert_array_equal(e.cpu().numpy(), oracle.gemm(a, bt.T))
    launches_before = ck.launch_count()

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        s = torch.cuda.current_stream().cuda_stream
        gemm.MakeInvoker().Run(garg, ck.StreamConfig(s, False))
        conv.MakeInvoker().Run(carg, ck.StreamConfig(s, False))
    assert ck.launch_count() == launches_before + 2

    for rep in range(2):  # new operand values in the same buffers, then replay
        a, bt = _ints(rng, (M, K)), _ints(rng, (N, K))
        inp, wei = _ints(rng, (Nb, H, H, C)), _ints(rng, (Kc, 3, 3, C))
        da.copy_(torch.from_numpy(a))
        db.copy_(torch.from_numpy(bt))
        di.copy_(torch.from_numpy(inp))
        dw.copy_(torch.from_numpy(wei))
        e.zero_()
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert ck.device_status() == 0
        np.testing.assert_array_equal(e.cpu().numpy(), oracle.gemm(a, bt.T))
        np.testing.assert_array_equal(out.cpu().numpy(), oracle.conv2d_fwd(inp, wei, (2, 2), (1, 1), (1, 1)))


def test_cluster_k_split_replays_from_a_graph(cuda_device):
    """A GEMM with few tiles and a long K runs as thread-block clusters whose K slices are summed through distributed
    shared memory: no scratch, no counters, so the captured launch takes the same plan as the eager one."""
    rng = np.random.default_rng(79)
    M, N, K = 256, 384, 8192
    a, bt = _ints(rng, (M, K)), _ints(rng, (N, K))
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    e = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    gemm = ck.DeviceGemm(capi.CKB_F16)
    arg = gemm.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), M, N, K, K, K, N)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        gemm.MakeInvoker().Run(arg, ck.StreamConfig(side.cuda_stream, False))
    eager_plan = capi.last_plan()
    side.synchronize()
    assert "cluster_k=0" not in eager_plan, eager_plan
    np.testing.assert_array_equal(e.cpu().numpy(), oracle.gemm(a, bt.T))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        gemm.MakeInvoker().Run(arg, ck.StreamConfig(torch.cuda.current_stream().cuda_stream, False))
    assert capi.last_plan() == eager_plan
    for rep in range(2):
        a, bt = _ints(rng, (M, K)), _ints(rng, (N, K))
        da.copy_(torch.from_numpy(a))
        db.copy_(torch.from_numpy(bt))
        e.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert ck.device_status() == 0
        np.testing.assert_array_equal(e.cpu().numpy(), oracle.gemm(a, bt.T))


def test_grouped_gemm_replays_from_a_graph_and_noalloc_refuses_capture(cuda_device):
    rng = np.random.default_rng(78)
    shapes = [(256, 128, 64), (200, 264, 136), (512, 384, 256)]
    A = [torch.from_numpy(_ints(rng, (m, k))).cuda() for m, n, k in shapes]
    B = [torch.from_numpy(_ints(rng, (n, k))).cuda() for m, n, k in shapes]
    E = [torch.zeros((m, n), dtype=torch.float16, device="cuda") for m, n, k in shapes]
    op = ck.DeviceGroupedGemm(capi.CKB_F16)
    arg = op.MakeArgument([x.data_ptr() for x in A], [x.data_ptr() for x in B], [[] for _ in shapes],
                          [x.data_ptr() for x in E], [ck.GemmDescHost(m, n, k, k, k, n, []) for m, n, k in shapes],
                          None, None, ck.PassThrough())
    ws = torch.empty(max(op.GetWorkSpaceSize(arg), 1), dtype=torch.uint8, device="cuda")
    op.SetWorkSpacePointer(arg, ws.data_ptr())
    op.MakeInvoker().Run(arg)  # eager
    torch.cuda.synchronize()
    for a, b, e in zip(A, B, E):
        np.testing.assert_array_equal(e.cpu().numpy(), oracle.gemm(a.cpu().numpy(), b.cpu().numpy().T))

    side = torch.cuda.Stream()
    marker = torch.zeros(4, device="cuda")
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        s = torch.cuda.current_stream().cuda_stream
        op.MakeInvoker().Run(arg, ck.StreamConfig(s, False))
        # the entry point with the fixed table shares its host staging among all calls: not capturable
        rc = capi.lib().ckb_grouped_gemm_run_noalloc(ctypes.byref(arg.desc), s)
        assert rc == capi.CKB_ERR_UNSUPPORTED and "graph" in capi.last_error()
        marker += 1  # the capture is still alive and records this
    ws.zero_()  # the replay has to bring the group table back by itself
    for rep in range(2):
        for x in A + B:
            x.copy_(torch.from_numpy(_ints(rng, tuple(x.shape))))
        for e in E:
            e.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert ck.device_status() == 0
        for a, b, e in zip(A, B, E):
            np.testing.assert_array_equal(e.cpu().numpy(), oracle.gemm(a.cpu().numpy(), b.cpu().numpy().T))
    assert marker.cpu().tolist() == [2.0] * 4


def test_release_scratch_and_run_again(cuda_device):
    rng = np.random.default_rng(79)
    M, N, K = 2048, 2560, 512
    a, bt = _ints(rng, (M, K)), _ints(rng, (N, K))
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    ref = oracle.gemm(a, bt.T)
    gemm = ck.DeviceGemm(capi.CKB_F16)
    for round_ in range(3):
        e = torch.zeros((M, N), dtype=torch.float16, device="cuda")
        arg = gemm.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), M, N, K, K, K, N, None, None, ck.PassThrough())
        gemm.MakeInvoker().Run(arg)
        torch.cuda.synchronize()
        np.testing.assert_array_equal(e.cpu().numpy(), ref)
        capi.check(capi.lib().ckb_release_scratch(None, 1 if round_ else 0))
    assert ck.device_status() == 0
