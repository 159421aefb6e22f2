"""GPU test of ckb_grouped_gemm_run_noalloc, the grouped-GEMM entry point for callers that cannot
allocate device memory (a fixed memory plan, another framework's planner, a latency-critical loop):
its group table lives in a fixed array inside the library instead of a caller-provided workspace.

The entry point is called through the C ABI twice in a row, with different group sets, and each
result must equal - bit for bit, the kernel is the same - what the workspace-taking entry point
ckb_grouped_gemm_run writes for the same descriptors, and must agree with the CPU oracle group by
group (the reference's check_err rule), so that a fault shared by both entry points cannot hide.
Device memory is watched at the driver level (cudaMemGetInfo): torch's own counters only see
torch's caching allocator, not a cudaMalloc made inside the library.  The second call is smaller than the first,
so entries left in the shared table by the first call must not leak into it.  The file name sorts
last so that a run that stops at the first failure has already run every other test; the test
needs no state from the others and passes alone in a fresh process."""
import ctypes

import numpy as np
import pytest
import torch

import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _make_arg(shapes, seed, with_bias):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    A = [torch.empty((m, k), dtype=torch.float16, device="cuda").uniform_(-1, 1, generator=gen) for m, n, k in shapes]
    B = [torch.empty((n, k), dtype=torch.float16, device="cuda").uniform_(-1, 1, generator=gen) for m, n, k in shapes]
    bias = [torch.empty((n,), dtype=torch.float16, device="cuda").uniform_(-1, 1, generator=gen) for m, n, k in shapes]
    op = ck.DeviceGroupedGemm()
    descs = [ck.GemmDescHost(m, n, k, k, k, n, [0] if with_bias else []) for m, n, k in shapes]

    def bind(E):
        return op.MakeArgument([x.data_ptr() for x in A], [x.data_ptr() for x in B],
                               [[b.data_ptr()] for b in bias] if with_bias else [], [e.data_ptr() for e in E],
                               descs, None, None, ck.AddRelu() if with_bias else ck.PassThrough())
    return op, bind, (A, B, bias)


def _run_both(shapes, seed, with_bias):
    op, bind, keep = _make_arg(shapes, seed, with_bias)
    E_ref = [torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda") for m, n, k in shapes]
    E_new = [torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda") for m, n, k in shapes]
    # existing entry point, caller-allocated workspace
    arg = bind(E_ref)
    ws = torch.empty(op.GetWorkSpaceSize(arg), dtype=torch.uint8, device="cuda")
    op.SetWorkSpacePointer(arg, ws.data_ptr())
    assert op.IsSupportedArgument(arg), capi.last_error()
    op.MakeInvoker().Run(arg)
    # new entry point: no workspace, nothing allocated by the call.  The first call on a device loads the module
    # and looks up the table's address; the call after it is the one whose device memory is watched.
    arg2 = bind(E_new)
    capi.check(capi.lib().ckb_grouped_gemm_run_noalloc(ctypes.byref(arg2.desc), None))
    torch.cuda.synchronize()
    for e in E_new:
        e.fill_(float("nan"))
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    capi.check(capi.lib().ckb_grouped_gemm_run_noalloc(ctypes.byref(arg2.desc), None))
    torch.cuda.synchronize()
    free_after = torch.cuda.mem_get_info()[0]
    assert free_after >= free_before, f"the call took {free_before - free_after} bytes of device memory"
    assert ck.device_status() == 0
    A, B, bias = keep
    fn = ck.AddRelu() if with_bias else ck.PassThrough()
    for g, (e_new, e_ref) in enumerate(zip(E_new, E_ref)):
        a, b = e_new.cpu().numpy(), e_ref.cpu().numpy()
        assert np.isfinite(b.astype(np.float32)).all()
        np.testing.assert_array_equal(a.view(np.uint16), b.view(np.uint16))
        ref = H.oracle_gemm(A[g].cpu().numpy(), B[g].cpu().numpy(), fn, bias[g].cpu().numpy() if with_bias else None)
        H.assert_close(a, ref)


def test_noalloc_matches_workspace_entry_point_on_two_calls_in_a_row(cuda_device):
    # call 1: many ragged groups, enough tiles for the CTA-pair kernel and a split tail wave
    shapes1 = [(256 * (1 + g % 5), 512 + 256 * (g % 3), 128 * (1 + g % 4)) for g in range(24)] + [(130, 72, 64), (1, 8, 8)]
    _run_both(shapes1, seed=1, with_bias=False)
    # call 2: fewer, different groups and a fused bias epilogue; the table still holds call 1's entries
    shapes2 = [(300, 520, 200), (64, 100, 72), (1000, 256, 512)]
    _run_both(shapes2, seed=2, with_bias=True)


def test_noalloc_rejects_more_groups_than_the_fixed_table_holds(cuda_device):
    n = capi.CKB_NOALLOC_MAX_GROUPS + 1
    t = torch.zeros((128, 64), dtype=torch.float16, device="cuda")
    op = ck.DeviceGroupedGemm()
    arg = op.MakeArgument([t.data_ptr()] * n, [t.data_ptr()] * n, [], [t.data_ptr()] * n,
                          [ck.GemmDescHost(128, 64, 64, 64, 64, 64)] * n)
    rc = capi.lib().ckb_grouped_gemm_run_noalloc(ctypes.byref(arg.desc), None)
    assert rc == capi.CKB_ERR_LIMIT
    assert str(capi.CKB_NOALLOC_MAX_GROUPS) in capi.last_error()
