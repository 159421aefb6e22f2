"""Shared helpers of the GPU parity tests: seeded inputs, device round trips through the C ABI,
and comparison against the CPU oracle with the reference's check_err rule."""
from __future__ import annotations

import numpy as np
import torch

import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from oracle import ck_oracle as oracle


def to_dev(x: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def rand_f16(rng, shape, kind="real"):
    if kind == "int":  # integers in [-5, 5]
        return rng.integers(-5, 6, size=shape).astype(np.float16)
    return rng.uniform(-1.0, 1.0, size=shape).astype(np.float16)


def run_gemm(a: np.ndarray, bt: np.ndarray, op: ck.ElementOp = None, d0=None, d1=None,
             ldd0=None, lde=None, time_kernel=False):
    """a: (M,K) row-major; bt: (N,K) = column-major B.  d0: (N,) bias (stride 0) or (M,N); d1: (M,N).
    Returns (E as numpy, avg_ms)."""
    op = op or ck.PassThrough()
    M, K = a.shape
    N = bt.shape[0]
    dtype = capi.CKB_I8 if a.dtype == np.int8 else capi.CKB_F16
    da, db = to_dev(a), to_dev(bt)
    lde = lde or N
    e = torch.full((M, lde), -77 if dtype == capi.CKB_I8 else float("nan"),
                   dtype=torch.int8 if dtype == capi.CKB_I8 else torch.float16, device="cuda")
    ds, lds, keep = [], [], []
    for d in (d0, d1):
        if d is None:
            continue
        t = to_dev(d)
        keep.append(t)
        ds.append(t.data_ptr())
        lds.append(0 if d.ndim == 1 else d.shape[1])
    gemm = ck.DeviceGemmMultipleD(dtype)
    arg = gemm.MakeArgument(da.data_ptr(), db.data_ptr(), ds, e.data_ptr(), M, N, K, a.shape[1],
                            bt.shape[1], lds, lde, None, None, op)
    assert gemm.IsSupportedArgument(arg), capi.last_error()
    ms = gemm.MakeInvoker().Run(arg, ck.StreamConfig(None, time_kernel))
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    out = e.cpu().numpy()
    return out, ms


def oracle_gemm(a, bt, op=None, d0=None, d1=None, fast=True):
    op = op or ck.PassThrough()
    M, N = a.shape[0], bt.shape[0]
    d0v = None if d0 is None else (np.broadcast_to(d0, (M, N)) if d0.ndim == 1 else d0)
    return oracle.gemm(a, bt.T, op.kind, op.params, d0v, d1, fast=fast)


def assert_close(out, ref, rtol=1e-3, atol=1e-3):
    """ck::utils::check_err rule (check_err.hpp:107-193): f16 rtol=atol=1e-3, integers exact."""
    bad, max_err = oracle.check_err(out, ref, rtol, atol)
    assert bad == 0, f"{bad} of {out.size} elements differ, max err {max_err}"
