"""GPU test of the kernel's give-up path: a bounded wait that runs out.

Every wait inside the kernel (mbarriers, the arrival counters of the K-split reduction, the flags of the balanced K
ranges) is a polling loop with a time limit; when it expires the waiting thread records a code in the device status word, the roles of its CTA drain and
the kernel returns, so that the context stays usable.  Here a test hook makes the reductions of a K-split GEMM wait
for one arrival more than will ever come (CKB_TEST_KSLICE_WAIT_EXTRA=1) under a limit of a few milliseconds
(CKB_WAIT_LIMIT_MS): every copy and MMA of the launch completes normally, only that wait gives up.  Nothing faults,
traps or spins without a limit.  The case runs in a child process because the limit is read once per process."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import ctypes, os, sys
import numpy as np
import torch
sys.path.insert(0, os.environ["CKB_REPO_ROOT"])
import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from oracle import ck_oracle as oracle

torch.cuda.set_device(0)
rng = np.random.default_rng(6)
M, N, K = 2048, 2560, 2560         # 80 pair tiles on 74 pairs: the 6 tail tiles are cut along K, parked and summed
a = rng.integers(-5, 6, (M, K)).astype(np.float16)
bt = rng.integers(-5, 6, (N, K)).astype(np.float16)
da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
e = torch.zeros((M, N), dtype=torch.float16, device="cuda")
g = ck.DeviceGemm(capi.CKB_F16)
arg = g.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), M, N, K, K, K, N)
ref = oracle.gemm(a, bt.T)

def status():
    w = ctypes.c_uint32(0)
    rc = capi.lib().ckb_device_status(ctypes.byref(w))
    return rc, w.value

# 1. a normal launch under the short limit: nothing expires
g.MakeInvoker().Run(arg)
assert "ksplit=4" in capi.last_plan() and "cluster_k=0" in capi.last_plan(), capi.last_plan()
rc, w = status()
assert (rc, w) == (capi.CKB_OK, 0), (rc, w)
assert (e.cpu().numpy() == ref).all()

# 2. the reductions wait for an arrival that never comes: the wait runs out, the kernel returns
os.environ["CKB_TEST_KSLICE_WAIT_EXTRA"] = "1"
e.zero_()
g.MakeInvoker().Run(arg)
rc, w = status()
assert rc == capi.CKB_ERR_DEVICE, (rc, w)
assert w >> 24 == 6, hex(w)                      # WAIT_KSLICES
assert "timed out" in capi.last_error()
rc, w = status()                                 # reading cleared the word
assert (rc, w) == (capi.CKB_OK, 0), (rc, w)

# 3. the same process keeps working: counters were reset, results are bit exact again (twice: the second launch
#    finds the counters as the first left them)
del os.environ["CKB_TEST_KSLICE_WAIT_EXTRA"]
for _ in range(2):
    e.zero_()
    g.MakeInvoker().Run(arg)
    rc, w = status()
    assert (rc, w) == (capi.CKB_OK, 0), (rc, w)
    assert (e.cpu().numpy() == ref).all()

# 4. the same for the flag waits of the balanced K ranges (pinned: 40 pair tiles dealt out over 74 pairs)
M, N, K = 1280, 2048, 2048
a = rng.integers(-5, 6, (M, K)).astype(np.float16)
bt = rng.integers(-5, 6, (N, K)).astype(np.float16)
da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
e = torch.zeros((M, N), dtype=torch.float16, device="cuda")
g = ck.DeviceGemm(capi.CKB_F16, tile_config=capi.tile_config(256, 2, balanced=1))
arg = g.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), M, N, K, K, K, N)
ref = oracle.gemm(a, bt.T)
g.MakeInvoker().Run(arg)
assert "balanced=0" not in capi.last_plan(), capi.last_plan()
assert status() == (capi.CKB_OK, 0)
assert (e.cpu().numpy() == ref).all()
os.environ["CKB_TEST_KSLICE_WAIT_EXTRA"] = "1"
g.MakeInvoker().Run(arg)
rc, w = status()
assert rc == capi.CKB_ERR_DEVICE and w >> 24 == 6, (rc, hex(w))
del os.environ["CKB_TEST_KSLICE_WAIT_EXTRA"]
for _ in range(2):                               # flags were cleared: bit exact again
    e.zero_()
    g.MakeInvoker().Run(arg)
    assert status() == (capi.CKB_OK, 0)
    assert (e.cpu().numpy() == ref).all()
print("wait-limit case passed")
'''


def test_a_bounded_wait_that_runs_out_is_reported_and_the_context_stays_usable(cuda_device):
    env = dict(os.environ, CKB_WAIT_LIMIT_MS="5", CKB_REPO_ROOT=ROOT)
    env.pop("CKB_TEST_KSLICE_WAIT_EXTRA", None)
    res = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert "wait-limit case passed" in res.stdout
