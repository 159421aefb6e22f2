"""GPU test of CKB_SM_LIMIT: a process that may use only part of the GPU (an MPS active-thread percentage, a green
context) tells the library how many SMs its launches can count on, because the K-split plans let CTAs wait for one
another and need every CTA of a launch resident at once.  With the limit set, every plan is made for that many
persistent CTAs; results must not change.  The limit is read once per process, so the cases run in a child process."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import os, sys
import numpy as np
import torch
sys.path.insert(0, os.environ["CKB_REPO_ROOT"])
import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from oracle import ck_oracle as oracle

torch.cuda.set_device(0)
limit = int(os.environ["CKB_SM_LIMIT"])
rng = np.random.default_rng(limit)
g = ck.DeviceGemm(capi.CKB_F16)
# whole waves + a K-split tail, a column-slice tail (short K), a cluster K split, a single small tile
for M, N, K in [(2048, 2560, 2560), (2048, 2560, 512), (256, 256, 8192), (300, 200, 72), (3840, 4096, 1024)]:
    a = rng.integers(-5, 6, (M, K)).astype(np.float16)
    bt = rng.integers(-5, 6, (N, K)).astype(np.float16)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    e = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    arg = g.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), M, N, K, K, K, N)
    for _ in range(2):
        g.MakeInvoker().Run(arg)
    plan = capi.last_plan()
    grid = int(plan.split("grid=")[1].split()[0])
    assert "cluster_k=0" not in plan or grid <= limit, plan     # persistent plans never launch more CTAs than the limit
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    assert (e.cpu().numpy() == oracle.gemm(a, bt.T)).all(), (M, N, K, plan)
# the convolution and the grouped GEMM plan for the same number of units
inp = rng.integers(-3, 4, (8, 30, 30, 64)).astype(np.float16)
wei = rng.integers(-3, 4, (256, 3, 3, 64)).astype(np.float16)
di, dw = torch.from_numpy(inp).cuda(), torch.from_numpy(wei).cuda()
out = torch.zeros((8, 15, 15, 256), dtype=torch.float16, device="cuda")
conv = ck.DeviceConvFwd()
carg = conv.MakeArgument(di.data_ptr(), dw.data_ptr(), out.data_ptr(), 8, 256, 64, (30, 30), (3, 3), (15, 15), (2, 2), (1, 1),
                         (1, 1), (1, 1))
conv.MakeInvoker().Run(carg)
assert int(capi.last_plan().split("grid=")[1].split()[0]) <= limit, capi.last_plan()
torch.cuda.synchronize()
assert ck.device_status() == 0
assert (out.cpu().numpy() == oracle.conv2d_fwd(inp, wei, (2, 2), (1, 1), (1, 1))).all()
print("sm-limit case passed")
'''


@pytest.mark.parametrize("limit", [74, 100, 20])
def test_plans_for_a_part_of_the_gpu_give_the_same_results(cuda_device, limit):
    env = dict(os.environ, CKB_SM_LIMIT=str(limit), CKB_REPO_ROOT=ROOT)
    res = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert "sm-limit case passed" in res.stdout
