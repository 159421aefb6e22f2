"""GPU parity tests of the grouped GEMM path against the CPU oracle, group by group."""
import numpy as np
import pytest
import torch

import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from tests import helpers as H

pytestmark = pytest.mark.gpu


def run_grouped(shapes, rng, op=None, with_bias=False, time_kernel=False, kind="real"):
    op = op or ck.PassThrough()
    As = [H.rand_f16(rng, (m, k), kind) for (m, n, k) in shapes]
    Bs = [H.rand_f16(rng, (n, k), kind) for (m, n, k) in shapes]
    biases = [H.rand_f16(rng, (n,)) for (m, n, k) in shapes] if with_bias else None
    dA, dB = [H.to_dev(x) for x in As], [H.to_dev(x) for x in Bs]
    dBias = [H.to_dev(x) for x in biases] if with_bias else None
    dE = [torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda") for (m, n, k) in shapes]
    gg = ck.DeviceGroupedGemm()
    descs = [ck.GemmDescHost(m, n, k, k, k, n, [0] if with_bias else []) for (m, n, k) in shapes]
    p_ds = [[b.data_ptr()] for b in dBias] if with_bias else []
    arg = gg.MakeArgument([x.data_ptr() for x in dA], [x.data_ptr() for x in dB], p_ds,
                          [x.data_ptr() for x in dE], descs, None, None, op)
    ws = torch.empty(gg.GetWorkSpaceSize(arg), dtype=torch.uint8, device="cuda")
    gg.SetWorkSpacePointer(arg, ws.data_ptr())
    assert gg.IsSupportedArgument(arg), capi.last_error()
    ms = gg.MakeInvoker().Run(arg, ck.StreamConfig(None, time_kernel))
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    outs = [e.cpu().numpy() for e in dE]
    refs = [H.oracle_gemm(As[i], Bs[i], op, biases[i] if with_bias else None) for i in range(len(shapes))]
    return outs, refs, ms


def test_small_groups_of_the_reference_example(cuda_device):
    """example/15_grouped_gemm/grouped_gemm_xdl_fp16.cpp:86-106: M = 256+256i, N = 128+128i, K = 64+64i."""
    shapes = [(256 + 256 * i, 128 + 128 * i, 64 + 64 * i) for i in range(4)]
    outs, refs, _ = run_grouped(shapes, np.random.default_rng(0))
    for o, r in zip(outs, refs):
        H.assert_close(o, r)


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_group_sets(cuda_device, seed):
    """test/grouped_gemm/grouped_gemm_fp16.cpp:18-49: 1..10 groups, M,N in 256*[1..10], K in 128*[1..10]."""
    rng = np.random.default_rng(seed)
    n = int(rng.integers(1, 11))
    shapes = [(256 * int(rng.integers(1, 11)), 256 * int(rng.integers(1, 11)), 128 * int(rng.integers(1, 11)))
              for _ in range(n)]
    outs, refs, _ = run_grouped(shapes, rng)
    for o, r in zip(outs, refs):
        H.assert_close(o, r)


def test_ragged_groups_and_single_row_group(cuda_device):
    shapes = [(300, 520, 200), (1, 8, 8), (64, 100, 72), (1000, 256, 512), (129, 264, 1032)]
    outs, refs, _ = run_grouped(shapes, np.random.default_rng(4))
    for o, r in zip(outs, refs):
        H.assert_close(o, r)


def test_grouped_with_bias_add(cuda_device):
    """example/28_grouped_gemm_bias: E_g = Add(C_g, bias_g) with a stride-0 D tensor per group."""
    shapes = [(256, 384, 128), (512, 128, 256), (130, 72, 64)]
    outs, refs, _ = run_grouped(shapes, np.random.default_rng(6), ck.Add(), with_bias=True)
    for o, r in zip(outs, refs):
        # Add rounds the accumulator to binary16 before adding the bias: allow one more binary16
        # spacing of |c| (|c| <= |e| + 1 here since |bias| <= 1).
        o32, r32 = o.astype(np.float32), r.astype(np.float32)
        ulp = np.spacing((np.abs(r32) + 1.0).astype(np.float16)).astype(np.float32)
        assert np.all(np.abs(o32 - r32) <= 1e-3 + 1e-3 * np.abs(r32) + ulp)


def test_integer_inputs_bit_exact(cuda_device):
    shapes = [(256, 512, 256), (768, 256, 640)]
    outs, refs, _ = run_grouped(shapes, np.random.default_rng(8), kind="int")
    for o, r in zip(outs, refs):
        np.testing.assert_array_equal(o.view(np.uint16), r.view(np.uint16))


def test_workspace_too_small_is_an_error(cuda_device):
    gg = ck.DeviceGroupedGemm()
    t = torch.zeros((256, 256), dtype=torch.float16, device="cuda")
    arg = gg.MakeArgument([t.data_ptr()], [t.data_ptr()], [], [t.data_ptr()],
                          [ck.GemmDescHost(256, 256, 256, 256, 256, 256)])
    ws = torch.empty(16, dtype=torch.uint8, device="cuda")
    gg.SetWorkSpacePointer(arg, ws.data_ptr(), 16)
    with pytest.raises(capi.CkbError) as ei:
        gg.MakeInvoker().Run(arg)
    assert ei.value.code == capi.CKB_ERR_WORKSPACE


def _full_size_64_groups(kind):
    """The 64-group configuration (M_g = 256*(1 + g mod 16), N = K = 4096) run once, every group compared with the
    oracle in full - the reference's example sends every group through check_err
    (example/15_grouped_gemm/grouped_gemm_xdl_fp16.cpp:245-246)."""
    G, N, K = 64, 4096, 4096
    Ms = [256 * (1 + g % 16) for g in range(G)]
    gen = torch.Generator(device="cuda").manual_seed(11939 + 5000)

    def make(shape):
        if kind == "int":  # integers in [-5, 5]: every fp32 partial sum is exact, so any summation order agrees
            return torch.randint(-5, 6, shape, generator=gen, device="cuda").to(torch.float16)
        return torch.empty(shape, dtype=torch.float16, device="cuda").uniform_(-1, 1, generator=gen)
    dA = [make((m, K)) for m in Ms]
    dB = [make((N, K)) for _ in Ms]
    dE = [torch.full((m, N), float("nan"), dtype=torch.float16, device="cuda") for m in Ms]
    gg = ck.DeviceGroupedGemm()
    arg = gg.MakeArgument([x.data_ptr() for x in dA], [x.data_ptr() for x in dB], [], [x.data_ptr() for x in dE],
                          [ck.GemmDescHost(m, N, K, K, K, N) for m in Ms])
    ws = torch.empty(gg.GetWorkSpaceSize(arg), dtype=torch.uint8, device="cuda")
    gg.SetWorkSpacePointer(arg, ws.data_ptr())
    assert gg.IsSupportedArgument(arg)
    ms = gg.MakeInvoker().Run(arg, ck.StreamConfig(None, True))
    torch.cuda.synchronize()
    assert ck.device_status() == 0 and ms > 0
    for g in range(G):
        out = dE[g].cpu().numpy()
        ref = H.oracle_gemm(dA[g].cpu().numpy(), dB[g].cpu().numpy())
        if kind == "int":
            np.testing.assert_array_equal(out.view(np.uint16), ref.view(np.uint16), err_msg=f"group {g}")
        else:
            bad, max_err = H.oracle.check_err(out, ref, 1e-3, 1e-3)
            assert bad == 0, f"group {g}: {bad} of {out.size} elements differ, max err {max_err}"


def test_full_size_64_groups(cuda_device):
    """Real-valued operands in [-1, 1]: all 64 groups within the reference's check_err rule (rtol = atol = 1e-3)."""
    _full_size_64_groups("real")


def test_full_size_64_groups_integer_inputs_bit_exact(cuda_device):
    """Integer-valued operands: all 64 groups bit for bit."""
    _full_size_64_groups("int")
