"""GPU parity tests of the GEMM path: CUDA kernels (through the C ABI) vs the CPU oracle.

Tolerances are the reference's (check_err.hpp:107-193): binary16 rtol = atol = 1e-3, integers
exact; integer-valued binary16 inputs must additionally match bit for bit."""
import numpy as np
import pytest
import torch

import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from oracle import ck_oracle as oracle
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [
    (128, 256, 64),      # one tile, one k block
    (128, 256, 256),
    (1, 8, 8),           # smallest rows
    (100, 200, 72),      # ragged in M, N and K
    (300, 520, 1000),    # several tiles, K tail
    (129, 257, 136),     # one past the tile edge
    (128, 64, 64),       # narrow tile (BN = 64)
    (128, 128, 128),     # BN = 128
    (1024, 1024, 1024),  # the reference's TestGemm size (test/gemm/gemm_util.hpp:150-158)
])
def test_gemm_f16_passthrough(cuda_device, M, N, K):
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    a, bt = H.rand_f16(rng, (M, K)), H.rand_f16(rng, (N, K))
    out, _ = H.run_gemm(a, bt)
    H.assert_close(out, H.oracle_gemm(a, bt))
    # GeneratorTensor_2{-5,5}-style integer inputs: order of accumulation cannot matter
    a, bt = H.rand_f16(rng, (M, K), "int"), H.rand_f16(rng, (N, K), "int")
    out, _ = H.run_gemm(a, bt)
    np.testing.assert_array_equal(out.view(np.uint16), H.oracle_gemm(a, bt).view(np.uint16))


EPILOGUES = [
    (ck.PassThrough, (), 0), (ck.Relu, (), 0), (ck.Scale, (0.25,), 0), (ck.FastGelu, (), 0),
    (ck.Add, (), 1), (ck.AddReluF16, (), 1), (ck.AddRelu, (), 1), (ck.AddHardswish, (), 1),
    (ck.Bilinear, (0.5, 2.0), 1), (ck.AddAddFastGelu, (), 2), (ck.AddReluAdd, (), 2),
]


@pytest.mark.parametrize("op_cls,args,nd", EPILOGUES)
@pytest.mark.parametrize("shape", [(256, 512, 256), (130, 72, 200)])
def test_gemm_f16_fused_epilogues(cuda_device, op_cls, args, nd, shape):
    M, N, K = shape
    rng = np.random.default_rng(11)
    a, bt = H.rand_f16(rng, (M, K)), H.rand_f16(rng, (N, K))
    bias, full = H.rand_f16(rng, (N,)), H.rand_f16(rng, (M, N))
    op = op_cls(*args)
    # one D: alternate between the broadcast row (stride 0) and a full matrix
    d0 = None if nd == 0 else (full if op_cls is ck.Bilinear else bias)
    d1 = full if nd == 2 else None
    out, _ = H.run_gemm(a, bt, op, d0, d1)
    ref = H.oracle_gemm(a, bt, op, d0, d1)
    if op_cls in (ck.Add, ck.AddReluF16):
        # These functors round the accumulator to binary16 BEFORE adding D (binary_element_wise_
        # operation.hpp:31-36), so a last-bit difference of the fp32 sum (accumulation order) moves
        # the binary16 sum by one ulp of |c| - two ulps when both sums are ties that round to even in
        # opposite directions - which can exceed rtol*|e|.  The check therefore adds one binary16
        # spacing of max(|e|, |c|) to the reference's bound.
        c = H.oracle_gemm(a, bt).astype(np.float32)
        o, r = out.astype(np.float32), ref.astype(np.float32)
        ulp = np.spacing(np.maximum(np.abs(r), np.abs(c)).astype(np.float16)).astype(np.float32)
        assert np.all(np.abs(o - r) <= 1e-3 + 1e-3 * np.abs(r) + ulp)
    else:
        H.assert_close(out, ref)


def test_device_epilogue_equals_host_functor_elementwise(cuda_device):
    """Pins each device epilogue to its host functor value by value: A = one column holding the
    accumulator values, B = a row of ones, so acc[m, n] = c[m] exactly."""
    M, N, K = 256, 64, 8
    rng = np.random.default_rng(3)
    c = np.concatenate([np.linspace(-8, 8, 200), [2049.0, -2049.0, 0.0, 1e-4, 6.0, -3.0, 3.0, 0.5],
                        rng.uniform(-70, 70, 48)]).astype(np.float16)
    a = np.zeros((M, K), np.float16)
    a[:, 0] = c
    bt = np.zeros((N, K), np.float16)
    bt[:, 0] = 1
    d0 = rng.uniform(-2, 2, (M, N)).astype(np.float16)
    d1 = rng.uniform(-2, 2, (M, N)).astype(np.float16)
    exact_ops = [ck.PassThrough(), ck.Relu(), ck.Scale(0.25), ck.Add(), ck.AddReluF16(), ck.AddRelu(),
                 ck.AddHardswish(), ck.Bilinear(0.5, 2.0), ck.AddReluAdd()]
    for op in exact_ops:  # no transcendental: must agree to the bit
        nd = capi.EPI_NUM_D.get(op.kind, 0)
        dd0, dd1 = (d0 if nd >= 1 else None), (d1 if nd >= 2 else None)
        out, _ = H.run_gemm(a, bt, op, dd0, dd1)
        ref = H.oracle_gemm(a, bt, op, dd0, dd1, fast=False)
        np.testing.assert_array_equal(out.view(np.uint16), ref.view(np.uint16), err_msg=type(op).__name__)
    for op in (ck.FastGelu(), ck.AddAddFastGelu()):  # expf vs exp: one binary16 ulp at most
        nd = capi.EPI_NUM_D.get(op.kind, 0)
        dd0, dd1 = (d0 if nd >= 1 else None), (d1 if nd >= 2 else None)
        out, _ = H.run_gemm(a, bt, op, dd0, dd1)
        ref = H.oracle_gemm(a, bt, op, dd0, dd1, fast=False)
        H.assert_close(out, ref)
        ulp = np.abs(out.view(np.int16).astype(np.int32) - ref.view(np.int16).astype(np.int32))
        assert ulp.max() <= 1


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 512), (200, 300, 272), (1, 16, 16), (1024, 1024, 1024)])
def test_gemm_int8_bit_exact(cuda_device, M, N, K):
    rng = np.random.default_rng(K)
    a = rng.integers(-5, 6, (M, K)).astype(np.int8)
    bt = rng.integers(-5, 6, (N, K)).astype(np.int8)
    for op in (ck.PassThrough(), ck.Relu(), ck.RequantReluRequant(0.03, 1.0), ck.RequantReluRequantRne(0.03, 14.0)):
        out, _ = H.run_gemm(a, bt, op)
        np.testing.assert_array_equal(out, H.oracle_gemm(a, bt, op), err_msg=type(op).__name__)


@pytest.mark.parametrize("kind", ["int8", "f16"])
def test_pair_tail_cut_into_four_ragged_column_slices(cuda_device, kind):
    """2560 x 2000: 80 pair tiles of 256 x 256 on 74 CTA pairs leave 6 tail tiles, each cut into four 64-column
    slices (32 B rows per CTA); the last column tile has 208 valid columns, so its fourth slice holds 16 of them.
    A column of canaries beside E (leading dimension 2008) must survive."""
    rng = np.random.default_rng(2560)
    M, N, K = 2560, 2000, 320
    if kind == "int8":
        a = rng.integers(-5, 6, (M, K)).astype(np.int8)
        bt = rng.integers(-5, 6, (N, K)).astype(np.int8)
        op = ck.RequantReluRequantRne(0.03, 14.0)
        d0 = None
    else:
        # a functor that reads a D tensor keeps the column-slice tail (D-less 16-bit GEMMs cut their tail along K)
        a, bt = H.rand_f16(rng, (M, K), "int"), H.rand_f16(rng, (N, K), "int")
        op, d0 = ck.AddRelu(), H.rand_f16(rng, (N,), "int")
    out, _ = H.run_gemm(a, bt, op, d0=d0, lde=N + 8)
    ref = H.oracle_gemm(a, bt, op, d0=d0)
    if kind == "int8":
        np.testing.assert_array_equal(out[:, :N], ref)
        assert (out[:, N:] == -77).all()
    else:
        np.testing.assert_array_equal(out[:, :N].view(np.uint16), ref.view(np.uint16))
        assert np.isnan(out[:, N:]).all()


def test_gemm_int8_full_range_inputs(cuda_device):
    """Full int8 range: accumulators exceed 2^24, PassThrough keeps the low byte of the int32 sum."""
    rng = np.random.default_rng(9)
    M, N, K = 128, 128, 2048
    a = rng.integers(-128, 128, (M, K)).astype(np.int8)
    bt = rng.integers(-128, 128, (N, K)).astype(np.int8)
    out, _ = H.run_gemm(a, bt)
    ref = (a.astype(np.int64) @ bt.T.astype(np.int64)).astype(np.int32).astype(np.int8)
    np.testing.assert_array_equal(out, ref)


def test_output_leading_dimension_and_canary(cuda_device):
    """E with lde > N: the padding columns must stay untouched (canary), ragged tile edges included."""
    rng = np.random.default_rng(21)
    M, N, K, lde = 200, 300, 136, 320
    a, bt = H.rand_f16(rng, (M, K)), H.rand_f16(rng, (N, K))
    out, _ = H.run_gemm(a, bt, lde=lde)
    H.assert_close(np.ascontiguousarray(out[:, :N]), H.oracle_gemm(a, bt))
    assert np.isnan(out[:, N:]).all()


def test_unaligned_output_uses_scalar_path(cuda_device):
    rng = np.random.default_rng(22)
    M, N, K = 130, 77, 64  # lde = 77: rows are not 16-byte aligned
    a, bt = H.rand_f16(rng, (M, K)), H.rand_f16(rng, (N, K))
    bias = H.rand_f16(rng, (N,))
    out, _ = H.run_gemm(a, bt, ck.AddRelu(), bias)
    H.assert_close(out, H.oracle_gemm(a, bt, ck.AddRelu(), bias))


def test_full_size_fp16_gemm_bit_exact(cuda_device):
    """3840 x 4096 x 4096, integer inputs in [-5, 5]: every output verified, bit for bit."""
    rng = np.random.default_rng(11939 + 1000)
    M, N, K = 3840, 4096, 4096
    a, bt = H.rand_f16(rng, (M, K), "int"), H.rand_f16(rng, (N, K), "int")
    out, ms = H.run_gemm(a, bt, time_kernel=True)
    assert ms > 0
    np.testing.assert_array_equal(out.view(np.uint16), H.oracle_gemm(a, bt).view(np.uint16))


def test_full_size_int8_requant_bit_exact(cuda_device):
    rng = np.random.default_rng(11939 + 2000)
    M, N, K = 3840, 4096, 4096
    a = rng.integers(-5, 6, (M, K)).astype(np.int8)
    bt = rng.integers(-5, 6, (N, K)).astype(np.int8)
    for op in (ck.RequantReluRequantRne(0.03, 14.0), ck.RequantReluRequant(0.03, 1.0)):
        out, _ = H.run_gemm(a, bt, op)
        ref = H.oracle_gemm(a, bt, op)
        np.testing.assert_array_equal(out, ref)
    # sanity of the value distribution: about half zeros, a saturated tail
    assert 0.3 < (ref == 0).mean() < 0.7


def test_full_size_add_add_fastgelu(cuda_device):
    rng = np.random.default_rng(11939 + 3000)
    M, N, K = 3840, 4096, 4096
    a, bt = H.rand_f16(rng, (M, K)), H.rand_f16(rng, (N, K))
    d0, d1 = H.rand_f16(rng, (N,)), H.rand_f16(rng, (M, N))
    out, _ = H.run_gemm(a, bt, ck.AddAddFastGelu(), d0, d1)
    H.assert_close(out, H.oracle_gemm(a, bt, ck.AddAddFastGelu(), d0, d1))


def test_linearity_property_at_full_size(cuda_device):
    """Size-independent property: with integer inputs, gemm(2A, B) == 2 * gemm(A, B) exactly."""
    rng = np.random.default_rng(5)
    M, N, K = 3840, 4096, 4096
    a = rng.integers(-2, 3, (M, K)).astype(np.float16)
    bt = rng.integers(-2, 3, (N, K)).astype(np.float16)
    e1, _ = H.run_gemm(a, bt)
    e2, _ = H.run_gemm((2 * a).astype(np.float16), bt)
    np.testing.assert_array_equal(e2.astype(np.float32), 2 * e1.astype(np.float32))


def test_run_returns_zero_without_timing_and_counts_launches(cuda_device):
    rng = np.random.default_rng(1)
    a, bt = H.rand_f16(rng, (128, 64)), H.rand_f16(rng, (64, 64))
    before = ck.launch_count()
    _, ms = H.run_gemm(a, bt, time_kernel=False)
    assert ms == 0.0 and ck.launch_count() == before + 1
    _, ms = H.run_gemm(a, bt, time_kernel=True)  # 1 warm-up + 10 timed (kernel_launch.hpp:32-61)
    assert ms > 0.0 and ck.launch_count() == before + 12


def test_output_offsets_beyond_2_gib(cuda_device):
    """E of 140 000 x 8192 halves is 2.29 GB: row offsets pass 2^31 bytes, so every address computation of the
    epilogue (staged tile stores and the scalar path of the ragged last rows) has to be 64-bit.  Row blocks at the
    start, around the 2 GiB mark and at the ragged end are compared bit-exactly with the oracle."""
    rng = np.random.default_rng(4242)
    M, N, K = 140_000, 8192, 32
    a = rng.integers(-5, 6, (M, K)).astype(np.float16)
    bt = rng.integers(-5, 6, (N, K)).astype(np.float16)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    e = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    gemm = ck.DeviceGemm(capi.CKB_F16)
    arg = gemm.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), M, N, K, K, K, N, None, None, ck.PassThrough())
    assert gemm.IsSupportedArgument(arg), capi.last_error()
    gemm.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    mark = (1 << 31) // (2 * N)  # first row whose byte offset is past 2 GiB
    for lo, hi in [(0, 256), (mark - 200, mark + 200), (M - 300, M)]:
        np.testing.assert_array_equal(e[lo:hi].cpu().numpy(), oracle.gemm(a[lo:hi], bt.T), err_msg=f"rows {lo}:{hi}")
    # nothing outside the ragged edge was left unwritten: every row has a non-zero element with these inputs
    assert bool((e != 0).any(dim=1).all())
