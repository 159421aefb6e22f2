"""GPU parity tests of the bfloat16 instances (ck::bhalf_t) against the CPU oracle.

The reference's bf16 tests use integer-valued inputs (test/gemm/gemm_bf16.cpp with GeneratorTensor_2),
for which the fp32 sum is exact and device == host bit for bit; that is asserted here.  With real-valued
inputs a different accumulation order can move the single final rounding by one bfloat16 ulp
(2^-8 relative), which is above check_err's rtol = 1e-3, so those cases allow one ulp."""
import numpy as np
import pytest
import torch

import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from oracle import ck_oracle as oracle

pytestmark = pytest.mark.gpu


def dev_bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda()


def run_gemm_bf16(a_bits, bt_bits, op=None, d0_bits=None, d1_bits=None):
    op = op or ck.PassThrough()
    M, K = a_bits.shape
    N = bt_bits.shape[0]
    da, db = dev_bf16(a_bits), dev_bf16(bt_bits)
    e = torch.zeros((M, N), dtype=torch.int16, device="cuda")
    keep, ds, lds = [], [], []
    for d in (d0_bits, d1_bits):
        if d is not None:
            t = dev_bf16(d)
            keep.append(t)
            ds.append(t.data_ptr())
            lds.append(0 if d.ndim == 1 else d.shape[1])
    gemm = ck.DeviceGemmMultipleD(capi.CKB_BF16)
    arg = gemm.MakeArgument(da.data_ptr(), db.data_ptr(), ds, e.data_ptr(), M, N, K, K, K, lds, N, None, None, op)
    assert gemm.IsSupportedArgument(arg), capi.last_error()
    gemm.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    return e.cpu().numpy().view(np.uint16)


def assert_within_one_ulp(out_bits, ref_bits):
    o, r = oracle.from_bf16(out_bits), oracle.from_bf16(ref_bits)
    ulp = np.maximum(np.abs(r), 2.0 ** -126) * 2.0 ** -7  # spacing of bfloat16 at |r| is at most |r| * 2^-7
    assert np.all(np.abs(o - r) <= ulp + 1e-3), float(np.max(np.abs(o - r) - ulp))


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (300, 520, 200), (1024, 1024, 1024), (129, 72, 136)])
def test_gemm_bf16_integer_inputs_bit_exact(cuda_device, M, N, K):
    rng = np.random.default_rng(M + N + K)
    a = oracle.to_bf16(rng.integers(-5, 6, (M, K)).astype(np.float32))
    bt = oracle.to_bf16(rng.integers(-5, 6, (N, K)).astype(np.float32))
    out = run_gemm_bf16(a, bt)
    np.testing.assert_array_equal(out, oracle.gemm(a, bt.T))


def test_gemm_bf16_real_inputs_and_epilogues(cuda_device):
    rng = np.random.default_rng(3)
    M, N, K = 384, 512, 256
    a = oracle.to_bf16(rng.uniform(-1, 1, (M, K)).astype(np.float32))
    bt = oracle.to_bf16(rng.uniform(-1, 1, (N, K)).astype(np.float32))
    bias = oracle.to_bf16(rng.uniform(-1, 1, (N,)).astype(np.float32))
    full = oracle.to_bf16(rng.uniform(-1, 1, (M, N)).astype(np.float32))
    for op, d0, d1 in [(ck.PassThrough(), None, None), (ck.Relu(), None, None), (ck.Scale(0.5), None, None),
                       (ck.FastGelu(), None, None), (ck.AddRelu(), bias, None), (ck.AddHardswish(), bias, None),
                       (ck.AddReluAdd(), bias, full)]:
        out = run_gemm_bf16(a, bt, op, d0, d1)
        d0v = None if d0 is None else np.broadcast_to(d0, (M, N))
        ref = oracle.gemm(a, bt.T, op.kind, op.params, d0v, d1)
        assert_within_one_ulp(out, ref)
        assert (out == ref).mean() > 0.97  # the rounding moves only where the fp32 sums differ


def test_bf16_functors_without_instances_are_unsupported(cuda_device):
    gemm = ck.DeviceGemmMultipleD(capi.CKB_BF16)
    arg = gemm.MakeArgument(0x1000, 0x2000, [0x3000], 0x4000, 256, 256, 256, 256, 256, [0], 256, None, None, ck.Add())
    assert not gemm.IsSupportedArgument(arg)


def test_conv_bf16_bias_relu(cuda_device):
    rng = np.random.default_rng(8)
    N, C, Hi, Wi, K = 2, 64, 15, 15, 128
    inp = oracle.to_bf16(rng.integers(-3, 4, (N, Hi, Wi, C)).astype(np.float32))
    wei = oracle.to_bf16(rng.integers(-3, 4, (K, 3, 3, C)).astype(np.float32))
    bias = oracle.to_bf16(rng.integers(-3, 4, (K,)).astype(np.float32))
    Ho = Wo = 8
    di, dw, db = dev_bf16(inp), dev_bf16(wei), dev_bf16(bias)
    out = torch.zeros((N, Ho, Wo, K), dtype=torch.int16, device="cuda")
    conv = ck.DeviceConvFwd(capi.CKB_BF16)
    arg = conv.MakeArgument(di.data_ptr(), dw.data_ptr(), out.data_ptr(), N, K, C, (Hi, Wi), (3, 3), (Ho, Wo),
                            (2, 2), (1, 1), (1, 1), (1, 1), None, None, ck.AddRelu(), p_bias=db.data_ptr())
    assert conv.IsSupportedArgument(arg), capi.last_error()
    conv.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    ref = oracle.conv2d_fwd(inp, wei, (2, 2), (1, 1), (1, 1), epilogue=oracle.EPI_ADD_RELU, bias=bias)
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint16), ref)


def test_grouped_bf16(cuda_device):
    rng = np.random.default_rng(9)
    shapes = [(256, 384, 128), (130, 72, 64), (512, 256, 320)]
    As = [oracle.to_bf16(rng.integers(-4, 5, (m, k)).astype(np.float32)) for m, n, k in shapes]
    Bs = [oracle.to_bf16(rng.integers(-4, 5, (n, k)).astype(np.float32)) for m, n, k in shapes]
    dA, dB = [dev_bf16(x) for x in As], [dev_bf16(x) for x in Bs]
    dE = [torch.zeros((m, n), dtype=torch.int16, device="cuda") for m, n, k in shapes]
    gg = ck.DeviceGroupedGemm(capi.CKB_BF16)
    arg = gg.MakeArgument([x.data_ptr() for x in dA], [x.data_ptr() for x in dB], [], [x.data_ptr() for x in dE],
                          [ck.GemmDescHost(m, n, k, k, k, n) for m, n, k in shapes])
    ws = torch.empty(gg.GetWorkSpaceSize(arg), dtype=torch.uint8, device="cuda")
    gg.SetWorkSpacePointer(arg, ws.data_ptr())
    assert gg.IsSupportedArgument(arg), capi.last_error()
    gg.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    for i in range(len(shapes)):
        np.testing.assert_array_equal(dE[i].cpu().numpy().view(np.uint16), oracle.gemm(As[i], Bs[i].T))
