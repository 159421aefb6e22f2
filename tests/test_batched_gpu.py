"""GPU parity tests of batched GEMM (DeviceBatchedGemm, device/device_batched_gemm.hpp:15-44) against the CPU
oracle applied batch by batch.  The reference's test (test/batched_gemm/batched_gemm_fp16.cpp and
profiler/include/profile_batched_gemm_impl.hpp) uses BatchStride = rows * stride of one matrix and
integer-valued inputs; both the packed and a padded batch stride are covered here, with bit-exact comparison."""
import numpy as np
import pytest
import torch

import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from oracle import ck_oracle as oracle

pytestmark = pytest.mark.gpu

ROW, COL = capi.CKB_ROW_MAJOR, capi.CKB_COL_MAJOR


def run_batched(dtype, a_layout, b_layout, a, b, pad=0, op=None):
    """a: (G, M, K) logical, b: (G, K, N) logical.  Returns E (G, M, N)."""
    G, M, K = a.shape
    N = b.shape[2]
    a_img = np.ascontiguousarray(a.transpose(0, 2, 1) if a_layout == COL else a)
    b_img = np.ascontiguousarray(b.transpose(0, 2, 1) if b_layout == COL else b)
    lda, ldb = a_img.shape[2], b_img.shape[2]
    bsa, bsb, bse = a_img.shape[1] * lda + pad, b_img.shape[1] * ldb + pad, M * N + pad

    def image(x, bs):  # batches `bs` elements apart
        flat = np.zeros(G * bs, dtype=x.dtype)
        for g in range(G):
            flat[g * bs:g * bs + x[g].size] = x[g].ravel()
        t = torch.from_numpy(flat.view(np.int16) if flat.dtype == np.uint16 else flat)
        return t.cuda()

    da, db = image(a_img, bsa), image(b_img, bsb)
    tdt = {capi.CKB_I8: torch.int8, capi.CKB_F16: torch.float16, capi.CKB_BF16: torch.int16}[dtype]
    e = torch.zeros(G * bse, dtype=tdt, device="cuda")
    op_ = ck.DeviceBatchedGemm(dtype, a_layout, b_layout)
    arg = op_.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), M, N, K, lda, ldb, N, bsa, bsb, bse, G,
                           None, None, op or ck.PassThrough())
    assert op_.IsSupportedArgument(arg), capi.last_error()
    op_.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    assert ck.device_status() == 0
    out = e.cpu().numpy()
    out = out.view(np.uint16) if dtype == capi.CKB_BF16 else out
    return np.stack([out[g * bse:g * bse + M * N].reshape(M, N) for g in range(G)])


def inputs(rng, dtype, G, M, N, K):
    a = rng.integers(-5, 6, (G, M, K))
    b = rng.integers(-5, 6, (G, K, N))
    if dtype == capi.CKB_I8:
        return a.astype(np.int8), b.astype(np.int8)
    if dtype == capi.CKB_BF16:
        return oracle.to_bf16(a.astype(np.float32)), oracle.to_bf16(b.astype(np.float32))
    return a.astype(np.float16), b.astype(np.float16)


def oracle_batched(a, b, op=None):
    op = op or ck.PassThrough()
    return np.stack([oracle.gemm(a[g], b[g], op.kind, op.params) for g in range(a.shape[0])])


@pytest.mark.parametrize("dtype", [capi.CKB_F16, capi.CKB_BF16, capi.CKB_I8], ids=["f16", "bf16", "i8"])
@pytest.mark.parametrize("layouts", [(ROW, COL), (ROW, ROW), (COL, ROW), (COL, COL)], ids=["mk_nk", "mk_kn", "km_kn", "km_nk"])
@pytest.mark.parametrize("G,M,N,K,pad", [(4, 256, 128, 64, 0), (3, 208, 144, 80, 32), (16, 128, 256, 128, 0)])
def test_batched_gemm_bit_exact(cuda_device, dtype, layouts, G, M, N, K, pad):
    rng = np.random.default_rng(G * 1000 + M + N + K + dtype)
    a, b = inputs(rng, dtype, G, M, N, K)
    out = run_batched(dtype, layouts[0], layouts[1], a, b, pad)
    np.testing.assert_array_equal(out, oracle_batched(a, b))


def test_batched_gemm_fills_the_machine_with_cta_pairs(cuda_device):
    """64 batches of 512 x 512 x 256: 512 tiles of 128 x 256, run as CTA pairs with a split tail wave."""
    rng = np.random.default_rng(1)
    a, b = inputs(rng, capi.CKB_F16, 64, 512, 512, 256)
    out = run_batched(capi.CKB_F16, ROW, COL, a, b)
    np.testing.assert_array_equal(out, oracle_batched(a, b))


def test_batched_gemm_unaligned_output_batch_stride_uses_scalar_stores(cuda_device):
    rng = np.random.default_rng(2)
    a, b = inputs(rng, capi.CKB_F16, 3, 128, 64, 64)
    out = run_batched(capi.CKB_F16, ROW, COL, a.copy(), b.copy(), pad=8)  # aligned
    ref = oracle_batched(a, b)
    np.testing.assert_array_equal(out, ref)
    # E batches 4 elements (8 bytes) off the 16-byte grid: A/B strides stay aligned, E falls back to scalar stores
    G, M, K = a.shape
    N = b.shape[2]
    da = torch.from_numpy(a).cuda()
    db = torch.from_numpy(np.ascontiguousarray(b.transpose(0, 2, 1))).cuda()
    bse = M * N + 4
    e = torch.zeros(G * bse, dtype=torch.float16, device="cuda")
    op_ = ck.DeviceBatchedGemm(capi.CKB_F16)
    arg = op_.MakeArgument(da.data_ptr(), db.data_ptr(), e.data_ptr(), M, N, K, K, K, N, M * K, N * K, bse, G)
    assert op_.IsSupportedArgument(arg), capi.last_error()
    op_.MakeInvoker().Run(arg)
    torch.cuda.synchronize()
    out = e.cpu().numpy()
    for g in range(G):
        np.testing.assert_array_equal(out[g * bse:g * bse + M * N].reshape(M, N), ref[g])


def test_batched_gemm_rejects_bad_batch_arguments(cuda_device):
    op_ = ck.DeviceBatchedGemm(capi.CKB_F16)
    ok = op_.MakeArgument(0x1000, 0x2000, 0x3000, 128, 128, 64, 64, 64, 128, 128 * 64, 128 * 64, 128 * 128, 4)
    assert op_.IsSupportedArgument(ok)
    assert not op_.IsSupportedArgument(
        op_.MakeArgument(0x1000, 0x2000, 0x3000, 128, 128, 64, 64, 64, 128, 128 * 64, 128 * 64, 128 * 128, 0))
    assert not op_.IsSupportedArgument(
        op_.MakeArgument(0x1000, 0x2000, 0x3000, 128, 128, 64, 64, 64, 128, 128 * 64 + 4, 128 * 64, 128 * 128, 4))
    assert "16 bytes" in capi.last_error()
