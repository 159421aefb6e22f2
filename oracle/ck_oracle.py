"""TEST INFRASTRUCTURE - ctypes binding of the CPU oracle (oracle/libck_oracle.so).

Only tests/, ``__graft_entry__.smoke()`` and ``bench.py``'s cpu_baseline / reference arm may
import this module.  The shipped package never does: its kernels have no CPU fallback.

The oracle restates Composable Kernel's host reference operators
(library/include/ck/library/reference_tensor_operation/cpu/reference_gemm.hpp:57-88,
reference_conv_fwd.hpp:132-185, reference_conv_fwd_bias_activation.hpp:74-128); see
ck_oracle.cpp for the function-by-function citations.  numpy arrays carry binary16 as
``np.float16`` and int8 as ``np.int8``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libck_oracle.so")

# Epilogue ids: identical to the CKB_EPI_* values of include/ckb200.h (asserted in tests).
EPI_PASSTHROUGH = 0
EPI_SCALE = 1
EPI_RELU = 2
EPI_FASTGELU = 3
EPI_ADD = 4
EPI_ADD_RELU_F16 = 5
EPI_BILINEAR = 6
EPI_ADD_ADD_FASTGELU = 7
EPI_ADD_RELU_ADD = 8
EPI_REQUANT_RELU_REQUANT = 9
EPI_REQUANT_RELU_REQUANT_RNE = 10
EPI_ADD_RELU = 11
EPI_ADD_HARDSWISH = 12


def build(force: bool = False) -> str:
    """Compile libck_oracle.so with the committed Makefile if it is missing or stale."""
    srcs = [os.path.join(_HERE, f) for f in ("ck_oracle.cpp", "ck_oracle_fast.cpp", "ck_epilogue.h", "Makefile")]
    stale = force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in srcs)
    if stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        i64, vp, fp = ctypes.c_int64, ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)
        gemm_args = [ctypes.c_int, ctypes.c_int, fp,
                     vp, i64, i64, vp, i64, i64, vp, i64, i64,
                     vp, i64, i64, vp, i64, i64, i64, i64, i64, ctypes.c_int]
        for name in ("oracle_gemm_naive", "oracle_gemm_fast"):
            getattr(L, name).argtypes = gemm_args
            getattr(L, name).restype = ctypes.c_int
        conv_args = [ctypes.c_int, fp, vp, vp, vp, vp, vp] + [ctypes.c_int] * 16
        for name in ("oracle_conv2d_fwd_naive", "oracle_conv2d_fwd_fast"):
            getattr(L, name).argtypes = conv_args
            getattr(L, name).restype = ctypes.c_int
        L.oracle_conv2d_fwd_naive_f32.argtypes = [vp, vp, vp] + [ctypes.c_int] * 16
        L.oracle_conv2d_fwd_naive_f32.restype = ctypes.c_int
        L.oracle_conv2d_fwd_naive_bf16.argtypes = conv_args
        L.oracle_conv2d_fwd_naive_bf16.restype = ctypes.c_int
        L.oracle_conv2d_fwd_naive_i8.argtypes = conv_args
        L.oracle_conv2d_fwd_naive_i8.restype = ctypes.c_int
        L.oracle_conv3d_fwd_naive.argtypes = ([ctypes.c_int, ctypes.c_int, fp] + [ctypes.c_void_p] * 5 +
                                              [ctypes.c_int] * 22)
        L.oracle_conv3d_fwd_naive.restype = ctypes.c_int
        L.oracle_conv_out_len.argtypes = [ctypes.c_int] * 6
        L.oracle_conv_out_len.restype = ctypes.c_int
        L.oracle_epilogue_f16.argtypes = [ctypes.c_int, fp, ctypes.c_float, ctypes.c_uint16, ctypes.c_uint16]
        L.oracle_epilogue_f16.restype = ctypes.c_uint16
        L.oracle_epilogue_i8.argtypes = [ctypes.c_int, fp, ctypes.c_int32]
        L.oracle_epilogue_i8.restype = ctypes.c_int8
        L.oracle_check_err_f16.argtypes = [vp, vp, i64, ctypes.c_double, ctypes.c_double,
                                           ctypes.POINTER(ctypes.c_double)]
        L.oracle_check_err_f16.restype = i64
        L.oracle_check_err_i8.argtypes = [vp, vp, i64, i64, ctypes.POINTER(i64)]
        L.oracle_check_err_i8.restype = i64
        L.oracle_hardware_concurrency.restype = ctypes.c_int
        _lib = L
    return _lib


def hardware_concurrency() -> int:
    return max(1, int(lib().oracle_hardware_concurrency()))


def _params(params: Optional[Sequence[float]]):
    arr = (ctypes.c_float * 4)(*([0.0] * 4))
    if params is not None:
        for i, v in enumerate(params):
            arr[i] = float(v)
    return arr


def _strides2(x: Optional[np.ndarray]):
    """Element strides of a 2-D array (0, 0 for None)."""
    if x is None:
        return None, 0, 0
    assert x.ndim == 2
    it = x.itemsize
    return x.ctypes.data, x.strides[0] // it, x.strides[1] // it


def gemm(a: np.ndarray, b: np.ndarray, epilogue: int = EPI_PASSTHROUGH,
         params: Optional[Sequence[float]] = None,
         d0: Optional[np.ndarray] = None, d1: Optional[np.ndarray] = None,
         fast: bool = True, threads: Optional[int] = None) -> np.ndarray:
    """E = epilogue(A @ B, D0, D1) with ReferenceGemm semantics.

    ``a`` is an (M, K) view, ``b`` a (K, N) view (any strides, so a column-major B is just
    ``bt.T``); ``d0`` / ``d1`` are (M, N) views (use ``np.broadcast_to`` for a stride-0 bias).
    float16 inputs give a float16 result, int8 inputs an int8 result, uint16 inputs are bfloat16
    bit patterns (see :func:`to_bf16`) and give bfloat16 bits.
    """
    assert a.ndim == 2 and b.ndim == 2 and a.shape[1] == b.shape[0]
    M, K = a.shape
    N = b.shape[1]
    if a.dtype == np.float16:
        dt = 0
    elif a.dtype == np.int8:
        dt = 1
    elif a.dtype == np.uint16:  # bfloat16 bit patterns (ck::bhalf_t)
        dt = 2
    else:
        raise TypeError(a.dtype)
    assert b.dtype == a.dtype
    e = np.empty((M, N), dtype=a.dtype)
    pa, asm, ask = _strides2(a)
    pb, bsk, bsn = _strides2(b)
    pe, esm, esn = _strides2(e)
    p0, d0m, d0n = _strides2(d0)
    p1, d1m, d1n = _strides2(d1)
    th = threads or hardware_concurrency()
    fn = lib().oracle_gemm_fast if fast else lib().oracle_gemm_naive
    rc = fn(dt, epilogue, _params(params), pa, asm, ask, pb, bsk, bsn, pe, esm, esn,
            p0, d0m, d0n, p1, d1m, d1n, M, N, K, th)
    if rc == 2 and fast:  # int8 range too large for the float-accumulating blocked form
        rc = lib().oracle_gemm_naive(dt, epilogue, _params(params), pa, asm, ask, pb, bsk, bsn,
                                     pe, esm, esn, p0, d0m, d0n, p1, d1m, d1n, M, N, K, th)
    if rc != 0:
        raise RuntimeError(f"oracle gemm failed rc={rc}")
    return e


def to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16), round to nearest even as ck::type_convert<bhalf_t>
    (include/ck/utility/data_type.hpp:953-990) does for finite values."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16(b: np.ndarray) -> np.ndarray:
    """bfloat16 bit patterns -> float32 (data_type.hpp:940-950)."""
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def conv_out_len(in_len, filter_len, stride, dilation, lpad, rpad) -> int:
    return int(lib().oracle_conv_out_len(in_len, filter_len, stride, dilation, lpad, rpad))


def conv2d_fwd(inp: np.ndarray, wei: np.ndarray, stride=(1, 1), dilation=(1, 1), pad=(0, 0),
               pad_right=None, epilogue: int = EPI_PASSTHROUGH,
               params: Optional[Sequence[float]] = None,
               bias: Optional[np.ndarray] = None, resi: Optional[np.ndarray] = None,
               fast: bool = True, threads: Optional[int] = None) -> np.ndarray:
    """NHWC float16 input (N,Hi,Wi,C), KYXC weights (K,Y,X,C) -> NHWK output (N,Ho,Wo,K).
    uint16 arrays are bfloat16 bit patterns, int8 arrays the int8 convolution (naive loops only for both)."""
    is_bf16 = inp.dtype == np.uint16
    assert inp.dtype in (np.float16, np.uint16, np.int8) and wei.dtype == inp.dtype
    dt = inp.dtype
    inp = np.ascontiguousarray(inp)
    wei = np.ascontiguousarray(wei)
    N, Hi, Wi, C = inp.shape
    K, Y, X, C2 = wei.shape
    assert C == C2
    pad_right = pad if pad_right is None else pad_right
    Ho = conv_out_len(Hi, Y, stride[0], dilation[0], pad[0], pad_right[0])
    Wo = conv_out_len(Wi, X, stride[1], dilation[1], pad[1], pad_right[1])
    out = np.empty((N, Ho, Wo, K), dtype=dt)
    pb = None
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=dt)
        assert bias.shape == (K,)
        pb = bias.ctypes.data
    pr = None
    if resi is not None:
        resi = np.ascontiguousarray(resi, dtype=dt)
        assert resi.shape == out.shape
        pr = resi.ctypes.data
    th = threads or hardware_concurrency()
    fn = lib().oracle_conv2d_fwd_fast if fast else lib().oracle_conv2d_fwd_naive
    if is_bf16:
        fn = lib().oracle_conv2d_fwd_naive_bf16
    if inp.dtype == np.int8:
        fn = lib().oracle_conv2d_fwd_naive_i8
    rc = fn(epilogue, _params(params), inp.ctypes.data, wei.ctypes.data, out.ctypes.data, pb, pr,
            N, K, C, Hi, Wi, Y, X, Ho, Wo, stride[0], stride[1], dilation[0], dilation[1],
            pad[0], pad[1], th)
    if rc != 0:
        raise RuntimeError(f"oracle conv failed rc={rc}")
    return out


def conv3d_fwd(inp: np.ndarray, wei: np.ndarray, stride=(1, 1, 1), dilation=(1, 1, 1), pad=(0, 0, 0),
               pad_right=None, epilogue: int = EPI_PASSTHROUGH, params: Optional[Sequence[float]] = None,
               bias: Optional[np.ndarray] = None, resi: Optional[np.ndarray] = None,
               threads: Optional[int] = None) -> np.ndarray:
    """NDHWC input (N,Di,Hi,Wi,C), KZYXC weights (K,Z,Y,X,C) -> NDHWK output (N,Do,Ho,Wo,K); naive loops.
    float16, int8, uint16 (bfloat16 bit patterns) or float32 (PassThrough only) arrays."""
    code = {np.dtype(np.float16): 0, np.dtype(np.int8): 1, np.dtype(np.uint16): 2, np.dtype(np.float32): 3}[inp.dtype]
    assert wei.dtype == inp.dtype
    inp, wei = np.ascontiguousarray(inp), np.ascontiguousarray(wei)
    N, Di, Hi, Wi, C = inp.shape
    K, Z, Y, X, C2 = wei.shape
    assert C == C2
    pad_right = pad if pad_right is None else pad_right
    Do, Ho, Wo = (conv_out_len(i, f, s, d, pl, pr) for i, f, s, d, pl, pr in
                  zip((Di, Hi, Wi), (Z, Y, X), stride, dilation, pad, pad_right))
    out = np.empty((N, Do, Ho, Wo, K), dtype=inp.dtype)
    pb = pr = None
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=inp.dtype)
        pb = bias.ctypes.data
    if resi is not None:
        resi = np.ascontiguousarray(resi, dtype=inp.dtype)
        assert resi.shape == out.shape
        pr = resi.ctypes.data
    rc = lib().oracle_conv3d_fwd_naive(code, epilogue, _params(params), inp.ctypes.data, wei.ctypes.data,
                                       out.ctypes.data, pb, pr, N, K, C, Di, Hi, Wi, Z, Y, X, Do, Ho, Wo, *stride,
                                       *dilation, *pad, threads or hardware_concurrency())
    if rc != 0:
        raise RuntimeError(f"oracle conv3d failed rc={rc}")
    return out


def conv1d_fwd(inp: np.ndarray, wei: np.ndarray, stride=1, dilation=1, pad=0, pad_right=None, **kw) -> np.ndarray:
    """NWC input (N,Wi,C), KXC weights (K,X,C) -> NWK output (N,Wo,K): the 3-D convolution with depth = height = 1."""
    pr = pad if pad_right is None else pad_right
    out = conv3d_fwd(inp[:, None, None], wei[:, None, None], (1, 1, stride), (1, 1, dilation), (0, 0, pad),
                     (0, 0, pr), **kw)
    return out[:, 0, 0]


def conv2d_fwd_f32(inp: np.ndarray, wei: np.ndarray, stride=(1, 1), dilation=(1, 1), pad=(0, 0),
                   pad_right=None, threads: Optional[int] = None) -> np.ndarray:
    """float32 PassThrough form of :func:`conv2d_fwd` (naive loops only)."""
    assert inp.dtype == np.float32 and wei.dtype == np.float32
    inp = np.ascontiguousarray(inp)
    wei = np.ascontiguousarray(wei)
    N, Hi, Wi, C = inp.shape
    K, Y, X, _ = wei.shape
    pad_right = pad if pad_right is None else pad_right
    Ho = conv_out_len(Hi, Y, stride[0], dilation[0], pad[0], pad_right[0])
    Wo = conv_out_len(Wi, X, stride[1], dilation[1], pad[1], pad_right[1])
    out = np.empty((N, Ho, Wo, K), dtype=np.float32)
    rc = lib().oracle_conv2d_fwd_naive_f32(inp.ctypes.data, wei.ctypes.data, out.ctypes.data,
                                           N, K, C, Hi, Wi, Y, X, Ho, Wo, stride[0], stride[1],
                                           dilation[0], dilation[1], pad[0], pad[1],
                                           threads or hardware_concurrency())
    if rc != 0:
        raise RuntimeError(f"oracle conv failed rc={rc}")
    return out


def epilogue_f16(epi: int, params, c: float, d0: float = 0.0, d1: float = 0.0) -> np.float16:
    bits = lib().oracle_epilogue_f16(epi, _params(params), float(c),
                                     int(np.float16(d0).view(np.uint16)),
                                     int(np.float16(d1).view(np.uint16)))
    return np.uint16(bits).view(np.float16)


def epilogue_i8(epi: int, params, acc: int) -> int:
    return int(lib().oracle_epilogue_i8(epi, _params(params), int(acc)))


def check_err(out: np.ndarray, ref: np.ndarray, rtol: float = 1e-3, atol: float = 1e-3):
    """ck::utils::check_err (check_err.hpp:107-193): returns (n_bad, max_err)."""
    out = np.ascontiguousarray(out)
    ref = np.ascontiguousarray(ref)
    assert out.shape == ref.shape and out.dtype == ref.dtype
    if out.dtype == np.float16:
        m = ctypes.c_double(0)
        bad = lib().oracle_check_err_f16(out.ctypes.data, ref.ctypes.data, out.size, rtol, atol,
                                         ctypes.byref(m))
        return int(bad), float(m.value)
    if out.dtype == np.int8:
        m = ctypes.c_int64(0)
        bad = lib().oracle_check_err_i8(out.ctypes.data, ref.ctypes.data, out.size, 0, ctypes.byref(m))
        return int(bad), int(m.value)
    raise TypeError(out.dtype)
