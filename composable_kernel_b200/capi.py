"""ctypes binding of the C ABI declared in include/ckb200.h.

The shared library holds sm_100a kernels only.  Loading fails loudly when it is missing; there
is no CPU substitute behind any of these calls.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t,
                    c_uint32, c_uint64, c_void_p)

HERE = os.path.dirname(os.path.abspath(__file__))
# CKB200_LIB selects another build of the library (e.g. one compiled with different tuning macros).
LIB_PATH = os.environ.get("CKB200_LIB") or os.path.join(HERE, "lib", "libckb200.so")

# ---- enums (include/ckb200.h) -------------------------------------------------------------------
CKB_OK, CKB_ERR_UNSUPPORTED, CKB_ERR_INVALID, CKB_ERR_CUDA, CKB_ERR_DEVICE, CKB_ERR_WORKSPACE, \
    CKB_ERR_LIMIT = range(7)
CKB_F16, CKB_I8, CKB_BF16 = 0, 1, 2
CKB_ROW_MAJOR, CKB_COL_MAJOR = 0, 1
(CKB_EPI_PASSTHROUGH, CKB_EPI_SCALE, CKB_EPI_RELU, CKB_EPI_FASTGELU, CKB_EPI_ADD,
 CKB_EPI_ADD_RELU_F16, CKB_EPI_BILINEAR, CKB_EPI_ADD_ADD_FASTGELU, CKB_EPI_ADD_RELU_ADD,
 CKB_EPI_REQUANT_RELU_REQUANT, CKB_EPI_REQUANT_RELU_REQUANT_RNE, CKB_EPI_ADD_RELU,
 CKB_EPI_ADD_HARDSWISH) = range(13)
CKB_MAX_DS = 2
CKB_NOALLOC_MAX_GROUPS = 256
CKB_ABI_VERSION = 2


def tile_config(bn: int = 0, cg: int = 0, no_ksplit: int = 0, kbatch: int = 0, balanced: int = 0) -> int:
    """CKB_TILE_CONFIG(bn, cg, no_ksplit) / CKB_TILE_CONFIG_KBATCH(bn, cg, kbatch) / CKB_TILE_CONFIG_BALANCED(bn, cg)
    of include/ckb200.h; 0 = the library's own choice."""
    return bn | (cg << 12) | (no_ksplit << 16) | (balanced << 17) | (kbatch << 20)

EPI_NUM_D = {CKB_EPI_ADD: 1, CKB_EPI_ADD_RELU_F16: 1, CKB_EPI_BILINEAR: 1, CKB_EPI_ADD_RELU: 1,
             CKB_EPI_ADD_HARDSWISH: 1, CKB_EPI_ADD_ADD_FASTGELU: 2, CKB_EPI_ADD_RELU_ADD: 2}


class GemmDesc(Structure):
    """struct ckb_gemm_desc"""
    _fields_ = [
        ("ab_dtype", c_int32), ("e_dtype", c_int32),
        ("a_layout", c_int32), ("b_layout", c_int32), ("e_layout", c_int32),
        ("epilogue", c_int32), ("n_ds", c_int32), ("tile_config", c_int32),
        ("M", c_int64), ("N", c_int64), ("K", c_int64),
        ("lda", c_int64), ("ldb", c_int64), ("lde", c_int64),
        ("ldd", c_int64 * CKB_MAX_DS),
        ("p_a", c_void_p), ("p_b", c_void_p),
        ("p_ds", c_void_p * CKB_MAX_DS),
        ("p_e", c_void_p),
        ("epi_params", c_float * 4),
    ]


class BatchedGemmDesc(Structure):
    """struct ckb_batched_gemm_desc"""
    _fields_ = [("gemm", GemmDesc), ("batch", c_int64), ("batch_stride_a", c_int64), ("batch_stride_b", c_int64),
                ("batch_stride_e", c_int64), ("batch_stride_d", c_int64 * CKB_MAX_DS)]


class GroupedGemmDesc(Structure):
    """struct ckb_grouped_gemm_desc"""
    _fields_ = [("group_count", c_int32), ("tile_config", c_int32), ("groups", POINTER(GemmDesc))]


class Conv2dFwdDesc(Structure):
    """struct ckb_conv2d_fwd_desc"""
    _fields_ = [
        ("dtype", c_int32), ("epilogue", c_int32),
        ("N", c_int32), ("K", c_int32), ("C", c_int32),
        ("Hi", c_int32), ("Wi", c_int32), ("Y", c_int32), ("X", c_int32),
        ("Ho", c_int32), ("Wo", c_int32),
        ("stride_h", c_int32), ("stride_w", c_int32),
        ("dilation_h", c_int32), ("dilation_w", c_int32),
        ("pad_h", c_int32), ("pad_w", c_int32),
        ("pad_h_right", c_int32), ("pad_w_right", c_int32),
        ("tile_config", c_int32),
        ("p_in", c_void_p), ("p_wei", c_void_p), ("p_out", c_void_p),
        ("p_bias", c_void_p), ("p_resi", c_void_p),
        ("epi_params", c_float * 4),
    ]


class Conv3dFwdDesc(Structure):
    """struct ckb_conv3d_fwd_desc"""
    _fields_ = [
        ("dtype", c_int32), ("epilogue", c_int32),
        ("N", c_int32), ("K", c_int32), ("C", c_int32),
        ("Di", c_int32), ("Hi", c_int32), ("Wi", c_int32),
        ("Z", c_int32), ("Y", c_int32), ("X", c_int32),
        ("Do", c_int32), ("Ho", c_int32), ("Wo", c_int32),
        ("stride_d", c_int32), ("stride_h", c_int32), ("stride_w", c_int32),
        ("dilation_d", c_int32), ("dilation_h", c_int32), ("dilation_w", c_int32),
        ("pad_d", c_int32), ("pad_h", c_int32), ("pad_w", c_int32),
        ("pad_d_right", c_int32), ("pad_h_right", c_int32), ("pad_w_right", c_int32),
        ("tile_config", c_int32),
        ("p_in", c_void_p), ("p_wei", c_void_p), ("p_out", c_void_p),
        ("p_bias", c_void_p), ("p_resi", c_void_p),
        ("epi_params", c_float * 4),
    ]


# name -> (restype, argtypes); every symbol include/ckb200.h declares.
SYMBOLS = {
    "ckb_abi_version": (c_int, []),
    "ckb_last_error": (c_char_p, []),
    "ckb_last_plan": (c_char_p, []),
    "ckb_launch_count": (c_uint64, []),
    "ckb_device_info": (c_int, [c_char_p, c_size_t, POINTER(c_int), POINTER(c_int), POINTER(c_int)]),
    "ckb_device_status": (c_int, [POINTER(c_uint32)]),
    "ckb_malloc": (c_int, [POINTER(c_void_p), c_size_t]),
    "ckb_free": (c_int, [c_void_p]),
    "ckb_memcpy_h2d": (c_int, [c_void_p, c_void_p, c_size_t]),
    "ckb_memcpy_d2h": (c_int, [c_void_p, c_void_p, c_size_t]),
    "ckb_memset": (c_int, [c_void_p, c_int, c_size_t]),
    "ckb_device_synchronize": (c_int, []),
    "ckb_release_scratch": (c_int, [c_void_p, c_int]),
    "ckb_gemm_supported": (c_int, [POINTER(GemmDesc)]),
    "ckb_gemm_run": (c_int, [POINTER(GemmDesc), c_void_p, c_int, POINTER(c_float)]),
    "ckb_batched_gemm_supported": (c_int, [POINTER(BatchedGemmDesc)]),
    "ckb_batched_gemm_run": (c_int, [POINTER(BatchedGemmDesc), c_void_p, c_int, POINTER(c_float)]),
    "ckb_grouped_gemm_supported": (c_int, [POINTER(GroupedGemmDesc)]),
    "ckb_grouped_gemm_workspace_size": (c_int, [POINTER(GroupedGemmDesc), POINTER(c_size_t)]),
    "ckb_grouped_gemm_run": (c_int, [POINTER(GroupedGemmDesc), c_void_p, c_size_t, c_void_p, c_int,
                                     POINTER(c_float)]),
    "ckb_grouped_gemm_run_noalloc": (c_int, [POINTER(GroupedGemmDesc), c_void_p]),
    "ckb_conv2d_fwd_supported": (c_int, [POINTER(Conv2dFwdDesc)]),
    "ckb_conv2d_fwd_run": (c_int, [POINTER(Conv2dFwdDesc), c_void_p, c_int, POINTER(c_float)]),
    "ckb_conv3d_fwd_supported": (c_int, [POINTER(Conv3dFwdDesc)]),
    "ckb_conv3d_fwd_run": (c_int, [POINTER(Conv3dFwdDesc), c_void_p, c_int, POINTER(c_float)]),
}

_lib = None


class CkbError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"ckb error {code}: {message}")
        self.code = code


def lib() -> ctypes.CDLL:
    """Loads libckb200.so (built by composable_kernel_b200.build).  Raises if it is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m composable_kernel_b200.build`. "
                "This package has no CPU fallback.")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error() -> str:
    return (lib().ckb_last_error() or b"").decode()


def last_plan() -> str:
    """Plan of the calling thread's last launch, e.g. 'gemm tile=128x256 cg=1 grid=144 ... cluster_k=8 ...'."""
    return (lib().ckb_last_plan() or b"").decode()


def check(rc: int) -> None:
    if rc != CKB_OK:
        raise CkbError(rc, last_error())
