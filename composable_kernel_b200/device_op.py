"""Python mirror of Composable Kernel's device-operation interface for the dense contraction path.

Same call sequence and names as the reference (include/ck/tensor_operation/gpu/device/
device_base.hpp:14-57): construct the op, ``MakeArgument``/``MakeArgumentPointer`` ->
``IsSupportedArgument`` -> ``MakeInvoker``/``MakeInvokerPointer`` -> ``Run(arg, StreamConfig)``,
which returns the average milliseconds when ``time_kernel`` is set and 0 otherwise
(device_utility/kernel_launch.hpp:61,67).  Pointers are raw device addresses (ints); the
library never owns tensor memory.  Every ``Run`` goes through the C ABI in include/ckb200.h.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

from . import capi
from .capi import (CKB_COL_MAJOR, CKB_F16, CKB_I8, CKB_ROW_MAJOR, Conv2dFwdDesc, GemmDesc,
                   GroupedGemmDesc)


# ---- element-wise operators (tensor_operation/gpu/element/*.hpp) ---------------------------------
@dataclass(frozen=True)
class ElementOp:
    kind: int
    params: tuple = (0.0, 0.0, 0.0, 0.0)


class PassThrough(ElementOp):
    """unary_element_wise_operation.hpp:13-25"""
    def __init__(self):
        super().__init__(capi.CKB_EPI_PASSTHROUGH)


class Scale(ElementOp):
    """unary_element_wise_operation.hpp:27-41"""
    def __init__(self, scale: float):
        super().__init__(capi.CKB_EPI_SCALE, (float(scale), 0.0, 0.0, 0.0))


class Relu(ElementOp):
    """unary_element_wise_operation.hpp:98-119"""
    def __init__(self):
        super().__init__(capi.CKB_EPI_RELU)


class FastGelu(ElementOp):
    """unary_element_wise_operation.hpp:121-135"""
    def __init__(self):
        super().__init__(capi.CKB_EPI_FASTGELU)


class Add(ElementOp):
    """binary_element_wise_operation.hpp:31-36 (half = half(c) + d0)"""
    def __init__(self):
        super().__init__(capi.CKB_EPI_ADD)


class AddReluF16(ElementOp):
    """example/03_gemm_bias_relu/gemm_bias_relu_xdl_fp16.cpp:34-43"""
    def __init__(self):
        super().__init__(capi.CKB_EPI_ADD_RELU_F16)


class AddRelu(ElementOp):
    """binary_element_wise_operation.hpp:123-129 (fp32, one rounding)"""
    def __init__(self):
        super().__init__(capi.CKB_EPI_ADD_RELU)


class AddHardswish(ElementOp):
    """binary_element_wise_operation.hpp:153-161"""
    def __init__(self):
        super().__init__(capi.CKB_EPI_ADD_HARDSWISH)


class Bilinear(ElementOp):
    """binary_element_wise_operation.hpp:93-116"""
    def __init__(self, alpha: float, beta: float):
        super().__init__(capi.CKB_EPI_BILINEAR, (float(alpha), float(beta), 0.0, 0.0))


class AddAddFastGelu(ElementOp):
    """element_wise_operation.hpp:115-140"""
    def __init__(self):
        super().__init__(capi.CKB_EPI_ADD_ADD_FASTGELU)


class AddReluAdd(ElementOp):
    """element_wise_operation.hpp:46-80"""
    def __init__(self):
        super().__init__(capi.CKB_EPI_ADD_RELU_ADD)


class RequantReluRequant(ElementOp):
    """example/14_gemm_xdl_requant_relu_requant/gemm_xdl_requant_relu_requant_int8.cpp:21-39
    (no rounding inside; the int8 store truncates toward zero)."""
    def __init__(self, scale_gemm: float, scale_relu: float):
        super().__init__(capi.CKB_EPI_REQUANT_RELU_REQUANT, (float(scale_gemm), float(scale_relu), 0.0, 0.0))


class RequantReluRequantRne(ElementOp):
    """sat_int8(rne(s1 * relu(rne(s0 * acc))))"""
    def __init__(self, scale_gemm: float, scale_relu: float):
        super().__init__(capi.CKB_EPI_REQUANT_RELU_REQUANT_RNE,
                         (float(scale_gemm), float(scale_relu), 0.0, 0.0))


@dataclass
class StreamConfig:
    """include/ck/stream_config.hpp:9-13"""
    stream_id: Optional[int] = None
    time_kernel: bool = False
    nrepeat: int = 10  # kernel_launch.hpp:32


class BaseArgument:
    """device_base.hpp:14-24"""
    def __init__(self):
        self.p_workspace_ = None
        self.workspace_bytes_ = 0


def _is_passthrough(op) -> bool:
    return op is None or (isinstance(op, ElementOp) and op.kind == capi.CKB_EPI_PASSTHROUGH)


def _fill_gemm_desc(d: GemmDesc, dtype, a_layout, b_layout, p_a, p_b, p_ds, p_e, M, N, K, sa, sb, sds,
                    se, cde_op: ElementOp):
    d.ab_dtype = dtype
    d.e_dtype = dtype
    d.a_layout = a_layout
    d.b_layout = b_layout
    d.e_layout = CKB_ROW_MAJOR
    d.epilogue = cde_op.kind
    d.n_ds = len(p_ds)
    d.M, d.N, d.K = int(M), int(N), int(K)
    d.lda, d.ldb, d.lde = int(sa), int(sb), int(se)
    for i in range(capi.CKB_MAX_DS):
        d.ldd[i] = int(sds[i]) if i < len(sds) else 0
        d.p_ds[i] = int(p_ds[i]) if i < len(p_ds) and p_ds[i] else None
    d.p_a = int(p_a) if p_a else None
    d.p_b = int(p_b) if p_b else None
    d.p_e = int(p_e) if p_e else None
    for i in range(4):
        d.epi_params[i] = float(cde_op.params[i])


class GemmArgument(BaseArgument):
    def __init__(self):
        super().__init__()
        self.desc = GemmDesc()
        self.ab_ops_passthrough = True


class _Invoker:
    def __init__(self, op):
        self._op = op

    def Run(self, arg, stream_config: StreamConfig = StreamConfig()) -> float:
        return self._op._run(arg, stream_config)


class BaseOperator:
    """device_base.hpp:37-57"""
    def IsSupportedArgument(self, arg) -> bool:
        raise NotImplementedError

    def GetTypeString(self) -> str:
        return type(self).__name__

    def GetWorkSpaceSize(self, arg) -> int:
        return 0

    def SetWorkSpacePointer(self, arg, p_workspace, workspace_bytes: Optional[int] = None) -> None:
        arg.p_workspace_ = p_workspace
        arg.workspace_bytes_ = workspace_bytes if workspace_bytes is not None else self.GetWorkSpaceSize(arg)

    def MakeInvoker(self):
        return _Invoker(self)

    MakeInvokerPointer = MakeInvoker


class DeviceGemmMultipleD(BaseOperator):
    """DeviceGemmMultipleD (device_gemm_multiple_d.hpp:32-53), realised by one sm_100a kernel.

    ``dtype`` is CKB_F16, CKB_BF16 or CKB_I8; layouts are the gemm layout tags of
    device/tensor_layout.hpp:13-25 (A and B in either order, E row-major).  ``tile_config`` is 0 (the library
    chooses tile shape and tail plan) or ``capi.tile_config(bn, cg, no_ksplit)``: one instance of an instance
    factory per value.
    """

    def __init__(self, dtype=CKB_F16, a_layout=CKB_ROW_MAJOR, b_layout=CKB_COL_MAJOR, tile_config=0):
        self.dtype, self.a_layout, self.b_layout, self.tile_config = dtype, a_layout, b_layout, tile_config

    def MakeArgument(self, p_a, p_b, p_ds: Sequence[int], p_e, M, N, K, StrideA, StrideB,
                     StrideDs: Sequence[int], StrideE, a_element_op=None, b_element_op=None,
                     cde_element_op: ElementOp = PassThrough()) -> GemmArgument:
        arg = GemmArgument()
        _fill_gemm_desc(arg.desc, self.dtype, self.a_layout, self.b_layout, p_a, p_b, list(p_ds), p_e,
                        M, N, K, StrideA, StrideB, list(StrideDs), StrideE, cde_element_op)
        arg.desc.tile_config = self.tile_config
        arg.ab_ops_passthrough = _is_passthrough(a_element_op) and _is_passthrough(b_element_op)
        return arg

    MakeArgumentPointer = MakeArgument

    def IsSupportedArgument(self, arg: GemmArgument) -> bool:
        # A/B element-ops are applied by the reference while copying global->LDS
        # (gridwise_gemm_xdl_cshuffle_v1.hpp:335-394); TMA cannot transform in flight.
        if not arg.ab_ops_passthrough:
            return False
        return capi.lib().ckb_gemm_supported(ctypes.byref(arg.desc)) == capi.CKB_OK

    def _run(self, arg: GemmArgument, sc: StreamConfig) -> float:
        if not self.IsSupportedArgument(arg):
            # device_gemm_xdl_cshuffle.hpp:475-481
            raise RuntimeError("wrong! GridwiseGemm has invalid setting: " + capi.last_error())
        ms = ctypes.c_float(0.0)
        rc = capi.lib().ckb_gemm_run(ctypes.byref(arg.desc), sc.stream_id,
                                     sc.nrepeat if sc.time_kernel else 0, ctypes.byref(ms))
        capi.check(rc)
        return float(ms.value)

    def GetTypeString(self) -> str:
        return "DeviceGemmMultipleD_B200_Tcgen05<128, 256|128|64, 128B>"


class DeviceGemm(DeviceGemmMultipleD):
    """DeviceGemm (device_gemm.hpp:24-40): no D tensors, one C element-op."""

    def MakeArgument(self, p_a, p_b, p_c, M, N, K, StrideA, StrideB, StrideC, a_element_op=None,
                     b_element_op=None, c_element_op: ElementOp = PassThrough()) -> GemmArgument:
        return super().MakeArgument(p_a, p_b, [], p_c, M, N, K, StrideA, StrideB, [], StrideC,
                                    a_element_op, b_element_op, c_element_op)

    MakeArgumentPointer = MakeArgument

    def GetTypeString(self) -> str:
        return "DeviceGemm_B200_Tcgen05<128, 256|128|64, 128B>"


class BatchedGemmArgument(BaseArgument):
    def __init__(self):
        super().__init__()
        self.desc = capi.BatchedGemmDesc()
        self.ab_ops_passthrough = True


class DeviceBatchedGemm(BaseOperator):
    """DeviceBatchedGemm (device_batched_gemm.hpp:15-44): `Batch` problems of one shape whose matrices lie
    BatchStrideA / BatchStrideB / BatchStrideC elements apart; all batches run in one launch."""

    def __init__(self, dtype=CKB_F16, a_layout=CKB_ROW_MAJOR, b_layout=CKB_COL_MAJOR):
        self.dtype, self.a_layout, self.b_layout = dtype, a_layout, b_layout

    def MakeArgument(self, p_a, p_b, p_c, M, N, K, StrideA, StrideB, StrideC, BatchStrideA, BatchStrideB,
                     BatchStrideC, Batch, a_element_op=None, b_element_op=None,
                     c_element_op: ElementOp = PassThrough()) -> BatchedGemmArgument:
        arg = BatchedGemmArgument()
        _fill_gemm_desc(arg.desc.gemm, self.dtype, self.a_layout, self.b_layout, p_a, p_b, [], p_c, M, N, K,
                        StrideA, StrideB, [], StrideC, c_element_op)
        arg.desc.batch = int(Batch)
        arg.desc.batch_stride_a, arg.desc.batch_stride_b = int(BatchStrideA), int(BatchStrideB)
        arg.desc.batch_stride_e = int(BatchStrideC)
        arg.ab_ops_passthrough = _is_passthrough(a_element_op) and _is_passthrough(b_element_op)
        return arg

    MakeArgumentPointer = MakeArgument

    def IsSupportedArgument(self, arg: BatchedGemmArgument) -> bool:
        if not arg.ab_ops_passthrough:
            return False
        return capi.lib().ckb_batched_gemm_supported(ctypes.byref(arg.desc)) == capi.CKB_OK

    def _run(self, arg: BatchedGemmArgument, sc: StreamConfig) -> float:
        if not self.IsSupportedArgument(arg):
            raise RuntimeError("wrong! GridwiseGemm has invalid setting: " + capi.last_error())
        ms = ctypes.c_float(0.0)
        capi.check(capi.lib().ckb_batched_gemm_run(ctypes.byref(arg.desc), sc.stream_id,
                                                   sc.nrepeat if sc.time_kernel else 0, ctypes.byref(ms)))
        return float(ms.value)

    def GetTypeString(self) -> str:
        return "DeviceBatchedGemm_B200_Tcgen05<128, 256|128|64, 128B>"


@dataclass
class GemmDescHost:
    """GemmDesc (device_grouped_gemm.hpp:11-17)"""
    M_: int
    N_: int
    K_: int
    stride_A_: int
    stride_B_: int
    stride_C_: int
    stride_Ds_: List[int] = field(default_factory=list)


class GroupedGemmArgument(BaseArgument):
    def __init__(self, n):
        super().__init__()
        self.group_descs = (GemmDesc * n)()
        self.desc = GroupedGemmDesc()
        self.desc.group_count = n
        self.desc.groups = ctypes.cast(self.group_descs, ctypes.POINTER(GemmDesc))
        self.ab_ops_passthrough = True


class DeviceGroupedGemm(BaseOperator):
    """DeviceGroupedGemm (device_grouped_gemm.hpp:19-44); workspace contract of
    device_grouped_gemm_xdl.hpp:816-819 (caller-allocated device memory)."""

    def __init__(self, dtype=CKB_F16, a_layout=CKB_ROW_MAJOR, b_layout=CKB_COL_MAJOR, tile_config=0):
        self.dtype, self.a_layout, self.b_layout, self.tile_config = dtype, a_layout, b_layout, tile_config

    def MakeArgument(self, p_a: Sequence[int], p_b: Sequence[int], p_ds: Sequence[Sequence[int]],
                     p_e: Sequence[int], gemm_descs: Sequence[GemmDescHost], a_element_op=None,
                     b_element_op=None, c_element_op: ElementOp = PassThrough()) -> GroupedGemmArgument:
        n = len(gemm_descs)
        # device_grouped_gemm_xdl.hpp:547-552
        if not (len(p_a) == n and len(p_b) == n and len(p_e) == n):
            raise RuntimeError("wrong! group_count_ != P_a/b/c.size")
        arg = GroupedGemmArgument(n)
        arg.desc.tile_config = self.tile_config
        for i, gd in enumerate(gemm_descs):
            ds = list(p_ds[i]) if p_ds else []
            _fill_gemm_desc(arg.group_descs[i], self.dtype, self.a_layout, self.b_layout, p_a[i],
                            p_b[i], ds, p_e[i], gd.M_, gd.N_, gd.K_, gd.stride_A_, gd.stride_B_,
                            list(gd.stride_Ds_), gd.stride_C_, c_element_op)
        arg.ab_ops_passthrough = _is_passthrough(a_element_op) and _is_passthrough(b_element_op)
        return arg

    MakeArgumentPointer = MakeArgument

    def IsSupportedArgument(self, arg: GroupedGemmArgument) -> bool:
        if not arg.ab_ops_passthrough:
            return False
        return capi.lib().ckb_grouped_gemm_supported(ctypes.byref(arg.desc)) == capi.CKB_OK

    def GetWorkSpaceSize(self, arg: GroupedGemmArgument) -> int:
        n = ctypes.c_size_t(0)
        capi.check(capi.lib().ckb_grouped_gemm_workspace_size(ctypes.byref(arg.desc), ctypes.byref(n)))
        return int(n.value)

    def _run(self, arg: GroupedGemmArgument, sc: StreamConfig) -> float:
        if not self.IsSupportedArgument(arg):
            raise RuntimeError("wrong! GridwiseGemm has invalid setting: " + capi.last_error())
        ms = ctypes.c_float(0.0)
        rc = capi.lib().ckb_grouped_gemm_run(ctypes.byref(arg.desc), arg.p_workspace_,
                                             arg.workspace_bytes_ or 0, sc.stream_id,
                                             sc.nrepeat if sc.time_kernel else 0, ctypes.byref(ms))
        capi.check(rc)
        return float(ms.value)

    def GetTypeString(self) -> str:
        return "DeviceGroupedGemm_B200_Tcgen05<128, 256|128|64, 128B>"


class ConvArgument(BaseArgument):
    def __init__(self):
        super().__init__()
        self.desc = Conv2dFwdDesc()
        self.in_wei_ops_passthrough = True


class DeviceConvFwd(BaseOperator):
    """DeviceConvFwd (device_conv_fwd.hpp:18-39) / DeviceConvFwdBiasActivation
    (device_conv_fwd_bias_activation.hpp:19-41) for channels-last tensors: 1-D NWC/KXC/NWK, 2-D NHWC/KYXC/NHWK or
    3-D NDHWC/KZYXC/NDHWK, chosen by the length of the spatial vectors (the NumDimSpatial of
    DeviceConvNDFwdXdl..., device_convnd_fwd_xdl_nhwc_kyxc_nhwk.hpp:76).  ``dtype`` is CKB_F16, CKB_BF16 or CKB_I8."""

    def __init__(self, dtype=CKB_F16, tile_config=0):
        self.dtype, self.tile_config = dtype, tile_config

    def MakeArgument(self, p_in, p_wei, p_out, N, K, C, input_spatial_lengths, filter_spatial_lengths,
                     output_spatial_lengths, conv_filter_strides, conv_filter_dilations,
                     input_left_pads, input_right_pads, in_element_op=None, wei_element_op=None,
                     out_element_op: ElementOp = PassThrough(), p_bias=None, p_resi=None) -> ConvArgument:
        vecs = [list(map(int, v)) for v in (input_spatial_lengths, filter_spatial_lengths, output_spatial_lengths,
                                            conv_filter_strides, conv_filter_dilations, input_left_pads,
                                            input_right_pads)]
        nd = len(vecs[0])
        arg = ConvArgument()
        arg.consistent = nd in (1, 2, 3) and all(len(v) == nd for v in vecs)
        if not arg.consistent:
            return arg
        if nd == 1:  # a 1-D problem is a 2-D one of height 1 (identity values for the missing dimension)
            ident = [1, 1, 1, 1, 1, 0, 0]
            vecs = [[i] + v for i, v in zip(ident, vecs)]
        in_sp, filt, out_sp, strides, dils, lpads, rpads = vecs
        if nd == 3:
            arg.desc = d = capi.Conv3dFwdDesc()
            d.Di, d.Hi, d.Wi = in_sp
            d.Z, d.Y, d.X = filt
            d.Do, d.Ho, d.Wo = out_sp
            d.stride_d, d.stride_h, d.stride_w = strides
            d.dilation_d, d.dilation_h, d.dilation_w = dils
            d.pad_d, d.pad_h, d.pad_w = lpads
            d.pad_d_right, d.pad_h_right, d.pad_w_right = rpads
        else:
            d = arg.desc
            d.Hi, d.Wi = in_sp
            d.Y, d.X = filt
            d.Ho, d.Wo = out_sp
            d.stride_h, d.stride_w = strides
            d.dilation_h, d.dilation_w = dils
            d.pad_h, d.pad_w = lpads
            d.pad_h_right, d.pad_w_right = rpads
        d.dtype = self.dtype
        d.tile_config = self.tile_config
        d.epilogue = out_element_op.kind
        d.N, d.K, d.C = int(N), int(K), int(C)
        d.p_in = int(p_in) if p_in else None
        d.p_wei = int(p_wei) if p_wei else None
        d.p_out = int(p_out) if p_out else None
        d.p_bias = int(p_bias) if p_bias else None
        d.p_resi = int(p_resi) if p_resi else None
        for i in range(4):
            d.epi_params[i] = float(out_element_op.params[i])
        arg.in_wei_ops_passthrough = _is_passthrough(in_element_op) and _is_passthrough(wei_element_op)
        return arg

    MakeArgumentPointer = MakeArgument

    @staticmethod
    def _is_3d(arg) -> bool:
        return isinstance(arg.desc, capi.Conv3dFwdDesc)

    def IsSupportedArgument(self, arg: ConvArgument) -> bool:
        if not getattr(arg, "consistent", True) or not arg.in_wei_ops_passthrough:
            return False
        fn = capi.lib().ckb_conv3d_fwd_supported if self._is_3d(arg) else capi.lib().ckb_conv2d_fwd_supported
        return fn(ctypes.byref(arg.desc)) == capi.CKB_OK

    def _run(self, arg: ConvArgument, sc: StreamConfig) -> float:
        if not self.IsSupportedArgument(arg):
            raise RuntimeError("wrong! GridwiseGemm has invalid setting: " + capi.last_error())
        ms = ctypes.c_float(0.0)
        fn = capi.lib().ckb_conv3d_fwd_run if self._is_3d(arg) else capi.lib().ckb_conv2d_fwd_run
        capi.check(fn(ctypes.byref(arg.desc), sc.stream_id, sc.nrepeat if sc.time_kernel else 0, ctypes.byref(ms)))
        return float(ms.value)

    def GetTypeString(self) -> str:
        return "DeviceConvNdFwd_B200_Tcgen05_Im2colTma<128, 256|128|64, 128B>"


def device_status() -> int:
    """0 when no kernel reported a bounded-wait time-out (synchronises the device)."""
    w = ctypes.c_uint32(0)
    capi.check(capi.lib().ckb_device_status(ctypes.byref(w)))
    return int(w.value)


def launch_count() -> int:
    return int(capi.lib().ckb_launch_count())
