"""CPU tests of the C-ABI boundary: the library loads, exports every symbol the header declares,
its structs have the layout the Python binding assumes, and argument validation (the
IsSupportedArgument side) works without a GPU.  No compute call is made here."""
import ctypes
import os
import re
import subprocess
import tempfile

import pytest

import composable_kernel_b200 as ck
from composable_kernel_b200 import capi
from oracle import ck_oracle as oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ckb200.h")


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ckb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = capi.lib()
    names = _declared_symbols()
    assert len(names) >= 18
    for n in names:
        assert hasattr(L, n), f"{n} declared in ckb200.h but not exported"
        assert n in capi.SYMBOLS, f"{n} has no ctypes prototype"
    assert L.ckb_abi_version() == capi.CKB_ABI_VERSION == 2


def test_struct_layout_matches_header():
    src = r'''
    #include "ckb200.h"
    #include <stdio.h>
    #include <stddef.h>
    int main(){ printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\n", sizeof(ckb_gemm_desc), sizeof(ckb_conv2d_fwd_desc),
      sizeof(ckb_grouped_gemm_desc), offsetof(ckb_gemm_desc, p_e), offsetof(ckb_gemm_desc, epi_params),
      offsetof(ckb_conv2d_fwd_desc, p_in), sizeof(ckb_batched_gemm_desc), offsetof(ckb_batched_gemm_desc, batch),
      offsetof(ckb_batched_gemm_desc, batch_stride_d), sizeof(ckb_conv3d_fwd_desc),
      offsetof(ckb_conv3d_fwd_desc, p_in)); return 0; }'''
    with tempfile.TemporaryDirectory() as td:
        c = os.path.join(td, "t.c")
        open(c, "w").write(src)
        exe = os.path.join(td, "t")
        subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe], check=True)
        out = subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split()
    want = [ctypes.sizeof(capi.GemmDesc), ctypes.sizeof(capi.Conv2dFwdDesc), ctypes.sizeof(capi.GroupedGemmDesc),
            capi.GemmDesc.p_e.offset, capi.GemmDesc.epi_params.offset, capi.Conv2dFwdDesc.p_in.offset,
            ctypes.sizeof(capi.BatchedGemmDesc), capi.BatchedGemmDesc.batch.offset,
            capi.BatchedGemmDesc.batch_stride_d.offset, ctypes.sizeof(capi.Conv3dFwdDesc),
            capi.Conv3dFwdDesc.p_in.offset]
    assert [int(x) for x in out] == want


def test_epilogue_ids_agree_between_header_binding_and_oracle():
    text = open(HEADER).read()
    for name, value in re.findall(r"(CKB_EPI_[A-Z0-9_]+)\s*=\s*(\d+)", text):
        if name.endswith("COUNT_"):
            continue
        assert getattr(capi, name) == int(value)
        assert getattr(oracle, name.replace("CKB_", "")) == int(value)


def test_gemm_supported_rules():
    op = ck.DeviceGemm()
    ok = op.MakeArgument(0x1000, 0x2000, 0x3000, 3840, 4096, 4096, 4096, 4096, 4096)
    assert op.IsSupportedArgument(ok)
    # ragged sizes are fine (TMA zero-fills); a pitch or base that is not a multiple of 16 bytes is served through a
    # padded copy by the plain GEMM and refused by the batched and grouped entry points
    assert op.IsSupportedArgument(op.MakeArgument(0x1000, 0x2000, 0x3000, 100, 37, 72, 72, 72, 37))
    assert op.IsSupportedArgument(op.MakeArgument(0x1000, 0x2000, 0x3000, 100, 37, 70, 70, 70, 37))
    bg = ck.DeviceBatchedGemm()
    assert not bg.IsSupportedArgument(bg.MakeArgument(0x1000, 0x2000, 0x3000, 100, 37, 70, 70, 70, 37, 7000, 2590, 3700, 2))
    assert "16 bytes" in capi.last_error()
    gg = ck.DeviceGroupedGemm()
    assert not gg.IsSupportedArgument(gg.MakeArgument([0x1000], [0x2000], [], [0x3000],
                                                      [ck.GemmDescHost(100, 37, 70, 70, 70, 37)]))
    # tile configurations: a pinned tile shape is part of the descriptor; malformed values are refused
    for tc in (capi.tile_config(256, 2), capi.tile_config(256, 1), capi.tile_config(128, 1), capi.tile_config(64, 1),
               capi.tile_config(256, 2, 1), capi.tile_config(0, 0, 1), capi.tile_config(kbatch=1), capi.tile_config(kbatch=4),
               capi.tile_config(128, 1, kbatch=8), capi.tile_config(256, 2, balanced=1), capi.tile_config(balanced=1)):
        pinned = ck.DeviceGemm(tile_config=tc)
        assert pinned.IsSupportedArgument(pinned.MakeArgument(0x1000, 0x2000, 0x3000, 512, 512, 512, 512, 512, 512))
    for tc in (capi.tile_config(96, 1), capi.tile_config(128, 2), capi.tile_config(256, 3), -1, 1 << 28,
               capi.tile_config(kbatch=3), capi.tile_config(256, 2, kbatch=4), capi.tile_config(256, 1, kbatch=2, balanced=1),
               capi.tile_config(no_ksplit=1, balanced=1), 1 << 18):
        pinned = ck.DeviceGemm(tile_config=tc)
        assert not pinned.IsSupportedArgument(pinned.MakeArgument(0x1000, 0x2000, 0x3000, 512, 512, 512, 512, 512, 512))
    assert not op.IsSupportedArgument(op.MakeArgument(0x1000, 0x2000, 0x3000, 0, 8, 8, 8, 8, 8))
    # non-PassThrough A/B element ops cannot be applied by TMA
    assert not op.IsSupportedArgument(op.MakeArgument(0x1000, 0x2000, 0x3000, 8, 8, 8, 8, 8, 8, ck.Scale(2.0)))
    # all four A/B layout combinations; the leading dimension rule follows the layout
    for la in (capi.CKB_ROW_MAJOR, capi.CKB_COL_MAJOR):
        for lb in (capi.CKB_ROW_MAJOR, capi.CKB_COL_MAJOR):
            g = ck.DeviceGemm(capi.CKB_F16, la, lb)
            lda = 64 if la == capi.CKB_ROW_MAJOR else 256  # M=256, N=512, K=64
            ldb = 64 if lb == capi.CKB_COL_MAJOR else 512
            assert g.IsSupportedArgument(g.MakeArgument(0x1000, 0x2000, 0x3000, 256, 512, 64, lda, ldb, 512))
    km = ck.DeviceGemm(capi.CKB_F16, capi.CKB_COL_MAJOR, capi.CKB_COL_MAJOR)
    assert not km.IsSupportedArgument(km.MakeArgument(0x1000, 0x2000, 0x3000, 256, 512, 64, 64, 64, 512))  # lda < M
    assert not ck.DeviceGemm(capi.CKB_F16, 7, capi.CKB_COL_MAJOR).IsSupportedArgument(
        ck.DeviceGemm(capi.CKB_F16, 7, capi.CKB_COL_MAJOR).MakeArgument(0x1000, 0x2000, 0x3000, 8, 8, 8, 8, 8, 8))
    # int8 epilogues are int8-only
    assert not op.IsSupportedArgument(op.MakeArgument(0x1000, 0x2000, 0x3000, 8, 8, 8, 8, 8, 8, None, None,
                                                      ck.RequantReluRequant(0.03, 1.0)))
    i8 = ck.DeviceGemm(capi.CKB_I8)
    assert i8.IsSupportedArgument(i8.MakeArgument(0x1000, 0x2000, 0x3000, 3840, 4096, 4096, 4096, 4096, 4096,
                                                  None, None, ck.RequantReluRequant(0.03, 1.0)))
    # Run on an unsupported argument throws like the reference (device_gemm_xdl_cshuffle.hpp:475-481)
    bad = op.MakeArgument(0x1000, 0x2000, 0x3000, 100, 37, 72, 64, 72, 37)  # lda < K
    with pytest.raises(RuntimeError, match="invalid setting"):
        op.MakeInvoker().Run(bad)


def test_multiple_d_and_grouped_validation():
    md = ck.DeviceGemmMultipleD()
    arg = md.MakeArgument(0x1000, 0x2000, [0x4000, 0x5000], 0x3000, 3840, 4096, 4096, 4096, 4096, [0, 4096], 4096,
                          None, None, ck.AddAddFastGelu())
    assert md.IsSupportedArgument(arg)
    arg = md.MakeArgument(0x1000, 0x2000, [0x4000], 0x3000, 3840, 4096, 4096, 4096, 4096, [0], 4096,
                          None, None, ck.AddAddFastGelu())
    assert not md.IsSupportedArgument(arg)  # functor reads two D tensors
    g = ck.DeviceGroupedGemm()
    descs = [ck.GemmDescHost(256 * (1 + i % 16), 4096, 4096, 4096, 4096, 4096) for i in range(64)]
    ga = g.MakeArgument([0x1000] * 64, [0x2000] * 64, [], [0x3000] * 64, descs)
    assert g.IsSupportedArgument(ga)
    assert g.GetWorkSpaceSize(ga) >= 64 * 256
    with pytest.raises(RuntimeError, match="group_count"):
        g.MakeArgument([0x1000] * 3, [0x2000] * 64, [], [0x3000] * 64, descs)


def test_conv_validation():
    conv = ck.DeviceConvFwd()
    mk = lambda **kw: conv.MakeArgument(0x1000, 0x2000, 0x3000, kw.get("N", 128), 256, kw.get("C", 192), (71, 71),
                                        (3, 3), kw.get("out", (36, 36)), kw.get("s", (2, 2)), (1, 1), (1, 1), (1, 1),
                                        None, None, ck.AddRelu(), p_bias=0x4000)
    assert conv.IsSupportedArgument(mk())
    assert not conv.IsSupportedArgument(mk(out=(35, 36)))      # inconsistent geometry
    assert conv.IsSupportedArgument(mk(C=12))                   # pixel pitch not 16-byte: served through a padded copy
    assert conv.IsSupportedArgument(mk(C=3))                    # the reference's OddC case
    assert not conv.IsSupportedArgument(mk(s=(9, 9), out=(8, 8)))  # stride beyond the TMA limit
