"""Times fp16 GEMMs (A row-major, B column-major, PassThrough) of the given shapes through the device-operation API
and, beside each, the same product through torch.matmul (cuBLAS) as a yardstick.

    python -m composable_kernel_b200.shape_sweep 512x512x8192 1024x1024x8192 [--no-splitk] [--reps 50]

Integer-valued operands in [-5, 5] (exact in fp32), so the two results are also compared bit for bit.  Times are
means over `reps` back-to-back launches between two CUDA events on the current stream, after 5 warm-up launches;
`--no-splitk` adds a column with the K split switched off (CKB_NO_SPLITK=1)."""
from __future__ import annotations

import argparse
import os

import torch

from . import capi
from .device_op import DeviceGemm, PassThrough, StreamConfig


def _time_us(fn, reps: int) -> float:
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / reps * 1e3


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("shapes", nargs="+", help="MxNxK")
    ap.add_argument("--reps", type=int, default=50)
    ap.add_argument("--no-splitk", action="store_true", help="also time the plan without the K split")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("shape_sweep needs a CUDA device")
    for text in args.shapes:
        M, N, K = (int(x) for x in text.lower().split("x"))
        a = torch.randint(-5, 6, (M, K), device="cuda").to(torch.float16)
        bt = torch.randint(-5, 6, (N, K), device="cuda").to(torch.float16)
        e = torch.empty((M, N), dtype=torch.float16, device="cuda")
        gemm = DeviceGemm(capi.CKB_F16)
        arg = gemm.MakeArgument(a.data_ptr(), bt.data_ptr(), e.data_ptr(), M, N, K, K, K, N, None, None, PassThrough())
        if not gemm.IsSupportedArgument(arg):
            print(f"{text}: not supported: {capi.last_error()}")
            continue
        invoker = gemm.MakeInvoker()
        cfg = StreamConfig(torch.cuda.current_stream().cuda_stream, False)
        os.environ.pop("CKB_NO_SPLITK", None)
        t_ours = _time_us(lambda: invoker.Run(arg, cfg), args.reps)
        t_plain = None
        if args.no_splitk:
            os.environ["CKB_NO_SPLITK"] = "1"
            t_plain = _time_us(lambda: invoker.Run(arg, cfg), args.reps)
            os.environ.pop("CKB_NO_SPLITK", None)
        ref = torch.empty((M, N), dtype=torch.float16, device="cuda")
        t_lib = _time_us(lambda: torch.matmul(a, bt.t(), out=ref), args.reps)
        tflops = 2.0 * M * N * K / 1e6
        line = f"{text:>18s}: {t_ours:8.1f} us {tflops / t_ours:7.0f} TFLOPS"
        if t_plain is not None:
            line += f" | without K split {t_plain:8.1f} us"
        line += f" | cuBLAS {t_lib:8.1f} us {tflops / t_lib:7.0f} TFLOPS | equal bits: {torch.equal(e, ref)}"
        print(line, flush=True)


if __name__ == "__main__":
    main()
