#!/usr/bin/env python
"""Benchmark of the dense-contraction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Headline workload (default): fp16 GEMM 3840 x 4096 x 4096, A row-major, B column-major, fp32
accumulate (the reference's example/01_gemm shape).  A "step" is one launch of the kernel over one
set of synthetic inputs already resident in HBM; several input sets are rotated so that a step
never finds its operands in L2.  Prints ONE JSON line on rank 0.

N > 1 (launched under torch.distributed.run, one rank per GPU): the headline GEMM runs as
independent replicas (weak scaling, no collective on the data path); the convolution is sharded
over the batch and the grouped GEMM over groups (FLOP-balanced), reported under "workloads".

--impl reference times the CPU restatement of the reference's own host operators (oracle/) on the
host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from composable_kernel_b200.sharding import batch_shard, grouped_gemm_shard  # noqa: E402

# fp16 GEMM 3840x4096x4096 on MI100: example/01_gemm/README.md:11-22 of the reference
PUBLISHED_MI100_TFLOPS = {"gemm_fp16": 107.657, "gemm_fastgelu": 101.525, "conv": 105.581}
FALLBACK_PEAK_TFLOPS = 1590.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"bf16_tflops": FALLBACK_PEAK_TFLOPS, "hbm_gbs": 6650.0}, "fallback"


def ncu_traffic(workload):
    """Per-launch DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of the workload's kernel,
    taken from the committed ncu summary profiles/dram_traffic_per_launch.txt ("name bytes" lines)."""
    path = os.path.join(ROOT, "profiles", "dram_traffic_per_launch.txt")
    if os.path.exists(path):
        for ln in open(path):
            parts = ln.split()
            if len(parts) >= 2 and parts[0] == workload:
                return float(parts[1])
    return None


# ------------------------------------------------------------------------------------------------
# clocks sampling (NVML, read-only) during the timed region
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    def __init__(self, index):
        self.samples, self.power, self.reasons, self.max_mhz = [], [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    self.power.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
                except Exception:
                    pass
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.001)

    def start(self):
        if self._nv:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples),
                "power_w": statistics.median(self.power) if self.power else None}


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------
class GemmWorkload:
    """C1 / C2 / C3: M=3840 N=4096 K=4096, A row-major, B column-major."""

    def __init__(self, name, torch, ck, capi):
        self.name, self.torch, self.ck, self.capi = name, torch, ck, capi
        self.M, self.N, self.K = 3840, 4096, 4096
        self.i8 = name == "gemm_int8"
        self.flop = 2 * self.M * self.N * self.K
        eb = 1 if self.i8 else 2
        self.bytes = eb * (self.M * self.K + self.K * self.N + self.M * self.N)
        if name == "gemm_fastgelu":
            self.bytes += 2 * self.N + 2 * self.M * self.N  # example/04...:202-204
        self.dtype = "i8" if self.i8 else "f16"
        self.unit = "TOPS" if self.i8 else "TFLOPS"
        self.desc = {
            "gemm_fp16": "fp16 GEMM 3840x4096x4096, A row-major, B column-major, fp32 accumulate, PassThrough",
            "gemm_int8": "int8 GEMM 3840x4096x4096 + Requant-ReLU-Requant (rne, s0=0.03, s1=14), int32 accumulate",
            "gemm_fastgelu": "fp16 GEMM 3840x4096x4096 + Add + Add + FastGelu (D0 bias stride 0, D1 MxN)",
        }[name]

    def host_inputs(self, seed):
        rng = np.random.default_rng(seed)
        M, N, K = self.M, self.N, self.K
        if self.i8:
            return [rng.integers(-5, 6, (M, K)).astype(np.int8), rng.integers(-5, 6, (N, K)).astype(np.int8)]
        if self.name == "gemm_fp16":
            return [rng.integers(-5, 6, (M, K)).astype(np.float16), rng.integers(-5, 6, (N, K)).astype(np.float16)]
        return [rng.uniform(-1, 1, (M, K)).astype(np.float16), rng.uniform(-1, 1, (N, K)).astype(np.float16),
                rng.uniform(-1, 1, (N,)).astype(np.float16), rng.uniform(-1, 1, (M, N)).astype(np.float16)]

    def op(self):
        ck = self.ck
        return {"gemm_fp16": ck.PassThrough(), "gemm_int8": ck.RequantReluRequantRne(0.03, 14.0),
                "gemm_fastgelu": ck.AddAddFastGelu()}[self.name]

    def make_set(self, host):
        torch = self.torch
        dev = [torch.from_numpy(h).cuda() for h in host]
        e = torch.empty((self.M, self.N), dtype=torch.int8 if self.i8 else torch.float16, device="cuda")
        return self.bind(dev, e)

    def bind(self, dev, e):
        ck, capi = self.ck, self.capi
        gemm = ck.DeviceGemmMultipleD(capi.CKB_I8 if self.i8 else capi.CKB_F16)
        ds = [t.data_ptr() for t in dev[2:]]
        lds = [0, self.N][:len(ds)]
        arg = gemm.MakeArgument(dev[0].data_ptr(), dev[1].data_ptr(), ds, e.data_ptr(), self.M, self.N, self.K,
                                self.K, self.K, lds, self.N, None, None, self.op())
        if not gemm.IsSupportedArgument(arg):
            raise RuntimeError("unsupported: " + capi.last_error())
        return {"op": gemm, "arg": arg, "inv": gemm.MakeInvoker(), "dev": dev, "e": e}

    def n_sets(self):
        return 4  # 4 x ~96 MB (fp16) of operands: a set is out of the 126 MB L2 before it is reused

    def oracle_rows(self, host, rows, oracle, threads):
        """Reference CPU path on the first `rows` rows of E; returns flop done."""
        a, bt = host[0][:rows], host[1]
        d0 = np.broadcast_to(host[2], (rows, self.N)) if len(host) > 2 else None
        d1 = host[3][:rows] if len(host) > 3 else None
        op = self.op()
        oracle.gemm(a, bt.T, op.kind, op.params, d0, d1, fast=False, threads=threads)
        return 2 * rows * self.N * self.K


class ConvWorkload:
    """C4: N128 C192 71x71 K256 3x3 s2 p1 + bias + ReLU; batch-sharded over ranks."""

    def __init__(self, torch, ck, capi, rank, world):
        self.name, self.torch, self.ck, self.capi = "conv", torch, ck, capi
        self.Ntot, self.C, self.Hi, self.Wi, self.K, self.Ho, self.Wo = 128, 192, 71, 71, 256, 36, 36
        b0, b1 = batch_shard(self.Ntot, rank, world)
        self.Nloc = b1 - b0
        self.flop_total = 2 * self.Ntot * self.K * self.Ho * self.Wo * self.C * 9
        self.flop = 2 * self.Nloc * self.K * self.Ho * self.Wo * self.C * 9
        self.traffic_scale = self.Nloc / self.Ntot  # the ncu summary states the 128-image launch
        self.bytes = 2 * (self.Nloc * self.C * self.Hi * self.Wi + self.K * self.C * 9 +
                          self.Nloc * self.K * self.Ho * self.Wo) + 2 * self.K
        self.dtype, self.unit = "f16", "TFLOPS"
        self.desc = ("fp16 conv2d fwd NHWC/KYXC/NHWK + bias + ReLU, N128 C192 71x71 K256 3x3 s2 p1 "
                     f"(batch shard {self.Nloc} per GPU)")
        self.rank = rank

    def host_inputs(self, seed):
        rng = np.random.default_rng(seed)
        return [rng.uniform(-1, 1, (self.Nloc, self.Hi, self.Wi, self.C)).astype(np.float16),
                rng.uniform(-1, 1, (self.K, 3, 3, self.C)).astype(np.float16),
                rng.uniform(-1, 1, (self.K,)).astype(np.float16)]

    def make_set(self, host):
        torch = self.torch
        dev = [torch.from_numpy(h).cuda() for h in host]
        e = torch.empty((self.Nloc, self.Ho, self.Wo, self.K), dtype=torch.float16, device="cuda")
        return self.bind(dev, e)

    def bind(self, dev, e):
        ck = self.ck
        conv = ck.DeviceConvFwd()
        arg = conv.MakeArgument(dev[0].data_ptr(), dev[1].data_ptr(), e.data_ptr(), self.Nloc, self.K, self.C,
                                (self.Hi, self.Wi), (3, 3), (self.Ho, self.Wo), (2, 2), (1, 1), (1, 1), (1, 1),
                                None, None, ck.AddRelu(), p_bias=dev[2].data_ptr())
        if not conv.IsSupportedArgument(arg):
            raise RuntimeError("unsupported: " + self.capi.last_error())
        return {"op": conv, "arg": arg, "inv": conv.MakeInvoker(), "dev": dev, "e": e}

    def n_sets(self):
        return 2  # one input shard is 248 MB at N=1; two sets stay beyond L2 down to 8 GPUs

    def oracle_rows(self, host, images, oracle, threads):
        oracle.conv2d_fwd(host[0][:images], host[1], (2, 2), (1, 1), (1, 1), epilogue=oracle.EPI_ADD_RELU,
                          bias=host[2], fast=False, threads=threads)
        return 2 * images * self.K * self.Ho * self.Wo * self.C * 9


class GroupedWorkload:
    """C5: 64 groups, M_g = 256*(1 + g mod 16), N = K = 4096; groups partitioned over ranks by LPT."""

    def __init__(self, torch, ck, capi, rank, world, groups=64):
        self.name, self.torch, self.ck, self.capi = "grouped", torch, ck, capi
        self.N = self.K = 4096
        all_m = [256 * (1 + g % 16) for g in range(groups)]
        self.mine = grouped_gemm_shard(all_m, rank, world)
        self.Ms = [all_m[g] for g in self.mine]
        self.flop_total = sum(2 * m * self.N * self.K for m in all_m)
        self.flop = sum(2 * m * self.N * self.K for m in self.Ms)
        # share of the 64-group benchmark launch (whose DRAM traffic the ncu summary states) that this GPU runs
        self.traffic_scale = self.flop / sum(2 * 256 * (1 + g % 16) * self.N * self.K for g in range(64))
        self.bytes = sum(2 * (m * self.K + self.K * self.N + m * self.N) for m in self.Ms)
        self.dtype, self.unit = "f16", "TFLOPS"
        self.desc = (f"fp16 grouped GEMM, {groups} groups M_g=256*(1+g%16) N=K=4096, "
                     f"{len(self.mine)} groups on this GPU (FLOP-balanced LPT)")

    def make_set(self, host=None):
        torch, ck = self.torch, self.ck
        gen = torch.Generator(device="cuda").manual_seed(11939 + 5000)
        dA = [torch.empty((m, self.K), dtype=torch.float16, device="cuda").uniform_(-1, 1, generator=gen) for m in self.Ms]
        dB = [torch.empty((self.N, self.K), dtype=torch.float16, device="cuda").uniform_(-1, 1, generator=gen) for _ in self.Ms]
        dE = [torch.empty((m, self.N), dtype=torch.float16, device="cuda") for m in self.Ms]
        gg = ck.DeviceGroupedGemm()
        arg = gg.MakeArgument([x.data_ptr() for x in dA], [x.data_ptr() for x in dB], [], [x.data_ptr() for x in dE],
                              [ck.GemmDescHost(m, self.N, self.K, self.K, self.K, self.N) for m in self.Ms])
        ws = torch.empty(gg.GetWorkSpaceSize(arg), dtype=torch.uint8, device="cuda")
        gg.SetWorkSpacePointer(arg, ws.data_ptr())
        if not gg.IsSupportedArgument(arg):
            raise RuntimeError("unsupported: " + self.capi.last_error())
        return {"op": gg, "arg": arg, "inv": gg.MakeInvoker(), "dev": (dA, dB, ws), "e": dE}

    def n_sets(self):
        return 1  # > 0.5 GB of operands per GPU even at 8 GPUs: far beyond L2


# ------------------------------------------------------------------------------------------------
def time_steps(torch, sets, steps, warmup, stream_cfg, dist_barrier):
    """W warm-up steps, then K timed steps bracketed by barrier + synchronize.  Returns
    (total_ms over the K steps, [mean launch ms] * K)."""
    n = len(sets)
    for i in range(warmup):
        s = sets[i % n]
        s["inv"].Run(s["arg"], stream_cfg)
    torch.cuda.synchronize()
    dist_barrier()
    torch.cuda.synchronize()
    # Two events around the K launches: nothing sits between consecutive kernels in the stream (a launch may
    # begin its start-up while the one before it drains), and the mean launch duration is total / K.
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        s = sets[i % n]
        s["inv"].Run(s["arg"], stream_cfg)
    stop.record()
    torch.cuda.synchronize()
    dist_barrier()
    torch.cuda.synchronize()
    total = start.elapsed_time(stop)
    return total, [total / steps] * steps


def sustained_run(torch, sets, seconds, kern_ms, stream_cfg, sampler):
    """The same launches back to back for at least `seconds`: the regime in which the part runs against its power
    cap (the timed region of the headline lasts milliseconds and runs at burst clocks).  Launches are queued in
    chunks of about 50 ms with a synchronise between chunks; clocks and power are sampled (read-only) from the
    first chunk's end on.  Returns (launches, elapsed ms, clocks)."""
    n = len(sets)
    chunk = max(1, int(50.0 / max(kern_ms, 1e-3)))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = 0
    t0 = time.perf_counter()
    start.record()
    while True:
        for i in range(chunk):
            s = sets[(launches + i) % n]
            s["inv"].Run(s["arg"], stream_cfg)
        launches += chunk
        torch.cuda.synchronize()
        if launches == chunk and sampler is not None:
            sampler.start()
        if time.perf_counter() - t0 >= seconds:
            break
    stop.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler is not None else None
    return launches, start.elapsed_time(stop), clocks


def metric_name(unit):
    return ("TFLOPS per GPU vs B200 dense peak; box TFLOPS over all GPUs" if unit == "TFLOPS"
            else "TOPS per GPU vs B200 dense peak; box TOPS over all GPUs")


def run_reference_arm(args, rank, world):
    """CPU restatement of the reference's host operators, all host threads, bounded sample."""
    if rank != 0:
        return
    from oracle import ck_oracle as oracle
    name = args.workload
    threads = oracle.hardware_concurrency()

    class _NoTorch:
        pass
    if name in ("gemm_fp16", "gemm_int8", "gemm_fastgelu"):
        wl = GemmWorkload(name, None, __import__("composable_kernel_b200"), None)
        host = wl.host_inputs(11939)
        unit_rows, full = 64, wl.M
    elif name == "conv":
        wl = ConvWorkload(None, __import__("composable_kernel_b200"), None, 0, 1)
        host = wl.host_inputs(11939)
        host[0] = host[0][:4]
        unit_rows, full = 1, wl.Ntot
    else:
        wl = GemmWorkload("gemm_fp16", None, __import__("composable_kernel_b200"), None)
        wl.desc = "fp16 grouped GEMM (one 256-row slice of a group: N=K=4096)"
        host = wl.host_inputs(11939)
        unit_rows, full = 64, wl.M
    # size the per-step sample to roughly one second
    t0 = time.perf_counter()
    flop = wl.oracle_rows(host, unit_rows, oracle, threads)
    dt = max(time.perf_counter() - t0, 1e-3)
    rows = int(max(unit_rows, min(full if name != "conv" else 4, unit_rows * (1.0 / dt))))
    for _ in range(args.warmup):
        wl.oracle_rows(host, rows, oracle, threads)
    t0 = time.perf_counter()
    done = 0
    for _ in range(args.steps):
        done += wl.oracle_rows(host, rows, oracle, threads)
    dt = time.perf_counter() - t0
    value = done / dt / 1e12
    sample = (f"{rows} of {full} output rows per step" if name != "conv" else f"{rows} of {full} images per step")
    line = {
        # same metric string as the GPU arm (the driver pairs the two lines); the path measured is named in config
        "impl": "reference", "metric": metric_name(wl.unit), "value": value,
        "unit": wl.unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": wl.dtype, "data": "synthetic", "config": {"workload": wl.desc, "sample": sample, "path": "CPU restatement of the reference's host operators, all host threads"},
        "cpu_baseline": {"value": value, "unit": wl.unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def print_role_cycles():
    """Role cycle counters of the last launch (profiling builds of the library only: -DCKB_TRACE exports
    ckb_trace_read; 16 words per CTA, see the top of csrc/ckb_kernel.cuh).  Means over the CTAs that ran the role."""
    import ctypes
    import numpy as np
    from composable_kernel_b200 import capi
    L = capi.lib()
    if not hasattr(L, "ckb_trace_read"):
        print("--role-cycles needs a library built with -DCKB_TRACE (python -m composable_kernel_b200.build "
              "--variant trace CKB_TRACE=1; CKB200_LIB=.../libckb200_trace.so)", file=sys.stderr)
        return
    n = 148
    buf = (ctypes.c_uint64 * (n * 16))()
    L.ckb_trace_read.argtypes = [ctypes.c_void_p, ctypes.c_int]
    if L.ckb_trace_read(buf, n * 16) != 0:
        print("ckb_trace_read failed: " + capi.last_error(), file=sys.stderr)
        return
    t = np.array(buf[:], dtype=np.int64).reshape(n, 16)
    mma = t[t[:, 7] > 0]  # CTAs whose MMA role ran (the leaders of CTA pairs)
    names = ["producer wait for a free stage", "producer loop", "MMA wait for operand data", "MMA wait for an accumulator",
             "MMA loop", "epilogue wait for the MMA", "epilogue loop", "stages issued", "MMA issue", "MMA commit"]
    out = {}
    for i, nm in enumerate(names):
        col = mma[:, i] if i in (2, 3, 4, 7, 8, 9) else t[:, i]
        out[nm] = {"mean": float(col.mean()), "min": int(col.min()), "max": int(col.max())}
    st = mma[:, 7].mean()
    out["per stage"] = {k: float(mma[:, i].mean() / st) for k, i in
                        (("MMA loop", 4), ("wait for data", 2), ("issue", 8), ("commit", 9))}
    print(json.dumps({"role_cycles": out}), file=sys.stderr)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemm_fp16",
                    choices=["gemm_fp16", "gemm_int8", "gemm_fastgelu", "conv", "grouped"])
    ap.add_argument("--no-extra", action="store_true", help="skip the other workloads / e2e / cpu baseline")
    ap.add_argument("--groups", type=int, default=64,
                    help="grouped workload: number of groups (64 = the benchmark; 16, one period of the group "
                         "sizes and about 1.1 GB, is the case small enough for a multi-pass profiler capture)")
    ap.add_argument("--sustain-seconds", type=float, default=2.0,
                    help="length of the back-to-back run behind each workload's \"sustained\" block (0 = skip)")
    ap.add_argument("--role-cycles", action="store_true",
                    help="with a -DCKB_TRACE build of the library (CKB200_LIB): print the per-role cycle counters "
                         "of the last launch of the workload on stderr")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return 0

    import torch
    import composable_kernel_b200 as ck
    from composable_kernel_b200 import capi
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the library has no CPU path")
    capi.lib()
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # keep NCCL's version banner off stdout: one JSON line only
        import torch.distributed as dist_mod
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    stream_cfg = ck.StreamConfig(torch.cuda.current_stream().cuda_stream, False)
    peaks, peak_kind = measured_peaks()

    def make_workload(name):
        if name == "conv":
            return ConvWorkload(torch, ck, capi, rank, world)
        if name == "grouped":
            return GroupedWorkload(torch, ck, capi, rank, world, args.groups)
        return GemmWorkload(name, torch, ck, capi)

    def measure(name, steps, warmup, sample_clocks=False):
        wl = make_workload(name)
        hosts = None
        if name == "grouped":
            sets = [wl.make_set() for _ in range(wl.n_sets())]
        else:
            hosts = [wl.host_inputs(11939 + 17 * i + 1000 * rank) for i in range(wl.n_sets())]
            sets = [wl.make_set(h) for h in hosts]
        sampler = ClockSampler(local_rank) if sample_clocks else None
        before = ck.launch_count()
        if sampler:
            sampler.start()
        total_ms, per = time_steps(torch, sets, steps, warmup, stream_cfg, barrier)
        clocks = sampler.stop() if sampler else None
        launches = ck.launch_count() - before - warmup
        if ck.device_status() != 0:
            raise RuntimeError("kernel reported a wait time-out")
        total_ms = max_over_ranks(total_ms)
        sharded = name in ("conv", "grouped")
        flop_job = (wl.flop_total if sharded else wl.flop * world)
        value = flop_job * steps / (total_ms * 1e-3) / 1e12
        kern_ms = statistics.mean(per)
        achieved = wl.flop / (kern_ms * 1e-3) / 1e12
        # `frac` is always against the burst measurement of the peak file (a cuBLAS bf16 GEMM timed alone, as these
        # launches are); the fraction against the sustained measurement is stated beside it, and the "sustained"
        # block below repeats the comparison in the regime where the power cap decides the clock.
        int8 = wl.dtype == "i8"
        peak = peaks["bf16_tflops"] * (2.0 if int8 else 1.0)
        peak_sus = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) * (2.0 if int8 else 1.0)
        peak_note = f"{peak_kind} bf16 burst" + (" x2: no int8 peak was measured, twice the bf16 figure is ASSUMED" if int8 else "")
        # the ncu figure is for the whole workload on one GPU; a shard's launch moves its share of it
        traffic = ncu_traffic(name)
        if traffic is not None:
            traffic *= getattr(wl, "traffic_scale", 1.0)
        res = {
            "workload": wl.desc, "value": value, "unit": wl.unit, "ms_per_step": total_ms / steps,
            "scaling": "strong" if sharded else "weak",
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s" if int8 else "TFLOP/s",
                         "frac": achieved / peak, "traffic": traffic,
                         "peak_source": peak_note, "frac_of_sustained_peak": achieved / peak_sus,
                         "timed_region_ms": total_ms,
                         "traffic_source": "ncu capture of one launch, profiles/dram_traffic_per_launch.txt (lines "
                                           "still dirty in L2 at kernel end are not counted)",
                         "kernel_ms": kern_ms, "hbm_gbs_algorithmic": wl.bytes / (kern_ms * 1e-3) / 1e9},
            "gpu_launches": launches,
        }
        if args.sustain_seconds > 0:
            n_l, ms_l, clk = sustained_run(torch, sets, args.sustain_seconds, kern_ms, stream_cfg,
                                           ClockSampler(local_rank))
            if ck.device_status() != 0:
                raise RuntimeError("kernel reported a wait time-out")
            rate = wl.flop * n_l / (ms_l * 1e-3) / 1e12
            mhz, mx = (clk or {}).get("sm_mhz"), (clk or {}).get("sm_max_mhz")
            res["sustained"] = {
                "value": rate, "unit": wl.unit, "launches": n_l, "seconds": ms_l * 1e-3, "kernel_ms": ms_l / n_l,
                "peak": peak_sus, "frac": rate / peak_sus,
                "peak_source": peak_note.replace("burst", "sustained"),
                "sm_mhz": mhz, "sm_max_mhz": mx, "power_w": (clk or {}).get("power_w"),
                "reasons": (clk or {}).get("reasons"),
                # what the same kernel would deliver at the maximum clock: separates kernel quality from the power cap
                "value_at_max_clock": rate * mx / mhz if mhz and mx else None,
            }
        return wl, sets, hosts, res, clocks

    wl, sets, hosts, head, clocks = measure(args.workload, args.steps, args.warmup, sample_clocks=True)
    if args.role_cycles and rank == 0:
        print_role_cycles()

    # ---- end to end through the public API with host buffers (pinned), copies inside the timed region
    e2e = None
    if hosts is not None:
        # Two lanes (stream + device buffers + pinned result each) alternate between steps, so that the
        # upload of step i+1 overlaps the download of step i on the full-duplex link.  Every step still
        # uploads all of its inputs from pinned host memory and downloads its whole result.
        e2e_steps = max(6, min(args.steps, 20))
        e2e_steps += e2e_steps % 2
        pinned_in = [torch.from_numpy(h).pin_memory() for h in hosts[0]]
        h2d = sum(t.numel() * t.element_size() for t in pinned_in)
        lanes = []
        for _ in range(2):
            st = torch.cuda.Stream()
            dev_in = [torch.empty_like(t, device="cuda") for t in pinned_in]
            e_dev = torch.empty_like(sets[0]["e"])
            e_host = torch.empty(e_dev.shape, dtype=e_dev.dtype).pin_memory()
            lanes.append({"stream": st, "dev_in": dev_in, "e_dev": e_dev, "e_host": e_host,
                          "bound": wl.bind(dev_in, e_dev), "cfg": ck.StreamConfig(st.cuda_stream, False)})
        d2h = lanes[0]["e_host"].numel() * lanes[0]["e_host"].element_size()

        def e2e_step(i, with_kernel=True):
            ln = lanes[i % 2]
            with torch.cuda.stream(ln["stream"]):
                for d, p in zip(ln["dev_in"], pinned_in):
                    d.copy_(p, non_blocking=True)
                if with_kernel:
                    ln["bound"]["inv"].Run(ln["bound"]["arg"], ln["cfg"])
                ln["e_host"].copy_(ln["e_dev"], non_blocking=True)

        def e2e_loop(with_kernel):
            for i in range(4):
                e2e_step(i, with_kernel)
            torch.cuda.synchronize()
            barrier()
            torch.cuda.synchronize()
            t_begin = time.perf_counter()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for ln in lanes:
                ln["stream"].wait_event(s)
            for i in range(e2e_steps):
                e2e_step(i, with_kernel)
            for ln in lanes:
                torch.cuda.current_stream().wait_stream(ln["stream"])
            e.record()
            torch.cuda.synchronize()
            wall = (time.perf_counter() - t_begin) * 1e3
            barrier()
            return max_over_ranks(s.elapsed_time(e)), wall

        ms, wall_ms = e2e_loop(True)
        # The same loop with the kernel launch left out: what the host-to-device and device-to-host copies cost by
        # themselves at this number of GPUs (every rank copies at the same time).  When this equals the end-to-end
        # time, the host side of the link bounds the step, not the kernel.
        copy_ms, _ = e2e_loop(False)
        sharded = args.workload in ("conv", "grouped")
        flop_job = wl.flop_total if sharded else wl.flop * world
        e2e = {"value": flop_job * e2e_steps / (ms * 1e-3) / 1e12, "unit": wl.unit,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
               "ms_per_step": ms / e2e_steps, "wall_ms_per_step": wall_ms / e2e_steps,
               "overlap": "two lanes: upload of step i+1 overlaps download of step i",
               "copy_only": {"ms_per_step": copy_ms / e2e_steps,
                             "h2d_gbs_per_gpu": h2d * e2e_steps / (copy_ms * 1e-3) / 1e9,
                             "d2h_gbs_per_gpu": d2h * e2e_steps / (copy_ms * 1e-3) / 1e9,
                             "share_of_e2e": copy_ms / ms,
                             "note": "same loop without the kernel launch, all ranks copying at once"}}
        del pinned_in, lanes

    # ---- CPU baseline (rank 0, N = 1): the reference's host path restated, bounded sample
    cpu = None
    if rank == 0 and world == 1 and not args.no_extra and hosts is not None:
        from oracle import ck_oracle as oracle
        threads = oracle.hardware_concurrency()
        unit = 64 if args.workload != "conv" else 1
        t0 = time.perf_counter()
        wl.oracle_rows(hosts[0], unit, oracle, threads)
        dt = max(time.perf_counter() - t0, 1e-3)
        full = wl.M if args.workload != "conv" else wl.Nloc
        rows = int(max(unit, min(full, unit * 12.0 / dt)))  # about 12 s of CPU work
        t0 = time.perf_counter()
        flop = wl.oracle_rows(hosts[0], rows, oracle, threads)
        dt = time.perf_counter() - t0
        what = "output rows" if args.workload != "conv" else "images"
        cpu = {"value": flop / dt / 1e12, "unit": wl.unit, "cores": threads, "kind": "port",
               "sample": f"first {rows} of {full} {what} of the same inputs, naive per-output loops, {dt:.1f} s"}

    del sets
    torch.cuda.empty_cache()

    # ---- the other configurations (not part of the headline timed region)
    others = {}
    if not args.no_extra:
        for name in ["gemm_fp16", "gemm_int8", "gemm_fastgelu", "conv", "grouped"]:
            if name == args.workload:
                continue
            _, s2, _, r2, _ = measure(name, 20, 3)
            others[name] = r2
            del s2
            torch.cuda.empty_cache()

    if rank == 0:
        pub = PUBLISHED_MI100_TFLOPS.get(args.workload)
        roof = dict(head["roofline"])
        line = {
            "metric": metric_name(wl.unit),
            "value": head["value"], "unit": wl.unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": head["scaling"],
            "vs_baseline": (head["value"] / pub) if pub else None,
            "dtype": wl.dtype, "data": "synthetic",
            "config": {"workload": head["workload"],
                       "l2": f"{wl.n_sets()} input sets rotated; operands of a step are beyond the 126 MB L2 when reused"
                             if wl.n_sets() > 1 else "operands per step far exceed the 126 MB L2",
                       "parallelism": ("replicas" if head["scaling"] == "weak" else "sharded, no collective") +
                                      f" x{world}",
                       "vs_baseline_note": "published number is the reference's MI100 figure for the same shape"},
            "roofline": {k: roof[k] for k in ("bound", "achieved", "peak", "unit", "frac", "traffic")},
            "roofline_detail": {k: roof[k] for k in ("peak_source", "frac_of_sustained_peak", "timed_region_ms",
                                                     "traffic_source", "kernel_ms", "hbm_gbs_algorithmic")},
            "sustained": head.get("sustained"),
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": head["gpu_launches"], "clocks": clocks,
            "workloads": others,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
