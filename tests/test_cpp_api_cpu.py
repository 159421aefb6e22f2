"""CPU tests of the C++ side of the boundary: the Composable-Kernel-compatible headers under
include/ck compile with g++ against libckb200.so, the host-only checks in tests/cpp pass, and the
example drivers (reference-style mains with the reference's template argument lists) build."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "composable_kernel_b200", "lib")


def test_host_api_checks_pass():
    from composable_kernel_b200 import capi
    capi.lib()  # the shared library must exist: the C++ layer links against it
    out_dir = os.path.join(ROOT, "tests", "cpp", "bin")
    os.makedirs(out_dir, exist_ok=True)
    exe = os.path.join(out_dir, "host_api_test")
    cmd = ["g++", "-std=c++17", "-O1", "-fexcess-precision=16", "-ffp-contract=off", "-pthread",
           "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "host_api_test.cpp"),
           "-o", exe, "-L", LIBDIR, "-lckb200", f"-Wl,-rpath,{LIBDIR}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout[-3000:]
    assert "all host API checks passed" in run.stdout


def test_work_plan_covers_every_tile_exactly_once():
    """Host-only sweep over the kernel's work decomposition (tile order, column-slice tail, K-split plans, batched
    and grouped tile tables), compiled by g++ alone from the header the kernel itself includes."""
    out_dir = os.path.join(ROOT, "tests", "cpp", "bin")
    os.makedirs(out_dir, exist_ok=True)
    exe = os.path.join(out_dir, "work_plan_test")
    cmd = ["g++", "-std=c++17", "-O2", "-I", os.path.join(ROOT, "composable_kernel_b200", "csrc"),
           os.path.join(ROOT, "tests", "cpp", "work_plan_test.cpp"), "-o", exe]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-3000:]
    assert "work plan checks passed" in run.stdout


def test_example_drivers_build():
    res = subprocess.run(["make", "-C", os.path.join(ROOT, "examples"), "-j4"], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    for name in ("gemm_xdl_fp16", "gemm_add_add_fastgelu_xdl_fp16", "gemm_xdl_requant_relu_requant_int8",
                 "grouped_gemm_xdl_fp16", "conv2d_fwd_xdl_bias_relu", "ck_profiler", "convnd_fwd_instance_engine",
                 "gemm_bilinear_xdl_fp16", "gemm_bias_relu_xdl_fp16", "grouped_gemm_bias_xdl_fp16",
                 "convnd_fwd_xdl_fp16", "convnd_fwd_xdl_int8", "client_gemm",
                 "client_gemm_add_add_fastgelu", "test_gemm_instances"):
        assert os.path.exists(os.path.join(ROOT, "examples", "bin", name))
