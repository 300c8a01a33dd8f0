"""The drop-in boundary exercised from C++, the reference's own host language: (1) a driver in the
shape of the reference's test programs (tests/cpp/dropin_suite.cpp: rand() inputs, cudaMalloc'd
buffers, blocking launchers, CPU oracle, the reference's comparison rule), linked against the shared
library through include/b200attn.h only; (2) when it has been built from the reference tree, the
reference's ONLY external caller (final/benchmark_pytorch_comparison.cu, unmodified) linked against
this library in place of the reference's own definition."""
import os
import re
import shutil
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def test_cpp_driver_in_the_shape_of_the_reference_tests(pkg, cuda, tmp_path):
    import build as oracle_build
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available to build the C++ driver")
    libdir = os.path.dirname(pkg.LIB_PATH)
    oracle_so = oracle_build.build_oracle()
    exe = str(tmp_path / "dropin_suite")
    subprocess.check_call([nvcc, "-O2", "-std=c++17", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "dropin_suite.cpp"),
                           "-o", exe, "-L", libdir, "-lb200attn", oracle_so, "-Xlinker", f"-rpath={libdir}",
                           "-Xlinker", f"-rpath={os.path.dirname(oracle_so)}"])
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    print(r.stdout[-3000:], r.stderr[-1000:])
    assert r.returncode == 0 and "ALL TESTS PASSED" in r.stdout
    assert r.stdout.count("PASSED") >= 22


def test_reference_external_caller_links_against_the_library(pkg, cuda):
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_benchmark_dropin")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/ref_benchmark_dropin not built (needs the reference tree)")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, LD_LIBRARY_PATH=os.path.dirname(pkg.LIB_PATH) + ":" + os.environ.get("LD_LIBRARY_PATH", "")))
    print(r.stdout[-2000:], r.stderr[-1000:])
    assert r.returncode == 0
    times = [float(x) for x in re.findall(r"Time: ([0-9.]+) ms", r.stdout)]
    assert len(times) == 4 and all(0.0 < t < 1.0 for t in times)   # its four shapes, each well under a millisecond
