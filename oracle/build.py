#!/usr/bin/env python3
"""Build the CPU oracle (test infrastructure, never shipped with the library).

  oracle/_build/liboracle.so   gcc -O2 build of attn_oracle.c (the C restatement)
  oracle/_ref/libref_attn.so   nvcc build of ref_shim.cu, which #includes the reference project's
                               own source files where they lie; only built when the reference tree
                               is present (it is not present on a GPU box; the prebuilt file
                               travels there instead)

Both are compiled without fast-math so that the restatement and the reference CPU code agree
bit for bit.  Run `python oracle/build.py` (add --force to rebuild).
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference project's tree: B200ATTN_REFERENCE_ROOT, else a directory `reference` beside this repository
REF_ROOT = os.environ.get("B200ATTN_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
ORACLE_SO = os.path.join(HERE, "_build", "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libref_attn.so")


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def build_oracle(force=False):
    src = os.path.join(HERE, "attn_oracle.c")
    if not force and _newer(ORACLE_SO, [src]):
        return ORACLE_SO
    os.makedirs(os.path.dirname(ORACLE_SO), exist_ok=True)
    cmd = ["gcc", "-O2", "-fPIC", "-shared", "-fno-fast-math", "-ffp-contract=off",
           "-o", ORACLE_SO, src, "-lm"]
    subprocess.check_call(cmd)
    return ORACLE_SO


def build_ref(force=False):
    """Returns the path of the reference shim library, or None if it cannot be had."""
    src = os.path.join(HERE, "ref_shim.cu")
    have_ref = os.path.isfile(os.path.join(REF_ROOT, "final", "attention.cu"))
    if not have_ref:
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, [src]):
        return REF_SO
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(os.path.dirname(REF_SO), exist_ok=True)
    cmd = [nvcc, "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
           "-Xcompiler", "-fPIC,-fno-fast-math,-ffp-contract=off", "-shared", "--fmad=true",
           "-w", f"-DREF_ROOT={REF_ROOT}", "-o", REF_SO, src]
    subprocess.check_call(cmd)
    return REF_SO


REF_DROPIN = os.path.join(HERE, "_ref", "ref_benchmark_dropin")


def build_ref_dropin(force=False):
    """The reference's only external caller (final/benchmark_pytorch_comparison.cu, compiled unmodified
    from the reference tree) linked against THIS library instead of the reference's own definition."""
    src = os.path.join(REF_ROOT, "final", "benchmark_pytorch_comparison.cu")
    lib = os.path.join(HERE, "..", "accelerated-final-project_b200", "lib", "libb200attn.so")
    if not os.path.isfile(src) or not os.path.exists(lib):
        return REF_DROPIN if os.path.exists(REF_DROPIN) else None
    if not force and _newer(REF_DROPIN, [src]):
        return REF_DROPIN
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(os.path.dirname(REF_DROPIN), exist_ok=True)
    libdir = os.path.dirname(os.path.abspath(lib))
    subprocess.check_call([nvcc, "-O3", "-w", "-gencode", "arch=compute_100a,code=sm_100a", src, "-o", REF_DROPIN,
                           "-L", libdir, "-lb200attn", "-Xlinker", "-rpath=$ORIGIN/../../accelerated-final-project_b200/lib"])
    return REF_DROPIN


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_oracle(force))
    print(build_ref(force))
    print(build_ref_dropin(force))
