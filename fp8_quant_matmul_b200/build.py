"""Builds libfp8bs.so (the CUDA kernels + C ABI) and the C++ harness programs in-tree.

    python -m fp8_quant_matmul_b200.build [--force] [-v] [--profile[=LEVEL]]

nvcc cross-compiles for sm_100a, so this works on a machine without a GPU.

--profile additionally builds lib/libfp8bs_prof.so, the same library compiled with -DFP8BS_PROFILE=LEVEL
(1: per-CTA time stamps of the kernel's phases; 2: plus cycle counters around every barrier wait; 3, the default:
plus a per-K-block time line of CTA 0).  The instrumented kernels write into a buffer that the extra export
fp8bs_debug_prof(long long* out, int n) copies back; csrc/gemm_kernel.cuh documents its layout.  The timers perturb
what they measure (a K block costs 10-15 % more), so that library is for finding out where time goes, never for
timing; nothing else in the package loads it.
"""
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
HOST = os.path.join(PKG_DIR, "host")
LIB_DIR = os.path.join(PKG_DIR, "lib")
BIN_DIR = os.path.join(PKG_DIR, "bin")
LIB_PATH = os.path.join(LIB_DIR, "libfp8bs.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build failed: %s\n%s" % (" ".join(cmd), proc.stdout))
    return proc.stdout


def build_library(force=False, verbose=False):
    """Compile csrc/*.cu into lib/libfp8bs.so; returns the path."""
    sources = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC))]
    sources.append(os.path.join(ROOT, "include", "fp8bs.h"))
    if not force and _newer(LIB_PATH, sources):
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [_nvcc()] + NVCC_FLAGS + ["-shared", "-o", LIB_PATH, os.path.join(CSRC, "fp8bs.cu")]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    out = _run(cmd)
    if verbose:
        print(out)
    return LIB_PATH


def build_profile_library(level=3):
    """Compile the instrumented variant lib/libfp8bs_prof.so (see the module docstring)."""
    os.makedirs(LIB_DIR, exist_ok=True)
    out = os.path.join(LIB_DIR, "libfp8bs_prof.so")
    _run([_nvcc()] + NVCC_FLAGS + ["-DFP8BS_PROFILE=%d" % int(level), "-shared", "-o", out, os.path.join(CSRC, "fp8bs.cu")])
    return out


def build_programs(force=False):
    """Compile the C++ harness programs host/check.cpp and host/sgemm.cpp into bin/."""
    built = []
    if not os.path.isdir(HOST):
        return built
    os.makedirs(BIN_DIR, exist_ok=True)
    for name in ("check", "sgemm"):
        src = os.path.join(HOST, name + ".cpp")
        if not os.path.exists(src):
            continue
        dst = os.path.join(BIN_DIR, name)
        deps = [src, LIB_PATH] + [os.path.join(HOST, f) for f in os.listdir(HOST) if f.endswith(".h")]
        if force or not _newer(dst, deps):
            _run([_nvcc(), "-O2", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-o", dst, src,
                  "-L", LIB_DIR, "-lfp8bs", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../lib"])
        built.append(dst)
    return built


def build_all(force=False, verbose=False):
    lib = build_library(force=force, verbose=verbose)
    progs = build_programs(force=force)
    return lib, progs


if __name__ == "__main__":
    lib, progs = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(lib)
    for arg in sys.argv[1:]:
        if arg.startswith("--profile"):
            print(build_profile_library(int(arg.split("=")[1]) if "=" in arg else 3))
    for p in progs:
        print(p)
