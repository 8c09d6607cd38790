"""Builds ``rpl_b200/lib/librpl.so`` in-tree with nvcc (sm_100a only) and gcc.

    python -m rpl_b200.build [--force] [--verbose]

The library carries the CUDA kernels, the ``rplb_*`` device-level C ABI and the
reference-named C API (``rpl_host.c``).  nvcc cross-compiles without a GPU.
"""
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIB_DIR = os.path.join(PKG, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_PATH = os.path.join(LIB_DIR, "librpl.so")

CU_SOURCES = ["runtime.cu", "quant_kernels.cu", "gemm_i8_simt.cu", "gemm_i8_tcgen05.cu", "gemm_i8_fused_quant.cu", "gemm_api.cu", "sharded.cu"]
C_SOURCES = ["rpl_host.c"]
HEADERS = ["common.cuh", "gemm_common.cuh", "gemm_tc_common.cuh"]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--default-stream", "legacy"]
CC = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
C_FLAGS = ["-std=c11", "-O2", "-Wall", "-fPIC"]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; librpl.so cannot be built")
    return exe


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    out = subprocess.run(cmd, capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("build step failed: %s\n%s%s" % (" ".join(cmd), out.stdout, out.stderr))
    if verbose and (out.stdout or out.stderr):
        print(out.stdout + out.stderr, flush=True)


def build(force=False, verbose=False, extra_nvcc=()):
    """Compile what is out of date and link ``librpl.so``.  Returns its path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    common = [os.path.join(CSRC, h) for h in HEADERS] + [os.path.join(INCLUDE, "rpl_b200.h"), os.path.abspath(__file__)]
    objs = []
    for src in CU_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src + ".o")
        if force or _stale(o, [s] + common):
            _run([_nvcc()] + NVCC_FLAGS + list(extra_nvcc) + ["-I", INCLUDE, "-I", CSRC, "-c", s, "-o", o], verbose)
        objs.append(o)
    for src in C_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src + ".o")
        if force or _stale(o, [s] + common):
            _run([CC] + C_FLAGS + ["-I", INCLUDE, "-c", s, "-o", o], verbose)
        objs.append(o)
    if force or _stale(LIB_PATH, objs):
        # The CUDA runtime is linked statically so the library stands alone.
        _run([_nvcc(), "-shared", "-o", LIB_PATH] + objs + ["-cudart", "static", "-Xlinker", "--no-undefined", "-lm", "-ldl"],
             verbose)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
