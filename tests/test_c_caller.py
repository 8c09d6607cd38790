"""A C program written against the reference's API (tests/c/drop_in_check.c),
compiled with gcc and linked against librpl.so: with the reference's own
include/rpl.h when that tree is present, and with include/rpl_b200.h."""
import os
import subprocess

import pytest

from conftest import ROOT

# The reference tree: RPL_REFERENCE, or a checkout named "reference" beside this repository.
REF_INCLUDE = os.path.join(os.environ.get("RPL_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference"), "include")
SRC = os.path.join(ROOT, "tests", "c", "drop_in_check.c")


def _build(tmp_path, lib, use_reference_header):
    from rpl_b200 import capi
    exe = str(tmp_path / ("dic_ref" if use_reference_header else "dic"))
    libdir = os.path.dirname(capi.LIB_PATH)
    cmd = ["/usr/bin/gcc", "-std=c11", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include")]
    if use_reference_header:
        cmd += ["-DUSE_REFERENCE_HEADER", "-I", REF_INCLUDE]
    cmd += [SRC, "-o", exe, "-L", libdir, "-lrpl", "-lm", "-Wl,-rpath," + libdir]
    out = subprocess.run(cmd, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    return exe


def _headers():
    hs = [False]
    if os.path.exists(os.path.join(REF_INCLUDE, "rpl.h")):
        hs.append(True)
    return hs


@pytest.mark.parametrize("use_reference_header", _headers())
def test_c_caller_compiles_and_links(tmp_path, lib, use_reference_header):
    """Both headers give a program that links; without a GPU it reports so and stops."""
    import torch
    exe = _build(tmp_path, lib, use_reference_header)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    if torch.cuda.is_available():
        assert out.returncode == 0, out.stdout + out.stderr
    else:
        assert out.returncode == 2 and "no CUDA device" in out.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("use_reference_header", _headers())
def test_c_caller_results_match_plain_c_loops(tmp_path, lib, cuda, use_reference_header):
    exe = _build(tmp_path, lib, use_reference_header)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "drop_in_check: OK" in out.stdout, out.stdout + out.stderr


@pytest.mark.skipif(not os.path.exists(os.path.join(os.path.dirname(REF_INCLUDE), "src", "rpl_nn.c")),
                    reason="reference tree absent")
def test_combined_library_keeps_the_rest_of_the_reference(tmp_path, lib):
    """The combined-library linking recipe: the reference's own objects (its INT8
    symbols weakened) next to this library's objects give one library in which the
    fp32 layers are the reference's and the INT8 path is this one."""
    import ctypes as C
    import glob
    from rpl_b200 import build
    ref = os.path.dirname(REF_INCLUDE)
    objs = []
    for src in sorted(glob.glob(os.path.join(ref, "src", "*.c"))):
        name = os.path.basename(src)[:-2]
        if name == "rpi_ml":                      # not part of the reference's own build
            continue
        o = str(tmp_path / (name + ".o"))
        subprocess.run(["/usr/bin/gcc", "-O1", "-fopenmp", "-fPIC", "-w", "-I", REF_INCLUDE, "-c", src, "-o", o], check=True)
        if name in ("rpl_core", "ops_extended", "rpl_quantization", "rpl_gpu"):
            subprocess.run(["objcopy", "--weaken", o], check=True)
        objs.append(o)
    ours = sorted(glob.glob(os.path.join(build.OBJ_DIR, "*.o")))
    out = str(tmp_path / "librpl_full.so")
    subprocess.run([build._nvcc(), "-shared", "-o", out] + objs + ours + ["-cudart", "static", "-Xcompiler", "-fopenmp", "-lm"],
                   check=True, capture_output=True)
    L = C.CDLL(out)
    for name in ("tensor_gemm", "linear_forward", "optimizer_adam_create", "rplb_minmax_f32", "quantized_linear_forward", "tensor_to_gpu"):
        assert hasattr(L, name), name
    # the INT8 entry point is this library's: it can report a CUDA error code
    L.rpl_cuda_last_error.restype = C.c_int
    assert L.rpl_cuda_last_error() == 0
