"""A C program written against the reference's API (tests/c/drop_in_check.c),
compiled with gcc and linked against librpl.so: with the reference's own
include/rpl.h when that tree is present, and with include/rpl_b200.h."""
import os
import subprocess

import pytest

from conftest import ROOT

REF_INCLUDE = os.path.join(os.environ.get("RPL_REFERENCE", "/root/reference"), "include")
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
