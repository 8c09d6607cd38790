"""The C-ABI library on a machine without a GPU: it loads, exports every
function include/rpl_b200.h declares, keeps the reference's struct layouts,
and refuses to compute (no CPU fallback)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from conftest import ROOT


def declared_functions():
    text = open(os.path.join(ROOT, "include", "rpl_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
    text = re.sub(r"typedef\s+struct\s*\w*\s*\{.*?\}\s*\w+\s*;", "", text, flags=re.S)
    text = re.sub(r"typedef\s+enum\s*\{.*?\}\s*\w+\s*;", "", text, flags=re.S)
    text = re.sub(r"typedef\s+[^;{}]*\(\s*\*\s*\w+\s*\)\s*\([^;{}]*\)\s*;", "", text)       # function-pointer types
    names = re.findall(r"\b([A-Za-z_]\w*)\s*\([^;{}]*\)\s*;", text)
    return sorted(set(names))


def test_header_parse_finds_the_api():
    names = declared_functions()
    for must in ("tensor_quantize_int8", "gemm_int8", "linear_int8", "tensor_dequantize_int8",
                 "tensor_quantize_per_channel", "rplb_linear_i8_dequant_f32", "rplb_minmax_f32"):
        assert must in names
    assert len(names) >= 50


def test_library_exports_every_declared_symbol(lib):
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_covers_every_declared_symbol():
    from rpl_b200 import capi
    assert sorted(capi.SIGNATURES) == declared_functions()


def test_struct_layouts_match_reference():
    from rpl_b200 import capi
    T, Q = capi.Tensor, capi.QuantizedTensor
    assert C.sizeof(T) == 152
    assert (T.size.offset, T._allocation.offset, T.device.offset, T.gpu_buffer.offset) == (84, 96, 112, 116)
    assert (T.is_leaf.offset, T.parent1.offset, T.backward_fn.offset) == (120, 128, 144)
    assert C.sizeof(Q) == 56 and (Q.scale.offset, Q.zero_point.offset, Q.size.offset, Q.dims.offset, Q.shape.offset) == (8, 12, 16, 20, 24)
    assert C.sizeof(capi.QParams) == 32
    assert C.sizeof(capi.PerChannelQuantizedTensor) == 72
    # the oracle's view of the reference structs agrees
    from oracle import loader
    assert C.sizeof(loader.RefTensor) == 152 and C.sizeof(loader.RefQuantizedTensor) == 56
    assert C.sizeof(loader.RefPerChannel) == 72


@pytest.mark.parametrize("n,world,align", [(65536, 8, 256), (65536, 1, 256), (10, 4, 1), (1000, 3, 256), (0, 2, 16), (12288, 8, 256)])
def test_shard_range_partitions_columns(lib, n, world, align):
    covered = 0
    for r in range(world):
        b, c = C.c_uint64(), C.c_uint64()
        assert lib.rplb_shard_range(n, world, r, align, C.byref(b), C.byref(c)) == 0
        assert b.value == covered                     # contiguous, in rank order
        if c.value and b.value + c.value < n:
            assert c.value % align == 0               # only the last block may be ragged
        covered += c.value
    assert covered == n
    from rpl_b200.sharded import shard_range
    assert [shard_range(n, world, r, align) for r in range(world)] == \
        [_c_range(lib, n, world, r, align) for r in range(world)]


def _c_range(lib, n, world, r, align):
    b, c = C.c_uint64(), C.c_uint64()
    lib.rplb_shard_range(n, world, r, align, C.byref(b), C.byref(c))
    return (b.value, c.value)


def test_shard_range_rejects_bad_rank(lib):
    b, c = C.c_uint64(), C.c_uint64()
    assert lib.rplb_shard_range(10, 2, 2, 1, C.byref(b), C.byref(c)) != 0
    assert b"rank" in lib.rplb_last_error()


def test_host_allocation_glue(lib):
    shape = (C.c_uint32 * 2)(3, 5)
    t = lib.tensor_create(2, shape, True)
    assert t and t.contents.size == 15 and t.contents.dims == 2
    assert list(t.contents.strides[:2]) == [5, 1]
    assert t.contents.data % 64 == 0 and t.contents.grad
    assert t.contents.is_leaf and t.contents.requires_grad
    lib.tensor_free(t)
    p = lib.rpitorch_aligned_alloc(64, 100)
    assert p and p % 64 == 0
    lib.rpitorch_aligned_free(p)
    cal = lib.calibrator_create()
    assert cal.contents.min_val > 3e38 and cal.contents.max_val < -3e38
    cal.contents.min_val, cal.contents.max_val = -2.0, 6.35
    lib.calibrator_compute_params(cal, True)
    assert cal.contents.scale == np.float32(6.35) / np.float32(127.0) and cal.contents.zero_point == 0
    lib.calibrator_compute_params(cal, False)
    assert cal.contents.scale == (np.float32(6.35) - np.float32(-2.0)) / np.float32(255.0)
    assert cal.contents.zero_point == int(np.round(np.float32(2.0) / np.float32(cal.contents.scale)))
    lib.calibrator_free(cal)


def test_no_cpu_fallback_without_a_device(lib):
    """Without a CUDA device the compute entry points must fail, not compute."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    assert lib.rplb_device_count() == 0
    x = np.ones(16, np.float32)
    q = np.zeros(16, np.int8)
    rc = lib.rplb_quantize_f32_i8(x.ctypes.data, q.ctypes.data, 16, 1.0, 0, None)
    assert rc != 0 and (q == 0).all()
    from rpl_b200 import capi
    shape = (C.c_uint32 * 1)(16)
    t = lib.tensor_create(1, shape, False)
    C.memmove(t.contents.data, x.ctypes.data, 64)
    assert not lib.tensor_quantize_int8(t, 1.0, 0)          # NULL, error on stderr
    assert lib.rpl_cuda_last_error() != 0
    lib.tensor_free(t)
    with pytest.raises(capi.RplError):
        capi.call("rplb_stream_sync", None)


@pytest.mark.parametrize("n,weights", [(65536, [1.0] * 8), (65536, [1 / 3.26, 1 / 3.85, 1 / 3.4, 1 / 3.5, 1 / 3.85, 1 / 3.3, 1 / 3.6, 1 / 3.45]),
                                       (700, [1, 2]), (200, [1, 5]), (1000, [3, 1, 1]), (12288, [1, 1.1, 0.9, 1])])
def test_weighted_shard_covers_the_columns_in_units_of_256(lib, n, weights):
    world = len(weights)
    w = (C.c_double * world)(*weights)
    counts = (C.c_uint64 * world)()
    assert lib.rplb_shard_weighted(n, world, 256, w, counts) == 0
    got = [int(c) for c in counts]
    assert sum(got) == n
    at = 0
    for c in got:
        if c and at + c < n:
            assert c % 256 == 0                               # only the block that ends the matrix may be ragged
        at += c
    units = (n + 255) // 256
    for c, wt in zip(got, weights):                           # within one unit of the exact proportional share
        assert abs((c + 255) // 256 - units * wt / sum(weights)) <= 1.0 + 1e-9
    if len(set(weights)) == 1:
        from rpl_b200.sharded import shard_range
        assert got == [shard_range(n, world, r, 256)[1] for r in range(world)]
    assert lib.rplb_shard_weighted(n, world, 256, (C.c_double * world)(*([0.0] * world)), counts) != 0
