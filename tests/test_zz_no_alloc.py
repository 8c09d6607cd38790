"""rplb_minmax_f32_static: the min/max reduction for callers that are not
allowed to allocate device memory (a plugin inside an application that owns
the GPU's memory budget, a real-time loop that cannot afford cudaMalloc's
implicit synchronisation).  Its scratch is a fixed array inside the library
image, so the call allocates nothing.

The file sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch


def _params(lib_call, name, x):
    from rpl_b200 import capi
    out = torch.full((8,), float("nan"), dtype=torch.float32, device=x.device)
    capi.call(name, C.c_void_p(x.data_ptr()), x.numel(), C.c_void_p(out.data_ptr()),
              C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return out.cpu().numpy().view(np.uint32)


@pytest.mark.gpu
def test_static_scratch_minmax_matches_the_allocating_entry_point(cuda, lib):
    from rpl_b200 import capi
    g = torch.Generator(device=cuda)
    g.manual_seed(77)
    # Two calls in a row share the array: the second must not see the first one's leftovers.
    first = torch.randn(3_000_003, device=cuda, generator=g) * 3.0
    first[12345] = -50.0
    second = torch.randn(70_001, device=cuda, generator=g)[1:] * 0.05      # misaligned view, small values
    for x in (first, second):
        want = _params(capi.call, "rplb_minmax_f32", x)
        got = _params(capi.call, "rplb_minmax_f32_static", x)
        assert np.array_equal(got, want)                                    # all eight words, bit for bit
    # and once more in the opposite order, back to back without a sync in between
    a = torch.empty(8, dtype=torch.float32, device=cuda)
    b = torch.empty(8, dtype=torch.float32, device=cuda)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    capi.call("rplb_minmax_f32_static", C.c_void_p(second.data_ptr()), second.numel(), C.c_void_p(a.data_ptr()), st)
    capi.call("rplb_minmax_f32_static", C.c_void_p(first.data_ptr()), first.numel(), C.c_void_p(b.data_ptr()), st)
    torch.cuda.synchronize()
    assert np.array_equal(a.cpu().numpy().view(np.uint32), _params(capi.call, "rplb_minmax_f32", second))
    assert np.array_equal(b.cpu().numpy().view(np.uint32), _params(capi.call, "rplb_minmax_f32", first))
    assert float(b[0]) == -50.0


def test_static_scratch_minmax_rejects_oversized_input(lib):
    """The size check comes before anything touches a device."""
    rc = lib.rplb_minmax_f32_static(None, (1 << 30) + 1, None, None)
    assert rc == -3
    assert b"exceed the limit" in lib.rplb_last_error()
