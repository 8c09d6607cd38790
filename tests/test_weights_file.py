"""Quantized weights on disk: host-side round trip (no GPU needed) and the byte
layout, which follows the reference's checkpoint framing
(src/rpl_training.c:924-936) with an int8 payload and per-channel scales."""
import ctypes as C
import struct

import numpy as np
import pytest


def _tensor(capi, q, scales, keep):
    t = capi.PerChannelQuantizedTensor()
    zps = np.zeros(scales.size, np.int32)
    keep += [q, scales, zps]
    t.data, t.scales, t.zero_points = q.ctypes.data, scales.ctypes.data, zps.ctypes.data
    t.num_channels, t.channel_size, t.dims = q.shape[0], q.size // q.shape[0], q.ndim
    for i, s in enumerate(q.shape):
        t.shape[i] = s
    return t


def test_round_trip_and_layout(lib, port, tmp_path):
    from rpl_b200 import capi
    rng = np.random.default_rng(4)
    ws = [(rng.standard_normal(s) * 0.05).astype(np.float32) for s in ((128, 784), (10, 128), (4, 3, 5))]
    keep, tensors = [], []
    for w in ws:
        q, sc, _ = port.quantize_per_channel(w, w.shape[0])
        tensors.append(_tensor(capi, q, sc, keep))
    arr = (C.POINTER(capi.PerChannelQuantizedTensor) * 3)(*[C.pointer(t) for t in tensors])
    path = str(tmp_path / "weights.rplq8").encode()
    assert lib.quantized_weights_save(path, arr, 3) == 0

    raw = open(path, "rb").read()
    n, tag, metric = struct.unpack_from("<IIf", raw, 0)
    assert (n, tag, metric) == (3, 0x38544E49, 0.0) and raw[4:8] == b"INT8"
    dims, s0, s1, size = struct.unpack_from("<IIII", raw, 12)
    assert (dims, s0, s1, size) == (2, 128, 784, 128 * 784)
    assert np.array_equal(np.frombuffer(raw, np.int8, size, 28), keep[0].ravel())
    nch = struct.unpack_from("<I", raw, 28 + size)[0]
    assert nch == 128 and np.array_equal(np.frombuffer(raw, np.float32, 128, 32 + size), keep[1])

    count = C.c_uint32()
    got = lib.quantized_weights_load(path, C.byref(count), False)
    assert got and count.value == 3
    for i, w in enumerate(ws):
        t = got[i].contents
        assert t.dims == w.ndim and list(t.shape[:w.ndim]) == list(w.shape)
        assert t.num_channels == w.shape[0] and t.channel_size == w.size // w.shape[0]
        q = np.ctypeslib.as_array(C.cast(t.data, C.POINTER(C.c_int8)), shape=(w.size,))
        sc = np.ctypeslib.as_array(C.cast(t.scales, C.POINTER(C.c_float)), shape=(w.shape[0],))
        zp = np.ctypeslib.as_array(C.cast(t.zero_points, C.POINTER(C.c_int32)), shape=(w.shape[0],))
        assert np.array_equal(q, keep[3 * i].ravel()) and np.array_equal(sc, keep[3 * i + 1]) and not zp.any()
        lib.per_channel_quantized_tensor_free(got[i])
    lib.rpitorch_aligned_free(C.cast(got, C.c_void_p))


def test_load_rejects_foreign_and_truncated_files(lib, tmp_path):
    count = C.c_uint32(77)
    p = tmp_path / "fp32.ckpt"
    p.write_bytes(struct.pack("<IIf", 1, 5, 0.25) + b"\0" * 64)          # the reference's fp32 framing: epoch 5
    assert not lib.quantized_weights_load(str(p).encode(), C.byref(count), False) and count.value == 77
    p = tmp_path / "short.rplq8"
    p.write_bytes(struct.pack("<IIf", 1, 0x38544E49, 0.0) + struct.pack("<IIII", 2, 4, 4, 16) + b"\1" * 7)
    assert not lib.quantized_weights_load(str(p).encode(), C.byref(count), False)
    assert not lib.quantized_weights_load(b"/nonexistent/file", C.byref(count), False)


@pytest.mark.gpu
def test_device_resident_weights_round_trip(lib, port, cuda, tmp_path):
    import torch
    from rpl_b200 import capi, device as D
    w = torch.randn((256, 512), device=cuda) * 0.02
    q, sc, zp = D.quantize_per_channel(w)
    t = capi.PerChannelQuantizedTensor()
    t.data, t.scales, t.zero_points = q.data_ptr(), sc.data_ptr(), zp.data_ptr()
    t.num_channels, t.channel_size, t.dims = 256, 512, 2
    t.shape[0], t.shape[1] = 256, 512
    arr = (C.POINTER(capi.PerChannelQuantizedTensor) * 1)(C.pointer(t))
    path = str(tmp_path / "dev.rplq8").encode()
    assert lib.quantized_weights_save(path, arr, 1) == 0
    count = C.c_uint32()
    got = lib.quantized_weights_load(path, C.byref(count), True)
    assert got and count.value == 1 and lib.rplb_pointer_kind(got[0].contents.data) == 2
    back = torch.empty_like(q)
    capi.call("rplb_copy", C.c_void_p(back.data_ptr()), C.c_void_p(got[0].contents.data), q.numel(), None)
    bs = torch.empty_like(sc)
    capi.call("rplb_copy", C.c_void_p(bs.data_ptr()), C.c_void_p(got[0].contents.scales), sc.numel() * 4, None)
    capi.call("rplb_stream_sync", None)
    assert torch.equal(back, q) and torch.equal(bs, sc)
    lib.per_channel_quantized_tensor_free(got[0])
    lib.rpitorch_aligned_free(C.cast(got, C.c_void_p))
