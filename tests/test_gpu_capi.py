"""The reference-named C API (tensor_quantize_int8, gemm_int8, linear_int8 ...)
called through ctypes the way a C program would, with host buffers and with
device buffers, against the CPU checker."""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import bits

pytestmark = pytest.mark.gpu


def same(a, b):
    return np.array_equal(bits(np.asarray(a)), bits(np.asarray(b)))


def host_tensor(lib, x):
    """A library-owned host Tensor holding a copy of x."""
    shape = (C.c_uint32 * x.ndim)(*x.shape)
    t = lib.tensor_create(x.ndim, shape, False)
    C.memmove(t.contents.data, np.ascontiguousarray(x).ctypes.data, x.nbytes)
    return t


def read_host(ptr, shape, dtype):
    n = int(np.prod(shape))
    buf = (C.c_char * (n * np.dtype(dtype).itemsize)).from_address(ptr)
    return np.frombuffer(buf, dtype=dtype, count=n).reshape(shape).copy()


def qt_view(capi, q, scale=1.0, zp=0):
    t = capi.QuantizedTensor()
    t.data = q.ctypes.data if isinstance(q, np.ndarray) else q.data_ptr()
    t.scale, t.zero_point, t.size, t.dims = scale, zp, int(np.prod(q.shape)), len(q.shape)
    for i, s in enumerate(q.shape):
        t.shape[i] = s
    return t


def test_quantize_dequantize_host_buffers(cuda, lib, port):
    rng = np.random.default_rng(21)
    x = (rng.standard_normal((33, 257)) * 3).astype(np.float32)
    t = host_tensor(lib, x)
    qt = lib.tensor_quantize_int8(t, 0.05, 3)
    assert qt and qt.contents.size == x.size and qt.contents.dims == 2 and list(qt.contents.shape[:2]) == [33, 257]
    assert qt.contents.data % 64 == 0 and lib.rplb_pointer_kind(qt.contents.data) == 0
    assert same(read_host(qt.contents.data, x.shape, np.int8), port.quantize(x, 0.05, 3))
    back = lib.tensor_dequantize_int8(qt)
    assert same(read_host(back.contents.data, x.shape, np.float32), port.dequantize(port.quantize(x, 0.05, 3), 0.05, 3))
    lib.tensor_free(back)
    lib.quantized_tensor_free(qt)

    qs = lib.tensor_quantize_int8_symmetric(t)
    wq, ws = port.quantize_symmetric(x)
    assert same(np.float32(qs.contents.scale), ws) and qs.contents.zero_point == 0
    assert same(read_host(qs.contents.data, x.shape, np.int8), wq)
    lib.quantized_tensor_free(qs)

    qa = lib.tensor_quantize_int8_asymmetric(t)
    wq, ws, wz = port.quantize_asymmetric(x)
    assert same(np.float32(qa.contents.scale), ws) and qa.contents.zero_point == wz
    assert same(read_host(qa.contents.data, x.shape, np.int8), wq)
    lib.quantized_tensor_free(qa)

    mn, mx = C.c_float(), C.c_float()
    lib.tensor_get_min_max(t, C.byref(mn), C.byref(mx))
    assert (np.float32(mn.value), np.float32(mx.value)) == port.minmax_serial(x)

    pc = lib.tensor_quantize_per_channel(t, 0)
    wq, wsc, wzp = port.quantize_per_channel(x, 33)
    assert pc.contents.num_channels == 33 and pc.contents.channel_size == 257
    assert same(read_host(pc.contents.data, x.shape, np.int8), wq)
    assert same(read_host(pc.contents.scales, (33,), np.float32), wsc)
    assert same(read_host(pc.contents.zero_points, (33,), np.int32), wzp)
    dq = lib.tensor_dequantize_per_channel(pc)
    assert same(read_host(dq.contents.data, x.shape, np.float32), port.dequantize_per_channel(wq, wsc))
    lib.tensor_free(dq)
    lib.per_channel_quantized_tensor_free(pc)
    assert lib.rpl_cuda_last_error() == 0
    lib.tensor_free(t)


def test_min_max_edge_cases(cuda, lib, port):
    mn, mx = C.c_float(123.0), C.c_float(456.0)
    empty = host_tensor(lib, np.zeros((0,), np.float32))
    lib.tensor_get_min_max(empty, C.byref(mn), C.byref(mx))
    assert (mn.value, mx.value) == (123.0, 456.0)            # untouched for size 0
    lib.tensor_free(empty)
    t = host_tensor(lib, np.array([np.nan, 1.0, -2.0], np.float32))
    lib.tensor_get_min_max(t, C.byref(mn), C.byref(mx))
    assert np.isnan(mn.value) and np.isnan(mx.value)         # seeded with a NaN first element
    lib.tensor_free(t)
    t = host_tensor(lib, np.array([1.0, np.nan, -2.0, 7.5], np.float32))
    lib.tensor_get_min_max(t, C.byref(mn), C.byref(mx))
    assert (mn.value, mx.value) == (-2.0, 7.5)
    lib.tensor_free(t)


def test_device_resident_tensors_stay_on_device(cuda, lib, port):
    rng = np.random.default_rng(22)
    x = (rng.standard_normal((16, 4096)) * 3).astype(np.float32)
    h = host_tensor(lib, x)
    d = lib.tensor_upload(h)
    assert d and d.contents.device == 1 and lib.rplb_pointer_kind(d.contents.data) == 2
    qt = lib.tensor_quantize_int8_symmetric(d)
    assert lib.rplb_pointer_kind(qt.contents.data) == 2
    wq, ws = port.quantize_symmetric(x)
    assert same(np.float32(qt.contents.scale), ws)
    back = lib.tensor_dequantize_int8(qt)
    assert back.contents.device == 1
    hb = lib.tensor_download(back)
    assert same(read_host(hb.contents.data, x.shape, np.float32), port.dequantize(wq, ws, 0))
    for t in (hb, back, d, h):
        lib.tensor_free(t)
    lib.quantized_tensor_free(qt)


@pytest.mark.parametrize("mnk", [(128, 128, 128), (33, 19, 77), (300, 520, 784)])
def test_gemm_int8_and_linear_int8_host_buffers(cuda, lib, port, mnk):
    from rpl_b200 import capi
    M, N, K = mnk
    rng = np.random.default_rng(M + N)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    W = rng.integers(-128, 128, (N, K), dtype=np.int8)
    B = np.ascontiguousarray(W.T)
    b = rng.integers(-128, 128, N, dtype=np.int8)
    out = np.zeros((M, N), np.int32)
    for fn in (lib.gemm_int8, lib.gemm_int8_fallback):
        fn(A.ctypes.data, B.ctypes.data, out.ctypes.data, M, N, K, 0.01, 0.01, 0.01, 0, 0)
        assert same(out, port.gemm_requant(A, B, 0.01, 0.01, 0.01))
    lib.gemm_int8(A.ctypes.data, B.ctypes.data, out.ctypes.data, M, N, K, 0.013, 0.021, 0.37, 3, -7)
    assert same(out, port.gemm_requant(A, B, 0.013, 0.021, 0.37, 3, -7))
    qa, qw, qb = qt_view(capi, A), qt_view(capi, W), qt_view(capi, b)
    lib.linear_int8(C.byref(qa), C.byref(qw), None, out.ctypes.data, M, K, N)
    assert same(out, port.linear(A, W))
    lib.linear_int8(C.byref(qa), C.byref(qw), C.byref(qb), out.ctypes.data, M, K, N)
    assert same(out, port.linear(A, W, b))
    assert lib.rpl_cuda_last_error() == 0


def test_linear_int8_dequant_mixed_residency(cuda, lib, port):
    """Weights resident on the device, activations and output in host memory."""
    from rpl_b200 import capi
    M, N, K = 200, 128, 784
    rng = np.random.default_rng(5)
    x = rng.random((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.05).astype(np.float32)
    wq, wsc, _ = port.quantize_per_channel(w, N)
    xq, xs = port.quantize_symmetric(x)
    wq_dev = torch.from_numpy(wq).to(cuda)
    pc = capi.PerChannelQuantizedTensor()
    pc.data, pc.scales = wq_dev.data_ptr(), wsc.ctypes.data
    pc.num_channels, pc.channel_size, pc.dims = N, K, 2
    qx = qt_view(capi, xq, float(xs))
    out = np.zeros((M, N), np.float32)
    lib.linear_int8_dequant(C.byref(qx), C.byref(pc), bias.ctypes.data, out.ctypes.data, M, K, N, True)
    assert same(out, port.linear_dequant(xq, wq, xs, wsc, bias, True))
    assert lib.rpl_cuda_last_error() == 0


def test_calibrator_and_model_quantize(cuda, lib, port):
    from rpl_b200 import capi
    rng = np.random.default_rng(8)
    batches = [(rng.standard_normal((64, 100)) * s).astype(np.float32) for s in (1.0, 4.0, 0.5)]
    cal = lib.calibrator_create()
    for b in batches:
        t = host_tensor(lib, b)
        lib.calibrator_update(cal, t)
        lib.tensor_free(t)
    allx = np.concatenate([b.ravel() for b in batches])
    assert cal.contents.num_samples == 3
    assert (np.float32(cal.contents.min_val), np.float32(cal.contents.max_val)) == port.minmax_seeded(allx)
    lib.calibrator_compute_params(cal, True)
    assert same(np.float32(cal.contents.scale), port.scale_symmetric(*port.minmax_seeded(allx)))
    lib.calibrator_compute_params(cal, False)
    s, z = port.params_asymmetric(*port.minmax_seeded(allx))
    assert same(np.float32(cal.contents.scale), s) and cal.contents.zero_point == z
    lib.calibrator_free(cal)

    params = [host_tensor(lib, b) for b in batches]
    arr = (C.POINTER(capi.Tensor) * 3)(*params)
    qm = lib.model_quantize(arr, 3, True)
    assert qm.contents.num_params == 3 and qm.contents.is_quantized
    for i, b in enumerate(batches):
        q = qm.contents.int8_params[i].contents
        wq, ws = port.quantize_symmetric(b)
        assert same(np.float32(q.scale), ws) and same(read_host(q.data, b.shape, np.int8), wq)
    lib.quantized_model_free(qm)
    r = host_tensor(lib, np.array([-1.0, 0.5, -0.0, 3.0], np.float32))
    lib.tensor_relu_inplace(r)
    assert same(read_host(r.contents.data, (4,), np.float32), port.relu(np.array([-1.0, 0.5, -0.0, 3.0], np.float32)))
    for t in params + [r]:
        lib.tensor_free(t)


def test_quantized_linear_layers_chain_like_the_mlp(cuda, lib, port):
    """quantized_linear_create / _forward (the INT8 counterpart of linear_create /
    linear_forward): a 784 -> 128 -> 10 MLP on host tensors and on device tensors."""
    rng = np.random.default_rng(31)
    X = rng.random((300, 784), dtype=np.float32)
    W1 = (rng.standard_normal((128, 784)) * 0.05).astype(np.float32)
    W2 = (rng.standard_normal((10, 128)) * 0.05).astype(np.float32)
    b1 = (rng.standard_normal(128) * 0.05).astype(np.float32)
    tw1, tw2, tb1, tx = (host_tensor(lib, a) for a in (W1, W2, b1, X))
    l1 = lib.quantized_linear_create(tw1, tb1)
    l2 = lib.quantized_linear_create(tw2, None)
    assert l1 and l2

    w1q, w1s, _ = port.quantize_per_channel(W1, 128)
    w2q, w2s, _ = port.quantize_per_channel(W2, 10)
    xq, xs = port.quantize_symmetric(X)
    h_want = port.linear_dequant(xq, w1q, xs, w1s, b1, relu=True)
    hq, hs = port.quantize_symmetric(h_want)
    y_want = port.linear_dequant(hq, w2q, hs, w2s, None, relu=False)

    h = lib.quantized_linear_forward(l1, tx, True)
    assert h and list(h.contents.shape[:2]) == [300, 128] and lib.rplb_pointer_kind(h.contents.data) == 0
    assert same(read_host(h.contents.data, (300, 128), np.float32), h_want)
    y = lib.quantized_linear_forward(l2, h, False)
    assert same(read_host(y.contents.data, (300, 10), np.float32), y_want)

    xd = lib.tensor_upload(tx)                         # same chain with device-resident activations
    hd = lib.quantized_linear_forward(l1, xd, True)
    yd = lib.quantized_linear_forward(l2, hd, False)
    assert yd.contents.device == 1 and lib.rplb_pointer_kind(yd.contents.data) == 2
    yh = lib.tensor_download(yd)
    assert same(read_host(yh.contents.data, (300, 10), np.float32), y_want)
    assert lib.rpl_cuda_last_error() == 0
    for t in (h, y, xd, hd, yd, yh, tw1, tw2, tb1, tx):
        lib.tensor_free(t)
    lib.quantized_linear_free(l1)
    lib.quantized_linear_free(l2)


def test_quantized_linear_host_pipeline(cuda, lib, port):
    """quantized_linear_submit_host / _drain: several calls in flight on page-locked
    host buffers, double-buffered on the device, each equal to the checker's result."""
    rng = np.random.default_rng(41)
    M, K, N = 1000, 256, 384
    W = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.05).astype(np.float32)
    tw, tb = host_tensor(lib, W), host_tensor(lib, bias)
    layer = lib.quantized_linear_create(tw, tb)
    wq, ws, _ = port.quantize_per_channel(W, N)
    xs = [torch.from_numpy((rng.standard_normal((M, K)) * (i + 1)).astype(np.float32)).pin_memory() for i in range(5)]
    outs = [torch.empty((M, N), dtype=torch.float32).pin_memory() for _ in xs]
    for x, o in zip(xs, outs):
        assert lib.quantized_linear_submit_host(layer, x.data_ptr(), M, o.data_ptr(), True, None) == 0
    assert lib.quantized_linear_drain(layer) == 0
    for x, o in zip(xs, outs):
        xq, s = port.quantize_symmetric(x.numpy())
        assert same(o.numpy(), port.linear_dequant(xq, wq, s, ws, bias, relu=True))
    # a different row count afterwards (buffers grow), then the blocking call on the same layer
    x2 = torch.from_numpy(rng.standard_normal((2 * M + 7, K)).astype(np.float32)).pin_memory()
    o2 = torch.empty((2 * M + 7, N), dtype=torch.float32).pin_memory()
    assert lib.quantized_linear_submit_host(layer, x2.data_ptr(), 2 * M + 7, o2.data_ptr(), False, None) == 0
    assert lib.quantized_linear_drain(layer) == 0
    xq, s = port.quantize_symmetric(x2.numpy())
    assert same(o2.numpy(), port.linear_dequant(xq, wq, s, ws, bias, relu=False))
    t = host_tensor(lib, xs[0].numpy())
    y = lib.quantized_linear_forward(layer, t, True)
    assert same(read_host(y.contents.data, (M, N), np.float32), outs[0].numpy())
    for p in (t, y, tw, tb):
        lib.tensor_free(p)
    lib.quantized_linear_free(layer)
    assert lib.rpl_cuda_last_error() == 0


def test_tensor_to_gpu_mirrors(cuda, lib, port):
    """The reference's accelerator hooks (include/rpl.h:105-108) on CUDA: a mirrored
    tensor keeps its host block, the INT8 calls read the mirror and answer in device
    memory, tensor_from_gpu brings the mirror back."""
    assert lib.rpl_gpu_init()
    rng = np.random.default_rng(43)
    x = (rng.standard_normal((24, 1024)) * 2).astype(np.float32)
    t = host_tensor(lib, x)
    host_block = t.contents.data
    lib.tensor_to_gpu(t)
    assert t.contents.device == 1 and t.contents.gpu_buffer != 0 and t.contents.data == host_block
    handle = t.contents.gpu_buffer
    lib.tensor_to_gpu(t)                                   # a second call changes nothing
    assert t.contents.gpu_buffer == handle

    # The mirror is what is read: change the host block, results still follow x.
    C.memset(host_block, 0, x.nbytes)
    qs = lib.tensor_quantize_int8_symmetric(t)
    wq, ws = port.quantize_symmetric(x)
    assert lib.rplb_pointer_kind(qs.contents.data) == 2 and same(np.float32(qs.contents.scale), ws)
    back = lib.tensor_dequantize_int8(qs)
    hb = lib.tensor_download(back)
    assert same(read_host(hb.contents.data, x.shape, np.float32), port.dequantize(wq, ws, 0))
    mn, mx = C.c_float(), C.c_float()
    lib.tensor_get_min_max(t, C.byref(mn), C.byref(mx))
    assert (np.float32(mn.value), np.float32(mx.value)) == port.minmax_serial(x)
    pc = lib.tensor_quantize_per_channel(t, 0)
    assert lib.rplb_pointer_kind(pc.contents.data) == 2
    lib.per_channel_quantized_tensor_free(pc)

    # In-place ReLU works on the mirror; tensor_from_gpu fills the host block with it.
    lib.tensor_relu_inplace(t)
    assert not read_host(host_block, x.shape, np.float32).any()
    lib.tensor_from_gpu(t)
    assert same(read_host(host_block, x.shape, np.float32), np.where(x < 0, np.float32(0), x))
    assert t.contents.device == 1 and t.contents.gpu_buffer == handle

    # Handles are distinct per tensor and reusable after tensor_free.
    u = host_tensor(lib, x[:2])
    lib.tensor_to_gpu(u)
    assert u.contents.gpu_buffer not in (0, handle)
    for p in (u, t, hb, back):
        lib.tensor_free(p)
    lib.quantized_tensor_free(qs)
    v = host_tensor(lib, x[:3])
    lib.tensor_to_gpu(v)
    lib.tensor_from_gpu(v)
    assert same(read_host(v.contents.data, (3, 1024), np.float32), x[:3])
    lib.tensor_free(v)
    lib.rpl_gpu_shutdown()
    assert lib.rpl_cuda_last_error() == 0


def test_shared_input_forward_like_attention_projections(cuda, lib, port):
    """quantized_linear_forward_shared_input: Q, K and V projections of one activation
    (src/rpl_attention.c:175-177), the activation quantized once; host and device inputs."""
    rng = np.random.default_rng(47)
    M, K = 200, 256
    widths = (256, 128, 384)
    x = rng.standard_normal((M, K)).astype(np.float32)
    Ws = [(rng.standard_normal((n, K)) * 0.05).astype(np.float32) for n in widths]
    bs = [(rng.standard_normal(n) * 0.05).astype(np.float32) for n in widths]
    tws, tbs = [host_tensor(lib, w) for w in Ws], [host_tensor(lib, b) for b in bs]
    layers = [lib.quantized_linear_create(tw, tb) for tw, tb in zip(tws, tbs)]
    assert all(layers)
    arr = (C.c_void_p * 3)(*layers)
    xq, s = port.quantize_symmetric(x)
    wants = []
    for w, b in zip(Ws, bs):
        wq, ws, _ = port.quantize_per_channel(w, w.shape[0])
        wants.append(port.linear_dequant(xq, wq, s, ws, b, relu=False))

    th = host_tensor(lib, x)
    outs = (C.POINTER(type(th.contents)) * 3)()
    assert lib.quantized_linear_forward_shared_input(arr, 3, th, outs, False) == 0
    for o, want, n in zip(outs, wants, widths):
        assert o.contents.device == 0 and list(o.contents.shape[:2]) == [M, n]
        assert same(read_host(o.contents.data, (M, n), np.float32), want)
        lib.tensor_free(o)

    td = lib.tensor_upload(th)
    outs = (C.POINTER(type(th.contents)) * 3)()
    assert lib.quantized_linear_forward_shared_input(arr, 3, td, outs, False) == 0
    for o, want, n, layer in zip(outs, wants, widths, layers):
        assert o.contents.device == 1
        h = lib.tensor_download(o)
        assert same(read_host(h.contents.data, (M, n), np.float32), want)
        single = lib.quantized_linear_forward(layer, td, False)            # the one-layer call gives the same bits
        hs = lib.tensor_download(single)
        assert same(read_host(hs.contents.data, (M, n), np.float32), want)
        for t in (o, h, single, hs):
            lib.tensor_free(t)

    # layers that do not share in_features are refused and nothing is returned
    odd = host_tensor(lib, Ws[0][:, :128].copy())
    lo = lib.quantized_linear_create(odd, None)
    bad = (C.c_void_p * 2)(layers[0], lo)
    outs2 = (C.POINTER(type(th.contents)) * 2)()
    assert lib.quantized_linear_forward_shared_input(bad, 2, th, outs2, False) != 0 and not outs2[0] and not outs2[1]
    lib.quantized_linear_free(lo)
    for l in layers:
        lib.quantized_linear_free(l)
    for t in tws + tbs + [th, td, odd]:
        lib.tensor_free(t)
    assert lib.rpl_cuda_last_error() == 0


def test_model_quantize_per_channel(cuda, lib, port):
    """The per-channel model quantizer the reference announces and leaves undone
    (src/rpl_quantization.c:286-292): weights per row of shape[0], biases with one scale."""
    from rpl_b200 import capi
    rng = np.random.default_rng(12)
    shapes = [(128, 784), (128,), (10, 128), (10,), (4, 3, 8)]
    arrays = [(rng.standard_normal(s) * 0.05).astype(np.float32) for s in shapes]
    params = [host_tensor(lib, a) for a in arrays]
    arr = (C.POINTER(capi.Tensor) * len(params))(*params)
    qm = C.cast(lib.model_quantize_per_channel(arr, len(params)), C.POINTER(capi.PerChannelQuantizedModel))
    assert qm and qm.contents.num_params == len(params) and qm.contents.is_quantized
    for i, a in enumerate(arrays):
        q = qm.contents.int8_params[i].contents
        assert q.dims == a.ndim and list(q.shape[:a.ndim]) == list(a.shape)
        if a.ndim >= 2:
            wq, ws, _ = port.quantize_per_channel(a, a.shape[0])
            assert q.num_channels == a.shape[0] and q.channel_size == a.size // a.shape[0]
        else:
            wq, s1 = port.quantize_symmetric(a)             # one scale for the whole tensor
            ws = np.array([s1], np.float32)
            assert q.num_channels == 1 and q.channel_size == a.size
        assert same(read_host(q.data, a.shape, np.int8), wq)
        assert same(read_host(q.scales, (q.num_channels,), np.float32), ws)
        assert not read_host(q.zero_points, (q.num_channels,), np.int32).any()
    lib.per_channel_quantized_model_free(qm)
    # the original entry point keeps ignoring its flag, as the reference does
    qm2 = lib.model_quantize(arr, len(params), True)
    wq, ws = port.quantize_symmetric(arrays[0])
    assert same(np.float32(qm2.contents.int8_params[0].contents.scale), ws)
    lib.quantized_model_free(qm2)
    for t in params:
        lib.tensor_free(t)


def test_a_give_up_is_reported_to_the_thread_that_launched_it(cuda, lib, port):
    """Two host threads: one provokes the bounded-wait give-up and leaves its code in place;
    the other sees a clear status and runs a tensor-core GEMM; the first then finds its code."""
    import threading
    from rpl_b200 import device as D
    rng = np.random.default_rng(2)
    A = rng.integers(-128, 128, (128, 256), dtype=np.int8)
    W = rng.integers(-128, 128, (256, 256), dtype=np.int8)
    want = port.linear(A, W)
    seen = {}
    gave_up, other_done = threading.Event(), threading.Event()

    def first():
        torch.cuda.set_device(0)
        st = torch.cuda.Stream()
        seen["rc"] = lib.rplb_selftest_bounded_wait_keep(C.c_void_p(st.cuda_stream))
        gave_up.set()
        other_done.wait(60)
        seen["first_status"] = D.kernel_status(True)
        seen["first_after"] = D.kernel_status(False)

    def second():
        torch.cuda.set_device(0)
        gave_up.wait(60)
        seen["second_status"] = D.kernel_status(False)
        D.gemm_backend(3)                                 # per thread: the tensor-core kernel, 128 x 256 tiles
        got = D.linear_i8(torch.from_numpy(A).to(cuda), torch.from_numpy(W).to(cuda))
        torch.cuda.synchronize()
        seen["second_ok"] = bool(np.array_equal(got.cpu().numpy(), want))
        seen["second_after"] = D.kernel_status(False)
        other_done.set()

    t1, t2 = threading.Thread(target=first), threading.Thread(target=second)
    t1.start(); t2.start(); t1.join(120); t2.join(120)
    assert seen == {"rc": 0, "second_status": 0, "second_ok": True, "second_after": 0, "first_status": 99, "first_after": 0}
    assert D.gemm_backend(0) == 0                         # this thread's setting was never touched by the other's


def test_scratch_cannot_grow_inside_a_capture(cuda, lib):
    """A graph keeps the scratch block's address: growing it during capture is refused with an error,
    and a reservation made beforehand makes the same capture work."""
    from rpl_b200 import capi, device as D
    side = torch.cuda.Stream()
    x = torch.randn(1 << 22, device=cuda)
    params = torch.empty(8, device=cuda)
    handle = C.c_void_p(side.cuda_stream)
    with torch.cuda.stream(side):
        g = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(g, stream=side, capture_error_mode="relaxed"):
                with pytest.raises(capi.RplError) as e:
                    D.minmax(x, params=params)            # this stream has no scratch block yet
                assert e.value.code == capi.RPLB_E_UNSUPPORTED
                torch.zeros(1, device=cuda)               # something capturable, so the graph is not empty
        finally:
            del g
    capi.call("rplb_scratch_reserve", handle, 1 << 20)
    with torch.cuda.stream(side):
        D.minmax(x, params=params)                        # outside a capture: fine, and now warm
        side.synchronize()
        want = params.clone()
        g = torch.cuda.CUDAGraph()
        params.zero_()
        with torch.cuda.graph(g, stream=side):
            D.minmax(x, params=params)
        g.replay()
        side.synchronize()
    assert torch.equal(params, want)
    del g
    capi.call("rplb_scratch_release", handle)
