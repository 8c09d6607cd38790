"""Seeded random sweeps over sizes, alignments and shapes, every result compared with the CPU
checker bit for bit and every output surrounded by guard values that must survive: the cases a
hand-picked list of shapes misses (a ragged edge that meets an alignment rule, a view that starts
in the middle of a 16-byte piece)."""
import numpy as np
import pytest
import torch

from conftest import bits

pytestmark = pytest.mark.gpu

GUARD_I8 = 0x55
GUARD_F32 = -7.0
GUARD_I32 = -1234567


def same(a, b):
    return np.array_equal(bits(np.asarray(a)), bits(np.asarray(b)))


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def host(t):
    return t.detach().cpu().numpy()


def _view_f32(x, offset, cuda):
    """x on the device as a view that starts `offset` floats into an allocation."""
    buf = torch.empty(x.size + offset + 8, dtype=torch.float32, device=cuda)
    view = buf[offset:offset + x.size]
    view.copy_(torch.from_numpy(x.reshape(-1)))
    return view


def _guarded(n, offset, dtype, fill, cuda):
    """(buffer, view of n elements starting `offset` elements in); the rest holds `fill`."""
    buf = torch.full((n + offset + 64,), fill, dtype=dtype, device=cuda)
    return buf, buf[offset:offset + n]


def _guards_intact(buf, offset, n, fill):
    h = host(buf)
    return bool((h[:offset] == fill).all() and (h[offset + n:] == fill).all())


def _sizes(rng, count):
    out = []
    for i in range(count):
        kind = i % 4
        if kind == 0:
            out.append(int(rng.integers(1, 200)))
        elif kind == 1:
            out.append(int(rng.integers(200, 100_000)))
        elif kind == 2:
            out.append(int(rng.integers(100_000, 2_000_000)))
        else:
            out.append(int(rng.integers(3_000_000, 5_000_000)))       # either side of the one-launch limit
    return out


def test_per_tensor_kernels_any_size_any_alignment(cuda, lib, port):
    from rpl_b200 import device as D
    rng = np.random.default_rng(20261125)
    for n in _sizes(rng, 20):
        x = (rng.standard_normal(n) * float(rng.choice([1e-3, 1.0, 37.0]))).astype(np.float32)
        if n > 10:
            x[int(rng.integers(0, n))] = np.float32(rng.choice([-1.0, 1.0])) * np.abs(x).max() * 3      # the extreme anywhere
        xin, xoff = int(rng.integers(0, 4)), int(rng.integers(0, 16))
        xv = _view_f32(x, xin, cuda)
        # explicit parameters
        scale, zp = float(rng.choice([0.011, 0.5, 3.0])), int(rng.integers(-20, 20))
        buf, q = _guarded(n, xoff, torch.int8, GUARD_I8, cuda)
        D.quantize(xv, scale, zp, out=q)
        assert same(host(q), port.quantize(x, scale, zp)), ("explicit", n, xin, xoff)
        assert _guards_intact(buf, xoff, n, GUARD_I8), ("explicit guards", n, xin, xoff)
        # symmetric
        buf, q = _guarded(n, xoff, torch.int8, GUARD_I8, cuda)
        _, params = D.quantize_symmetric(xv, out=q)
        wq, ws = port.quantize_symmetric(x)
        assert same(host(q), wq) and same(host(params)[D.QPARAM_SCALE_SYM], ws), ("symmetric", n, xin, xoff)
        assert _guards_intact(buf, xoff, n, GUARD_I8), ("symmetric guards", n, xin, xoff)
        # asymmetric
        buf, q = _guarded(n, xoff, torch.int8, GUARD_I8, cuda)
        _, params = D.quantize_asymmetric(xv, out=q)
        wq, ws, wz = port.quantize_asymmetric(x)
        hp = host(params)
        assert same(host(q), wq) and same(hp[D.QPARAM_SCALE_ASYM], ws) and int(hp.view(np.int32)[D.QPARAM_ZP_ASYM]) == wz, \
            ("asymmetric", n, xin, xoff)
        assert _guards_intact(buf, xoff, n, GUARD_I8), ("asymmetric guards", n, xin, xoff)
        # dequantize of what was just produced, into a guarded fp32 view
        fbuf, f = _guarded(n, xin, torch.float32, GUARD_F32, cuda)
        D.dequantize(q, float(ws), wz, out=f)
        assert same(host(f), port.dequantize(wq, ws, wz)), ("dequantize", n, xin, xoff)
        assert _guards_intact(fbuf, xin, n, GUARD_F32), ("dequantize guards", n, xin, xoff)
    torch.cuda.synchronize()


def test_per_channel_any_shape_any_alignment(cuda, lib, port):
    from rpl_b200 import device as D
    rng = np.random.default_rng(99)
    shapes = [(int(rng.integers(1, 300)), int(rng.integers(1, 5000))) for _ in range(10)]
    shapes += [(int(rng.integers(1, 12)), int(rng.integers(8192, 60000))) for _ in range(4)]      # rows staged in shared memory
    shapes += [(3, 70001), (2, 131072 + 4)]                                                      # rows too long to stage
    for Cn, L in shapes:
        x = (rng.standard_normal((Cn, L)) * np.exp(rng.standard_normal((Cn, 1)))).astype(np.float32)
        xin, xoff = int(rng.integers(0, 4)), int(rng.integers(0, 16))
        xv = _view_f32(x, xin, cuda).view(Cn, L)
        buf, q = _guarded(Cn * L, xoff, torch.int8, GUARD_I8, cuda)
        _, scales, zps = D.quantize_per_channel(xv, Cn, out=q.view(Cn, L))
        wq, wscales, wzps = port.quantize_per_channel(x, Cn)
        assert same(host(q).reshape(Cn, L), wq), ("per channel", Cn, L, xin, xoff)
        assert same(host(scales), wscales) and np.array_equal(host(zps), wzps), ("per channel scales", Cn, L)
        assert _guards_intact(buf, xoff, Cn * L, GUARD_I8), ("per channel guards", Cn, L, xin, xoff)
        fbuf, f = _guarded(Cn * L, xin, torch.float32, GUARD_F32, cuda)
        D.dequantize_per_channel(q.view(Cn, L), scales, out=f.view(Cn, L))
        assert same(host(f).reshape(Cn, L), port.dequantize_per_channel(wq, wscales)), ("dequantize per channel", Cn, L)
        assert _guards_intact(fbuf, xin, Cn * L, GUARD_F32), ("dequantize per channel guards", Cn, L)
    torch.cuda.synchronize()


@pytest.mark.parametrize("which", [0, 1, 3])
def test_gemm_int8_any_shape_with_zero_points(cuda, lib, port, which):
    """gemm_int8's contraction, B as [K,N]: any K (the tensor-core kernel reads B in place when N % 16 == 0 and
    K % 16 == 0, else the dp4a kernel or a transposed copy runs), zero points on and off, output at an aligned and
    at an unaligned address."""
    from rpl_b200 import device as D
    prev = D.gemm_backend(which)
    try:
        rng = np.random.default_rng(4242 + which)
        for i in range(14):
            M, N, K = int(rng.integers(1, 500)), int(rng.integers(1, 400)), int(rng.integers(1, 700))
            if which == 3 or i % 2 == 0:
                K = 16 * max(1, K // 16)
            if i % 3 == 0:
                N = 16 * max(1, N // 16)
            if which == 3 and K % 16:
                continue
            A = rng.integers(-128, 128, (M, K), dtype=np.int8)
            B = rng.integers(-128, 128, (K, N), dtype=np.int8)
            sa, sb, sc = float(rng.random() * 0.1 + 0.01), float(rng.random() * 0.1 + 0.01), float(rng.random() + 0.5)
            za, zb = (int(rng.integers(-9, 9)), int(rng.integers(-9, 9))) if i % 2 else (0, 0)
            ooff = int(rng.choice([0, 4, 1, 3]))
            buf, o = _guarded(M * N, ooff, torch.int32, GUARD_I32, cuda)
            D.gemm_i8_requant(dev(A, cuda), dev(B, cuda), sa, sb, sc, za, zb, out=o.view(M, N))
            want = port.gemm_requant(A, B, sa, sb, sc, za, zb)
            assert same(host(o).reshape(M, N), want), (which, M, N, K, za, zb, ooff)
            assert _guards_intact(buf, ooff, M * N, GUARD_I32), ("guards", which, M, N, K, ooff)
        torch.cuda.synchronize()
        assert D.kernel_status(True) == 0
    finally:
        D.gemm_backend(prev)


@pytest.mark.parametrize("which", [1, 3, 4, 5])
def test_int8_output_and_absmax_into_column_blocks(cuda, lib, port, which):
    from rpl_b200 import device as D
    prev = D.gemm_backend(which)
    try:
        rng = np.random.default_rng(31337 + which)
        for _ in range(10):
            M, N, K = int(rng.integers(1, 700)), int(rng.integers(1, 600)), 16 * int(rng.integers(1, 50))
            A = rng.integers(-128, 128, (M, K), dtype=np.int8)
            W = rng.integers(-128, 128, (N, K), dtype=np.int8)
            ws = ((rng.random(N) + 0.5) * 3e-4).astype(np.float32)
            bias = (rng.standard_normal(N) * 0.1).astype(np.float32)
            sa, so, zo = np.float32(0.0117), np.float32(0.021), int(rng.integers(-5, 5))
            a_dev, o_dev = dev(np.array([sa], np.float32), cuda), dev(np.array([so], np.float32), cuda)
            want = port.linear_dequant(A, W, sa, ws, bias, True)
            pad = int(rng.integers(0, 20))
            wide = torch.full((M, N + pad + int(rng.integers(1, 20))), GUARD_I8, dtype=torch.int8, device=cuda)
            got = D.linear_i8_requant_i8(dev(A, cuda), dev(W, cuda), a_dev, dev(ws, cuda), o_dev, zo, dev(bias, cuda), True,
                                         out=wide[:, pad:pad + N])
            assert same(host(got), port.quantize(want, so, zo)), ("int8 out", which, M, N, K, pad)
            assert (host(wide[:, :pad]) == GUARD_I8).all() and (host(wide[:, pad + N:]) == GUARD_I8).all(), ("int8 guards", which, M, N, K, pad)
            padf = 4 * int(rng.integers(0, 4))
            widef = torch.full((M, N + padf + (4 - N % 4) % 4 + 4 * int(rng.integers(0, 3))), GUARD_F32, device=cuda)
            gotf, amax, nxt = D.linear_i8_dequant_absmax(dev(A, cuda), dev(W, cuda), a_dev, dev(ws, cuda), dev(bias, cuda), True,
                                                        out=widef[:, padf:padf + N])
            top = np.float32(np.abs(want).max())
            assert same(host(gotf), want), ("fp32 out", which, M, N, K, padf)
            assert same(host(amax)[0], top) and same(host(nxt)[0], top / np.float32(127.0)), ("absmax", which, M, N, K)
            assert (host(widef[:, :padf]) == GUARD_F32).all() and (host(widef[:, padf + N:]) == GUARD_F32).all(), ("fp32 guards", which, M, N, K, padf)
        torch.cuda.synchronize()
        assert D.kernel_status(True) == 0
    finally:
        D.gemm_backend(prev)


def test_quantize_fused_into_the_layer_any_shape(cuda, lib, port):
    """rplb_quantize_linear_dequant_f32 over both of its kernels (dp4a for N <= 16 and K <= 512, tensor cores for
    N <= 128 and K <= 896), fp32 activation at a 16-byte aligned view, output a column block with guards."""
    from rpl_b200 import device as D
    rng = np.random.default_rng(555)
    shapes = [(int(rng.integers(1, 3000)), int(rng.integers(1, 17)), 4 * int(rng.integers(1, 129))) for _ in range(8)]
    shapes += [(int(rng.integers(1, 1500)), int(rng.integers(17, 129)), 16 * int(rng.integers(1, 57))) for _ in range(8)]
    for M, N, K in shapes:
        x = (rng.standard_normal((M, K)) * 2.0).astype(np.float32)
        W = rng.integers(-128, 128, (N, K), dtype=np.int8)
        ws = ((rng.random(N) + 0.5) * 1e-3).astype(np.float32)
        bias = rng.standard_normal(N).astype(np.float32)
        sa = np.float32(0.03)
        relu = bool(rng.integers(0, 2))
        want = port.linear_dequant(port.quantize(x, sa, 0), W, sa, ws, bias, relu)
        pad = 4 * int(rng.integers(0, 4))
        wide = torch.full((M, N + pad + int(rng.integers(1, 9))), GUARD_F32, device=cuda)
        stats = torch.zeros(2, device=cuda)
        xv = _view_f32(x, 4 * int(rng.integers(0, 2)), cuda).view(M, K)
        got = D.quantize_linear_dequant(xv, dev(W, cuda), dev(np.array([sa], np.float32), cuda), dev(ws, cuda), dev(bias, cuda), relu,
                                        out=wide[:, pad:pad + N], stats=stats)
        top = np.float32(np.abs(want).max())
        assert same(host(got), want), (M, N, K, pad)
        assert same(host(stats)[0], top) and same(host(stats)[1], top / np.float32(127.0)), ("stats", M, N, K)
        assert (host(wide[:, :pad]) == GUARD_F32).all() and (host(wide[:, pad + N:]) == GUARD_F32).all(), ("guards", M, N, K, pad)
    torch.cuda.synchronize()
    assert D.kernel_status(True) == 0


def test_reference_named_api_with_host_buffers_any_shape(cuda, lib, port):
    """The calls a program written against the reference makes (host pointers in, library-owned host results out),
    over random shapes: quantize in its three forms, per channel, dequantize, gemm_int8 with zero points and
    linear_int8 with and without bias."""
    import ctypes as C

    from rpl_b200 import capi

    def host_tensor(x):
        shape = (C.c_uint32 * x.ndim)(*x.shape)
        t = lib.tensor_create(x.ndim, shape, False)
        C.memmove(t.contents.data, np.ascontiguousarray(x).ctypes.data, x.nbytes)
        return t

    def read(ptr, shape, dtype):
        n = int(np.prod(shape))
        buf = (C.c_char * (n * np.dtype(dtype).itemsize)).from_address(ptr)
        return np.frombuffer(buf, dtype=dtype, count=n).reshape(shape).copy()

    def qt_view(q):
        t = capi.QuantizedTensor()
        t.data = q.ctypes.data
        t.scale, t.zero_point, t.size, t.dims = 1.0, 0, int(q.size), q.ndim
        for i, s in enumerate(q.shape):
            t.shape[i] = s
        return t

    rng = np.random.default_rng(8086)
    for _ in range(10):
        rows, cols = int(rng.integers(1, 400)), int(rng.integers(1, 3000))
        x = (rng.standard_normal((rows, cols)) * float(rng.choice([0.01, 1.0, 50.0]))).astype(np.float32)
        t = host_tensor(x)
        scale, zp = float(rng.choice([0.02, 0.7])), int(rng.integers(-30, 30))
        qt = lib.tensor_quantize_int8(t, scale, zp)
        assert same(read(qt.contents.data, x.shape, np.int8), port.quantize(x, scale, zp)), ("explicit", rows, cols)
        back = lib.tensor_dequantize_int8(qt)
        assert same(read(back.contents.data, x.shape, np.float32), port.dequantize(port.quantize(x, scale, zp), scale, zp))
        lib.tensor_free(back)
        lib.quantized_tensor_free(qt)
        qs = lib.tensor_quantize_int8_symmetric(t)
        wq, ws = port.quantize_symmetric(x)
        assert same(np.float32(qs.contents.scale), ws) and same(read(qs.contents.data, x.shape, np.int8), wq), ("symmetric", rows, cols)
        lib.quantized_tensor_free(qs)
        qa = lib.tensor_quantize_int8_asymmetric(t)
        wq, ws, wz = port.quantize_asymmetric(x)
        assert same(np.float32(qa.contents.scale), ws) and qa.contents.zero_point == wz, ("asymmetric", rows, cols)
        assert same(read(qa.contents.data, x.shape, np.int8), wq), ("asymmetric", rows, cols)
        lib.quantized_tensor_free(qa)
        pc = lib.tensor_quantize_per_channel(t, 0)
        wq, wsc, _ = port.quantize_per_channel(x, rows)
        assert same(read(pc.contents.data, x.shape, np.int8), wq) and same(read(pc.contents.scales, (rows,), np.float32), wsc), \
            ("per channel", rows, cols)
        lib.per_channel_quantized_tensor_free(pc)
        lib.tensor_free(t)
    for i in range(10):
        M, N, K = int(rng.integers(1, 400)), int(rng.integers(1, 400)), int(rng.integers(1, 900))
        if i % 2:
            N, K = 16 * max(1, N // 16), 16 * max(1, K // 16)          # the shapes the tensor cores take in place
        A = rng.integers(-128, 128, (M, K), dtype=np.int8)
        W = rng.integers(-128, 128, (N, K), dtype=np.int8)
        B = np.ascontiguousarray(W.T)
        b = rng.integers(-128, 128, N, dtype=np.int8)
        out = np.full((M, N), GUARD_I32, np.int32)
        za, zb = (int(rng.integers(-9, 9)), int(rng.integers(-9, 9))) if i % 3 else (0, 0)
        lib.gemm_int8(A.ctypes.data, B.ctypes.data, out.ctypes.data, M, N, K, 0.013, 0.021, 0.37, za, zb)
        assert same(out, port.gemm_requant(A, B, 0.013, 0.021, 0.37, za, zb)), ("gemm_int8", M, N, K, za, zb)
        qa, qw, qb = qt_view(A), qt_view(W), qt_view(b)
        lib.linear_int8(C.byref(qa), C.byref(qw), None, out.ctypes.data, M, K, N)
        assert same(out, port.linear(A, W)), ("linear_int8", M, N, K)
        lib.linear_int8(C.byref(qa), C.byref(qw), C.byref(qb), out.ctypes.data, M, K, N)
        assert same(out, port.linear(A, W, b)), ("linear_int8 + bias", M, N, K)
    assert lib.rpl_cuda_last_error() == 0


def test_reference_named_api_from_several_host_threads(cuda, lib, port):
    """The reference's functions are stateless and re-entrant; so are these.  Four host threads call gemm_int8
    (shapes that need the library's scratch memory: a transposed copy of B, row and column sums for the zero
    points), linear_int8 and the symmetric quantize at the same time, each on its own data."""
    import ctypes as C
    import threading

    from rpl_b200 import capi

    def work(seed, failures):
        try:
            rng = np.random.default_rng(seed)
            for i in range(12):
                M, N, K = int(rng.integers(100, 400)), int(rng.integers(17, 300)), 16 * int(rng.integers(4, 40))
                if i % 2:
                    N |= 1                                      # B[K,N] cannot be read in place: transposed copy in scratch
                A = rng.integers(-128, 128, (M, K), dtype=np.int8)
                B = rng.integers(-128, 128, (K, N), dtype=np.int8)
                out = np.zeros((M, N), np.int32)
                za, zb = int(rng.integers(-9, 9)), int(rng.integers(-9, 9))
                lib.gemm_int8(A.ctypes.data, B.ctypes.data, out.ctypes.data, M, N, K, 0.013, 0.021, 0.37, za, zb)
                if not same(out, port.gemm_requant(A, B, 0.013, 0.021, 0.37, za, zb)):
                    failures.append(("gemm_int8", seed, i, M, N, K, za, zb))
                x = (rng.standard_normal((int(rng.integers(1, 200)), int(rng.integers(1, 5000)))) * 3).astype(np.float32)
                shape = (C.c_uint32 * 2)(*x.shape)
                t = lib.tensor_create(2, shape, False)
                C.memmove(t.contents.data, x.ctypes.data, x.nbytes)
                qs = lib.tensor_quantize_int8_symmetric(t)
                wq, ws = port.quantize_symmetric(x)
                n = x.size
                got = np.frombuffer((C.c_char * n).from_address(qs.contents.data), dtype=np.int8, count=n).reshape(x.shape)
                if not (same(np.float32(qs.contents.scale), ws) and same(got, wq)):
                    failures.append(("quantize_symmetric", seed, i, x.shape))
                lib.quantized_tensor_free(qs)
                lib.tensor_free(t)
        except Exception as e:                                  # a failure inside a thread must reach the test
            failures.append(("exception", seed, repr(e)))

    failures = []
    threads = [threading.Thread(target=work, args=(1000 + k, failures)) for k in range(4)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not failures, failures[:5]
    assert lib.rpl_cuda_last_error() == 0


def test_two_devices_in_one_process_from_two_threads(lib, port):
    """One host thread per GPU in the same process (the library's caches are keyed by device, its switches and
    status words by thread): quantize and GEMM on both devices at once, each against the checker."""
    import threading

    from rpl_b200 import device as D
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")

    def work(ordinal, failures):
        try:
            torch.cuda.set_device(ordinal)
            d = torch.device("cuda", ordinal)
            rng = np.random.default_rng(50 + ordinal)
            for i in range(8):
                M, N, K = int(rng.integers(100, 900)), int(rng.integers(17, 600)), 16 * int(rng.integers(4, 40))
                x = (rng.standard_normal((M, K)) * 2).astype(np.float32)
                W = rng.integers(-128, 128, (N, K), dtype=np.int8)
                ws = ((rng.random(N) + 0.5) * 1e-3).astype(np.float32)
                D.gemm_backend([0, 3, 4, 5][i % 4])
                xq, params = D.quantize_symmetric(torch.from_numpy(x).to(d))
                got = D.linear_i8_dequant(xq, torch.from_numpy(W).to(d), params[D.QPARAM_SCALE_SYM:D.QPARAM_SCALE_SYM + 1],
                                          torch.from_numpy(ws).to(d))
                torch.cuda.synchronize(d)
                hq, hs = port.quantize_symmetric(x)
                if not (same(host(xq), hq) and same(host(got), port.linear_dequant(hq, W, hs, ws))):
                    failures.append((ordinal, i, M, N, K))
            D.gemm_backend(0)
            if D.kernel_status(True) != 0:
                failures.append((ordinal, "status"))
        except Exception as e:
            failures.append((ordinal, repr(e)))

    failures = []
    threads = [threading.Thread(target=work, args=(k, failures)) for k in range(2)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    torch.cuda.set_device(0)
    assert not failures, failures[:5]
