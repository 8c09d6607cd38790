"""INT8 contraction kernels (dp4a and tcgen05) against the CPU checker:
int32 results bit for bit, fp32 epilogue within 1e-5 relative (exact equality
is expected and checked first)."""
import numpy as np
import pytest
import torch

from conftest import bits

pytestmark = pytest.mark.gpu

SIMT, TC, TC_SINGLE, TC_PAIR, TC_WIDE, TC_NARROW = 1, 2, 3, 4, 5, 6      # rplb_gemm_backend codes


def same(a, b):
    return np.array_equal(bits(np.asarray(a)), bits(np.asarray(b)))


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def host(t):
    return t.detach().cpu().numpy()


@pytest.fixture(params=[0, 1], ids=["tma_store", "register_store"])
def backend(request):
    """Every test runs with both store paths of the tensor-core epilogue: 32 x 32 chunks through
    TMA tensor stores (where the output's alignment allows it) and rows stored from registers."""
    from rpl_b200 import device as D
    prev = D.gemm_backend(0)
    prev_epi = D.gemm_epilogue(request.param)
    yield D
    D.gemm_backend(prev)
    D.gemm_epilogue(prev_epi)
    assert D.kernel_status(True) == 0


def rel_close(got, want, tol=1e-5):
    denom = np.maximum(np.abs(want), 1e-30)
    return bool((np.abs(got - want) / denom <= tol).all())


def test_golden_vectors_both_kernels(cuda, lib, golden, backend):
    D = backend
    A, W, b = dev(golden["A"], cuda), dev(golden["W"], cuda), dev(golden["bias_i8"], cuda)
    B = dev(np.ascontiguousarray(golden["W"].T), cuda)
    sa, sb, sc = (float(v) for v in golden["gemm_params"])
    D.gemm_backend(SIMT)
    assert same(host(D.linear_i8(A, W)), golden["linear_raw"])
    assert same(host(D.linear_i8(A, W, b)), golden["linear_bias"])
    assert same(host(D.gemm_i8_requant(A, B)), golden["gemm_unit"])
    assert same(host(D.gemm_i8_requant(A, B, sa, sb, sc)), golden["gemm_scaled"])
    assert same(host(D.gemm_i8_requant(A, B, sa, sb, sc, 3, -7)), golden["gemm_zp"])
    two, twoT = dev(np.array([[127, 127]], np.int8), cuda), dev(np.array([[127], [127]], np.int8), cuda)
    got = [int(D.gemm_i8_requant(two, twoT)[0, 0]), int(D.gemm_i8_requant(two, twoT, 0.5, 0.5, 2.0)[0, 0]),
           int(D.gemm_i8_requant(two, twoT, 1, 1, 1, 3, -2)[0, 0])]
    assert got == [32258, 4032, 31992]


# K = 129 is not a multiple of 16, so the golden pair above cannot reach the
# tensor-core kernel; these shapes can (K % 16 == 0), ragged M and N included.
TC_SHAPES = [(128, 256, 128), (1, 16, 16), (37, 23, 144), (130, 300, 784), (512, 512, 512), (257, 10, 128),
             (300, 1000, 4096), (128, 256, 16), (1000, 129, 2064)]


@pytest.mark.parametrize("mnk", TC_SHAPES)
def test_tcgen05_raw_and_bias(cuda, lib, port, backend, mnk):
    D = backend
    M, N, K = mnk
    rng = np.random.default_rng(M * 31 + N * 7 + K)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    W = rng.integers(-128, 128, (N, K), dtype=np.int8)
    b = rng.integers(-128, 128, N, dtype=np.int8)
    want = port.linear(A, W)
    for which in (TC_SINGLE, TC_PAIR, TC_WIDE, TC):
        D.gemm_backend(which)
        got = host(D.linear_i8(dev(A, cuda), dev(W, cuda)))
        torch.cuda.synchronize()
        assert D.kernel_status(True) == 0
        assert same(got, want), which
        assert same(host(D.linear_i8(dev(A, cuda), dev(W, cuda), dev(b, cuda))), port.linear(A, W, b)), which
    D.gemm_backend(SIMT)
    assert same(host(D.linear_i8(dev(A, cuda), dev(W, cuda))), want)


@pytest.mark.parametrize("mnk", [(64, 64, 64), (130, 300, 784), (512, 512, 512), (33, 77, 19), (5, 3, 1)])
@pytest.mark.parametrize("which", [SIMT, TC_SINGLE, TC_PAIR, TC_WIDE])
def test_requant_epilogue(cuda, lib, port, backend, mnk, which):
    D = backend
    M, N, K = mnk
    if which != SIMT and K % 16:
        pytest.skip("tensor-core kernel needs K % 16 == 0")
    rng = np.random.default_rng(M + N + K)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    B = rng.integers(-128, 128, (K, N), dtype=np.int8)
    D.gemm_backend(which)
    for args in ((1, 1, 1, 0, 0), (0.013, 0.021, 0.37, 0, 0), (0.5, 0.5, 1e-3, 0, 0)):
        assert same(host(D.gemm_i8_requant(dev(A, cuda), dev(B, cuda), *args)), port.gemm_requant(A, B, *args))
    if which == SIMT:
        for args in ((0.013, 0.021, 0.37, 3, -7), (1, 1, 1, -128, 127), (0.3, 0.3, 1e-4, 5, 0)):
            assert same(host(D.gemm_i8_requant(dev(A, cuda), dev(B, cuda), *args)), port.gemm_requant(A, B, *args))


@pytest.mark.parametrize("mnk", [(128, 256, 128), (37, 23, 144), (130, 300, 784), (256, 10, 128), (512, 512, 512)])
@pytest.mark.parametrize("which", [SIMT, TC_SINGLE, TC_PAIR, TC_WIDE])
@pytest.mark.parametrize("relu", [False, True])
def test_fused_dequant_epilogue(cuda, lib, port, backend, mnk, which, relu):
    D = backend
    M, N, K = mnk
    rng = np.random.default_rng(M * 3 + N * 5 + K * 7)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    W = rng.integers(-128, 128, (N, K), dtype=np.int8)
    ws = ((rng.random(N) + 0.5) * 2e-4).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.05).astype(np.float32)
    a_scale = np.float32(0.0231)
    D.gemm_backend(which)
    a_dev = dev(np.array([a_scale], np.float32), cuda)
    for b in (bias, None):
        want = port.linear_dequant(A, W, a_scale, ws, b, relu)
        got = host(D.linear_i8_dequant(dev(A, cuda), dev(W, cuda), a_dev, dev(ws, cuda),
                                       dev(b, cuda) if b is not None else None, relu))
        assert rel_close(got, want, 1e-5)
        assert same(got, want)


def test_fused_epilogue_writes_a_column_block_in_place(cuda, lib, port, backend):
    """Output row stride larger than N: what an N-sharded rank does."""
    D = backend
    M, N, K, NT = 200, 256, 256, 768
    rng = np.random.default_rng(9)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    W = rng.integers(-128, 128, (N, K), dtype=np.int8)
    ws = ((rng.random(N) + 0.5) * 1e-4).astype(np.float32)
    want = port.linear_dequant(A, W, 0.01, ws, None, False)
    a_dev = dev(np.array([0.01], np.float32), cuda)
    for which in (SIMT, TC_SINGLE, TC_PAIR, TC_WIDE):
        D.gemm_backend(which)
        full = torch.full((M, NT), -7.0, device=cuda)
        D.linear_i8_dequant(dev(A, cuda), dev(W, cuda), a_dev, dev(ws, cuda), out=full[:, 256:512])
        h = host(full)
        assert same(h[:, 256:512], want)
        assert (h[:, :256] == -7.0).all() and (h[:, 512:] == -7.0).all()


def test_config1_512_cubed_end_to_end(cuda, lib, port, backend):
    """fp32 N(0,1) 512x512 pair, per-tensor symmetric, raw / requantized / fp32 outputs."""
    D = backend
    rng = np.random.default_rng(0x5EED0010)
    A = rng.standard_normal((512, 512)).astype(np.float32)
    Bt = rng.standard_normal((512, 512)).astype(np.float32)      # stored [N,K]
    qa, pa = D.quantize_symmetric(dev(A, cuda))
    qb, pb = D.quantize_symmetric(dev(Bt, cuda))
    wqa, sa = port.quantize_symmetric(A)
    wqb, sb = port.quantize_symmetric(Bt)
    assert same(host(qa), wqa) and same(host(qb), wqb)
    for which in (SIMT, TC_SINGLE, TC_PAIR, TC_WIDE):
        D.gemm_backend(which)
        assert same(host(D.linear_i8(qa, qb)), port.linear(wqa, wqb))
        Bkn = np.ascontiguousarray(wqb.T)
        sc = np.float32(sa * sb * 64)
        assert same(host(D.gemm_i8_requant(qa, dev(Bkn, cuda), sa, sb, sc)), port.gemm_requant(wqa, Bkn, sa, sb, sc))
        ws = np.full(512, sb, np.float32)
        got = host(D.linear_i8_dequant(qa, qb, pa[D.QPARAM_SCALE_SYM:D.QPARAM_SCALE_SYM + 1], dev(ws, cuda)))
        assert same(got, port.linear_dequant(wqa, wqb, sa, ws))


def test_tcgen05_matches_dp4a_at_projection_size(cuda, lib, backend):
    """4096 x 4096 x 4096 (a CPU loop would take minutes): the two kernels must
    agree on every int32, and linearity in A must hold."""
    D = backend
    g = torch.Generator(device=cuda)
    g.manual_seed(3)
    A = torch.randint(-128, 128, (4096, 4096), device=cuda, generator=g, dtype=torch.int8)
    W = torch.randint(-128, 128, (4096, 4096), device=cuda, generator=g, dtype=torch.int8)
    D.gemm_backend(TC_PAIR)
    c_tc = D.linear_i8(A, W)
    D.gemm_backend(TC_SINGLE)
    assert torch.equal(D.linear_i8(A, W), c_tc)
    D.gemm_backend(TC_WIDE)
    assert torch.equal(D.linear_i8(A, W), c_tc)
    D.gemm_backend(SIMT)
    c_simt = D.linear_i8(A, W)
    assert torch.equal(c_tc, c_simt)
    # column sums: sum_n C[m,n] == A[m,:] . (sum_n W[n,:])
    colsum = W.to(torch.int64).sum(0)
    want = (A[:64].to(torch.int64) * colsum[None, :]).sum(1)
    assert torch.equal(c_tc[:64].to(torch.int64).sum(1), want)


def test_sampled_tiles_vs_checker_at_projection_size(cuda, lib, port, backend):
    D = backend
    g = torch.Generator(device=cuda)
    g.manual_seed(4)
    M, N, K = 2048, 4096, 4096
    A = torch.randint(-128, 128, (M, K), device=cuda, generator=g, dtype=torch.int8)
    W = torch.randint(-128, 128, (N, K), device=cuda, generator=g, dtype=torch.int8)
    D.gemm_backend(TC)
    Cd = D.linear_i8(A, W)
    rng = np.random.default_rng(1)
    for _ in range(8):
        m0, n0 = int(rng.integers(0, M - 128)), int(rng.integers(0, N - 128))
        want = port.linear(host(A[m0:m0 + 128]), host(W[n0:n0 + 128]))
        assert same(host(Cd[m0:m0 + 128, n0:n0 + 128]), want)


@pytest.mark.parametrize("mnk", [(130, 300, 784), (512, 512, 512), (64, 40, 16), (130, 304, 784), (37, 48, 144)])
@pytest.mark.parametrize("which", [TC_SINGLE, TC_PAIR, TC_WIDE])
def test_zero_points_on_the_tensor_core_path(cuda, lib, port, backend, mnk, which):
    """gemm_int8 with za, zb != 0: the tensor-core kernels correct the plain product
    with row sums of A and column sums of B in the epilogue."""
    D = backend
    M, N, K = mnk
    rng = np.random.default_rng(M + 2 * N + 3 * K)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    B = rng.integers(-128, 128, (K, N), dtype=np.int8)
    D.gemm_backend(which)
    for args in ((0.013, 0.021, 0.37, 3, -7), (1, 1, 1, -128, 127), (0.3, 0.3, 1e-4, 5, 0), (1, 1, 1, 0, 9)):
        got = host(D.gemm_i8_requant(dev(A, cuda), dev(B, cuda), *args))
        assert same(got, port.gemm_requant(A, B, *args)), args


@pytest.mark.parametrize("mnk", [(130, 300, 784), (512, 512, 512), (65, 10, 128)])
@pytest.mark.parametrize("which", [SIMT, TC_SINGLE, TC_PAIR, TC_WIDE])
def test_epilogue_reports_absmax_for_the_next_layer(cuda, lib, port, backend, mnk, which):
    D = backend
    M, N, K = mnk
    rng = np.random.default_rng(M * 11 + N)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    W = rng.integers(-128, 128, (N, K), dtype=np.int8)
    ws = ((rng.random(N) + 0.5) * 2e-4).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.05).astype(np.float32)
    a_dev = dev(np.array([0.0231], np.float32), cuda)
    D.gemm_backend(which)
    for relu in (False, True):
        out, absmax, scale = D.linear_i8_dequant_absmax(dev(A, cuda), dev(W, cuda), a_dev, dev(ws, cuda), dev(bias, cuda), relu)
        want = port.linear_dequant(A, W, np.float32(0.0231), ws, bias, relu)
        assert same(host(out), want)
        wq, wscale = port.quantize_symmetric(want)
        assert same(host(scale)[0], wscale) and float(absmax.item()) == float(np.abs(want).max())
        # the next layer's quantizer, fed the reported scale, reproduces the two-pass result
        assert same(host(D.quantize_dev(out, scale)), wq)


@pytest.mark.parametrize("mnk", [(130, 300, 784), (512, 512, 512), (65, 10, 128), (256, 256, 256)])
@pytest.mark.parametrize("which", [SIMT, TC_SINGLE, TC_PAIR, TC_WIDE])
def test_int8_output_with_a_static_scale(cuda, lib, port, backend, mnk, which):
    D = backend
    M, N, K = mnk
    rng = np.random.default_rng(M * 13 + K)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    W = rng.integers(-128, 128, (N, K), dtype=np.int8)
    ws = ((rng.random(N) + 0.5) * 2e-4).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.05).astype(np.float32)
    a_dev = dev(np.array([0.0231], np.float32), cuda)
    D.gemm_backend(which)
    for out_scale, zp, relu in ((0.05, 0, True), (0.031, -9, False), (1e-3, 4, False)):
        want = port.quantize(port.linear_dequant(A, W, np.float32(0.0231), ws, bias, relu), np.float32(out_scale), zp)
        got = D.linear_i8_requant_i8(dev(A, cuda), dev(W, cuda), a_dev, dev(ws, cuda),
                                     dev(np.array([out_scale], np.float32), cuda), zp, dev(bias, cuda), relu)
        assert same(host(got), want), (out_scale, zp, relu)


def test_empty_and_degenerate_shapes(cuda, lib, port, backend):
    D = backend
    z = lambda *s: torch.zeros(s, dtype=torch.int8, device=cuda)
    # K = 0: every sum is empty, the int8 bias still applies
    b = dev(np.array([5, -7, 9], np.int8), cuda)
    out = D.linear_i8(z(4, 0), z(3, 0), b)
    assert host(out).tolist() == [[5, -7, 9]] * 4
    # M = 0 and N = 0: nothing is written, nothing fails
    assert D.linear_i8(z(0, 16), z(3, 16)).shape == (0, 3)
    assert D.linear_i8(z(4, 16), z(0, 16)).shape == (4, 0)
    assert D.gemm_i8_requant(z(0, 16), z(16, 5)).shape == (0, 5)
    # a tall problem on the dp4a kernel: more than 65535 row tiles
    rng = np.random.default_rng(0)
    A = rng.integers(-128, 128, (65536 * 64 + 70, 20), dtype=np.int8)
    W = rng.integers(-128, 128, (3, 20), dtype=np.int8)
    D.gemm_backend(SIMT)
    assert same(host(D.linear_i8(dev(A, cuda), dev(W, cuda))), port.linear(A, W))


def test_bounded_wait_gives_up_and_reports(cuda, lib, port, backend):
    """A wait on a barrier that nothing signals must end by itself (about a
    millisecond here), leave its code in the status word, and leave the library
    usable: the next GEMM runs and is correct."""
    import ctypes as C
    from rpl_b200 import capi
    D = backend
    assert D.kernel_status(True) == 0
    capi.call("rplb_selftest_bounded_wait", C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert D.kernel_status(False) == 0                  # the self-test clears what it provoked
    rng = np.random.default_rng(1)
    A = rng.integers(-128, 128, (128, 256), dtype=np.int8)
    W = rng.integers(-128, 128, (256, 256), dtype=np.int8)
    D.gemm_backend(TC_SINGLE)
    assert same(host(D.linear_i8(dev(A, cuda), dev(W, cuda))), port.linear(A, W))


@pytest.mark.parametrize("mnk", [(128, 256, 128), (130, 304, 784), (37, 48, 144), (512, 512, 512), (1000, 1040, 2064),
                                 (257, 16, 16)])
def test_gemm_int8_reads_b_kn_in_place(cuda, lib, port, backend, mnk):
    """gemm_int8's B [K,N] with N % 16 == 0 reaches the tensor cores without a transposed
    copy (MN-major operand); ragged M, N and K tails included."""
    D = backend
    M, N, K = mnk
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    B = rng.integers(-128, 128, (K, N), dtype=np.int8)
    for which in (TC_SINGLE, TC):
        D.gemm_backend(which)
        before = D.launch_count()
        got = host(D.gemm_i8_requant(dev(A, cuda), dev(B, cuda), 0.013, 0.021, 0.37))
        assert D.launch_count() - before == 1                  # the GEMM alone: no transpose pass
        assert same(got, port.gemm_requant(A, B, 0.013, 0.021, 0.37)), which
    assert same(host(D.gemm_i8_requant(dev(A, cuda), dev(B, cuda))), port.gemm_requant(A, B))


# (M, N, K): tensor-core route (N <= 128, K <= 896, K % 16 == 0) and dp4a route (N <= 16, K <= 512, K % 4 == 0)
FUSED_SHAPES = [(1000, 128, 784), (128, 128, 128), (300, 100, 896), (65, 17, 16), (4096, 64, 400), (257, 128, 880),
                (1000, 10, 128), (33, 16, 512), (5, 1, 4), (700, 3, 100), (2048, 10, 132)]


@pytest.mark.parametrize("mnk", FUSED_SHAPES)
@pytest.mark.parametrize("relu", [False, True])
def test_quantize_fused_into_the_layer(cuda, lib, port, backend, mnk, relu):
    """rplb_quantize_linear_dequant_f32: the int8 activation is never written, the result is the one the
    two-step path gives (quantize with the given scale, then the contraction with the fused epilogue)."""
    from rpl_b200 import capi
    D = backend
    M, N, K = mnk
    rng = np.random.default_rng(M + 3 * N + 7 * K)
    x = (rng.standard_normal((M, K)) * 2.0).astype(np.float32)
    x[0, :4] = [0.5 * 0.03, 1.5 * 0.03, -2.5 * 0.03, 1e9]            # ties and a value far outside the range
    wq = rng.integers(-128, 128, (N, K), dtype=np.int8)
    ws = ((rng.random(N) + 0.5) * 1e-3).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    sa = np.float32(0.03)
    xq = port.quantize(x, sa, 0)
    want = port.linear_dequant(xq, wq, sa, ws, bias, relu)
    a_dev = dev(np.array([sa], np.float32), cuda)
    stats = torch.zeros(2, device=cuda)
    wide = torch.full((M, N + 12), -3.0, device=cuda)                  # a column block of a wider matrix
    for out in (None, wide[:, 4:4 + N]):
        got = D.quantize_linear_dequant(dev(x, cuda), dev(wq, cuda), a_dev, dev(ws, cuda), dev(bias, cuda), relu, out=out, stats=stats)
        torch.cuda.synchronize()
        assert D.kernel_status(True) == 0
        assert same(host(got), want)
        amax = np.float32(np.abs(want).max())
        assert same(host(stats)[0], amax) and same(host(stats)[1], amax / np.float32(127.0))
    assert (host(wide[:, :4]) == -3.0).all() and (host(wide[:, 4 + N:]) == -3.0).all()
    # the same bits as the two-step device path
    two = D.linear_i8_dequant(D.quantize_dev(dev(x, cuda), a_dev), dev(wq, cuda), a_dev, dev(ws, cuda), dev(bias, cuda), relu)
    assert same(host(two), want)


def test_quantize_fused_refuses_other_shapes(cuda, lib, backend):
    from rpl_b200 import capi
    D = backend
    s = torch.ones(1, device=cuda)
    for M, N, K in ((64, 129, 128), (64, 128, 912), (64, 64, 24), (64, 17, 516)):
        with pytest.raises(capi.RplError) as e:
            D.quantize_linear_dequant(torch.zeros((M, K), device=cuda), torch.zeros((N, K), dtype=torch.int8, device=cuda), s,
                                      torch.ones(N, device=cuda))
        assert e.value.code == capi.RPLB_E_UNSUPPORTED


@pytest.mark.parametrize("mnk", [(1000, 128, 784), (128, 128, 128), (300, 100, 896), (65, 17, 16), (257, 10, 128),
                                 (20000, 128, 784), (19000, 10, 128)])
@pytest.mark.parametrize("relu", [False, True])
def test_kernel_for_few_output_features(cuda, lib, port, backend, mnk, relu):
    """The tensor-core kernel with the whole weight matrix resident in shared memory (backend 6, and the automatic
    choice once every SM gets a tile): same bits as the checker, absmax included."""
    from rpl_b200 import capi
    D = backend
    M, N, K = mnk
    rng = np.random.default_rng(M + N + K)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    W = rng.integers(-128, 128, (N, K), dtype=np.int8)
    ws = ((rng.random(N) + 0.5) * 2e-4).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.05).astype(np.float32)
    a_scale = np.float32(0.0231)
    want = port.linear_dequant(A, W, a_scale, ws, bias, relu)
    a_dev = dev(np.array([a_scale], np.float32), cuda)
    for which in (TC_NARROW, 0):
        D.gemm_backend(which)
        got, amax, nxt = D.linear_i8_dequant_absmax(dev(A, cuda), dev(W, cuda), a_dev, dev(ws, cuda), dev(bias, cuda), relu)
        torch.cuda.synchronize()
        assert D.kernel_status(True) == 0
        assert same(host(got), want), which
        assert same(host(amax)[0], np.float32(np.abs(want).max()))
        # the scale of the next layer's activation, written by the last warp through (no second kernel)
        assert same(host(nxt)[0], np.float32(np.abs(want).max()) / np.float32(127.0))
    D.gemm_backend(TC_NARROW)
    with pytest.raises(capi.RplError):                       # other epilogues and wider layers are refused, not emulated
        D.linear_i8(dev(A, cuda), dev(W, cuda))
    with pytest.raises(capi.RplError):
        D.linear_i8_dequant(dev(A[:64], cuda), torch.zeros((256, K), dtype=torch.int8, device=cuda), a_dev, torch.ones(256, device=cuda))


def _random_shapes(count, seed):
    rng = np.random.default_rng(seed)
    shapes = []
    for _ in range(count):
        M = int(rng.integers(1, 900))
        N = int(rng.integers(1, 700))
        K = 16 * int(rng.integers(1, 80))                   # the tensor-core kernels need K % 16 == 0
        shapes.append((M, N, K))
    return shapes


@pytest.mark.parametrize("which", [SIMT, TC_SINGLE, TC_PAIR, TC_WIDE])
def test_seeded_random_shapes_every_kernel(cuda, lib, port, backend, which):
    """Sixteen shapes drawn from a fixed seed (ragged M and N, K from 16 to 1264), every contraction kernel, the
    raw int32 result and the fp32 epilogue with bias and ReLU into a column block of a wider matrix: the same bits
    as the checker, and nothing written outside the block."""
    D = backend
    D.gemm_backend(which)
    for M, N, K in _random_shapes(16, 20261125):
        rng = np.random.default_rng(M * 1009 + N * 31 + K)
        A = rng.integers(-128, 128, (M, K), dtype=np.int8)
        W = rng.integers(-128, 128, (N, K), dtype=np.int8)
        ws = ((rng.random(N) + 0.5) * 3e-4).astype(np.float32)
        bias = (rng.standard_normal(N) * 0.1).astype(np.float32)
        sa = np.float32(0.0117)
        assert same(host(D.linear_i8(dev(A, cuda), dev(W, cuda))), port.linear(A, W)), (which, M, N, K)
        pad = 4 * int(rng.integers(0, 4))                   # a 16-byte multiple keeps the TMA-store path reachable
        wide = torch.full((M, N + pad + 5), -7.0, device=cuda)
        got = D.linear_i8_dequant(dev(A, cuda), dev(W, cuda), dev(np.array([sa], np.float32), cuda), dev(ws, cuda), dev(bias, cuda), True,
                                  out=wide[:, pad:pad + N])
        want = port.linear_dequant(A, W, sa, ws, bias, True)
        assert same(host(got), want), (which, M, N, K)
        assert (host(wide[:, :pad]) == -7.0).all() and (host(wide[:, pad + N:]) == -7.0).all(), (which, M, N, K)
    torch.cuda.synchronize()
    assert D.kernel_status(True) == 0


def test_seeded_random_shapes_kernel_for_few_output_features(cuda, lib, port, backend):
    """The same sweep for the kernel that keeps the weights in shared memory (N <= 128, K <= 896): column blocks whose
    width is not a multiple of four leave their ragged edge from registers, not through a tensor store."""
    D = backend
    D.gemm_backend(TC_NARROW)
    rng0 = np.random.default_rng(777)
    for _ in range(12):
        M, N, K = int(rng0.integers(1, 1500)), int(rng0.integers(1, 129)), 16 * int(rng0.integers(1, 57))
        rng = np.random.default_rng(M * 1009 + N * 31 + K)
        A = rng.integers(-128, 128, (M, K), dtype=np.int8)
        W = rng.integers(-128, 128, (N, K), dtype=np.int8)
        ws = ((rng.random(N) + 0.5) * 3e-4).astype(np.float32)
        bias = (rng.standard_normal(N) * 0.1).astype(np.float32)
        sa = np.float32(0.0117)
        pad = 4 * int(rng.integers(0, 4))
        wide = torch.full((M, N + pad + (4 - N % 4) % 4 + 4), -7.0, device=cuda)       # row stride a multiple of 16 bytes
        got = D.linear_i8_dequant(dev(A, cuda), dev(W, cuda), dev(np.array([sa], np.float32), cuda), dev(ws, cuda), dev(bias, cuda), True,
                                  out=wide[:, pad:pad + N])
        want = port.linear_dequant(A, W, sa, ws, bias, True)
        assert same(host(got), want), (M, N, K)
        assert (host(wide[:, :pad]) == -7.0).all() and (host(wide[:, pad + N:]) == -7.0).all(), (M, N, K)
    torch.cuda.synchronize()
    assert D.kernel_status(True) == 0
