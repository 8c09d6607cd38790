"""Quantize / dequantize kernels against the CPU checker, bit for bit."""
import numpy as np
import pytest
import torch

from conftest import bits

pytestmark = pytest.mark.gpu


def same(a, b):
    return np.array_equal(bits(np.asarray(a)), bits(np.asarray(b)))


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def host(t):
    return t.detach().cpu().numpy()


def sweep_tensor(rng, shape, sigma=3.0, outliers=1e-3):
    x = (rng.standard_normal(shape) * sigma).astype(np.float32)
    m = rng.random(shape) < outliers
    x[m] = np.where(rng.random(int(m.sum())) < 0.5, -50.0, 50.0)
    return x


def test_golden_vectors_on_gpu(cuda, lib, golden):
    from rpl_b200 import device as D
    x = dev(golden["kat_x"], cuda)
    assert same(host(D.quantize(x, 1.0, 0)), golden["kat_q_s1_z0"])
    assert same(host(D.quantize(x, 1.0, 5)), golden["kat_q_s1_z5"])
    assert same(host(D.dequantize(dev(golden["kat_q_s1_z5"], cuda), 1.0, 5)), golden["kat_dq_s1_z5"])
    q, p = D.quantize_symmetric(x)
    assert same(host(q), golden["kat_q_sym"]) and same(host(p)[D.QPARAM_SCALE_SYM], golden["kat_scale_sym"])
    q, p = D.quantize_symmetric(dev(np.zeros(8, np.float32), cuda))
    assert same(host(q), golden["zeros_q_sym"]) and host(p)[D.QPARAM_SCALE_SYM] == 0.0
    odd = dev(golden["odd_x"], cuda)
    for zp, key in ((0, "odd_q_s1_z0"), (7, "odd_q_s1_z7"), (-7, "odd_q_s1_zm7")):
        assert same(host(D.quantize(odd, 1.0, zp)), golden[key])
    q, p = D.quantize_symmetric(dev(golden["withnan_x"], cuda))
    assert same(host(q), golden["withnan_q_sym"]) and same(host(p)[D.QPARAM_SCALE_SYM], golden["withnan_scale_sym"])
    x = dev(golden["x"], cuda)
    assert same(host(D.quantize(x, 0.05, 3)), golden["x_q_explicit"])
    q, p = D.quantize_symmetric(x)
    assert same(host(q), golden["x_q_sym"]) and same(host(p)[D.QPARAM_SCALE_SYM], golden["x_scale_sym"])
    q, p = D.quantize_asymmetric(x)
    hp = host(p)
    assert same(host(q), golden["x_q_asym"]) and same(hp[D.QPARAM_SCALE_ASYM], golden["x_scale_asym"])
    assert int(hp.view(np.int32)[D.QPARAM_ZP_ASYM]) == int(golden["x_zp_asym"])
    q, sc, zp = D.quantize_per_channel(x)
    assert same(host(q), golden["x_q_pc"]) and same(host(sc), golden["x_scales_pc"]) and same(host(zp), golden["x_zps_pc"])
    q, sc, _ = D.quantize_per_channel(dev(golden["w"], cuda))
    assert same(host(q), golden["w_q_pc"]) and same(host(sc), golden["w_scales_pc"])
    assert same(host(D.dequantize(dev(golden["x_q_sym"], cuda), float(golden["x_scale_sym"]), 0)), golden["x_dq_sym"])
    assert same(host(D.dequantize(dev(golden["x_q_asym"], cuda), float(golden["x_scale_asym"]), int(golden["x_zp_asym"]))),
                golden["x_dq_asym"])
    assert same(host(D.relu_(dev(golden["relu_in"], cuda))), golden["relu_out"])


@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 1023, 1024, 1025, 4096 * 3 + 7, 1 << 20])
def test_per_tensor_sizes(cuda, lib, port, n):
    from rpl_b200 import device as D
    rng = np.random.default_rng(n + 1)
    x = sweep_tensor(rng, (n,))
    xd = dev(x, cuda)
    for scale, zp in ((0.05, 0), (0.37, -11), (1e-3, 90)):
        assert same(host(D.quantize(xd, scale, zp)), port.quantize(x, scale, zp))
    q, p = D.quantize_symmetric(xd)
    hp = host(p)
    wq, ws = port.quantize_symmetric(x)
    assert same(hp[D.QPARAM_SCALE_SYM], ws) and same(host(q), wq)
    mn, mx = port.minmax_seeded(x)
    assert same(hp[D.QPARAM_MIN], mn) and same(hp[D.QPARAM_MAX], mx)
    q, p = D.quantize_asymmetric(xd)
    wq, ws, wz = port.quantize_asymmetric(x)
    hp = host(p)
    if n:
        assert same(host(q), wq) and same(hp[D.QPARAM_SCALE_ASYM], ws) and int(hp.view(np.int32)[D.QPARAM_ZP_ASYM]) == wz
    qh = port.quantize(x, 0.05, 0)
    assert same(host(D.dequantize(dev(qh, cuda), 0.05, 0)), port.dequantize(qh, 0.05, 0))
    assert same(host(D.dequantize(dev(qh, cuda), 0.3, -17)), port.dequantize(qh, 0.3, -17))


def test_misaligned_views_take_the_scalar_path(cuda, lib, port):
    from rpl_b200 import device as D
    rng = np.random.default_rng(3)
    x = sweep_tensor(rng, (5000,))
    base = dev(x, cuda)
    for off in (1, 2, 3):
        v = base[off:off + 4001]
        hv = x[off:off + 4001]
        out = torch.zeros(4003, dtype=torch.int8, device=cuda)[off % 2:off % 2 + 4001]
        assert same(host(D.quantize(v, 0.07, 2, out=out)), port.quantize(hv, 0.07, 2))
        q, p = D.quantize_symmetric(v)
        wq, ws = port.quantize_symmetric(hv)
        assert same(host(q), wq) and same(host(p)[D.QPARAM_SCALE_SYM], ws)


@pytest.mark.parametrize("shape", [(1, 4), (10, 128), (128, 784), (7, 1031), (64, 4096), (5, 8192), (3, 8196),
                                   (2, 40000), (300, 12), (4, 1 << 18),
                                   # rows kept on chip in registers + shared memory (32 to 232 KiB), ragged lengths included
                                   (5, 16384), (300, 8200), (700, 16384), (9, 18432), (7, 18428), (450, 12292),
                                   (3, 20000), (310, 28672), (149, 24004), (4, 59392), (40, 32768),
                                   # long rows (the two-pass kernel)
                                   (3, 59396), (4, 65536), (40, 65540), (2, 100000),
                                   (37, 131072), (3, 262144), (2, 262148), (2, 300000)])
def test_per_channel_shapes(cuda, lib, port, shape):
    from rpl_b200 import capi, device as D
    rng = np.random.default_rng(shape[0] * 7919 + shape[1])
    x = sweep_tensor(rng, shape)
    if shape[0] > 2:
        x[1] = 0.0                                   # an all-zero channel: scale 0, every value -128
    wq, wsc, wzp = port.quantize_per_channel(x, shape[0])
    for staging in (1, 0):                           # rows of 32 to 232 KiB: kept on chip, or two passes
        prev = capi.load().rplb_per_channel_staging(staging)
        q, sc, zp = D.quantize_per_channel(dev(x, cuda))
        capi.load().rplb_per_channel_staging(prev)
        assert same(host(sc), wsc) and same(host(zp), wzp) and same(host(q), wq), staging
    assert same(host(D.dequantize_per_channel(q, sc)), port.dequantize_per_channel(wq, wsc))


@pytest.mark.parametrize("length", [16384, 32768, 65536, 131072, 262144])
def test_per_channel_extreme_in_one_part_only(cuda, lib, port, length):
    """Long rows: the value that sets a channel's scale sits at one place only, a
    different one per row, next to a NaN that the min/max compares must skip."""
    from rpl_b200 import device as D
    rng = np.random.default_rng(length)
    rows = 19
    x = (rng.standard_normal((rows, length)) * 0.5).astype(np.float32)
    for r in range(rows):
        pos = (r * (length // 16) + 13 * r) % length
        x[r, pos] = np.float32((100.0 + r) * (-1.0 if r % 2 else 1.0))
        x[r, (pos + length // 2) % length] = np.nan            # skipped by the min/max compares
    x[5, :] = np.float32(-0.0)
    q, sc, zp = D.quantize_per_channel(dev(x, cuda))
    wq, wsc, wzp = port.quantize_per_channel(x, rows)
    assert same(host(sc), wsc) and same(host(zp), wzp) and same(host(q), wq)


def test_round_trip_and_idempotence_at_sweep_size(cuda, lib):
    """2^26 elements (too slow to compare element-wise on every run against a
    scalar CPU loop): properties that hold for any size."""
    from rpl_b200 import device as D
    g = torch.Generator(device=cuda)
    g.manual_seed(11)
    n = 1 << 26
    x = torch.randn(n, device=cuda, generator=g) * 3.0
    x[::1009] = 50.0
    x[5::2003] = -50.0
    q, p = D.quantize_symmetric(x)
    scale = float(p[D.QPARAM_SCALE_SYM].item())
    assert scale == float(np.float32(50.0) / np.float32(127.0))
    assert int(q.max()) == 127 and int(q.min()) == -127
    y = D.dequantize(q, scale, 0)
    assert float((y - x).abs().max()) <= scale * 0.50001
    q2, p2 = D.quantize_symmetric(y)                 # quantizing the dequantized tensor changes nothing
    assert torch.equal(q, q2) and abs(float(p2[D.QPARAM_SCALE_SYM].item()) - scale) <= scale * 2.4e-7
    qc, sc, _ = D.quantize_per_channel(x.view(-1, 4096))
    yc = D.dequantize_per_channel(qc, sc)
    assert bool(((yc - x.view(-1, 4096)).abs() <= sc[:, None] * 0.50001).all())
    # explicit-scale kernel agrees with the two-pass entry point
    assert torch.equal(D.quantize(x, scale, 0), q)
    assert torch.equal(D.quantize_dev(x, p[D.QPARAM_SCALE_SYM:D.QPARAM_SCALE_SYM + 1]), q)


def test_sampled_parity_at_sweep_size(cuda, lib, port):
    """2^26 elements: compare 64 random 4096-element windows with the checker."""
    from rpl_b200 import device as D
    g = torch.Generator(device=cuda)
    g.manual_seed(12)
    n = 1 << 26
    x = torch.randn(n, device=cuda, generator=g) * 3.0
    x[::997] = 50.0
    q, p = D.quantize_symmetric(x)
    scale = host(p)[D.QPARAM_SCALE_SYM]
    rng = np.random.default_rng(0)
    for start in rng.integers(0, n - 4096, 64):
        s = int(start)
        hx = host(x[s:s + 4096])
        assert same(host(q[s:s + 4096]), port.quantize(hx, scale, 0))


def test_near_tie_inputs_and_extreme_parameters(cuda, lib, port):
    """Inputs a few ulps either side of (k + 0.5) * scale and k * scale, where a
    reciprocal multiply and a true division can round differently; scales and
    zero points outside the fast path's range."""
    from rpl_b200 import device as D
    rng = np.random.default_rng(99)
    for scale in (np.float32(0.39370078), np.float32(1.0 / 3.0), np.float32(2.3622048), np.float32(1e-3),
                  np.float32(7.0), np.float32(50.0) / np.float32(127.0)):
        k = rng.integers(-150, 150, 200_000)
        half = (k + 0.5).astype(np.float32) * scale
        whole = k.astype(np.float32) * scale
        x = np.concatenate([half, whole])
        ulps = rng.integers(-4, 5, x.size)
        x = (x.view(np.int32) + ulps).view(np.float32)
        xd = dev(x, cuda)
        for zp in (0, 3, -128, 1000):
            assert same(host(D.quantize(xd, float(scale), zp)), port.quantize(x, scale, zp))
    x = sweep_tensor(rng, (100_003,))
    xd = dev(x, cuda)
    for scale, zp in ((1e-41, 0), (3e38, 0), (1e-30, 5), (0.05, 2**31 - 1), (0.05, -2**31), (0.05, 2**30 + 7),
                      (float("inf"), 0), (0.0, 0), (-0.25, 4), (float("nan"), 0)):
        assert same(host(D.quantize(xd, scale, zp)), port.quantize(x, scale, zp)), (scale, zp)
    q = rng.integers(-128, 128, 100_003, dtype=np.int8)
    qd = dev(q, cuda)
    for scale, zp in ((0.1, 2**21 - 1), (0.1, -(2**21) + 1), (0.1, 2**21), (0.1, -(2**22)), (0.1, 2**31 - 1), (0.1, -2**31), (3e38, 7)):
        assert same(host(D.dequantize(qd, scale, zp)), port.dequantize(q, scale, zp)), (scale, zp)


def test_scale_from_a_combined_pair_is_the_single_gpu_scale(cuda, lib, port):
    """Row-sharded activations: (-min, max) pairs are max-reduced across ranks and the scale is derived
    from the combined pair.  For a few thousand absmax bit patterns that scale must be the very bits
    tensor_quantize_int8_symmetric computes (an IEEE division by 127, not a multiplication by 1/127)."""
    from rpl_b200 import device as D
    rng = np.random.default_rng(17)
    vals = np.concatenate([np.abs(rng.standard_normal(1500)).astype(np.float32) * 5,
                           rng.integers(0x00800000, 0x7F000000, 1500).astype(np.uint32).view(np.float32),
                           np.array([0.0, 1e-45, 1.1754944e-38, 127.0, 3.4028235e38], np.float32)])
    params = torch.empty(8, dtype=torch.float32, device=cuda)
    pair = torch.empty(2, dtype=torch.float32, device=cuda)
    got_direct, got_pair = [], []
    for v in vals:
        x = torch.tensor([float(v), -float(v) / 2, 0.0, float(v) / 4], device=cuda)
        D.minmax(x, params=params)
        got_direct.append(params[D.QPARAM_SCALE_SYM].clone())
        D.qparams_to_pair(params, pair)
        # what another rank with smaller extremes contributes changes nothing
        other = torch.tensor([float(v) / 8, float(v) / 3], device=cuda)
        torch.maximum(pair, other, out=pair)
        params.zero_()
        D.qparams_from_pair(pair, params)
        got_pair.append(params[D.QPARAM_SCALE_SYM].clone())
    a = torch.stack(got_direct).cpu().numpy()
    b = torch.stack(got_pair).cpu().numpy()
    want = np.array([port.scale_symmetric(np.float32(-v / 2), np.float32(v)) for v in vals], np.float32)
    assert same(a, want) and same(b, want)


@pytest.mark.parametrize("n", [4, 5, 7, 1000, 8192, 8193, 100003, 1 << 20, (1 << 21) + 2, 3500000, 4000000])
def test_one_launch_and_two_launch_per_tensor_quantize_agree(cuda, lib, port, n):
    """Tensors that fit in the registers of one resident grid are quantized by one cooperative launch that reads
    them once; the two-kernel route is the same arithmetic.  Both must give the checker's bits (sizes around the
    CTA granule, odd tails, a NaN and an outlier far from the rest included); 4000000 exceeds the one-launch limit."""
    from rpl_b200 import capi, device as D
    rng = np.random.default_rng(n)
    x = sweep_tensor(rng, n)
    if n > 10:
        x[n // 3] = np.nan
        x[n - 1] = -77.5
    wq, ws = port.quantize_symmetric(x)
    aq, asc, azp = port.quantize_asymmetric(x)
    L = capi.load()
    for onepass in (1, 0):
        prev = L.rplb_quantize_onepass(onepass)
        try:
            launches = D.launch_count()
            q, p = D.quantize_symmetric(dev(x, cuda))
            used = D.launch_count() - launches
            q2, p2 = D.quantize_asymmetric(dev(x, cuda))
            torch.cuda.synchronize()
        finally:
            L.rplb_quantize_onepass(prev)
        assert D.kernel_status(True) == 0
        assert same(host(q), wq) and same(host(p)[D.QPARAM_SCALE_SYM], ws), onepass
        assert same(host(q2), aq) and same(host(p2)[D.QPARAM_SCALE_ASYM], asc), onepass
        assert int(host(p2).view(np.int32)[D.QPARAM_ZP_ASYM]) == azp
        if onepass and n <= 3500000:
            assert used == 1                                   # one kernel, not two or three
    # back to back on one stream: the barrier's counters are left at zero
    for _ in range(3):
        q, p = D.quantize_symmetric(dev(x, cuda))
    assert same(host(q), wq)
