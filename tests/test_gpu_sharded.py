"""The quantized Linear with rows and columns split over ranks (rplb_sharded_linear_*)
and the GEMM that takes rows still arriving from other GPUs.

One GPU: the arrival words are set before the launch (so nothing really waits), a wait that
nothing satisfies runs out by itself and is reported, and the layer with world = 1.
Two or more GPUs: a child process per GPU, NVLS off; every rank's int8 activation and scale
must be the bits one GPU computes, and so must the outputs."""
import ctypes as C
import os
import socket
import subprocess

import numpy as np
import pytest
import torch

from conftest import ROOT, bits

pytestmark = pytest.mark.gpu


def same(a, b):
    return np.array_equal(bits(np.asarray(a)), bits(np.asarray(b)))


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def _problem(M, N, K, seed):
    rng = np.random.default_rng(seed)
    xq = rng.integers(-128, 128, (M, K), dtype=np.int8)
    wq = rng.integers(-128, 128, (N, K), dtype=np.int8)
    ws = ((rng.random(N) + 0.5) * 1e-3).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    return xq, wq, ws, bias


@pytest.mark.parametrize("mnk,first,count", [((1000, 300, 256), 3, 2), ((128, 256, 128), 0, 1), ((700, 520, 784), 5, 1),
                                             ((1024, 256, 512), 0, 0), ((2048, 512, 256), 12, 4)])
@pytest.mark.parametrize("which", [3, 5])
def test_arriving_rows_with_words_already_set(cuda, lib, port, mnk, first, count, which):
    """Same bits as the plain call whatever block the walk starts from, from both kernels that can wait for rows
    (128-row tiles: one arrival word each; 256-row tiles: two)."""
    from rpl_b200 import device as D
    prev = D.gemm_backend(which)
    M, N, K = mnk
    xq, wq, ws, bias = _problem(M, N, K, M + N + K)
    sa = np.float32(0.0173)
    want = port.linear_dequant(xq, wq, sa, ws, bias, relu=True)
    blocks = (M + 127) // 128
    epoch = 0xFFFFFFF0                                     # close to the wrap: words further on count as arrived
    ready = torch.full((blocks,), epoch + 3, dtype=torch.int64, device=cuda).to(torch.int32)   # wraps to small values
    ready[first:first + count] = 0                         # local blocks are never looked at
    got = D.linear_i8_dequant_arriving(dev(xq, cuda), dev(wq, cuda), torch.tensor([sa], device=cuda), dev(ws, cuda), ready,
                                       epoch, first, count, bias=dev(bias, cuda), relu=True)
    torch.cuda.synchronize()
    D.gemm_backend(prev)
    assert D.kernel_status(True) == 0
    assert same(got.cpu().numpy(), want)


def test_arriving_rows_that_never_arrive_end_in_a_status_code(cuda, lib, port):
    """A block whose word nothing sets: the wait runs out by itself (about a second), the kernel
    returns, the status word says 5, and the next GEMM of this thread works."""
    from rpl_b200 import capi, device as D
    M, N, K = 256, 256, 128
    xq, wq, ws, bias = _problem(M, N, K, 5)
    ready = torch.zeros(2, dtype=torch.int32, device=cuda)
    a_scale = torch.tensor([0.01], device=cuda)
    D.linear_i8_dequant_arriving(dev(xq, cuda), dev(wq, cuda), a_scale, dev(ws, cuda), ready, 7, 0, 1)
    torch.cuda.synchronize()
    assert D.kernel_status(False) == 5
    prev = D.gemm_backend(3)                                # the tensor-core kernel, whatever the size
    with pytest.raises(capi.RplError):                      # refused until the caller has looked
        D.linear_i8_dequant(dev(xq, cuda), dev(wq, cuda), a_scale, dev(ws, cuda))
    assert D.kernel_status(True) == 0
    got = D.linear_i8_dequant(dev(xq, cuda), dev(wq, cuda), a_scale, dev(ws, cuda))
    D.gemm_backend(prev)
    assert same(got.cpu().numpy(), port.linear_dequant(xq, wq, np.float32(0.01), ws))
    with pytest.raises(capi.RplError):                      # K % 16 != 0: refused, not emulated
        D.linear_i8_dequant_arriving(dev(xq[:, :24].copy(), cuda), dev(wq[:, :24].copy(), cuda), a_scale, dev(ws, cuda), ready, 7, 0, 1)


@pytest.mark.parametrize("mnk", [(384, 512, 256), (100, 300, 64), (1000, 1280, 784)])
def test_row_sharded_layer_on_one_rank(cuda, lib, port, mnk):
    from rpl_b200 import device as D
    from rpl_b200.sharded import RowShardedLinear
    M, N, K = mnk
    rng = np.random.default_rng(N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    wq, ws, _ = D.quantize_per_channel(dev(W, cuda))
    layer = RowShardedLinear(wq, ws, dev(bias, cuda), n_total=N, max_rows=M, rank=0, world=1)
    assert (layer.col_begin, layer.col_count) == (0, N) and layer.rows(M) == (0, M)
    hq, hs = port.quantize_symmetric(x)
    hwq, hws, _ = port.quantize_per_channel(W, N)
    want = port.linear_dequant(hq, hwq, hs, hws, bias, relu=False)
    for _ in range(2):
        out = layer.forward(dev(x, cuda), M)
        torch.cuda.synchronize()
        xq, scale = layer.activation(M)
        assert same(xq.cpu().numpy(), hq) and same(scale.cpu().numpy()[0], hs)
        assert same(out.cpu().numpy(), want)
    full = layer.gather(out, M)
    assert torch.equal(full, out)
    # the forward pass in its two halves (what a caller does to put a timing event between them)
    halves = torch.zeros((M, N), device=cuda)
    layer.quantize(dev(x, cuda), M)
    layer.gemm(M, halves)
    torch.cuda.synchronize()
    assert torch.equal(halves, out)
    # host buffers through the pipelined entry point, two calls in flight
    xh = torch.from_numpy(x).pin_memory()
    outs = [torch.empty((M, N), dtype=torch.float32).pin_memory() for _ in range(3)]
    for o in outs:
        layer.submit_host(xh, M, o, row_blocks=3)
    layer.drain()
    for o in outs:
        assert same(o.numpy(), want)
    with pytest.raises(Exception):
        layer.forward(dev(x, cuda), M + 1)                  # more rows than the layer was created for
    layer.close()
    assert D.kernel_status(True) == 0


@pytest.mark.parametrize("which", [3, 5])
def test_arriving_rows_seeded_random_shapes(cuda, lib, port, which):
    """Random shapes and random local ranges (odd first blocks, ranges that end in the ragged last block) through
    both kernels that can wait for rows; every word already set, so nothing waits and the result must not depend
    on where the walk starts."""
    from rpl_b200 import device as D
    prev = D.gemm_backend(which)
    try:
        rng = np.random.default_rng(2718 + which)
        for _ in range(10):
            M, N, K = int(rng.integers(1, 2500)), int(rng.integers(1, 700)), 16 * int(rng.integers(1, 40))
            xq, wq, ws, bias = _problem(M, N, K, M * 7 + N)
            sa = np.float32(0.0173)
            blocks = (M + 127) // 128
            first = int(rng.integers(0, blocks))
            count = int(rng.integers(0, blocks - first + 1))
            epoch = int(rng.integers(1, 1 << 31))
            ready = torch.full((blocks,), epoch, dtype=torch.int64, device=cuda).to(torch.int32)
            ready[first:first + count] = 0                     # local blocks are never looked at
            got = D.linear_i8_dequant_arriving(dev(xq, cuda), dev(wq, cuda), torch.tensor([sa], device=cuda), dev(ws, cuda), ready,
                                               epoch, first, count, bias=dev(bias, cuda), relu=False)
            torch.cuda.synchronize()
            assert D.kernel_status(True) == 0, (which, M, N, K, first, count)
            assert same(got.cpu().numpy(), port.linear_dequant(xq, wq, sa, ws, bias, relu=False)), (which, M, N, K, first, count)
    finally:
        D.gemm_backend(prev)


def test_host_pipeline_seeded_random_shapes(cuda, lib, port):
    """The host-buffer entry point with random row counts and row-block counts (1 to 16), calls in flight reusing
    the two slots, on a layer created once for the largest."""
    from rpl_b200 import device as D
    from rpl_b200.sharded import RowShardedLinear
    rng = np.random.default_rng(1618)
    N, K, max_rows = 520, 256, 3000
    W = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    wq, ws, _ = D.quantize_per_channel(dev(W, cuda))
    hwq, hws, _ = port.quantize_per_channel(W, N)
    layer = RowShardedLinear(wq, ws, dev(bias, cuda), n_total=N, max_rows=max_rows, rank=0, world=1)
    pending = []
    for _ in range(8):
        M = int(rng.integers(1, max_rows + 1))
        x = (rng.standard_normal((M, K)) * float(rng.choice([0.1, 1.0, 9.0]))).astype(np.float32)
        xh = torch.from_numpy(x).pin_memory()
        o = torch.full((M, N), -7.0, dtype=torch.float32).pin_memory()
        layer.submit_host(xh, M, o, relu=True, row_blocks=int(rng.integers(1, 17)))
        pending.append((x, xh, o))
    layer.drain()
    for x, _, o in pending:
        hq, hs = port.quantize_symmetric(x)
        assert same(o.numpy(), port.linear_dequant(hq, hwq, hs, hws, bias, relu=True)), x.shape
    layer.close()
    assert D.kernel_status(True) == 0


# ---------------------------------------------------------------------------- two or more GPUs
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port_no, result_dir):
    import datetime

    import torch.distributed as dist

    from oracle.loader import Port
    from rpl_b200 import device as D
    from rpl_b200.sharded import RowShardedLinear
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port_no), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev_ = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    try:
        cpu = Port()
        n_total, K, max_rows = 1024 + 256 * world, 256, 1100
        rng = np.random.default_rng(91)                                   # same stream on every rank
        W = (rng.standard_normal((n_total, K)) * 0.05).astype(np.float32)
        bias = rng.standard_normal(n_total).astype(np.float32)
        hwq, hws, _ = cpu.quantize_per_channel(W, n_total)
        layer = None
        for M, scale in ((1100, 1.0), (1100, 3.0), (640, 0.5), (100, 2.0)):   # the buffers are reused; ragged and tiny M
            x = (rng.standard_normal((M, K)) * scale).astype(np.float32)
            if layer is None:
                b, c = RowShardedLinearColumns(n_total, world, rank)
                wq, ws, _ = D.quantize_per_channel(torch.from_numpy(W[b:b + c]).to(dev_))
                layer = RowShardedLinear(wq, ws, torch.from_numpy(bias[b:b + c]).to(dev_), n_total=n_total, max_rows=max_rows,
                                         rank=rank, world=world)
            r0, rc = layer.rows(M)
            x_local = torch.from_numpy(x[r0:r0 + rc]).to(dev_) if rc else torch.empty((0, K), device=dev_)
            out = layer.forward(x_local, M, relu=True)
            torch.cuda.synchronize()
            assert D.kernel_status(True) == 0
            hq, hs = cpu.quantize_symmetric(x)
            xq, a_scale = layer.activation(M)
            assert np.array_equal(xq.cpu().numpy(), hq), "int8 activation differs on rank %d, M %d" % (rank, M)
            assert np.float32(a_scale.item()) == hs
            b, c = layer.col_begin, layer.col_count
            want = cpu.linear_dequant(hq, hwq[b:b + c], hs, hws[b:b + c], bias[b:b + c], relu=True)
            assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32)), "rank %d, M %d" % (rank, M)
            full = layer.gather(out, M)
            torch.cuda.synchronize()
            want_full = cpu.linear_dequant(hq, hwq, hs, hws, bias, relu=True)
            assert np.array_equal(full.cpu().numpy().view(np.uint32), want_full.view(np.uint32))
            # the same through host buffers, two calls in flight
            xh = torch.from_numpy(np.ascontiguousarray(x[r0:r0 + rc])).pin_memory() if rc else torch.empty((1, K)).pin_memory()
            outs = [torch.empty((M, c), dtype=torch.float32).pin_memory() for _ in range(2)]
            for o in outs:
                layer.submit_host(xh, M, o, relu=True, row_blocks=4)
            layer.drain()
            for o in outs:
                assert np.array_equal(o.numpy().view(np.uint32), want.view(np.uint32)), "host path, rank %d, M %d" % (rank, M)
        dist.barrier()
        layer.close()
        # an uneven column split (in proportion to 1, 2, 3 ...: what a caller does for GPUs of unequal speed)
        from rpl_b200.sharded import weighted_column_counts
        counts = weighted_column_counts(n_total, [1.0 + r for r in range(world)])
        b, c = sum(counts[:rank]), counts[rank]
        wq, ws, _ = D.quantize_per_channel(torch.from_numpy(W[b:b + c]).to(dev_))
        layer = RowShardedLinear(wq, ws, torch.from_numpy(bias[b:b + c]).to(dev_), n_total=n_total, max_rows=max_rows,
                                 rank=rank, world=world, column_counts=counts)
        assert (layer.col_begin, layer.col_count) == (b, c)
        # route 1: the rows travel by stores from a kernel; kernel 5: 256-row tiles, two arrival words per tile
        drawn = [(int(rng.integers(1, max_rows + 1)), int(rng.integers(0, 2)), int(rng.choice([0, 3, 5]))) for _ in range(6)]
        for M, route, kernel in [(900, 0, 0), (1100, 1, 5), (640, 1, 0), (900, 0, 5)] + drawn:   # then six drawn from the shared seed
            layer.transfer(route)
            D.gemm_backend(kernel)
            x = rng.standard_normal((M, K)).astype(np.float32)
            r0, rc = layer.rows(M)
            out = layer.forward(torch.from_numpy(np.ascontiguousarray(x[r0:r0 + rc])).to(dev_), M)
            full = layer.gather(out, M)
            torch.cuda.synchronize()
            hq, hs = cpu.quantize_symmetric(x)
            xq, _ = layer.activation(M)
            assert np.array_equal(xq.cpu().numpy(), hq), "int8 activation, route %d, rank %d" % (route, rank)
            want_full = cpu.linear_dequant(hq, hwq, hs, hws, bias, relu=False)
            assert np.array_equal(out.cpu().numpy().view(np.uint32), want_full[:, b:b + c].view(np.uint32)), "uneven split, rank %d" % rank
            assert np.array_equal(full.cpu().numpy().view(np.uint32), want_full.view(np.uint32)), "gather with an uneven split, rank %d" % rank
            assert D.kernel_status(True) == 0
        D.gemm_backend(0)
        dist.barrier()
        layer.close()
        # two layers in a chain, each with its own communicator: column blocks of the first are gathered, every
        # rank takes its rows of the result as its share of the second layer's input (with four ranks the last one
        # owns no column of the second layer and still quantizes and sends its rows)
        n2 = 768
        W2 = (rng.standard_normal((n2, n_total)) * 0.05).astype(np.float32)
        hw2q, hw2s, _ = cpu.quantize_per_channel(W2, n2)
        b1, c1 = RowShardedLinearColumns(n_total, world, rank)
        w1q, w1s, _ = D.quantize_per_channel(torch.from_numpy(W[b1:b1 + c1]).to(dev_))
        first = RowShardedLinear(w1q, w1s, torch.from_numpy(bias[b1:b1 + c1]).to(dev_), n_total=n_total, max_rows=max_rows,
                                 rank=rank, world=world)
        b2, c2 = RowShardedLinearColumns(n2, world, rank)
        if c2:
            w2q, w2s, _ = D.quantize_per_channel(torch.from_numpy(W2[b2:b2 + c2]).to(dev_))
        else:
            w2q, w2s = torch.empty((0, n_total), dtype=torch.int8, device=dev_), torch.empty(0, device=dev_)
        second = RowShardedLinear(w2q, w2s, None, n_total=n2, max_rows=max_rows, rank=rank, world=world)
        for M in (1000, 333):
            x = rng.standard_normal((M, K)).astype(np.float32)
            r0, rc = first.rows(M)
            h_block = first.forward(torch.from_numpy(np.ascontiguousarray(x[r0:r0 + rc])).to(dev_), M, relu=True)
            h_full = first.gather(h_block, M)
            r0b, rcb = second.rows(M)
            y_block = second.forward(h_full[r0b:r0b + rcb].contiguous(), M)
            y_full = second.gather(y_block, M)
            torch.cuda.synchronize()
            hq, hs = cpu.quantize_symmetric(x)
            want_h = cpu.linear_dequant(hq, hwq, hs, hws, bias, relu=True)
            h2q, h2s = cpu.quantize_symmetric(want_h)
            want_y = cpu.linear_dequant(h2q, hw2q, h2s, hw2s, None, relu=False)
            assert np.array_equal(h_full.cpu().numpy().view(np.uint32), want_h.view(np.uint32)), "chain, first layer, rank %d" % rank
            assert np.array_equal(y_full.cpu().numpy().view(np.uint32), want_y.view(np.uint32)), "chain, second layer, rank %d" % rank
            assert D.kernel_status(True) == 0
        dist.barrier()
        second.close()
        first.close()
        with open(os.path.join(result_dir, "ok%d" % rank), "w") as f:
            f.write("ok")
    finally:
        dist.destroy_process_group()


def RowShardedLinearColumns(n_total, world, rank):
    from rpl_b200.sharded import shard_range
    return shard_range(n_total, world, rank, 256)


def test_rows_and_columns_split_over_gpus(cuda, lib, tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two or more GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(os.path.join(str(tmp_path), "ok%d" % r)) for r in range(world))


def test_c_program_runs_the_sharded_layer(cuda, lib, tmp_path):
    """tests/c/sharded_check.c: a C host, one process per GPU (as many as there are, up to 4),
    only rplb_* calls; it checks slabs of a config-5-shaped GEMM against plain C loops."""
    from rpl_b200 import capi
    exe = str(tmp_path / "sharded_check")
    libdir = os.path.dirname(capi.LIB_PATH)
    cmd = ["/usr/bin/gcc", "-std=c11", "-O2", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "c", "sharded_check.c"), "-o", exe, "-L", libdir, "-lrpl", "-lm", "-Wl,-rpath," + libdir]
    out = subprocess.run(cmd, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    world = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([exe, str(world)], capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0 and "sharded_check: OK" in out.stdout, out.stdout + out.stderr
