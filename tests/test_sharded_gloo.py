"""The N>1 host logic on CPU: two gloo ranks split the output columns, each
computes its block (with the CPU checker standing in for the GPU kernels) and
the all-gather reassembles the full matrix; a scalar max-all-reduce gives the
per-tensor scale of a row-sharded activation."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, n_total, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle.loader import Port
        from rpl_b200.sharded import ShardedQuantizedLinear, gather_columns, global_absmax_scale, shard_range
        P = Port()
        rng = np.random.default_rng(123)                      # same data on every rank
        M, K = 37, 64
        x = rng.standard_normal((M, K)).astype(np.float32)
        w = (rng.standard_normal((n_total, K)) * 0.02).astype(np.float32)
        xq, xs = P.quantize_symmetric(x)
        wq, wsc, _ = P.quantize_per_channel(w, n_total)
        b, c = shard_range(n_total, world, rank, 256)
        block = P.linear_dequant(xq, wq[b:b + c], xs, wsc[b:b + c]) if c else np.zeros((M, 0), np.float32)
        full = gather_columns(torch.from_numpy(block), n_total, world)
        want = P.linear_dequant(xq, wq, xs, wsc)
        ok_gather = np.array_equal(full.numpy().view(np.uint32), want.view(np.uint32))
        layer = ShardedQuantizedLinear(None, None, None, n_total=n_total, rank=rank, world=world)
        ok_layer = torch.equal(layer.gather(torch.from_numpy(block)), full)
        # row-sharded activation: each rank sees half the rows, the scale must be the global one
        rows = np.array_split(np.arange(M), world)[rank]
        mn, mx = P.minmax_seeded(x[rows])
        local = torch.tensor([max(abs(float(mn)), abs(float(mx)))], dtype=torch.float32)
        scale = global_absmax_scale(local)
        ok_scale = np.float32(scale.item()) == xs
        np.save(os.path.join(result_dir, "r%d.npy" % rank), np.array([ok_gather, ok_layer, ok_scale]))
    finally:
        dist.destroy_process_group()


def _run(n_total, tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), n_total, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert np.load(os.path.join(str(tmp_path), "r%d.npy" % r)).all(), "rank %d" % r


def test_two_ranks_even_split(tmp_path):
    _run(1024, tmp_path)


def test_two_ranks_ragged_split(tmp_path):
    _run(700, tmp_path)            # blocks of 512 and 188 columns: padded gather, trimmed unpack


def test_two_ranks_one_empty(tmp_path):
    _run(200, tmp_path)            # a single 256-column unit: rank 1 owns nothing
