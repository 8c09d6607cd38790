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


# ---------------------------------------------------------------------------- rows of the activation split over ranks
def _rows_worker(rank, world, port, M, result_dir):
    """The row-sharded protocol of rplb_sharded_linear_forward with the CPU checker standing in for the kernels:
    local min/max, max-all-reduce of (-min, max), scale from the combined pair, local quantize, exchange of the
    int8 rows.  Every rank must end up with the int8 activation and scale a single rank computes."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle.loader import Port
        from rpl_b200.sharded import shard_range
        P = Port()
        K = 48
        x = (np.random.default_rng(M).standard_normal((M, K)) * 2.5).astype(np.float32)     # same on every rank
        r0, rc = shard_range(M, world, rank, 128)
        mine = x[r0:r0 + rc]
        lo, hi = (P.minmax_seeded(mine) if rc else (np.float32(np.inf), np.float32(-np.inf)))
        pair = torch.tensor([-float(lo), float(hi)], dtype=torch.float32)
        dist.all_reduce(pair, op=dist.ReduceOp.MAX)
        scale = P.scale_symmetric(np.float32(-pair[0].item()), np.float32(pair[1].item()))
        q_mine = P.quantize(mine, scale, 0) if rc else np.zeros((0, K), np.int8)
        # exchange: every rank places its rows at their offset (the peer copies of the GPU path)
        pieces = [None] * world
        dist.all_gather_object(pieces, (r0, q_mine))
        full = np.zeros((M, K), np.int8)
        covered = 0
        for b, rows in pieces:
            full[b:b + rows.shape[0]] = rows
            covered += rows.shape[0]
        want_q, want_s = P.quantize_symmetric(x)
        ok = covered == M and want_s == scale and np.array_equal(full, want_q)
        # rows are dealt in multiples of 128 (one arrival word per block), contiguous and in rank order
        ok = ok and (rc == 0 or r0 % 128 == 0) and (rc % 128 == 0 or r0 + rc == M)
        np.save(os.path.join(result_dir, "rows%d.npy" % rank), np.array([ok]))
    finally:
        dist.destroy_process_group()


def _run_rows(M, tmp_path):
    world = 2
    mp.spawn(_rows_worker, args=(world, _free_port(), M, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert np.load(os.path.join(str(tmp_path), "rows%d.npy" % r)).all(), "rank %d" % r


def test_row_sharded_quantize_even(tmp_path):
    _run_rows(1024, tmp_path)


def test_row_sharded_quantize_ragged(tmp_path):
    _run_rows(1100, tmp_path)          # 9 blocks of 128 rows: 5 and 4, the last one ragged


def test_row_sharded_quantize_one_rank_without_rows(tmp_path):
    _run_rows(100, tmp_path)           # a single block: rank 1 contributes the neutral pair (-inf, -inf)
