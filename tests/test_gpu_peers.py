"""The GEMM whose epilogue also stores into other ranks' buffers
(rplb_linear_i8_dequant_f32_peers).

On one GPU the further destinations are other buffers of the same device, which
exercises the kernel's stores; with two or more GPUs a child process per GPU
shares its output over rplb_ipc_export / rplb_ipc_open and every rank ends up
with the whole matrix without a gather pass.
"""
import ctypes as C
import os
import socket

import numpy as np
import pytest
import torch

from conftest import bits

pytestmark = pytest.mark.gpu


def same(a, b):
    return np.array_equal(bits(np.asarray(a)), bits(np.asarray(b)))


@pytest.mark.parametrize("mnk,relu,round_up", [((300, 512, 256), False, False), ((129, 250, 64), True, False), ((128, 256, 128), False, False),
                                              ((129, 250, 64), True, True), ((200, 301, 128), False, True)])
def test_extra_destinations_on_one_device(cuda, lib, port, mnk, relu, round_up):
    from rpl_b200 import capi, device as D
    from rpl_b200.sharded import _RawBlock
    M, N, K = mnk
    n_total, begin = N + 256 + 8, 256                 # this "rank" owns columns [256, 256 + N) of a wider matrix
    if round_up:
        # a row stride of whole 16-byte pieces under a block whose width is not: tensor stores for the whole
        # chunks, the ragged last chunk from registers, the staged copy for the peers either way
        n_total = (n_total + 3) // 4 * 4
    rng = np.random.default_rng(61)
    xq = rng.integers(-128, 128, (M, K), dtype=np.int8)
    wq = rng.integers(-128, 128, (N, K), dtype=np.int8)
    ws = (rng.random(N, dtype=np.float32) + 0.5) * 1e-2
    bias = rng.standard_normal(N).astype(np.float32)
    sa = np.float32(0.037)
    want = port.linear_dequant(xq, wq, sa, ws, bias, relu=relu)

    x, w = torch.from_numpy(xq).to(cuda), torch.from_numpy(wq).to(cuda)
    a_scale = torch.tensor([sa], device=cuda)
    local = torch.full((M, n_total), -7.0, device=cuda)
    other = torch.full((M, n_total), -7.0, device=cuda)
    raw = C.c_void_p()
    capi.call("rplb_malloc", C.byref(raw), M * n_total * 4)
    try:
        third = torch.as_tensor(_RawBlock(raw.value, (M, n_total)), device=cuda)     # the view PeerOutput uses
        assert third.data_ptr() == raw.value and third.shape == (M, n_total)
        third.fill_(-7.0)
        peers = [other.data_ptr() + begin * 4, raw.value + begin * 4]
        D.linear_i8_dequant_peers(x, w, a_scale, torch.from_numpy(ws).to(cuda), local[:, begin:begin + N], peers,
                                  bias=torch.from_numpy(bias).to(cuda), relu=relu)
        torch.cuda.synchronize()
        for buf in (local, other, third):
            got = buf.cpu().numpy()
            assert same(got[:, begin:begin + N], want)
            assert (got[:, :begin] == -7.0).all() and (got[:, begin + N:] == -7.0).all()   # nothing outside the block
        del third
    finally:
        capi.call("rplb_free", raw.value)
    assert D.kernel_status(True) == 0


def test_peers_call_refuses_what_it_cannot_do(cuda, lib):
    from rpl_b200 import capi, device as D
    x = torch.zeros((16, 24), dtype=torch.int8, device=cuda)              # K = 24: not a multiple of 16
    w = torch.zeros((16, 24), dtype=torch.int8, device=cuda)
    out = torch.zeros((16, 16), device=cuda)
    other = torch.zeros((16, 16), device=cuda)
    s = torch.ones(1, device=cuda)
    with pytest.raises(capi.RplError):
        D.linear_i8_dequant_peers(x, w, s, torch.ones(16, device=cuda), out, [other.data_ptr()])
    with pytest.raises(capi.RplError):
        D.linear_i8_dequant_peers(x[:, :16].contiguous(), w[:, :16].contiguous(), s, torch.ones(16, device=cuda), out,
                                  [other.data_ptr()] * 8)                 # more than 7 peers


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port_no, result_dir):
    import torch.distributed as dist

    from oracle.loader import Port
    from rpl_b200 import device as D
    from rpl_b200.sharded import PeerOutput, ShardedQuantizedLinear, shard_range
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port_no), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=60))
    try:
        M, K, n_total = 384, 256, 1280 + 256 * world
        rng = np.random.default_rng(71)                                     # same stream on every rank
        x = rng.standard_normal((M, K)).astype(np.float32)
        W = (rng.standard_normal((n_total, K)) * 0.05).astype(np.float32)
        bias = rng.standard_normal(n_total).astype(np.float32)
        begin, count = shard_range(n_total, world, rank, 256)
        wq, ws, _ = D.quantize_per_channel(torch.from_numpy(W[begin:begin + count]).to(dev))
        layer = ShardedQuantizedLinear(wq, ws, torch.from_numpy(bias[begin:begin + count]).to(dev), n_total=n_total,
                                       rank=rank, world=world)
        shared = PeerOutput(M, n_total, dev)
        xd = torch.from_numpy(x).to(dev)
        for scale in (1.0, 3.0):                                            # twice: the buffers are reused
            full = layer.forward_gathered(xd * scale, shared)
            torch.cuda.synchronize()
            got = full.cpu().numpy()
            cpu = Port()
            xq, sa = cpu.quantize_symmetric((x * np.float32(scale)).astype(np.float32))
            wq_all, ws_all, _ = cpu.quantize_per_channel(W, n_total)
            want = cpu.linear_dequant(xq, wq_all, sa, ws_all, bias, relu=False)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), "rank %d, scale %g" % (rank, scale)
        assert D.kernel_status(True) == 0
        shared.close()
        with open(os.path.join(result_dir, "ok%d" % rank), "w") as f:
            f.write("ok")
    finally:
        dist.destroy_process_group()


def test_every_rank_gets_the_whole_output_without_a_gather(cuda, lib, tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two or more GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(os.path.join(str(tmp_path), "ok%d" % r)) for r in range(world))
