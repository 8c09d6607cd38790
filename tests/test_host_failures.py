"""Failures made on the host, none of which needs (or touches) a GPU: an
allocator that refuses, a communicator that cannot be set up, a corrupted
weight file, a rank that leaves between steps.  The library reports each through
its error codes, in the convention of the reference's accelerator file (one line
on stderr, a NULL result: src/rpl_gpu.c:95-111), and stays usable."""
import ctypes as C
import os
import socket
import struct
import subprocess
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def test_refusing_allocator_is_reported_not_fatal(lib):
    from rpl_b200 import capi
    seen = []

    def refuse(out, nbytes):
        seen.append(int(nbytes))
        return 2                                    # cudaErrorMemoryAllocation

    def release(ptr):
        return 0

    alloc, free = capi.ALLOC_FN(refuse), capi.FREE_FN(release)
    capi.call("rplb_set_allocator", alloc, free)
    try:
        p = C.c_void_p(123)
        rc = lib.rplb_malloc(C.byref(p), 4096)
        assert rc == 2 and not p.value and seen == [4096]
        assert b"allocator" in lib.rplb_last_error()
        # a reference-named producer: NULL result, code kept for rpl_cuda_last_error, nothing leaked or crashed
        shape = (C.c_uint32 * 2)(8, 8)
        assert not lib.tensor_create_device(2, shape)
        assert lib.rpl_cuda_last_error() == 2
        # the library's own scratch block goes through the same hook
        assert lib.rplb_scratch_reserve(None, 1 << 16) != 0
    finally:
        capi.call("rplb_set_allocator", C.cast(None, capi.ALLOC_FN), C.cast(None, capi.FREE_FN))
    with pytest.raises(capi.RplError):              # one function without the other is refused
        capi.call("rplb_set_allocator", alloc, C.cast(None, capi.FREE_FN))
    t = lib.tensor_create((2), shape, False)        # host allocations were never affected
    assert t
    lib.tensor_free(t)


def test_communicator_set_up_failure_is_an_error_code():
    """world > 1 needs NCCL: when the library cannot be loaded the create call says so
    and returns no layer.  Runs in a child process because the loader remembers its
    first attempt."""
    code = (
        "import ctypes as C, sys\n"
        "sys.path.insert(0, %r)\n"
        "from rpl_b200 import capi\n"
        "L = capi.load()\n"
        "h = C.c_void_p(7)\n"
        "ident = (C.c_char * 128)()\n"
        "rc = L.rplb_sharded_linear_create(C.byref(h), 0, 2, ident, None, 256, 64, 512, None, None, None)\n"
        "assert rc == capi.RPLB_E_COMM and not h.value, (rc, h.value)\n"
        "assert b'cannot load' in L.rplb_last_error(), L.rplb_last_error()\n"
        "assert L.rplb_nccl_unique_id(ident) == capi.RPLB_E_COMM\n"
        "rc = L.rplb_sharded_linear_create(C.byref(h), 3, 2, ident, None, 256, 64, 512, None, None, None)\n"
        "assert rc == capi.RPLB_E_BAD_ARG\n"
        "print('ok')\n" % ROOT)
    env = dict(os.environ, RPLB_NCCL_LIBRARY="/nonexistent/libnccl.so.2")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=120)
    assert out.returncode == 0 and "ok" in out.stdout, out.stdout + out.stderr


def test_sharded_create_checks_its_arguments(lib):
    from rpl_b200 import capi
    h = C.c_void_p()
    assert lib.rplb_sharded_linear_create(C.byref(h), 0, 9, None, None, 256, 64, 512, None, None, None) == capi.RPLB_E_BAD_ARG
    assert lib.rplb_sharded_linear_create(C.byref(h), 0, 1, None, None, 0, 64, 512, None, None, None) == capi.RPLB_E_BAD_ARG
    assert lib.rplb_sharded_linear_create(C.byref(h), 0, 2, None, None, 256, 24, 512, None, None, None) == capi.RPLB_E_UNSUPPORTED
    assert lib.rplb_sharded_linear_create(C.byref(h), 0, 2, None, None, 256, 64, 512, None, None, None) == capi.RPLB_E_BAD_ARG
    assert not h.value
    assert lib.rplb_sharded_linear_drain(None) == 0
    lib.rplb_sharded_linear_free(None)


def _weights_file(dims, shape, size, nch, payload=None):
    head = struct.pack("<IIf", 1, 0x38544E49, 0.0) + struct.pack("<I", dims) + struct.pack("<%dI" % dims, *shape)
    body = struct.pack("<I", size) + (payload if payload is not None else b"\1" * size)
    return head + body + struct.pack("<I", nch) + struct.pack("<%df" % nch, *([0.5] * nch))


@pytest.mark.parametrize("dims,shape,size,nch", [
    (2, (4, 4), 12, 4),        # size is not the product of the shape
    (2, (4, 6), 24, 5),        # channel count is none of the extents (and does not divide the size)
    (2, (4, 6), 24, 3),        # divides the size but is not an extent
])
def test_load_rejects_inconsistent_headers(lib, tmp_path, dims, shape, size, nch):
    p = tmp_path / "bad.rplq8"
    p.write_bytes(_weights_file(dims, shape, size, nch))
    count = C.c_uint32(5)
    assert not lib.quantized_weights_load(str(p).encode(), C.byref(count), False) and count.value == 5


def test_load_accepts_the_consistent_neighbours(lib, tmp_path):
    for shape, nch in (((4, 6), 4), ((4, 6), 6), ((4, 6), 1)):
        p = tmp_path / "good.rplq8"
        p.write_bytes(_weights_file(2, shape, 24, nch))
        count = C.c_uint32()
        got = lib.quantized_weights_load(str(p).encode(), C.byref(count), False)
        assert got and count.value == 1 and got[0].contents.channel_size == 24 // nch
        lib.per_channel_quantized_tensor_free(got[0])
        lib.rpitorch_aligned_free(C.cast(got, C.c_void_p))


# ---------------------------------------------------------------------------- a rank that leaves between steps
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _member(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    from rpl_b200.sharded import Membership, RankLeft
    store = dist.distributed_c10d._get_default_store()
    members = Membership(store, rank, world)
    steps_done, left = 0, None
    try:
        for step in range(4):
            try:
                members.check(step)                     # before anything is launched for this step
            except RankLeft as e:
                left = e.ranks
                break
            t = torch.tensor([float(rank + step)])
            dist.all_reduce(t, op=dist.ReduceOp.MAX)    # the step's exchange
            steps_done += 1
            if rank == 1 and step == 1:
                members.leave(step + 1)                 # between steps: nothing of this rank is in flight
                break
            members.arrive(step + 1)
    finally:
        np.save(os.path.join(result_dir, "m%d.npy" % rank), np.array([steps_done, -1 if left is None else left[0]]))
        if rank == 1:
            import time
            time.sleep(1.0)                             # let the other rank read the store before it goes away
        dist.destroy_process_group()


def test_a_rank_that_leaves_between_steps_is_noticed_before_the_next_launch(tmp_path):
    mp.spawn(_member, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    r0 = np.load(os.path.join(str(tmp_path), "m0.npy"))
    r1 = np.load(os.path.join(str(tmp_path), "m1.npy"))
    assert list(r1) == [2, -1]                          # rank 1 ran two steps and left
    assert list(r0) == [2, 1]                           # rank 0 ran the same two, then learned that rank 1 had gone
