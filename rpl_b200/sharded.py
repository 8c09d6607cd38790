"""Column-parallel (N-split) quantized Linear over one process per GPU.

The INT8 GEMM shards over output columns: rank r owns rows
``[begin, begin+count)`` of the ``[N, K]`` weight (with their per-channel
scales and bias entries), holds the whole int8 activation, and produces the
matching column block of the output.  Nothing is exchanged inside the GEMM.
``torch.distributed`` is used for the two optional exchange steps around it:
one max-all-reduce of a scalar when the activation itself is row-sharded, and
an all-gather of fp32 column blocks when a consumer needs the whole matrix.
"""
import torch
import torch.distributed as dist


def shard_range(n, world, rank, align=256):
    """(begin, count) of rank's column block; mirrors ``rplb_shard_range``.

    Blocks are contiguous, in rank order, multiples of ``align`` columns (the
    tensor-core tile width) except possibly the last non-empty one.
    """
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad world/rank")
    align = max(int(align), 1)
    units = (n + align - 1) // align
    base, extra = divmod(units, world)
    u0 = rank * base + min(rank, extra)
    u1 = u0 + base + (1 if rank < extra else 0)
    b, e = min(u0 * align, n), min(u1 * align, n)
    return (b, e - b)


def gather_columns(block, n_total, world=None, group=None, align=256):
    """All-gather the fp32 column blocks ``[M, count_r]`` into ``[M, n_total]``.

    Works on any backend (NCCL on GPUs, gloo on CPU).  Ragged blocks are padded
    to the widest block for the collective and trimmed while unpacking.
    """
    world = world if world is not None else dist.get_world_size(group)
    M = block.shape[0]
    counts = [shard_range(n_total, world, r, align)[1] for r in range(world)]
    widest = max(counts) if counts else 0
    send = block
    if block.shape[1] != widest:
        send = block.new_zeros((M, widest))
        send[:, : block.shape[1]] = block
    send = send.contiguous()
    recv = [torch.empty_like(send) for _ in range(world)]
    dist.all_gather(recv, send, group=group)
    out = block.new_empty((M, n_total))
    for r in range(world):
        b, c = shard_range(n_total, world, r, align)
        if c:
            out[:, b:b + c] = recv[r][:, :c]
    return out


def global_absmax_scale(local_absmax, group=None):
    """Per-tensor symmetric scale of an activation whose rows are spread over
    ranks: max-all-reduce of one float, then absmax / 127 in fp32 (the same
    division the single-device reduction performs)."""
    t = local_absmax.clone()
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t / 127.0
