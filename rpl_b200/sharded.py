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
    # One [world * M, widest] landing buffer: the collective writes it in place,
    # with no per-rank list to flatten.
    recv = send.new_empty((world * M, widest))
    dist.all_gather_into_tensor(recv, send, group=group)
    recv = recv.view(world, M, widest)
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
    # Tensor / tensor is an IEEE division on every backend; tensor / python scalar is
    # turned into a multiplication by the rounded reciprocal on CUDA, which differs in the last bit.
    return t / torch.full_like(t, 127.0)


class RankLeft(RuntimeError):
    """Raised before a step is launched when other ranks have announced that they are gone."""

    def __init__(self, ranks, step):
        super().__init__("rank(s) %s left before step %d" % (ranks, step))
        self.ranks, self.step = list(ranks), step


class Membership:
    """Who is still taking part, kept in the process group's key-value store.

    A step of the sharded layer contains collectives, so a rank that has gone must be
    noticed on the host, before the next launch: nothing may wait for it on the GPU.
    A rank calls ``arrive(step)`` when it is ready for a step and ``leave(step)``
    instead when it stops (only between steps, with none of its kernels or
    collectives in flight); ``check(step)`` waits until every other rank has done one
    or the other and raises ``RankLeft`` naming those that left.
    """

    def __init__(self, store, rank, world, timeout_s=20.0):
        self.store, self.rank, self.world, self.timeout_s = store, rank, world, timeout_s

    def _key(self, rank, step):
        return "rplb/member/%d/%d" % (step, rank)

    def arrive(self, step):
        self.store.set(self._key(self.rank, step), "here")

    def leave(self, step):
        self.store.set(self._key(self.rank, step), "left")

    def check(self, step):
        import datetime
        if step == 0:
            return
        others = [r for r in range(self.world) if r != self.rank]
        self.store.wait([self._key(r, step) for r in others], datetime.timedelta(seconds=self.timeout_s))
        gone = [r for r in others if self.store.get(self._key(r, step)) == b"left"]
        if gone:
            raise RankLeft(gone, step)


class ShardedQuantizedLinear:
    """One rank's column block of a quantized Linear: ``y[:, b:b+c] = x . W[b:b+c, :]^T``.

    Holds the int8 weight rows of this rank with their per-channel scales (and
    an fp32 bias slice) in device memory.  ``forward`` quantizes the fp32
    activation per tensor (symmetric) and runs the INT8 GEMM with the fused
    fp32 epilogue; both are ``librpl.so`` kernels.  Mirrors the shapes of the
    reference's ``linear_forward`` (weights ``[out, in]``, ``x . W^T + b``,
    src/rpl_nn.c:55-77) on the INT8 path of ``linear_int8``.
    """

    def __init__(self, wq, w_scales, bias=None, n_total=None, rank=0, world=1, relu=False, group=None,
                 shard_reduction=True):
        self.wq, self.w_scales, self.bias = wq, w_scales, bias
        self.rank, self.world, self.group = rank, world, group
        self.shard_reduction = shard_reduction
        self.n_total = int(n_total if n_total is not None else wq.shape[0])
        self.relu = relu
        self._xq = None
        self._params = None
        self._pair = None
        self._dev_in = None
        self._dev_out = None
        self._copy_stream = None
        self._side = None

    @classmethod
    def from_fp32(cls, w_shard, bias=None, **kw):
        from . import device as D
        wq, scales, _ = D.quantize_per_channel(w_shard)
        return cls(wq, scales, bias, **kw)

    def quantize_activation(self, x):
        """Per-tensor symmetric quantization of the fp32 activation ``[M,K]``.

        Returns ``(xq, a_scale)``: the int8 activation and its scale as a
        one-element device tensor.  With more than one rank (every rank holds the
        whole activation) the min/max pass is split by rows: each rank reduces its
        row block, one scalar max-all-reduce makes the result global, and the
        quantize pass runs locally with that scale.
        """
        from . import device as D
        M, K = x.shape
        if self._xq is None or self._xq.shape != x.shape or self._xq.device != x.device:
            self._xq = torch.empty((M, K), dtype=torch.int8, device=x.device)
            self._params = torch.empty(8, dtype=torch.float32, device=x.device)
        a_scale = self._params[D.QPARAM_SCALE_SYM:D.QPARAM_SCALE_SYM + 1]
        if self.world > 1 and self.shard_reduction and dist.is_initialized():
            r0, rc = shard_range(M, self.world, self.rank, 1)
            self._reduce_scale(x[r0:r0 + rc])
            D.quantize_dev(x, a_scale, out=self._xq)
        else:
            D.quantize_symmetric(x, out=self._xq, params=self._params)
        return self._xq, a_scale

    def gemm(self, xq, a_scale, out=None, row_chunks=None, after_chunk=None):
        """INT8 GEMM of the quantized activation against this rank's weight rows,
        fused fp32 epilogue; returns the column block ``[M, count]``.

        ``row_chunks`` splits the GEMM into that many row blocks (same results);
        ``after_chunk(i, r0, r1)`` is called after block i has been launched.
        """
        from . import device as D
        M = xq.shape[0]
        count = self.wq.shape[0]
        if out is None:
            out = torch.empty((M, count), dtype=torch.float32, device=xq.device)
        if not row_chunks or row_chunks <= 1:
            D.linear_i8_dequant(xq, self.wq, a_scale, self.w_scales, self.bias, self.relu, out=out)
            return out
        step = (M + row_chunks - 1) // row_chunks
        step = (step + 127) // 128 * 128
        for i, r0 in enumerate(range(0, M, step)):
            r1 = min(M, r0 + step)
            D.linear_i8_dequant(xq[r0:r1], self.wq, a_scale, self.w_scales, self.bias, self.relu, out=out[r0:r1])
            if after_chunk is not None:
                after_chunk(i, r0, r1)
        return out

    def forward(self, x, out=None, row_chunks=None, after_chunk=None):
        """x: fp32 CUDA [M,K] -> fp32 column block [M, count] (quantize, then GEMM)."""
        xq, a_scale = self.quantize_activation(x)
        return self.gemm(xq, a_scale, out=out, row_chunks=row_chunks, after_chunk=after_chunk)

    def activation_scale(self, x):
        """The per-tensor symmetric scale of ``x`` (one-element device tensor) without
        quantizing: the min/max pass only, row-sharded with one scalar all-reduce when
        there is more than one rank."""
        from . import device as D
        M, K = x.shape
        if self._xq is None or self._xq.shape != x.shape or self._xq.device != x.device:
            self._xq = torch.empty((M, K), dtype=torch.int8, device=x.device)
            self._params = torch.empty(8, dtype=torch.float32, device=x.device)
        a_scale = self._params[D.QPARAM_SCALE_SYM:D.QPARAM_SCALE_SYM + 1]
        if self.world > 1 and self.shard_reduction and dist.is_initialized():
            r0, rc = shard_range(M, self.world, self.rank, 1)
            self._reduce_scale(x[r0:r0 + rc])
        else:
            D.minmax(x, params=self._params)
        return a_scale

    def _reduce_scale(self, rows):
        """min/max of this rank's rows, a max-all-reduce of (-min, max), and the parameters
        from the combined pair: all arithmetic stays in the library's kernels (the division
        by 127 is the IEEE one of the single-GPU reduction)."""
        from . import device as D
        D.minmax(rows, params=self._params)
        if self._pair is None:
            self._pair = torch.empty(2, dtype=torch.float32, device=rows.device)
        D.qparams_to_pair(self._params, self._pair)
        dist.all_reduce(self._pair, op=dist.ReduceOp.MAX, group=self.group)
        D.qparams_from_pair(self._pair, self._params)

    def forward_overlapped(self, x, out=None, row_chunks=4, gemm_events=None):
        """Same result as ``forward``; the quantize pass is pipelined under the GEMM.

        The scale needs every element, so the min/max pass runs first.  After that
        the quantize kernel (HBM-bound) and the GEMM (tensor-bound) want different
        resources: the activation is quantized in ``row_chunks`` row blocks on a
        second stream and the GEMM of a block starts as soon as that block is ready.
        ``gemm_events``, if given, receives a (start, end) CUDA event pair per GEMM launch.
        """
        from . import device as D
        M, K = x.shape
        count = self.wq.shape[0]
        if out is None:
            out = torch.empty((M, count), dtype=torch.float32, device=x.device)
        main = torch.cuda.current_stream(x.device)
        if self._side is None:
            self._side = torch.cuda.Stream(device=x.device)
        a_scale = self.activation_scale(x)
        ready = torch.cuda.Event()
        ready.record(main)                      # scale known; every earlier reader of _xq is done
        self._side.wait_event(ready)
        step = (M + row_chunks - 1) // row_chunks
        step = (step + 127) // 128 * 128
        blocks = [(r0, min(M, r0 + step)) for r0 in range(0, M, step)]
        blocks.reverse()                        # the end of x is what the min/max pass left in L2
        done = []
        with torch.cuda.stream(self._side):
            for r0, r1 in blocks:
                D.quantize_dev(x[r0:r1], a_scale, out=self._xq[r0:r1])
                ev = torch.cuda.Event()
                ev.record(self._side)
                done.append(ev)
        for (r0, r1), ev in zip(blocks, done):
            main.wait_event(ev)
            if gemm_events is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(main)
            D.linear_i8_dequant(self._xq[r0:r1], self.wq, a_scale, self.w_scales, self.bias, self.relu, out=out[r0:r1])
            if gemm_events is not None:
                e1.record(main)
                gemm_events.append((e0, e1))
        return out

    def forward_host(self, x_host, out_host, row_chunks=8):
        """Host buffers in, host buffers out (page-locked for full PCIe speed).

        The activation is copied to the device, quantized, and the GEMM runs in
        row blocks; each finished block is copied back on a second stream while
        the next one computes.  Returns after ``out_host`` is complete.
        """
        M, K = x_host.shape
        dev = self.wq.device
        if self._dev_in is None or self._dev_in.shape != x_host.shape:
            self._dev_in = torch.empty((M, K), dtype=torch.float32, device=dev)
            self._dev_out = torch.empty((M, self.wq.shape[0]), dtype=torch.float32, device=dev)
            self._copy_stream = torch.cuda.Stream(device=dev)
        main = torch.cuda.current_stream(dev)
        self._copy_stream.wait_stream(main)          # earlier readers of _dev_out are done
        self._dev_in.copy_(x_host, non_blocking=True)

        def ship(i, r0, r1):
            ev = torch.cuda.Event()
            ev.record(main)
            self._copy_stream.wait_event(ev)
            with torch.cuda.stream(self._copy_stream):
                out_host[r0:r1].copy_(self._dev_out[r0:r1], non_blocking=True)

        self.forward(self._dev_in, out=self._dev_out, row_chunks=row_chunks, after_chunk=ship)
        main.wait_stream(self._copy_stream)
        main.synchronize()
        return out_host

    def forward_gathered(self, x, peer_output):
        """``forward`` + ``gather`` in one pass: this rank's columns are written into
        ``peer_output.local`` and into every other rank's buffer by the GEMM epilogue.
        After the closing fence ``peer_output.local`` holds the whole ``[M, n_total]``."""
        from . import device as D
        xq, a_scale = self.quantize_activation(x)
        begin, count = shard_range(self.n_total, self.world, self.rank, 256)
        if count != self.wq.shape[0] or peer_output.n_total != self.n_total or peer_output.M != x.shape[0]:
            raise ValueError("this rank's weight rows or the shared output do not match the column split")
        peer_output.fence()                       # the previous contents are no longer read anywhere
        if count:
            block = peer_output.local[:, begin:begin + count]
            D.linear_i8_dequant_peers(xq, self.wq, a_scale, self.w_scales, block,
                                      peer_output.peer_block_ptrs(begin), bias=self.bias, relu=self.relu)
        peer_output.fence()                       # every rank's stores have landed
        return peer_output.local

    def gather(self, block, group=None):
        """Full ``[M, n_total]`` output on every rank (NCCL all-gather of column blocks)."""
        if self.world == 1:
            return block
        return gather_columns(block, self.n_total, self.world, group)


class _RawBlock:
    """A device block that torch can view without owning it."""

    def __init__(self, ptr, shape, typestr="<f4"):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 2, "strides": None}


class PeerOutput:
    """The whole ``[M, n_total]`` fp32 output on every rank, written by the GEMMs themselves.

    Each rank allocates its ``[M, n_total]`` buffer with the library's allocator,
    exports it, and opens the buffers of the other ranks of the node
    (``rplb_ipc_export`` / ``rplb_ipc_open``; the handles travel through the process
    group).  ``ShardedQuantizedLinear.forward_gathered`` then stores every output tile
    into all of them from the GEMM's epilogue, so no gather pass follows the GEMM.
    """

    def __init__(self, M, n_total, device, group=None):
        import ctypes as C

        from . import capi
        self.M, self.n_total, self.group = int(M), int(n_total), group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._capi = capi
        base = C.c_void_p()
        capi.call("rplb_malloc", C.byref(base), self.M * self.n_total * 4)
        self.base = int(base.value)
        self.local = torch.as_tensor(_RawBlock(self.base, (self.M, self.n_total)), device=device)
        handle = (C.c_char * 64)()
        capi.call("rplb_ipc_export", self.base, handle)
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self.peer_bases = {}
        for r, h in enumerate(handles):
            if r == self.rank:
                continue
            opened = C.c_void_p()
            capi.call("rplb_ipc_open", (C.c_char * 64).from_buffer_copy(h), C.byref(opened))
            self.peer_bases[r] = int(opened.value)
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)

    def peer_block_ptrs(self, begin):
        """Addresses of column ``begin`` of row 0 in every other rank's buffer."""
        return [b + int(begin) * 4 for _, b in sorted(self.peer_bases.items())]

    def fence(self):
        """Orders the ranks on their streams: everything a rank enqueued before the
        fence has completed on every rank before anything enqueued after it starts."""
        dist.all_reduce(self._flag, group=self.group)

    def close(self):
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier(group=self.group)
        for b in self.peer_bases.values():
            self._capi.call("rplb_ipc_close", b)
        self.peer_bases = {}
        if dist.is_initialized():
            dist.barrier(group=self.group)          # nobody frees while a peer still has the block open
        self.local = None
        if self.base:
            self._capi.call("rplb_free", self.base)
            self.base = 0


class HostPipeline:
    """Back-to-back forward calls on host buffers with the PCIe directions overlapped.

    ``forward_host`` finishes a call before the next one starts, so the host->device
    copy of the next activation waits behind the device->host copy of the current
    output although the link is full duplex.  Here every call is only enqueued
    (``submit``): inputs and outputs are double-buffered on the device, the upload of
    call n+1 runs on its own stream while call n computes and downloads, and
    ``drain`` waits for everything.  Each call still uploads its whole activation and
    downloads its whole output; results are the same bits as ``forward``.
    """

    def __init__(self, layer, rows, in_features, depth=2, row_chunks=8):
        dev = layer.wq.device
        self.layer, self.depth, self.row_chunks = layer, depth, row_chunks
        self.din = [torch.empty((rows, in_features), dtype=torch.float32, device=dev) for _ in range(depth)]
        self.dout = [torch.empty((rows, layer.wq.shape[0]), dtype=torch.float32, device=dev) for _ in range(depth)]
        self.s_in = torch.cuda.Stream(device=dev)
        self.s_out = torch.cuda.Stream(device=dev)
        self.compute_done = [None] * depth
        self.out_done = [None] * depth
        self.calls = 0

    def submit(self, x_host, out_host):
        i = self.calls % self.depth
        main = torch.cuda.current_stream(self.din[i].device)
        if self.compute_done[i] is not None:
            self.s_in.wait_event(self.compute_done[i])        # din[i] was last read by call n - depth
        else:
            self.s_in.wait_stream(main)
        with torch.cuda.stream(self.s_in):
            self.din[i].copy_(x_host, non_blocking=True)
            uploaded = torch.cuda.Event()
            uploaded.record(self.s_in)
        main.wait_event(uploaded)
        if self.out_done[i] is not None:
            main.wait_event(self.out_done[i])                 # dout[i] was last downloaded by call n - depth
        dout = self.dout[i]

        def ship(_, r0, r1):
            ev = torch.cuda.Event()
            ev.record(main)
            self.s_out.wait_event(ev)
            with torch.cuda.stream(self.s_out):
                out_host[r0:r1].copy_(dout[r0:r1], non_blocking=True)

        self.layer.forward(self.din[i], out=dout, row_chunks=self.row_chunks, after_chunk=ship)
        self.compute_done[i] = torch.cuda.Event()
        self.compute_done[i].record(main)
        self.out_done[i] = torch.cuda.Event()
        self.out_done[i].record(self.s_out)
        self.calls += 1

    def drain(self):
        self.s_out.synchronize()
        torch.cuda.current_stream(self.din[0].device).synchronize()


def weighted_column_counts(n_total, speeds, align=256):
    """Column counts per rank in proportion to ``speeds`` (``rplb_shard_weighted``): multiples of ``align``
    by largest remainder.  Every rank must call it with the same numbers."""
    import ctypes as C

    from . import capi
    world = len(speeds)
    w = (C.c_double * world)(*[float(v) for v in speeds])
    counts = (C.c_uint64 * world)()
    capi.call("rplb_shard_weighted", int(n_total), world, int(align), w, counts)
    return [int(c) for c in counts]


class RowShardedLinear:
    """Binding of ``rplb_sharded_linear_*``: the quantized Linear with output columns AND
    activation rows split over the ranks, run entirely by ``librpl.so`` (its own NCCL
    communicator, peer copies of the int8 rows under the GEMM).

    ``torch.distributed`` is used once, to hand rank 0's NCCL id to the other ranks.
    ``wq`` / ``w_scales`` / ``bias`` are this rank's weight rows (``columns(n_total, ...)``
    tells which), already in device memory.
    """

    def __init__(self, wq, w_scales, bias, n_total, max_rows, rank=0, world=1, group=None, column_counts=None):
        import ctypes as C

        from . import capi
        self._capi, self._C = capi, C
        self.rank, self.world, self.n_total, self.max_rows = rank, world, int(n_total), int(max_rows)
        self.wq, self.w_scales, self.bias = wq, w_scales, bias          # keep the tensors alive
        self.K = int(wq.shape[1])
        ident = None
        if world > 1:
            raw = (C.c_char * capi.RPLB_NCCL_ID_BYTES)()
            if rank == 0:
                capi.call("rplb_nccl_unique_id", raw)
            box = [bytes(raw.raw)]
            dist.broadcast_object_list(box, src=0, group=group)
            ident = (C.c_char * capi.RPLB_NCCL_ID_BYTES).from_buffer_copy(box[0])
        self.handle = C.c_void_p()
        counts = (C.c_uint64 * world)(*[int(c) for c in column_counts]) if column_counts is not None else None
        capi.call("rplb_sharded_linear_create_split", C.byref(self.handle), rank, world, ident, None, self.max_rows, self.K,
                  self.n_total, counts, C.c_void_p(wq.data_ptr()), C.c_void_p(w_scales.data_ptr()),
                  C.c_void_p(bias.data_ptr()) if bias is not None else None)
        b, c = C.c_uint64(), C.c_uint64()
        capi.call("rplb_sharded_linear_columns", self.handle, C.byref(b), C.byref(c))
        self.col_begin, self.col_count = int(b.value), int(c.value)
        if self.col_count != wq.shape[0]:
            raise ValueError("this rank owns %d columns, %d weight rows were given" % (self.col_count, wq.shape[0]))

    def rows(self, M):
        """(begin, count) of this rank's rows of an ``[M, K]`` activation."""
        b, c = self._C.c_uint64(), self._C.c_uint64()
        self._capi.call("rplb_sharded_linear_rows", self.handle, int(M), self._C.byref(b), self._C.byref(c))
        return int(b.value), int(c.value)

    def forward(self, x_local, M, out=None, relu=False):
        """x_local: this rank's fp32 rows ``[rows(M)[1], K]`` on the device -> fp32 column block ``[M, col_count]``."""
        C = self._C
        if out is None:
            out = torch.empty((M, self.col_count), dtype=torch.float32, device=self.wq.device)
        ldo = out.stride(0) if M > 1 else max(self.col_count, out.stride(0))
        self._capi.call("rplb_sharded_linear_forward", self.handle, C.c_void_p(x_local.data_ptr()), int(M),
                        C.c_void_p(out.data_ptr()), int(ldo), 1 if relu else 0,
                        C.c_void_p(torch.cuda.current_stream().cuda_stream))
        return out

    def quantize(self, x_local, M):
        """First half of ``forward``: scale agreement, quantization of the local rows, start of their transfer."""
        C = self._C
        self._capi.call("rplb_sharded_linear_quantize", self.handle, C.c_void_p(x_local.data_ptr()), int(M),
                        C.c_void_p(torch.cuda.current_stream().cuda_stream))

    def gemm(self, M, out, relu=False):
        """Second half of ``forward``: the contraction over all ``M`` rows of the activation quantized last."""
        C = self._C
        ldo = out.stride(0) if M > 1 else max(self.col_count, out.stride(0))
        self._capi.call("rplb_sharded_linear_gemm", self.handle, int(M), C.c_void_p(out.data_ptr()), int(ldo),
                        1 if relu else 0, C.c_void_p(torch.cuda.current_stream().cuda_stream))
        return out

    def transfer(self, which):
        """0 = the int8 rows travel by copy-engine peer copies (default), 1 = by stores from a second quantize kernel."""
        self._capi.call("rplb_sharded_linear_transfer", self.handle, int(which))

    def activation(self, M):
        """The whole int8 activation as this rank holds it after a forward, and its scale (views, not copies)."""
        C = self._C
        q, s = C.c_void_p(), C.c_void_p()
        self._capi.call("rplb_sharded_linear_activation", self.handle, C.byref(q), C.byref(s))
        dev = self.wq.device
        xq = torch.as_tensor(_RawBlock(q.value, (M, self.K), "|i1"), device=dev)
        scale = torch.as_tensor(_RawBlock(s.value, (1,)), device=dev)
        return xq, scale

    def gather(self, block, M):
        C = self._C
        full = torch.empty((M, self.n_total), dtype=torch.float32, device=block.device)
        self._capi.call("rplb_sharded_linear_gather", self.handle, C.c_void_p(block.data_ptr()), int(block.stride(0)), int(M),
                        C.c_void_p(full.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
        return full

    def submit_host(self, x_local_host, M, out_host, relu=False, row_blocks=0, stream=None):
        C = self._C
        self._capi.call("rplb_sharded_linear_submit_host", self.handle, C.c_void_p(x_local_host.data_ptr()), int(M),
                        C.c_void_p(out_host.data_ptr()), 1 if relu else 0, int(row_blocks),
                        C.c_void_p(stream.cuda_stream) if stream is not None else None)

    def drain(self):
        self._capi.call("rplb_sharded_linear_drain", self.handle)

    def close(self):
        if self.handle:
            self._capi.load().rplb_sharded_linear_free(self.handle)
            self.handle = None
