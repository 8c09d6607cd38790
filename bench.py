"""Benchmark of the INT8 quantized-inference hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (default): the large sharded INT8 GEMM, M=65536, K=8192, N=65536.
A is fp32 ~ N(0,1), quantized per tensor (symmetric) every step; the weight is
fp32 ~ N(0,0.02) stored [N,K], quantized per output channel once at set-up
(weights are static) and split over the output columns across the ranks; the
output is fp32 acc*sA*sW[n], left column-sharded.  One step = quantize(A) +
GEMM + dequantizing epilogue on every rank; the metric counts 2*M*N*K integer
operations per step over the whole job ("strong" scaling: N is split).

Prints one JSON line (rank 0).  `value` is timed with inputs resident in HBM;
`e2e` repeats the step through the host-buffer API with the host->device copy
of A and the device->host copy of the output inside the timed region.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "int8_gemm_tops_quant_gemm_dequant"
UNIT = "TOPS"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c5", choices=["c1", "c2", "c3", "c5"],
                    help="c5 = large sharded GEMM (the benchmark); c1 512^3, c2 quantized MLP, c3 transformer "
                         "projections: secondary single-GPU lines, device-resident timing only")
    ap.add_argument("--m", type=int, default=65536)
    ap.add_argument("--n", type=int, default=65536)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer pass")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-sweep", action="store_true", help="skip the quantize/dequantize GB/s figures")
    ap.add_argument("--no-clocks", action="store_true", help="no nvidia-smi sampling and no pre-roll (for profiler runs)")
    ap.add_argument("--sweep-only", action="store_true", help="only the quantize/dequantize GB/s figures (for profiler runs)")
    ap.add_argument("--overlap", type=int, default=-1,
                    help="row blocks for pipelining the quantize pass under the GEMM (0 = sequential, "
                         "-1 = choose: pipelined when a rank's GEMM is short enough for the quantize pass to matter)")
    ap.add_argument("--gemm-backend", type=int, default=0, help="rplb_gemm_backend code (0 auto, 3 tcgen05 128x256 tiles, 4 CTA pair, 5 256x256 tiles per CTA)")
    ap.add_argument("--gemm-epilogue", type=int, default=0, help="rplb_gemm_epilogue code (0 TMA tensor stores where possible, 1 stores from registers)")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="target CPU time of the baseline sample")
    ap.add_argument("--gather", action="store_true",
                    help="with N > 1 also time the all-gather of the fp32 column blocks into [M, N] on every rank (own line, not part of value)")
    return ap.parse_args()


def workload_name(a):
    if (a.m, a.n, a.k) == (65536, 65536, 8192):
        return "large sharded INT8 GEMM M=65536 K=8192 N=65536 (A per-tensor, W per-channel, fp32 out)"
    return "INT8 GEMM M=%d K=%d N=%d (A per-tensor, W per-channel, fp32 out)" % (a.m, a.k, a.n)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_burst": float(d["bf16_tflops"]),
                "bf16_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []
        self.t_begin = None
        self.t_end = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        import datetime
        sm, smax, reasons, watts = [], None, set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            if self.t_begin is not None and self.t_end is not None:
                # keep only samples taken inside the timed region
                try:
                    ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                except ValueError:
                    continue
                if not (self.t_begin <= ts <= self.t_end):
                    continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            try:
                watts.append(float(f[3]))
            except ValueError:
                pass
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        med = sm[len(sm) // 2] if sm else None
        watts.sort()
        return {"sm_mhz": med, "sm_max_mhz": smax, "reasons": sorted(reasons), "samples": len(sm),
                "power_w": watts[len(watts) // 2] if watts else None}


# --------------------------------------------------------------------------- CPU legs
class CpuPath:
    """The reference's CPU implementation of one step, on a bounded sample:
    tensor_quantize_int8_symmetric on a slab of rows of A, linear_int8 of the
    slab against a block of weight rows, fp32 scaling of the accumulators.
    Uses oracle/_ref (the reference's own compiled code) when it is present,
    else the C restatement."""

    def __init__(self, K, target_seconds):
        import numpy as np
        from oracle.loader import Port, Ref, ref_available
        self.np = np
        self.kind = "reference" if ref_available() else "port"
        self.impl = Ref() if self.kind == "reference" else Port()
        self.cores = Port().num_threads()
        self.K = K
        rng = np.random.default_rng(0x5EED0050)
        # Probe the host's rate on a small case, then size the sample.
        a = rng.standard_normal((64, K)).astype(np.float32)
        w = rng.integers(-127, 128, (1024, K), dtype=np.int8)
        t0 = time.perf_counter()
        q, _ = self.impl.quantize_symmetric(a)
        self.impl.linear(q, w)
        rate = 2.0 * 64 * 1024 * K / max(time.perf_counter() - t0, 1e-6)
        self.cols = 8192
        rows = int(rate * target_seconds / (2.0 * self.cols * K))
        self.rows = max(64, min(65536, (rows // 64) * 64))
        self.a = rng.standard_normal((self.rows, K)).astype(np.float32)
        wf = (rng.standard_normal((self.cols, K)) * 0.02).astype(np.float32)
        self.wq, self.ws, _ = self.impl.quantize_per_channel(wf) if self.kind == "reference" else \
            self.impl.quantize_per_channel(wf, self.cols)
        del wf
        self.ops = 2.0 * self.rows * self.cols * K

    def step(self):
        np = self.np
        q, s = self.impl.quantize_symmetric(self.a)
        if self.kind == "reference":
            acc = self.impl.linear(q, self.wq)
            out = (acc.astype(np.float32) * np.float32(s)) * self.ws[None, :]
        else:
            out = self.impl.linear_dequant(q, self.wq, s, self.ws)
        return out

    def describe(self):
        return ("%d rows of A x %d weight rows, K=%d: quantize(A slab) + linear_int8 + fp32 scaling of the "
                "accumulators%s" % (self.rows, self.cols, self.K,
                                    " (scaling done with numpy: the reference has no fused epilogue)"
                                    if self.kind == "reference" else ""))


def run_reference_arm(a):
    """`--impl reference`: the reference's CPU path on the host cores, rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cpu = CpuPath(a.k, max(2.0, min(a.cpu_seconds, 120.0 / max(a.steps + a.warmup, 1))))
    for _ in range(a.warmup):
        cpu.step()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        cpu.step()
    dt = (time.perf_counter() - t0) / max(a.steps, 1)
    tops = cpu.ops / dt / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": workload_name(a), "sample_per_step": cpu.describe()},
        "cpu_baseline": {"value": tops, "unit": UNIT, "cores": cpu.cores, "kind": cpu.kind, "sample": cpu.describe()},
        "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def event_ms(pairs):
    return [a.elapsed_time(b) for a, b in pairs]


def quantize_sweep_one(torch, D, dev, peaks, n):
    """Quantize / dequantize GB/s on n fp32 elements, rows of 4096: N(0,3) with outliers at +/-50."""
    g = torch.Generator(device=dev)
    g.manual_seed(0x5EED0040)
    x = torch.randn(n, device=dev, generator=g) * 3.0
    x[::1009] = 50.0
    x[5::2003] = -50.0
    q = torch.empty(n, dtype=torch.int8, device=dev)
    params = torch.empty(8, dtype=torch.float32, device=dev)
    back = torch.empty(n, dtype=torch.float32, device=dev)
    x2 = x.view(-1, 4096)
    cases = [
        ("quantize_explicit_scale", 5.0, lambda: D.quantize(x, 0.3937, 0, out=q)),
        ("quantize_per_tensor_symmetric", 9.0, lambda: D.quantize_symmetric(x, out=q, params=params)),
        ("minmax", 4.0, lambda: D.minmax(x, params=params)),
        ("quantize_per_channel_rows4096", 5.0, lambda: D.quantize_per_channel(x2, out=q.view(-1, 4096))),
        # the other reading of "rows of 4096 channels": 4096 channels of n/4096 elements each.  A channel is
        # read twice by its CTA; the second read comes from L2 while the ~1184 channels in flight fit there
        # (5 B/element of HBM traffic), otherwise both passes go to HBM (9 B/element).
        ("quantize_per_channel_4096_channels", 5.0 if (n // 4096) * 4 * 1184 <= 100e6 else 9.0,
         lambda: D.quantize_per_channel(x.view(4096, -1), out=q.view(4096, -1))),
        ("dequantize", 5.0, lambda: D.dequantize(q, 0.3937, 0, out=back)),
    ]
    res = {"elements": n, "unit": "GB/s", "peak_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"]}
    launches = 0
    for name, bytes_per_elem, fn in cases:
        for _ in range(3):
            fn()
        # 20 launches between one pair of events (a kernel here can last ~50 us: an event
        # pair around every launch would time the launch gap as well), 5 such groups.
        reps, groups = 20, 5
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(groups)]
        before = D.launch_count()
        for a, b in evs:
            a.record()
            for _ in range(reps):
                fn()
            b.record()
        torch.cuda.synchronize()
        launches += D.launch_count() - before
        ms = sorted(t / reps for t in event_ms(evs))
        med = ms[len(ms) // 2]
        gbs = bytes_per_elem * n / (med * 1e-3) / 1e9
        res[name] = {"ms": med, "gbs": gbs, "bytes_per_elem": bytes_per_elem, "frac": gbs / peaks["hbm_gbs"]}
    res["launches"] = launches
    return res


def quantize_sweep(torch, D, dev, peaks):
    """The memory-bound sweep: 2^26 elements (256 MiB, larger than L2) is the quoted
    size; 2^20 (fits in L2: launch- and L2-bound) and 2^30 (4 GiB) ride along."""
    res = quantize_sweep_one(torch, D, dev, peaks, 1 << 26)
    res["other_sizes"] = {}
    for n in (1 << 20, 1 << 30):
        r = quantize_sweep_one(torch, D, dev, peaks, n)
        res["other_sizes"][str(n)] = {k: {"ms": v["ms"], "gbs": v["gbs"], "frac": v["frac"]} for k, v in r.items()
                                      if isinstance(v, dict)}
        res["launches"] += r["launches"]
        torch.cuda.empty_cache()
    return res


def smi_id(torch, dev, local):
    """What `nvidia-smi -i` should be given for this rank's GPU."""
    try:
        u = str(torch.cuda.get_device_properties(dev).uuid)
        return u if u.startswith("GPU-") else "GPU-" + u
    except Exception:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
        ids = [v for v in vis.split(",") if v]
        return ids[local] if local < len(ids) else str(local)


def run_ours(a):
    import torch
    import torch.distributed as dist

    from rpl_b200 import device as D
    from rpl_b200.sharded import ShardedQuantizedLinear, shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: librpl has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        # A short timeout: a rank that falls out of step fails in minutes, not in ten.
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    peaks = measured_peaks()
    M, N, K = a.m, a.n, a.k
    D.gemm_backend(a.gemm_backend)
    D.gemm_epilogue(a.gemm_epilogue)
    if a.sweep_only:
        print(json.dumps({"quantize_sweep": quantize_sweep(torch, D, dev, peaks)}), flush=True)
        return

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- synthetic inputs (same A on every rank; W rows by global index) ----
    g = torch.Generator(device=dev)
    g.manual_seed(0x5EED0050)
    A = torch.randn((M, K), device=dev, generator=g)
    begin, count = shard_range(N, world, rank, 256)
    wq = torch.empty((count, K), dtype=torch.int8, device=dev)
    wsc = torch.empty(count, dtype=torch.float32, device=dev)
    blk = 4096
    for r0 in range(0, count, blk):
        r1 = min(count, r0 + blk)
        g.manual_seed(0x5EED0051 + (begin + r0))
        w = torch.randn((r1 - r0, K), device=dev, generator=g) * 0.02
        q, s, _ = D.quantize_per_channel(w)
        wq[r0:r1] = q
        wsc[r0:r1] = s
    del w, q, s
    layer = ShardedQuantizedLinear(wq, wsc, None, n_total=N, rank=rank, world=world)
    if a.overlap < 0:
        # Measured on one B200 (ms per step, sequential -> pipelined): 8192 columns per
        # rank (the 8-GPU share) 4.48 -> 4.13 with six row blocks; 16384 columns 8.06 -> 8.20;
        # 32768 columns 15.3 -> 15.7; all 65536 columns 29.7 -> 30.6.  The blocks cost the
        # GEMM about as much as they hide except when the GEMM itself is only a few ms.
        a.overlap = 6 if float(M) * count * K <= 5.0e12 else 0
    out = torch.empty((M, count), dtype=torch.float32, device=dev)
    ops_total = 2.0 * M * N * K
    ops_rank = 2.0 * M * count * K

    # ---- device-resident timing ----
    step_fn = (lambda: layer.forward_overlapped(A, out=out, row_chunks=a.overlap)) if a.overlap > 1 else \
        (lambda: layer.forward(A, out=out))
    for _ in range(max(a.warmup, 3)):
        step_fn()
    torch.cuda.synchronize()
    if D.kernel_status(True) != 0:
        raise RuntimeError("the tcgen05 kernel reported an expired wait during warm-up")
    gemm_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(a.steps)]
    quant_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(a.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(smi_id(torch, dev, local))
    # The sampler needs a moment to start: keep the GPU under the same load
    # until it has, then open the timed region.
    if not a.no_clocks:
        sampler.start()
        # Every rank must run the same number of pre-roll steps (a step contains a
        # collective when N > 1): rank 0 sizes it for about a second and tells the others.
        t_pre = time.time()
        step_fn()
        torch.cuda.synchronize()
        n_pre = torch.tensor([max(1, min(2000, int(1.0 / max(time.time() - t_pre, 1e-4))))], device=dev)
        if world > 1:
            dist.broadcast(n_pre, src=0)
        for _ in range(int(n_pre.item())):
            step_fn()
        torch.cuda.synchronize()
    barrier()
    sampler.t_begin = time.time()
    launches0 = D.launch_count()
    e0.record()
    gemm_pairs = []
    for i in range(a.steps):
        if a.overlap > 1:
            layer.forward_overlapped(A, out=out, row_chunks=a.overlap, gemm_events=gemm_pairs)
            continue
        quant_ev[i][0].record()
        xq, a_scale = layer.quantize_activation(A)
        quant_ev[i][1].record()
        gemm_ev[i][0].record()
        layer.gemm(xq, a_scale, out=out)
        gemm_ev[i][1].record()
    e1.record()
    barrier()
    sampler.t_end = time.time()
    launches = D.launch_count() - launches0
    time.sleep(0.15)
    clocks = sampler.stop()
    if D.kernel_status(True) != 0:
        raise RuntimeError("the tcgen05 kernel reported an expired wait")
    ms = e0.elapsed_time(e1) / a.steps
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    if a.overlap > 1:
        gemm_ms = sum(event_ms(gemm_pairs)) / a.steps
        quant_ms = max(ms - gemm_ms, 0.0)               # what of the quantize pass is not hidden under the GEMM
    else:
        gemm_ms = sum(event_ms(gemm_ev)) / a.steps
        quant_ms = sum(event_ms(quant_ev)) / a.steps
    per_rank = torch.tensor([gemm_ms, quant_ms, ms], device=dev)
    if world > 1:
        gathered = [torch.empty_like(per_rank) for _ in range(world)]
        dist.all_gather(gathered, per_rank)
        per_rank = torch.stack(gathered)
    else:
        per_rank = per_rank.reshape(1, 3)
    per_rank = [[round(float(v), 4) for v in row] for row in per_rank.cpu()]

    # ---- optional: all-gather of the column blocks, timed on its own ----
    gather = None
    if a.gather and world > 1:
        full = layer.gather(out)                            # warm-up: NCCL channels and buffers
        del full
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 3
        g0.record()
        for _ in range(reps):
            full = layer.gather(out)
            del full
        g1.record()
        barrier()
        tg = torch.tensor([g0.elapsed_time(g1) / reps], device=dev)
        dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        received = float(M) * (N - count) * 4
        gather = {"ms": float(tg.item()), "received_bytes_per_rank": received,
                  "GB/s_per_rank_in": received / (float(tg.item()) * 1e-3) / 1e9,
                  "what": "NCCL all-gather of fp32 [M, N/G] blocks plus unpack into row-major [M, N] on every rank"}

    # ---- optional: the same step with the gather fused into the GEMM epilogue ----
    if a.gather and world > 1:
        from rpl_b200.sharded import PeerOutput
        shared = PeerOutput(M, N, dev)
        for _ in range(2):
            layer.forward_gathered(A, shared)
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(a.steps):
            layer.forward_gathered(A, shared)
        f1.record()
        barrier()
        tf = torch.tensor([f0.elapsed_time(f1) / a.steps], device=dev)
        dist.all_reduce(tf, op=dist.ReduceOp.MAX)
        same_block = bool(torch.equal(shared.local[:256, begin:begin + count], out[:256]))
        other = (rank + 1) % world
        ob, oc = shard_range(N, world, other, 256)
        probe = out[:256, :min(oc, 1024)].contiguous()       # the neighbour's first rows and columns, for a cross-check
        probes = [torch.empty_like(probe) for _ in range(world)]
        dist.all_gather(probes, probe)
        same_remote = bool(torch.equal(shared.local[:256, ob:ob + min(oc, 1024)], probes[other]))
        gather["fused"] = {"ms_per_step": float(tf.item()), "value": ops_total / (float(tf.item()) * 1e-3) / 1e12, "unit": UNIT,
                           "what": "quantize + GEMM whose epilogue stores every tile into all ranks' [M, N] buffers over NVLink (peer stores), fences included",
                           "matches_sharded_run": same_block and same_remote}
        shared.close()
        del shared

    # ---- end to end through host buffers ----
    e2e = None
    if not a.no_e2e:
        xh = oh = None
        try:
            xh = torch.empty((M, K), dtype=torch.float32, pin_memory=True)
            oh = torch.empty((M, count), dtype=torch.float32, pin_memory=True)
            have = 1
        except RuntimeError:
            have = 0
        agreed = torch.tensor([have], device=dev)
        if world > 1:
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)          # all ranks take the same branch
        if int(agreed.item()) == 0:
            e2e = {"value": None, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                   "error": "page-locked host buffers (%.1f GiB per rank) could not be allocated" % ((M * K + M * count) * 4 / 2**30)}
        else:
            xh.copy_(A)
            torch.cuda.synchronize()
            # The reference-facing C ABI with host buffers: a QuantizedLinear layer over this rank's
            # device-resident int8 weights, quantized_linear_submit_host / _drain.  Every call uploads
            # its whole activation and downloads its whole output; the upload of call n+1 overlaps the
            # download of call n (PCIe is full duplex).  Quantize and GEMM run on torch's current
            # stream, which after the drain has also waited for the downloads, so the events see it all.
            import ctypes as C
            from rpl_b200 import capi
            L = capi.load()
            clayer = L.quantized_linear_wrap(wq.data_ptr(), wsc.data_ptr(), None, K, count)
            if not clayer:
                raise RuntimeError("quantized_linear_wrap failed")
            estream = torch.cuda.Stream(device=dev)         # quantize and GEMM of the e2e calls run here
            estream.wait_stream(torch.cuda.current_stream())
            main = C.c_void_p(estream.cuda_stream)

            def submit():
                rc = L.quantized_linear_submit_host(clayer, xh.data_ptr(), M, oh.data_ptr(), False, main)
                if rc != 0:
                    raise RuntimeError("quantized_linear_submit_host failed with %d" % rc)

            submit()
            if L.quantized_linear_drain(clayer) != 0:
                raise RuntimeError("quantized_linear_drain failed")
            esteps = max(2, min(a.steps, 6))
            barrier()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            launches_e0 = D.launch_count()
            s0.record(estream)
            for _ in range(esteps):
                submit()
            if L.quantized_linear_drain(clayer) != 0:
                raise RuntimeError("quantized_linear_drain failed")
            s1.record(estream)
            barrier()
            e2e_launches = D.launch_count() - launches_e0
            te = torch.tensor([s0.elapsed_time(s1) / esteps], device=dev)
            if world > 1:
                dist.all_reduce(te, op=dist.ReduceOp.MAX)
            same = bool(torch.equal(oh[:256].to(dev), out[:256]))
            e2e = {"value": ops_total / (float(te.item()) * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": float(te.item()),
                   "steps": esteps, "h2d_bytes_per_step": int(M * K * 4) * world, "d2h_bytes_per_step": int(M * N * 4),
                   "api": "quantized_linear_submit_host / quantized_linear_drain (C ABI, page-locked host buffers)",
                   "matches_device_run": same, "gpu_launches": int(e2e_launches)}
            L.quantized_linear_free(clayer)
        del xh, oh

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # DRAM traffic of the GEMM from an ncu capture at 16384 x 16384 x 8192
    # (dram read + write): 6.99 B per output element at K = 8192.
    gemm_launches_per_step = max(1, len(gemm_pairs) // max(a.steps, 1)) if a.overlap > 1 else 1
    traffic = 6.99 * M * count / gemm_launches_per_step if K == 8192 else None
    int8_peak = 2.0 * peaks["bf16_sustained"]
    achieved = ops_rank / (gemm_ms * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": ops_total / (ms_max * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
        "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms_max, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": workload_name(a), "parallelism": "N-split over %d rank(s), output left column-sharded" % world,
                   "columns_per_rank": count,
                   "schedule": ("quantize pass pipelined under the GEMM in %d row blocks" % a.overlap) if a.overlap > 1
                   else "min/max, quantize, GEMM one after the other", "l2": "no flush: per-step inputs and outputs exceed L2 (A %.1f GiB fp32, out %.1f GiB per rank)"
                   % (M * K * 4 / 2**30, M * count * 4 / 2**30)},
        "breakdown_ms": {"quantize_A": quant_ms, "gemm_with_epilogue": gemm_ms,
                         "per_rank_gemm_quant_step": per_rank},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOP/s",
                     "frac": achieved / int8_peak, "traffic": traffic, "traffic_unit": "bytes per launch (ncu dram read+write, scaled by output elements)",
                     "algorithmic_bytes": float(M * K + count * K + 4 * M * count) / gemm_launches_per_step,
                     "launches_per_step": gemm_launches_per_step, "kernel": "gemm_i8_tc_kernel",
                     "peak_note": "2 x bf16_tflops_sustained of %s (int8 dense = 2 x bf16 dense)" % peaks["source"],
                     "frac_of_nominal_4500": achieved / 4500.0},
        "clocks": clocks, "gpu_launches": int(launches), "e2e": e2e,
    }
    if gather is not None:
        line["gather"] = gather
    if world == 1 and not a.no_sweep:
        line["quantize_sweep"] = quantize_sweep(torch, D, dev, peaks)
    if world == 1 and not a.no_cpu:
        del A, out
        cpu = CpuPath(K, a.cpu_seconds)
        cpu.step()
        t0 = time.perf_counter()
        cpu.step()
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": cpu.ops / dt / 1e12, "unit": UNIT, "cores": cpu.cores, "kind": cpu.kind,
                                "sample": cpu.describe(), "seconds": dt}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_secondary(a):
    """Secondary configurations on one GPU: device-resident timing, same metric."""
    import torch

    from rpl_b200 import device as D
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    peaks = measured_peaks()
    D.gemm_backend(a.gemm_backend)
    g = torch.Generator(device=dev)
    g.manual_seed(0x5EED0000 + int(a.workload[1]) * 16)
    one = lambda p: p[D.QPARAM_SCALE_SYM:D.QPARAM_SCALE_SYM + 1]
    if a.workload == "c1":
        name = "INT8 GEMM 512x512x512: A, B fp32 N(0,1), both per-tensor symmetric, fp32 out acc*sA*sB"
        A = torch.randn((512, 512), device=dev, generator=g)
        Bt = torch.randn((512, 512), device=dev, generator=g)          # stored [N,K]
        bq, pb = D.quantize_symmetric(Bt)
        ws = pb[D.QPARAM_SCALE_SYM].repeat(512).contiguous()
        out = torch.empty((512, 512), device=dev)
        aq, pa = torch.empty((512, 512), dtype=torch.int8, device=dev), torch.empty(8, device=dev)
        ops, hbm_bytes = 2.0 * 512 ** 3, None

        def step():
            D.quantize_symmetric(A, out=aq, params=pa)
            D.linear_i8_dequant(aq, bq, one(pa), ws, out=out)
        note = "launch-latency bound: 0.27 GOP is ~0.1 us of tensor work"
    elif a.workload == "c2":
        name = "quantized MLP 784->128->10, batch 65536: X U[0,1) per tensor, W N(0,0.05) per channel, ReLU, fp32 logits"
        Bn = 65536
        X = torch.rand((Bn, 784), device=dev, generator=g)
        w1q, w1s, _ = D.quantize_per_channel(torch.randn((128, 784), device=dev, generator=g) * 0.05)
        w2q, w2s, _ = D.quantize_per_channel(torch.randn((10, 128), device=dev, generator=g) * 0.05)
        b1 = torch.randn(128, device=dev, generator=g) * 0.05
        b2 = torch.randn(10, device=dev, generator=g) * 0.05
        xq, px = torch.empty((Bn, 784), dtype=torch.int8, device=dev), torch.empty(8, device=dev)
        h, hq, ph = torch.empty((Bn, 128), device=dev), torch.empty((Bn, 128), dtype=torch.int8, device=dev), torch.empty(8, device=dev)
        logits = torch.empty((Bn, 10), device=dev)
        ops = 2.0 * Bn * (784 * 128 + 128 * 10)
        # X read twice (min/max, quantize) + int8 X written and read + hidden fp32 written and read once,
        # int8 hidden written and read + logits
        hbm_bytes = Bn * (784 * (4 + 4 + 1 + 1) + 128 * (4 + 4 + 1 + 1) + 10 * 4)

        stats = torch.empty(2, device=dev)
        import ctypes as C
        from rpl_b200 import capi

        def step():
            D.quantize_symmetric(X, out=xq, params=px)
            # layer 1: fused dequant + bias + ReLU; the epilogue also reports max|h| and the scale of h
            capi.call("rplb_linear_i8_dequant_f32_absmax", C.c_void_p(xq.data_ptr()), C.c_void_p(w1q.data_ptr()),
                      C.c_void_p(h.data_ptr()), Bn, 784, 128, 128, C.c_void_p(one(px).data_ptr()),
                      C.c_void_p(w1s.data_ptr()), C.c_void_p(b1.data_ptr()), 1, C.c_void_p(stats[0:1].data_ptr()),
                      C.c_void_p(stats[1:2].data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
            D.quantize_dev(h, stats[1:2], out=hq)
            D.linear_i8_dequant(hq, w2q, stats[1:2], w2s, b2, relu=False, out=logits)
        note = "HBM-bound: 13.3 GOP over ~0.7 GB of traffic"
    else:
        name = "transformer projections: tokens 32768 x d_model 4096, Q/K/V/O weights 4096x4096 per channel, bias, fp32 out"
        T, Dm = 32768, 4096
        X = torch.randn((T, Dm), device=dev, generator=g)
        ws_ = [D.quantize_per_channel(torch.randn((Dm, Dm), device=dev, generator=g) * 0.02) for _ in range(4)]
        bs = [torch.randn(Dm, device=dev, generator=g) * 0.02 for _ in range(4)]
        outs = [torch.empty((T, Dm), device=dev) for _ in range(4)]
        xq, px = torch.empty((T, Dm), dtype=torch.int8, device=dev), torch.empty(8, device=dev)
        ops, hbm_bytes = 4 * 2.0 * T * Dm * Dm, None

        def step():
            D.quantize_symmetric(X, out=xq, params=px)
            for (wq, wsc, _), b, o in zip(ws_, bs, outs):
                D.linear_i8_dequant(xq, wq, one(px), wsc, b, out=o)
        note = "X quantized once per step, four GEMMs with fused per-channel dequant + bias"
    # These steps are a handful of short kernels: replay them from a CUDA graph so
    # that the host's launch cost does not show up as GPU idle time.  The library
    # allocates its per-stream scratch on first use, so warm up on the capture stream.
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(max(a.warmup, 3)):
            step()
    side.synchronize()
    l0 = D.launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        step()
    per_step = D.launch_count() - l0
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    if D.kernel_status(True) != 0:
        raise RuntimeError("the tcgen05 kernel reported an expired wait")
    ms = e0.elapsed_time(e1) / a.steps
    line = {"metric": METRIC, "value": ops / (ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": 1, "steps": a.steps,
            "warmup": max(a.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": {"workload": name, "note": note, "replay": "CUDA graph of one step"},
            "gpu_launches": int(per_step * a.steps)}
    if hbm_bytes:
        gbs = hbm_bytes / (ms * 1e-3) / 1e9
        line["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": gbs / peaks["hbm_gbs"], "traffic": None}
    else:
        t = ops / (ms * 1e-3) / 1e12
        line["roofline"] = {"bound": "tensor", "achieved": t, "peak": 2.0 * peaks["bf16_sustained"], "unit": "TOP/s",
                            "frac": t / (2.0 * peaks["bf16_sustained"]), "traffic": None}
    print(json.dumps(line), flush=True)


def main():
    a = parse_args()
    if a.impl != "reference" and a.workload != "c5":
        run_secondary(a)
        return
    if a.impl == "reference":
        # torchrun pins OMP_NUM_THREADS to 1; the CPU arm is meant to use every host
        # core, and the OpenMP runtime reads the variable when it is first loaded.
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
        run_reference_arm(a)
    else:
        run_ours(a)


if __name__ == "__main__":
    main()
