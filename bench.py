"""Benchmark of the INT8 quantized-inference hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (default): the large sharded INT8 GEMM, M=65536, K=8192, N=65536.
A is fp32 ~ N(0,1), quantized per tensor (symmetric) every step; the weight is
fp32 ~ N(0,0.02) stored [N,K], quantized per output channel once at set-up
(weights are static) and split over the output columns across the ranks; the
output is fp32 acc*sA*sW[n], left column-sharded.  The rows of A are split over
the ranks too: every rank holds its rows in fp32, the ranks agree on the scale
with one max-all-reduce, each quantizes its rows and sends the int8 rows to the
others over NVLink while the GEMM already runs.  One step = that on every rank;
the metric counts 2*M*N*K integer operations per step over the whole job
("strong" scaling: the work is split).  The schedule is the same at every N.

Prints one JSON line (rank 0).  `value` is timed with inputs resident in HBM;
`e2e` repeats the step through the C ABI's host-buffer call with the
host->device copy of each rank's rows of A and the device->host copy of its
output block inside the timed region.  After the timed regions samples of the
results are compared with the CPU oracle (`parity`).
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
    ap.add_argument("--no-secondary", action="store_true", help="skip the 512^3 / MLP / projection lines")
    ap.add_argument("--no-parity", action="store_true", help="skip the checks against the CPU oracle after the timed region")
    ap.add_argument("--no-probe", action="store_true", help="skip the cuBLASLt INT8 probe (torch._int_mm)")
    ap.add_argument("--schedule", default="rows", choices=["rows", "replicated"],
                    help="rows: every rank holds, quantizes and sends only its rows of A (the default at every N); "
                         "replicated: every rank holds and quantizes all of A (comparison only, N > 1)")
    ap.add_argument("--no-numa", action="store_true", help="allocate the page-locked host buffers wherever the process happens to run "
                    "(default: on the CPUs next to the rank's GPU)")
    ap.add_argument("--balance", action="store_true", help="N > 1: re-split the columns in proportion to each GPU's GEMM speed measured "
                    "under load before the timed region (off by default: measured, the ranking of the GPUs of a node under "
                    "their power cap does not hold from one second to the next, and the re-split cost 0-3 %)")
    ap.add_argument("--no-balance", action="store_true", help="accepted for older command lines: the even split is the default")
    ap.add_argument("--transfer", type=int, default=0, help="N > 1: how the int8 rows reach the other ranks: 0 copy engines (default), "
                    "1 stores from a second quantize kernel (comparison)")
    ap.add_argument("--balance-threshold", type=float, default=1.06,
                    help="N > 1: re-split the columns only when the slowest rank's GEMM takes this many times the fastest's")
    ap.add_argument("--no-clocks", action="store_true", help="no nvidia-smi sampling and no pre-roll (for profiler runs)")
    ap.add_argument("--sweep-only", action="store_true", help="only the quantize/dequantize GB/s figures (for profiler runs)")
    ap.add_argument("--sweep-elements", type=int, default=0, help="with --sweep-only: that one tensor size instead of 2^26, 2^20 and 2^30")
    ap.add_argument("--overlap", type=int, default=0,
                    help="replicated schedule only: row blocks for pipelining the quantize pass under the GEMM (0 = sequential)")
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


class Checker:
    """The CPU oracle as a checker of sampled results: the reference's own compiled code
    (oracle/_ref) when it is present, else the C restatement.  Never timed, never shipped."""

    def __init__(self):
        from oracle.loader import Port, Ref, ref_available
        self.port = Port()
        self.ref = Ref() if ref_available() else None
        self.name = "reference" if self.ref is not None else "port"
        self.checked = 0
        self.mismatches = 0
        self.notes = []

    def scale(self, lo, hi):
        return self.port.scale_symmetric(lo, hi)            # fmaxf(|min|,|max|) / 127.0f, IEEE division

    def quantize(self, x, scale):
        return (self.ref or self.port).quantize(x, scale, 0)

    def tile(self, xq, wq, scale, ws):
        """fp32 outputs of int8 rows xq against int8 weight rows wq: accumulate, then (float)acc * sA, then * sW[n]."""
        import numpy as np
        if self.ref is not None:
            acc = self.ref.linear(xq, wq)
            return (acc.astype(np.float32) * np.float32(scale)) * ws[None, :]
        return self.port.linear_dequant(xq, wq, scale, ws)

    def expect(self, ok, what):
        self.checked += 1
        if not ok:
            self.mismatches += 1
            if len(self.notes) < 8:
                self.notes.append(what)

    def result(self):
        r = {"checked": self.checked, "mismatches": self.mismatches, "oracle": self.name}
        if self.notes:
            r["first_mismatches"] = self.notes
        return r


def check_quantize_windows(torch, chk, x, q, scale_dev, windows, what, seed=7):
    """`windows` windows of 4096 elements of a quantized tensor against the oracle, plus its scale."""
    import numpy as np
    n = x.numel()
    lo, hi = float(x.min().item()), float(x.max().item())       # exact operations: any device may take them
    want_scale = chk.scale(np.float32(lo), np.float32(hi))
    got_scale = np.float32(scale_dev.item())
    chk.expect(want_scale.tobytes() == got_scale.tobytes(), "%s: scale %r, oracle %r" % (what, got_scale, want_scale))
    rng = np.random.default_rng(seed)
    xf, qf = x.reshape(-1), q.reshape(-1)
    for _ in range(windows):
        o = int(rng.integers(0, max(1, n - 4096)))
        xs = xf[o:o + 4096].cpu().numpy()
        chk.expect(np.array_equal(chk.quantize(xs, want_scale), qf[o:o + 4096].cpu().numpy()), "%s: window at %d" % (what, o))


def quantize_sweep_one(torch, D, dev, peaks, n, chk=None):
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
        # the other reading of "rows of 4096 channels": 4096 channels of n/4096 elements each.  Channels of up
        # to 232 KiB are kept on chip (registers + shared memory) and read from HBM once (5 B/element);
        # longer ones are read twice by their CTA, the second time from L2 while the ~1184 channels in
        # flight fit there, otherwise from HBM (9 B/element).
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
    if chk is not None and n >= (1 << 26):
        D.quantize_symmetric(x, out=q, params=params)
        torch.cuda.synchronize()
        check_quantize_windows(torch, chk, x, q, params[D.QPARAM_SCALE_SYM], 64, "per-tensor quantize of 2^%d elements" % (n.bit_length() - 1))
    return res


def quantize_sweep(torch, D, dev, peaks, chk=None):
    """The memory-bound sweep: 2^26 elements (256 MiB, larger than L2) is the quoted
    size; 2^20 (fits in L2: launch- and L2-bound) and 2^30 (4 GiB) ride along."""
    res = quantize_sweep_one(torch, D, dev, peaks, 1 << 26, chk)
    res["other_sizes"] = {}
    for n in (1 << 20, 1 << 30):
        r = quantize_sweep_one(torch, D, dev, peaks, n, chk)
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


class NearGpu:
    """While active, the process runs on the CPUs next to its GPU, so that page-locked
    buffers allocated inside land in that NUMA node's memory (each rank's PCIe traffic
    then stays off the inter-socket link).  Affinity is put back afterwards; reading
    NVML's affinity mask changes nothing on the GPU."""

    def __init__(self, torch, dev):
        self.cpus, self.saved = None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(dev).uuid)
            uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if hasattr(uuid, "encode") else uuid)
            words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
            cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
            allowed = os.sched_getaffinity(0)
            self.cpus = (cpus & allowed) or None
        except Exception:
            self.cpus = None

    def __enter__(self):
        if self.cpus:
            try:
                self.saved = os.sched_getaffinity(0)
                os.sched_setaffinity(0, self.cpus)
            except OSError:
                self.saved = None
        return self

    def __exit__(self, *exc):
        if self.saved:
            try:
                os.sched_setaffinity(0, self.saved)
            except OSError:
                pass


def int8_probe(torch, dev, seconds=2.0):
    """What the vendor's INT8 GEMM (cuBLASLt through torch._int_mm) reaches on this GPU, 8192^3:
    best single call and a back-to-back loop of about `seconds` under the power cap.  A ceiling to
    read the roofline fraction against; it is not on the product path."""
    n = 8192
    a = torch.randint(-128, 128, (n, n), device=dev, dtype=torch.int8)
    b = torch.randint(-128, 128, (n, n), device=dev, dtype=torch.int8)
    ops = 2.0 * n ** 3
    for _ in range(3):
        torch._int_mm(a, b)
    torch.cuda.synchronize()
    best = 1e9
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    reps = max(10, int(seconds * 1e3 / best))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        torch._int_mm(a, b)
    e1.record()
    torch.cuda.synchronize()
    sustained = e0.elapsed_time(e1) / reps
    return {"burst_tops": ops / (best * 1e-3) / 1e12, "sustained_tops": ops / (sustained * 1e-3) / 1e12, "shape": "8192^3",
            "what": "torch._int_mm (cuBLASLt INT8) on this GPU in this run, outside the timed region"}


def rows_of_a(torch, dev, M, K, r0, rc):
    """Rows [r0, r0 + rc) of the synthetic activation ~ N(0,1): generated in blocks of 4096 rows, each from
    its own seed, so that a rank makes exactly its rows and every split of the rows gives the same matrix."""
    out = torch.empty((rc, K), dtype=torch.float32, device=dev)
    g = torch.Generator(device=dev)
    blk = 4096
    b = r0 // blk
    while b * blk < r0 + rc:
        g.manual_seed(0x5EED0050 + 7919 * b)
        rows = torch.randn((min(blk, M - b * blk), K), device=dev, generator=g)
        lo, hi = max(r0, b * blk), min(r0 + rc, (b + 1) * blk)
        out[lo - r0:hi - r0] = rows[lo - b * blk:hi - b * blk]
        b += 1
    return out


def check_main_results(torch, dist, chk, layer, A_local, out, wq, wsc, M, K, world, rank, dev):
    """Samples of the timed run's results against the oracle: the agreed scale, windows of this rank's int8
    rows, the int8 activation as every rank holds it (block checksums must agree across ranks), and 128 x 128
    tiles of this rank's output block, half of them on rows that came from other ranks."""
    import numpy as np
    r0, rc = layer.rows(M)
    xq, scale_dev = layer.activation(M)
    lo = torch.tensor([float(A_local.min().item()) if rc else float("inf")], device=dev)
    hi = torch.tensor([float(A_local.max().item()) if rc else float("-inf")], device=dev)
    if world > 1:
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    want_scale = chk.scale(np.float32(lo.item()), np.float32(hi.item()))
    got_scale = np.float32(scale_dev.item())
    chk.expect(want_scale.tobytes() == got_scale.tobytes(), "activation scale %r, oracle %r" % (got_scale, want_scale))
    rng = np.random.default_rng(1000 + rank)
    for _ in range(32 if rc else 0):
        m, k0 = int(rng.integers(0, rc)), int(rng.integers(0, max(1, K - 4096)))
        xs = A_local[m, k0:k0 + 4096].cpu().numpy()
        chk.expect(np.array_equal(chk.quantize(xs, want_scale), xq[r0 + m, k0:k0 + 4096].cpu().numpy()),
                   "int8 activation, row %d" % (r0 + m))
    if world > 1:
        # every rank must hold the same int8 activation: per-row checksums (a plain and a weighted sum of the
        # row's 8-byte words, modulo 2^64) are compared with rank 0's
        words = xq.view(-1, K).view(torch.int64) if K % 8 == 0 else xq.view(-1, K).to(torch.int64)
        wts = torch.arange(words.shape[1], device=dev, dtype=torch.int64) * 2 + 1
        sums = torch.stack([words.sum(1), (words * wts).sum(1)])
        ref = sums.clone()
        dist.broadcast(ref, src=0)
        chk.expect(bool(torch.equal(ref, sums)), "int8 activation differs from rank 0's copy")
    count = wq.shape[0]
    tiles = 64 if world == 1 else 32
    ws_host = wsc.cpu().numpy()
    for t in range(tiles if count else 0):
        if world > 1 and t % 2 == 1 and M > rc:             # rows that arrived from another rank
            m0 = (r0 + rc + int(rng.integers(0, M - rc - 127))) % M
            m0 = min(m0, M - 128)
        else:
            m0 = r0 + int(rng.integers(0, max(1, rc - 127))) if rc >= 128 else int(rng.integers(0, max(1, M - 127)))
        n0 = int(rng.integers(0, max(1, count - 127)))
        rows = min(128, M - m0)
        want = chk.tile(xq[m0:m0 + rows].cpu().numpy(), wq[n0:n0 + 128].cpu().numpy(), want_scale, ws_host[n0:n0 + 128])
        got = out[m0:m0 + rows, n0:n0 + 128].cpu().numpy()
        chk.expect(np.array_equal(got.view(np.uint32), want.view(np.uint32)), "output tile at (%d, %d)" % (m0, n0))


def run_ours(a):
    import torch
    import torch.distributed as dist

    from rpl_b200 import device as D
    from rpl_b200.sharded import RowShardedLinear, ShardedQuantizedLinear, shard_range

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
    chk = None
    if not a.no_parity:
        os.environ["OMP_NUM_THREADS"] = str(max(1, (os.cpu_count() or 1) // max(world, 1)))   # torchrun pins it to 1
        chk = Checker()
    if a.sweep_only:
        if a.sweep_elements:
            print(json.dumps({"quantize_sweep": quantize_sweep_one(torch, D, dev, peaks, a.sweep_elements, chk),
                              "parity": chk.result() if chk else None}), flush=True)
            return
        print(json.dumps({"quantize_sweep": quantize_sweep(torch, D, dev, peaks, chk),
                          "parity": chk.result() if chk else None}), flush=True)
        return

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    replicated = a.schedule == "replicated" and world > 1
    # ---- synthetic inputs: this rank's rows of A (all of A under the replicated schedule), its rows of W ----
    r0, rc = (0, M) if replicated else shard_range(M, world, rank, 128)
    A_local = rows_of_a(torch, dev, M, K, r0, rc)
    ops_total = 2.0 * M * N * K

    def weight_rows(begin, count):
        """Rows [begin, begin + count) of the synthetic weight ~ N(0, 0.02), quantized per output channel: generated
        in units of 256 rows, each from its own seed, so that every split of the columns yields the same matrix."""
        g = torch.Generator(device=dev)
        wq = torch.empty((count, K), dtype=torch.int8, device=dev)
        wsc = torch.empty(count, dtype=torch.float32, device=dev)
        u = begin // 256
        while u * 256 < begin + count:
            g.manual_seed(0x5EED0051 + 104729 * u)
            w = torch.randn((min(256, N - u * 256), K), device=dev, generator=g) * 0.02
            q, sc, _ = D.quantize_per_channel(w)
            lo, hi = max(begin, u * 256), min(begin + count, (u + 1) * 256)
            wq[lo - begin:hi - begin] = q[lo - u * 256:hi - u * 256]
            wsc[lo - begin:hi - begin] = sc[lo - u * 256:hi - u * 256]
            u += 1
        return wq, wsc

    class State:
        pass
    st = State()

    def build(column_counts):
        """This rank's weights, output block and layer for a split of the columns (None = even)."""
        if column_counts is None:
            st.begin, st.count = shard_range(N, world, rank, 256)
        else:
            st.begin, st.count = sum(column_counts[:rank]), column_counts[rank]
        st.wq, st.wsc = weight_rows(st.begin, st.count)
        st.out = torch.empty((M, st.count), dtype=torch.float32, device=dev)
        if replicated:
            st.old = ShardedQuantizedLinear(st.wq, st.wsc, None, n_total=N, rank=rank, world=world)
            st.layer = None
        else:
            st.layer = RowShardedLinear(st.wq, st.wsc, None, n_total=N, max_rows=M, rank=rank, world=world, column_counts=column_counts)
            if a.transfer:
                st.layer.transfer(a.transfer)

    build(None)

    def quantize_half():
        if replicated:
            st.old.quantize_activation(A_local)
        else:
            st.layer.quantize(A_local, M)

    def gemm_half():
        if replicated:
            st.old.gemm(st.old._xq, st.old._params[D.QPARAM_SCALE_SYM:D.QPARAM_SCALE_SYM + 1], out=st.out)
        else:
            st.layer.gemm(M, st.out)

    # ---- N > 1: the GPUs of a node do not sustain the same clock under their power cap, and a step ends when the
    # slowest rank does.  Measure every rank's GEMM under sustained load and deal the columns out in proportion to speed. ----
    balance = None
    if world > 1 and not replicated and a.balance and not a.no_balance:
        from rpl_b200.sharded import weighted_column_counts
        # About a second of steps first: what counts is the clock each GPU settles at under its power cap, and a
        # cold GPU runs faster than that.  Every rank runs the same number of steps (a step contains a collective).
        t_pre = time.time()
        for _ in range(3):
            quantize_half()
            gemm_half()
        torch.cuda.synchronize()
        n_pre = torch.tensor([max(1, min(2000, int(1.0 / max((time.time() - t_pre) / 3, 1e-4))))], device=dev)
        dist.broadcast(n_pre, src=0)
        for _ in range(int(n_pre.item())):
            quantize_half()
            gemm_half()
        pairs = []
        for _ in range(8):
            quantize_half()
            e_a, e_b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e_a.record()
            gemm_half()
            e_b.record()
            pairs.append((e_a, e_b))
        torch.cuda.synchronize()
        mine = torch.tensor([sum(event_ms(pairs)) / len(pairs)], device=dev, dtype=torch.float64)
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        times = [float(t.item()) for t in every]
        counts = weighted_column_counts(N, [1.0 / t for t in times])
        even = [shard_range(N, world, r, 256)[1] for r in range(world)]
        # Run-to-run noise of a GPU's GEMM time is about 2 %: re-split only for a spread well above that.
        spread = max(times) / min(times)
        if spread < a.balance_threshold:
            counts = even
        balance = {"gemm_ms_even_split": [round(t, 4) for t in times], "spread": round(spread, 4), "threshold": a.balance_threshold,
                   "columns_even_split": even, "columns": counts}
        if counts != even and min(counts) > 0:
            dist.barrier()
            st.layer.close()
            del st.out, st.wq, st.wsc
            torch.cuda.empty_cache()
            build(counts)
    count, out, wq, wsc, layer = st.count, st.out, st.wq, st.wsc, st.layer
    ops_rank = 2.0 * M * count * K

    def step_fn():
        quantize_half()
        gemm_half()

    # ---- device-resident timing ----
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
    for i in range(a.steps):
        quant_ev[i][0].record()
        quantize_half()
        quant_ev[i][1].record()
        gemm_ev[i][0].record()
        gemm_half()
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

    # ---- samples of the results against the oracle (outside every timed region) ----
    if chk is not None and layer is not None:
        check_main_results(torch, dist, chk, layer, A_local, out, wq, wsc, M, K, world, rank, dev)

    # ---- every element of the full-size output: the tensor-core kernel against the dp4a kernel ----
    if chk is not None and layer is not None and world == 1 and count:
        try:
            other = torch.empty_like(out)
        except RuntimeError:
            other = None
        if other is not None:
            xq_all, scale_dev = layer.activation(M)
            D.gemm_backend(1)
            D.linear_i8_dequant(xq_all, wq, scale_dev, wsc, out=other)
            D.gemm_backend(a.gemm_backend)
            torch.cuda.synchronize()
            chk.expect(bool(torch.equal(other, out)), "tcgen05 and dp4a kernels disagree somewhere in the %d x %d output" % (M, count))
            del other
            torch.cuda.empty_cache()

    # ---- optional: all-gather of the column blocks, timed on its own ----
    gather = None
    if a.gather and world > 1 and layer is not None:
        full = layer.gather(out, M)                         # warm-up: NCCL channels and buffers
        del full
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 3
        g0.record()
        for _ in range(reps):
            full = layer.gather(out, M)
            del full
        g1.record()
        barrier()
        tg = torch.tensor([g0.elapsed_time(g1) / reps], device=dev)
        dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        received = float(M) * (N - count) * 4
        gather = {"ms": float(tg.item()), "received_bytes_per_rank": received,
                  "GB/s_per_rank_in": received / (float(tg.item()) * 1e-3) / 1e9,
                  "what": "NCCL all-gather of fp32 [M, N/G] blocks plus unpack into row-major [M, N] on every rank"}

    # ---- end to end through host buffers ----
    e2e = None
    if not a.no_e2e and layer is not None:
        xh = oh = None
        try:
            near = NearGpu(torch, dev)
            if a.no_numa:
                near.cpus = None
            with near:
                xh = torch.empty((max(rc, 1), K), dtype=torch.float32, pin_memory=True)
                oh = torch.empty((M, max(count, 1)), dtype=torch.float32, pin_memory=True)
                oh.zero_()                                  # touch the pages while the process is near its GPU
            have = 1
        except RuntimeError:
            have = 0
        agreed = torch.tensor([have], device=dev)
        if world > 1:
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)          # all ranks take the same branch
        if int(agreed.item()) == 0:
            e2e = {"value": None, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                   "error": "page-locked host buffers (%.1f GiB per rank) could not be allocated" % ((rc * K + M * count) * 4 / 2**30)}
        else:
            if rc:
                xh[:rc].copy_(A_local)
            torch.cuda.synchronize()
            # The C ABI's host-buffer call (rplb_sharded_linear_submit_host / _drain): every call uploads this
            # rank's rows of A and downloads its whole output block, row block by row block while the next
            # block computes; the upload of call n+1 overlaps the download of call n (PCIe is full duplex).
            # Quantize and GEMM run on `estream`, which after the drain has also waited for the downloads,
            # so the events see it all.
            estream = torch.cuda.Stream(device=dev)
            estream.wait_stream(torch.cuda.current_stream())

            def submit():
                layer.submit_host(xh, M, oh, row_blocks=8, stream=estream)

            submit()
            layer.drain()
            esteps = max(2, min(a.steps, 6))
            barrier()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            launches_e0 = D.launch_count()
            s0.record(estream)
            for _ in range(esteps):
                submit()
            layer.drain()
            s1.record(estream)
            barrier()
            e2e_launches = D.launch_count() - launches_e0
            te = torch.tensor([s0.elapsed_time(s1) / esteps], device=dev)
            if world > 1:
                dist.all_reduce(te, op=dist.ReduceOp.MAX)
            same = bool(torch.equal(oh[:256].to(dev), out[:256])) and bool(torch.equal(oh[M - 256:].to(dev), out[M - 256:]))
            if chk is not None:
                chk.expect(same, "host-buffer call differs from the device-resident run")
            e2e = {"value": ops_total / (float(te.item()) * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": float(te.item()),
                   "steps": esteps, "h2d_bytes_per_step": int(M * K * 4), "d2h_bytes_per_step": int(M * N * 4),
                   "api": "rplb_sharded_linear_submit_host / rplb_sharded_linear_drain (C ABI, page-locked host buffers; "
                          "every rank uploads its own rows of A and downloads its own output columns)",
                   "matches_device_run": same, "gpu_launches": int(e2e_launches),
                   "host_buffers": "page-locked, allocated on the CPUs next to the GPU (%d CPUs)" % len(near.cpus) if near.cpus
                   else "page-locked, no CPU affinity set"}
        del xh, oh

    parity = None
    if chk is not None:
        counts = torch.tensor([chk.checked, chk.mismatches], device=dev)
        if world > 1:
            dist.all_reduce(counts)
        parity = chk.result()
        parity["checked"], parity["mismatches"] = int(counts[0].item()), int(counts[1].item())
        parity["what"] = ("per rank: the agreed scale, 32 windows of the int8 activation, per-block checksums of the whole int8 "
                          "activation against rank 0's, %d output tiles of 128 x 128 (half on rows received from other ranks), "
                          "the host-buffer result against the device-resident one%s" % (64 if world == 1 else 32, "; every element of the output against "
                          "the dp4a kernel's" if world == 1 else ""))

    if layer is not None:
        if world > 1:
            dist.barrier()
        layer.close()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # DRAM traffic of the GEMM from ncu captures at 16384 x 16384 x 8192 (dram read + write) per output element
    # at K = 8192: 9.42 B for the kernel with 256 x 256 tiles (the library's choice for a GEMM this long),
    # 7.13 B for the kernel with 128 x 256 tiles.
    wide = a.gemm_backend == 5 or (a.gemm_backend == 0 and float(M) * count * K >= 1.1e12 and K >= 6144)
    traffic = (9.42 if wide else 7.13) * M * count if K == 8192 and a.gemm_backend in (0, 3, 5) else None
    int8_peak = 2.0 * peaks["bf16_sustained"]
    achieved = ops_rank / (gemm_ms * 1e-3) / 1e12
    sched = ("every rank: min/max of its rows, max-all-reduce of (-min, max), quantize its rows, peer copies of the int8 rows "
             "to the other ranks under the GEMM, GEMM over all rows (waits per 128-row block)") if not replicated else \
        "replicated A: every rank quantizes all rows (comparison schedule)"
    line = {
        "metric": METRIC, "value": ops_total / (ms_max * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
        "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms_max, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": workload_name(a), "parallelism": "output columns and activation rows split over %d rank(s), output left column-sharded" % world,
                   "columns_per_rank": count, "rows_per_rank": rc, "schedule": sched,
                   "column_split": ("in proportion to each rank's GEMM speed measured under sustained load before the timed region" if balance and balance["columns"] != balance["columns_even_split"]
                                    else "even"),
                   "l2": "no flush: per-step inputs and outputs exceed L2 (A rows %.2f GiB fp32, int8 A %.2f GiB, out %.1f GiB per rank)"
                   % (rc * K * 4 / 2**30, M * K / 2**30, M * count * 4 / 2**30)},
        "breakdown_ms": {"quantize_A_and_scale_agreement": quant_ms, "gemm_with_epilogue": gemm_ms,
                         "per_rank_gemm_quant_step": per_rank},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOP/s",
                     "frac": achieved / int8_peak, "traffic": traffic, "traffic_unit": "bytes per launch (ncu dram read+write, scaled by output elements)",
                     "algorithmic_bytes": float(M * K + count * K + 4 * M * count),
                     "launches_per_step": 1, "kernel": "gemm_i8_tc_wide_kernel" if wide else "gemm_i8_tc_kernel",
                     "peak_note": "2 x bf16_tflops_sustained of %s (int8 dense = 2 x bf16 dense)" % peaks["source"],
                     "frac_of_nominal_4500": achieved / 4500.0,
                     "ms_x_mhz": gemm_ms * clocks["sm_mhz"] if clocks.get("sm_mhz") else None},
        "clocks": clocks, "gpu_launches": int(launches), "e2e": e2e, "parity": parity,
    }
    if balance is not None:
        line["balance"] = balance
    if gather is not None:
        line["gather"] = gather
    del A_local, out
    st.out = st.layer = None
    torch.cuda.empty_cache()
    if world == 1 and not a.no_sweep:
        line["quantize_sweep"] = quantize_sweep(torch, D, dev, peaks, chk)
        if chk is not None:
            line["parity"].update(chk.result())
    if world == 1 and not a.no_secondary:
        del wq, wsc
        st.wq = st.wsc = None
        torch.cuda.empty_cache()
        line["secondary"] = {}
        for wl in ("c1", "c2", "c3"):
            b = argparse.Namespace(**vars(a))
            b.workload, b.steps = wl, 50 if wl != "c3" else 10
            line["secondary"][wl] = secondary_line(torch, D, dev, peaks, b, chk)
            torch.cuda.empty_cache()
        if chk is not None:
            line["parity"].update(chk.result())
    if world == 1 and not a.no_probe:
        # Last of the GPU legs: seconds of dense tensor work leave the board at its power cap, which the
        # memory-bound figures above must not inherit.
        line["roofline"]["int8_probe"] = int8_probe(torch, dev)
        p = line["roofline"]["int8_probe"]
        p["frac_of_probe_sustained"] = achieved / p["sustained_tops"]
    if world == 1 and not a.no_cpu:
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


def timed_replay(torch, D, dev, step, steps, warmup):
    """ms per step of `step` replayed from a CUDA graph (these steps are a handful of short kernels: the
    host's launch cost must not show up as GPU idle time), and the library's launches per step."""
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(max(warmup, 3)):                     # also sizes the library's scratch block of this stream
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
    for _ in range(steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    if D.kernel_status(True) != 0:
        raise RuntimeError("the tcgen05 kernel reported an expired wait")
    return e0.elapsed_time(e1) / steps, per_step


def layers_through_c_api(torch, capi, C, dev, shapes, X, reps, what, shared=False):
    """ms per pass of quantized Linear layers driven through the reference-style C objects (quantized_linear_create /
    _forward / _forward_shared_input) on device-resident tensors: what a C caller of the layer API pays per call."""
    L = capi.load()

    def dev_tensor(t):
        shape = (C.c_uint32 * t.dim())(*t.shape)
        p = L.tensor_create_device(t.dim(), shape)
        capi.call("rplb_copy", C.c_void_p(p.contents.data), C.c_void_p(t.data_ptr()), t.numel() * 4, None)
        return p

    g = torch.Generator(device=dev)
    g.manual_seed(99)
    layers = []
    for (n_out, n_in, _) in shapes:
        w = dev_tensor(torch.randn((n_out, n_in), device=dev, generator=g) * 0.05)
        b = dev_tensor(torch.randn(n_out, device=dev, generator=g) * 0.05)
        capi.call("rplb_stream_sync", None)
        layers.append(L.quantized_linear_create(w, b))
        L.tensor_free(w)
        L.tensor_free(b)
    x = dev_tensor(X)
    capi.call("rplb_stream_sync", None)

    def one_pass():
        if shared:
            arr = (C.c_void_p * len(layers))(*layers)
            outs = (C.POINTER(capi.Tensor) * len(layers))()
            if L.quantized_linear_forward_shared_input(arr, len(layers), x, outs, False) != 0:
                raise RuntimeError("quantized_linear_forward_shared_input failed")
            for o in outs:
                L.tensor_free(o)
        else:
            cur = x
            for layer, (_, _, relu) in zip(layers, shapes):
                nxt = L.quantized_linear_forward(layer, cur, relu)
                if not nxt:
                    raise RuntimeError("quantized_linear_forward failed")
                if cur is not x:
                    L.tensor_free(cur)
                cur = nxt
            L.tensor_free(cur)

    one_pass()
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        one_pass()
        ts.append(time.perf_counter() - t0)
    ts.sort()
    for layer in layers:
        L.quantized_linear_free(layer)
    L.tensor_free(x)
    return {"ms": ts[len(ts) // 2] * 1e3, "what": what}


def secondary_line(torch, D, dev, peaks, a, chk=None):
    """One of the smaller configurations on one GPU: device-resident timing, same metric; where the
    configuration is what a drop-in user calls with host buffers (512^3), that call is timed too."""
    import ctypes as C

    import numpy as np

    from rpl_b200 import capi
    g = torch.Generator(device=dev)
    g.manual_seed(0x5EED0000 + int(a.workload[1]) * 16)
    one = lambda p: p[D.QPARAM_SCALE_SYM:D.QPARAM_SCALE_SYM + 1]
    extra = {}
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
        # The call a drop-in user makes: gemm_int8(A, B, C, 512, 512, 512, ...) of the reference's API with
        # host buffers (upload, kernel, download, synchronize), beside the reference's CPU code on the same bytes.
        L = capi.load()
        rng = np.random.default_rng(0x5EED0010)
        Ah = rng.integers(-127, 128, (512, 512), dtype=np.int8)
        Bh = rng.integers(-127, 128, (512, 512), dtype=np.int8)
        Ch = np.zeros((512, 512), np.int32)
        args = (Ah.ctypes.data, Bh.ctypes.data, Ch.ctypes.data, 512, 512, 512, 0.011, 0.013, 0.37, 0, 0)
        for _ in range(5):
            L.gemm_int8(*args)
        ts = []
        for _ in range(30):
            t0 = time.perf_counter()
            L.gemm_int8(*args)
            ts.append(time.perf_counter() - t0)
        ts.sort()
        extra["gemm_int8_host_call"] = {"ms": ts[len(ts) // 2] * 1e3, "gops": ops / ts[len(ts) // 2] / 1e9,
                                        "what": "gemm_int8 of the reference's C API, host buffers in and out, per call (median of 30)"}
        # linear_int8 of the reference's API on device-resident int8 tensors (the call synchronises before it returns)
        qa, qb = capi.QuantizedTensor(), capi.QuantizedTensor()
        qa.data, qb.data = aq.data_ptr(), bq.data_ptr()
        acc = torch.empty((512, 512), dtype=torch.int32, device=dev)
        for _ in range(5):
            L.linear_int8(C.byref(qa), C.byref(qb), None, C.c_void_p(acc.data_ptr()), 512, 512, 512)
        ts = []
        for _ in range(50):
            t0 = time.perf_counter()
            L.linear_int8(C.byref(qa), C.byref(qb), None, C.c_void_p(acc.data_ptr()), 512, 512, 512)
            ts.append(time.perf_counter() - t0)
        ts.sort()
        extra["linear_int8_device_call"] = {"us": ts[len(ts) // 2] * 1e6,
                                            "what": "linear_int8 of the reference's C API, device-resident operands, launch + synchronize per call (median of 50)"}
        if chk is not None:
            cpu = chk.ref or chk.port
            cpu.gemm_requant(Ah, Bh, 0.011, 0.013, 0.37)
            tc = []
            for _ in range(5):
                t0 = time.perf_counter()
                want = cpu.gemm_requant(Ah, Bh, 0.011, 0.013, 0.37)
                tc.append(time.perf_counter() - t0)
            tc.sort()
            extra["gemm_int8_cpu_" + chk.name] = {"ms": tc[len(tc) // 2] * 1e3, "gops": ops / tc[len(tc) // 2] / 1e9,
                                                  "cores": chk.port.num_threads()}
            chk.expect(np.array_equal(Ch, want), "512^3 gemm_int8 through the C API")
    elif a.workload == "c2":
        name = "quantized MLP 784->128->10, batch 65536: X U[0,1) per tensor, W N(0,0.05) per channel, ReLU, fp32 logits"
        Bn = 65536
        X = torch.rand((Bn, 784), device=dev, generator=g)
        w1q, w1s, _ = D.quantize_per_channel(torch.randn((128, 784), device=dev, generator=g) * 0.05)
        w2q, w2s, _ = D.quantize_per_channel(torch.randn((10, 128), device=dev, generator=g) * 0.05)
        b1 = torch.randn(128, device=dev, generator=g) * 0.05
        b2 = torch.randn(10, device=dev, generator=g) * 0.05
        xq, px = torch.empty((Bn, 784), dtype=torch.int8, device=dev), torch.empty(8, device=dev)
        h = torch.empty((Bn, 128), device=dev)
        logits = torch.empty((Bn, 10), device=dev)
        ops = 2.0 * Bn * (784 * 128 + 128 * 10)
        # X read twice (min/max, quantize) + int8 X written and read + hidden fp32 written and read once
        # (its quantize rides inside the last layer: no int8 copy of it) + logits
        hbm_bytes = Bn * (784 * (4 + 4 + 1 + 1) + 128 * (4 + 4) + 10 * 4)
        stats = torch.empty(2, device=dev)

        def step():
            D.quantize_symmetric(X, out=xq, params=px)
            # layer 1 (the kernel for few output features): fused dequant + bias + ReLU; the epilogue also
            # reports max|h| and the scale of h
            capi.call("rplb_linear_i8_dequant_f32_absmax", C.c_void_p(xq.data_ptr()), C.c_void_p(w1q.data_ptr()),
                      C.c_void_p(h.data_ptr()), Bn, 784, 128, 128, C.c_void_p(one(px).data_ptr()),
                      C.c_void_p(w1s.data_ptr()), C.c_void_p(b1.data_ptr()), 1, C.c_void_p(stats[0:1].data_ptr()),
                      C.c_void_p(stats[1:2].data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
            # layer 2: h is quantized with that scale on its way into the contraction (N = 10: dp4a kernel)
            D.quantize_linear_dequant(h, w2q, stats[1:2], w2s, b2, relu=False, out=logits)
        note = "HBM-bound: 13.3 GOP over ~0.6 GB of traffic; three kernels after the min/max pass"
        extra["c_api"] = layers_through_c_api(torch, capi, C, dev, [(128, 784, True), (10, 128, False)], X, 5,
                                              "quantized_linear_create + quantized_linear_forward per layer (device-resident tensors; "
                                              "each call allocates its output and synchronises)")
    else:
        name = ("transformer projections: tokens 32768 x d_model 4096, Q/K/V as one GEMM with N = 12288 plus O (N = 4096), "
                "weights per channel, bias, fp32 out")
        T, Dm = 32768, 4096
        X = torch.randn((T, Dm), device=dev, generator=g)
        ws_ = [D.quantize_per_channel(torch.randn((Dm, Dm), device=dev, generator=g) * 0.02) for _ in range(4)]
        bs = [torch.randn(Dm, device=dev, generator=g) * 0.02 for _ in range(4)]
        wqkv = torch.cat([w[0] for w in ws_[:3]]).contiguous()                      # [12288, 4096] int8
        sqkv = torch.cat([w[1] for w in ws_[:3]]).contiguous()
        bqkv = torch.cat(bs[:3]).contiguous()
        qkv = torch.empty((T, 3 * Dm), device=dev)
        o = torch.empty((T, Dm), device=dev)
        xq, px = torch.empty((T, Dm), dtype=torch.int8, device=dev), torch.empty(8, device=dev)
        ops, hbm_bytes = 4 * 2.0 * T * Dm * Dm, None

        def step():
            D.quantize_symmetric(X, out=xq, params=px)
            D.linear_i8_dequant(xq, wqkv, one(px), sqkv, bqkv, out=qkv)
            D.linear_i8_dequant(xq, ws_[3][0], one(px), ws_[3][1], bs[3], out=o)
        note = "X quantized once per step; Q/K/V in one launch (N = 12288), O in a second; fused per-channel dequant + bias"
        extra["c_api"] = layers_through_c_api(torch, capi, C, dev, [(Dm, Dm, False)] * 4, X, 3,
                                              "quantized_linear_forward_shared_input over four layers (device-resident tensors; the call "
                                              "allocates its outputs and synchronises)", shared=True)
    ms, per_step = timed_replay(torch, D, dev, step, a.steps, a.warmup)
    if a.workload == "c3" and chk is not None:
        # tiles of the fused Q/K/V output and of O against the oracle
        step()
        torch.cuda.synchronize()
        sa = np.float32(px[D.QPARAM_SCALE_SYM].item())
        rng = np.random.default_rng(3)
        for t in range(12):
            m0 = int(rng.integers(0, T - 128))
            wmat, smat, bvec, res = (wqkv, sqkv, bqkv, qkv) if t < 9 else (ws_[3][0], ws_[3][1], bs[3], o)
            n0 = int(rng.integers(0, wmat.shape[0] - 128))
            want = chk.tile(xq[m0:m0 + 128].cpu().numpy(), wmat[n0:n0 + 128].cpu().numpy(), sa, smat[n0:n0 + 128].cpu().numpy())
            want = want + bvec[n0:n0 + 128].cpu().numpy()[None, :]
            got = res[m0:m0 + 128, n0:n0 + 128].cpu().numpy()
            chk.expect(np.array_equal(got.view(np.uint32), want.astype(np.float32).view(np.uint32)), "projection tile (%d, %d)" % (m0, n0))
    line = {"metric": METRIC, "value": ops / (ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": 1, "steps": a.steps,
            "warmup": max(a.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": {"workload": name, "note": note, "replay": "CUDA graph of one step"},
            "gpu_launches": int(per_step * a.steps)}
    line.update(extra)
    if hbm_bytes:
        gbs = hbm_bytes / (ms * 1e-3) / 1e9
        line["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": gbs / peaks["hbm_gbs"], "traffic": None}
    else:
        t = ops / (ms * 1e-3) / 1e12
        line["roofline"] = {"bound": "tensor", "achieved": t, "peak": 2.0 * peaks["bf16_sustained"], "unit": "TOP/s",
                            "frac": t / (2.0 * peaks["bf16_sustained"]), "traffic": None}
    return line


def run_secondary(a):
    """`--workload c1|c2|c3` on its own: one JSON line for that configuration."""
    import torch

    from rpl_b200 import device as D
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    D.gemm_backend(a.gemm_backend)
    D.gemm_epilogue(a.gemm_epilogue)
    chk = None if a.no_parity else Checker()
    line = secondary_line(torch, D, dev, measured_peaks(), a, chk)
    if chk is not None:
        line["parity"] = chk.result()
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
