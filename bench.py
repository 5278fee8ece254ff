"""Benchmark of the semiring batched-matmul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference-cuda]

A step is one logbmm forward + backward (loss = c.sum()) over a batch of `--batch` problems of
size 1024x1024x1024 per GPU (the "1024^3 per batch element" throughput configuration); the
metric is semiring multiply-accumulates per second, 3*B*M*K*N per step (forward, grad_a and
grad_b each touch every (m,k,n) triple once).  The same step for maxbmm is timed beside it and
reported under "also".  Inputs are seeded synthetic tensors, larger than the L2 cache.

A step takes about a millisecond, so the timed region runs every counted step `inner_repeats` times
back to back (chosen so that the region lasts about two seconds; ms_per_step is per single step):
long enough for the clock sampler to see the region itself and for the power cap to settle.

With N > 1 (torchrun, one process per GPU) every rank runs the same per-GPU workload on its own
batch shard; there is no data-path collective.  The time is the maximum over ranks of the
CUDA-event duration, the value the total over ranks.  "configs" then holds the sharded forms of the
other benchmark configurations: the chain (CRF) configuration by batch shards and by batch x
chain-chunk shards (one NCCL all-gather), the banded configuration by batch shards, and the
strong-scaling form of the throughput configuration (global batch 64).

`--impl reference` times the reference's own CPU formulation of logbmm — the broadcast-reduce
PyTorch expression of its README and tests — on the host cores, on a bounded sample of the
same workload.  `--impl reference-cuda` times the reference's own CUDA kernels, recompiled for
sm_100a by baseline/build_ref.py, on the same workload on one GPU.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SIZE = 1024
N_SMS = 148
SFU_PER_SM_CLK = 16     # ex2 results per SM per clock
FP32_PER_SM_CLK = 128   # FP32 lanes per SM per clock
TARGET_REGION_S = 2.0   # length of the timed region of the headline


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p.get("hbm_gbs", 6650.0), "sm_max_mhz": p.get("sm_max_mhz", 1965.0),
                "bf16_tflops": p.get("bf16_tflops", 1590.0),
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", 1400.0), "source": "measured"}
    return {"hbm_gbs": 6650.0, "sm_max_mhz": 1965.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi (100 ms period); every sample carries the host
    time at which it was read, so that `window(t0, t1)` reports on exactly the samples taken inside a region."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append((time.perf_counter(), parts))

    def stop(self):
        if self.proc is None:
            return
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()

    def window(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        mhz, reasons, mx = [], set(), None
        for t, s in list(self.samples):
            if not (t0 <= t <= t1):
                continue
            try:
                mhz.append(float(s[0]))
                mx = float(s[1])
            except ValueError:
                continue
            for name, flag in zip(self.NAMES, s[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz), "sm_mhz_min": mhz[0] if mhz else None, "sm_mhz_max": mhz[-1] if mhz else None}


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference's own formulation on the host cores
# ------------------------------------------------------------------------------------------------

def cpu_logbmm_sample(rows, chunk, repeats=1):
    """The reference's CPU formulation (broadcast-reduce expression + autograd), timed on `rows` rows
    of one 1024^3 batch element, in chunks of `chunk` rows.  Returns (MAC/s, seconds, threads)."""
    import oracle
    gen = torch.Generator().manual_seed(5)
    a = torch.randn(1, rows, SIZE, generator=gen)
    b = torch.randn(1, SIZE, SIZE, generator=gen)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        for s in range(0, rows, chunk):
            oracle.expr_fwd_bwd(oracle.MODE_LOG, a[:, s:s + chunk], b)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    macs = 3.0 * rows * SIZE * SIZE
    return macs / best, best, torch.get_num_threads()


def host_threads():
    """All host threads this process may use (torchrun pins OMP_NUM_THREADS=1 per rank; undo that
    for the single rank that runs the CPU arm)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def workload_config(args):
    return {"workload": "logbmm fwd+bwd, a,b:(%d,%d,%d) fp32 N(0,1) seed 5 per GPU, loss=c.sum()" % (
        args.batch, SIZE, SIZE), "batch_per_gpu": args.batch, "M": SIZE, "K": SIZE, "N": SIZE,
        "parallelism": "batch-sharded, no collective", "l2": "working set %d MB per GPU, larger than L2" % (
            6 * args.batch * 4 * SIZE * SIZE >> 20)}


def run_reference(args, rank, world):
    if rank != 0:
        return
    host_threads()
    rows, chunk = 512, 64
    for _ in range(args.warmup):
        cpu_logbmm_sample(chunk, chunk)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        value, _, threads = cpu_logbmm_sample(rows, chunk)
    dt = (time.perf_counter() - t0) / args.steps
    macs = 3.0 * rows * SIZE * SIZE
    value = macs / dt
    sample = "per step: %d rows of one 1024x1024x1024 batch element, forward + autograd backward, %d-row chunks" % (
        rows, chunk)
    line = {
        "impl": "reference", "metric": "logbmm fwd+bwd semiring MAC/s", "value": value, "unit": "MAC/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args),
        "cpu_baseline": {"value": value, "unit": "MAC/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "MAC/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# The reference's own CUDA kernels (baseline/_ref, built by baseline/build_ref.py), one GPU
# ------------------------------------------------------------------------------------------------

def run_reference_cuda(args, rank, world):
    """harvardnlp/genbmm's kernels recompiled for sm_100a, through its own Python operators
    (genbmm.logbmm / maxbmm + autograd), on the workload of the headline and on configs 1-3 and 5.
    Nothing of this package is loaded in this process."""
    if rank != 0:
        return
    ref = os.path.join(ROOT, "baseline", "_ref")
    line = {"impl": "reference-cuda"}
    try:
        if not os.path.isdir(ref):
            raise RuntimeError("baseline/_ref is absent (run baseline/build_ref.py where the reference checkout is)")
        sys.path.insert(0, ref)
        import _genbmm  # noqa: F401  (the reference's extension; its Python files import it by this name)
        import genbmm.genmul as rg
        import genbmm.sparse as rs
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
    except Exception as exc:
        line["unavailable"] = "%s: %s" % (type(exc).__name__, str(exc).splitlines()[0] if str(exc) else "")
        print(json.dumps(line), flush=True)
        return
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)

    def fwd_bwd_ms(fn, a, b, iters, warm):
        a, b = a.to(dev).requires_grad_(True), b.to(dev).requires_grad_(True)

        def step():
            c = fn(a, b)
            torch.autograd.grad(c, (a, b), torch.ones_like(c))
        return median_ms(step, iters, warm)

    B = args.batch
    gen = torch.Generator().manual_seed(5)
    a = torch.randn(B, SIZE, SIZE, generator=gen)
    b = torch.randn(B, SIZE, SIZE, generator=gen)
    steps = max(1, min(args.steps, 5))
    t_log = fwd_bwd_ms(rg.logbmm, a, b, steps, 1) / 1e3
    t_max = fwd_bwd_ms(rg.maxbmm, a, b, steps, 1) / 1e3
    macs = 3.0 * B * SIZE ** 3
    configs = {}
    g1 = torch.Generator().manual_seed(0)
    x, y = torch.rand(32, 64, 64, generator=g1), torch.rand(32, 64, 64, generator=g1)
    configs["cfg1_logbmm_32x64x64x64"] = {"ms": fwd_bwd_ms(rg.logbmm, x, y, 50, 10)}
    g2 = torch.Generator().manual_seed(1)
    x = (torch.randn(256, 128, 128, generator=g2) * 8).round() / 8
    y = (torch.randn(256, 128, 128, generator=g2) * 8).round() / 8
    configs["cfg2_maxbmm_256x128x128x128"] = {"ms": fwd_bwd_ms(rg.maxbmm, x, y, 50, 10)}
    configs["cfg2_prodmaxbmm_256x128x128x128"] = {"ms": fwd_bwd_ms(rg.prodmaxbmm, x, y, 50, 10)}
    g3 = torch.Generator().manual_seed(2)
    x, y = 2 * torch.randn(64, 256, 256, generator=g3), 2 * torch.randn(64, 256, 256, generator=g3)
    configs["cfg3_samplebmm_64x256x256x256"] = {"ms": fwd_bwd_ms(rg.samplebmm, x, y, 20, 5)}
    g5 = torch.Generator().manual_seed(4)
    x, y = torch.randn(32, 8192, 129, generator=g5), torch.randn(32, 8192, 129, generator=g5)
    for name in ("multiply", "multiply_log", "multiply_max"):
        def band(p, q, name=name):
            return getattr(rs.BandedMatrix(p, 64, 64), name)(rs.BandedMatrix(q, 64, 64)).data
        configs["cfg5_banded_%s_32x8192x129" % name] = {"ms": fwd_bwd_ms(band, x, y, 5, 1)}
    line.update({
        "metric": "logbmm fwd+bwd semiring MAC/s", "value": macs / t_log, "unit": "MAC/s", "n_gpus": 1,
        "steps": steps, "warmup": 1, "ms_per_step": t_log * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(args),
        "also": {"maxbmm_ms_per_step": t_max * 1e3,
                 "maxbmm_fwd_bwd_mac_per_s": (B * SIZE ** 3 + 2.0 * B * SIZE * SIZE) / t_max},
        "configs": configs,
        "what": "harvardnlp/genbmm's own CUDA kernels and Python operators, built for sm_100a by "
                "baseline/build_ref.py (dispatch-macro rename only), median of CUDA-event timings"})
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# timing helpers
# ------------------------------------------------------------------------------------------------

def median_ms(fn, iters, warmup):
    """Median CUDA-event duration (ms) of `iters` calls of fn on the current stream, one event pair per call,
    after `warmup` untimed calls."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
    evs[0].record()
    for i in range(iters):
        fn()
        evs[i + 1].record()
    torch.cuda.synchronize()
    return statistics.median(evs[i].elapsed_time(evs[i + 1]) for i in range(iters))


def region_ms(fn, calls, sync):
    """CUDA-event duration (ms) of `calls` back-to-back calls of fn, sync() on both sides."""
    sync()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(calls):
        fn()
    stop.record()
    sync()
    return start.elapsed_time(stop)


class Ranks:
    """The process group of the run (or none at N = 1): barrier + synchronize, maximum over ranks."""

    def __init__(self, dev, world):
        self.dev, self.world, self.dist = dev, world, None
        if world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=dev)
            self.dist = dist

    def sync(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max(self, x):
        t = torch.tensor([float(x)], device=self.dev, dtype=torch.float64)
        if self.dist is not None:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self):
        if self.dist is not None:
            self.dist.barrier()
            self.dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# roofline bounds of the benchmark configurations (fwd + bwd), from the pipe rates at the maximum SM clock
# ------------------------------------------------------------------------------------------------

def bounds(peaks):
    clk = peaks["sm_max_mhz"] * 1e6
    return {"sfu": N_SMS * SFU_PER_SM_CLK * clk,            # ex2 per second
            "max": N_SMS * FP32_PER_SM_CLK / 2 * clk,        # max-plus MACs per second (add + max per MAC)
            "fma": N_SMS * FP32_PER_SM_CLK * clk,            # FFMA per second
            "hbm": peaks["hbm_gbs"] * 1e9,                   # bytes per second
            "tf32": peaks["bf16_tflops"] * 1e12 / 2}         # dense TF32 FLOP/s, derived: bf16 / 2


def with_bound(entry, bound_s, what, peaks=None, tensor_flops=None):
    entry["bound"] = what
    entry["bound_ms"] = bound_s * 1e3
    entry["frac"] = bound_s * 1e3 / entry["ms"]
    if tensor_flops is not None:   # the factorised log products run on the tensor cores: second denominator
        t = tensor_flops / bounds(peaks)["tf32"]
        entry["tensor_bound_ms"] = t * 1e3
        entry["frac_of_tensor_bound"] = t * 1e3 / entry["ms"]
    return entry


def route_bytes(B, M, K, N, prod):
    """Algorithmic bytes of the index-routed backward: idx and g in, grad_a and grad_b out (plus the gathered
    operand values for prod-max)."""
    return 4.0 * (2 * B * M * N + B * M * K + B * K * N + ((B * M * K + B * K * N) if prod else 0))


CFG5_TRIPLES = 135428672          # valid (i, ja, jo) triples per batch element at n = 8192, 129 diagonals each


def cfg5_bound(mode, batch, pk):
    v = batch * CFG5_TRIPLES
    n, wa, wo = 8192, 129, 257
    fwd_bytes = 4.0 * batch * n * (2 * wa + wo)
    bwd_bytes = 4.0 * batch * n * (4 * wa + 2 * wo)
    if mode == "multiply":
        return max(3 * v / pk["fma"], (fwd_bytes + bwd_bytes) / pk["hbm"]), "FFMA 128/clk/SM (3V) vs HBM bytes"
    if mode == "multiply_max":
        return v / pk["max"] + bwd_bytes / pk["hbm"], "fwd add+max 64 MAC/clk/SM + bwd routing bytes / HBM"
    return 2 * v / pk["sfu"], "SFU ex2 16/clk/SM, 2 exp per triple"


# ------------------------------------------------------------------------------------------------
# the other configurations on one GPU
# ------------------------------------------------------------------------------------------------

def fwd_bwd_median(gb, fn, args, iters, warm):
    leaves = [x.detach().requires_grad_(True) for x in args[:2]]
    rest = list(args[2:])

    def step():
        c = fn(*leaves, *rest)
        c = c.data if isinstance(c, gb.BandedMatrix) else c
        torch.autograd.grad(c, leaves, torch.ones_like(c))

    return median_ms(step, iters, warm)


def chain_elements(elements, lo=0, hi=511, dev=None, C=256):
    """Potentials of the chain configuration: batch element e is N(0,1) from seed 3000 + e, positions [lo, hi)
    (so that any rank can draw exactly its shard).  Generated on the host, element by element."""
    out = torch.empty((len(elements), hi - lo, C, C), device=dev)
    for i, e in enumerate(elements):
        full = torch.randn(511, C, C, generator=torch.Generator().manual_seed(3000 + e))
        out[i].copy_(full[lo:hi])
    return out


def band_elements(elements, dev):
    xs, ys = [], []
    for e in elements:
        g = torch.Generator().manual_seed(4000 + e)
        xs.append(torch.randn(8192, 129, generator=g))
        ys.append(torch.randn(8192, 129, generator=g))
    return torch.stack(xs).to(dev), torch.stack(ys).to(dev)


def measure_configs(gb, dev, peaks, quick=False):
    """Forward+backward time of the other benchmark configurations on one GPU: inputs drawn on the host from
    the configuration's seed, 10 warm-up and 50 timed iterations, median of per-iteration CUDA-event times,
    each with its bound (pipe rates at the maximum SM clock, measured HBM rate) and the fraction reached."""
    from genbmm_b200 import crf
    pk = bounds(peaks)
    it, warm = (10, 3) if quick else (50, 10)
    res = {}
    gen = torch.Generator().manual_seed(0)
    a, b = (torch.rand(32, 64, 64, generator=gen).to(dev) for _ in range(2))
    t = fwd_bwd_median(gb, gb.logbmm, (a, b), it, warm)
    res["cfg1_logbmm_32x64x64x64"] = with_bound(
        {"ms": t, "mac_per_s": 3 * 32 * 64 ** 3 / t * 1e3}, 2 * 32 * 64 ** 3 / pk["sfu"],
        "SFU ex2 16/clk/SM, 2 exp per triple")
    gen = torch.Generator().manual_seed(1)
    a, b = ((torch.randn(256, 128, 128, generator=gen) * 8).round().div(8).to(dev) for _ in range(2))
    for name in ("maxbmm", "prodmaxbmm"):
        t = fwd_bwd_median(gb, getattr(gb, name), (a, b), it, warm)
        bound = 256 * 128 ** 3 / pk["max"] + route_bytes(256, 128, 128, 128, name == "prodmaxbmm") / pk["hbm"]
        res["cfg2_%s_256x128x128x128" % name] = with_bound(
            {"ms": t, "mac_per_s": 256 * 128 ** 3 / t * 1e3}, bound, "fwd 64 MAC/clk/SM + bwd routing bytes / HBM")
    gen = torch.Generator().manual_seed(2)
    a, b = (2 * torch.randn(64, 256, 256, generator=gen) for _ in range(2))
    u = torch.rand(64, 256, 256, generator=gen)
    t = fwd_bwd_median(gb, gb.samplebmm, (a.to(dev), b.to(dev), u.to(dev)), it, warm)
    bound = 2 * 64 * 256 ** 3 / pk["sfu"] + route_bytes(64, 256, 256, 256, False) / pk["hbm"]
    res["cfg3_samplebmm_64x256x256x256"] = with_bound(
        {"ms": t, "mac_per_s": 64 * 256 ** 3 / t * 1e3}, bound,
        "SFU: one exp per triple for the logsumexp and one for the inverse-CDF pass, + bwd routing bytes / HBM")
    del a, b, u
    pot = chain_elements(range(16), dev=dev)
    triples = 16 * 510 * 256 ** 3
    t = median_ms(lambda: crf.marginals(pot), it, max(3, warm // 2))
    res["cfg4_crf_B16_T512_C256"] = with_bound(
        {"ms": t, "mac_per_s": 3 * triples / t * 1e3}, 2 * triples / pk["sfu"], "SFU ex2 16/clk/SM, 2 exp per triple "
        "(the factorised tensor-core path is not bound by it)", peaks, tensor_flops=3 * 3 * 2.0 * triples)
    del pot
    x, y = band_elements(range(32), dev)
    for name in ("multiply", "multiply_log", "multiply_max"):
        def band(p, q, name=name):
            return getattr(gb.BandedMatrix(p, 64, 64), name)(gb.BandedMatrix(q, 64, 64))
        t = fwd_bwd_median(gb, band, (x, y), it, max(3, warm // 2))
        bound, what = cfg5_bound(name, 32, pk)
        res["cfg5_banded_%s_32x8192x129" % name] = with_bound(
            {"ms": t, "mac_per_s": 3.0 * 32 * CFG5_TRIPLES / t * 1e3}, bound, what)
    return res


def host_cost(gb, dev):
    """Host microseconds per call of the small configurations: wall-clock per eager forward+backward issued
    back to back without synchronising (what the host spends launching), against one CUDA-graph replay of
    the same step."""
    out = {}
    gen = torch.Generator().manual_seed(0)
    cases = {"cfg1_logbmm": (gb.logbmm, torch.rand(32, 64, 64, generator=gen), torch.rand(32, 64, 64, generator=gen)),
             "cfg2_maxbmm": (gb.maxbmm, torch.randn(256, 128, 128, generator=gen),
                             torch.randn(256, 128, 128, generator=gen))}
    for name, (fn, a, b) in cases.items():
        a, b = a.to(dev).requires_grad_(True), b.to(dev).requires_grad_(True)
        ones = torch.ones(a.shape[0], a.shape[1], b.shape[2], device=dev)

        def step():
            return torch.autograd.grad(fn(a, b), (a, b), ones)

        for _ in range(20):
            step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(200):
            step()
        host_us = (time.perf_counter() - t0) / 200 * 1e6
        torch.cuda.synchronize()
        entry = {"eager_host_us_per_step": host_us, "eager_gpu_us_per_step": median_ms(step, 100, 10) * 1e3}
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(3):
                    step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            entry["graph_replay_us_per_step"] = median_ms(graph.replay, 100, 10) * 1e3
        except Exception as exc:
            entry["graph_replay_us_per_step"] = None
            entry["graph_error"] = repr(exc)[:200]
        out[name] = entry
    return out


# ------------------------------------------------------------------------------------------------
# the sharded forms of the configurations, N ranks
# ------------------------------------------------------------------------------------------------

def measure_sharded(gb, dev, ranks, rank, world, peaks, quick=False):
    """cfg4 by batch shards and by batch x chain-chunk shards, cfg5 by batch shards, and the strong-scaling
    throughput configuration (global batch 64), each as the maximum over ranks of the median per-iteration
    CUDA-event time; `single_gpu_ms` is the same whole problem run by rank 0 alone in the same job, and
    `efficiency` = single_gpu_ms / (N x ms)."""
    from genbmm_b200 import crf
    from genbmm_b200.sharded import shard_bounds
    it, warm = (5, 2) if quick else (20, 5)
    res = {}

    def both(name, sharded_fn, single_fn, extra=None):
        ranks.sync()
        # the lower of two medians: one run of this leg came out 2.3 times slower than the same call measured a
        # minute earlier in the same process and than every other run of it
        ms = ranks.max(min(median_ms(sharded_fn, it, warm), median_ms(sharded_fn, it, 1)))
        entry = {"ms": ms}
        if world > 1:
            ranks.sync()
            single = median_ms(single_fn(), it, warm) if rank == 0 else 0.0
            single = ranks.max(single)
            entry["single_gpu_ms"] = single
            entry["efficiency"] = single / (world * ms)
        if extra:
            entry.update(extra)
        res[name] = entry
        torch.cuda.empty_cache()

    # ---- cfg4, pure batch shards: 16 chains, 16 / N per rank, no communication
    lo, hi = shard_bounds(16, rank, world)
    pot = chain_elements(range(lo, hi), dev=dev)

    def single_cfg4():
        full = chain_elements(range(16), dev=dev)
        return lambda: crf.marginals(full)

    both("cfg4_crf_batch_sharded", lambda: crf.marginals(pot), single_cfg4,
         {"chains_per_gpu": hi - lo, "collective": "none"})
    del pot
    # ---- cfg4, batch x chain-chunk: every rank holds positions [lo, hi) of all 16 chains; one all-gather of the
    # 16 partial products (16 x 256 x 256 fp32 = 4 MB per rank), then every rank finishes log2(N) levels
    clo, chi = rank * 511 // world, (rank + 1) * 511 // world
    chunk = chain_elements(range(16), clo, chi, dev=dev)

    def chunk_step():
        x = chunk.detach().requires_grad_(True)
        if world > 1:
            logz = crf.sharded_log_partition(x)
        else:
            logz = crf.log_partition(x)
        torch.autograd.grad(logz.sum(), x)

    both("cfg4_crf_chain_chunk_sharded", chunk_step, single_cfg4,
         {"positions_per_gpu": chi - clo, "collective": "one NCCL all-gather of 16x256x256 fp32 (4 MB per rank)"})
    if world > 1:   # the exchange step alone
        part = torch.randn(16, 256, 256, device=dev)
        outs = [torch.empty_like(part) for _ in range(world)]
        res["cfg4_crf_chain_chunk_sharded"]["all_gather_ms"] = ranks.max(
            median_ms(lambda: ranks.dist.all_gather(outs, part), it, warm))
        del part, outs
    del chunk
    # ---- cfg5: batch 32 sharded, three semirings
    lo, hi = shard_bounds(32, rank, world)
    x, y = band_elements(range(lo, hi), dev)
    for name in ("multiply", "multiply_log", "multiply_max"):
        def band_step(p, q, name=name):
            a, b = p.detach().requires_grad_(True), q.detach().requires_grad_(True)
            r = getattr(gb.BandedMatrix(a, 64, 64), name)(gb.BandedMatrix(b, 64, 64)).data
            torch.autograd.grad(r, (a, b), torch.ones_like(r))

        def single_band(name=name):
            fx, fy = band_elements(range(32), dev)
            return lambda: band_step(fx, fy, name)

        both("cfg5_banded_%s_batch_sharded" % name, lambda: band_step(x, y), single_band,
             {"batch_per_gpu": hi - lo, "collective": "none"})
        from genbmm_b200 import _native
        _native.release_workspaces()
    del x, y
    # ---- strong scaling of the throughput configuration: global batch 64
    per = 64 // world
    gen = torch.Generator().manual_seed(50 + rank)
    a = torch.randn(per, SIZE, SIZE, generator=gen).to(dev).requires_grad_(True)
    b = torch.randn(per, SIZE, SIZE, generator=gen).to(dev).requires_grad_(True)
    ones = torch.ones(per, SIZE, SIZE, device=dev)
    for name, fn in (("logbmm", gb.logbmm), ("maxbmm", gb.maxbmm)):
        def strong_step(fn=fn):
            torch.autograd.grad(fn(a, b), (a, b), ones)

        def single_strong(fn=fn):
            g2 = torch.Generator().manual_seed(50)
            fa = torch.randn(64, SIZE, SIZE, generator=g2).to(dev).requires_grad_(True)
            fb = torch.randn(64, SIZE, SIZE, generator=g2).to(dev).requires_grad_(True)
            fo = torch.ones(64, SIZE, SIZE, device=dev)
            return lambda: torch.autograd.grad(fn(fa, fb), (fa, fb), fo)

        macs = (3.0 if name == "logbmm" else 1.0) * 64 * SIZE ** 3
        both("strong_%s_global_batch_64" % name, strong_step, single_strong, {"batch_per_gpu": per})
        res["strong_%s_global_batch_64" % name]["mac_per_s"] = macs / res["strong_%s_global_batch_64" % name]["ms"] * 1e3
    return res


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------

def run_ours(args, rank, world, local):
    import genbmm_b200 as gb
    from genbmm_b200 import _native
    from genbmm_b200.host import HostPipeline, bind_host_near

    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU path"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # pinned host buffers next to this rank's GPU: the end-to-end number is bound by host memory and the PCIe
    # roots, not by the kernels.  At N = 1 the full core set is given back before the CPU baseline leg (the
    # buffers are pinned where they were allocated).
    all_cores = os.sched_getaffinity(0) if hasattr(os, "sched_getaffinity") else None
    near = bind_host_near(dev)
    ranks = Ranks(dev, world)
    lib = _native.load()
    peaks = read_peaks()

    B = args.batch
    gen = torch.Generator().manual_seed(5 + rank)
    a_h = torch.randn(B, SIZE, SIZE, generator=gen).pin_memory()
    b_h = torch.randn(B, SIZE, SIZE, generator=gen).pin_memory()
    a = a_h.to(dev).requires_grad_(True)
    b = b_h.to(dev).requires_grad_(True)
    ones = torch.ones(B, SIZE, SIZE, device=dev)
    macs_log = 3.0 * B * SIZE ** 3

    def step_log():
        c = gb.logbmm(a, b)
        return torch.autograd.grad(c, (a, b), ones)

    def step_max():
        c = gb.maxbmm(a, b)
        return torch.autograd.grad(c, (a, b), ones)

    # ---- headline: device-resident inputs ------------------------------------------------
    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(args.warmup):
        step_log()
    est = ranks.max(region_ms(step_log, 3, ranks.sync) / 3)         # three more untimed-for-the-record steps
    repeats = max(1, min(4000, math.ceil(TARGET_REGION_S * 1e3 / (args.steps * est))))
    if args.inner_repeats > 0:
        repeats = args.inner_repeats
    ranks.sync()
    launches0 = lib.gbmm_launch_count()
    t_host0 = time.perf_counter()
    region = region_ms(step_log, args.steps * repeats, ranks.sync)
    t_host1 = time.perf_counter()
    launches = lib.gbmm_launch_count() - launches0
    t_log = ranks.max(region) / 1e3 / repeats                        # seconds per `steps` steps
    clocks = sampler.window(t_host0, t_host1)
    # the same step in a short burst (`steps` steps, a few tens of milliseconds: before the power cap has pulled
    # the clock down), after a pause: what a timed region of that length reports
    time.sleep(1.0)
    for _ in range(3):
        step_log()
    t_burst = ranks.max(region_ms(step_log, args.steps, ranks.sync)) / 1e3
    if clocks.get("sm_mhz"):
        clocks["ms_per_step_x_sm_ghz"] = t_log / args.steps * 1e3 * clocks["sm_mhz"] / 1e3

    # ---- the same step for maxbmm ---------------------------------------------------------
    for _ in range(args.warmup):
        step_max()
    max_rep = max(1, repeats // 6)
    t0m = time.perf_counter()
    t_max = ranks.max(region_ms(step_max, args.steps * max_rep, ranks.sync)) / 1e3 / max_rep
    clocks_max = sampler.window(t0m, time.perf_counter())
    macs_max = (1.0 * B * SIZE ** 3) + 2.0 * B * SIZE * SIZE

    # ---- end to end: pinned host inputs in, gradients and loss back to the host ----------
    # genbmm_b200.host.HostPipeline: the package's call for host-resident operands.  It cuts the batch into
    # chunks on three streams so that the two PCIe directions overlap the kernels; every chunk goes through
    # the public operator (genbmm_b200.logbmm + torch.autograd.grad).
    ga_h = torch.empty(B, SIZE, SIZE).pin_memory()
    gb_h = torch.empty(B, SIZE, SIZE).pin_memory()
    pipe = HostPipeline(B, SIZE, SIZE, SIZE, chunks=args.e2e_chunks if args.e2e_chunks == "tapered" else int(args.e2e_chunks),
                        device=dev, graph=bool(args.e2e_graph))

    def step_e2e():
        return pipe.step(a_h, b_h, ga_h, gb_h)

    e2e_steps = max(2, min(args.steps, 50))
    for _ in range(3):       # with --e2e-graph 1 the pipeline captures its kernels at the second
        step_e2e()
    t_e2e = ranks.max(region_ms(step_e2e, e2e_steps, ranks.sync) / e2e_steps) / 1e3
    h2d = 2 * B * SIZE * SIZE * 4
    d2h = 2 * B * SIZE * SIZE * 4 + 8
    # the copies alone: the same bytes over the same two copy streams in the same chunks, both directions at
    # once, nothing computed — the bound of the end-to-end step on this host
    s_in, s_out = pipe.s_in, pipe.s_out

    def copies_only():
        cur = torch.cuda.current_stream()
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        for lo, hi in pipe.bounds:
            with torch.cuda.stream(s_in):
                pipe.a[lo:hi].copy_(a_h[lo:hi], non_blocking=True)
                pipe.b[lo:hi].copy_(b_h[lo:hi], non_blocking=True)
            with torch.cuda.stream(s_out):
                ga_h[lo:hi].copy_(pipe.a[lo:hi], non_blocking=True)
                gb_h[lo:hi].copy_(pipe.b[lo:hi], non_blocking=True)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)

    for _ in range(2):
        copies_only()
    t_copy = ranks.max(region_ms(copies_only, e2e_steps, ranks.sync) / e2e_steps) / 1e3
    del pipe

    # ---- per-kernel durations for the roofline (this rank's GPU) ---------------------------
    # The step is dominated by the three TMA-fed products of the factorised path (forward, grad_a,
    # grad_b), run as 3xTF32 on tcgen05; the library brackets each product launch with CUDA events
    # on request.  The same products on the FP32 pipe are timed beside them.
    ad, bd = a.detach(), b.detach()
    names = ("fwd_product", "grad_a_product", "grad_b_product")

    def product_ms(tensor_cores):
        ms = {k: [] for k in names}
        lib.gbmm_profile_enable(1)
        for _ in range(max(3, min(args.steps, 10))):
            out_f, rmax, cmax, flg = _native.logbmm_fast_forward(ad, bd, tensor_cores=tensor_cores)
            _native.logbmm_fast_backward(ad, bd, ones, out_f, rmax, cmax, flg, tensor_cores=tensor_cores)
            for i, k in enumerate(names):
                ms[k].append(float(lib.gbmm_profile_last_ms(i)))
        lib.gbmm_profile_enable(0)
        return {k: sorted(v)[len(v) // 2] / 1e3 for k, v in ms.items()}, int(flg.sum().item())

    kernels, flagged_tiles = product_ms(True)
    kernels_fp32, _ = product_ms(False)
    dominant = max(kernels, key=kernels.get)
    flops = 2.0 * B * SIZE ** 3                 # one multiply-add per (m,k,n) triple in each product
    tensor_flops = 3.0 * flops                  # executed on the tensor cores: three TF32 MMAs per triple
    tf32_peak = peaks["bf16_tflops"] * 1e12 / 2  # dense TF32 runs at half the measured bf16 rate (derived)
    fp32_peak = N_SMS * FP32_PER_SM_CLK * 2 * peaks["sm_max_mhz"] * 1e6
    achieved = tensor_flops / kernels[dominant]
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        with open(tpath) as f:
            t = json.load(f).get("tc_pair_gemm_kernel")
        if t and dominant in t.get("dram_bytes_per_launch", {}):
            traffic = t["dram_bytes_per_launch"][dominant] * (B / t["batch"])

    # ---- a library TF32 product on this GPU, for the denominator's sake -------------------
    tf32_lib = None
    try:
        was = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        x = torch.randn(8192, 8192, device=dev)
        y = torch.randn(8192, 8192, device=dev)
        best = min(region_ms(lambda: torch.matmul(x, y), 1, torch.cuda.synchronize) for _ in range(10))
        tf32_lib = 2.0 * 8192 ** 3 / (best / 1e3) / 1e12
        torch.backends.cuda.matmul.allow_tf32 = was
        del x, y
    except Exception:
        pass

    # ---- the exact (SFU) kernels on the same step, for the record --------------------------
    def step_exact():
        o = _native.forward(ad, bd, 0, want_maxes=False)[0]
        _native.backward(ad, bd, ones, o, None, 0)

    n_exact = max(2, min(args.steps, 5))
    t_exact = region_ms(step_exact, n_exact, torch.cuda.synchronize) / n_exact / 1e3 if not args.quick else None
    sfu_peak = N_SMS * SFU_PER_SM_CLK * peaks["sm_max_mhz"] * 1e6
    sampler.stop()

    line = {
        "metric": "logbmm fwd+bwd semiring MAC/s", "value": world * macs_log * args.steps / t_log, "unit": "MAC/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_log / args.steps * 1e3,
        "inner_repeats": repeats, "timed_region_s": t_log * repeats,
        "burst": {"ms_per_step": t_burst / args.steps * 1e3, "value": world * macs_log * args.steps / t_burst,
                  "what": "the same %d steps once, after a one-second pause (region of a few tens of ms)" % args.steps},
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args), "clocks": clocks,
        "e2e": {"value": world * macs_log / t_e2e, "unit": "MAC/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": t_e2e * 1e3,
                "api": "genbmm_b200.host.HostPipeline.step -> genbmm_b200.logbmm + torch.autograd.grad per chunk",
                "copies_only_ms": t_copy * 1e3, "frac_of_copy_bound": t_copy / t_e2e,
                "copy_gb_per_s_per_direction": h2d / t_copy / 1e9,
                "host_cores_bound": None if near is None else len(near)},
        "gpu_launches": int(launches), "gpu_launches_per_step": launches / (args.steps * repeats),
        "roofline": {
            "bound": "tensor", "kernel": "tc_pair_gemm_kernel (%s)" % dominant, "achieved": achieved / 1e12,
            "peak": tf32_peak / 1e12, "unit": "TFLOP/s", "frac": achieved / tf32_peak, "traffic": traffic,
            "peak_source": "DERIVED, not measured: dense TF32 taken as bf16_tflops (burst) of MEASURED_PEAKS.json "
                           "/ 2 (%s); achieved counts the executed tensor FLOPs, 3 TF32 MMAs per multiply-add "
                           "(3xTF32 split); tf32_library_tflops is a cuBLAS TF32 8192^3 product timed in this "
                           "run" % peaks["source"],
            "frac_of_sustained_peak": achieved / (peaks["bf16_tflops_sustained"] * 1e12 / 2),
            "tf32_library_tflops": tf32_lib,
            "frac_of_tf32_library": None if not tf32_lib else achieved / (tf32_lib * 1e12),
            "useful_tflops": flops / kernels[dominant] / 1e12,
            "kernel_ms": {k: v * 1e3 for k, v in kernels.items()},
            "step_frac_of_tensor_bound": (3 * tensor_flops / tf32_peak) / (t_log / args.steps),
            "flagged_tiles": flagged_tiles,
        },
        "also": {"fp32_pipe_product_ms": {k: v * 1e3 for k, v in kernels_fp32.items()},
                 "fp32_pipe_product_frac_of_fp32_peak": flops / max(kernels_fp32.values()) / fp32_peak,
                 "maxbmm_fwd_bwd_mac_per_s": world * macs_max * args.steps / t_max,
                 "maxbmm_ms_per_step": t_max / args.steps * 1e3,
                 "maxbmm_clocks": clocks_max,
                 "maxbmm_frac_of_fp32_bound": (B * SIZE ** 3 / bounds(peaks)["max"] + route_bytes(
                     B, SIZE, SIZE, SIZE, False) / bounds(peaks)["hbm"]) / (t_max / args.steps)},
    }
    if t_exact is not None:
        line["also"].update({"exact_sfu_path_ms_per_step": t_exact * 1e3,
                             "exact_sfu_path_mac_per_s": macs_log / t_exact,
                             "exact_sfu_path_frac_of_sfu_bound": (2.0 * B * SIZE ** 3 / sfu_peak) / t_exact})
    del a, b, ones, ad, bd, a_h, b_h, ga_h, gb_h
    torch.cuda.empty_cache()
    if not args.no_configs:
        try:
            if world == 1:
                line["configs"] = measure_configs(gb, dev, peaks, args.quick)
                line["host_cost"] = host_cost(gb, dev)
                _native.release_workspaces()
                torch.cuda.empty_cache()
            sharded = measure_sharded(gb, dev, ranks, rank, world, peaks, args.quick)
            line.setdefault("configs", {}).update(sharded)
        except Exception as exc:  # the headline must not depend on the side measurements
            line.setdefault("configs", {})["error"] = repr(exc)[:300]
    if rank == 0 and world == 1 and not args.no_reference_cuda:
        # the reference's own kernels on this GPU, in a process of their own (nothing of it is loaded here)
        try:
            r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference-cuda", "--batch",
                                str(args.batch), "--steps", "3"], capture_output=True, text=True, timeout=900)
            ref = json.loads(r.stdout.strip().splitlines()[-1])
            line["also"]["reference_cuda"] = ref if "unavailable" in ref else {
                "logbmm_ms_per_step": ref["ms_per_step"], "maxbmm_ms_per_step": ref["also"]["maxbmm_ms_per_step"],
                "configs_ms": {k: v["ms"] for k, v in ref["configs"].items()}, "what": ref["what"]}
            if "unavailable" not in ref:
                line["also"]["reference_cuda"]["logbmm_speedup"] = ref["ms_per_step"] / (t_log / args.steps * 1e3)
                line["also"]["reference_cuda"]["maxbmm_speedup"] = (ref["also"]["maxbmm_ms_per_step"] /
                                                                    (t_max / args.steps * 1e3))
        except Exception as exc:
            line["also"]["reference_cuda"] = {"unavailable": repr(exc)[:200]}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        if all_cores is not None:
            os.sched_setaffinity(0, all_cores)
        host_threads()
        value, secs, threads = cpu_logbmm_sample(8192, 64)
        line["cpu_baseline"] = {
            "value": value, "unit": "MAC/s", "cores": threads, "kind": "port",
            "sample": "8192 rows x 1024 x 1024 (the work of 8 of the 32 batch elements of a step), forward + "
                      "autograd backward of the broadcast-reduce expression in 64-row chunks, %.1f s" % secs}
    if rank == 0:
        print(json.dumps(line), flush=True)
    ranks.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-cuda"])
    ap.add_argument("--batch", type=int, default=32, help="1024^3 problems per GPU per step")
    ap.add_argument("--inner-repeats", type=int, default=0,
                    help="run every counted step this many times (0: as many as make the timed region 2 s)")
    ap.add_argument("--e2e-chunks", default="8",
                    help="batch chunks of the host pipeline (end-to-end leg): a count, or 'tapered'")
    ap.add_argument("--e2e-graph", type=int, default=0, help="1: the host pipeline replays one CUDA graph per chunk")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-cuda", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the side measurements of configs 1-5")
    ap.add_argument("--quick", action="store_true", help="few iterations of every side measurement (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif args.impl == "reference-cuda":
        run_reference_cuda(args, rank, world)
    else:
        run_ours(args, rank, world, local)


if __name__ == "__main__":
    main()
