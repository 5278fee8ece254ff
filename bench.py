"""Benchmark of the semiring batched-matmul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one logbmm forward + backward (loss = c.sum()) over a batch of `--batch` problems of
size 1024x1024x1024 per GPU (the "1024^3 per batch element" throughput configuration); the
metric is semiring multiply-accumulates per second, 3*B*M*K*N per step (forward, grad_a and
grad_b each touch every (m,k,n) triple once).  The same step for maxbmm is timed beside it and
reported under "also".  Inputs are seeded synthetic tensors, larger than the L2 cache.

With N > 1 (torchrun, one process per GPU) every rank runs the same per-GPU workload on its own
batch shard; there is no data-path collective.  The time is the maximum over ranks of the
CUDA-event duration, the value the total over ranks.

`--impl reference` times the reference's own CPU formulation of logbmm — the broadcast-reduce
PyTorch expression of its README and tests — on the host cores, on a bounded sample of the
same workload.
"""
import argparse
import json
import os
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
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

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
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                mhz.append(float(s[0]))
                mx = float(s[1])
            except ValueError:
                continue
            for name, flag in zip(names, s[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


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


def workload_config(args):
    return {"workload": "logbmm fwd+bwd, a,b:(%d,%d,%d) fp32 N(0,1) seed 5 per GPU, loss=c.sum()" % (
        args.batch, SIZE, SIZE), "batch_per_gpu": args.batch, "M": SIZE, "K": SIZE, "N": SIZE,
        "parallelism": "batch-sharded, no collective", "l2": "working set %d MB per GPU, larger than L2" % (
            6 * args.batch * 4 * SIZE * SIZE >> 20)}


def time_steps(fn, steps, warmup, sync):
    """CUDA-event time of `steps` calls of fn on the current stream, after `warmup` untimed calls."""
    for _ in range(warmup):
        fn()
    sync()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    sync()
    return start.elapsed_time(stop) / 1e3


def measure_configs(gb, dev):
    """Forward+backward time of the other benchmark configurations (seeded synthetic inputs made on
    the device; parity of the same shapes is covered by the test-suite).  Reported under "configs"."""
    from genbmm_b200 import crf
    res = {}
    gen = torch.Generator(device=dev)

    def fwd_bwd(fn, args, n_iter=5):
        leaves = [x.detach().requires_grad_(True) for x in args[:2]]
        rest = list(args[2:])

        def step():
            c = fn(*leaves, *rest)
            c = c.data if isinstance(c, gb.BandedMatrix) else c
            torch.autograd.grad(c, leaves, torch.ones_like(c))

        return time_steps(step, n_iter, 2, torch.cuda.synchronize) / n_iter

    gen.manual_seed(0)
    a, b = (torch.rand(32, 64, 64, device=dev, generator=gen) for _ in range(2))
    t = fwd_bwd(gb.logbmm, (a, b), 20)
    res["cfg1_logbmm_32x64x64x64"] = {"ms": t * 1e3, "mac_per_s": 3 * 32 * 64 ** 3 / t}
    gen.manual_seed(1)
    a, b = ((torch.randn(256, 128, 128, device=dev, generator=gen) * 8).round() / 8 for _ in range(2))
    for name in ("maxbmm", "prodmaxbmm"):
        t = fwd_bwd(getattr(gb, name), (a, b), 10)
        res["cfg2_%s_256x128x128x128" % name] = {"ms": t * 1e3, "mac_per_s": 256 * 128 ** 3 / t}
    gen.manual_seed(2)
    a, b = (2 * torch.randn(64, 256, 256, device=dev, generator=gen) for _ in range(2))
    u = torch.rand(64, 256, 256, device=dev, generator=gen)
    t = fwd_bwd(gb.samplebmm, (a, b, u), 10)
    res["cfg3_samplebmm_64x256x256x256"] = {"ms": t * 1e3, "mac_per_s": 64 * 256 ** 3 / t}
    gen.manual_seed(3)
    pot = torch.randn(16, 511, 256, 256, device=dev, generator=gen)

    def crf_step():
        crf.marginals(pot)

    t = time_steps(crf_step, 3, 1, torch.cuda.synchronize) / 3
    res["cfg4_crf_B16_T512_C256"] = {"ms": t * 1e3, "mac_per_s": 3 * 16 * 510 * 256 ** 3 / t}
    del pot
    gen.manual_seed(4)
    x, y = (torch.randn(32, 8192, 129, device=dev, generator=gen) for _ in range(2))
    triples = 32 * 135428672  # valid (i, ja, jo) triples per forward at n=8192, 129 diagonals each
    for name in ("multiply", "multiply_log", "multiply_max"):
        def band(p, q, name=name):
            return getattr(gb.BandedMatrix(p, 64, 64), name)(gb.BandedMatrix(q, 64, 64))
        t = fwd_bwd(band, (x, y), 3)
        res["cfg5_banded_%s_32x8192x129" % name] = {"ms": t * 1e3, "mac_per_s": 3 * triples / t}
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=32, help="1024^3 problems per GPU per step")
    ap.add_argument("--e2e-chunks", type=int, default=16, help="batch chunks of the host pipeline (end-to-end leg)")
    ap.add_argument("--e2e-graph", type=int, default=0, help="1: the host pipeline replays one CUDA graph per chunk")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the side measurements of configs 1-5")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import genbmm_b200 as gb
    from genbmm_b200 import _native

    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU path"
    torch.cuda.set_device(local)
    # pinned host buffers next to this rank's GPU: the end-to-end number is bound by host memory and the PCIe
    # roots, not by the kernels.  At N = 1 the full core set is given back before the CPU baseline leg (the
    # buffers are pinned where they were allocated).
    from genbmm_b200.host import bind_host_near
    all_cores = os.sched_getaffinity(0) if hasattr(os, "sched_getaffinity") else None
    near = bind_host_near(torch.device("cuda", local))
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    def sync():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

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
    for _ in range(args.warmup):
        step_log()
    sync()
    sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step_log()
    stop.record()
    sync()
    t_log = torch.tensor([start.elapsed_time(stop) / 1e3], device=dev)
    if dist is not None:
        dist.all_reduce(t_log, op=dist.ReduceOp.MAX)
    t_log = float(t_log.item())

    # ---- the same step for maxbmm ---------------------------------------------------------
    t_max = torch.tensor([time_steps(step_max, args.steps, args.warmup, sync)], device=dev)
    if dist is not None:
        dist.all_reduce(t_max, op=dist.ReduceOp.MAX)
    t_max = float(t_max.item())
    macs_max = (1.0 * B * SIZE ** 3) + 2.0 * B * SIZE * SIZE

    # ---- end to end: pinned host inputs in, gradients and loss back to the host ----------
    ga_h = torch.empty(B, SIZE, SIZE).pin_memory()
    gb_h = torch.empty(B, SIZE, SIZE).pin_memory()

    # genbmm_b200.host.HostPipeline: the package's call for host-resident operands; it overlaps the
    # two PCIe directions with the kernels by cutting the batch into chunks on three streams
    from genbmm_b200.host import HostPipeline
    pipe = HostPipeline(B, SIZE, SIZE, SIZE, chunks=args.e2e_chunks, device=dev, graph=bool(args.e2e_graph))

    def step_e2e():
        return pipe.step(a_h, b_h, ga_h, gb_h)

    e2e_steps = max(2, min(args.steps, 50))
    # three untimed steps first (with --e2e-graph 1 the pipeline captures its kernels at the second)
    t_e2e = torch.tensor([time_steps(step_e2e, e2e_steps, 3, sync) / e2e_steps], device=dev)
    if dist is not None:
        dist.all_reduce(t_e2e, op=dist.ReduceOp.MAX)
    t_e2e = float(t_e2e.item())
    h2d = 2 * B * SIZE * SIZE * 4
    d2h = 2 * B * SIZE * SIZE * 4 + 4
    # extend the load until nvidia-smi (100 ms period) has seen it for about a second, so that the
    # clock record covers a sustained run of the same step
    t_end = time.perf_counter() + 1.0
    while time.perf_counter() < t_end:
        for _ in range(20):
            step_log()
        torch.cuda.synchronize()
    clocks = sampler.stop()

    # ---- per-kernel durations for the roofline (this rank's GPU) ---------------------------
    # The step is dominated by the three TMA-fed products of the factorised path (forward, grad_a,
    # grad_b), run as 3xTF32 on tcgen05; the library brackets each product launch with CUDA events
    # on request.  The same products on the FP32 pipe are timed beside them.
    lib = _native.load()
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
    peaks = read_peaks()
    flops = 2.0 * B * SIZE ** 3                 # one multiply-add per (m,k,n) triple in each product
    tensor_flops = 3.0 * flops                  # executed on the tensor cores: three TF32 MMAs per triple
    tf32_peak = peaks["bf16_tflops"] * 1e12 / 2  # dense TF32 runs at half the measured bf16 rate
    fp32_peak = N_SMS * FP32_PER_SM_CLK * 2 * peaks["sm_max_mhz"] * 1e6
    achieved = tensor_flops / kernels[dominant]
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        with open(tpath) as f:
            t = json.load(f).get("tc_pair_gemm_kernel")
        if t:
            traffic = t["dram_bytes_per_launch"] * (B / t["batch"])

    # ---- the exact (SFU) kernels on the same step, for the record --------------------------
    out_e = _native.forward(ad, bd, 0, want_maxes=False)[0]

    def step_exact():
        o = _native.forward(ad, bd, 0, want_maxes=False)[0]
        _native.backward(ad, bd, ones, o, None, 0)

    t_exact = time_steps(step_exact, max(2, min(args.steps, 5)), 2, torch.cuda.synchronize) / max(
        2, min(args.steps, 5))
    sfu_peak = N_SMS * SFU_PER_SM_CLK * peaks["sm_max_mhz"] * 1e6
    del out_e

    line = {
        "metric": "logbmm fwd+bwd semiring MAC/s", "value": world * macs_log * args.steps / t_log, "unit": "MAC/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_log / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args), "clocks": clocks,
        "e2e": {"value": world * macs_log / t_e2e, "unit": "MAC/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": t_e2e * 1e3,
                "host_cores_bound": None if near is None else len(near)},
        "gpu_launches": 9 * args.steps,
        "roofline": {
            "bound": "tensor", "kernel": "tc_pair_gemm_kernel (%s)" % dominant, "achieved": achieved / 1e12,
            "peak": tf32_peak / 1e12, "unit": "TFLOP/s", "frac": achieved / tf32_peak, "traffic": traffic,
            "peak_source": "dense TF32 = bf16_tflops of MEASURED_PEAKS.json / 2 (%s); achieved counts the "
                           "executed tensor FLOPs, 3 TF32 MMAs per multiply-add (3xTF32 split)" % peaks["source"],
            "frac_of_sustained_peak": achieved / (peaks["bf16_tflops_sustained"] * 1e12 / 2),
            "useful_tflops": flops / kernels[dominant] / 1e12,
            "kernel_ms": {k: v * 1e3 for k, v in kernels.items()},
            "flagged_tiles": flagged_tiles,
        },
        "also": {"fp32_pipe_product_ms": {k: v * 1e3 for k, v in kernels_fp32.items()},
                 "fp32_pipe_product_frac_of_fp32_peak": flops / max(kernels_fp32.values()) / fp32_peak,
                 "exact_sfu_path_ms_per_step": t_exact * 1e3,
                 "exact_sfu_path_mac_per_s": macs_log / t_exact,
                 "exact_sfu_path_frac_of_sfu_bound": (2.0 * B * SIZE ** 3 / sfu_peak) / t_exact,
                 "maxbmm_fwd_bwd_mac_per_s": world * macs_max * args.steps / t_max,
                 "maxbmm_ms_per_step": t_max / args.steps * 1e3,
                 "maxbmm_frac_of_fp32_bound": (macs_max * 2 / (N_SMS * FP32_PER_SM_CLK * peaks["sm_max_mhz"] * 1e6))
                 / (t_max / args.steps)},
    }
    if rank == 0 and world == 1 and not args.no_configs:
        try:
            line["configs"] = measure_configs(gb, dev)
        except Exception as exc:  # the headline must not depend on the side measurements
            line["configs"] = {"error": repr(exc)}
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
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
