"""Host-resident operands: logbmm forward + backward with the PCIe copies overlapped.

A caller whose operands live in (pinned) host memory pays two copies per step, each of the size
of the operands; done one after the other with the kernels they cost more than the kernels.
`HostPipeline` cuts the batch into chunks and runs three CUDA streams — host-to-device copies,
kernels, device-to-host copies — so that chunk i+1 is arriving and chunk i-1 is leaving while
chunk i is being multiplied (PCIe is full duplex; the GPU has separate copy engines for the two
directions).  Device buffers are allocated once and reused by every step.

    pipe = HostPipeline(B, M, K, N, chunks=4)
    loss = pipe.step(a_host, b_host, grad_a_host, grad_b_host)   # loss = logbmm(a, b).sum()

The reference has no counterpart: it takes device tensors only (matmul_cuda.cpp:65).
"""
import torch

from . import _native


def bind_host_near(device):
    """Restrict this process to the CPU cores NVML lists as local to `device` (its NUMA node), so that pinned
    host buffers allocated afterwards — first touched by this process — sit next to the GPU's PCIe root and
    ranks on different sockets do not all stream through one.  Reads GPU properties only; changes nothing but
    this process's own CPU affinity.  Returns the cores chosen, or None when NVML or the affinity call is
    unavailable, or none of the local cores is allowed to this process."""
    import os
    try:
        import pynvml
        dev = torch.device(device)
        props = torch.cuda.get_device_properties(dev)
        bus_id = "%08x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus_id.encode())
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        local = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1}
        cores = sorted(local & os.sched_getaffinity(0))
        if not cores:
            return None
        os.sched_setaffinity(0, cores)
        return cores
    except Exception:
        return None


def chunk_bounds(B, chunks):
    """[lo, hi) batch ranges of the pipeline's chunks.  An integer gives that many equal chunks.  "tapered" gives
    small chunks at both ends and larger ones between (1, 1, 2, then about B / 8 each, then 2, 1, 1): the
    device-to-host copies cannot start before the first chunk has arrived and been multiplied, and the last
    chunk's results leave after everything else is done, so the first and the last chunk are pure latency while
    the number of chunks is what the host pays for."""
    if chunks == "tapered":
        if B < 12:
            sizes = [1] * B
        else:
            mid = max(2, B // 8)
            head = [1, 1, 2]
            rest = B - 2 * sum(head)
            sizes = head + [mid] * (rest // mid) + ([rest % mid] if rest % mid else []) + head[::-1]
        out, lo = [], 0
        for n in sizes:
            out.append((lo, lo + n))
            lo += n
        assert lo == B
        return out
    if isinstance(chunks, (list, tuple)):   # explicit chunk sizes
        assert sum(chunks) == B and all(n > 0 for n in chunks)
        out, lo = [], 0
        for n in chunks:
            out.append((lo, lo + n))
            lo += n
        return out
    chunks = max(1, min(int(chunks), B))
    return [(i * B // chunks, (i + 1) * B // chunks) for i in range(chunks)]


class HostPipeline:
    def __init__(self, B, M, K, N, chunks=4, device=None, tensor_cores=True, graph=False):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.shape = (B, M, K, N)
        self.tensor_cores = tensor_cores
        # Default (graph=False): every chunk is one call of the package's own operator, genbmm_b200.logbmm, and
        # one torch.autograd.grad — the path a user of the drop-in API takes.
        # graph=True: the second step captures the kernels of every chunk (forward, loss, backward) into one
        # CUDA graph per chunk, all in one memory pool, on static gradient buffers through the C-ABI calls
        # directly, and later steps replay them between the copies, which stay ordinary stream copies; the
        # host then issues about a hundred calls per step instead of several hundred.  Off by default: a
        # 32 x 1024^3 step is bound by the PCIe copies, not by the host (measured 7.4 ms with graphs against
        # 6.6-6.9 ms without on one GPU, 31.5 ms either way with eight ranks sharing one host's links).
        self.use_graph = graph
        self._graphs = None
        self._warm = False
        self.bounds = chunk_bounds(B, chunks)
        with torch.cuda.device(self.device):
            self.a = torch.empty((B, M, K), device=self.device)
            self.b = torch.empty((B, K, N), device=self.device)
            self.grad_a = torch.empty_like(self.a) if graph else None
            self.grad_b = torch.empty_like(self.b) if graph else None
            self.ones = torch.ones((max(hi - lo for lo, hi in self.bounds), M, N), device=self.device)
            self.loss = torch.zeros((), device=self.device, dtype=torch.float64)
            self.s_in = torch.cuda.Stream(self.device)
            self.s_out = torch.cuda.Stream(self.device)
            self.ev_in = [torch.cuda.Event() for _ in self.bounds]
            self.ev_done = [torch.cuda.Event() for _ in self.bounds]
            self.ev_step = torch.cuda.Event()

    def step(self, a_host, b_host, grad_a_host, grad_b_host):
        """One forward + backward of loss = logbmm(a, b).sum().  All four host tensors should be
        pinned; the gradients are complete in grad_*_host when this returns.  Returns the loss."""
        B, M, K, N = self.shape
        assert tuple(a_host.shape) == (B, M, K) and tuple(b_host.shape) == (B, K, N)
        with torch.cuda.device(self.device):
            if self.use_graph and self._warm and self._graphs is None:
                # the first step ran directly (every kernel loaded, allocator filled): capture now
                torch.cuda.synchronize(self.device)
                graphs, pool = [], None
                for i in range(len(self.bounds)):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, pool=pool):
                        self._compute_static(i)
                    pool = g.pool()
                    graphs.append(g)
                self._graphs = graphs
            comp = torch.cuda.current_stream(self.device)
            self.loss.zero_()
            # the copy streams start after whatever the compute stream was doing with the buffers
            self.ev_step.record(comp)
            self.s_in.wait_event(self.ev_step)
            self.s_out.wait_event(self.ev_step)
            with torch.cuda.stream(self.s_in):
                for i, (lo, hi) in enumerate(self.bounds):
                    self.a[lo:hi].copy_(a_host[lo:hi], non_blocking=True)
                    self.b[lo:hi].copy_(b_host[lo:hi], non_blocking=True)
                    self.ev_in[i].record(self.s_in)
            for i, (lo, hi) in enumerate(self.bounds):
                comp.wait_event(self.ev_in[i])
                if self._graphs is not None:
                    self._graphs[i].replay()
                    ga, gb = self.grad_a[lo:hi], self.grad_b[lo:hi]
                elif self.use_graph:
                    self._compute_static(i)
                    ga, gb = self.grad_a[lo:hi], self.grad_b[lo:hi]
                else:
                    ga, gb = self._compute(i)
                self.ev_done[i].record(comp)
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(self.ev_done[i])
                    grad_a_host[lo:hi].copy_(ga, non_blocking=True)
                    grad_b_host[lo:hi].copy_(gb, non_blocking=True)
                    if not self.use_graph:   # allocated on the compute stream, last read on the copy stream
                        ga.record_stream(self.s_out)
                        gb.record_stream(self.s_out)
            comp.wait_stream(self.s_out)
            self._warm = True
            return float(self.loss.item())

    def _compute(self, i):
        """Chunk i through the public operator: c = genbmm_b200.logbmm(a, b), its share of the loss, and
        autograd for both gradients."""
        from .genmul import logbmm
        lo, hi = self.bounds[i]
        a, b = self.a[lo:hi].requires_grad_(True), self.b[lo:hi].requires_grad_(True)
        c = logbmm(a, b) if self.tensor_cores else _FP32Log.apply(a, b)
        self.loss += c.detach().sum(dtype=torch.float64)
        return torch.autograd.grad(c, (a, b), self.ones[: hi - lo])

    def _compute_static(self, i):
        """Kernels of chunk i on the current stream through the C-ABI calls, into static buffers (what a CUDA
        graph can capture): forward, its share of the loss, backward into the chunk's rows of the gradient
        buffers."""
        lo, hi = self.bounds[i]
        a, b = self.a[lo:hi], self.b[lo:hi]
        out, rowmax, colmax, flags, factors = _native.logbmm_fast_forward(
            a, b, tensor_cores=self.tensor_cores, keep_factors=True)
        self.loss += out.sum(dtype=torch.float64)
        _native.logbmm_fast_backward(a, b, self.ones[: hi - lo], out, rowmax, colmax, flags,
                                     tensor_cores=self.tensor_cores, factors=factors,
                                     out_grads=(self.grad_a[lo:hi], self.grad_b[lo:hi]))


class _FP32Log(torch.autograd.Function):
    """logbmm on the FP32-pipe factorised kernels (HostPipeline(tensor_cores=False))."""

    @staticmethod
    def forward(ctx, a, b):
        out, rowmax, colmax, flags = _native.logbmm_fast_forward(a, b, tensor_cores=False)
        ctx.save_for_backward(a, b, out, rowmax, colmax, flags)
        return out

    @staticmethod
    def backward(ctx, g):
        a, b, out, rowmax, colmax, flags = ctx.saved_tensors
        return _native.logbmm_fast_backward(a, b, g.contiguous(), out, rowmax, colmax, flags, tensor_cores=False)
