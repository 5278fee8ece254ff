"""Linear-chain CRF log-partition by a log-semiring tree reduction — a caller of logbmm.

The reference has no such module (its README names PyTorch-Struct as the caller that does this);
this is the smallest driver for the benchmark configuration "linear-chain CRF, T positions,
C states": potentials pot:(B, T-1, C, C), the chain product

    P[b] = pot[b,0] (x) pot[b,1] (x) ... (x) pot[b,T-2],   (A (x) B)[i,j] = logsumexp_k A[i,k] + B[k,j]

evaluated as balanced pairwise trees over the power-of-two runs of the chain (level l of a run is one
logbmm call with batch B * run / 2^(l+1)); logZ[b] = logsumexp_{i,j} P[b]; the edge
marginals are d(sum_b logZ[b]) / d pot, obtained by autograd through the tree.

`bmm` is the semiring product to use (default: genbmm_b200.logbmm); tests on CPU pass the
broadcast-reduce expression instead.
"""
import torch
import torch.distributed as dist
from torch.autograd.function import once_differentiable


def _default_bmm():
    from .genmul import logbmm
    return logbmm


def _bit_reversed(x, k):
    """x:(2**k, ...) -> the same matrices in bit-reversed order of the first index, as one strided copy
    (bit reversal = splitting the index into k binary digits and reversing their order).  Its own inverse."""
    if k <= 1:
        return x.contiguous()
    rest = x.shape[1:]
    y = x.reshape((2,) * k + tuple(rest))
    y = y.permute(tuple(range(k - 1, -1, -1)) + tuple(range(k, k + len(rest))))
    return y.reshape((2 ** k,) + tuple(rest)).contiguous()


def _runs(L):
    """(start, length, padded length) of the runs a chain of L matrices is cut into.  When the next power of
    two is at most an eighth longer than L the chain is one run, padded with identity matrices (which
    multiply away); otherwise one run per power of two of L's binary expansion, longest first."""
    n = 1 << max(L - 1, 0).bit_length()
    if n - L <= L // 8:
        return [(0, L, n)]
    out, s = [], 0
    for bit in range(L.bit_length() - 1, -1, -1):
        if L & (1 << bit):
            out.append((s, 1 << bit, 1 << bit))
            s += 1 << bit
    return out


class _ChainMajor(torch.autograd.Function):
    """pot (B, L, C, C) -> one tensor per run of the chain (see _runs): (n, B, C, C), n a power of two, with the
    run's chain positions in bit-reversed order.

    In that order the matrices at even positions are the first half and the ones at odd positions the second
    half, and the pairwise products come out in the bit-reversed order of their own index, so every level of
    the tree multiplies the first half by the second half: contiguous views, no copies.  Padding matrices are
    the semiring's identity (0 on the diagonal, -1e9 elsewhere).  first_order_only=True (GPU, float32, one
    run) moves the matrices with the library's block gather in both directions; otherwise both directions
    are torch operations and second-order gradients pass through."""

    @staticmethod
    def forward(ctx, pot, first_order_only=False):
        ctx.shape = pot.shape
        B, L, C, D = pot.shape
        runs = _runs(L)
        ctx.maps = None
        if (first_order_only and pot.is_cuda and pot.dtype == torch.float32 and pot.is_contiguous()
                and len(runs) == 1 and (C * D) % 4 == 0):
            # one pass of the library's block gather instead of torch's strided copies
            from . import _native
            n = runs[0][2]
            fwd, bwd = _chain_maps(B, L, n, pot.device)
            ctx.maps = bwd
            return (_native.gather_blocks(pot, fwd, C * D, side=C).view(n, B, C, D),)
        out = []
        for s, m, n in runs:
            src = pot[:, s:s + m].transpose(0, 1)
            if n != m:
                full = torch.empty((n, B, C, D), dtype=pot.dtype, device=pot.device)
                full[:m].copy_(src)
                full[m:] = -1e9
                full[m:].diagonal(dim1=-2, dim2=-1).zero_()
                src = full
            out.append(_bit_reversed(src, n.bit_length() - 1))
        return tuple(out)

    @staticmethod
    def backward(ctx, *grads):
        if ctx.maps is not None:
            # taken only together with the fused tree levels, which are first-order themselves
            from . import _native
            B, L, C, D = ctx.shape
            return _native.gather_blocks(grads[0].detach().contiguous(), ctx.maps, C * D).view(ctx.shape), None
        # differentiable torch operations: a double backward passes through here
        parts = [_bit_reversed(g, n.bit_length() - 1)[:m].transpose(0, 1) for (s, m, n), g in zip(_runs(ctx.shape[1]),
                                                                                                    grads)]
        return torch.cat(parts, 1), None


_map_cache = {}


def _chain_maps(B, L, n, device):
    """Block indices for the chain-major bit-reversed layout of one run of L matrices padded to n = 2**k:
    forward[r * B + b] = b * L + bitrev(r), or -1 where bitrev(r) >= L (an identity pad);
    backward[b * L + c] = bitrev(c) * B + b."""
    key = (B, L, n, str(device))
    if key not in _map_cache:
        k = n.bit_length() - 1
        r = torch.arange(n, device=device)
        rev = torch.zeros_like(r)
        for bit in range(k):
            rev |= ((r >> bit) & 1) << (k - 1 - bit)
        b = torch.arange(B, device=device)
        fwd = torch.where(rev[:, None] < L, b[None, :] * L + rev[:, None], torch.full((), -1, device=device))
        bwd = rev[None, :L] * B + b[:, None]
        if len(_map_cache) > 8:
            _map_cache.clear()
        _map_cache[key] = (fwd.reshape(-1).contiguous(), bwd.reshape(-1).contiguous())
    return _map_cache[key]


class _Halves(torch.autograd.Function):
    """(2p, B, C, C) -> the first and the second half as (p*B, C, C) views; the backward joins the two gradients
    in one copy (autograd through two slices would zero-fill and add two full-size tensors)."""

    @staticmethod
    def forward(ctx, x):
        L, B, C, D = x.shape
        p = L // 2
        ctx.shape = (p, B, C, D)
        return x[:p].view(p * B, C, D), x[p:].view(p * B, C, D)

    @staticmethod
    def backward(ctx, g_left, g_right):
        p, B, C, D = ctx.shape
        return torch.cat((g_left.reshape(p, B, C, D), g_right.reshape(p, B, C, D)), 0)


class _PairLevel(torch.autograd.Function):
    """One level of the tree on the GPU: x (2p, B, C, C) -> (p, B, C, C), first half (x) second half, through the
    factorised tensor-core logbmm.  The backward hands the two halves of one gradient buffer to the kernels as
    their outputs, so nothing is joined or copied.  First-order only: a double backward through this node raises
    (pass `bmm=genbmm_b200.logbmm` to chain_product for second-order gradients; logbmm implements them)."""

    @staticmethod
    def forward(ctx, x):
        from . import _native
        L, B, C, D = x.shape
        p = L // 2
        left, right = x[:p].view(p * B, C, D), x[p:].view(p * B, C, D)
        out, rowmax, colmax, flags, factors = _native.logbmm_fast_forward(left, right, tensor_cores=True,
                                                                          keep_factors=True)
        from .genmul import _keep_factors
        if not _keep_factors(left, right):
            factors = None      # the backward rebuilds them
        ctx.save_for_backward(x, out, rowmax, colmax, flags, factors)
        return out.view(p, B, C, D)

    @staticmethod
    @once_differentiable
    def backward(ctx, g):
        from . import _native
        x, out, rowmax, colmax, flags, factors = ctx.saved_tensors
        L, B, C, D = x.shape
        p = L // 2
        gx = torch.empty_like(x)
        _native.logbmm_fast_backward(x[:p].view(p * B, C, D), x[p:].view(p * B, C, D),
                                     g.contiguous().view(p * B, C, D), out, rowmax, colmax, flags, tensor_cores=True,
                                     out_grads=(gx[:p].view(p * B, C, D), gx[p:].view(p * B, C, D)), factors=factors)
        return gx


def _fused_levels(x, bmm):
    """The GPU fast path applies to float32 CUDA chains reduced with the default product, at sizes the
    tensor-core logbmm takes anyway."""
    if bmm is not None or not x.is_cuda or x.dtype != torch.float32:
        return False
    from .genmul import _log_path
    return _log_path(x.shape[2], x.shape[3], x.shape[3]) == "tensor"


def chain_product(pot, bmm=None):
    """(B, L, C, C) -> (B, C, C): the log-semiring product of the L matrices of each chain.

    The chain is cut into power-of-two runs (_runs); each run is
    reduced by a balanced pairwise tree (level l is one product with batch B * run / 2^(l+1)) on a
    chain-major, bit-reversed copy (see _ChainMajor), and the few run products are multiplied in order."""
    fused = _fused_levels(pot, bmm)
    bmm = bmm or _default_bmm()
    B, L, C, D = pot.shape
    assert C == D, "transition matrices must be square"
    parts = []
    for x in _ChainMajor.apply(pot, fused):
        while x.shape[0] > 1:
            if fused:
                x = _PairLevel.apply(x)
            else:
                left, right = _Halves.apply(x)
                x = bmm(left, right).view(x.shape[0] // 2, B, C, C)
        parts.append(x[0])
    out = parts[0]
    for nxt in parts[1:]:
        out = bmm(out.contiguous(), nxt.contiguous())
    return out


def log_partition(pot, bmm=None):
    """logZ:(B,) of chains with potentials pot:(B, T-1, C, C)."""
    return chain_product(pot, bmm).flatten(1).logsumexp(1)


def marginals(pot, bmm=None):
    """(logZ, edge marginals) — the marginals have pot's shape and sum to 1 over each (C, C) slice."""
    pot = pot.detach().requires_grad_(True)
    logz = log_partition(pot, bmm)
    grad, = torch.autograd.grad(logz.sum(), pot)
    return logz.detach(), grad


class GraphedMarginals:
    """marginals() for one fixed shape, captured once into a CUDA graph and replayed.

    The tree has log2(T) levels and each level is a handful of launches in either direction; at the upper
    levels the products are tiny and the host cannot issue launches as fast as the GPU retires them.  The
    capture records the whole forward and backward (layout conversion, every level, the final logsumexp and
    its gradient) on static buffers, so a call is one copy into the input buffer and one graph launch.

        run = GraphedMarginals((B, T - 1, C, C), device)
        logz, marg = run(pot)        # views of the graph's own output buffers: copy them to keep them

    Nothing in the captured region synchronises with the host: the guard flags of the factorised logbmm are
    consumed on the device."""

    def __init__(self, shape, device, dtype=torch.float32, warmup=3):
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError("GraphedMarginals needs a CUDA device")
        self.pot = torch.zeros(shape, dtype=dtype, device=device)
        with torch.cuda.device(device):
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(max(warmup, 1)):      # loads every kernel and fills the driver-side caches
                    marginals(self.pot)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.logz, self.grad = marginals(self.pot)

    def __call__(self, pot):
        if tuple(pot.shape) != tuple(self.pot.shape) or pot.dtype != self.pot.dtype:
            raise RuntimeError("captured for %s %s, got %s %s" % (tuple(self.pot.shape), self.pot.dtype,
                                                                  tuple(pot.shape), pot.dtype))
        self.pot.copy_(pot)
        self.graph.replay()
        return self.logz, self.grad


class _GatherKeepOwnGrad(torch.autograd.Function):
    """All-gather along a new leading rank axis.  Every rank goes on to compute the same
    replicated loss from the gathered tensor, so the gradient each rank needs is just the slice
    of its own contribution: the backward takes that slice and communicates nothing."""

    @staticmethod
    def forward(ctx, x, group):
        world = dist.get_world_size(group)
        ctx.rank = dist.get_rank(group)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.stack(parts, 0)

    @staticmethod
    def backward(ctx, grad):
        return grad[ctx.rank], None


def sharded_log_partition(pot_chunk, group=None, bmm=None):
    """logZ when the chain is split across ranks by position: rank r holds the contiguous chunk
    pot_chunk:(B, L_r, C, C) (chunks in rank order make up the chain).  Each rank reduces its chunk
    with the local tree, the partial products (B, C, C) are all-gathered — the one exchange step
    of this path — and every rank finishes the remaining log2(world) levels redundantly.
    Differentiating the result w.r.t. pot_chunk gives this rank's slice of the marginals."""
    partial = chain_product(pot_chunk, bmm)
    gathered = _GatherKeepOwnGrad.apply(partial, group)            # (world, B, C, C)
    full = chain_product(gathered.transpose(0, 1).contiguous(), bmm)
    return full.flatten(1).logsumexp(1)
