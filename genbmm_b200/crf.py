"""Linear-chain CRF log-partition by a log-semiring tree reduction — a caller of logbmm.

The reference has no such module (its README names PyTorch-Struct as the caller that does this);
this is the smallest driver for the benchmark configuration "linear-chain CRF, T positions,
C states": potentials pot:(B, T-1, C, C), the chain product

    P[b] = pot[b,0] (x) pot[b,1] (x) ... (x) pot[b,T-2],   (A (x) B)[i,j] = logsumexp_k A[i,k] + B[k,j]

evaluated as a balanced pairwise tree (an unpaired last matrix is carried up a level), so level l
is one logbmm call with batch B * (T-1) / 2^(l+1); logZ[b] = logsumexp_{i,j} P[b]; the edge
marginals are d(sum_b logZ[b]) / d pot, obtained by autograd through the tree.

`bmm` is the semiring product to use (default: genbmm_b200.logbmm); tests on CPU pass the
broadcast-reduce expression instead.
"""
import torch
import torch.distributed as dist


def _default_bmm():
    from .genmul import logbmm
    return logbmm


def chain_product(pot, bmm=None):
    """(B, L, C, C) -> (B, C, C): the log-semiring product of the L matrices of each chain."""
    bmm = bmm or _default_bmm()
    x = pot
    B, _, C, D = x.shape
    assert C == D, "transition matrices must be square"
    while x.shape[1] > 1:
        L = x.shape[1]
        pairs = L // 2
        left = x[:, 0:2 * pairs:2].reshape(B * pairs, C, C).contiguous()
        right = x[:, 1:2 * pairs:2].reshape(B * pairs, C, C).contiguous()
        y = bmm(left, right).view(B, pairs, C, C)
        x = torch.cat([y, x[:, L - 1:]], 1) if L % 2 else y
    return x[:, 0]


def log_partition(pot, bmm=None):
    """logZ:(B,) of chains with potentials pot:(B, T-1, C, C)."""
    return chain_product(pot, bmm).flatten(1).logsumexp(1)


def marginals(pot, bmm=None):
    """(logZ, edge marginals) — the marginals have pot's shape and sum to 1 over each (C, C) slice."""
    pot = pot.detach().requires_grad_(True)
    logz = log_partition(pot, bmm)
    grad, = torch.autograd.grad(logz.sum(), pot)
    return logz.detach(), grad


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
