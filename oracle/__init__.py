"""CPU oracle for genbmm's semiring products — TEST INFRASTRUCTURE, not the product.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
import this package.  It wraps oracle/genbmm_oracle.c (a plain-C restatement of
the reference's kernels, compiled by oracle/build.py) with numpy in/out, and
adds the broadcast-reduce PyTorch expressions the reference's README and tests
use as the definition of the dense operators.

Parity pinning: the reference holds no golden vectors; the fixtures under
tests/golden/ were produced by running the reference's own Python code
(genbmm/sparse.py and the dense expressions of genbmm/test_cuda.py:17,
README.md:30-65) and this oracle is checked against them.
"""
import ctypes

import numpy as np

from . import build as _build

_LIB = None

_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_int64


def lib():
    """Load (building if needed) the compiled oracle."""
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(_build.build())
        for suf in ("f32", "f64"):
            getattr(_LIB, "orc_dense_fwd_" + suf).argtypes = [_I, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L]
            getattr(_LIB, "orc_sample_margin_" + suf).argtypes = [_P, _P, _P, _P, _L, _L, _L, _L]
            getattr(_LIB, "orc_dense_bwd_" + suf).argtypes = [_I, _P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L]
            getattr(_LIB, "orc_dense_bwdbwd_" + suf).argtypes = [_P] * 9 + [_L] * 4
            getattr(_LIB, "orc_band_fwd_" + suf).argtypes = [_I, _P, _I, _I, _P, _I, _I, _P, _P, _P, _L, _L]
            getattr(_LIB, "orc_band_bwd_" + suf).argtypes = [_I, _P, _I, _I, _P, _I, _I, _P, _P, _P, _L, _L]
            getattr(_LIB, "orc_band_bwdbwd_" + suf).argtypes = [_P, _I, _I, _P, _I, _I] + [_P] * 7 + [_L, _L]
            getattr(_LIB, "orc_band_transpose_" + suf).argtypes = [_P, _I, _I, _P, _L, _L]
            for n in ("dense_fwd", "sample_margin", "dense_bwd", "dense_bwdbwd", "band_fwd", "band_bwd",
                      "band_transpose"):
                getattr(_LIB, "orc_%s_%s" % (n, suf)).restype = None
    return _LIB


def _np(x, dtype):
    """numpy view/copy of a numpy array or CPU torch tensor, C-contiguous, of `dtype`."""
    if hasattr(x, "detach"):
        x = x.detach().cpu().numpy()
    return np.ascontiguousarray(x, dtype=dtype)


def _ptr(x):
    return None if x is None else x.ctypes.data_as(_P)


def _suf(dtype):
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        return "f32"
    if dtype == np.float64:
        return "f64"
    raise ValueError("oracle supports float32 and float64 only")


MODE_LOG, MODE_MAX, MODE_SAMPLE, MODE_PRODMAX = 0, 1, 2, 3
BAND_LOG, BAND_MAX, BAND_MUL = 0, 1, 3


def dense_fwd(mode, a, b, u=None, dtype=np.float32):
    """Reference forward (matmul_cuda_kernel.cu:13-152).  Returns (out, aux):
    aux is `maxes` for mode 0 and the int32 index tensor for modes 1-3."""
    a, b = _np(a, dtype), _np(b, dtype)
    B, M, K = a.shape
    N = b.shape[2]
    assert b.shape == (B, K, N)
    out = np.zeros((B, M, N), dtype)
    maxes = np.zeros((B, M, N), dtype) if mode == 0 else None
    idx = np.zeros((B, M, N), np.int32) if mode != 0 else None
    if mode == 2:
        u = _np(u, dtype)
        assert u.shape == (B, M, N)
    getattr(lib(), "orc_dense_fwd_" + _suf(dtype))(mode, _ptr(a), _ptr(b), _ptr(u) if mode == 2 else None,
                                                   _ptr(out), _ptr(maxes), _ptr(idx), B, M, K, N)
    return out, (maxes if mode == 0 else idx)


def sample_margin(a, b, u, dtype=np.float32):
    """Distance (in probability mass, fp64) of each uniform from the nearest CDF step."""
    a, b, u = _np(a, dtype), _np(b, dtype), _np(u, dtype)
    B, M, K = a.shape
    N = b.shape[2]
    margin = np.zeros((B, M, N), np.float64)
    getattr(lib(), "orc_sample_margin_" + _suf(dtype))(_ptr(a), _ptr(b), _ptr(u), _ptr(margin), B, M, K, N)
    return margin


def dense_bwd(mode, a, b, g, part=None, aux=None, dtype=np.float32):
    """Reference backward (matmul_cuda_kernel.cu:159-217, 336-456).  `part`/`aux` are the forward's
    (out, maxes) for mode 0; `aux` the int32 indices for modes 1-3.  Returns (grad_a, grad_b)."""
    a, b, g = _np(a, dtype), _np(b, dtype), _np(g, dtype)
    B, M, K = a.shape
    N = b.shape[2]
    dA, dB = np.zeros_like(a), np.zeros_like(b)
    if mode == 0:
        part, maxes, idx = _np(part, dtype), _np(aux, dtype), None
    else:
        part, maxes, idx = None, None, _np(aux, np.int32)
    getattr(lib(), "orc_dense_bwd_" + _suf(dtype))(mode, _ptr(a), _ptr(b), _ptr(g), _ptr(part), _ptr(maxes),
                                                   _ptr(idx), _ptr(dA), _ptr(dB), B, M, K, N)
    return dA, dB


def dense_bwdbwd(a, b, g, part, maxes, h, dtype=np.float32):
    """Second-order terms of the log product (matmul_cuda_kernel.cu:220-331) for the cotangent `h`
    of grad_a.  Returns (d/da, d/db, d/dgrad_out)."""
    a, b, g, part, maxes, h = (_np(x, dtype) for x in (a, b, g, part, maxes, h))
    B, M, K = a.shape
    N = b.shape[2]
    dA, dB, dG = np.zeros_like(a), np.zeros_like(b), np.zeros_like(g)
    getattr(lib(), "orc_dense_bwdbwd_" + _suf(dtype))(_ptr(a), _ptr(b), _ptr(g), _ptr(part), _ptr(maxes),
                                                      _ptr(h), _ptr(dA), _ptr(dB), _ptr(dG), B, M, K, N)
    return dA, dB, dG


def band_fwd(mode, a, a_lu, a_ld, b, b_lu, b_ld, dtype=np.float32):
    """Reference banded forward (banded_cuda_kernel.cu:13-100, 354-402).
    Returns (out, indices, maxes), all zero-initialised as the dispatcher does."""
    a, b = _np(a, dtype), _np(b, dtype)
    B, n, Wa = a.shape
    assert Wa == a_lu + a_ld + 1 and b.shape == (B, n, b_lu + b_ld + 1)
    Wo = Wa + b.shape[2] - 1
    out = np.zeros((B, n, Wo), dtype)
    idx = np.zeros((B, n, Wo), np.int32)
    maxes = np.zeros((B, n, Wo), dtype)
    getattr(lib(), "orc_band_fwd_" + _suf(dtype))(mode, _ptr(a), a_lu, a_ld, _ptr(b), b_lu, b_ld, _ptr(out),
                                                  _ptr(idx), _ptr(maxes), B, n)
    return out, idx, maxes


def band_bwd(mode, a, a_lu, a_ld, b, b_lu, b_ld, g, part, dtype=np.float32):
    """Reference banded backward w.r.t. the first operand (banded_cuda_kernel.cu:104-152, 404-450)."""
    a, b, g = _np(a, dtype), _np(b, dtype), _np(g, dtype)
    part = _np(part, dtype) if part is not None else g
    B, n, _ = a.shape
    dA = np.zeros_like(a)
    getattr(lib(), "orc_band_bwd_" + _suf(dtype))(mode, _ptr(a), a_lu, a_ld, _ptr(b), b_lu, b_ld, _ptr(g),
                                                  _ptr(part), _ptr(dA), B, n)
    return dA


def band_bwdbwd(a, a_lu, a_ld, b, b_lu, b_ld, g, part, h_a, h_b=None, dtype=np.float32):
    """Second-order terms of the banded log product (banded_cuda_kernel.cu:154-350, 453-546): for
    L = <grad_a, h_a> + <grad_b, h_b> returns (dL/da, dL/db, dL/dg).  The reference has h_a only."""
    a, b, g, part, h_a = (_np(x, dtype) for x in (a, b, g, part, h_a))
    h_b = np.zeros_like(b) if h_b is None else _np(h_b, dtype)
    B, n, _ = a.shape
    dA, dB, dG = np.zeros_like(a), np.zeros_like(b), np.zeros_like(g)
    getattr(lib(), "orc_band_bwdbwd_" + _suf(dtype))(_ptr(a), a_lu, a_ld, _ptr(b), b_lu, b_ld, _ptr(g), _ptr(part),
                                                     _ptr(h_a), _ptr(h_b), _ptr(dA), _ptr(dB), _ptr(dG), B, n)
    return dA, dB, dG


def band_transpose(x, lu, ld, dtype=np.float32):
    """BandedMatrix.transpose() data (sparse.py:214-218, 65-70, 33-47); result bands are (ld, lu)."""
    x = _np(x, dtype)
    B, n, _ = x.shape
    out = np.zeros_like(x)
    getattr(lib(), "orc_band_transpose_" + _suf(dtype))(_ptr(x), lu, ld, _ptr(out), B, n)
    return out


def band_fwd_bwd(mode, a, a_lu, a_ld, b, b_lu, b_ld, g, dtype=np.float32):
    """Forward plus both gradients, routed the way the reference's autograd Functions do it:
    grad_a by one backward call, grad_b by a second call with the operands swapped and the
    cotangent / saved output band-transposed (sparse.py:415-447 mul, 523-545 log, 585-637 max —
    the max product runs a second, swapped forward to get indices in b's band coordinate)."""
    o_lu, o_ld = a_lu + b_ld, a_ld + b_lu
    out, idx, maxes = band_fwd(mode, a, a_lu, a_ld, b, b_lu, b_ld, dtype)
    gT = band_transpose(g, o_lu, o_ld, dtype)
    if mode == BAND_MUL:
        dA = band_bwd(3, a, a_lu, a_ld, b, b_lu, b_ld, g, None, dtype)
        dB = band_bwd(3, b, b_lu, b_ld, a, a_lu, a_ld, gT, None, dtype)
    elif mode == BAND_LOG:
        dA = band_bwd(0, a, a_lu, a_ld, b, b_lu, b_ld, g, out, dtype)
        outT = band_transpose(out, o_lu, o_ld, dtype)
        dB = band_bwd(0, b, b_lu, b_ld, a, a_lu, a_ld, gT, outT, dtype)
    else:
        _, idx2, _ = band_fwd(1, b, b_lu, b_ld, a, a_lu, a_ld, dtype)
        dA = band_bwd(1, a, a_lu, a_ld, b, b_lu, b_ld, g, idx.astype(dtype), dtype)
        dB = band_bwd(1, b, b_lu, b_ld, a, a_lu, a_ld, gT, idx2.astype(dtype), dtype)
    return out, idx, maxes, dA, dB


# --------------------------------------------------------------------------------------------
# The reference's own definition of the dense operators: broadcast-reduce PyTorch expressions
# (README.md:30-65, genbmm/test_cuda.py:17).  Used as the timed CPU baseline and as a second
# opinion on the C restatement.  The (B,M,K,N) intermediate is capped by chunking over batch.
# --------------------------------------------------------------------------------------------

def expr_forward(mode, a, b):
    """c for torch CPU tensors a:(B,M,K), b:(B,K,N) by the reference's broadcast expression."""
    s = a.unsqueeze(-1) + b.unsqueeze(-3) if mode != MODE_PRODMAX else a.unsqueeze(-1) * b.unsqueeze(-3)
    if mode in (MODE_LOG, MODE_SAMPLE):
        return s.logsumexp(-2)
    return s.max(-2)[0]


def expr_fwd_bwd(mode, a, b, g=None, chunk_bytes=1 << 30):
    """Forward + autograd backward of the broadcast expression, chunked over batch.
    Returns (c, grad_a, grad_b) as torch CPU tensors."""
    import torch

    B, M, K = a.shape
    N = b.shape[2]
    per = M * K * N * a.element_size()
    step = max(1, int(chunk_bytes // max(per, 1)))
    cs, gas, gbs = [], [], []
    for s in range(0, B, step):
        ac = a[s:s + step].detach().clone().requires_grad_(True)
        bc = b[s:s + step].detach().clone().requires_grad_(True)
        c = expr_forward(mode, ac, bc)
        gc = torch.ones_like(c) if g is None else g[s:s + step]
        ga, gb = torch.autograd.grad(c, (ac, bc), gc)
        cs.append(c.detach())
        gas.append(ga)
        gbs.append(gb)
    return torch.cat(cs), torch.cat(gas), torch.cat(gbs)


# --------------------------------------------------------------------------------------------
# Linear-chain CRF (benchmark configuration 4): left-to-right semiring products in float64 with
# autograd for the edge marginals.  The reference has no such routine; this restates the
# configuration's definition (chain product of the potentials, logZ = logsumexp of its entries).
# --------------------------------------------------------------------------------------------

def crf_log_partition(pot):
    """(logZ, marginals) for torch CPU potentials pot:(B, L, C, C), in float64, sequentially."""
    import torch

    pot = pot.detach().double().requires_grad_(True)
    p = pot[:, 0]
    for t in range(1, pot.shape[1]):
        p = (p.unsqueeze(-1) + pot[:, t].unsqueeze(-3)).logsumexp(-2)
    logz = p.flatten(1).logsumexp(1)
    grad, = torch.autograd.grad(logz.sum(), pot)
    return logz.detach(), grad


def crf_alpha_beta(pot):
    """(logZ, edge marginals) of ONE chain, pot:(L, C, C), by the forward-backward recursions in float64
    numpy — O(L C^2) time and memory, so the full benchmark size (L = 511, C = 256) takes a second, where
    autograd through a float64 chain product would hold every intermediate.

    With alpha_t[j] = log-mass of the prefixes that end edge t in state j and beta_t[j] = log-mass of the
    suffixes that follow edge t from state j,

        alpha_t[j] = logsumexp_i alpha_{t-1}[i] + pot[t, i, j]      (alpha_{-1} = 0)
        beta_t[i]  = logsumexp_j pot[t+1, i, j] + beta_{t+1}[j]     (beta_{L-1} = 0)
        logZ       = logsumexp_j alpha_{L-1}[j]
        marginal[t, i, j] = exp(alpha_{t-1}[i] + pot[t, i, j] + beta_t[j] - logZ)

    which is d logZ / d pot[t, i, j] for logZ = logsumexp of all entries of the chain product, the
    definition `crf_log_partition` differentiates; tests check the two against each other."""
    p = _np(pot, np.float64)
    L, C, _ = p.shape

    def lse(x, axis):
        m = x.max(axis=axis, keepdims=True)
        return (m + np.log(np.exp(x - m).sum(axis=axis, keepdims=True))).squeeze(axis)

    alpha = np.zeros((L + 1, C))          # alpha[t + 1] = alpha_t, alpha[0] = alpha_{-1} = 0
    for t in range(L):
        alpha[t + 1] = lse(alpha[t][:, None] + p[t], 0)
    beta = np.zeros((L, C))
    for t in range(L - 2, -1, -1):
        beta[t] = lse(p[t + 1] + beta[t + 1][None, :], 1)
    logz = lse(alpha[L], 0)
    marg = np.exp(alpha[:L, :, None] + p + beta[:, None, :] - logz)
    return float(logz), marg
