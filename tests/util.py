"""Shared helpers of the test-suite: seeded inputs of the benchmark configurations and comparators."""
import numpy as np
import torch

# tolerance of the log / sum semirings: 1e-5 relative (fp32), with an absolute floor for values
# that happen to lie near zero
RTOL, ATOL = 1e-5, 2e-6


def assert_close(got, want, rtol=RTOL, atol=ATOL, what="", term_sum=None):
    """|got - want| <= atol + rtol |want|.  For sums of signed terms (the ordinary semiring) a result may be
    the small difference of large terms; `term_sum` = the same sum over the terms' absolute values then also
    admits 1e-6 of it, the componentwise bound of a float32 sum (a few ulp of the terms' total)."""
    got = got.detach().cpu().numpy() if hasattr(got, "detach") else np.asarray(got)
    want = np.asarray(want)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    bad = ~np.isclose(got, want, rtol=rtol, atol=atol, equal_nan=True)
    if term_sum is not None:
        bad &= ~(np.abs(got - want) <= 1e-6 * np.asarray(term_sum))
    if bad.any():
        i = np.argwhere(bad)[0]
        raise AssertionError("%s: %d of %d differ; first at %s: got %r want %r" % (
            what, bad.sum(), bad.size, tuple(i), got[tuple(i)], want[tuple(i)]))


def assert_equal_bits(got, want, what=""):
    """Bit-for-bit equality (distinguishes +0/-0)."""
    got = got.detach().cpu().numpy() if hasattr(got, "detach") else np.asarray(got)
    want = np.asarray(want)
    assert got.shape == want.shape and got.dtype == want.dtype, (what, got.shape, want.shape, got.dtype, want.dtype)
    g = got.view(np.uint32) if got.dtype == np.float32 else got
    w = want.view(np.uint32) if want.dtype == np.float32 else want
    bad = g != w
    if bad.any():
        i = np.argwhere(bad)[0]
        raise AssertionError("%s: %d of %d differ; first at %s: got %r want %r" % (
            what, bad.sum(), bad.size, tuple(i), got[tuple(i)], want[tuple(i)]))


def cfg1(B=32, M=64, K=64, N=64):
    g = torch.Generator().manual_seed(0)
    return torch.rand(B, M, K, generator=g), torch.rand(B, K, N, generator=g)


def cfg2(B=256, M=128, K=128, N=128):
    g = torch.Generator().manual_seed(1)
    a = (torch.randn(B, M, K, generator=g) * 8).round() / 8
    b = (torch.randn(B, K, N, generator=g) * 8).round() / 8
    return a, b


def cfg3(B=64, M=256, K=256, N=256):
    g = torch.Generator().manual_seed(2)
    a = 2 * torch.randn(B, M, K, generator=g)
    b = 2 * torch.randn(B, K, N, generator=g)
    u = torch.rand(B, M, N, generator=g)
    return a, b, u


def cfg5(B=32, n=8192, lu=64, ld=64):
    g = torch.Generator().manual_seed(4)
    return torch.randn(B, n, lu + ld + 1, generator=g), torch.randn(B, n, lu + ld + 1, generator=g)


def band_inside(B, n, lu, ld):
    i = np.arange(n)[:, None]
    j = np.arange(lu + ld + 1)[None, :]
    o = i + j - lu
    return np.broadcast_to((o >= 0) & (o < n), (B, n, lu + ld + 1))


def assert_valid_sample(a, b, u, idx, tol=1e-5):
    """Every drawn index k brackets its uniform: cdf(k-1) - tol <= u <= cdf(k) + tol in fp64
    (or no k can: u ~ 0 or u beyond the total mass, where the reference leaves index 0)."""
    a, b, u = (np.asarray(x, dtype=np.float64) for x in (a, b, u))
    idx = np.asarray(idx).astype(np.int64)
    s = a[:, :, :, None] + b[:, None, :, :]
    s = s - s.max(2, keepdims=True)
    p = np.exp(s)
    p /= p.sum(2, keepdims=True)
    cdf = np.cumsum(p, axis=2)
    hi = np.take_along_axis(cdf, idx[:, :, None, :], 2)[:, :, 0, :]
    lo = hi - np.take_along_axis(p, idx[:, :, None, :], 2)[:, :, 0, :]
    ok = (lo - tol <= u) & (u <= hi + tol)
    # the strict double inequality also fails when the fp32 running sum lands exactly on u:
    # u then sits on a CDF step, and the reference leaves index 0
    on_step = np.abs(cdf - u[:, :, None, :]).min(2) <= tol
    none = (idx == 0) & ((u <= tol) | (u >= 1 - tol) | on_step)
    bad = ~(ok | none)
    if bad.any():
        w = np.argwhere(bad)[:4]
        detail = ["%s idx=%d u=%.8f lo=%.8f hi=%.8f" % (tuple(i), idx[tuple(i)], u[tuple(i)], lo[tuple(i)],
                                                      hi[tuple(i)]) for i in w]
        raise AssertionError("%d sampled indices do not bracket their uniform: %s" % (bad.sum(), "; ".join(detail)))


def rel_err(got, want, term_sum=None, rtol=RTOL, atol=ATOL):
    """The largest error in units in which `assert_close` passes at `rtol`: max |got - want| / (atol / rtol +
    |want|), the denominator widened to term_sum / 10 where that is larger (1e-6 of the terms' magnitudes)."""
    got = got.detach().cpu().numpy() if hasattr(got, "detach") else np.asarray(got)
    want = np.asarray(want, dtype=np.float64)
    den = atol / rtol + np.abs(want)
    if term_sum is not None:
        den = np.maximum(den, np.asarray(term_sum, dtype=np.float64) * (1e-6 / rtol))
    err = np.abs(got.astype(np.float64) - want) / den
    return float(np.nanmax(err)) if err.size else 0.0
