"""The kernels behind the headline numbers against the float64 oracle, called the way a user calls
them (`genbmm_b200.logbmm` + autograd): the CTA-pair tensor-core kernel in all three of its operand
forms, an operand-scale sweep of the default logbmm path, and the full-size chain and banded
configurations on more than one batch element.

Tolerances.  Log semiring: rtol 1e-5, atol 2e-6 (util.RTOL / util.ATOL).  Where a gradient is a sum
of terms of both signs (a signed cotangent) no float32 algorithm can meet a bound relative to the
cancelled sum; those comparisons also admit 1e-6 of the same sum taken over the terms' magnitudes
(the oracle run on |g|), which is what `assert_close(term_sum=...)` implements.  Every test prints the
error it measured, so the margins can be read from the log.
"""
import numpy as np
import pytest
import torch

import oracle
from util import assert_close, assert_equal_bits, cfg5, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gb():
    import genbmm_b200
    return genbmm_b200


def op_fwd_bwd(gb, a, b, g):
    ad, bd = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    c = gb.logbmm(ad, bd)
    ga, gb_ = torch.autograd.grad(c, (ad, bd), g.cuda())
    return c.detach(), ga, gb_


@pytest.mark.parametrize("cotangent", ["ones", "uniform", "signed"])
def test_benchmark_shape_all_three_products_against_oracle(gb, cotangent):
    """1024^3 (the shape the bench times): forward, grad_a and grad_b all run on the CTA-pair tcgen05
    kernel (A K-major / B MN-major, both K-major, both MN-major).  The oracle covers 96 rows of out and
    grad_a and 96 columns of grad_b of one batch element — the same number of (m,k,n) triples each."""
    gen = torch.Generator().manual_seed(9)
    a, b = torch.randn(2, 1024, 1024, generator=gen), torch.randn(2, 1024, 1024, generator=gen)
    g = {"ones": torch.ones(2, 1024, 1024), "uniform": torch.rand(2, 1024, 1024, generator=gen),
         "signed": torch.randn(2, 1024, 1024, generator=gen)}[cotangent]
    c, ga, gb_ = op_fwd_bwd(gb, a, b, g)
    # rows: out and grad_a need every column of b
    want, maxes = oracle.dense_fwd(0, a[:1, :96], b[:1], dtype=np.float64)
    dA, _ = oracle.dense_bwd(0, a[:1, :96], b[:1], g[:1, :96], want, maxes, dtype=np.float64)
    # columns: grad_b[:, :, :96] needs every row of a and the 96 columns of out and g
    want_c, maxes_c = oracle.dense_fwd(0, a[:1], b[:1, :, :96], dtype=np.float64)
    _, dB = oracle.dense_bwd(0, a[:1], b[:1, :, :96], g[:1, :, :96], want_c, maxes_c, dtype=np.float64)
    ta = tb = None
    if cotangent == "signed":
        ta, _ = oracle.dense_bwd(0, a[:1, :96], b[:1], g[:1, :96].abs(), want, maxes, dtype=np.float64)
        _, tb = oracle.dense_bwd(0, a[:1], b[:1, :, :96], g[:1, :, :96].abs(), want_c, maxes_c, dtype=np.float64)
    print("1024^3 %s: max rel err out %.2e grad_a %.2e grad_b %.2e" % (
        cotangent, rel_err(c[:1, :96], want), rel_err(ga[:1, :96], dA, ta), rel_err(gb_[:1, :, :96], dB, tb)))
    assert_close(c[:1, :96], want, what="fwd rows")
    assert_close(c[:1, :, :96], want_c, what="fwd columns")
    assert_close(ga[:1, :96], dA, what="grad_a", term_sum=ta)
    assert_close(gb_[:1, :, :96], dB, what="grad_b", term_sum=tb)


def test_pair_kernel_odd_shape_fully_against_oracle(gb):
    """An odd shape big enough that forward, grad_a and grad_b all take the CTA-pair kernel (reduction x
    smaller result side >= 512 x 1024 in each): ragged last tiles in every direction, unaligned pitches,
    whole result against float64."""
    B, M, K, N = 1, 741, 1030, 713
    assert min(K * min(M, N), N * min(M, K), M * min(K, N)) >= 512 * 1024
    gen = torch.Generator().manual_seed(77)
    a, b = torch.randn(B, M, K, generator=gen), torch.randn(B, K, N, generator=gen)
    g = torch.rand(B, M, N, generator=gen)
    c, ga, gb_ = op_fwd_bwd(gb, a, b, g)
    want, maxes = oracle.dense_fwd(0, a, b, dtype=np.float64)
    dA, dB = oracle.dense_bwd(0, a, b, g, want, maxes, dtype=np.float64)
    print("741x1030x713: max rel err out %.2e grad_a %.2e grad_b %.2e" % (
        rel_err(c, want), rel_err(ga, dA), rel_err(gb_, dB)))
    assert_close(c, want, what="fwd")
    assert_close(ga, dA, what="grad_a")
    assert_close(gb_, dB, what="grad_b")


@pytest.mark.parametrize("K", [64, 1024])
@pytest.mark.parametrize("std", [0.1, 1.0, 5.0, 20.0])
def test_default_path_operand_scale_sweep(gb, std, K):
    """The default path of logbmm (factorised, 3xTF32 on tcgen05, lg2.approx epilogue) as the operands'
    spread grows: row maximum + column maximum overshoots max_k(a+b) by more and more, the factorised sum
    shrinks towards the guard threshold (2^-90) and result tiles start to take the exact kernels."""
    from genbmm_b200 import _native, genmul
    B, M, N = 2, 192, 160
    assert genmul._log_path(M, K, N) == "tensor"
    gen = torch.Generator().manual_seed(int(std * 10) + K)
    a, b = std * torch.randn(B, M, K, generator=gen), std * torch.randn(B, K, N, generator=gen)
    g = torch.rand(B, M, N, generator=gen)
    c, ga, gb_ = op_fwd_bwd(gb, a, b, g)
    flags = _native.logbmm_fast_forward(a.cuda(), b.cuda(), tensor_cores=True)[3]
    want, maxes = oracle.dense_fwd(0, a, b, dtype=np.float64)
    dA, dB = oracle.dense_bwd(0, a, b, g, want, maxes, dtype=np.float64)
    print("std %-4g K %-4d flagged tiles %d of %d; max rel err out %.2e grad_a %.2e grad_b %.2e" % (
        std, K, int(flags.sum()), flags.numel(), rel_err(c, want), rel_err(ga, dA), rel_err(gb_, dB)))
    # a + b and the saved result are float32 numbers as large as max|c| (150 at std 20): their spacing there is
    # a relative error of every weight exp(a + b - c), whatever computes it (at std 20 every tile is flagged
    # and it is the exact kernels that are measured).  1.1e-5 up to std 1, 1.8e-5 at std 5, 4e-5 at std 20.
    rtol_w = 1e-5 + 2 * float(np.spacing(np.float32(np.abs(want).max())))
    assert rtol_w < 5e-5
    assert_close(c, want, what="fwd")
    assert_close(ga, dA, rtol_w, what="grad_a")
    assert_close(gb_, dB, rtol_w, what="grad_b")


def test_config4_marginals_against_forward_backward_recursions():
    """cfg4 at full size (B 16, T 512, C 256): log-partition and every edge marginal of batch elements 0 and
    15 against the float64 alpha/beta recursions.  A marginal is a product of nine levels of softmax
    weights, each within 1e-5: rtol 2e-4 (measured error printed)."""
    from genbmm_b200 import crf
    gen = torch.Generator().manual_seed(3)
    pot = torch.randn(16, 511, 256, 256, generator=gen)
    logz, marg = crf.marginals(pot.cuda())
    for bi in (0, 15):
        want_z, want_m = oracle.crf_alpha_beta(pot[bi])
        got = marg[bi].cpu().numpy()
        print("cfg4 element %d: logZ rel err %.2e, marginals max rel err %.2e" % (
            bi, abs(float(logz[bi]) - want_z) / abs(want_z), rel_err(got, want_m, atol=1e-12)))
        assert abs(float(logz[bi]) - want_z) <= 1e-5 * abs(want_z)
        assert_close(got, want_m, 2e-4, 1e-12, what="marginals of element %d" % bi)


@pytest.mark.parametrize("element", [0, 15, 31])
def test_config5_against_oracle_on_three_batch_elements(element):
    """cfg5 (n 8192, 129 diagonals, batch 32): the three banded products, forward and both gradients, of
    batch elements 0, 15 and 31 of the full-size call against the oracle."""
    from genbmm_b200 import _native
    a, b = cfg5()
    lu = ld = 64
    ad, bd = a.cuda(), b.cuda()
    g = torch.rand(32, 8192, 257, generator=torch.Generator().manual_seed(44))
    gd = g.cuda()
    s = slice(element, element + 1)
    for mode in (3, 0, 1):
        out, idx, _ = _native.forward_band(ad, lu, ld, bd, lu, ld, mode)
        part = out if mode == 0 else idx
        ga, gb_ = _native.backward_band(ad, lu, ld, bd, lu, ld, gd, part, mode, both=True)
        dt = np.float32 if mode == 1 else np.float64
        wout, widx, _, dA, dB = oracle.band_fwd_bwd(mode, a[s], lu, ld, b[s], lu, ld, g[s], dtype=dt)
        if mode == 1:
            assert_equal_bits(out[s], wout)
            assert_equal_bits(idx[s], widx)
            assert_equal_bits(ga[s], dA)
            assert_equal_bits(gb_[s], dB)
            continue
        bound = (None, None, None)
        if mode == 3:  # signed terms: 1e-6 of the same sums over magnitudes
            t_out, _, _, t_dA, t_dB = oracle.band_fwd_bwd(3, a[s].abs(), lu, ld, b[s].abs(), lu, ld, g[s].abs(),
                                                          dtype=np.float64)
            bound = (t_out, t_dA, t_dB)
        print("cfg5 element %d mode %d: max rel err out %.2e grad_a %.2e grad_b %.2e" % (
            element, mode, rel_err(out[s], wout, bound[0]), rel_err(ga[s], dA, bound[1]),
            rel_err(gb_[s], dB, bound[2])))
        assert_close(out[s], wout, term_sum=bound[0], what="out")
        assert_close(ga[s], dA, term_sum=bound[1], what="grad_a")
        assert_close(gb_[s], dB, term_sum=bound[2], what="grad_b")
