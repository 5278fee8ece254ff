"""Randomised shapes for the bit-exact operators: max-plus / prod-max (dense) and multiply_max (banded) against
the oracle, values, indices and both gradients, on shapes drawn so that every kernel choice is hit — reductions
that are or are not multiples of 4, below and above the short-reduction limit, ragged tiles in both result
dimensions, bands narrower and wider than the tile sizes, and special values (ties, -inf, a NaN, rows that stay
below the reference's -1e9 floor)."""
import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings, strategies as st

import oracle
from util import assert_close, assert_equal_bits, assert_valid_sample

pytestmark = pytest.mark.gpu

SETTINGS = dict(max_examples=100, deadline=None, derandomize=True,
                suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])


def special(x, gen, how):
    """Sprinkle the values the reference's strict `>` from -1e9 treats specially."""
    if how == 1:
        x[..., ::3] = float("-inf")
    if how == 2:
        x.view(-1)[torch.randint(0, x.numel(), (1,), generator=gen)] = float("nan")
    if how == 3:
        x[:, 0] = -2e9
    return x


@settings(**SETTINGS)
@given(B=st.integers(1, 3), M=st.sampled_from([1, 7, 33, 64, 65, 100, 129, 150]),
       K=st.sampled_from([1, 3, 4, 8, 20, 60, 128, 130, 132, 288, 292, 300, 516, 1028]),
       N=st.sampled_from([1, 5, 31, 32, 33, 64, 97, 140]), mode=st.sampled_from([1, 3]), how=st.integers(0, 3), seed=st.integers(0, 10 ** 6))
def test_dense_max_semirings_random_shapes(B, M, K, N, mode, how, seed):
    import genbmm_b200 as gb
    from genbmm_b200 import _native
    gen = torch.Generator().manual_seed(seed)
    a = special((torch.randn(B, M, K, generator=gen) * 4).round() / 4, gen, how)
    b = (torch.randn(B, K, N, generator=gen) * 4).round() / 4
    g = torch.rand(B, M, N, generator=gen)
    ad, bd = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    fn = gb.maxbmm if mode == 1 else gb.prodmaxbmm
    c = fn(ad, bd)
    ga, gb_ = torch.autograd.grad(c, (ad, bd), g.cuda())
    out, idx = oracle.dense_fwd(mode, a, b)
    dA, dB = oracle.dense_bwd(mode, a, b, g, None, idx)
    _, idx_gpu = _native.forward(a.cuda(), b.cuda(), mode)
    assert_equal_bits(c, out, "value")
    assert_equal_bits(idx_gpu, idx, "index")
    # a NaN operand under prod-max makes NaN gradients wherever it is routed to: compare those as bits too
    assert_equal_bits(ga, dA, "grad_a")
    assert_equal_bits(gb_, dB, "grad_b")


@settings(**SETTINGS)
@given(B=st.integers(1, 2), n=st.sampled_from([128, 129, 191, 256, 333, 420]), alu=st.sampled_from([16, 31, 64, 90]),
       ald=st.sampled_from([15, 33, 64, 90]), blu=st.sampled_from([16, 40, 64, 90]), bld=st.sampled_from([15, 31, 64, 90]), how=st.integers(0, 3), seed=st.integers(0, 10 ** 6))
def test_banded_max_random_bands(B, n, alu, ald, blu, bld, how, seed):
    import genbmm_b200 as gb
    from genbmm_b200 import _native
    gen = torch.Generator().manual_seed(seed)
    a = special((torch.randn(B, n, alu + ald + 1, generator=gen) * 2).round() / 2, gen, how)
    b = (torch.randn(B, n, blu + bld + 1, generator=gen) * 2).round() / 2
    g = torch.rand(B, n, alu + ald + blu + bld + 1, generator=gen)
    ad, bd = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    r = gb.BandedMatrix(ad, alu, ald).multiply_max(gb.BandedMatrix(bd, blu, bld))
    ga, gb_ = torch.autograd.grad(r.data, (ad, bd), g.cuda())
    out, idx, _, dA, dB = oracle.band_fwd_bwd(1, a, alu, ald, b, blu, bld, g)
    _, idx_gpu, _ = _native.forward_band(a.cuda(), alu, ald, b.cuda(), blu, bld, 1)
    assert_equal_bits(r.data.detach(), out, "value")
    assert_equal_bits(idx_gpu, idx, "index")
    assert_equal_bits(ga, dA, "grad_a")
    assert_equal_bits(gb_, dB, "grad_b")


@settings(**SETTINGS)
@given(B=st.integers(1, 3), M=st.sampled_from([1, 10, 64, 65, 128, 130, 200]),
       K=st.sampled_from([1, 5, 16, 33, 64, 100, 128, 257, 512]), N=st.sampled_from([1, 13, 64, 100, 129, 200]), scale=st.sampled_from([0.1, 1.0, 5.0]), seed=st.integers(0, 10 ** 6))
def test_logbmm_random_shapes(B, M, K, N, scale, seed):
    """logbmm through the rule that picks its path (32x32-tile exact kernels, 128x64-tile exact kernels, 3xTF32
    tensor-core products with the underflow guard) against the float64 oracle at the stated 1e-5."""
    import genbmm_b200 as gb
    gen = torch.Generator().manual_seed(seed)
    a, b = scale * torch.randn(B, M, K, generator=gen), scale * torch.randn(B, K, N, generator=gen)
    g = torch.randn(B, M, N, generator=gen)
    ad, bd = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    c = gb.logbmm(ad, bd)
    ga, gb_ = torch.autograd.grad(c, (ad, bd), g.cuda())
    want, maxes = oracle.dense_fwd(0, a, b, dtype=np.float64)
    dA, dB = oracle.dense_bwd(0, a, b, g, want, maxes, dtype=np.float64)
    tA, tB = oracle.dense_bwd(0, a, b, g.abs(), want, maxes, dtype=np.float64)
    # a + b and the saved result are float32 numbers as large as max|c|: their spacing there is a relative error of
    # every weight exp(a + b - c), whatever computes it (tests/test_gpu_parity_full.py derives the same bound)
    rtol_w = 1e-5 + 2 * float(np.spacing(np.float32(np.abs(want).max())))
    assert rtol_w < 3e-5
    # the cotangent has both signs: a gradient may be the small difference of large terms, each carrying that
    # relative error, so the bound is rtol_w of the sum of the terms' magnitudes (the oracle on |g|)
    assert_close(c, want, what="fwd")
    assert_close(ga, dA, rtol_w, what="grad_a", term_sum=tA * (rtol_w / 1e-6))
    assert_close(gb_, dB, rtol_w, what="grad_b", term_sum=tB * (rtol_w / 1e-6))


@settings(**SETTINGS)
@given(B=st.integers(1, 2), n=st.sampled_from([1, 9, 70, 128, 131, 300, 420]), alu=st.sampled_from([0, 3, 20, 40, 70]),
       ald=st.sampled_from([0, 5, 31, 64]), blu=st.sampled_from([0, 2, 33, 64]), bld=st.sampled_from([0, 7, 31, 70]), mode=st.sampled_from([0, 3]), seed=st.integers(0, 10 ** 6))
def test_banded_sum_and_log_random_bands(B, n, alu, ald, blu, bld, mode, seed):
    """multiply and multiply_log over every path the band widths and n select (direct kernels, FP32 block
    kernels, 3xTF32 on the tensor cores from skewed copies) against the float64 oracle."""
    import genbmm_b200 as gb
    gen = torch.Generator().manual_seed(seed)
    a = torch.randn(B, n, alu + ald + 1, generator=gen)
    b = torch.randn(B, n, blu + bld + 1, generator=gen)
    g = torch.randn(B, n, alu + ald + blu + bld + 1, generator=gen) if mode == 3 else \
        torch.rand(B, n, alu + ald + blu + bld + 1, generator=gen)
    ad, bd = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    method = "multiply" if mode == 3 else "multiply_log"
    r = getattr(gb.BandedMatrix(ad, alu, ald), method)(gb.BandedMatrix(bd, blu, bld))
    ga, gb_ = torch.autograd.grad(r.data, (ad, bd), g.cuda())
    out, _, _, dA, dB = oracle.band_fwd_bwd(mode, a, alu, ald, b, blu, bld, g, dtype=np.float64)
    bound = (None, None, None)
    if mode == 3:  # signed terms: the same sums over absolute values bound the rounding error
        t_out, _, _, t_dA, t_dB = oracle.band_fwd_bwd(mode, a.abs(), alu, ald, b.abs(), blu, bld, g.abs(),
                                                      dtype=np.float64)
        bound = (t_out, t_dA, t_dB)
    assert_close(r.data.detach(), out, what=method, term_sum=bound[0])
    assert_close(ga, dA, what=method + " grad_a", term_sum=bound[1])
    assert_close(gb_, dB, what=method + " grad_b", term_sum=bound[2])


@settings(**dict(SETTINGS, max_examples=60))
@given(B=st.integers(1, 2), M=st.sampled_from([1, 9, 64, 70, 130]), K=st.sampled_from([1, 4, 17, 64, 129, 256]),
       N=st.sampled_from([1, 8, 65, 100, 128]), seed=st.integers(0, 10 ** 6))
def test_samplebmm_random_shapes(B, M, K, N, seed):
    """samplebmm with explicit uniforms: the index is the oracle's wherever the uniform is more than 1e-5 away
    from a step of the float64 CDF, a bracketing index elsewhere; gradients are the one-hot routing of the
    cotangent through the indices drawn, bit for bit."""
    import genbmm_b200 as gb
    from genbmm_b200 import _native, genmul
    gen = torch.Generator().manual_seed(seed)
    a, b = 2 * torch.randn(B, M, K, generator=gen), 2 * torch.randn(B, K, N, generator=gen)
    u, g = torch.rand(B, M, N, generator=gen), torch.rand(B, M, N, generator=gen)
    ad, bd = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    c = gb.samplebmm(ad, bd, u.cuda())
    ga, gb_ = torch.autograd.grad(c, (ad, bd), g.cuda())
    assert_close(c, oracle.dense_fwd(0, a, b, dtype=np.float64)[0], what="sample value")
    fast = genmul._log_path(M, K, N) == "tensor"
    _, idx_gpu = _native.forward(a.cuda(), b.cuda(), 2, u.cuda(), fast_log=fast)
    idx_gpu = idx_gpu.cpu().numpy()
    _, idx = oracle.dense_fwd(2, a, b, u)
    firm = oracle.sample_margin(a, b, u) > 1e-5
    assert np.array_equal(idx_gpu[firm], idx[firm])
    assert_valid_sample(a, b, u, idx_gpu)
    dA, dB = oracle.dense_bwd(2, a, b, g, None, idx_gpu)
    assert_equal_bits(ga, dA, "sample grad_a")
    assert_equal_bits(gb_, dB, "sample grad_b")
