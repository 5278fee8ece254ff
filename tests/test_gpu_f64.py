"""Double-precision entry points (the reference dispatches its kernels over double too,
matmul_cuda_kernel.cu:489, banded_cuda_kernel.cu:389) against the float64 oracle."""
import numpy as np
import pytest
import torch

import oracle
from util import assert_close, band_inside

pytestmark = pytest.mark.gpu

SHAPES = [(2, 33, 17, 21), (1, 64, 64, 64), (3, 5, 1, 7), (2, 16, 40, 16)]


@pytest.fixture(scope="module")
def gb():
    import genbmm_b200
    return genbmm_b200


def rand(shape, seed, ties=False):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(*shape, generator=gen, dtype=torch.float64)
    return (x * 4).round() / 4 if ties else x


@pytest.mark.parametrize("shape", SHAPES)
def test_logbmm_f64(gb, shape):
    B, M, K, N = shape
    a, b, g = rand((B, M, K), 1), rand((B, K, N), 2), rand((B, M, N), 3)
    ad, bd = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    c = gb.logbmm(ad, bd)
    assert c.dtype == torch.float64
    ga, gb_ = torch.autograd.grad(c, (ad, bd), g.cuda())
    want, maxes = oracle.dense_fwd(0, a, b, dtype=np.float64)
    dA, dB = oracle.dense_bwd(0, a, b, g, want, maxes, dtype=np.float64)
    assert_close(c, want, 1e-12, 1e-12, "logbmm f64")
    assert_close(ga, dA, 1e-11, 1e-12, "grad_a")
    assert_close(gb_, dB, 1e-11, 1e-12, "grad_b")


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("name,mode", [("maxbmm", 1), ("prodmaxbmm", 3)])
def test_max_semirings_f64_bit_exact(gb, shape, name, mode):
    B, M, K, N = shape
    a, b, g = rand((B, M, K), 4, ties=True), rand((B, K, N), 5, ties=True), rand((B, M, N), 6)
    from genbmm_b200 import _native
    out, idx = _native.forward(a.cuda(), b.cuda(), mode)
    want, widx = oracle.dense_fwd(mode, a, b, dtype=np.float64)
    assert np.array_equal(out.cpu().numpy(), want) and np.array_equal(idx.cpu().numpy(), widx)
    ad, bd = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    c = getattr(gb, name)(ad, bd)
    ga, gb_ = torch.autograd.grad(c, (ad, bd), g.cuda())
    dA, dB = oracle.dense_bwd(mode, a, b, g, None, widx, dtype=np.float64)
    assert np.array_equal(ga.cpu().numpy(), dA) and np.array_equal(gb_.cpu().numpy(), dB)


def test_samplebmm_f64(gb):
    B, M, K, N = 2, 20, 30, 10
    a, b = 2 * rand((B, M, K), 7), 2 * rand((B, K, N), 8)
    u = torch.rand(B, M, N, generator=torch.Generator().manual_seed(9), dtype=torch.float64)
    from genbmm_b200 import _native
    out, idx = _native.forward(a.cuda(), b.cuda(), 2, u.cuda())
    want, widx = oracle.dense_fwd(2, a, b, u, dtype=np.float64)
    assert_close(out, want, 1e-12, 1e-12, "sample value")
    margin = oracle.sample_margin(a, b, u, dtype=np.float64)
    sure = margin > 1e-9  # a uniform this far from every CDF step has one right answer
    assert sure.mean() > 0.99
    assert np.array_equal(idx.cpu().numpy()[sure], widx[sure])


@pytest.mark.parametrize("case", [(2, 9, 2, 1, 1, 2), (1, 40, 5, 4, 0, 3), (2, 70, 20, 15, 18, 17)])
@pytest.mark.parametrize("method,mode", [("multiply", 3), ("multiply_log", 0), ("multiply_max", 1)])
def test_banded_f64(gb, case, method, mode):
    B, n, alu, ald, blu, bld = case
    a = rand((B, n, alu + ald + 1), 10, ties=mode == 1)
    b = rand((B, n, blu + bld + 1), 11, ties=mode == 1)
    g = rand((B, n, alu + ald + blu + bld + 1), 12)
    ad, bd = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    r = getattr(gb.BandedMatrix(ad, alu, ald), method)(gb.BandedMatrix(bd, blu, bld))
    assert r.data.dtype == torch.float64
    ga, gb_ = torch.autograd.grad(r.data, (ad, bd), g.cuda())
    out, idx, _, dA, dB = oracle.band_fwd_bwd(mode, a, alu, ald, b, blu, bld, g, dtype=np.float64)
    if mode == 1:
        assert np.array_equal(r.data.detach().cpu().numpy(), out)
        assert np.array_equal(ga.cpu().numpy(), dA) and np.array_equal(gb_.cpu().numpy(), dB)
    else:
        assert_close(r.data, out, 1e-11, 1e-12, method)
        assert_close(ga, dA, 1e-10, 1e-12, method + " grad_a")
        assert_close(gb_, dB, 1e-10, 1e-12, method + " grad_b")
    inside = band_inside(B, n, alu + bld, ald + blu)
    assert (r.data.detach().cpu().numpy()[~inside] == 0).all()
