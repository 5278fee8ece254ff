"""The factorised (TMA-fed FP32 product) path of logbmm against the oracle, the exact path and
the cases its guard exists for."""
import numpy as np
import pytest
import torch

import oracle
from util import assert_close

pytestmark = pytest.mark.gpu

SHAPES = [(3, 7, 9, 8), (2, 33, 17, 65), (2, 130, 70, 67), (1, 128, 128, 64), (2, 129, 257, 130),
          (1, 256, 512, 384), (2, 5, 1, 3), (1, 1, 1, 1), (1, 300, 40, 5)]


@pytest.fixture(scope="module")
def nat():
    from genbmm_b200 import _native
    return _native


def fast_fwd_bwd(nat, a, b, g, tc=False):
    ad, bd, gd = a.cuda(), b.cuda(), g.cuda()
    out, rowmax, colmax, flags, factors = nat.logbmm_fast_forward(ad, bd, check=True, tensor_cores=tc,
                                                                  keep_factors=True)
    ga, gb = nat.logbmm_fast_backward(ad, bd, gd, out, rowmax, colmax, flags, check=True, tensor_cores=tc)
    if tc:  # reusing the forward's split operands gives the same bits as rebuilding them
        assert factors is not None
        ga2, gb2 = nat.logbmm_fast_backward(ad, bd, gd, out, rowmax, colmax, flags, check=True, tensor_cores=True,
                                            factors=factors)
        assert torch.equal(ga, ga2) and torch.equal(gb, gb2)
    return out, ga, gb, flags


@pytest.mark.parametrize("path", ["fp32", "tcgen05", "tcgen05-unsplit"])
@pytest.mark.parametrize("shape", SHAPES)
def test_fast_path_matches_oracle(nat, shape, path, monkeypatch):
    """The FP32-pipe products and the tensor-core products in both operand forms: a tf32 hi and a lo copy per
    operand (GENBMM_B200_TC_SPLIT=0), and one unsplit copy split in shared memory by the product kernel
    (GENBMM_B200_TC_SPLIT=1; half the workspace, selectable)."""
    tc = path != "fp32"
    if path == "tcgen05-unsplit":
        monkeypatch.setenv("GENBMM_B200_TC_SPLIT", "1")
    B, M, K, N = shape
    gen = torch.Generator().manual_seed(sum(shape))
    a, b = torch.randn(B, M, K, generator=gen), torch.randn(B, K, N, generator=gen)
    g = torch.randn(B, M, N, generator=gen)
    out, ga, gb, flags = fast_fwd_bwd(nat, a, b, g, tc)
    want, maxes = oracle.dense_fwd(0, a, b, dtype=np.float64)
    dA, dB = oracle.dense_bwd(0, a, b, g, want, maxes, dtype=np.float64)
    # the cotangent has both signs: a gradient may be the small difference of large terms, so the same
    # sums over the terms' magnitudes (the oracle on |g|) bound the rounding error (util.assert_close)
    tA, tB = oracle.dense_bwd(0, a, b, g.abs(), want, maxes, dtype=np.float64)
    assert int(flags.sum()) == 0          # well-conditioned inputs never need the guard
    assert_close(out, want, what="fwd")
    assert_close(ga, dA, what="grad_a", term_sum=tA)
    assert_close(gb, dB, what="grad_b", term_sum=tB)
    # and agrees with the exact SFU path
    exact, _ = nat.forward(a.cuda(), b.cuda(), 0)
    assert torch.allclose(out, exact, rtol=1e-5, atol=2e-6)


@pytest.mark.parametrize("tc", [False, True], ids=["fp32", "tcgen05"])
def test_guard_recomputes_underflowing_tiles(nat, tc):
    """Row and column supports that do not meet: row maximum + column maximum overshoots the true
    maximum by hundreds of nats, the factorised sum underflows, the tile is flagged and redone."""
    gen = torch.Generator().manual_seed(1)
    B, M, K, N = 2, 200, 96, 260
    a, b = torch.randn(B, M, K, generator=gen), torch.randn(B, K, N, generator=gen)
    g = torch.rand(B, M, N, generator=gen)
    a[:, :60, :48] -= 400.0      # rows 0..59 live on k >= 48 ...
    b[:, 48:, :70] -= 400.0      # ... columns 0..69 live on k < 48
    out, ga, gb, flags = fast_fwd_bwd(nat, a, b, g, tc)
    nflag = int(flags.sum())
    assert 0 < nflag < flags.numel()      # some tiles take the exact kernels, some the fast ones
    want, maxes = oracle.dense_fwd(0, a, b, dtype=np.float64)
    dA, dB = oracle.dense_bwd(0, a, b, g, want, maxes, dtype=np.float64)
    # results near -400 are stored with the float32 spacing there (3e-5), and so is a + b: the weights
    # exp(a + b - c) of any float32 implementation inherit that as a relative error
    rtol_w = 1e-5 + 2 * float(np.spacing(np.float32(np.abs(want).max())))
    assert 5e-5 < rtol_w < 1e-4
    assert_close(out, want, what="fwd")
    assert_close(ga, dA, rtol_w, what="grad_a")
    assert_close(gb, dB, rtol_w, what="grad_b")
    # the exact path, given the same inputs, agrees to the same tolerance
    ea, eb = nat.backward(a.cuda(), b.cuda(), g.cuda(), out, None, 0)
    assert torch.allclose(ga, ea, rtol=rtol_w, atol=2e-6) and torch.allclose(gb, eb, rtol=rtol_w, atol=2e-6)


def test_guard_with_semiring_zero_fills(nat):
    """-1e9 fills (the usual semiring zero): forward values, flagged or not, match the oracle."""
    gen = torch.Generator().manual_seed(2)
    B, M, K, N = 2, 200, 96, 260
    a, b = torch.randn(B, M, K, generator=gen), torch.randn(B, K, N, generator=gen)
    a[:, 150:, :] = -1e9         # fully masked rows
    a[:, :40, ::2] = -1e9        # half of the reduction masked
    b[:, 1::2, :40] = -1e9       # the other half masked for these columns: nothing survives
    b[:, :, 200:] -= 1e9
    out, _, _, flags = nat.logbmm_fast_forward(a.cuda(), b.cuda(), check=True)
    assert int(flags.sum()) > 0
    want, _ = oracle.dense_fwd(0, a, b)
    assert_close(out, want, what="fwd")


def test_guard_keeps_the_reference_floor(nat):
    """Everything below the reference's -1e9 floor gives -inf, as matmul_cuda_kernel.cu:31-43 does."""
    a = torch.full((1, 130, 64), -3e9)
    b = torch.zeros(1, 64, 140)
    a[0, 5, :] = 0.25
    out, _, _, flags = nat.logbmm_fast_forward(a.cuda(), b.cuda(), check=True)
    want, _ = oracle.dense_fwd(0, a, b)
    assert int(flags.sum()) > 0
    assert torch.isinf(out[0, 0]).all() and np.isinf(want[0, 0]).all()
    assert_close(out[0, 5], want[0, 5])
    # rows of -inf
    a = torch.randn(1, 40, 64)
    a[0, 3] = float("-inf")
    b = torch.randn(1, 64, 50)
    out, _, _, _ = nat.logbmm_fast_forward(a.cuda(), b.cuda(), check=True)
    want, _ = oracle.dense_fwd(0, a, b, dtype=np.float64)
    assert_close(out, want)


def test_autograd_uses_fast_path_for_large_products(monkeypatch):
    import genbmm_b200 as gb
    gen = torch.Generator().manual_seed(3)
    a, b = torch.randn(2, 192, 160, generator=gen), torch.randn(2, 160, 136, generator=gen)
    g = torch.rand(2, 192, 136, generator=gen)
    res = {}
    for mode in ("tensor", "fp32", "exact"):
        monkeypatch.setenv("GENBMM_B200_LOGBMM", mode)
        ad, bd = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
        c = gb.logbmm(ad, bd)
        res[mode] = (c.detach(),) + torch.autograd.grad(c, (ad, bd), g.cuda())
    want, maxes = oracle.dense_fwd(0, a, b, dtype=np.float64)
    dA, dB = oracle.dense_bwd(0, a, b, g, want, maxes, dtype=np.float64)
    for mode in ("tensor", "fp32", "exact"):
        assert_close(res[mode][0], want, what=mode + " fwd")
        assert_close(res[mode][1], dA, what=mode + " grad_a")
        assert_close(res[mode][2], dB, what=mode + " grad_b")


def test_tensor_core_path_at_the_benchmark_shape(nat):
    """1024^3: 3xTF32 on tcgen05 against the float64 oracle on a slice and against the FP32-pipe path."""
    gen = torch.Generator().manual_seed(9)
    a, b = torch.randn(2, 1024, 1024, generator=gen), torch.randn(2, 1024, 1024, generator=gen)
    g = torch.randn(2, 1024, 1024, generator=gen)
    out, ga, gb, flags = fast_fwd_bwd(nat, a, b, g, tc=True)
    ref, ra, rb, _ = fast_fwd_bwd(nat, a, b, g, tc=False)
    assert int(flags.sum()) == 0
    want, maxes = oracle.dense_fwd(0, a[:1, :96], b[:1], dtype=np.float64)
    dA, _ = oracle.dense_bwd(0, a[:1, :96], b[:1], g[:1, :96], want, maxes, dtype=np.float64)
    tA, _ = oracle.dense_bwd(0, a[:1, :96], b[:1], g[:1, :96].abs(), want, maxes, dtype=np.float64)
    assert_close(out[:1, :96], want, what="fwd")
    assert_close(ga[:1, :96], dA, what="grad_a", term_sum=tA)
    assert torch.allclose(out, ref, rtol=1e-5, atol=2e-6)
    # mixed-sign cotangents: each gradient is a sum of 1024 terms of both signs, so the two paths are
    # compared against the sum of the terms' magnitudes (the same gradients for |g|), each path being
    # within 1e-6 of it from the exact result; tests/test_gpu_parity_full.py holds the oracle comparison
    # of grad_b at this shape
    _, ta, tb, _ = fast_fwd_bwd(nat, a, b, g.abs(), tc=False)
    ea, eb = ((ga - ra).abs() / ta).max().item(), ((gb - rb).abs() / tb).max().item()
    print("max |tc - fp32| / sum|terms|: grad_a %.3e grad_b %.3e" % (ea, eb))
    assert ea <= 2e-6 and eb <= 2e-6


def test_host_pipeline_matches_the_plain_call():
    """Chunked H2D / kernels / D2H overlap gives the same loss and gradients as one plain call."""
    import genbmm_b200 as gb
    from genbmm_b200.host import HostPipeline
    gen = torch.Generator().manual_seed(4)
    B, M, K, N = 6, 192, 160, 136
    a_h = torch.randn(B, M, K, generator=gen).pin_memory()
    b_h = torch.randn(B, K, N, generator=gen).pin_memory()
    ga_h, gb_h = torch.empty(B, M, K).pin_memory(), torch.empty(B, K, N).pin_memory()
    pipe = HostPipeline(B, M, K, N, chunks=4, graph=True)
    # buffers are reused across steps: the first step is issued directly, the second captures one CUDA graph
    # per chunk, the third replays them on new contents of the host tensors
    first = pipe.step(a_h, b_h, ga_h, gb_h)
    ga_first = ga_h.clone()
    assert pipe.step(a_h, b_h, ga_h, gb_h) == first and torch.equal(ga_h, ga_first)
    a_h.copy_(torch.randn(B, M, K, generator=gen))
    ga_h.zero_(); gb_h.zero_()
    loss = pipe.step(a_h, b_h, ga_h, gb_h)
    assert pipe._graphs is not None and len(pipe._graphs) == 4
    torch.cuda.synchronize()
    plain = HostPipeline(B, M, K, N, chunks=4)
    ga_p, gb_p = torch.empty(B, M, K).pin_memory(), torch.empty(B, K, N).pin_memory()
    for _ in range(2):
        assert plain.step(a_h, b_h, ga_p, gb_p) == loss
    assert plain._graphs is None and torch.equal(ga_p, ga_h) and torch.equal(gb_p, gb_h)
    ad, bd = a_h.cuda().requires_grad_(True), b_h.cuda().requires_grad_(True)
    c = gb.logbmm(ad, bd)
    want_a, want_b = torch.autograd.grad(c.sum(), (ad, bd))
    assert abs(loss - float(c.detach().sum().double())) <= 1e-5 * abs(loss)
    assert torch.allclose(ga_h.cuda(), want_a, rtol=1e-5, atol=2e-6)
    assert torch.allclose(gb_h.cuda(), want_b, rtol=1e-5, atol=2e-6)
    # chunks of unequal sizes (small at both ends) give the same gradients
    tapered = HostPipeline(B, M, K, N, chunks="tapered")
    assert len(tapered.bounds) == B
    ga_t, gb_t = torch.empty(B, M, K).pin_memory(), torch.empty(B, K, N).pin_memory()
    loss_t = tapered.step(a_h, b_h, ga_t, gb_t)
    assert abs(loss_t - loss) <= 1e-9 * abs(loss)
    assert torch.equal(ga_t, ga_p) and torch.equal(gb_t, gb_p)


_FIXUP_CHILD = r"""
import sys, numpy as np, torch
sys.path.insert(0, sys.argv[1])
from genbmm_b200 import _native as nat
gen = torch.Generator().manual_seed(1)
B, M, K, N = 40, 200, 96, 260
a, b = torch.randn(B, M, K, generator=gen), torch.randn(B, K, N, generator=gen)
g = torch.rand(B, M, N, generator=gen)
a[:, :60, :48] -= 400.0
b[:, 48:, :70] -= 400.0
a[::3] = torch.randn(a[::3].shape, generator=gen)     # every third element has no flagged tile
ad, bd, gd = a.cuda(), b.cuda(), g.cuda()
out, rowmax, colmax, flags = nat.logbmm_fast_forward(ad, bd, check=True, tensor_cores=True)
ga, gb = nat.logbmm_fast_backward(ad, bd, gd, out, rowmax, colmax, flags, check=True, tensor_cores=True)
np.savez(sys.argv[2], out=out.cpu().numpy(), ga=ga.cpu().numpy(), gb=gb.cpu().numpy(), nflag=int(flags.sum()))
"""


def test_fixup_work_list_over_several_rounds(tmp_path):
    """The exact fix-up kernels on one CTA (400 tiles: two rounds of its 256-entry work list) and on the
    default grid give the same bits: a tile's result does not depend on who gathers it."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = []
    for cap in ("1", None):
        env = dict(os.environ)
        env.pop("GENBMM_B200_FIXUP_CTAS", None)
        if cap:
            env["GENBMM_B200_FIXUP_CTAS"] = cap
        path = str(tmp_path / ("fix_%s.npz" % cap))
        subprocess.run([sys.executable, "-c", _FIXUP_CHILD, root, path], env=env, check=True, timeout=300)
        res.append(np.load(path))
    one, many = res
    assert int(one["nflag"]) == int(many["nflag"]) > 0
    for k in ("out", "ga", "gb"):
        assert np.array_equal(one[k], many[k]), k
    assert np.isfinite(one["out"]).all()
