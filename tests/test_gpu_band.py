"""Parity of the banded CUDA kernels (through the C ABI) with the CPU oracle and the golden fixtures."""
import numpy as np
import pytest
import torch

import oracle
from util import assert_close, assert_equal_bits, band_inside, cfg5

pytestmark = pytest.mark.gpu

# (B, n, a_lu, a_ld, b_lu, b_ld)
CASES = [(2, 5, 2, 1, 1, 2), (3, 8, 0, 3, 2, 0), (2, 6, 3, 3, 3, 3), (1, 4, 5, 4, 0, 0), (2, 9, 1, 1, 2, 2),
         (1, 1, 0, 0, 0, 0), (2, 70, 4, 7, 9, 2), (2, 300, 20, 13, 5, 31), (1, 40, 64, 64, 64, 64),
         (3, 33, 0, 0, 3, 1),
         # bands >= 32 wide and n >= 128: the tensor-core path (sum, log), with odd sizes and offsets
         (2, 300, 20, 15, 18, 17), (1, 128, 40, 3, 5, 40), (2, 517, 64, 64, 64, 64), (1, 257, 0, 40, 35, 0),
         (1, 1000, 31, 1, 0, 33), (2, 130, 100, 90, 70, 120), (3, 700, 33, 30, 31, 40), (2, 1029, 64, 64, 64, 64),
         (1, 400, 50, 0, 0, 50)]
MODES = [("multiply", 3), ("multiply_log", 0), ("multiply_max", 1)]


@pytest.fixture(scope="module")
def gb():
    import genbmm_b200
    return genbmm_b200


def run(gb, method, a, alu, ald, b, blu, bld, g):
    ad, bd = a.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    r = getattr(gb.BandedMatrix(ad, alu, ald), method)(gb.BandedMatrix(bd, blu, bld))
    ga, gb_ = torch.autograd.grad(r.data, (ad, bd), g.cuda())
    r.data = r.data.detach()
    return r, ga, gb_


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("method,mode", MODES)
def test_band_products_match_oracle(gb, case, method, mode):
    B, n, alu, ald, blu, bld = case
    gen = torch.Generator().manual_seed(sum(case) + mode)
    a = torch.randn(B, n, alu + ald + 1, generator=gen)
    b = torch.randn(B, n, blu + bld + 1, generator=gen)
    g = torch.rand(B, n, alu + ald + blu + bld + 1, generator=gen)
    if mode == 1:  # ties on purpose
        a, b = (a * 4).round() / 4, (b * 4).round() / 4
    r, ga, gb_ = run(gb, method, a, alu, ald, b, blu, bld, g)
    assert (r.lu, r.ld) == (alu + bld, ald + blu)
    if mode == 1:
        out, idx, _, dA, dB = oracle.band_fwd_bwd(mode, a, alu, ald, b, blu, bld, g)
        assert_equal_bits(r.data, out, "max value")
        from genbmm_b200 import _native
        _, idx_gpu, _ = _native.forward_band(a.cuda(), alu, ald, b.cuda(), blu, bld, 1)
        assert_equal_bits(idx_gpu, idx, "max index")
        assert_equal_bits(ga, dA, "max grad_a")
        assert_equal_bits(gb_, dB, "max grad_b")
    else:
        out, _, _, dA, dB = oracle.band_fwd_bwd(mode, a, alu, ald, b, blu, bld, g, dtype=np.float64)
        bound = (None, None, None)
        if mode == 3:  # signed terms: the same sums over absolute values bound the rounding error
            t_out, _, _, t_dA, t_dB = oracle.band_fwd_bwd(mode, a.abs(), alu, ald, b.abs(), blu, bld, g.abs(),
                                                          dtype=np.float64)
            bound = (t_out, t_dA, t_dB)
        assert_close(r.data, out, what=method, term_sum=bound[0])
        assert_close(ga, dA, what=method + " grad_a", term_sum=bound[1])
        assert_close(gb_, dB, what=method + " grad_b", term_sum=bound[2])
    inside = band_inside(B, n, alu + bld, ald + blu)
    assert (r.data.cpu().numpy()[~inside] == 0).all()


@pytest.mark.parametrize("case", [c for c in CASES if c[1] >= 128 and min(c[2] + c[3], c[4] + c[5]) >= 31])
@pytest.mark.parametrize("path", ["auto", "hilo", "convert", "block"])
def test_sum_semiring_both_paths(gb, case, monkeypatch, path):
    """The ordinary product and its gradients as 3xTF32 on the tensor cores and on the FP32 block kernels
    (GENBMM_B200_BAND=block), with signed cotangents.  The tensor-core path has three feeds: one zero-padded
    skewed fp32 copy per operand, fetched by TMA and split into tf32 hi + lo in shared memory (default when
    every tile fits one accumulation chunk); a hi and a lo copy (GENBMM_B200_BAND_SPLIT=0, and always for
    wider bands); operand tiles converted from the band tensors themselves by SIMT warps
    (GENBMM_B200_BAND_CV=1).  Bound: 1e-6 of the sum of the terms' magnitudes."""
    monkeypatch.setenv("GENBMM_B200_BAND", "block" if path == "block" else "auto")
    if path == "convert":
        monkeypatch.setenv("GENBMM_B200_BAND_CV", "1")
    if path == "hilo":
        monkeypatch.setenv("GENBMM_B200_BAND_SPLIT", "0")
    B, n, alu, ald, blu, bld = case
    gen = torch.Generator().manual_seed(sum(case))
    a = torch.randn(B, n, alu + ald + 1, generator=gen)
    b = torch.randn(B, n, blu + bld + 1, generator=gen)
    g = torch.randn(B, n, alu + ald + blu + bld + 1, generator=gen)
    r, ga, gb_ = run(gb, "multiply", a, alu, ald, b, blu, bld, g)
    out, _, _, dA, dB = oracle.band_fwd_bwd(3, a, alu, ald, b, blu, bld, g, dtype=np.float64)
    t_out, _, _, t_dA, t_dB = oracle.band_fwd_bwd(3, a.abs(), alu, ald, b.abs(), blu, bld, g.abs(), dtype=np.float64)
    assert_close(r.data, out, what="multiply", term_sum=t_out)
    assert_close(ga, dA, what="grad_a", term_sum=t_dA)
    assert_close(gb_, dB, what="grad_b", term_sum=t_dB)
    inside = band_inside(B, n, alu + bld, ald + blu)
    assert (r.data.cpu().numpy()[~inside] == 0).all()


@pytest.mark.parametrize("case", [c for c in CASES if c[1] >= 128 and min(c[2] + c[3], c[4] + c[5]) >= 31])
@pytest.mark.parametrize("feed", ["hilo", "convert", "scale-fused"])
def test_log_semiring_other_tensor_feeds(gb, case, monkeypatch, feed):
    """The log product on the tensor-core feeds that are not the default (hi + lo copies,
    GENBMM_B200_BAND_SPLIT=0; SIMT-converted tiles, GENBMM_B200_BAND_CV=1) and, on the default feed, with the
    gradients' factor exp(x - max) applied by the product's epilogue instead of a separate pass
    (GENBMM_B200_BAND_SCALE=fused); the default is what test_band_products_match_oracle runs for these shapes."""
    if feed == "scale-fused":
        monkeypatch.setenv("GENBMM_B200_BAND_SCALE", "fused")
    else:
        monkeypatch.setenv("GENBMM_B200_BAND_CV" if feed == "convert" else "GENBMM_B200_BAND_SPLIT",
                           "1" if feed == "convert" else "0")
    B, n, alu, ald, blu, bld = case
    gen = torch.Generator().manual_seed(sum(case))
    a = torch.randn(B, n, alu + ald + 1, generator=gen)
    b = torch.randn(B, n, blu + bld + 1, generator=gen)
    g = torch.rand(B, n, alu + ald + blu + bld + 1, generator=gen)
    r, ga, gb_ = run(gb, "multiply_log", a, alu, ald, b, blu, bld, g)
    out, _, _, dA, dB = oracle.band_fwd_bwd(0, a, alu, ald, b, blu, bld, g, dtype=np.float64)
    assert_close(r.data, out, what="multiply_log")
    assert_close(ga, dA, what="grad_a")
    assert_close(gb_, dB, what="grad_b")


@pytest.mark.parametrize("case", [c for c in CASES if c[1] >= 128 and min(c[2] + c[3], c[4] + c[5]) >= 31]
                         + [(2, 640, 64, 64, 64, 64), (1, 333, 100, 20, 10, 90), (2, 256, 31, 0, 0, 31),
                            (1, 700, 150, 100, 120, 140)])
@pytest.mark.parametrize("blocks", ["warp-ranges", "warp-ranges-64", "lockstep"])
def test_max_semiring_both_block_kernels(gb, case, monkeypatch, blocks):
    """multiply_max on the kernels that read skewed copies: blocks whose warps walk their own reduction ranges
    (64 x 32, the default, and 64 x 64 with GENBMM_B200_BAND_MAX_COLS=64) and 128 x 64 blocks in lockstep
    (GENBMM_B200_BAND_MAX=block).  Values and indices bit for bit, with ties and with rows that nothing lifts
    above -1e9."""
    if blocks == "lockstep":
        monkeypatch.setenv("GENBMM_B200_BAND_MAX", "block")
    if blocks == "warp-ranges-64":
        monkeypatch.setenv("GENBMM_B200_BAND_MAX_COLS", "64")
    B, n, alu, ald, blu, bld = case
    gen = torch.Generator().manual_seed(sum(case) + 5)
    a = (torch.randn(B, n, alu + ald + 1, generator=gen) * 2).round() / 2
    b = (torch.randn(B, n, blu + bld + 1, generator=gen) * 2).round() / 2
    a[:, n // 3] = -2e9          # a row whose terms all stay below the reference's floor
    b[:, n // 2, ::2] = float("-inf")
    from genbmm_b200 import _native
    out_gpu, idx_gpu, _ = _native.forward_band(a.cuda(), alu, ald, b.cuda(), blu, bld, 1)
    g = torch.rand(B, n, alu + ald + blu + bld + 1, generator=gen)
    out, idx, _, _, _ = oracle.band_fwd_bwd(1, a, alu, ald, b, blu, bld, g)
    assert_equal_bits(out_gpu, out, "max value")
    assert_equal_bits(idx_gpu, idx, "max index")


@pytest.mark.parametrize("case", [(2, 300, 20, 15, 18, 17), (2, 517, 64, 64, 64, 64), (1, 257, 0, 40, 35, 0),
                                  (3, 33, 0, 0, 3, 1), (2, 130, 100, 90, 70, 120), (1, 1001, 33, 30, 31, 40)])
@pytest.mark.parametrize("route", ["thread-per-row", "warp-per-row"])
def test_max_backward_both_routings(gb, case, monkeypatch, route):
    """The index-routed gradients of multiply_max with grad_b by the thread-per-row kernel (default) and by the
    warp-per-row kernel (GENBMM_B200_BAND_ROUTE_B=w): bit for bit the oracle's sums, on indices with ties, -1
    entries and odd row lengths."""
    if route == "warp-per-row":
        monkeypatch.setenv("GENBMM_B200_BAND_ROUTE_B", "w")
    B, n, alu, ald, blu, bld = case
    gen = torch.Generator().manual_seed(sum(case) + 11)
    a = (torch.randn(B, n, alu + ald + 1, generator=gen) * 2).round() / 2
    b = (torch.randn(B, n, blu + bld + 1, generator=gen) * 2).round() / 2
    a[:, n // 3] = -2e9
    g = torch.randn(B, n, alu + ald + blu + bld + 1, generator=gen)
    r, ga, gb_ = run(gb, "multiply_max", a, alu, ald, b, blu, bld, g)
    out, idx, _, dA, dB = oracle.band_fwd_bwd(1, a, alu, ald, b, blu, bld, g)
    assert_equal_bits(r.data, out, "max value")
    assert_equal_bits(ga, dA, "max grad_a")
    assert_equal_bits(gb_, dB, "max grad_b")


@pytest.mark.parametrize("ci", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("method,name", [("multiply", "mul"), ("multiply_log", "log"), ("multiply_max", "max")])
def test_band_products_match_reference_fixture(gb, golden, ci, method, name):
    B, n, alu, ald, blu, bld = (int(v) for v in golden["band%d_dims" % ci])
    f = lambda k: torch.from_numpy(golden["band%d_%s" % (ci, k)]).float()
    r, ga, gb_ = run(gb, method, f("a"), alu, ald, f("b"), blu, bld, f("g"))
    inside = band_inside(B, n, alu + bld, ald + blu)
    assert_close(r.data.cpu().numpy()[inside], golden["band%d_%s_out" % (ci, name)][inside], what=name)
    assert_close(ga, golden["band%d_%s_ga" % (ci, name)] * band_inside(B, n, alu, ald), what=name + " grad_a")
    assert_close(gb_, golden["band%d_%s_gb" % (ci, name)] * band_inside(B, n, blu, bld), what=name + " grad_b")


def test_reference_test_property(gb):
    """genbmm/test_cuda.py:81-109: b.multiply_log(a.transpose()) against the CPU loops."""
    gen = torch.Generator().manual_seed(0)
    B, n, lu, ld = 4, 5, 3, 4
    band = gb.banddiag(torch.rand(B, n, n, generator=gen), lu, ld)[0]
    band2 = gb.banddiag(torch.rand(B, n, n, generator=gen), lu, ld)[0]
    x, y = gb.BandedMatrix(band.cuda(), lu, ld), gb.BandedMatrix(band2.cuda(), lu, ld)
    got = y.multiply_log(x.transpose())
    xt = oracle.band_transpose(band, lu, ld)
    want, _, _ = oracle.band_fwd(0, band2, lu, ld, xt, ld, lu, dtype=np.float64)
    assert_close(got.data, want)


def test_config5_full_size(gb):
    """n=8192, 129 diagonals: the oracle on a batch slice, then properties at full size."""
    from genbmm_b200 import _native
    a, b = cfg5()
    lu = ld = 64
    ad, bd = a.cuda(), b.cuda()
    gen = torch.Generator().manual_seed(44)
    g = torch.rand(32, 8192, 257, generator=gen)
    gd = g.cuda()
    for mode in (3, 0, 1):
        out, idx, _ = _native.forward_band(ad, lu, ld, bd, lu, ld, mode)
        part = out if mode == 0 else idx
        ga, gb_ = _native.backward_band(ad, lu, ld, bd, lu, ld, gd, part, mode, both=True)
        dt = np.float32 if mode == 1 else np.float64
        wout, widx, _, dA, dB = oracle.band_fwd_bwd(mode, a[:1], lu, ld, b[:1], lu, ld, g[:1], dtype=dt)
        if mode == 1:
            assert_equal_bits(out[:1], wout)
            assert_equal_bits(idx[:1], widx)
            assert_equal_bits(ga[:1], dA)
            assert_equal_bits(gb_[:1], dB)
        else:
            bound = (None, None, None)
            if mode == 3:  # signed terms: see assert_close
                t_out, _, _, t_dA, t_dB = oracle.band_fwd_bwd(3, a[:1].abs(), lu, ld, b[:1].abs(), lu, ld, g[:1].abs(),
                                                              dtype=np.float64)
                bound = (t_out, t_dA, t_dB)
            assert_close(out[:1], wout, term_sum=bound[0])
            assert_close(ga[:1], dA, term_sum=bound[1])
            assert_close(gb_[:1], dB, term_sum=bound[2])
    # linearity of the ordinary product at full size
    out1 = _native.forward_band(ad, lu, ld, bd, lu, ld, 3)[0]
    out2 = _native.forward_band(2 * ad, lu, ld, bd, lu, ld, 3)[0]
    assert torch.allclose(out2, 2 * out1, rtol=1e-6, atol=1e-6)
    # max-plus: doubling both operands (exact in binary floating point) doubles every in-matrix
    # result and leaves the argmax where it was
    o1, i1, _ = _native.forward_band(ad, lu, ld, bd, lu, ld, 1)
    o2, i2, _ = _native.forward_band(2 * ad, lu, ld, 2 * bd, lu, ld, 1)
    inside = torch.from_numpy(band_inside(32, 8192, 128, 128).copy()).cuda()
    assert torch.equal(i1, i2)
    assert torch.equal(o2[inside], 2 * o1[inside])
    # log bounds max
    ol = _native.forward_band(ad, lu, ld, bd, lu, ld, 0)[0]
    assert (ol[inside] >= o1[inside] - 1e-4).all() and (ol[inside] <= o1[inside] + np.log(129.0) + 1e-4).all()


def test_wide_band_falls_back_to_global_reads(gb):
    """Bands too wide for shared-memory staging take the unstaged path."""
    B, n, lu, ld = 1, 600, 150, 149
    gen = torch.Generator().manual_seed(3)
    a, b = torch.randn(B, n, 300, generator=gen), torch.randn(B, n, 300, generator=gen)
    g = torch.rand(B, n, 599, generator=gen)
    for method, mode in MODES:
        r, ga, gb_ = run(gb, method, a, lu, ld, b, lu, ld, g)
        out, idx, _, dA, dB = oracle.band_fwd_bwd(mode, a, lu, ld, b, lu, ld, g, dtype=np.float64)
        bound = (None, None, None)
        if mode == 3:
            t_out, _, _, t_dA, t_dB = oracle.band_fwd_bwd(3, a.abs(), lu, ld, b.abs(), lu, ld, g.abs(), dtype=np.float64)
            bound = (t_out, t_dA, t_dB)
        assert_close(r.data, out, what=method, term_sum=bound[0])
        assert_close(ga, dA, what=method + " grad_a", term_sum=bound[1])
        assert_close(gb_, dB, what=method + " grad_b", term_sum=bound[2])


def test_band_rejects_bad_inputs(gb):
    a = torch.rand(2, 5, 3)
    with pytest.raises(RuntimeError, match="a must be a CUDA tensor"):
        gb.BandedMatrix(a, 1, 1).multiply(gb.BandedMatrix(a.cuda(), 1, 1))
    with pytest.raises(AssertionError):
        gb.BandedMatrix(a.cuda(), 2, 2)


@pytest.mark.parametrize("lu,ld", [(9, 8), (20, 20)], ids=["block", "tensor"])
def test_band_log_guard_recomputes_flagged_row_blocks(gb, monkeypatch, lu, ld):
    """Operand rows whose supports miss each other make the factorised sum underflow: the row
    block is flagged and goes through the exact kernels, forward and backward (17-wide bands: the
    FP32 block kernels; 41-wide: the tensor-core kernels)."""
    from genbmm_b200 import _native
    B, n = 2, 200
    gen = torch.Generator().manual_seed(5)
    a, b = torch.randn(B, n, lu + ld + 1, generator=gen), torch.randn(B, n, lu + ld + 1, generator=gen)
    g = torch.rand(B, n, 2 * (lu + ld) + 1, generator=gen)
    a[:, 70:90, :lu] -= 300.0       # rows 70..89 of a live on the upper half of the band ...
    b[:, 40:120, lu:] -= 300.0      # ... the b rows they meet live on the lower half
    out, ga, gb_ = run(gb, "multiply_log", a, lu, ld, b, lu, ld, g)
    want, _, _, dA, dB = oracle.band_fwd_bwd(0, a, lu, ld, b, lu, ld, g, dtype=np.float64)
    # results near -600 are stored with the float32 spacing there (6e-5), and so is a + b: the weights
    # exp(a + b - out) of any float32 implementation inherit that as a relative error
    rtol_w = 1e-5 + 2 * float(np.spacing(np.float32(np.abs(want).max())))
    assert 5e-5 < rtol_w < 2e-4
    assert_close(out.data, want, what="fwd")
    assert_close(ga, dA, rtol_w, what="grad_a")
    assert_close(gb_, dB, rtol_w, what="grad_b")
    # and the exact kernels alone agree
    monkeypatch.setenv("GENBMM_B200_BANDLOG", "exact")
    out2, ga2, gb2 = run(gb, "multiply_log", a, lu, ld, b, lu, ld, g)
    assert torch.allclose(out.data, out2.data, rtol=1e-5, atol=2e-6)
    assert torch.allclose(ga, ga2, rtol=rtol_w, atol=2e-6) and torch.allclose(gb_, gb2, rtol=rtol_w, atol=2e-6)


@pytest.mark.parametrize("ci", [0, 1, 2, 3, 4])
def test_band_log_second_order_matches_reference_fixture(gb, golden, ci):
    """genbmm/test_cuda.py:113-143: gradient of (grad_a, grad_b) w.r.t. (a, b, cotangent); the fixture is
    float64 autograd through the reference's multiply_log_simple; the reference's own test accepts 1e-2."""
    B, n, alu, ald, blu, bld = (int(v) for v in golden["band%d_dims" % ci])
    f = lambda k: torch.from_numpy(golden["band%d_%s" % (ci, k)]).float().cuda()
    a, b, g = f("a").requires_grad_(True), f("b").requires_grad_(True), f("g").requires_grad_(True)
    r = gb.BandedMatrix(a, alu, ald).multiply_log(gb.BandedMatrix(b, blu, bld))
    ga, gb_ = torch.autograd.grad(r.data, (a, b), g, create_graph=True)
    hh = torch.autograd.grad((ga, gb_), (a, b, g), (f("log_h_a"), f("log_h_b")))
    ins = lambda lu, ld: band_inside(B, n, lu, ld)
    assert_close(hh[0], golden["band%d_log_hh_a" % ci] * ins(alu, ald), 1e-4, 1e-5, "d/da")
    assert_close(hh[1], golden["band%d_log_hh_b" % ci] * ins(blu, bld), 1e-4, 1e-5, "d/db")
    assert_close(hh[2], golden["band%d_log_hh_g" % ci] * ins(alu + bld, ald + blu), 1e-4, 1e-5, "d/dg")


@pytest.mark.parametrize("B,n,alu,ald,blu,bld", [(2, 70, 3, 2, 1, 4), (1, 33, 0, 0, 2, 2), (3, 129, 17, 9, 12, 20)])
def test_backbackward_band_entry_matches_oracle(B, n, alu, ald, blu, bld):
    """The reference's call shape `backbackward_band(a, .., grad_out, part, maxes, grad_out_a, 0)`:
    cotangent of grad_a only (banded_cuda_kernel.cu:453-546)."""
    from genbmm_b200 import _native
    rng = np.random.default_rng(n)
    mk = lambda w: rng.standard_normal((B, n, w)).astype(np.float32)
    a, b = mk(alu + ald + 1), mk(blu + bld + 1)
    wo = alu + bld + ald + blu + 1
    g, h = mk(wo), mk(alu + ald + 1)
    out, _, _ = oracle.band_fwd(0, a, alu, ald, b, blu, bld)
    want = oracle.band_bwdbwd(a, alu, ald, b, blu, bld, g, out, h)
    t = lambda x: torch.from_numpy(x).cuda()
    got = _native.backbackward_band(t(a), alu, ald, t(b), blu, bld, t(g), t(out), None, t(h), 0)
    for w, r, name in zip(want, got, ("grad_a", "grad_b", "grad_grad")):
        assert_close(r, w, 2e-4, 2e-5, name)
