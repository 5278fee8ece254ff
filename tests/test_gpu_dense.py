"""Parity of the dense CUDA kernels (through the C ABI) with the CPU oracle and the golden fixtures."""
import numpy as np
import pytest
import torch

import oracle
from util import assert_close, assert_equal_bits, assert_valid_sample, cfg1, cfg2, cfg3

pytestmark = pytest.mark.gpu

SHAPES = [(1, 1, 1, 1), (2, 5, 1, 3), (3, 7, 9, 8), (2, 33, 17, 65), (2, 130, 70, 67), (1, 128, 128, 64),
          (2, 129, 257, 130), (4, 64, 64, 64), (3, 6, 10, 7), (1, 200, 33, 4)]


@pytest.fixture(scope="module")
def gb():
    import genbmm_b200
    return genbmm_b200


def dev(x):
    return x.cuda().contiguous()


def run_fwd_bwd(fn, a, b, g, *extra):
    ad, bd = dev(a).requires_grad_(True), dev(b).requires_grad_(True)
    c = fn(ad, bd, *extra)
    ga, gb_ = torch.autograd.grad(c, (ad, bd), dev(g))
    return c.detach(), ga, gb_


def tied(shape, gen):
    return (torch.randn(*shape, generator=gen) * 8).round() / 8


@pytest.mark.parametrize("tiles", ["auto", "large", "small"])
@pytest.mark.parametrize("shape", SHAPES + [(40, 64, 64, 64), (3, 100, 150, 40)])
def test_logbmm_matches_oracle(gb, shape, tiles, monkeypatch):
    """The exact log kernels: 128x64 tiles (GENBMM_B200_SMALL=0), 32x32 tiles with both gradients in one launch
    (=1), and the rule that picks between them by how many CTAs the large tiles would give."""
    if tiles != "auto":   # "auto" is the operator as a user gets it (factorised tensor-core path when large)
        monkeypatch.setenv("GENBMM_B200_LOGBMM", "exact")
        monkeypatch.setenv("GENBMM_B200_SMALL", "0" if tiles == "large" else "1")
    B, M, K, N = shape
    gen = torch.Generator().manual_seed(sum(shape))
    a, b, g = torch.randn(B, M, K, generator=gen), torch.randn(B, K, N, generator=gen), torch.rand(B, M, N, generator=gen)
    c, ga, gb_ = run_fwd_bwd(gb.logbmm, a, b, g)
    out, maxes = oracle.dense_fwd(0, a, b, dtype=np.float64)
    dA, dB = oracle.dense_bwd(0, a, b, g, out, maxes, dtype=np.float64)
    assert_close(c, out, what="logbmm fwd")
    assert_close(ga, dA, what="logbmm grad_a")
    assert_close(gb_, dB, what="logbmm grad_b")


@pytest.mark.parametrize("ci", [0, 1, 2, 3])
def test_logbmm_matches_reference_fixture(gb, golden, ci):
    f = lambda k: golden["dense%d_log_%s" % (ci, k)]
    c, ga, gb_ = run_fwd_bwd(gb.logbmm, torch.from_numpy(f("a")).float(), torch.from_numpy(f("b")).float(),
                             torch.from_numpy(f("back")).float())
    assert_close(c, f("c"), what="fwd")
    assert_close(ga, f("ga"), what="grad_a")
    assert_close(gb_, f("gb"), what="grad_b")


# reductions longer than 128 steps: the register-staged kernel, or with GENBMM_B200_MAX_TMA=1 and K a multiple of 4
# the TMA-staged one (ragged tiles, a partial last stage, a stage count that is not a multiple of the ring)
MAX_SHAPES = SHAPES + [(2, 130, 260, 70), (1, 300, 516, 200), (3, 64, 132, 64), (1, 129, 1028, 65),
                       (2, 70, 416, 33), (2, 70, 288, 33), (3, 65, 20, 31), (1, 200, 128, 100), (1, 70, 2052, 90)]


@pytest.mark.parametrize("staging", ["auto", "tma", "warp-routing", "lockstep-short"])
@pytest.mark.parametrize("shape", MAX_SHAPES)
@pytest.mark.parametrize("name,mode", [("maxbmm", 1), ("prodmaxbmm", 3)])
def test_max_semirings_bit_exact(gb, shape, name, mode, staging, monkeypatch):
    if staging == "tma":
        monkeypatch.setenv("GENBMM_B200_MAX_TMA", "1")
    if staging == "warp-routing":   # grad_b of short reductions by the warp-per-column kernel too
        monkeypatch.setenv("GENBMM_B200_ROUTE_B", "w")
    if staging == "lockstep-short":  # reductions of up to 288 steps on the 128 x 64 lockstep kernels as well
        monkeypatch.setenv("GENBMM_B200_MAX_SHORT", "block")
    B, M, K, N = shape
    gen = torch.Generator().manual_seed(7 + sum(shape))
    a, b, g = tied((B, M, K), gen), tied((B, K, N), gen), torch.rand(B, M, N, generator=gen)
    fn = getattr(gb, name)
    c, ga, gb_ = run_fwd_bwd(fn, a, b, g)
    out, idx = oracle.dense_fwd(mode, a, b)
    dA, dB = oracle.dense_bwd(mode, a, b, g, None, idx)
    assert_equal_bits(c, out, name + " value")
    from genbmm_b200 import _native
    _, idx_gpu = _native.forward(dev(a), dev(b), mode)
    assert_equal_bits(idx_gpu, idx, name + " index")
    assert_equal_bits(ga, dA, name + " grad_a")
    assert_equal_bits(gb_, dB, name + " grad_b")


@pytest.mark.parametrize("ci", [0, 1, 2, 3])
@pytest.mark.parametrize("name,op,mode", [("maxbmm", "max", 1), ("prodmaxbmm", "prodmax", 3)])
def test_max_semirings_match_reference_fixture(gb, golden, ci, name, op, mode):
    f = lambda k: golden["dense%d_%s_%s" % (ci, op, k)]
    from genbmm_b200 import _native
    a, b = torch.from_numpy(f("a")), torch.from_numpy(f("b"))
    c, ga, gb_ = run_fwd_bwd(getattr(gb, name), a, b, torch.from_numpy(f("back")))
    assert_equal_bits(c, f("c"), "value")
    _, idx = _native.forward(dev(a), dev(b), mode)
    assert_equal_bits(idx, f("idx_low"), "lowest-k index")
    assert_close(ga, f("ga"), 1e-6, 1e-6, "grad_a")
    assert_close(gb_, f("gb"), 1e-6, 1e-6, "grad_b")


def test_max_edge_semantics(gb):
    """-1e9 floor, -1 index, NaN and signed zeros (matmul_cuda_kernel.cu:60-73)."""
    from genbmm_b200 import _native
    a = torch.tensor([[[-2e9, -3e9, -1e10], [-0.0, 0.0, -0.0], [float("nan"), 1.0, 1.0], [0.0, -0.0, 0.0]]])
    b = torch.zeros(1, 3, 2)
    b[0, :, 1] = -0.0
    for mode in (1, 3):
        out, idx = _native.forward(dev(a), dev(b), mode)
        want, widx = oracle.dense_fwd(mode, a, b)
        assert_equal_bits(out, want, "mode %d value" % mode)
        assert_equal_bits(idx, widx, "mode %d index" % mode)
    # a long reduction whose maximum sits in a late tile and is tied with a later one
    a = torch.full((1, 3, 100), -5.0)
    a[0, 0, 37] = a[0, 0, 90] = 2.0
    a[0, 1, 99] = 1.0
    b = torch.zeros(1, 100, 5)
    out, idx = _native.forward(dev(a), dev(b), 1)
    want, widx = oracle.dense_fwd(1, a, b)
    assert_equal_bits(out, want)
    assert_equal_bits(idx, widx)
    assert int(idx[0, 0, 0]) == 37 and int(idx[0, 1, 0]) == 99 and int(idx[0, 2, 0]) == 0


def test_log_edge_semantics(gb):
    """-1e9 fills, -inf rows and the -1e9 floor of the running maximum (matmul_cuda_kernel.cu:31)."""
    gen = torch.Generator().manual_seed(3)
    a = torch.randn(2, 9, 40, generator=gen)
    b = torch.randn(2, 40, 11, generator=gen)
    a[:, 0, :] = -1e9
    a[:, 1, :] = float("-inf")
    a[:, 2, ::2] = -1e9
    b[:, 5:30, 3] = float("-inf")
    c = gb.logbmm(dev(a), dev(b))
    want, _ = oracle.dense_fwd(0, a, b, dtype=np.float64)
    assert_close(c, want.astype(np.float32), what="masked logbmm")
    assert torch.isinf(c[:, 1, :]).all() and (c[:, 1, :] < 0).all()


@pytest.mark.parametrize("shape", [(2, 5, 1, 3), (3, 7, 9, 8), (2, 33, 17, 65), (2, 130, 70, 67), (2, 64, 256, 64)])
def test_samplebmm(gb, shape):
    from genbmm_b200 import _native
    B, M, K, N = shape
    gen = torch.Generator().manual_seed(11 + sum(shape))
    a, b = 2 * torch.randn(B, M, K, generator=gen), 2 * torch.randn(B, K, N, generator=gen)
    u, g = torch.rand(B, M, N, generator=gen), torch.rand(B, M, N, generator=gen)
    c, ga, gb_ = run_fwd_bwd(gb.samplebmm, a, b, g, dev(u))
    out, idx = oracle.dense_fwd(2, a, b, u)
    assert_close(c, oracle.dense_fwd(0, a, b, dtype=np.float64)[0], what="sample value")
    # the same kernels the operator picked (large products take their logsumexp from the tensor-core forward)
    from genbmm_b200 import genmul
    fast = genmul._log_path(M, K, N) == "tensor"
    _, idx_gpu = _native.forward(dev(a), dev(b), 2, dev(u), fast_log=fast)
    idx_gpu = idx_gpu.cpu().numpy()
    margin = oracle.sample_margin(a, b, u)
    firm = margin > 1e-5
    # away from CDF steps the index is exact; on a step either neighbour is a valid draw
    assert np.array_equal(idx_gpu[firm], idx[firm])
    assert_valid_sample(a, b, u, idx_gpu)
    assert firm.mean() > 0.99
    # gradients are the one-hot routing of the cotangent through the indices the GPU drew
    dA, dB = oracle.dense_bwd(2, a, b, g, None, idx_gpu)
    assert_equal_bits(ga, dA, "sample grad_a")
    assert_equal_bits(gb_, dB, "sample grad_b")
    # u = 0 can satisfy no strict inequality: the reference leaves index 0
    for fl in (False, fast):
        _, idx0 = _native.forward(dev(a), dev(b), 2, torch.zeros(B, M, N).cuda(), fast_log=fl)
        assert int(idx0.abs().max()) == 0


def test_samplebmm_draws_its_own_uniforms(gb):
    a, b = torch.randn(2, 8, 16).cuda(), torch.randn(2, 16, 8).cuda()
    c = gb.samplebmm(a, b)
    assert_close(c, oracle.dense_fwd(0, a.cpu(), b.cpu(), dtype=np.float64)[0])


def test_config1_logbmm(gb):
    a, b = cfg1()
    c, ga, gb_ = run_fwd_bwd(gb.logbmm, a, b, torch.ones(32, 64, 64))
    out, maxes = oracle.dense_fwd(0, a, b, dtype=np.float64)
    dA, dB = oracle.dense_bwd(0, a, b, np.ones((32, 64, 64)), out, maxes, dtype=np.float64)
    assert_close(c, out)
    assert_close(ga, dA)
    assert_close(gb_, dB)
    # the reference's own formulation (genbmm/test_cuda.py:17)
    want = (a.double().unsqueeze(-1) + b.double().unsqueeze(-3)).logsumexp(-2)
    assert_close(c, want.numpy())


def test_config2_max_and_prodmax(gb):
    from genbmm_b200 import _native
    a, b = cfg2()
    for name, mode in (("maxbmm", 1), ("prodmaxbmm", 3)):
        for g in (torch.ones(256, 128, 128), torch.rand(256, 128, 128, generator=torch.Generator().manual_seed(9))):
            c, ga, gb_ = run_fwd_bwd(getattr(gb, name), a, b, g)
            out, idx = oracle.dense_fwd(mode, a, b)
            dA, dB = oracle.dense_bwd(mode, a, b, g, None, idx)
            assert_equal_bits(c, out, name)
            assert_equal_bits(_native.forward(dev(a), dev(b), mode)[1], idx, name + " idx")
            assert_equal_bits(ga, dA, name + " grad_a")
            assert_equal_bits(gb_, dB, name + " grad_b")
    # ties really occur in this configuration
    s = a[:8].unsqueeze(-1) + b[:8].unsqueeze(-3)
    assert ((s == s.max(-2, keepdim=True)[0]).sum(-2) > 1).float().mean() > 0.02


def test_config3_samplebmm(gb):
    from genbmm_b200 import _native
    a, b, u = cfg3()
    out_gpu, idx_gpu = _native.forward(dev(a), dev(b), 2, dev(u), fast_log=True)  # what samplebmm runs at this size
    out, idx = oracle.dense_fwd(2, a, b, u)
    assert_close(out_gpu, out, what="value")
    margin = oracle.sample_margin(a, b, u)
    firm = margin > 1e-5
    idx_gpu = idx_gpu.cpu().numpy()
    assert np.array_equal(idx_gpu[firm], idx[firm])
    # bracket tolerance from the data: the kernel's running sum is float32 over K = 256 terms (K * eps), and
    # its logsumexp is the tensor-core forward's, within rtol * |out| + atol of exact, which every probability
    # exp(a + b - out) inherits as a relative error
    tol = 256 * float(np.finfo(np.float32).eps) + 1e-5 * float(np.abs(out).max()) + 2e-6
    assert tol < 3e-4
    for lo in range(0, 64, 9):      # eight of the 64 batch elements, spread over the batch
        assert_valid_sample(a[lo:lo + 1], b[lo:lo + 1], u[lo:lo + 1], idx_gpu[lo:lo + 1], tol=tol)
    assert (~firm).mean() < 0.01


def test_throughput_shape_properties(gb):
    """1024^3 per batch element: full oracle for one element, then size-independent properties."""
    from genbmm_b200 import _native
    gen = torch.Generator().manual_seed(5)
    a, b = torch.randn(2, 1024, 1024, generator=gen), torch.randn(2, 1024, 1024, generator=gen)
    ad, bd = dev(a), dev(b)
    out, idx = _native.forward(ad, bd, 1)
    want, widx = oracle.dense_fwd(1, a[:1], b[:1])
    assert_equal_bits(out[:1], want)
    assert_equal_bits(idx[:1], widx)
    # the index reproduces the value, and no earlier k does better or equal
    k = idx.long()
    av = torch.gather(ad, 2, k[:, :, :256])            # a[b, m, idx[b, m, n]] for n < 256
    bv = torch.gather(bd[:, :, :256], 1, k[:, :, :256])  # b[b, idx[b, m, n], n]
    assert torch.equal(av + bv, out[:, :, :256])
    # log: shifting a row of a by t shifts that row of c by t; gradients of c.sum() are
    # softmax weights: non-negative, grad_a rows sum to N, grad_b columns sum to M
    c, ga, gb_ = run_fwd_bwd(gb.logbmm, a, b, torch.ones(2, 1024, 1024))
    want, maxes = oracle.dense_fwd(0, a[:1, :64], b[:1], dtype=np.float64)
    assert_close(c[:1, :64], want)
    dA, _ = oracle.dense_bwd(0, a[:1, :64], b[:1], np.ones((1, 64, 1024)), want, maxes, dtype=np.float64)
    assert_close(ga[:1, :64], dA)
    assert (ga >= 0).all() and (gb_ >= 0).all()
    assert_close(ga.sum(2), np.full((2, 1024), 1024.0), 1e-4, 1e-3)
    assert_close(gb_.sum(1), np.full((2, 1024), 1024.0), 1e-4, 1e-3)
    a2 = a.clone()
    a2[:, 5, :] += 3.0
    c2 = gb.logbmm(dev(a2), bd)
    assert_close(c2[:, 5], (c[:, 5] + 3.0).cpu().numpy(), 1e-5, 1e-5)
    # the max-plus value bounds the log value from below, within log K from above
    assert (c >= out - 1e-4).all() and (c <= out + np.log(1024.0) + 1e-4).all()


def test_rejects_what_the_reference_rejects(gb):
    a, b = torch.rand(2, 3, 4), torch.rand(2, 4, 5)
    with pytest.raises(RuntimeError, match="a must be a CUDA tensor"):
        gb.logbmm(a, b.cuda())
    with pytest.raises(RuntimeError, match="b must be contiguous"):
        gb.maxbmm(a.cuda(), torch.rand(2, 5, 4).cuda().transpose(1, 2))
    with pytest.raises(RuntimeError):
        gb.logbmm(a.cuda(), torch.rand(2, 7, 5).cuda())


def test_empty_inputs(gb):
    from genbmm_b200 import _native
    out, idx = _native.forward(torch.zeros(0, 3, 4).cuda(), torch.zeros(0, 4, 5).cuda(), 1)
    assert out.shape == (0, 3, 5)
    out, idx = _native.forward(torch.zeros(2, 3, 0).cuda(), torch.zeros(2, 0, 5).cuda(), 1)
    assert (out == -1e9).all() and (idx == -1).all()
    out, _ = _native.forward(torch.zeros(2, 3, 0).cuda(), torch.zeros(2, 0, 5).cuda(), 0)
    assert torch.isinf(out).all()


def test_half_inputs_round_trip(gb):
    a, b = torch.randn(2, 9, 12).cuda().half(), torch.randn(2, 12, 7).cuda().half()
    c = gb.logbmm(a, b)
    assert c.dtype == torch.float16
    want, _ = oracle.dense_fwd(0, a.float().cpu(), b.float().cpu(), dtype=np.float64)
    assert_close(c.float(), want, 2e-3, 2e-3)


@pytest.mark.parametrize("ci", [0, 1, 2, 3])
def test_logbmm_second_order_matches_reference_fixture(gb, golden, ci):
    """genbmm/test_cuda.py:30-42: grad of (grad_a, grad_b) w.r.t. (a, b, back); the reference's own
    test accepts rtol 1e-2, the fixture (float64 autograd of the dense expression) is met at 1e-4."""
    f = lambda k: torch.from_numpy(golden["dense%d_log_%s" % (ci, k)]).float().cuda()
    a, b, back = f("a").requires_grad_(True), f("b").requires_grad_(True), f("back").requires_grad_(True)
    c = gb.logbmm(a, b)
    g = torch.autograd.grad(c, (a, b), back, create_graph=True)
    h = torch.autograd.grad((g[0], g[1]), (a, b, back), (f("h_a"), f("h_b")))
    for got, name in zip(h, ("hh_a", "hh_b", "hh_back")):
        assert_close(got, golden["dense%d_log_%s" % (ci, name)], 1e-4, 1e-5, name)
    # the cotangent of grad_a alone: the case the reference's kernels implement
    c = gb.logbmm(a, b)
    g = torch.autograd.grad(c, (a, b), back, create_graph=True)
    h = torch.autograd.grad(g[0], (a, b, back), f("h_a"))
    for got, name in zip(h, ("ha_only_a", "ha_only_b", "ha_only_back")):
        assert_close(got, golden["dense%d_log_%s" % (ci, name)], 1e-4, 1e-5, name)


@pytest.mark.parametrize("shape", [(2, 33, 17, 65), (2, 130, 70, 67), (1, 129, 200, 130)])
def test_logbmm_second_order_matches_oracle(gb, shape):
    from genbmm_b200 import _native
    B, M, K, N = shape
    gen = torch.Generator().manual_seed(sum(shape))
    a, b = torch.randn(B, M, K, generator=gen), torch.randn(B, K, N, generator=gen)
    g, h = torch.rand(B, M, N, generator=gen), torch.randn(B, M, K, generator=gen)
    out, maxes = oracle.dense_fwd(0, a, b, dtype=np.float64)
    wa, wb, wg = oracle.dense_bwdbwd(a, b, g, out, maxes, h, dtype=np.float64)
    part = torch.from_numpy(out).float().cuda()
    da, db, dg = _native.backbackward(a.cuda(), b.cuda(), g.cuda(), part, None, h.cuda(), 0)
    assert_close(da, wa, 1e-4, 2e-5, "d/da")
    assert_close(db, wb, 1e-4, 2e-5, "d/db")
    assert_close(dg, wg, 1e-4, 2e-5, "d/dgrad_out")


@pytest.mark.parametrize("shape", [(2, 33, 17, 65), (2, 130, 70, 67), (2, 192, 160, 136)])
def test_compiled_binding_and_python_binding_give_the_same_bits(gb, shape):
    """genbmm_b200.logbmm etc. are the C++ autograd functions of genbmm_b200/_shim.so when that module is built;
    the Python autograd Functions of genmul.py over ctypes are the other binding of the same C ABI."""
    from genbmm_b200 import genmul
    if genmul._shim is None:
        pytest.skip("compiled binding not built")
    B, M, K, N = shape
    gen = torch.Generator().manual_seed(sum(shape))
    a, b, g = tied((B, M, K), gen), tied((B, K, N), gen), torch.rand(B, M, N, generator=gen)
    u = torch.rand(B, M, N, generator=gen)
    pairs = [(gb.logbmm, genmul.LogMatMul.apply, ()), (gb.maxbmm, genmul.MaxMatMul.apply, ()),
             (gb.prodmaxbmm, genmul.ProdMaxMatMul.apply, ()),
             (gb.samplebmm, genmul.SampleMatMul.apply, (dev(u),))]
    for compiled, python, extra in pairs:
        got = run_fwd_bwd(compiled, a, b, g, *extra)
        want = run_fwd_bwd(python, a, b, g, *extra)
        for x, y in zip(got, want):
            assert torch.equal(x, y)
    # half precision in, half precision out, through both
    ah, bh = dev(a).half(), dev(b).half()
    assert torch.equal(gb.logbmm(ah, bh), genmul.LogMatMul.apply(ah, bh)) and gb.logbmm(ah, bh).dtype == torch.float16
    # second order through the compiled binding equals second order through the Python one
    res = []
    for fn in (gb.logbmm, genmul.LogMatMul.apply):
        ad, bd, gd = dev(a).requires_grad_(True), dev(b).requires_grad_(True), dev(g).requires_grad_(True)
        ga, gb_ = torch.autograd.grad(fn(ad, bd), (ad, bd), gd, create_graph=True)
        res.append(torch.autograd.grad((ga * ga).sum() + (gb_ * gb_).sum(), (ad, bd, gd)))
    for x, y in zip(*res):
        assert torch.equal(x, y)
    # float64 takes the float64 kernels in both
    c64 = gb.logbmm(dev(a).double(), dev(b).double())
    assert c64.dtype == torch.float64 and torch.equal(c64, genmul.LogMatMul.apply(dev(a).double(), dev(b).double()))
