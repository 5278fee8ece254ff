"""State the fast paths keep between calls, and what a caller sees when a kernel gives up.

Nothing here makes a kernel give up: the error word a product kernel would set is written by the test itself
(a fake word), and the kernels that react to it are run on that.
"""
import numpy as np
import pytest
import torch

import oracle
from util import assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nat():
    from genbmm_b200 import _native
    return _native


def test_error_word_turns_the_output_into_nan_and_is_reported(nat):
    lib = nat.load()
    st = torch.cuda.current_stream().cuda_stream
    out = torch.ones(100_003, device="cuda")
    word = torch.zeros(64, dtype=torch.int32, device="cuda")
    assert lib.gbmm_poison_on_error(word.data_ptr(), out.data_ptr(), out.numel(), st) == 0
    assert lib.gbmm_logbmm_check(word.data_ptr(), st) == 0
    assert bool((out == 1).all())            # word clear: nothing is touched
    word[0] = 1                               # what a product kernel does when a bounded wait runs out
    assert lib.gbmm_poison_on_error(word.data_ptr(), out.data_ptr(), out.numel(), st) == 0
    assert lib.gbmm_logbmm_check(word.data_ptr(), st) == 3
    assert bool(torch.isnan(out).all())      # the whole output, not just a tile
    assert lib.gbmm_poison_on_error(None, out.data_ptr(), 1, st) == 1


def test_fast_paths_leave_their_error_word_clear(nat):
    """After ordinary calls the words read as zero through both check entries (dense workspace, banded
    workspace, built-in scratch of the no-allocation forward)."""
    lib = nat.load()
    st = torch.cuda.current_stream().cuda_stream
    a, b = torch.randn(2, 200, 160, device="cuda"), torch.randn(2, 160, 136, device="cuda")
    out, rowmax, colmax, flags, ws = nat.logbmm_fast_forward(a, b, tensor_cores=True, keep_factors=True)
    assert lib.gbmm_logbmm_check(ws.data_ptr(), st) == 0 and bool(torch.isfinite(out).all())
    o2 = torch.empty_like(out)
    assert lib.gbmm_logbmm_forward_noalloc_f32(a.data_ptr(), b.data_ptr(), o2.data_ptr(), 2, 200, 160, 136, st) == 0
    assert lib.gbmm_logbmm_forward_noalloc_check(st) == 0
    x, y = torch.randn(2, 300, 41, device="cuda"), torch.randn(2, 300, 41, device="cuda")
    r, _, _, token = nat.forward_band(x, 20, 20, y, 20, 20, 0, want_token=True)
    assert token is not None and lib.gbmm_logbmm_check(token.ws.buf.data_ptr(), st) == 0
    assert bool(torch.isfinite(r).all())


@pytest.mark.parametrize("method,mode", [("multiply", 3), ("multiply_log", 0), ("multiply_max", 1)])
def test_same_shape_banded_products_on_two_streams(method, mode):
    """Two products of the same dimensions issued on two streams with nothing ordering them: each stream has
    its own workspace, so both match the oracle (with one shared workspace they would race on the operand
    copies).  Forward and backward, several rounds to give an overlap every chance."""
    import genbmm_b200 as gb
    B, n, lu, ld = 4, 2048, 40, 40
    gen = torch.Generator().manual_seed(21 + mode)
    data = [torch.randn(B, n, lu + ld + 1, generator=gen) for _ in range(4)]
    if mode == 1:
        data = [(x * 4).round() / 4 for x in data]
    g = torch.rand(B, n, 2 * (lu + ld) + 1, generator=gen)
    dt = np.float32 if mode == 1 else np.float64
    want = [oracle.band_fwd_bwd(mode, data[2 * i], lu, ld, data[2 * i + 1], lu, ld, g, dtype=dt) for i in range(2)]
    # sum semiring: terms of both signs, so the same sums over magnitudes bound the rounding (util.assert_close)
    mags = [oracle.band_fwd_bwd(3, data[2 * i].abs(), lu, ld, data[2 * i + 1].abs(), lu, ld, g, dtype=dt)
            if mode == 3 else None for i in range(2)]
    dev = [x.cuda() for x in data]
    gd = g.cuda()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    for _ in range(3):
        got = []
        for i, s in enumerate(streams):
            with torch.cuda.stream(s):
                a, b = dev[2 * i].clone().requires_grad_(True), dev[2 * i + 1].clone().requires_grad_(True)
                r = getattr(gb.BandedMatrix(a, lu, ld), method)(gb.BandedMatrix(b, lu, ld))
                ga, gb_ = torch.autograd.grad(r.data, (a, b), gd)
                got.append((r.data.detach(), ga, gb_))
        torch.cuda.synchronize()
        for (out, ga, gb_), (wout, _, _, dA, dB), mag in zip(got, want, mags):
            if mode == 1:
                assert np.array_equal(out.cpu().numpy(), wout)
                assert np.array_equal(ga.cpu().numpy(), dA) and np.array_equal(gb_.cpu().numpy(), dB)
            else:
                ts = (None, None, None) if mag is None else (mag[0], mag[3], mag[4])
                assert_close(out, wout, term_sum=ts[0])
                assert_close(ga, dA, term_sum=ts[1])
                assert_close(gb_, dB, term_sum=ts[2])
    from genbmm_b200 import _native
    kinds = {k[0] for k in _native._ws_cache}
    assert len([k for k in _native._ws_cache if k[2] in (streams[0].cuda_stream, streams[1].cuda_stream)]) >= 2, kinds
    _native.release_workspaces()
    assert not _native._ws_cache


def test_backward_after_an_intervening_product_rebuilds_its_operands():
    """The backward reuses the forward's converted operands only while nothing else wrote into that
    workspace: a second product of the same shape in between must not leak into the first one's gradients."""
    import genbmm_b200 as gb
    B, n, lu, ld = 2, 512, 33, 33
    gen = torch.Generator().manual_seed(8)
    x, y, x2, y2 = (torch.randn(B, n, lu + ld + 1, generator=gen) for _ in range(4))
    g = torch.rand(B, n, 2 * (lu + ld) + 1, generator=gen)
    a, b = x.cuda().requires_grad_(True), y.cuda().requires_grad_(True)
    r = gb.BandedMatrix(a, lu, ld).multiply_log(gb.BandedMatrix(b, lu, ld))
    gb.BandedMatrix(x2.cuda(), lu, ld).multiply_log(gb.BandedMatrix(y2.cuda(), lu, ld))   # same workspace
    ga, gb_ = torch.autograd.grad(r.data, (a, b), g.cuda())
    _, _, _, dA, dB = oracle.band_fwd_bwd(0, x, lu, ld, y, lu, ld, g, dtype=np.float64)
    assert_close(ga, dA)
    assert_close(gb_, dB)


def test_fused_chain_levels_refuse_a_double_backward():
    """The chain driver's fused tree level is first-order only; asking for second-order gradients through it
    raises instead of returning zeros, and the unfused path (bmm given) computes them."""
    import genbmm_b200 as gb
    from genbmm_b200 import crf
    pot = torch.randn(2, 8, 128, 128, device="cuda", requires_grad=True)
    logz = crf.log_partition(pot)
    g, = torch.autograd.grad(logz.sum(), pot, create_graph=True)
    with pytest.raises(RuntimeError):
        g.square().sum().backward()
    pot2 = torch.randn(1, 4, 24, 24, device="cuda", requires_grad=True)
    logz = crf.log_partition(pot2, bmm=gb.logbmm)
    g, = torch.autograd.grad(logz.sum(), pot2, create_graph=True)
    gg, = torch.autograd.grad(g.square().sum(), pot2)
    assert bool(torch.isfinite(gg).all()) and float(gg.abs().max()) > 0


def test_launch_counter_counts_kernels(nat):
    lib = nat.load()
    a, b = torch.randn(2, 40, 30, device="cuda"), torch.randn(2, 30, 20, device="cuda")
    before = lib.gbmm_launch_count()
    nat.forward(a, b, 0)             # exact log forward: one kernel
    assert lib.gbmm_launch_count() - before == 1
    before = lib.gbmm_launch_count()
    nat.forward(a, b, 2, torch.rand(2, 40, 20, device="cuda"))   # sample: log forward + pick
    assert lib.gbmm_launch_count() - before == 2
