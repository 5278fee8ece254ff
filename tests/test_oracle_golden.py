"""The CPU oracle against the fixtures generated from the reference's own Python code.

Dense: the broadcast-reduce expressions of README.md:30-65 / genbmm/test_cuda.py:17 and their
autograd gradients.  Banded: genbmm/sparse.py's multiply_simple / multiply_log_simple /
multiply_max_simple loops, transpose, to_dense and multiply_back_simple.
"""
import numpy as np
import pytest

import oracle

DENSE = [0, 1, 2, 3]
BAND = [0, 1, 2, 3, 4]


def close(x, y, rtol=1e-9, atol=1e-12):
    return np.allclose(x, y, rtol=rtol, atol=atol)


@pytest.mark.parametrize("ci", DENSE)
def test_dense_log_f64(golden, ci):
    g = lambda k: golden["dense%d_log_%s" % (ci, k)]
    out, maxes = oracle.dense_fwd(0, g("a"), g("b"), dtype=np.float64)
    assert close(out, g("c"))
    dA, dB = oracle.dense_bwd(0, g("a"), g("b"), g("back"), out, maxes, dtype=np.float64)
    assert close(dA, g("ga")) and close(dB, g("gb"))
    # second order: the reference's kernels differentiate <grad_a, h_a> only
    hA, hB, hG = oracle.dense_bwdbwd(g("a"), g("b"), g("back"), out, maxes, g("h_a"), dtype=np.float64)
    assert close(hA, g("ha_only_a"), 1e-7, 1e-10)
    assert close(hB, g("ha_only_b"), 1e-7, 1e-10)
    assert close(hG, g("ha_only_back"), 1e-7, 1e-10)


@pytest.mark.parametrize("ci", DENSE)
def test_dense_log_f32_within_tolerance(golden, ci):
    g = lambda k: golden["dense%d_log_%s" % (ci, k)]
    out, maxes = oracle.dense_fwd(0, g("a"), g("b"), dtype=np.float32)
    assert np.allclose(out, g("c"), rtol=1e-5, atol=1e-6)
    dA, dB = oracle.dense_bwd(0, g("a"), g("b"), g("back"), out, maxes, dtype=np.float32)
    assert np.allclose(dA, g("ga"), rtol=1e-5, atol=1e-6)
    assert np.allclose(dB, g("gb"), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("ci", DENSE)
@pytest.mark.parametrize("op,mode", [("max", 1), ("prodmax", 3)])
def test_dense_max_bit_exact(golden, ci, op, mode):
    g = lambda k: golden["dense%d_%s_%s" % (ci, op, k)]
    out, idx = oracle.dense_fwd(mode, g("a"), g("b"))
    assert np.array_equal(out, g("c"))
    assert np.array_equal(idx, g("idx_low"))          # lowest k among ties
    dA, dB = oracle.dense_bwd(mode, g("a"), g("b"), g("back"), None, idx)
    # routed sums: same addends; the order over n / m may differ from autograd's by rounding
    assert np.allclose(dA, g("ga"), rtol=1e-6, atol=1e-6)
    assert np.allclose(dB, g("gb"), rtol=1e-6, atol=1e-6)
    # where torch.max itself returned the lowest index (observed, not promised) the routing is identical
    assert np.array_equal(g("idx_torch"), g("idx_low"))


@pytest.mark.parametrize("ci", DENSE)
def test_dense_sample_value_and_index_rule(golden, ci):
    g = lambda k: golden["dense%d_log_%s" % (ci, k)]
    a, b = g("a"), g("b")
    rng = np.random.default_rng(7 + ci)
    u = rng.random(g("c").shape)
    out, idx = oracle.dense_fwd(2, a, b, u, dtype=np.float64)
    assert close(out, g("c"))
    # inverse-CDF rule restated independently (matmul_cuda_kernel.cu:109-118)
    p = np.exp(a[:, :, :, None] + b[:, None, :, :] - out[:, :, None, :])
    cdf = np.cumsum(p, axis=2)
    lo = np.concatenate([np.zeros_like(cdf[:, :, :1]), cdf[:, :, :-1]], axis=2)
    hit = (lo < u[:, :, None, :]) & (cdf > u[:, :, None, :])
    want = np.where(hit.any(2), hit.argmax(2), 0)
    margin = oracle.sample_margin(a, b, u, dtype=np.float64)
    ok = margin > 1e-9
    assert np.array_equal(idx[ok], want[ok].astype(np.int32))
    # gradient of a sample is a one-hot routing of the cotangent
    dA, dB = oracle.dense_bwd(2, a, b, g("back"), None, idx, dtype=np.float64)
    onehot = (np.arange(a.shape[2])[None, None, :, None] == idx[:, :, None, :])
    assert close(dA, (onehot * g("back")[:, :, None, :]).sum(3))
    assert close(dB, (onehot * g("back")[:, :, None, :]).sum(1))


def _dims(golden, ci):
    return [int(v) for v in golden["band%d_dims" % ci]]


def _inside(B, n, lu, ld):
    i = np.arange(n)[:, None]
    j = np.arange(lu + ld + 1)[None, :]
    o = i + j - lu
    return np.broadcast_to((o >= 0) & (o < n), (B, n, lu + ld + 1))


@pytest.mark.parametrize("ci", BAND)
def test_band_layout_and_transpose(golden, ci):
    B, n, alu, ald, blu, bld = _dims(golden, ci)
    a = golden["band%d_a" % ci]
    dense = golden["band%d_dense_a" % ci]
    # storage rule pinned by genbmm/test_sparse.py:18-24: band[c, lu - c + r] = dense[r, c]
    for c in range(n):
        for j in range(alu + ald + 1):
            r = c + j - alu
            want = dense[:, r, c] if 0 <= r < n else 0.0
            assert np.array_equal(a[:, c, j], np.broadcast_to(want, (B,)))
    assert np.array_equal(oracle.band_transpose(a, alu, ald, dtype=np.float64), golden["band%d_a_T" % ci])


@pytest.mark.parametrize("ci", BAND)
@pytest.mark.parametrize("name,mode", [("mul", 3), ("log", 0), ("max", 1)])
def test_band_products_f64(golden, ci, name, mode):
    B, n, alu, ald, blu, bld = _dims(golden, ci)
    g = lambda k: golden["band%d_%s" % (ci, k)]
    out, idx, maxes, dA, dB = oracle.band_fwd_bwd(mode, g("a"), alu, ald, g("b"), blu, bld, g("g"),
                                                  dtype=np.float64)
    inside = _inside(B, n, alu + bld, ald + blu)
    assert close(out[inside], g(name + "_out")[inside])
    assert np.all(out[~inside] == 0.0)               # banded_cuda_kernel.cu:38 leaves them zero
    # the reference loops only write in-matrix cells, so autograd sees the cotangent there only;
    # so does the kernel formulation (o outside [0,n) contributes nothing)
    assert close(dA, g(name + "_ga") * _inside(B, n, alu, ald), 1e-8, 1e-11)
    assert close(dB, g(name + "_gb") * _inside(B, n, blu, bld), 1e-8, 1e-11)


@pytest.mark.parametrize("ci", BAND)
def test_band_mul_back_simple(golden, ci):
    B, n, alu, ald, blu, bld = _dims(golden, ci)
    g = lambda k: golden["band%d_%s" % (ci, k)]
    dA = oracle.band_bwd(3, g("a"), alu, ald, g("b"), blu, bld, g("g"), None, dtype=np.float64)
    # multiply_back_simple (sparse.py:382-401) returns the band-transposed gradient and also
    # fills cells outside the matrix; compare inside
    want = oracle.band_transpose(g("mul_back_simple"), ald, alu, dtype=np.float64)
    inside = _inside(B, n, alu, ald)
    assert close(dA[inside], want[inside], 1e-8, 1e-11)


@pytest.mark.parametrize("ci", BAND)
def test_band_log_second_order_f64(golden, ci):
    """Autograd through the reference's multiply_log_simple (float64) pins the restated kernels A/B/C."""
    B, n, alu, ald, blu, bld = _dims(golden, ci)
    g = lambda k: golden["band%d_%s" % (ci, k)]
    dA, dB, dG = oracle.band_bwdbwd(g("a"), alu, ald, g("b"), blu, bld, g("g"), g("log_out"), g("log_h_a"),
                                    g("log_h_b"), dtype=np.float64)
    ins = lambda lu, ld: _inside(B, n, lu, ld)
    np.testing.assert_allclose(dA, g("log_hh_a") * ins(alu, ald), rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(dB, g("log_hh_b") * ins(blu, bld), rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(dG, g("log_hh_g") * ins(alu + bld, ald + blu), rtol=1e-9, atol=1e-11)
