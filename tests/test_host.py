"""CPU-side checks: the C-ABI library loads and exports what the header declares, the host
mirror rejects what the reference rejects, and the pure-torch band utilities match the
reference fixtures.  No kernel is launched here."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "genbmm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gbmm_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from genbmm_b200 import _native
    lib = ctypes.CDLL(_native.library_path()) if os.path.exists(_native.library_path()) else _native.load()
    names = header_symbols()
    assert "gbmm_dense_forward_f32" in names and "gbmm_band_backward_f32" in names
    for name in names:
        assert hasattr(lib, name), name
    assert set(names) >= set(_native.exported_symbols())


def test_status_strings_and_argument_validation_without_a_gpu():
    from genbmm_b200 import _native
    lib = _native.load()
    assert lib.gbmm_abi_version() >= 1
    assert lib.gbmm_status_string(0) == b"ok"
    assert lib.gbmm_status_string(1) == b"invalid argument"
    # validation happens before any CUDA call, so these return without a device
    assert lib.gbmm_dense_forward_f32(9, None, None, None, None, None, 1, 1, 1, 1, None, 0, None) == 1
    assert lib.gbmm_dense_forward_f32(0, None, None, None, None, None, 1, 1, 1, 1, None, 0, None) == 1
    assert lib.gbmm_dense_forward_f32(0, None, None, None, None, None, 0, 1, 1, 1, None, 0, None) == 0
    assert lib.gbmm_dense_forward_f32(0, None, None, None, None, None, -1, 1, 1, 1, None, 0, None) == 1
    assert lib.gbmm_band_forward_f32(2, None, 1, 1, None, 1, 1, None, None, None, 1, 4, None, 0, None) == 1
    assert lib.gbmm_band_forward_f32(3, None, -1, 1, None, 1, 1, None, None, None, 1, 4, None, 0, None) == 1
    assert lib.gbmm_band_backward_f32(0, None, 1, 1, None, 1, 1, None, None, None, None, 0, 4, None, 0, None) == 0


def test_host_mirror_rejects_cpu_and_strided_tensors():
    import genbmm_b200 as gb
    a, b = torch.rand(2, 3, 4), torch.rand(2, 4, 5)
    for fn in (gb.logbmm, gb.maxbmm, gb.samplebmm, gb.prodmaxbmm):
        with pytest.raises(RuntimeError, match="a must be a CUDA tensor"):
            fn(a, b)
    with pytest.raises(RuntimeError, match="a must be a CUDA tensor"):
        gb.BandedMatrix(torch.rand(2, 5, 3), 1, 1).multiply_log(gb.BandedMatrix(torch.rand(2, 5, 3), 1, 1))
    with pytest.raises(RuntimeError, match="a must be a CUDA tensor"):
        gb.logbmm(a.double(), b.double())   # float64 has kernels of its own, and the same checks
    with pytest.raises(RuntimeError, match="not supported"):
        gb.logbmm(a.long(), b.long())


def test_public_names_match_the_reference():
    import genbmm_b200 as gb
    from genbmm_b200 import genmul, sparse
    for name in ("logbmm", "samplebmm", "maxbmm", "prodmaxbmm", "BandedMatrix", "banddiag"):
        assert hasattr(gb, name)
    for name in ("LogMatMul", "LogMatMulBack", "MaxMatMul", "SampleMatMul", "ProdMaxMatMul", "trans"):
        assert hasattr(genmul, name)
    for name in ("banddiag", "repdiag", "Transpose", "BandedMatrix", "BandedMul", "BandedLogMul", "BandedMaxMul",
                 "bandedbmm", "bandedlogbmm", "bandedmaxbmm"):
        assert hasattr(sparse, name)
    for m in ("band_shift", "band_pad", "band_unshift", "col_shift", "col_unshift", "to_dense", "_expand", "op",
              "transpose", "multiply", "multiply_log", "multiply_max", "multiply_back"):
        assert hasattr(sparse.BandedMatrix, m)


@pytest.mark.parametrize("ci", [0, 1, 2, 3, 4])
def test_band_utilities_match_reference_fixture(golden, ci):
    import genbmm_b200 as gb
    B, n, alu, ald, blu, bld = (int(v) for v in golden["band%d_dims" % ci])
    dense = torch.from_numpy(golden["band%d_dense_a" % ci])
    band, same = gb.banddiag(dense, alu, ald)
    assert same is dense
    assert np.array_equal(band.numpy(), golden["band%d_a" % ci])
    x = gb.BandedMatrix(band, alu, ald)
    assert np.array_equal(x.transpose().data.numpy(), golden["band%d_a_T" % ci])
    assert (x.transpose().lu, x.transpose().ld) == (ald, alu)
    assert np.array_equal(x.to_dense().numpy(), golden["band%d_a_dense" % ci])
    # transpose is an involution on in-matrix cells and its autograd is the transpose back
    assert np.array_equal(x.transpose().transpose().data.numpy(), golden["band%d_a" % ci])
    v = band.clone().requires_grad_(True)
    gb.BandedMatrix(v, alu, ald).transpose().data.sum().backward()
    i = np.arange(n)[:, None] + np.arange(alu + ald + 1)[None, :] - alu
    assert np.array_equal(v.grad.numpy(), np.broadcast_to(((i >= 0) & (i < n)).astype(np.float64), v.shape))


def test_band_layout_operations():
    """Dense meaning of op / col_shift / band_shift / band_pad / _expand (genbmm/test_sparse.py:43-55, 96-107)."""
    import genbmm_b200 as gb
    gen = torch.Generator().manual_seed(1)
    B, n = 2, 7
    for lu, ld in ((1, 1), (2, 0), (0, 3), (3, 2)):
        dense = torch.rand(B, n, n, generator=gen)
        x = gb.BandedMatrix(gb.banddiag(dense, lu, ld)[0], lu, ld)
        mid = x.to_dense()
        plus = x.op(x, lambda p, q: p + q)
        assert (plus.lu, plus.ld) == (lu, ld) and torch.equal(plus.to_dense(), mid + mid)
        sym = x.op(x.transpose(), lambda p, q: p + q)
        assert sym.lu == sym.ld == max(lu, ld)
        assert torch.equal(sym.to_dense(), mid + mid.transpose(-2, -1))
        # col_shift moves the stored columns: dense column c becomes column c - t
        for t in (1, -1, 2):
            s = x.col_shift(t)
            assert (s.lu, s.ld) == (lu - t, ld + t)
            assert s.data.shape == x.data.shape
            if t > 0:
                assert torch.equal(s.data[:, :-t], x.data[:, t:]) and (s.data[:, -t:] == 0).all()
            else:
                assert torch.equal(s.data[:, -t:], x.data[:, :t]) and (s.data[:, :-t] == 0).all()
        assert torch.equal(x.col_unshift().data[:, 1:], x.data[:, :-1])
        e = x._expand(lu + 2, ld + 1)
        assert torch.equal(e.to_dense(), mid)
        p = x.band_pad(2)
        assert (p.lu, p.ld) == (lu + 2, ld + 2) and torch.equal(p.to_dense(), mid)
        if lu + ld >= 1:
            sh = x.band_shift(1)
            assert (sh.lu, sh.ld) == (lu + 1, ld - 1)
            assert torch.equal(sh.data[:, :, :-1], x.data[:, :, 1:]) and (sh.data[:, :, -1] == 0).all()
            un = x.band_unshift()
            assert (un.lu, un.ld) == (lu - 1, ld + 1)
            assert torch.equal(un.data[:, :, 1:], x.data[:, :, :-1])
    y = gb.BandedMatrix(torch.zeros(1, 3, 3), 1, 1, fill=-1e9)
    assert (y.band_pad(1).data[:, :, 0] == -1e9).all() and (y.to_dense()[0, 0, 2] == -1e9)


def test_band_forward_token_is_valid_only_until_the_workspace_is_written_again():
    """Host logic of the operand reuse between a banded forward and its backward (no GPU involved)."""
    from genbmm_b200 import _native
    ws = _native._Workspace((2, 128, 20, 20, 20, 20), None)
    ws.generation, ws.holds = 5, 0
    tok = _native.BandForwardToken(ws, 0)
    assert tok.valid_for(ws, 0)
    assert not tok.valid_for(ws, 3)                       # another semiring's copies
    other = _native._Workspace(ws.dims, None)
    other.generation, other.holds = 5, 0
    assert not tok.valid_for(other, 0)                    # another stream's (or a rebuilt) workspace
    ws.generation += 1                                    # any later call that writes into it
    assert not tok.valid_for(ws, 0)
    ws.generation -= 1
    ws.holds = None                                       # a call that left the copies incomplete
    assert not tok.valid_for(ws, 0)


def test_host_pipeline_chunk_bounds():
    """Equal chunks and the tapered form cover the batch exactly once, in order."""
    from genbmm_b200.host import chunk_bounds
    for B in (1, 2, 5, 11, 12, 16, 31, 32, 64, 100):
        for chunks in (1, 3, 8, 200, "tapered"):
            bounds = chunk_bounds(B, chunks)
            assert bounds[0][0] == 0 and bounds[-1][1] == B
            assert all(lo < hi for lo, hi in bounds)
            assert all(bounds[i][1] == bounds[i + 1][0] for i in range(len(bounds) - 1))
    assert [hi - lo for lo, hi in chunk_bounds(32, "tapered")] == [1, 1, 2, 4, 4, 4, 4, 4, 4, 2, 1, 1]
