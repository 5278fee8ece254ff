"""genbmm_b200 — semiring batched matrix products for PyTorch on B200 (sm_100a).

Drop-in for harvardnlp/genbmm's public surface (genbmm/__init__.py:1-2):

    import genbmm_b200 as genbmm
    c = genbmm.logbmm(a, b)          # also maxbmm, samplebmm, prodmaxbmm
    z = genbmm.BandedMatrix(data, lu, ld).multiply_log(other)

Everything runs on hand-written CUDA kernels reached through a C-ABI shared library
(include/genbmm_b200.h); importing this package loads that library and fails if it is absent.
"""
from . import _native

_native.load()

from .genmul import logbmm, maxbmm, prodmaxbmm, samplebmm  # noqa: E402
from .sparse import BandedMatrix, banddiag  # noqa: E402

__all__ = ["logbmm", "samplebmm", "maxbmm", "prodmaxbmm", "BandedMatrix", "banddiag"]
