"""The no-allocation logbmm forward (gbmm_logbmm_forward_noalloc_f32), called through the C ABI.

It serves callers that may not allocate device memory where they need the product (a region
that forbids new reservations, a latency-bound loop, a host framework with fixed buffers): its
scratch is a fixed 32 MiB array inside the library.  The test drives it with ctypes and raw
pointers, twice in a row with different problems (the array keeps the first call's contents
when the second starts), and compares with the existing forward entry point.  This file sorts
last on purpose so that a stop-at-first-failure run has already run every other test.
"""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 2e-6  # the tolerance of the log semiring everywhere in this suite


def _call(lib, a, b, out):
    B, M, K = a.shape
    N = b.shape[2]
    out.fill_(float("nan"))
    st = lib.gbmm_logbmm_forward_noalloc_f32(a.data_ptr(), b.data_ptr(), out.data_ptr(), B, M, K, N,
                                             torch.cuda.current_stream().cuda_stream)
    assert st == 0, lib.gbmm_status_string(st)
    return out


def test_no_alloc_forward_matches_the_allocating_entry_points():
    from genbmm_b200 import _native
    lib = _native.load()
    gen = torch.Generator().manual_seed(0)
    first = (torch.randn(3, 300, 200, generator=gen).cuda(), torch.randn(3, 200, 260, generator=gen).cuda())
    second = (torch.randn(2, 70, 33, generator=gen).cuda(), torch.randn(2, 33, 50, generator=gen).cuda())
    second[0][:, :10, :16] -= 400.0   # rows and columns whose supports miss each other:
    second[1][:, 16:, :12] -= 400.0   # exercises the flagged-tile recomputation as well
    outs = [torch.empty(3, 300, 260, device="cuda"), torch.empty(2, 70, 50, device="cuda")]
    wants = [(_native.forward(a, b, 0)[0], _native.logbmm_fast_forward(a, b)[0]) for a, b in (first, second)]
    # the first call on a device looks up the scratch address (and loads the kernels)
    _call(lib, *second, outs[1])
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for (a, b), out in zip((first, second), outs):   # two calls in a row, nothing else in between
        _call(lib, a, b, out)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before   # the two calls reserved no device memory
    for got, (want_exact, want_fast), (a, b) in zip(outs, wants, (first, second)):
        assert torch.allclose(got, want_exact, rtol=RTOL, atol=ATOL)
        assert torch.equal(got, want_fast)   # same kernels, same arithmetic
        # and against the float64 CPU oracle, like every other forward in this suite
        want = oracle.dense_fwd(0, a.cpu(), b.cpu(), dtype=np.float64)[0]
        assert np.allclose(got.cpu().numpy(), want, rtol=RTOL, atol=ATOL)


def test_no_alloc_forward_rejects_what_does_not_fit():
    from genbmm_b200 import _native
    lib = _native.load()
    limit = lib.gbmm_logbmm_forward_noalloc_max_bytes()
    assert limit == 32 << 20
    assert lib.gbmm_logbmm_forward_noalloc_need_bytes(3, 1024, 1024, 1024) <= limit
    assert lib.gbmm_logbmm_forward_noalloc_need_bytes(4, 1024, 1024, 1024) > limit
    x = torch.zeros(1, device="cuda")
    st = lib.gbmm_logbmm_forward_noalloc_f32(x.data_ptr(), x.data_ptr(), x.data_ptr(), 4, 1024, 1024, 1024, None)
    assert st == 5 and b"scratch" in lib.gbmm_status_string(st)
    assert lib.gbmm_logbmm_forward_noalloc_f32(None, None, None, 1, 8, 8, 8, None) == 1
