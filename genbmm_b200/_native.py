"""Host-side binding of the C-ABI library, shaped like the reference's `_genbmm` module.

The reference's Python code calls a pybind11 extension `_genbmm` with six functions
(matmul_cuda.cpp:165-172) that take torch tensors, allocate their outputs and return lists of
tensors.  This module offers the same functions with the same argument order and the same
error messages for the same mistakes, implemented by allocating the outputs with torch and
passing raw device pointers plus the current CUDA stream to libgenbmm_b200.so through ctypes.

There is no CPU path: a tensor that is not on a CUDA device is rejected exactly as the
reference's CHECK_CUDA does, and a missing library is an ImportError.
"""
import ctypes
import os
import threading

import torch

from . import build as _build

_P, _I, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64

_SIGNATURES = {
    "gbmm_status_string": ([_I], ctypes.c_char_p),
    "gbmm_abi_version": ([], _I),
    "gbmm_dense_forward_workspace_bytes": ([_I, _L, _L, _L, _L], _L),
    "gbmm_dense_forward_f32": ([_I, _P, _P, _P, _P, _P, _L, _L, _L, _L, _P, _L, _P], _I),
    "gbmm_dense_sample_pick_f32": ([_P, _P, _P, _P, _P, _L, _L, _L, _L, _P], _I),
    "gbmm_dense_backward_f32": ([_I, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _P], _I),
    "gbmm_dense_backbackward_f32": ([_P] * 9 + [_L] * 4 + [_P], _I),
    "gbmm_dense_forward_f64": ([_I, _P, _P, _P, _P, _P, _L, _L, _L, _L, _P], _I),
    "gbmm_dense_backward_f64": ([_I, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _P], _I),
    "gbmm_band_forward_f64": ([_I, _P, _I, _I, _P, _I, _I, _P, _P, _P, _L, _L, _P], _I),
    "gbmm_band_backward_f64": ([_I, _P, _I, _I, _P, _I, _I, _P, _P, _P, _P, _L, _L, _P], _I),
    "gbmm_band_workspace_bytes": ([_L, _L], _L),
    "gbmm_band_forward_f32": ([_I, _P, _I, _I, _P, _I, _I, _P, _P, _P, _L, _L, _P, _L, _P], _I),
    "gbmm_band_backward_f32": ([_I, _P, _I, _I, _P, _I, _I, _P, _P, _P, _P, _L, _L, _P, _L, _P], _I),
    "gbmm_band_backbackward_f32": ([_P, _I, _I, _P, _I, _I, _P, _P, _P, _P, _P, _P, _P, _L, _L, _P], _I),
    "gbmm_band_max_eligible": ([_L, _I, _I, _I, _I], _I),
    "gbmm_band_max_workspace_bytes": ([_L, _L, _I, _I, _I, _I], _L),
    "gbmm_band_max_workspace_init": ([_P, _L, _P], _I),
    "gbmm_band_max_forward_f32": ([_P, _I, _I, _P, _I, _I, _P, _P, _L, _L, _P, _L, _P], _I),
    "gbmm_band_tc_eligible": ([_I, _L, _I, _I, _I, _I], _I),
    "gbmm_band_tc_workspace_bytes": ([_I, _L, _L, _I, _I, _I, _I], _L),
    "gbmm_band_tc_workspace_init": ([_P, _L, _P], _I),
    "gbmm_band_tc_forward_f32": ([_I, _P, _I, _I, _P, _I, _I, _P, _L, _L, _P, _L, _P], _I),
    "gbmm_band_tc_backward_f32": ([_I, _P, _I, _I, _P, _I, _I, _P, _P, _P, _P, _L, _L, _P, _L, _I, _P], _I),
    "gbmm_logbmm_workspace_bytes": ([_I, _L, _L, _L, _L], _L),
    "gbmm_logbmm_flag_count": ([_L, _L, _L], _L),
    "gbmm_logbmm_forward_f32": ([_P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _P], _I),
    "gbmm_logbmm_backward_f32": ([_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _P], _I),
    "gbmm_logbmm_check": ([_P, _P], _I),
    "gbmm_logbmm_tc_workspace_bytes": ([_I, _L, _L, _L, _L], _L),
    "gbmm_logbmm_tc_forward_f32": ([_P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _P], _I),
    "gbmm_logbmm_tc_backward_f32": ([_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _P], _I),
    "gbmm_logbmm_forward_noalloc_max_bytes": ([], _L),
    "gbmm_logbmm_forward_noalloc_need_bytes": ([_L, _L, _L, _L], _L),
    "gbmm_logbmm_forward_noalloc_f32": ([_P, _P, _P, _L, _L, _L, _L, _P], _I),
    "gbmm_logbmm_forward_noalloc_check": ([_P], _I),
    "gbmm_launch_count": ([], ctypes.c_uint64),
    "gbmm_poison_on_error": ([_P, _P, _L, _P], _I),
    "gbmm_gather_blocks_f32": ([_P, _P, _P, _L, _L, _I, _P], _I),
    "gbmm_profile_enable": ([_I], None),
    "gbmm_profile_last_ms": ([_I], ctypes.c_float),
}

_lib = None


def library_path():
    return _build.LIB


def load():
    """dlopen libgenbmm_b200.so (building it first when a toolkit is present and it is stale)."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB
    try:
        if _build.stale():
            _build.build()
    except Exception as exc:  # no nvcc, or a compile error
        if not os.path.exists(path):
            raise ImportError(
                "genbmm_b200: the CUDA library %s is missing and could not be built (%s). "
                "There is no CPU fallback; run `python -m genbmm_b200.build`." % (path, exc))
    lib = ctypes.CDLL(path)
    for name, (args, res) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = library and header out of step
        fn.argtypes = args
        fn.restype = res
    _lib = lib
    return lib


def exported_symbols():
    return sorted(_SIGNATURES)


def _check(status, what):
    if status != 0:
        msg = load().gbmm_status_string(status).decode()
        raise RuntimeError("%s failed: %s (status %d)" % (what, msg, status))


def _check_input(x, name, dtype=torch.float32):
    # same conditions and messages as CHECK_CUDA / CHECK_CONTIGUOUS, matmul_cuda.cpp:65-67
    if not x.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor" % name)
    if not x.is_contiguous():
        raise RuntimeError("%s must be contiguous" % name)
    if x.dtype != dtype:
        raise RuntimeError("%s must be %s (got %s)" % (name, dtype, x.dtype))


def _compute_dtype(x):
    """float32 or float64 kernels; anything else is an error here (the operators widen half / bfloat16)."""
    return torch.float64 if x.dtype == torch.float64 else torch.float32


def _stream(dev):
    return torch.cuda.current_stream(dev).cuda_stream


def _ptr(x):
    return None if x is None else x.data_ptr()


MODE_LOG, MODE_MAX, MODE_SAMPLE, MODE_PRODMAX = 0, 1, 2, 3
BAND_LOG, BAND_MAX, BAND_MUL = 0, 1, 3


def forward(a, b, mode, u=None, want_maxes=True, fast_log=False):
    """`_genbmm.forward(a, b, mode)` -> [out, aux]; aux = maxes (mode 0) or int32 indices.

    Mode 2 (sample) takes the uniforms `u`:(B,M,N); when None they are drawn with torch.rand
    on the device, as the reference does inside its dispatcher (matmul_cuda_kernel.cu:517);
    fast_log=True takes its logsumexp from the factorised tensor-core forward (float32 only).
    """
    dt = _compute_dtype(a)
    _check_input(a, "a", dt)
    _check_input(b, "b", dt)
    if a.dim() != 3 or b.dim() != 3 or a.shape[0] != b.shape[0] or a.shape[2] != b.shape[1]:
        raise RuntimeError("expected a:(B,M,K) and b:(B,K,N), got %s and %s" % (tuple(a.shape), tuple(b.shape)))
    if b.device != a.device:
        raise RuntimeError("a and b must be on the same device")
    if mode not in (0, 1, 2, 3):
        raise RuntimeError("unknown mode %r" % (mode,))
    B, M, K = a.shape
    N = b.shape[2]
    with torch.cuda.device(a.device):
        out = torch.empty((B, M, N), dtype=a.dtype, device=a.device)
        if mode == MODE_LOG:
            aux = torch.empty_like(out) if want_maxes else None
        else:
            aux = torch.empty((B, M, N), dtype=torch.int32, device=a.device)
        if mode == MODE_SAMPLE:
            if u is None:
                u = torch.rand((B, M, N), dtype=a.dtype, device=a.device)
            _check_input(u, "u", dt)
            if tuple(u.shape) != (B, M, N):
                raise RuntimeError("u must have shape %s" % ((B, M, N),))
        if dt == torch.float64:
            st = load().gbmm_dense_forward_f64(mode, _ptr(a), _ptr(b), _ptr(u) if mode == MODE_SAMPLE else None,
                                               _ptr(out), _ptr(aux), B, M, K, N, _stream(a.device))
            _check(st, "gbmm_dense_forward_f64")
            return [out, aux]
        if mode == MODE_SAMPLE and fast_log and K > 0:
            # the logsumexp from the factorised tensor-core forward, then only the inverse-CDF pass
            out = logbmm_fast_forward(a, b, tensor_cores=True)[0]
            st = load().gbmm_dense_sample_pick_f32(_ptr(a), _ptr(b), _ptr(u), _ptr(out), _ptr(aux), B, M, K, N,
                                                   _stream(a.device))
            _check(st, "gbmm_dense_sample_pick_f32")
            return [out, aux]
        nbytes = load().gbmm_dense_forward_workspace_bytes(mode, B, M, K, N)
        ws = torch.empty((nbytes,), dtype=torch.uint8, device=a.device) if nbytes > 0 else None
        st = load().gbmm_dense_forward_f32(mode, _ptr(a), _ptr(b), _ptr(u) if mode == MODE_SAMPLE else None,
                                           _ptr(out), _ptr(aux), B, M, K, N, _ptr(ws), nbytes, _stream(a.device))
    _check(st, "gbmm_dense_forward_f32")
    return [out, aux]


def backward(a, b, grad_output, part, maxes, mode):
    """`_genbmm.backward(a, b, grad_output, part, maxes, mode)` -> [grad_a, grad_b].

    mode 0: `part` is the forward output; `maxes` is accepted for signature compatibility and
    not read.  Modes 1-3: `part` holds the saved indices (int32, or the float copy the
    reference's Python passes, genmul.py:63).  Unlike the reference, mode 0 fills grad_b too.
    """
    dt = _compute_dtype(a)
    _check_input(a, "a", dt)
    _check_input(b, "b", dt)
    _check_input(grad_output, "grad_output", dt)
    B, M, K = a.shape
    N = b.shape[2]
    if tuple(grad_output.shape) != (B, M, N):
        raise RuntimeError("grad_output must have shape %s" % ((B, M, N),))
    with torch.cuda.device(a.device):
        if mode == MODE_LOG:
            _check_input(part, "part", dt)
            pf, aux = part, None
        else:
            if part.dtype != torch.int32:
                part = part.to(torch.int32)
            _check_input(part, "part", torch.int32)
            pf, aux = None, part
        if tuple(part.shape) != (B, M, N):
            raise RuntimeError("part must have shape %s" % ((B, M, N),))
        grad_a = torch.empty_like(a)
        grad_b = torch.empty_like(b)
        if dt == torch.float64:
            st = load().gbmm_dense_backward_f64(mode, _ptr(a), _ptr(b), _ptr(grad_output), _ptr(pf), _ptr(aux),
                                                _ptr(grad_a), _ptr(grad_b), B, M, K, N, _stream(a.device))
            _check(st, "gbmm_dense_backward_f64")
            return [grad_a, grad_b]
        st = load().gbmm_dense_backward_f32(mode, _ptr(a), _ptr(b), _ptr(grad_output), _ptr(pf), _ptr(aux),
                                            _ptr(grad_a), _ptr(grad_b), B, M, K, N, _stream(a.device))
    _check(st, "gbmm_dense_backward_f32")
    return [grad_a, grad_b]


def backbackward(a, b, grad_output, part, maxes, grad_out_a, mode=0, grad_out_b=None):
    """`_genbmm.backbackward(a, b, grad_output, part, maxes, grad_out_a, mode)` -> [grad_a, grad_b,
    grad_grad] for the log product (mode 0 only, as in the reference, matmul_cuda_kernel.cu:583).
    `grad_out_a` / `grad_out_b` are the cotangents of the first-order grad_a / grad_b (the reference
    has the first only); `maxes` is accepted for signature compatibility and not read."""
    if mode != MODE_LOG:
        raise RuntimeError("backbackward is defined for mode 0 (log) only")
    for x, name in ((a, "a"), (b, "b"), (grad_output, "grad_output"), (part, "part")):
        _check_input(x, name)
    B, M, K = a.shape
    N = b.shape[2]
    with torch.cuda.device(a.device):
        h_a = torch.zeros_like(a) if grad_out_a is None else grad_out_a.contiguous()
        h_b = torch.zeros_like(b) if grad_out_b is None else grad_out_b.contiguous()
        _check_input(h_a, "grad_out_a")
        _check_input(h_b, "grad_out_b")
        d_a, d_b, d_g = torch.empty_like(a), torch.empty_like(b), torch.empty_like(grad_output)
        if min(B, M, K, N) == 0:
            return [d_a.zero_(), d_b.zero_(), d_g.zero_()]
        st = load().gbmm_dense_backbackward_f32(_ptr(a), _ptr(b), _ptr(grad_output), _ptr(part), _ptr(h_a),
                                                _ptr(h_b), _ptr(d_a), _ptr(d_b), _ptr(d_g), B, M, K, N,
                                                _stream(a.device))
    _check(st, "gbmm_dense_backbackward_f32")
    return [d_a, d_b, d_g]


def _check_band(a, a_lu, a_lb, b, b_lu, b_lb):
    _check_input(a, "a", _compute_dtype(a))
    _check_input(b, "b", _compute_dtype(a))
    if a.dim() != 3 or b.dim() != 3 or a.shape[:2] != b.shape[:2]:
        raise RuntimeError("expected a:(B,n,Wa) and b:(B,n,Wb), got %s and %s" % (tuple(a.shape), tuple(b.shape)))
    if a.shape[2] != a_lu + a_lb + 1 or b.shape[2] != b_lu + b_lb + 1:
        raise RuntimeError("band widths do not match lu + ld + 1")
    if b.device != a.device:
        raise RuntimeError("a and b must be on the same device")


# Workspaces of the banded fast paths, kept between calls: their padding (zeros for the tensor-core path, -inf
# for the max-plus path) is written once, when a workspace is created; the library never rewrites it.
#
# One workspace per (device, stream, kind): a workspace is only ever touched by kernels of the stream it was
# created on, so two products on different streams never share scratch, and a workspace that is dropped goes
# back to the allocator pool of the stream that used it.  A workspace is replaced when the problem's dimensions
# change.  At most _WS_MAX of them are kept (the oldest is dropped); `release_workspaces()` drops all of them.
# cfg5-sized problems (32 x 8192, 129 diagonals) keep about 2.3 GB per stream this way.
_WS_MAX = 8
_ws_lock = threading.Lock()
_ws_cache = {}       # (kind, device index, stream handle) -> _Workspace, in order of last use


class _Workspace:
    """`generation` counts the calls that wrote operands into `buf`; `holds` is the banded mode whose forward
    wrote them last (None after a call that left them incomplete)."""
    __slots__ = ("dims", "buf", "generation", "holds")

    def __init__(self, dims, buf):
        self.dims, self.buf, self.generation, self.holds = dims, buf, 0, None


def release_workspaces(device=None):
    """Drop the cached workspaces of the banded fast paths (all devices, or one).  The memory returns to
    torch's allocator; the next banded call builds a new workspace."""
    with _ws_lock:
        for key in [k for k in _ws_cache if device is None or k[1] == torch.device(device).index]:
            del _ws_cache[key]


def _cached_workspace(kind, dims, need, device, init):
    dev = device.index if device.index is not None else torch.cuda.current_device()
    stream = _stream(device)
    key = (kind, dev, stream)
    with _ws_lock:
        hit = _ws_cache.pop(key, None)
        if hit is None or hit.dims != dims or hit.buf.numel() < need:
            hit = None
            buf = torch.empty((need,), dtype=torch.uint8, device=device)
            _check(init(_ptr(buf), buf.numel(), stream), "workspace init")
            hit = _Workspace(dims, buf)
        _ws_cache[key] = hit            # most recently used last
        while len(_ws_cache) > _WS_MAX:
            del _ws_cache[next(iter(_ws_cache))]
    return hit


def _band_tc_workspace(mode, backward, B, n, bands, device):
    """The cached workspace (_Workspace) for these dimensions on this device and stream, or None when the
    tensor-core path is not taken (GENBMM_B200_BAND=block keeps the FP32 block kernels, GENBMM_B200_BANDLOG=exact
    the direct ones).  A backward-sized workspace also serves the forward.
    For the ordinary (sum) semiring the 3xTF32 result is about 1.7 times further from the exact sum than the
    FP32 block kernel's, both a few units in the last place of the sum of the terms' magnitudes."""
    if os.environ.get("GENBMM_B200_BAND", "auto") == "block" or os.environ.get("GENBMM_B200_BANDLOG") == "exact":
        return None
    lib = load()
    need = lib.gbmm_band_tc_workspace_bytes(1 if backward else 0, B, n, *bands)
    return _cached_workspace("tc", (B, n) + tuple(bands), need, device, lib.gbmm_band_tc_workspace_init)


def _band_max_workspace(B, n, bands, device):
    """Cached workspace (a tensor) of the fast max-plus forward, or None when GENBMM_B200_BAND=block."""
    if os.environ.get("GENBMM_B200_BAND", "auto") == "block":
        return None
    lib = load()
    need = lib.gbmm_band_max_workspace_bytes(B, n, *bands)
    return _cached_workspace("max", (B, n) + tuple(bands), need, device, lib.gbmm_band_max_workspace_init).buf


class BandForwardToken:
    """What a banded tensor-core forward left in its workspace, for the backward of the same operands: the
    workspace and the value of its generation counter right after the forward.  The backward may reuse the
    forward's converted operands, row maxima and guard flags only while the counter still has that value, i.e.
    while no other call has written into that workspace."""
    __slots__ = ("ws", "generation", "mode")

    def __init__(self, ws, mode):
        self.ws, self.generation, self.mode = ws, ws.generation, mode

    def valid_for(self, ws, mode):
        return ws is self.ws and ws.generation == self.generation and ws.holds == mode and mode == self.mode


def _band_workspace(B, n, device):
    if os.environ.get("GENBMM_B200_BANDLOG", "auto") == "exact":
        return None
    return torch.empty((max(int(load().gbmm_band_workspace_bytes(B, n)), 256),), dtype=torch.uint8, device=device)


def forward_band(a, a_lu, a_lb, b, b_lu, b_lb, mode, want_maxes=False, want_token=False):
    """`_genbmm.forward_band(a, a_lu, a_lb, b, b_lu, b_lb, mode)` -> [out, indices, maxes].

    Only the outputs the mode defines are produced (the reference allocates and zero-fills all
    three every call, banded_cuda_kernel.cu:373-387); the others are returned as None, and the
    log mode's `maxes` only on request (the backward does not need it).
    want_token=True appends a BandForwardToken (or None when the tensor-core path was not taken) that
    `backward_band(reuse=...)` accepts.
    """
    _check_band(a, a_lu, a_lb, b, b_lu, b_lb)
    if mode not in (BAND_LOG, BAND_MAX, BAND_MUL):
        raise RuntimeError("unknown banded mode %r" % (mode,))
    B, n, Wa = a.shape
    Wo = Wa + b.shape[2] - 1
    token = None

    def result(out, idx, maxes):
        return [out, idx, maxes, token] if want_token else [out, idx, maxes]

    with torch.cuda.device(a.device):
        out = torch.empty((B, n, Wo), dtype=a.dtype, device=a.device)
        idx = torch.empty((B, n, Wo), dtype=torch.int32, device=a.device) if mode == BAND_MAX else None
        maxes = torch.empty_like(out) if (mode == BAND_LOG and want_maxes) else None
        bands = (a_lu, a_lb, b_lu, b_lb)
        if a.dtype == torch.float64:
            st = load().gbmm_band_forward_f64(mode, _ptr(a), a_lu, a_lb, _ptr(b), b_lu, b_lb, _ptr(out), _ptr(idx),
                                              _ptr(maxes), B, n, _stream(a.device))
            _check(st, "gbmm_band_forward_f64")
            return result(out, idx, maxes)
        if mode == BAND_MAX and load().gbmm_band_max_eligible(n, *bands):
            mx_ws = _band_max_workspace(B, n, bands, a.device)
            if mx_ws is not None:
                st = load().gbmm_band_max_forward_f32(_ptr(a), a_lu, a_lb, _ptr(b), b_lu, b_lb, _ptr(out), _ptr(idx),
                                                      B, n, _ptr(mx_ws), mx_ws.numel(), _stream(a.device))
                _check(st, "gbmm_band_max_forward_f32")
                return result(out, idx, maxes)
        tc = None
        if maxes is None and load().gbmm_band_tc_eligible(mode, n, *bands):
            tc = _band_tc_workspace(mode, False, B, n, bands, a.device)
        if tc is not None:
            tc.generation += 1
            tc.holds = None
            st = load().gbmm_band_tc_forward_f32(mode, _ptr(a), a_lu, a_lb, _ptr(b), b_lu, b_lb, _ptr(out), B, n,
                                                 _ptr(tc.buf), tc.buf.numel(), _stream(a.device))
            _check(st, "gbmm_band_tc_forward_f32")
            tc.holds = mode
            token = BandForwardToken(tc, mode)
            return result(out, idx, maxes)
        ws = _band_workspace(B, n, a.device) if mode == BAND_LOG else None
        st = load().gbmm_band_forward_f32(mode, _ptr(a), a_lu, a_lb, _ptr(b), b_lu, b_lb, _ptr(out), _ptr(idx),
                                          _ptr(maxes), B, n, _ptr(ws), 0 if ws is None else ws.numel(),
                                          _stream(a.device))
    _check(st, "gbmm_band_forward_f32")
    return result(out, idx, maxes)


def backward_band(a, a_lu, a_lb, b, b_lu, b_lb, grad_output, part, mode, both=False, reuse=None):
    """`_genbmm.backward_band(a, a_lu, a_lb, b, b_lu, b_lb, grad_output, part, mode)` -> [grad_a].

    With both=True returns [grad_a, grad_b], grad_b computed directly by a second kernel rather
    than by the reference's swap-and-transpose route (sparse.py:436-446).  `part` is the forward
    output (mode 0), the int32 or float indices in a's band coordinate (mode 1), ignored (mode 3).
    reuse = the BandForwardToken of the forward of these very operands (for callers that kept a and b alive
    and unmodified since, as autograd does): while no other call has written into that forward's workspace,
    its converted operands, row maxima and guard flags are reused instead of rebuilt.
    """
    _check_band(a, a_lu, a_lb, b, b_lu, b_lb)
    _check_input(grad_output, "grad_output", _compute_dtype(a))
    B, n, Wa = a.shape
    Wo = Wa + b.shape[2] - 1
    if tuple(grad_output.shape) != (B, n, Wo):
        raise RuntimeError("grad_output must have shape %s" % ((B, n, Wo),))
    with torch.cuda.device(a.device):
        if mode == BAND_MAX:
            if part.dtype != torch.int32:
                part = part.to(torch.int32)
            _check_input(part, "part", torch.int32)
        elif mode == BAND_LOG:
            _check_input(part, "part", _compute_dtype(a))
        else:
            part = None
        if part is not None and tuple(part.shape) != (B, n, Wo):
            raise RuntimeError("part must have shape %s" % ((B, n, Wo),))
        grad_a = torch.empty_like(a)
        grad_b = torch.empty_like(b) if both else None
        if a.dtype == torch.float64:
            st = load().gbmm_band_backward_f64(mode, _ptr(a), a_lu, a_lb, _ptr(b), b_lu, b_lb, _ptr(grad_output),
                                               _ptr(part), _ptr(grad_a), _ptr(grad_b), B, n, _stream(a.device))
            _check(st, "gbmm_band_backward_f64")
            return [grad_a, grad_b] if both else [grad_a]
        bands = (a_lu, a_lb, b_lu, b_lb)
        tc = None
        if load().gbmm_band_tc_eligible(mode, n, *bands):
            tc = _band_tc_workspace(mode, True, B, n, bands, a.device)
        if tc is not None:
            ready = 1 if (reuse is not None and reuse.valid_for(tc, mode)) else 0
            tc.generation += 1
            tc.holds = None
            st = load().gbmm_band_tc_backward_f32(mode, _ptr(a), a_lu, a_lb, _ptr(b), b_lu, b_lb, _ptr(grad_output),
                                                  _ptr(part), _ptr(grad_a), _ptr(grad_b), B, n, _ptr(tc.buf),
                                                  tc.buf.numel(), ready, _stream(a.device))
            _check(st, "gbmm_band_tc_backward_f32")
            return [grad_a, grad_b] if both else [grad_a]
        ws = _band_workspace(B, n, a.device) if mode == BAND_LOG else None
        st = load().gbmm_band_backward_f32(mode, _ptr(a), a_lu, a_lb, _ptr(b), b_lu, b_lb, _ptr(grad_output),
                                           _ptr(part), _ptr(grad_a), _ptr(grad_b), B, n, _ptr(ws),
                                           0 if ws is None else ws.numel(), _stream(a.device))
    _check(st, "gbmm_band_backward_f32")
    return [grad_a, grad_b] if both else [grad_a]


# ---- factorised fast path of logbmm -----------------------------------------------------------

def _workspace(nbytes, device):
    return torch.empty((max(int(nbytes), 256),), dtype=torch.uint8, device=device)


def logbmm_fast_forward(a, b, check=False, tensor_cores=False, keep_factors=False):
    """c = logbmm(a, b) by the factorised kernels.  Returns (out, rowmax, colmax, flags); the last
    three are what `logbmm_fast_backward` needs.  Requires K > 0.  tensor_cores=True runs the
    product as 3xTF32 on tcgen05 instead of the FP32 pipe.  keep_factors=True appends the
    workspace holding the split exponentiated operands (None on the FP32 pipe) for
    `logbmm_fast_backward(factors=...)`; it is four times the size of a and b."""
    _check_input(a, "a")
    _check_input(b, "b")
    if a.dim() != 3 or b.dim() != 3 or a.shape[0] != b.shape[0] or a.shape[2] != b.shape[1]:
        raise RuntimeError("expected a:(B,M,K) and b:(B,K,N), got %s and %s" % (tuple(a.shape), tuple(b.shape)))
    B, M, K = a.shape
    N = b.shape[2]
    lib = load()
    with torch.cuda.device(a.device):
        out = torch.empty((B, M, N), dtype=a.dtype, device=a.device)
        rowmax = torch.empty((B, M), dtype=a.dtype, device=a.device)
        colmax = torch.empty((B, N), dtype=a.dtype, device=a.device)
        flags = torch.empty((max(lib.gbmm_logbmm_flag_count(B, M, N), 1),), dtype=torch.int32, device=a.device)
        sizer = lib.gbmm_logbmm_tc_workspace_bytes if tensor_cores else lib.gbmm_logbmm_workspace_bytes
        fn = lib.gbmm_logbmm_tc_forward_f32 if tensor_cores else lib.gbmm_logbmm_forward_f32
        ws = _workspace(sizer(0, B, M, K, N), a.device)
        st = fn(_ptr(a), _ptr(b), _ptr(out), _ptr(rowmax), _ptr(colmax), _ptr(flags), _ptr(ws), ws.numel(), B, M,
                K, N, _stream(a.device))
        _check(st, "gbmm_logbmm_forward_f32")
        if check:
            _check(lib.gbmm_logbmm_check(_ptr(ws), _stream(a.device)), "gbmm_logbmm_forward_f32 (device)")
    if keep_factors:
        return out, rowmax, colmax, flags, (ws if tensor_cores else None)
    return out, rowmax, colmax, flags


def logbmm_fast_backward(a, b, grad_output, out, rowmax, colmax, flags, check=False, tensor_cores=False,
                         out_grads=None, factors=None):
    """(grad_a, grad_b) of logbmm by the factorised kernels, from what the fast forward saved.
    `out_grads` = (grad_a, grad_b) buffers to fill instead of allocating new ones; `factors` = the
    workspace `logbmm_fast_forward(keep_factors=True)` returned for the same a, b (tensor cores only)."""
    for x, name in ((a, "a"), (b, "b"), (grad_output, "grad_output"), (out, "out"), (rowmax, "rowmax"),
                    (colmax, "colmax")):
        _check_input(x, name)
    B, M, K = a.shape
    N = b.shape[2]
    lib = load()
    with torch.cuda.device(a.device):
        grad_a, grad_b = (torch.empty_like(a), torch.empty_like(b)) if out_grads is None else out_grads
        _check_input(grad_a, "grad_a")
        _check_input(grad_b, "grad_b")
        sizer = lib.gbmm_logbmm_tc_workspace_bytes if tensor_cores else lib.gbmm_logbmm_workspace_bytes
        fn = lib.gbmm_logbmm_tc_backward_f32 if tensor_cores else lib.gbmm_logbmm_backward_f32
        ws = _workspace(sizer(1, B, M, K, N), a.device)
        args = [_ptr(a), _ptr(b), _ptr(grad_output), _ptr(out), _ptr(rowmax), _ptr(colmax), _ptr(flags),
                _ptr(grad_a), _ptr(grad_b)]
        if tensor_cores:
            if factors is not None and (factors.device != a.device or
                                        factors.numel() < lib.gbmm_logbmm_tc_workspace_bytes(0, B, M, K, N)):
                raise RuntimeError("factors do not belong to a forward of these shapes on this device")
            args.append(None if factors is None else _ptr(factors))
        st = fn(*args, _ptr(ws), ws.numel(), B, M, K, N, _stream(a.device))
        _check(st, "gbmm_logbmm_backward_f32")
        if check:
            _check(lib.gbmm_logbmm_check(_ptr(ws), _stream(a.device)), "gbmm_logbmm_backward_f32 (device)")
    return grad_a, grad_b


def backbackward_band(a, a_lu, a_lb, b, b_lu, b_lb, grad_output, part, maxes, grad_out_a, mode=0, grad_out_b=None):
    """`_genbmm.backbackward_band(a, a_lu, a_lb, b, b_lu, b_lb, grad_output, part, maxes, grad_out_a,
    mode)` -> [grad_a, grad_b, grad_grad] for the banded log product (mode 0).  `grad_out_a` /
    `grad_out_b` are the cotangents of the first-order grad_a / grad_b; `maxes` is not read."""
    if mode != BAND_LOG:
        raise RuntimeError("backbackward_band is defined for mode 0 (log) only")
    _check_band(a, a_lu, a_lb, b, b_lu, b_lb)
    _check_input(grad_output, "grad_output")
    _check_input(part, "part")
    B, n, _ = a.shape
    with torch.cuda.device(a.device):
        h_a = torch.zeros_like(a) if grad_out_a is None else grad_out_a.contiguous()
        h_b = torch.zeros_like(b) if grad_out_b is None else grad_out_b.contiguous()
        _check_input(h_a, "grad_out_a")
        _check_input(h_b, "grad_out_b")
        d_a, d_b, d_g = torch.empty_like(a), torch.empty_like(b), torch.empty_like(grad_output)
        st = load().gbmm_band_backbackward_f32(_ptr(a), a_lu, a_lb, _ptr(b), b_lu, b_lb, _ptr(grad_output),
                                               _ptr(part), _ptr(h_a), _ptr(h_b), _ptr(d_a), _ptr(d_b), _ptr(d_g),
                                               B, n, _stream(a.device))
    _check(st, "gbmm_band_backbackward_f32")
    return [d_a, d_b, d_g]


def gather_blocks(src, index, elems, side=0):
    """dst block d <- src block index[d] (blocks of `elems` contiguous floats); index[d] < 0 gives the log
    semiring's identity matrix of side `side`.  `src` float32 contiguous on the GPU, `index` int64 on it."""
    _check_input(src, "src")
    _check_input(index, "index", torch.int64)
    if src.numel() % elems or elems % 4:
        raise RuntimeError("src must consist of whole blocks of a multiple of 4 elements")
    with torch.cuda.device(src.device):
        dst = torch.empty((index.numel(), elems), dtype=src.dtype, device=src.device)
        st = load().gbmm_gather_blocks_f32(_ptr(src), _ptr(dst), _ptr(index), index.numel(), elems, side,
                                           _stream(src.device))
    _check(st, "gbmm_gather_blocks_f32")
    return dst
