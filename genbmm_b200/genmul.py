"""Dense semiring batched matrix products as torch.autograd.Functions.

Same public names and call shapes as the reference's genbmm/genmul.py:100-103:
`logbmm(a, b)`, `maxbmm(a, b)`, `samplebmm(a, b)`, `prodmaxbmm(a, b)` on 3-D CUDA tensors
a:(B,M,K), b:(B,K,N), each returning c:(B,M,N) of a's dtype.  Additive: `samplebmm` takes
an optional third argument, the uniforms that drive the sample.

The public names are bound to the compiled PyTorch binding (genbmm_b200/_shim.so, C++ autograd functions)
when it is built, else to the Python autograd Functions of this file over the ctypes binding; both call the
same C-ABI entry points.

Differences from the reference that a caller can observe:
  * the logbmm backward makes no transposed copies (genmul.py:38-41 makes six);
  * half / bfloat16 inputs are computed in float32 and cast back; float64 runs float64 kernels of its own
    (plain tiled ones: a checking path, not a fast one);
  * inputs must be contiguous CUDA tensors, as in the reference (matmul_cuda.cpp:65-67).
"""
import os

import torch

from . import _native


def trans(s):
    return s.transpose(-2, -1).contiguous()


def _as_f32(x, name):
    """The tensor the kernels compute on: float32 and float64 as they are, half and bfloat16 widened to
    float32 (results are cast back to the input's dtype)."""
    if x.dtype in (torch.float32, torch.float64):
        return x
    if x.dtype in (torch.float16, torch.bfloat16):
        return x.float()
    raise RuntimeError("%s: dtype %s is not supported" % (name, x.dtype))


def _log_path(M, K, N):
    """Which kernels logbmm uses: "exact" (SFU, one exponential per term), "fp32" (factorised
    products on the FP32 pipe) or "tensor" (factorised products as 3xTF32 on tcgen05).  The
    factorised paths pay off once the product amortises their preparation kernels; the tensor
    cores are the default for those.  GENBMM_B200_LOGBMM=exact|fp32|tensor overrides the rule."""
    mode = os.environ.get("GENBMM_B200_LOGBMM", "auto")
    if K == 0 or M == 0 or N == 0 or mode == "exact":
        return "exact"
    if mode in ("fp32", "fast"):
        return "fp32"
    if mode == "tensor":
        return "tensor"
    return "tensor" if M * K * N >= 128 * 128 * 64 else "exact"


def _keep_factors(a, b):
    """Whether the tensor-core forward's split exponentiated operands (four times the bytes of a and b) stay
    alive until the backward, which then does not rebuild them (two HBM-bound passes saved).  The reference
    saves only a, b, out and maxes, and a chain of products keeps one such set per product alive, so large ones
    are kept only while the device has room for them several times over.
    GENBMM_B200_KEEP_FACTORS=1 always keeps them, =0 never does."""
    mode = os.environ.get("GENBMM_B200_KEEP_FACTORS", "auto")
    if mode in ("0", "1"):
        return mode == "1"
    nbytes = 4 * (a.numel() + b.numel()) * 4
    if nbytes <= (1 << 30):
        return True
    free, _ = torch.cuda.mem_get_info(a.device)
    return free >= 4 * nbytes


class LogMatMulBack(torch.autograd.Function):
    """First-order gradients of logbmm as a differentiable node (genmul.py:11-24).

    forward returns (grad_a, grad_b) in one call.  `aux` is None after the exact forward, or
    (rowmax, colmax, flags, tensor_cores, factors) of the factorised forward.
    """

    @staticmethod
    def forward(ctx, a, b, grad_out, part, aux):
        ctx.save_for_backward(a, b, grad_out, part)
        if aux is None:
            grad_a, grad_b = _native.backward(a, b, grad_out, part, None, _native.MODE_LOG)
        else:
            grad_a, grad_b = _native.logbmm_fast_backward(a, b, grad_out, part, *aux[:3], tensor_cores=aux[3],
                                                          factors=aux[4])
        return grad_a, grad_b

    @staticmethod
    def backward(ctx, h_a, h_b):
        a, b, grad_out, part = ctx.saved_tensors
        if a.dtype == torch.float64:
            raise RuntimeError("logbmm: second-order gradients are implemented for float32 inputs only")
        d_a, d_b, d_g = _native.backbackward(a, b, grad_out, part, None,
                                             None if h_a is None else h_a.float(), 0,
                                             None if h_b is None else h_b.float())
        return d_a, d_b, d_g, None, None


class LogMatMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        a32, b32 = _as_f32(a, "a"), _as_f32(b, "b")
        ctx.aux = None
        path = _log_path(a32.shape[1], a32.shape[2], b32.shape[-1]) if a32.dim() == 3 and b32.dim() == 3 else "exact"
        if a32.dtype == torch.float64:
            path = "exact"  # the factorised paths are float32 kernels
        if path != "exact":
            tc = path == "tensor"
            keep = tc and _keep_factors(a32, b32)
            out, rowmax, colmax, flags, factors = _native.logbmm_fast_forward(a32, b32, tensor_cores=tc,
                                                                              keep_factors=True)
            ctx.aux = (rowmax, colmax, flags, tc, factors if keep else None)
        else:
            out, _ = _native.forward(a32, b32, _native.MODE_LOG, want_maxes=False)
        ctx.save_for_backward(a32, b32, out)
        ctx.dtypes = (a.dtype, b.dtype)
        return out.to(a.dtype)

    @staticmethod
    def backward(ctx, grad_output):
        a, b, out = ctx.saved_tensors
        grad_a, grad_b = LogMatMulBack.apply(a, b, grad_output.contiguous().to(a.dtype), out, ctx.aux)
        return grad_a.to(ctx.dtypes[0]), grad_b.to(ctx.dtypes[1])


class _IndexRouted(torch.autograd.Function):
    """Shared shape of the three index-routed products (genmul.py:50-97)."""

    MODE = None

    @classmethod
    def _forward(cls, ctx, a, b, u=None):
        a32, b32 = _as_f32(a, "a"), _as_f32(b, "b")
        fast = (cls.MODE == _native.MODE_SAMPLE and a32.dtype == torch.float32 and a32.dim() == 3 and b32.dim() == 3
                and _log_path(a32.shape[1], a32.shape[2], b32.shape[-1]) == "tensor")
        out, switches = _native.forward(a32, b32, cls.MODE, u, fast_log=fast)
        ctx.save_for_backward(a32, b32, switches)
        ctx.dtypes = (a.dtype, b.dtype)
        return out.to(a.dtype)

    @classmethod
    def _backward(cls, ctx, grad_output):
        a, b, switches = ctx.saved_tensors
        grad_a, grad_b = _native.backward(a, b, grad_output.contiguous().to(a.dtype), switches, switches, cls.MODE)
        return grad_a.to(ctx.dtypes[0]), grad_b.to(ctx.dtypes[1])


class MaxMatMul(_IndexRouted):
    MODE = _native.MODE_MAX

    @staticmethod
    def forward(ctx, a, b):
        return MaxMatMul._forward(ctx, a, b)

    @staticmethod
    def backward(ctx, grad_output):
        return MaxMatMul._backward(ctx, grad_output)


class SampleMatMul(_IndexRouted):
    MODE = _native.MODE_SAMPLE

    @staticmethod
    def forward(ctx, a, b, u=None):
        return SampleMatMul._forward(ctx, a, b, u)

    @staticmethod
    def backward(ctx, grad_output):
        return SampleMatMul._backward(ctx, grad_output) + (None,)


class ProdMaxMatMul(_IndexRouted):
    MODE = _native.MODE_PRODMAX

    @staticmethod
    def forward(ctx, a, b):
        return ProdMaxMatMul._forward(ctx, a, b)

    @staticmethod
    def backward(ctx, grad_output):
        return ProdMaxMatMul._backward(ctx, grad_output)


def _load_shim():
    """The compiled PyTorch binding (csrc/shim/torch_shim.cpp: the same four operators as C++ autograd
    functions over the same C ABI), or None when it is not built or GENBMM_B200_BINDING=ctypes asks for the
    Python autograd Functions above.  Both bindings run the same kernels and give the same bits; the compiled
    one costs a fraction of the host time per call."""
    if os.environ.get("GENBMM_B200_BINDING", "shim") == "ctypes":
        return None
    from . import build as _build
    try:
        if not os.path.exists(_build.SHIM):
            _build.build_shim()
        from . import _shim
        if _shim.abi_version() != _native.load().gbmm_abi_version():
            return None
        return _shim
    except Exception:  # no host compiler, or a torch whose ABI the module was not built for
        return None


_shim = _load_shim()

if _shim is not None:
    logbmm = _shim.logbmm
    maxbmm = _shim.maxbmm
    prodmaxbmm = _shim.prodmaxbmm
else:
    logbmm = LogMatMul.apply
    maxbmm = MaxMatMul.apply
    prodmaxbmm = ProdMaxMatMul.apply


def samplebmm(a, b, u=None):
    """log-sum-exp value whose gradient is a one-hot sample from softmax_k(a+b).

    `u`:(B,M,N) uniforms in [0,1) select the sample; omitted, they are drawn on the device.
    """
    if _shim is not None:
        return _shim.samplebmm(a, b, u)
    return SampleMatMul.apply(a, b, u)
