"""Generates tests/golden/genbmm_golden.npz from the reference's own Python code.

Run once, in a container that has the reference checkout (no GPU needed):

    python tests/golden/make_golden.py /path/to/genbmm

It imports the reference's `genbmm/sparse.py` (its CPU triple loops, band
constructors and transpose) and evaluates the dense broadcast-reduce
expressions the reference's README and tests use as the definition of
logbmm / maxbmm / prodmaxbmm, on small seeded inputs, and stores inputs and
outputs.  Dense and banded cases are computed in float64 (the reference code
run under torch.set_default_dtype(float64)) and, for the bit-exact max
semirings, in float32 on inputs that are multiples of 1/8.

The committed .npz is what the tests read; the reference checkout is never
needed at test time.
"""
import sys

import numpy as np
import torch

if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py /path/to/genbmm-checkout")
REF = sys.argv[1]
sys.path.insert(0, REF)
from genbmm.sparse import BandedMatrix, banddiag  # noqa: E402

OUT = {}


def put(name, t):
    OUT[name] = t.detach().cpu().numpy() if hasattr(t, "detach") else np.asarray(t)


def dense_cases():
    shapes = [(3, 7, 9, 8), (2, 6, 10, 6), (1, 1, 1, 1), (2, 5, 1, 3)]
    for ci, (B, M, K, N) in enumerate(shapes):
        gen = torch.Generator().manual_seed(100 + ci)
        # log semiring, float64: value, first and second order gradients (test_cuda.py:12-42)
        a = torch.rand(B, M, K, generator=gen, dtype=torch.float64).requires_grad_(True)
        b = torch.rand(B, K, N, generator=gen, dtype=torch.float64).requires_grad_(True)
        back = torch.rand(B, M, N, generator=gen, dtype=torch.float64).requires_grad_(True)
        h_a = torch.rand(B, M, K, generator=gen, dtype=torch.float64)
        h_b = torch.rand(B, K, N, generator=gen, dtype=torch.float64)
        c = (a[:, :, :, None] + b[:, None, :, :]).logsumexp(-2)
        g = torch.autograd.grad(c, (a, b), back, create_graph=True)
        hh = torch.autograd.grad((g[0], g[1]), (a, b, back), (h_a, h_b))
        # the reference's double-backward kernels only see the cotangent of grad_a
        # (genmul.py:18-24): store that term on its own as well
        c2 = (a[:, :, :, None] + b[:, None, :, :]).logsumexp(-2)
        g2 = torch.autograd.grad(c2, (a, b), back, create_graph=True)
        ha_only = torch.autograd.grad(g2[0], (a, b, back), h_a)
        pre = "dense%d_log_" % ci
        for k, v in dict(a=a, b=b, back=back, h_a=h_a, h_b=h_b, c=c, ga=g[0], gb=g[1], hh_a=hh[0], hh_b=hh[1],
                         hh_back=hh[2], ha_only_a=ha_only[0], ha_only_b=ha_only[1],
                         ha_only_back=ha_only[2]).items():
            put(pre + k, v)
        # max-plus / prod-max, float32 on multiples of 1/8 (ties on purpose)
        for op in ("max", "prodmax"):
            a = (torch.randn(B, M, K, generator=gen) * 8).round() / 8
            b = (torch.randn(B, K, N, generator=gen) * 8).round() / 8
            back = torch.rand(B, M, N, generator=gen)
            a.requires_grad_(True)
            b.requires_grad_(True)
            s = a.unsqueeze(-1) + b.unsqueeze(-3) if op == "max" else a.unsqueeze(-1) * b.unsqueeze(-3)
            c, idx = s.max(-2)
            # lowest k among the maxima, computed explicitly (not relying on torch.max's choice)
            ar = torch.arange(K).view(1, 1, K, 1)
            low = torch.where(s == c.unsqueeze(-2), ar, K).min(-2)[0]
            ga, gb = torch.autograd.grad(c, (a, b), back)
            pre = "dense%d_%s_" % (ci, op)
            for k, v in dict(a=a, b=b, back=back, c=c, idx_torch=idx.int(), idx_low=low.int(), ga=ga,
                             gb=gb).items():
                put(pre + k, v)


def band_of(x, lu, ld):
    return banddiag(x, lu, ld)[0].contiguous()


def banded_cases():
    cases = [(2, 5, 2, 1, 1, 2), (3, 8, 0, 3, 2, 0), (2, 6, 3, 3, 3, 3), (1, 4, 5, 4, 0, 0), (2, 9, 1, 1, 2, 2)]
    for ci, (B, n, alu, ald, blu, bld) in enumerate(cases):
        gen = torch.Generator().manual_seed(200 + ci)
        pre = "band%d_" % ci
        put(pre + "dims", np.array([B, n, alu, ald, blu, bld]))
        da = torch.rand(B, n, n, generator=gen)
        db = torch.rand(B, n, n, generator=gen)
        xa = band_of(da, alu, ald)
        xb = band_of(db, blu, bld)
        put(pre + "dense_a", da)
        put(pre + "a", xa)
        put(pre + "b", xb)
        put(pre + "a_T", BandedMatrix(xa, alu, ald).transpose().data)
        put(pre + "a_dense", BandedMatrix(xa, alu, ald).to_dense())
        olu, old = alu + bld, ald + blu
        gout = torch.rand(B, n, olu + old + 1, generator=gen)
        put(pre + "g", gout)
        for name, fill in (("mul", 0), ("log", 0), ("max", 0)):
            A = xa.clone().requires_grad_(True)
            Bm = xb.clone().requires_grad_(True)
            X, Y = BandedMatrix(A, alu, ald, fill), BandedMatrix(Bm, blu, bld, fill)
            fn = {"mul": X.multiply_simple, "log": X.multiply_log_simple, "max": X.multiply_max_simple}[name]
            R = fn(Y)
            assert (R.lu, R.ld) == (olu, old)
            # in-matrix mask: cells the loops wrote
            ga, gb = torch.autograd.grad(R.data, (A, Bm), gout.to(R.data.dtype))
            put(pre + name + "_out", R.data)
            put(pre + name + "_ga", ga)
            put(pre + name + "_gb", gb)
        X, Y = BandedMatrix(xa, alu, ald), BandedMatrix(xb, blu, bld)
        G = BandedMatrix(gout, olu, old)
        put(pre + "mul_back_simple", X.multiply_back_simple(Y, G).data)
        # second order of the log product (genbmm/test_cuda.py:113-143): gradient of
        # <grad_a, h_a> + <grad_b, h_b> w.r.t. (a, b, cotangent), by autograd through the loops
        A = xa.clone().requires_grad_(True)
        Bm = xb.clone().requires_grad_(True)
        go = gout.clone().requires_grad_(True)
        R = BandedMatrix(A, alu, ald, 0).multiply_log_simple(BandedMatrix(Bm, blu, bld, 0))
        ga, gb = torch.autograd.grad(R.data, (A, Bm), go, create_graph=True)
        ha = torch.rand(ga.shape, generator=gen)
        hb = torch.rand(gb.shape, generator=gen)
        hh = torch.autograd.grad((ga, gb), (A, Bm, go), (ha, hb))
        for k, v in dict(h_a=ha, h_b=hb, hh_a=hh[0], hh_b=hh[1], hh_g=hh[2]).items():
            put(pre + "log_" + k, v)


def main():
    torch.manual_seed(0)
    dense_cases()
    torch.set_default_dtype(torch.float64)
    banded_cases()
    torch.set_default_dtype(torch.float32)
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "genbmm_golden.npz")
    np.savez_compressed(path, **OUT)
    print(path, len(OUT), "arrays", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
