"""Builds the reference's own CUDA extension for sm_100a into baseline/_ref/ (git-ignored).

    python baseline/build_ref.py [path to the genbmm checkout]

Without an argument the checkout is taken from $GENBMM_REFERENCE, else from a directory named `reference` beside
this repository.

This is the second baseline of bench.py (`--impl reference-cuda`): harvardnlp/genbmm's kernels, unchanged,
recompiled for the B200, so that a speed-up can be quoted against the code this package replaces on the
same GPU and not only against a CPU.  Nothing under baseline/_ref is imported by the package.

The checkout is copied to a scratch directory and built there (the checkout itself is never written).
Two mechanical edits make it compile against current PyTorch and without a GPU in the build container:
  * `AT_DISPATCH_FLOATING_TYPES[_AND_HALF](x.type(), ...)` -> `x.scalar_type()` (the macro no longer accepts
    the deprecated type object), and `x.type().is_cuda()` -> `x.is_cuda()`;
  * setup.py builds the extension even when torch.cuda.is_available() is false at build time.
No kernel, launch configuration or Python file of the reference is touched.
"""
import glob
import os
import re
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def default_checkout():
    return os.environ.get("GENBMM_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(src=None):
    src = src or default_checkout()
    if not os.path.isdir(src):
        raise RuntimeError("reference checkout not found at %s" % src)
    work = tempfile.mkdtemp(prefix="genbmm_ref_")
    tree = os.path.join(work, "genbmm_src")
    shutil.copytree(src, tree)
    for name in ("matmul_cuda_kernel.cu", "banded_cuda_kernel.cu", "matmul_cuda.cpp"):
        path = os.path.join(tree, name)
        text = open(path).read()
        text = re.sub(r"(AT_DISPATCH_[A-Z_]+\(\s*\w+)\.type\(\)", r"\1.scalar_type()", text)
        text = text.replace(".type().is_cuda()", ".is_cuda()")
        open(path, "w").write(text)
    setup = os.path.join(tree, "setup.py")
    text = open(setup).read().replace("if torch.cuda.is_available():", "if True:")
    open(setup, "w").write(text)
    env = dict(os.environ, TORCH_CUDA_ARCH_LIST="10.0a", MAX_JOBS="4")
    subprocess.run([sys.executable, "setup.py", "build_ext", "--inplace"], cwd=tree, env=env, check=True)
    so = glob.glob(os.path.join(tree, "_genbmm*.so"))
    if not so:
        raise RuntimeError("the extension was not produced")
    os.makedirs(OUT, exist_ok=True)
    shutil.copy2(so[0], OUT)
    dst = os.path.join(OUT, "genbmm")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    shutil.copytree(os.path.join(tree, "genbmm"), dst)
    shutil.rmtree(work, ignore_errors=True)
    return OUT


if __name__ == "__main__":
    print(build(*(sys.argv[1:2])))
