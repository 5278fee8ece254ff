"""In-tree build of the CUDA library: nvcc, sm_100a only.

    python -m genbmm_b200.build            # build if sources are newer than the library
    python -m genbmm_b200.build --force

Produces genbmm_b200/libgenbmm_b200.so, a plain C-ABI shared library (no torch, no Python
in it) whose entry points are declared in include/genbmm_b200.h.  The CUDA runtime is linked
statically so the library does not depend on which libcudart the host process loaded.
"""
import concurrent.futures
import contextlib
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "csrc", "_obj")
LIB = os.path.join(HERE, "libgenbmm_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math=false", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; genbmm_b200 needs the CUDA toolkit to build its sm_100a kernels")


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps():
    return sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h"))


def stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(s) > t for s in _deps())


def _compile(src):
    obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
    extra = os.environ.get("GENBMM_B200_NVCC_EXTRA", "").split()   # e.g. -DGBMM_BAND_BOX=64 (experiments)
    cmd = [_nvcc(), *[f for f in NVCC_FLAGS if f != "--use_fast_math=false"], *extra, "-I", INCLUDE, "-c", src,
           "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, " ".join(cmd), r.stdout + r.stderr))
    return obj, r.stderr


@contextlib.contextmanager
def _build_lock():
    """One builder at a time across processes (several ranks importing a stale tree at once): the others wait and
    then find the library up to date."""
    import fcntl
    with open(os.path.join(HERE, ".build.lock"), "w") as fh:
        fcntl.flock(fh, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(fh, fcntl.LOCK_UN)


def build(force=False, verbose=False):
    """Compile every .cu under csrc/ for sm_100a and link libgenbmm_b200.so.  Returns its path."""
    if not force and not stale():
        return LIB
    with _build_lock():
        if not force and not stale():
            return LIB
        return _build_locked(verbose)


def _build_locked(verbose):
    os.makedirs(OBJ, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        results = list(ex.map(_compile, sources()))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    tmp = "%s.tmp.%d" % (LIB, os.getpid())   # linked beside the library and renamed over it: never half written
    cmd = [_nvcc(), "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
           "-Xcompiler", "-fPIC", "-Xlinker", "--wrap=__cudaPushCallConfiguration", "-o", tmp, *objs]
    # --wrap: every kernel launch of the library goes through the counter in csrc/capi.cu (gbmm_launch_count)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (" ".join(cmd), r.stdout + r.stderr))
    os.replace(tmp, LIB)
    return LIB


SHIM_SRC = os.path.join(CSRC, "shim", "torch_shim.cpp")
SHIM = os.path.join(HERE, "_shim.so")


def shim_stale():
    if not os.path.exists(SHIM):
        return True
    t = os.path.getmtime(SHIM)
    return any(os.path.getmtime(s) > t for s in [SHIM_SRC] + glob.glob(os.path.join(INCLUDE, "*.h")))


def build_shim(force=False):
    """Compile csrc/shim/torch_shim.cpp (host C++ only: the PyTorch binding of the C ABI with the operators as
    C++ autograd functions) into genbmm_b200/_shim.so, linked against libgenbmm_b200.so beside it.  Built with
    the host compiler directly, in tree, so the module that is imported is the file that was built and nothing
    is compiled at import time.  Returns its path."""
    if not force and not shim_stale():
        return SHIM
    with _build_lock():
        if not force and not shim_stale():
            return SHIM
        return _build_shim_locked()


def _build_shim_locked():
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ext
    # the system compiler first: a module built by this image's /opt/gcc wrapper (what $CXX names here) crashed
    # when a C++ exception crossed it
    cxx = next((c for c in ("/usr/bin/g++", shutil.which("g++"), os.environ.get("CXX")) if c and os.path.exists(c)),
               None)
    if cxx is None:
        raise RuntimeError("no C++ compiler for the torch shim")
    cuda_home = os.path.dirname(os.path.dirname(_nvcc()))
    inc = ext.include_paths() + [sysconfig.get_paths()["include"], INCLUDE, os.path.join(cuda_home, "include")]
    libdirs = [os.path.join(os.path.dirname(torch.__file__), "lib"), os.path.join(cuda_home, "lib64")]
    tmp = "%s.tmp.%d" % (SHIM, os.getpid())
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-w",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI), "-DTORCH_EXTENSION_NAME=_shim",
           "-DTORCH_API_INCLUDE_EXTENSION_H", *["-I" + i for i in inc], SHIM_SRC, "-o", tmp,
           *["-L" + d for d in libdirs], "-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10_cuda",
           "-ltorch_cuda", "-lcudart", "-L" + HERE, "-l:libgenbmm_b200.so", "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("torch shim failed to build:\n%s\n%s" % (" ".join(cmd), (r.stdout + r.stderr)[-4000:]))
    os.replace(tmp, SHIM)
    return SHIM


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv or "--verbose" in sys.argv))
    print(build_shim(force="--force" in sys.argv))
