"""Build recipe of the CPU oracle (test infrastructure, not the product).

Compiles oracle/genbmm_oracle.c into oracle/_build/libgenbmm_oracle.so with the
first C compiler that accepts -fopenmp, else without OpenMP.
"""
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build", "libgenbmm_oracle.so")
SOURCES = [os.path.join(HERE, "genbmm_oracle.c"), os.path.join(HERE, "oracle_impl.h")]
CFLAGS = ["-O2", "-fPIC", "-fno-fast-math", "-ffp-contract=off", "-Wall"]


def _stale():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    return any(os.path.getmtime(s) > t for s in SOURCES)


def build(force=False):
    """Compile the oracle if it is missing or older than its sources; return its path."""
    if not force and not _stale():
        return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    compilers = [c for c in ("/usr/bin/gcc", shutil.which("gcc"), os.environ.get("CC"), shutil.which("cc")) if c]
    errors = []
    for omp in (["-fopenmp"], []):
        for cc in compilers:
            cmd = [cc, *CFLAGS, *omp, "-shared", "-o", OUT, SOURCES[0], "-lm"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode == 0:
                return OUT
            errors.append(" ".join(cmd) + "\n" + r.stderr[-400:])
    raise RuntimeError("could not compile the CPU oracle:\n" + "\n".join(errors))


if __name__ == "__main__":
    print(build(force=True))
