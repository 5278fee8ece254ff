/*
 * TEST INFRASTRUCTURE — not part of the product.
 *
 * CPU oracle for the semiring batched matrix products of harvardnlp/genbmm:
 * a plain-C restatement of the reference's CUDA kernels and Python loops,
 * compiled once for float and once for double (see oracle_impl.h for the
 * per-function citations).  Only the test-suite, the smoke check and the CPU
 * baseline leg of the benchmark may load this library; the product never does.
 *
 * Pinning: the reference ships no golden vectors.  This oracle is pinned to
 * outputs of the reference's own Python code (genbmm/sparse.py loops and the
 * dense broadcast expressions its tests compare against) through the
 * fixtures under tests/golden/, produced by tests/golden/make_golden.py.
 */
#include <math.h>
#include <stdint.h>

#define REAL float
#define SUF f32
#define EXP expf
#define LOG logf
#include "oracle_impl.h"
#undef REAL
#undef SUF
#undef EXP
#undef LOG

#define REAL double
#define SUF f64
#define EXP exp
#define LOG log
#include "oracle_impl.h"
#undef REAL
#undef SUF
#undef EXP
#undef LOG

int orc_abi_version(void) { return 1; }
