/*
 * TEST INFRASTRUCTURE — not part of the product.
 *
 * Body of the CPU oracle, included twice by genbmm_oracle.c: once with
 * REAL=float (the arithmetic the reference's CUDA kernels perform when given
 * fp32 tensors) and once with REAL=double (a higher-precision yardstick for
 * the tolerance-based comparisons).  Every function restates, loop for loop,
 * one kernel or Python routine of harvardnlp/genbmm; the file:line it follows
 * is given above each function (paths are relative to the genbmm project).
 *
 * Layout conventions (all row-major, contiguous):
 *   dense   a:(B,M,K)  b:(B,K,N)  out/aux/g:(B,M,N)
 *   banded  data:(B,n,W), W = lu+ld+1, data[b,i,j] = Dense[b, i+j-lu, i]
 */

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUF)

/* ------------------------------------------------------------------ dense */

/* matmul_cuda_kernel.cu:13-45 (mode 0, log), :47-75 (mode 1, max),
 * :77-121 (mode 2, sample), :124-152 (mode 3, prod-max).
 * `maxes` is written for mode 0, `idx` for modes 1-3.  For mode 2 the index
 * keeps the dispatcher's zero initial value (matmul_cuda_kernel.cu:516) when
 * no k passes the strict double inequality. */
void FN(orc_dense_fwd_)(int mode, const REAL *a, const REAL *b, const REAL *u,
                        REAL *out, REAL *maxes, int32_t *idx, int64_t B,
                        int64_t M, int64_t K, int64_t N) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t n = 0; n < B; ++n)
    for (int64_t row = 0; row < M; ++row) {
      const REAL *ar = a + (n * M + row) * K;
      const REAL *bn = b + n * K * N;
      for (int64_t col = 0; col < N; ++col) {
        const int64_t o = (n * M + row) * N + col;
        if (mode == 0 || mode == 2) {
          REAL val = 0, m = (REAL)-1e9;
          for (int64_t i = 0; i < K; ++i) {
            REAL v = ar[i] + bn[i * N + col];
            if (v > m) m = v;
          }
          for (int64_t i = 0; i < K; ++i) {
            REAL v = ar[i] + bn[i * N + col];
            val += EXP(v - m);
          }
          out[o] = LOG(val) + m;
          if (mode == 0) {
            if (maxes) maxes[o] = m;
          } else {
            REAL total = 0, r = u[o];
            int32_t pick = 0;
            for (int64_t i = 0; i < K; ++i) {
              REAL v = ar[i] + bn[i * N + col] - out[o];
              REAL e = EXP(v);
              if (total < r && total + e > r) {
                pick = (int32_t)i;
                break;
              }
              total += e;
            }
            idx[o] = pick;
          }
        } else {
          REAL m = (REAL)-1e9;
          int32_t ind = -1;
          for (int64_t i = 0; i < K; ++i) {
            REAL v = (mode == 1) ? ar[i] + bn[i * N + col]
                                 : ar[i] * bn[i * N + col];
            if (v > m) {
              m = v;
              ind = (int32_t)i;
            }
          }
          out[o] = m;
          idx[o] = ind;
        }
      }
    }
}

/* Distance of each uniform draw from the nearest step of the sampling CDF,
 * evaluated in double whatever REAL is.  Used by the tests to decide where a
 * sampled index is well defined: the fp32 running sum of
 * matmul_cuda_kernel.cu:109-118 depends on the last ulp of exp(), so two
 * correct implementations may pick neighbouring k when u sits on a step. */
void FN(orc_sample_margin_)(const REAL *a, const REAL *b, const REAL *u,
                            double *margin, int64_t B, int64_t M, int64_t K,
                            int64_t N) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t n = 0; n < B; ++n)
    for (int64_t row = 0; row < M; ++row)
      for (int64_t col = 0; col < N; ++col) {
        const REAL *ar = a + (n * M + row) * K;
        const REAL *bn = b + n * K * N;
        double m = -1e9, val = 0;
        for (int64_t i = 0; i < K; ++i) {
          double v = (double)ar[i] + (double)bn[i * N + col];
          if (v > m) m = v;
        }
        for (int64_t i = 0; i < K; ++i)
          val += exp((double)ar[i] + (double)bn[i * N + col] - m);
        double lse = log(val) + m, total = 0;
        double r = (double)u[(n * M + row) * N + col];
        double best = fabs(r);
        for (int64_t i = 0; i < K; ++i) {
          total += exp((double)ar[i] + (double)bn[i * N + col] - lse);
          double d = fabs(total - r);
          if (d < best) best = d;
        }
        margin[(n * M + row) * N + col] = best;
      }
}

/* matmul_cuda_kernel.cu:159-184 (log grad_a), :190-217 (log grad_b — the
 * kernel the Python side emulates with transposed copies, genmul.py:38-41),
 * :336-395 (max and sample routing), :399-456 (prod-max routing).
 * `part` is the forward output and `maxes` its shift for mode 0; `idx` the
 * saved int32 indices for modes 1-3.  Sums run in ascending n (grad_a) and
 * ascending m (grad_b), as in the kernels. */
void FN(orc_dense_bwd_)(int mode, const REAL *a, const REAL *b, const REAL *g,
                        const REAL *part, const REAL *maxes,
                        const int32_t *idx, REAL *dA, REAL *dB, int64_t B,
                        int64_t M, int64_t K, int64_t N) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t n = 0; n < B; ++n)
    for (int64_t row = 0; row < M; ++row)
      for (int64_t col = 0; col < K; ++col) {
        REAL val = 0;
        for (int64_t k = 0; k < N; ++k) {
          const int64_t o = (n * M + row) * N + k;
          if (mode == 0) {
            REAL m = maxes[o];
            val += (EXP(a[(n * M + row) * K + col] + b[(n * K + col) * N + k] -
                        m) /
                    EXP(part[o] - m)) *
                   g[o];
          } else if (mode == 3) {
            if ((REAL)col == (REAL)idx[o])
              val += b[(n * K + col) * N + k] * g[o];
          } else {
            if ((REAL)col == (REAL)idx[o]) val += g[o];
          }
        }
        dA[(n * M + row) * K + col] = val;
      }
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t n = 0; n < B; ++n)
    for (int64_t row = 0; row < K; ++row)
      for (int64_t col = 0; col < N; ++col) {
        REAL val = 0;
        for (int64_t k = 0; k < M; ++k) {
          const int64_t o = (n * M + k) * N + col;
          if (mode == 0) {
            REAL m = maxes[o];
            REAL v = EXP(a[(n * M + k) * K + row] + b[(n * K + row) * N + col] -
                         m);
            val += (v / EXP(part[o] - m)) * g[o];
          } else if (mode == 3) {
            if ((REAL)row == (REAL)idx[o])
              val += a[(n * M + k) * K + row] * g[o];
          } else {
            if ((REAL)row == (REAL)idx[o]) val += g[o];
          }
        }
        dB[(n * K + row) * N + col] = val;
      }
}

/* matmul_cuda_kernel.cu:220-258 (w.r.t. a), :261-303 (w.r.t. b), :305-331
 * (w.r.t. grad_out): second-order terms of the log product.  `h` is the
 * cotangent of grad_a (shape of a).  Complexity O(B*M*K*N*K), so only for
 * small cases. */
void FN(orc_dense_bwdbwd_)(const REAL *a, const REAL *b, const REAL *g,
                           const REAL *part, const REAL *maxes, const REAL *h,
                           REAL *dA, REAL *dB, REAL *dG, int64_t B, int64_t M,
                           int64_t K, int64_t N) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t n = 0; n < B; ++n)
    for (int64_t row = 0; row < M; ++row)
      for (int64_t col = 0; col < K; ++col) {
        REAL val = 0;
        for (int64_t k = 0; k < N; ++k) {
          const int64_t o = (n * M + row) * N + k;
          REAL m = maxes[o], z = EXP(part[o] - m);
          REAL s = EXP(a[(n * M + row) * K + col] + b[(n * K + col) * N + k] -
                       m) / z;
          REAL inner = 0;
          for (int64_t k2 = 0; k2 < K; ++k2) {
            REAL s2 = EXP(a[(n * M + row) * K + k2] +
                          b[(n * K + k2) * N + k] - m) / z;
            REAL v = (col == k2) ? s - s * s2 : -s * s2;
            inner += v * h[(n * M + row) * K + k2];
          }
          val += inner * g[o];
        }
        dA[(n * M + row) * K + col] = val;
      }
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t n = 0; n < B; ++n)
    for (int64_t row = 0; row < K; ++row)
      for (int64_t col = 0; col < N; ++col) {
        REAL val = 0;
        for (int64_t k = 0; k < M; ++k) {
          const int64_t o = (n * M + k) * N + col;
          REAL m = maxes[o], z = EXP(part[o] - m);
          REAL s = EXP(a[(n * M + k) * K + row] + b[(n * K + row) * N + col] -
                       m) / z;
          REAL inner = 0;
          for (int64_t k2 = 0; k2 < K; ++k2) {
            REAL s2 = EXP(a[(n * M + k) * K + k2] +
                          b[(n * K + k2) * N + col] - m) / z;
            REAL v = (row == k2) ? s - s * s2 : -s * s2;
            inner += v * h[(n * M + k) * K + k2];
          }
          val += inner * g[o];
        }
        dB[(n * K + row) * N + col] = val;
      }
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t n = 0; n < B; ++n)
    for (int64_t row = 0; row < M; ++row)
      for (int64_t col = 0; col < N; ++col) {
        const int64_t o = (n * M + row) * N + col;
        REAL val = 0, m = maxes[o];
        for (int64_t k = 0; k < K; ++k)
          val += (EXP(a[(n * M + row) * K + k] + b[(n * K + k) * N + col] - m) /
                  EXP(part[o] - m)) *
                 h[(n * M + row) * K + k];
        dG[o] = val;
      }
}

/* ----------------------------------------------------------------- banded */

/* banded_cuda_kernel.cu:13-100.  mode 0 log (out, maxes), 1 max (out, idx),
 * 3 ordinary product (out).  Cells whose dense column o lies outside [0,n)
 * are left untouched; the caller zero-fills the outputs first, as the
 * dispatcher does (banded_cuda_kernel.cu:373-387).  The same loops are the
 * CPU routines sparse.py:268-294 (mul), :296-323 (max), :325-363 (log). */
void FN(orc_band_fwd_)(int mode, const REAL *a, int a_lu, int a_ld,
                       const REAL *b, int b_lu, int b_ld, REAL *out,
                       int32_t *idx, REAL *maxes, int64_t B, int64_t n) {
  const int Wa = a_lu + a_ld + 1, Wb = b_lu + b_ld + 1;
  const int r_lu = a_lu + b_ld, r_ld = a_ld + b_lu, Wo = r_lu + r_ld + 1;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bt = 0; bt < B; ++bt)
    for (int64_t i = 0; i < n; ++i)
      for (int j = 0; j < Wo; ++j) {
        const int64_t o = i + (j - r_lu);
        if (o < 0 || o >= n) continue;
        const REAL *ai = a + (bt * n + i) * Wa;
        const REAL *bo = b + (bt * n + o) * Wb;
        const int64_t oi = (bt * n + i) * Wo + j;
        if (mode == 1) {
          REAL m = (REAL)-1e9;
          int32_t ind = -1;
          for (int k = 0; k < Wa; ++k) {
            int64_t pos = i + (k - a_lu);
            int64_t k2 = (pos - o) + b_lu;
            if (k2 < 0 || k2 >= Wb) continue;
            if (pos < 0 || pos >= n) continue;
            REAL v = ai[k] + bo[k2];
            if (v > m) {
              m = v;
              ind = k;
            }
          }
          out[oi] = m;
          idx[oi] = ind;
        } else if (mode == 3) {
          REAL val = 0;
          for (int k = 0; k < Wa; ++k) {
            int64_t pos = i + (k - a_lu);
            int64_t k2 = (pos - o) + b_lu;
            if (k2 < 0 || k2 >= Wb) continue;
            if (pos < 0 || pos >= n) continue;
            val += ai[k] * bo[k2];
          }
          out[oi] = val;
        } else if (mode == 0) {
          REAL val = 0, m = (REAL)-1e9;
          for (int k = 0; k < Wa; ++k) {
            int64_t pos = i + (k - a_lu);
            if (pos < 0 || pos >= n) continue;
            int64_t k2 = (pos - o) + b_lu;
            if (k2 < 0 || k2 >= Wb) continue;
            REAL v = ai[k] + bo[k2];
            if (v > m) m = v;
          }
          for (int k = 0; k < Wa; ++k) {
            int64_t pos = i + (k - a_lu);
            if (pos < 0 || pos >= n) continue;
            int64_t k2 = (pos - o) + b_lu;
            if (k2 < 0 || k2 >= Wb) continue;
            val += EXP(ai[k] + bo[k2] - m);
          }
          out[oi] = LOG(val) + m;
          if (maxes) maxes[oi] = m;
        }
      }
}

/* banded_cuda_kernel.cu:104-152: gradient w.r.t. the first operand only.
 * `part` is the forward output for mode 0 and the float-cast argmax index
 * for mode 1 (sparse.py:610); unused for mode 3.  Cells whose dense column
 * lies outside [0,n) are left untouched (zero-filled by the caller). */
void FN(orc_band_bwd_)(int mode, const REAL *a, int a_lu, int a_ld,
                       const REAL *b, int b_lu, int b_ld, const REAL *g,
                       const REAL *part, REAL *dA, int64_t B, int64_t n) {
  const int Wa = a_lu + a_ld + 1, Wb = b_lu + b_ld + 1;
  const int r_lu = a_lu + b_ld, r_ld = a_ld + b_lu, Wo = r_lu + r_ld + 1;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bt = 0; bt < B; ++bt)
    for (int64_t i = 0; i < n; ++i)
      for (int j = 0; j < Wa; ++j) {
        const int64_t o = i + (j - a_lu);
        if (o < 0 || o >= n) continue;
        REAL val = 0;
        for (int k = 0; k < Wo; ++k) {
          const int64_t pos = i + (k - r_lu);
          const int64_t k2 = (o - pos) + b_lu;
          if (k2 < 0 || k2 >= Wb) continue;
          if (pos < 0 || pos >= n) continue;
          const int64_t gi = (bt * n + i) * Wo + k;
          if (mode == 3) {
            val += b[(bt * n + pos) * Wb + k2] * g[gi];
          } else if (mode == 1) {
            REAL v = ((REAL)j == part[gi]) ? 1 : 0;
            val += v * g[gi];
          } else if (mode == 0) {
            REAL v = a[(bt * n + i) * Wa + j] + b[(bt * n + pos) * Wb + k2] -
                     part[gi];
            val += EXP(v) * g[gi];
          }
        }
        dA[(bt * n + i) * Wa + j] = val;
      }
}

/* banded_cuda_kernel.cu:154-350 (kernels A, B, C): second-order terms of the
 * log product.  The reference differentiates grad_a only and contracts with
 * its cotangent h_a[i][m]; here the contracted value of an inner triple is
 * h_a[i][m] + h_b[o2][m2], which also covers the cotangent of grad_b (h_b all
 * zero gives the reference's three outputs exactly).  The reference's
 * exp(x - mx) / exp(part - mx) is written exp(x - part). */
void FN(orc_band_bwdbwd_)(const REAL *a, int a_lu, int a_ld, const REAL *b,
                          int b_lu, int b_ld, const REAL *g, const REAL *part,
                          const REAL *ha, const REAL *hb, REAL *dA, REAL *dB,
                          REAL *dG, int64_t B, int64_t n) {
  const int Wa = a_lu + a_ld + 1, Wb = b_lu + b_ld + 1;
  const int r_lu = a_lu + b_ld, r_ld = a_ld + b_lu, Wo = r_lu + r_ld + 1;
#define INNER_(i_, k_, jsel_, s_, res_)                                       \
  do {                                                                        \
    const int64_t o2_ = (i_) + ((k_) - r_lu);                                 \
    REAL inner_ = 0;                                                          \
    for (int m = 0; m < Wa; ++m) {                                            \
      const int64_t pin_ = (i_) + (m - a_lu), m2_ = (pin_ - o2_) + b_lu;      \
      if (m2_ < 0 || m2_ >= Wb || pin_ < 0 || pin_ >= n) continue;            \
      REAL s2_ = EXP(a[(bt * n + (i_)) * Wa + m] +                            \
                     b[(bt * n + o2_) * Wb + m2_] -                           \
                     part[(bt * n + (i_)) * Wo + (k_)]);                      \
      REAL v_ = ((jsel_) == m) ? (s_) - (s_) * s2_ : -(s_) * s2_;             \
      inner_ += v_ * (ha[(bt * n + (i_)) * Wa + m] +                          \
                      hb[(bt * n + o2_) * Wb + m2_]);                         \
    }                                                                         \
    res_ = inner_;                                                            \
  } while (0)
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bt = 0; bt < B; ++bt)
    for (int64_t i = 0; i < n; ++i)
      for (int j = 0; j < Wa; ++j) { /* kernel A */
        const int64_t o = i + (j - a_lu);
        if (o < 0 || o >= n) continue;
        REAL val = 0;
        for (int k = 0; k < Wo; ++k) {
          const int64_t pos = i + (k - r_lu), k2 = (o - pos) + b_lu;
          if (k2 < 0 || k2 >= Wb || pos < 0 || pos >= n) continue;
          REAL s = EXP(a[(bt * n + i) * Wa + j] + b[(bt * n + pos) * Wb + k2] -
                       part[(bt * n + i) * Wo + k]);
          REAL inner;
          INNER_(i, k, j, s, inner);
          val += inner * g[(bt * n + i) * Wo + k];
        }
        dA[(bt * n + i) * Wa + j] = val;
      }
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bt = 0; bt < B; ++bt)
    for (int64_t pos = 0; pos < n; ++pos)
      for (int k2 = 0; k2 < Wb; ++k2) { /* kernel B */
        const int64_t check = pos + (k2 - b_lu);
        if (check < 0 || check >= n) continue;
        REAL val = 0;
        for (int k = 0; k < Wo; ++k) {
          const int64_t i = pos - (k - r_lu);
          const int64_t j = k2 + pos - b_lu - (i - a_lu);
          if (j < 0 || j >= Wa || i < 0 || i >= n) continue;
          REAL s = EXP(a[(bt * n + i) * Wa + j] + b[(bt * n + pos) * Wb + k2] -
                       part[(bt * n + i) * Wo + k]);
          REAL inner;
          INNER_(i, k, (int)j, s, inner);
          val += inner * g[(bt * n + i) * Wo + k];
        }
        dB[(bt * n + pos) * Wb + k2] = val;
      }
#undef INNER_
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bt = 0; bt < B; ++bt)
    for (int64_t i = 0; i < n; ++i)
      for (int j = 0; j < Wo; ++j) { /* kernel C */
        const int64_t o = i + (j - r_lu);
        if (o < 0 || o >= n) continue;
        REAL val = 0;
        for (int k = 0; k < Wa; ++k) {
          const int64_t pos = i + (k - a_lu), k2 = (pos - o) + b_lu;
          if (k2 < 0 || k2 >= Wb || pos < 0 || pos >= n) continue;
          val += EXP(a[(bt * n + i) * Wa + k] + b[(bt * n + o) * Wb + k2] -
                     part[(bt * n + i) * Wo + j]) *
                 (ha[(bt * n + i) * Wa + k] + hb[(bt * n + o) * Wb + k2]);
        }
        dG[(bt * n + i) * Wo + j] = val;
      }
}

/* sparse.py:33-47 with :65-70 — BandedMatrix.transpose() as
 * repdiag(data.flip(-1), lu, ld): out[i,j] = data[i+j-ld, lu+ld-j], zero
 * where the source row is outside [0,n).  The result has (lu,ld) swapped. */
void FN(orc_band_transpose_)(const REAL *x, int lu, int ld, REAL *out,
                             int64_t B, int64_t n) {
  const int W = lu + ld + 1;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bt = 0; bt < B; ++bt)
    for (int64_t i = 0; i < n; ++i)
      for (int j = 0; j < W; ++j) {
        const int64_t src = i + j - ld;
        out[(bt * n + i) * W + j] =
            (src < 0 || src >= n) ? (REAL)0
                                  : x[(bt * n + src) * W + (lu + ld - j)];
      }
}

#undef FN
#undef CAT
#undef CAT_
