// Double-precision versions of the operators (the reference dispatches its kernels over
// float, double and half: matmul_cuda_kernel.cu:489, banded_cuda_kernel.cu:389).  These are plain
// shared-memory tiled kernels, one result per thread: B200's FP64 rate is a small fraction of its FP32
// rate, and the reference's users reach for double to check gradients, not for throughput.
// Semantics are the reference's, statement for statement: running maximum from -1e9, strict `>`
// (lowest k on ties, index -1 when nothing exceeds -1e9), the sample's strict double inequality on an
// ascending running sum with default index 0, out-of-matrix band cells 0.
#include "band.cuh"
#include "genbmm_b200.h"

namespace gbmm {
namespace {

constexpr int T = 16;
constexpr double kFloorD = -1e9;

__device__ __forceinline__ double dadd(double x, double y) { return __dadd_rn(x, y); }
__device__ __forceinline__ double dmul(double x, double y) { return __dmul_rn(x, y); }

// ---- dense forward ----------------------------------------------------------------------------
// mode 0 log (aux = maxes or null), 1 max, 2 sample (u), 3 prod-max; aux = int32 indices for 1..3
template <int MODE>
__global__ void __launch_bounds__(T * T) dense_fwd_f64(const double* __restrict__ a, const double* __restrict__ b,
                                                       const double* __restrict__ u, double* __restrict__ out,
                                                       void* __restrict__ aux, int M, int K, int N, int tiles_m,
                                                       int tiles_n) {
  __shared__ double sa[T][T + 1], sb[T][T + 1];
  const int tx = threadIdx.x % T, ty = threadIdx.x / T;
  const int64_t id = blockIdx.x;
  const int n0 = (int)(id % tiles_n) * T, m0 = (int)((id / tiles_n) % tiles_m) * T;
  const int64_t bt = id / ((int64_t)tiles_n * tiles_m);
  const double* ab = a + bt * M * K;
  const double* bb = b + bt * K * N;
  const int m = m0 + ty, n = n0 + tx;
  double mx = kFloorD, s = 0.0;
  int ind = (MODE == 2) ? 0 : -1;
  auto load = [&](int k0) {
    sa[ty][tx] = (m < M && k0 + tx < K) ? ab[(int64_t)m * K + k0 + tx] : 0.0;
    sb[ty][tx] = (k0 + ty < K && n < N) ? bb[(int64_t)(k0 + ty) * N + n] : 0.0;
  };
  for (int k0 = 0; k0 < K; k0 += T) {
    load(k0);
    __syncthreads();
    const int kend = min(T, K - k0);
    for (int kk = 0; kk < kend; ++kk) {
      const double v = MODE == 3 ? dmul(sa[ty][kk], sb[kk][tx]) : dadd(sa[ty][kk], sb[kk][tx]);
      if (MODE == 1 || MODE == 3) {
        if (v > mx) {
          mx = v;
          ind = k0 + kk;
        }
      } else {
        if (v > mx) {
          s = s * exp(mx - v) + 1.0;
          mx = v;
        } else {
          s += exp(v - mx);
        }
      }
    }
    __syncthreads();
  }
  const double res = (MODE == 1 || MODE == 3) ? mx : log(s) + mx;
  if (MODE == 2) {  // second walk: inverse CDF of the softmax weights against the uniform
    const double r = (m < M && n < N) ? u[(bt * M + m) * N + n] : 0.0;
    double total = 0.0;
    for (int k0 = 0; k0 < K; k0 += T) {
      load(k0);
      __syncthreads();
      const int kend = min(T, K - k0);
      for (int kk = 0; kk < kend; ++kk) {
        const double p = exp(dadd(sa[ty][kk], sb[kk][tx]) - res);
        if (total < r && total + p > r) ind = k0 + kk;
        total += p;
      }
      __syncthreads();
    }
  }
  if (m < M && n < N) {
    const int64_t o = (bt * M + m) * N + n;
    out[o] = res;
    if (MODE == 0) {
      if (aux) static_cast<double*>(aux)[o] = mx;
    } else {
      static_cast<int*>(aux)[o] = ind;
    }
  }
}

// ---- dense log backward -------------------------------------------------------------------------
// grad_a[m,k] = sum_n exp(a[m,k] + b[k,n] - c[m,n]) g[m,n]
__global__ void __launch_bounds__(T * T) dense_log_bwd_a_f64(const double* __restrict__ a, const double* __restrict__ b,
                                                             const double* __restrict__ c, const double* __restrict__ g,
                                                             double* __restrict__ grad_a, int M, int K, int N,
                                                             int tiles_m, int tiles_k) {
  __shared__ double sb[T][T + 1], sc[T][T + 1], sg[T][T + 1];
  const int tx = threadIdx.x % T, ty = threadIdx.x / T;
  const int64_t id = blockIdx.x;
  const int k0 = (int)(id % tiles_k) * T, m0 = (int)((id / tiles_k) % tiles_m) * T;
  const int64_t bt = id / ((int64_t)tiles_k * tiles_m);
  const int m = m0 + ty, k = k0 + tx;
  const double av = (m < M && k < K) ? a[(bt * M + m) * K + k] : 0.0;
  double acc = 0.0;
  for (int n0 = 0; n0 < N; n0 += T) {
    // sb[kk][nn] = b[k0+kk][n0+nn];  sc/sg[mm][nn]
    sb[ty][tx] = (k0 + ty < K && n0 + tx < N) ? b[(bt * K + k0 + ty) * N + n0 + tx] : 0.0;
    const bool okc = m0 + ty < M && n0 + tx < N;
    sc[ty][tx] = okc ? c[(bt * M + m0 + ty) * N + n0 + tx] : 0.0;
    sg[ty][tx] = okc ? g[(bt * M + m0 + ty) * N + n0 + tx] : 0.0;
    __syncthreads();
    const int nend = min(T, N - n0);
    for (int nn = 0; nn < nend; ++nn) acc += exp(av + sb[tx][nn] - sc[ty][nn]) * sg[ty][nn];
    __syncthreads();
  }
  if (m < M && k < K) grad_a[(bt * M + m) * K + k] = acc;
}

// grad_b[k,n] = sum_m exp(a[m,k] + b[k,n] - c[m,n]) g[m,n]
__global__ void __launch_bounds__(T * T) dense_log_bwd_b_f64(const double* __restrict__ a, const double* __restrict__ b,
                                                             const double* __restrict__ c, const double* __restrict__ g,
                                                             double* __restrict__ grad_b, int M, int K, int N,
                                                             int tiles_k, int tiles_n) {
  __shared__ double sa[T][T + 1], sc[T][T + 1], sg[T][T + 1];
  const int tx = threadIdx.x % T, ty = threadIdx.x / T;
  const int64_t id = blockIdx.x;
  const int n0 = (int)(id % tiles_n) * T, k0 = (int)((id / tiles_n) % tiles_k) * T;
  const int64_t bt = id / ((int64_t)tiles_n * tiles_k);
  const int k = k0 + ty, n = n0 + tx;
  const double bv = (k < K && n < N) ? b[(bt * K + k) * N + n] : 0.0;
  double acc = 0.0;
  for (int m0 = 0; m0 < M; m0 += T) {
    // sa[mm][kk] = a[m0+mm][k0+kk];  sc/sg[mm][nn]
    sa[ty][tx] = (m0 + ty < M && k0 + tx < K) ? a[(bt * M + m0 + ty) * K + k0 + tx] : 0.0;
    const bool okc = m0 + ty < M && n0 + tx < N;
    sc[ty][tx] = okc ? c[(bt * M + m0 + ty) * N + n0 + tx] : 0.0;
    sg[ty][tx] = okc ? g[(bt * M + m0 + ty) * N + n0 + tx] : 0.0;
    __syncthreads();
    const int mend = min(T, M - m0);
    for (int mm = 0; mm < mend; ++mm) acc += exp(sa[mm][ty] + bv - sc[mm][tx]) * sg[mm][tx];
    __syncthreads();
  }
  if (k < K && n < N) grad_b[(bt * K + k) * N + n] = acc;
}

// ---- dense index routing (max / sample / prod-max backward) ------------------------------------------
// One thread per gradient element; sums in ascending n (grad_a) / ascending m (grad_b), the reference's order
// (matmul_cuda_kernel.cu:336-456).  O(B M K N) compares like the reference; fine for a checking path.
template <bool MUL>
__global__ void __launch_bounds__(256) route_a_f64(const double* __restrict__ b, const int* __restrict__ idx,
                                                   const double* __restrict__ g, double* __restrict__ grad_a,
                                                   int64_t total, int M, int K, int N) {
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= total) return;
  const int k = (int)(e % K);
  const int64_t row = e / K, bt = row / M;
  double acc = 0.0;
  for (int n = 0; n < N; ++n)
    if (idx[row * N + n] == k) acc = dadd(acc, MUL ? dmul(b[(bt * K + k) * N + n], g[row * N + n]) : g[row * N + n]);
  grad_a[e] = acc;
}
template <bool MUL>
__global__ void __launch_bounds__(256) route_b_f64(const double* __restrict__ a, const int* __restrict__ idx,
                                                   const double* __restrict__ g, double* __restrict__ grad_b,
                                                   int64_t total, int M, int K, int N) {
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= total) return;
  const int n = (int)(e % N), k = (int)((e / N) % K);
  const int64_t bt = e / ((int64_t)N * K);
  double acc = 0.0;
  for (int m = 0; m < M; ++m) {
    const int64_t o = (bt * M + m) * N + n;
    if (idx[o] == k) acc = dadd(acc, MUL ? dmul(a[(bt * M + m) * K + k], g[o]) : g[o]);
  }
  grad_b[e] = acc;
}

// ---- banded ---------------------------------------------------------------------------------------
// banded_cuda_kernel.cu:13-100; one thread per result band cell
template <int MODE>
__global__ void __launch_bounds__(256) band_fwd_f64(const double* __restrict__ a, const double* __restrict__ b,
                                                    double* __restrict__ out, int* __restrict__ idx,
                                                    double* __restrict__ maxes, BandDims d, int64_t cells) {
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= cells) return;
  const int Wa = d.Wa(), Wb = d.Wb(), Wo = d.Wo(), r_lu = d.r_lu();
  const int64_t n = d.n;
  const int j = (int)(e % Wo);
  const int64_t i = (e / Wo) % n, bt = e / (Wo * n);
  const int64_t o = i + j - r_lu;
  double res = 0.0, mx = kFloorD;
  int ind = -1;
  if (o >= 0 && o < n) {
    const double* ai = a + (bt * n + i) * Wa;
    const double* bo = b + (bt * n + o) * Wb;
    auto term = [&](int k, double* v) -> bool {
      const int64_t pos = i + k - d.a_lu, k2 = pos - o + d.b_lu;
      if (k2 < 0 || k2 >= Wb || pos < 0 || pos >= n) return false;
      *v = MODE == 3 ? dmul(ai[k], bo[k2]) : dadd(ai[k], bo[k2]);
      return true;
    };
    double v;
    if (MODE == 3) {
      for (int k = 0; k < Wa; ++k)
        if (term(k, &v)) res = dadd(res, v);
    } else {
      for (int k = 0; k < Wa; ++k)
        if (term(k, &v) && v > mx) {
          mx = v;
          ind = k;
        }
      res = mx;
      if (MODE == 0) {
        double s = 0.0;
        for (int k = 0; k < Wa; ++k)
          if (term(k, &v)) s += exp(v - mx);
        res = log(s) + mx;
      }
    }
  } else {
    ind = 0;
    mx = 0.0;
  }
  out[e] = res;
  if (MODE == 1) idx[e] = ind;
  if (MODE == 0 && maxes) maxes[e] = mx;
}

// banded_cuda_kernel.cu:104-152 (grad_a) and its operand-swapped use for grad_b (sparse.py:436-446),
// the latter computed directly here.  part: saved output (log) / indices (max).
template <int MODE, bool FOR_B>
__global__ void __launch_bounds__(256) band_bwd_f64(const double* __restrict__ a, const double* __restrict__ b,
                                                    const double* __restrict__ g, const double* __restrict__ part,
                                                    const int* __restrict__ pidx, double* __restrict__ grad,
                                                    BandDims d, int64_t cells) {
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= cells) return;
  const int Wa = d.Wa(), Wb = d.Wb(), Wo = d.Wo(), r_lu = d.r_lu();
  const int64_t n = d.n;
  double val = 0.0;
  if (!FOR_B) {
    const int ja = (int)(e % Wa);
    const int64_t i = (e / Wa) % n, bt = e / (Wa * n);
    const int64_t p = i + ja - d.a_lu;
    if (p >= 0 && p < n) {
      for (int jo = 0; jo < Wo; ++jo) {
        const int64_t o = i + jo - r_lu, k2 = p - o + d.b_lu;
        if (k2 < 0 || k2 >= Wb || o < 0 || o >= n) continue;
        const int64_t q = (bt * n + i) * Wo + jo;
        double w;
        if (MODE == 3) w = b[(bt * n + o) * Wb + k2];
        if (MODE == 1) w = (pidx[q] == ja) ? 1.0 : 0.0;
        if (MODE == 0) w = exp(a[e] + b[(bt * n + o) * Wb + k2] - part[q]);
        val = dadd(val, dmul(w, g[q]));
      }
    }
  } else {
    const int k2 = (int)(e % Wb);
    const int64_t o = (e / Wb) % n, bt = e / (Wb * n);
    const int64_t p = o + k2 - d.b_lu;
    if (p >= 0 && p < n) {
      // rows i whose band reaches column p, in ascending order
      for (int64_t i = max((int64_t)0, p - d.a_ld); i <= min(n - 1, p + d.a_lu); ++i) {
        const int ja = (int)(p - i + d.a_lu);
        const int64_t jo = o - i + r_lu;
        if (jo < 0 || jo >= Wo) continue;
        const int64_t q = (bt * n + i) * Wo + jo;
        double w;
        if (MODE == 3) w = a[(bt * n + i) * Wa + ja];
        if (MODE == 1) w = (pidx[q] == ja) ? 1.0 : 0.0;
        if (MODE == 0) w = exp(a[(bt * n + i) * Wa + ja] + b[e] - part[q]);
        val = dadd(val, dmul(w, g[q]));
      }
    }
  }
  grad[e] = val;
}

int check_dims(int64_t B, int64_t M, int64_t K, int64_t N) {
  if (B < 0 || M < 0 || K < 0 || N < 0) return GBMM_ERR_INVALID_ARG;
  const int64_t lim = (1LL << 31) - 64;
  if (M >= lim || K >= lim || N >= lim) return GBMM_ERR_UNSUPPORTED;
  return GBMM_OK;
}

}  // namespace
}  // namespace gbmm

using namespace gbmm;

extern "C" int gbmm_dense_forward_f64(int mode, const double* a, const double* b, const double* u, double* out,
                                      void* aux, int64_t B, int64_t M, int64_t K, int64_t N, void* stream) {
  if (mode < 0 || mode > 3) return GBMM_ERR_INVALID_ARG;
  const int rc = check_dims(B, M, K, N);
  if (rc != GBMM_OK) return rc;
  if (B == 0 || M == 0 || N == 0) return GBMM_OK;
  if ((K > 0 && (!a || !b)) || !out || (mode != GBMM_MODE_LOG && !aux) || (mode == GBMM_MODE_SAMPLE && !u))
    return GBMM_ERR_INVALID_ARG;
  const int64_t tm = ceil_div(M, T), tn = ceil_div(N, T), blocks = B * tm * tn;
  if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)blocks;
  const int m = (int)M, k = (int)K, n = (int)N;
  switch (mode) {
    case 0: dense_fwd_f64<0><<<grid, T * T, 0, st>>>(a, b, u, out, aux, m, k, n, (int)tm, (int)tn); break;
    case 1: dense_fwd_f64<1><<<grid, T * T, 0, st>>>(a, b, u, out, aux, m, k, n, (int)tm, (int)tn); break;
    case 2: dense_fwd_f64<2><<<grid, T * T, 0, st>>>(a, b, u, out, aux, m, k, n, (int)tm, (int)tn); break;
    default: dense_fwd_f64<3><<<grid, T * T, 0, st>>>(a, b, u, out, aux, m, k, n, (int)tm, (int)tn); break;
  }
  return launch_status();
}

extern "C" int gbmm_dense_backward_f64(int mode, const double* a, const double* b, const double* grad_out,
                                       const double* part, const void* aux, double* grad_a, double* grad_b, int64_t B,
                                       int64_t M, int64_t K, int64_t N, void* stream) {
  if (mode < 0 || mode > 3) return GBMM_ERR_INVALID_ARG;
  const int rc = check_dims(B, M, K, N);
  if (rc != GBMM_OK) return rc;
  if (B == 0 || K == 0 || (M == 0 && N == 0)) return GBMM_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int m = (int)M, k = (int)K, n = (int)N;
  if (M == 0 || N == 0) {  // nothing flows back: the gradients are zero
    if (grad_a && M > 0 && cudaMemsetAsync(grad_a, 0, sizeof(double) * B * M * K, st) != cudaSuccess) return GBMM_ERR_LAUNCH;
    if (grad_b && N > 0 && cudaMemsetAsync(grad_b, 0, sizeof(double) * B * K * N, st) != cudaSuccess) return GBMM_ERR_LAUNCH;
    return GBMM_OK;
  }
  if (!a || !b || !grad_out) return GBMM_ERR_INVALID_ARG;
  if (mode == GBMM_MODE_LOG) {
    if (!part) return GBMM_ERR_INVALID_ARG;
    const int64_t tm = ceil_div(M, T), tk = ceil_div(K, T), tn = ceil_div(N, T);
    if (B * tm * tk >= (1LL << 31) || B * tk * tn >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
    if (grad_a)
      dense_log_bwd_a_f64<<<(unsigned)(B * tm * tk), T * T, 0, st>>>(a, b, part, grad_out, grad_a, m, k, n, (int)tm,
                                                                    (int)tk);
    if (grad_b)
      dense_log_bwd_b_f64<<<(unsigned)(B * tk * tn), T * T, 0, st>>>(a, b, part, grad_out, grad_b, m, k, n, (int)tk,
                                                                    (int)tn);
    return launch_status();
  }
  if (!aux) return GBMM_ERR_INVALID_ARG;
  const int* idx = static_cast<const int*>(aux);
  const int64_t ea = B * M * K, eb = B * K * N;
  if (ceil_div(ea, 256) >= (1LL << 31) || ceil_div(eb, 256) >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  const bool mul = mode == GBMM_MODE_PRODMAX;
  if (grad_a) {
    if (mul) route_a_f64<true><<<(unsigned)ceil_div(ea, 256), 256, 0, st>>>(b, idx, grad_out, grad_a, ea, m, k, n);
    else route_a_f64<false><<<(unsigned)ceil_div(ea, 256), 256, 0, st>>>(b, idx, grad_out, grad_a, ea, m, k, n);
  }
  if (grad_b) {
    if (mul) route_b_f64<true><<<(unsigned)ceil_div(eb, 256), 256, 0, st>>>(a, idx, grad_out, grad_b, eb, m, k, n);
    else route_b_f64<false><<<(unsigned)ceil_div(eb, 256), 256, 0, st>>>(a, idx, grad_out, grad_b, eb, m, k, n);
  }
  return launch_status();
}

static int check_band_f64(int mode, int64_t B, int64_t n, int a_lu, int a_ld, int b_lu, int b_ld) {
  if (mode != GBMM_BAND_LOG && mode != GBMM_BAND_MAX && mode != GBMM_BAND_MUL) return GBMM_ERR_INVALID_ARG;
  if (B < 0 || n < 0 || a_lu < 0 || a_ld < 0 || b_lu < 0 || b_ld < 0) return GBMM_ERR_INVALID_ARG;
  if (n >= (1LL << 31) - 64 || (int64_t)a_lu + a_ld + b_lu + b_ld >= (1 << 24)) return GBMM_ERR_UNSUPPORTED;
  return GBMM_OK;
}

extern "C" int gbmm_band_forward_f64(int mode, const double* a, int a_lu, int a_ld, const double* b, int b_lu,
                                     int b_ld, double* out, int32_t* idx, double* maxes, int64_t B, int64_t n,
                                     void* stream) {
  const int rc = check_band_f64(mode, B, n, a_lu, a_ld, b_lu, b_ld);
  if (rc != GBMM_OK) return rc;
  if (B == 0 || n == 0) return GBMM_OK;
  if (!a || !b || !out || (mode == GBMM_BAND_MAX && !idx)) return GBMM_ERR_INVALID_ARG;
  const BandDims d{n, a_lu, a_ld, b_lu, b_ld};
  const int64_t cells = B * n * d.Wo(), blocks = ceil_div(cells, 256);
  if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (mode == GBMM_BAND_LOG) band_fwd_f64<0><<<(unsigned)blocks, 256, 0, st>>>(a, b, out, idx, maxes, d, cells);
  if (mode == GBMM_BAND_MAX) band_fwd_f64<1><<<(unsigned)blocks, 256, 0, st>>>(a, b, out, idx, maxes, d, cells);
  if (mode == GBMM_BAND_MUL) band_fwd_f64<3><<<(unsigned)blocks, 256, 0, st>>>(a, b, out, idx, maxes, d, cells);
  return launch_status();
}

extern "C" int gbmm_band_backward_f64(int mode, const double* a, int a_lu, int a_ld, const double* b, int b_lu,
                                      int b_ld, const double* grad_out, const void* part, double* grad_a,
                                      double* grad_b, int64_t B, int64_t n, void* stream) {
  const int rc = check_band_f64(mode, B, n, a_lu, a_ld, b_lu, b_ld);
  if (rc != GBMM_OK) return rc;
  if (B == 0 || n == 0) return GBMM_OK;
  if (!a || !b || !grad_out || (mode != GBMM_BAND_MUL && !part)) return GBMM_ERR_INVALID_ARG;
  const BandDims d{n, a_lu, a_ld, b_lu, b_ld};
  const int64_t ca = B * n * d.Wa(), cb = B * n * d.Wb();
  if (ceil_div(ca, 256) >= (1LL << 31) || ceil_div(cb, 256) >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const double* pd = mode == GBMM_BAND_LOG ? static_cast<const double*>(part) : nullptr;
  const int* pi = mode == GBMM_BAND_MAX ? static_cast<const int*>(part) : nullptr;
  const unsigned ga = (unsigned)ceil_div(ca, 256), gb = (unsigned)ceil_div(cb, 256);
  if (grad_a) {
    if (mode == GBMM_BAND_LOG) band_bwd_f64<0, false><<<ga, 256, 0, st>>>(a, b, grad_out, pd, pi, grad_a, d, ca);
    if (mode == GBMM_BAND_MAX) band_bwd_f64<1, false><<<ga, 256, 0, st>>>(a, b, grad_out, pd, pi, grad_a, d, ca);
    if (mode == GBMM_BAND_MUL) band_bwd_f64<3, false><<<ga, 256, 0, st>>>(a, b, grad_out, pd, pi, grad_a, d, ca);
  }
  if (grad_b) {
    if (mode == GBMM_BAND_LOG) band_bwd_f64<0, true><<<gb, 256, 0, st>>>(a, b, grad_out, pd, pi, grad_b, d, cb);
    if (mode == GBMM_BAND_MAX) band_bwd_f64<1, true><<<gb, 256, 0, st>>>(a, b, grad_out, pd, pi, grad_b, d, cb);
    if (mode == GBMM_BAND_MUL) band_bwd_f64<3, true><<<gb, 256, 0, st>>>(a, b, grad_out, pd, pi, grad_b, d, cb);
  }
  return launch_status();
}
