// Second-order terms of the log-semiring product (what autograd needs under create_graph=True).
//
// The first-order gradients are grad_a[m,k] = sum_n s g and grad_b[k,n] = sum_m s g with the
// softmax weight s[m,k,n] = exp(a[m,k] + b[k,n] - c[m,n]).  For cotangents h_a of grad_a and
// h_b of grad_b the scalar  L = <grad_a, h_a> + <grad_b, h_b> = sum s g (h_a[m,k] + h_b[k,n])
// has, with  H = h_a[m,k] + h_b[k,n]  and  t[m,n] = sum_k s H,
//   dL/da[m,k] = sum_n g s (H - t),   dL/db[k,n] = sum_m g s (H - t),   dL/dg[m,n] = t[m,n]
// (ds/da[m,k'] = s (delta_kk' - s[m,k',n]) folded in).  Two passes of O(B*M*K*N) replace the
// reference's three kernels, two of which are O(B*M*K*N*K) (matmul_cuda_kernel.cu:220-331), and
// also cover the cotangent of grad_b, which the reference reaches through transposed copies.
//
// Same 128x64 tiling as the first-order kernels; single-buffered (these are rarely the hot path).
#include "tile.cuh"

namespace gbmm {
namespace {

constexpr int BR = 128, BC = 64, BK = 16, NT = 256;
constexpr int LDR = BR + 4, LDC = BC + 4;

struct TileCoord {
  int bt, r0, c0;
  __device__ __forceinline__ TileCoord(int tiles_r, int tiles_c) {
    const int64_t id = blockIdx.x;
    c0 = (int)(id % tiles_c) * BC;
    r0 = (int)((id / tiles_c) % tiles_r) * BR;
    bt = (int)(id / ((int64_t)tiles_c * tiles_r));
  }
};

__device__ __forceinline__ void store_tile(float* __restrict__ dst, int64_t pitch, int rows, int cols,
                                           const TileCoord& tc, const Micro8x4& mt, const float (&acc)[8][4]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = tc.r0 + mt.row(i);
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = tc.c0 + mt.col(j);
      if (c < cols) dst[(int64_t)r * pitch + c] = acc[i][j];
    }
  }
}

// t[m,n] = sum_k exp(a+b-c) (h_a[m,k] + h_b[k,n]); tile rows m, columns n, reduction over k.
__global__ void __launch_bounds__(NT) log_bwd2_t_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                        const float* __restrict__ c, const float* __restrict__ ha,
                                                        const float* __restrict__ hb, float* __restrict__ t, int M,
                                                        int K, int N, int tiles_r, int tiles_c) {
  __shared__ __align__(16) float sa[BK * LDR], sha[BK * LDR], sb[BK * LDC], shb[BK * LDC];
  const TileCoord tc(tiles_r, tiles_c);
  const Micro8x4 mt;
  const int64_t oa = (int64_t)tc.bt * M * K, ob = (int64_t)tc.bt * K * N, oc = (int64_t)tc.bt * M * N;
  float acc[8][4], cl[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = tc.r0 + mt.row(i), n = tc.c0 + mt.col(j);
      acc[i][j] = 0.f;
      cl[i][j] = (m < M && n < N) ? -kLog2e * __ldg(c + oc + (int64_t)m * N + n) : 0.f;
    }
  TileLoader<BR, BK, NT, true> la, lha;
  TileLoader<BC, BK, NT, false> lb, lhb;
  const int nt = (K + BK - 1) / BK;
  for (int tt = 0; tt < nt; ++tt) {
    // padded reduction steps: a = -inf gives weight 0, h = 0
    la.load(a + oa, K, 1, tc.r0, tt * BK, M, K, false, __int_as_float(0xff800000));
    lha.load(ha + oa, K, 1, tc.r0, tt * BK, M, K, false, 0.f);
    lb.load(b + ob, 1, N, tc.c0, tt * BK, N, K, false, 0.f);
    lhb.load(hb + ob, 1, N, tc.c0, tt * BK, N, K, false, 0.f);
    __syncthreads();
    la.store(sa, LDR);
    lha.store(sha, LDR);
    lb.store(sb, LDC);
    lhb.store(shb, LDC);
    __syncthreads();
#pragma unroll 4
    for (int kk = 0; kk < BK; ++kk) {
      float x[8], hx[8], y[4], hy[4];
      mt.load_x(sa + kk * LDR, LDR, x);
      mt.load_x(sha + kk * LDR, LDR, hx);
      mt.load_y(sb + kk * LDC, y);
      mt.load_y(shb + kk * LDC, hy);
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          acc[i][j] = fmaf(ex2_approx(fmaf(x[i] + y[j], kLog2e, cl[i][j])), hx[i] + hy[j], acc[i][j]);
    }
  }
  store_tile(t + oc, N, M, N, tc, mt, acc);
}

// dL/da[m,k] = sum_n g s (h_a[m,k] + h_b[k,n] - t[m,n]); tile rows m, columns k, reduction over n.
__global__ void __launch_bounds__(NT) log_bwd2_a_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                        const float* __restrict__ c, const float* __restrict__ g,
                                                        const float* __restrict__ t, const float* __restrict__ ha,
                                                        const float* __restrict__ hb, float* __restrict__ out,
                                                        int M, int K, int N, int tiles_r, int tiles_c) {
  __shared__ __align__(16) float sc[BK * LDR], sg[BK * LDR], st[BK * LDR], sb[BK * LDC], shb[BK * LDC];
  const TileCoord tc(tiles_r, tiles_c);
  const Micro8x4 mt;
  const int64_t oa = (int64_t)tc.bt * M * K, ob = (int64_t)tc.bt * K * N, oc = (int64_t)tc.bt * M * N;
  float acc[8][4], av[8][4], hv[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = tc.r0 + mt.row(i), k = tc.c0 + mt.col(j);
      const bool ok = m < M && k < K;
      acc[i][j] = 0.f;
      av[i][j] = ok ? __ldg(a + oa + (int64_t)m * K + k) : 0.f;
      hv[i][j] = ok ? __ldg(ha + oa + (int64_t)m * K + k) : 0.f;
    }
  TileLoader<BR, BK, NT, true> lc, lg, lt;
  TileLoader<BC, BK, NT, true> lb, lhb;
  const int nt = (N + BK - 1) / BK;
  for (int tt = 0; tt < nt; ++tt) {
    lc.load(c + oc, N, 1, tc.r0, tt * BK, M, N, false, __int_as_float(0x7f800000));
    lg.load(g + oc, N, 1, tc.r0, tt * BK, M, N, false, 0.f);
    lt.load(t + oc, N, 1, tc.r0, tt * BK, M, N, false, 0.f);
    lb.load(b + ob, N, 1, tc.c0, tt * BK, K, N, false, 0.f);
    lhb.load(hb + ob, N, 1, tc.c0, tt * BK, K, N, false, 0.f);
    __syncthreads();
    lc.store_scaled(sc, LDR, -kLog2e);
    lg.store(sg, LDR);
    lt.store(st, LDR);
    lb.store(sb, LDC);
    lhb.store(shb, LDC);
    __syncthreads();
#pragma unroll 4
    for (int kk = 0; kk < BK; ++kk) {
      float cv[8], gv[8], tv[8], bv[4], hy[4];
      mt.load_x(sc + kk * LDR, LDR, cv);
      mt.load_x(sg + kk * LDR, LDR, gv);
      mt.load_x(st + kk * LDR, LDR, tv);
      mt.load_y(sb + kk * LDC, bv);
      mt.load_y(shb + kk * LDC, hy);
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float w = ex2_approx(fmaf(av[i][j] + bv[j], kLog2e, cv[i])) * gv[i];
          acc[i][j] = fmaf(w, (hv[i][j] + hy[j]) - tv[i], acc[i][j]);
        }
    }
  }
  store_tile(out + oa, K, M, K, tc, mt, acc);
}

// dL/db[k,n] = sum_m g s (h_a[m,k] + h_b[k,n] - t[m,n]); tile rows k, columns n, reduction over m.
__global__ void __launch_bounds__(NT) log_bwd2_b_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                        const float* __restrict__ c, const float* __restrict__ g,
                                                        const float* __restrict__ t, const float* __restrict__ ha,
                                                        const float* __restrict__ hb, float* __restrict__ out,
                                                        int M, int K, int N, int tiles_r, int tiles_c) {
  __shared__ __align__(16) float sa[BK * LDR], sha[BK * LDR], sc[BK * LDC], sg[BK * LDC], st[BK * LDC];
  const TileCoord tc(tiles_r, tiles_c);
  const Micro8x4 mt;
  const int64_t oa = (int64_t)tc.bt * M * K, ob = (int64_t)tc.bt * K * N, oc = (int64_t)tc.bt * M * N;
  float acc[8][4], bv[8][4], hv[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = tc.r0 + mt.row(i), n = tc.c0 + mt.col(j);
      const bool ok = k < K && n < N;
      acc[i][j] = 0.f;
      bv[i][j] = ok ? __ldg(b + ob + (int64_t)k * N + n) : 0.f;
      hv[i][j] = ok ? __ldg(hb + ob + (int64_t)k * N + n) : 0.f;
    }
  TileLoader<BR, BK, NT, false> la, lha;
  TileLoader<BC, BK, NT, false> lc, lg, lt;
  const int nt = (M + BK - 1) / BK;
  for (int tt = 0; tt < nt; ++tt) {
    la.load(a + oa, 1, K, tc.r0, tt * BK, K, M, false, 0.f);
    lha.load(ha + oa, 1, K, tc.r0, tt * BK, K, M, false, 0.f);
    lc.load(c + oc, 1, N, tc.c0, tt * BK, N, M, false, __int_as_float(0x7f800000));
    lg.load(g + oc, 1, N, tc.c0, tt * BK, N, M, false, 0.f);
    lt.load(t + oc, 1, N, tc.c0, tt * BK, N, M, false, 0.f);
    __syncthreads();
    la.store(sa, LDR);
    lha.store(sha, LDR);
    lc.store_scaled(sc, LDC, -kLog2e);
    lg.store(sg, LDC);
    lt.store(st, LDC);
    __syncthreads();
#pragma unroll 4
    for (int kk = 0; kk < BK; ++kk) {
      float xa[8], hx[8], cv[4], gv[4], tv[4];
      mt.load_x(sa + kk * LDR, LDR, xa);
      mt.load_x(sha + kk * LDR, LDR, hx);
      mt.load_y(sc + kk * LDC, cv);
      mt.load_y(sg + kk * LDC, gv);
      mt.load_y(st + kk * LDC, tv);
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float w = ex2_approx(fmaf(xa[i] + bv[i][j], kLog2e, cv[j])) * gv[j];
          acc[i][j] = fmaf(w, (hx[i] + hv[i][j]) - tv[j], acc[i][j]);
        }
    }
  }
  store_tile(out + ob, N, K, N, tc, mt, acc);
}

}  // namespace
}  // namespace gbmm

using namespace gbmm;

extern "C" int gbmm_dense_backbackward_f32(const float* a, const float* b, const float* grad_out,
                                           const float* part, const float* h_a, const float* h_b, float* d_a,
                                           float* d_b, float* d_grad_out, int64_t B, int64_t M, int64_t K,
                                           int64_t N, void* stream) {
  if (B < 0 || M < 0 || K < 0 || N < 0) return GBMM_ERR_INVALID_ARG;
  if (B == 0 || M == 0 || K == 0 || N == 0) return GBMM_ERR_UNSUPPORTED;  // nothing to differentiate
  if (!a || !b || !grad_out || !part || !h_a || !h_b || !d_a || !d_b || !d_grad_out) return GBMM_ERR_INVALID_ARG;
  const int64_t lim = (1LL << 31) - 256;
  if (M >= lim || K >= lim || N >= lim) return GBMM_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int m = (int)M, k = (int)K, n = (int)N;
  {
    const int64_t tr = ceil_div(M, BR), tcn = ceil_div(N, BC), blocks = B * tr * tcn;
    if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
    log_bwd2_t_kernel<<<(unsigned)blocks, NT, 0, st>>>(a, b, part, h_a, h_b, d_grad_out, m, k, n, (int)tr,
                                                       (int)tcn);
    if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
  }
  {
    const int64_t tr = ceil_div(M, BR), tcn = ceil_div(K, BC), blocks = B * tr * tcn;
    if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
    log_bwd2_a_kernel<<<(unsigned)blocks, NT, 0, st>>>(a, b, part, grad_out, d_grad_out, h_a, h_b, d_a, m, k, n,
                                                       (int)tr, (int)tcn);
    if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
  }
  {
    const int64_t tr = ceil_div(K, BR), tcn = ceil_div(N, BC), blocks = B * tr * tcn;
    if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
    log_bwd2_b_kernel<<<(unsigned)blocks, NT, 0, st>>>(a, b, part, grad_out, d_grad_out, h_a, h_b, d_b, m, k, n,
                                                       (int)tr, (int)tcn);
  }
  return launch_status();
}
