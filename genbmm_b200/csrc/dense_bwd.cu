// Dense semiring backward kernels.
//
// log semiring (replaces matmul_cuda_kernel.cu:159-217 and the transposed copies of
// genmul.py:38-41): the softmax weight w = exp(a[m,k] + b[k,n] - c[m,n]) is recomputed tile
// by tile from the saved forward output; nothing of size B*M*K*N is stored.
//   grad_a[m,k] = sum_n w * g[m,n]   (CTA owns a 128x64 tile of grad_a, walks n)
//   grad_b[k,n] = sum_m w * g[m,n]   (CTA owns a 128x64 tile of grad_b, walks m)
// Both read a, b, c, g in their natural layouts; no transposed copy is made.
//
// max / sample / prod-max (replaces matmul_cuda_kernel.cu:336-456, which scan all K*N
// candidates per output): the saved int32 index routes each g[m,n] to one cell,
//   grad_a[m,idx] += g[m,n] (* b[idx,n]),   grad_b[idx,n] += g[m,n] (* a[m,idx]),
// accumulated in shared-memory rows/columns in ascending n (grad_a) and ascending m
// (grad_b), the order of the reference's loops.  An index outside [0,K) routes nowhere.
#include "dense.cuh"
#include <cstdlib>

#include "tile.cuh"

namespace gbmm {
namespace {

constexpr int BR = 128, BC = 64, BK = 16, NT = 256;
constexpr int LDR = BR + 4, LDC = BC + 4;

__device__ __forceinline__ float pinf_f() { return __int_as_float(0x7f800000); }

struct TileCoord {
  int bt, r0, c0;
  __device__ __forceinline__ TileCoord(int64_t id, int tiles_r, int tiles_c) {
    c0 = (int)(id % tiles_c) * BC;
    r0 = (int)((id / tiles_c) % tiles_r) * BR;
    bt = (int)(id / ((int64_t)tiles_c * tiles_r));
  }
};

template <bool ACCUMULATE>
__device__ __forceinline__ void store_tile(float* __restrict__ dst, int64_t pitch, int rows, int cols,
                                           const TileCoord& tc, const Micro8x4& mt, const float (&acc)[8][4]) {
  const bool vec = aligned16(dst) && (pitch % 4 == 0);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = tc.r0 + mt.row(i);
    if (r >= rows) continue;
    const int cb = tc.c0 + mt.col(0);
    if (vec && cb + 3 < cols) {
      float4* p = reinterpret_cast<float4*>(dst + (int64_t)r * pitch + cb);
      float4 v = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
      if (ACCUMULATE) {
        const float4 old = *p;
        v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
      }
      *p = v;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (cb + j < cols) {
          float* p = dst + (int64_t)r * pitch + cb + j;
          *p = ACCUMULATE ? *p + acc[i][j] : acc[i][j];
        }
    }
  }
}

// In FLAGGED mode (used behind the factorised fast path, dense_fast.cu) only the terms whose
// (m,n) lies in a 128x128 result tile marked in `flags` are summed, and the sum is added to
// what the fast kernels already wrote; a CTA with no marked tile in its strip returns at once.
// flags is indexed [batch][m/128][n/128].

// grad_a tile: rows m, columns k, reduction over n.
template <bool FLAGGED>
__device__ __forceinline__ void log_bwd_a_tile(const TileCoord& tc, float (&sc)[2][BK * LDR],
                                               float (&sg)[2][BK * LDR], float (&sb)[2][BK * LDC],
                                               const float* __restrict__ a, const float* __restrict__ b,
                                               const float* __restrict__ c, const float* __restrict__ g,
                                               float* __restrict__ grad_a, int M, int K, int N, int tiles_r,
                                               const int* __restrict__ flags) {
  const Micro8x4 mt;
  const float* ab = a + (int64_t)tc.bt * M * K;
  const float* bb = b + (int64_t)tc.bt * K * N;
  const float* cb = c + (int64_t)tc.bt * M * N;
  const float* gb = g + (int64_t)tc.bt * M * N;
  const bool vec_n = (N % 4 == 0);
  const bool vec_b = vec_n && aligned16(bb), vec_c = vec_n && aligned16(cb), vec_g = vec_n && aligned16(gb);
  const int nt = (N + BK - 1) / BK;
  constexpr int GRP = 128 / BK;  // reduction tiles per 128-wide flag tile
  const int ngrp = FLAGGED ? (N + 127) / 128 : 1;
  const int* frow = FLAGGED ? flags + ((int64_t)tc.bt * tiles_r + tc.r0 / 128) * ngrp : nullptr;

  float acc[8][4], av[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = tc.r0 + mt.row(i), k = tc.c0 + mt.col(j);
      acc[i][j] = 0.f;
      av[i][j] = (m < M && k < K) ? __ldg(ab + (int64_t)m * K + k) : 0.f;
    }

  TileLoader<BR, BK, NT, true> lc, lg;
  TileLoader<BC, BK, NT, true> lb;
  // c is staged as -c*log2(e), so that exp(a+b-c) = 2^((a+b)*log2e + staged): one FADD, one FFMA,
  // one MUFU and the accumulating FFMA per term.  Padding: c = +inf makes the weight 0 and g = 0
  // removes the term.
  for (int grp = 0; grp < ngrp; ++grp) {
    if (FLAGGED && __ldg(frow + grp) == 0) continue;
    const int t_begin = FLAGGED ? grp * GRP : 0;
    const int t_end = FLAGGED ? min(nt, t_begin + GRP) : nt;
    if (t_begin >= t_end) continue;
    lc.load(cb, N, 1, tc.r0, t_begin * BK, M, N, vec_c, pinf_f());
    lg.load(gb, N, 1, tc.r0, t_begin * BK, M, N, vec_g, 0.f);
    lb.load(bb, N, 1, tc.c0, t_begin * BK, K, N, vec_b, 0.f);
    __syncthreads();  // the previous group's last tile is fully consumed
    lc.store_scaled(sc[0], LDR, -kLog2e);
    lg.store(sg[0], LDR);
    lb.store(sb[0], LDC);
    __syncthreads();
    for (int t = t_begin; t < t_end; ++t) {
      const int cur = (t - t_begin) & 1;
      if (t + 1 < t_end) {
        lc.load(cb, N, 1, tc.r0, (t + 1) * BK, M, N, vec_c, pinf_f());
        lg.load(gb, N, 1, tc.r0, (t + 1) * BK, M, N, vec_g, 0.f);
        lb.load(bb, N, 1, tc.c0, (t + 1) * BK, K, N, vec_b, 0.f);
      }
#pragma unroll
      for (int kk = 0; kk < BK; ++kk) {
        float cv[8], gv[8], bv[4];
        mt.load_x(sc[cur] + kk * LDR, LDR, cv);
        mt.load_x(sg[cur] + kk * LDR, LDR, gv);
        mt.load_y(sb[cur] + kk * LDC, bv);
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            acc[i][j] = fmaf(ex2_approx(fmaf(av[i][j] + bv[j], kLog2e, cv[i])), gv[i], acc[i][j]);
      }
      if (t + 1 < t_end) {
        lc.store_scaled(sc[cur ^ 1], LDR, -kLog2e);
        lg.store(sg[cur ^ 1], LDR);
        lb.store(sb[cur ^ 1], LDC);
      }
      __syncthreads();
    }
  }
  store_tile<FLAGGED>(grad_a + (int64_t)tc.bt * M * K, K, M, K, tc, mt, acc);
}

// One tile per CTA (FLAGGED false: grid = `total` tiles), or a capped grid whose CTAs gather the tiles with a
// marked flag in their strip and work through them.
template <bool FLAGGED>
__global__ void __launch_bounds__(NT) dense_log_bwd_a_kernel(const float* __restrict__ a,
                                                             const float* __restrict__ b,
                                                             const float* __restrict__ c,
                                                             const float* __restrict__ g,
                                                             float* __restrict__ grad_a, int M, int K, int N,
                                                             int tiles_r, int tiles_c,
                                                             const int* __restrict__ flags, int64_t total,
                                                             const int* error, int64_t out_count) {
  __shared__ __align__(16) float sc[2][BK * LDR];
  __shared__ __align__(16) float sg[2][BK * LDR];
  __shared__ __align__(16) float sb[2][BK * LDC];
  if (!FLAGGED) {
    log_bwd_a_tile<false>(TileCoord(blockIdx.x, tiles_r, tiles_c), sc, sg, sb, a, b, c, g, grad_a, M, K, N,
                          tiles_r, flags);
    return;
  }
  // the product kernel before this one gave up on a bounded wait: the whole gradient becomes NaN
  if (poison_if_failed(error, grad_a, out_count)) return;
  __shared__ int list[NT];
  __shared__ int count;
  const int ngrp = (N + 127) / 128;
  auto flagged = [&](int64_t id) {
    const TileCoord t(id, tiles_r, tiles_c);
    const int* frow = flags + ((int64_t)t.bt * tiles_r + t.r0 / 128) * ngrp;
    bool any = false;
    for (int q = 0; q < ngrp; ++q) any |= (__ldg(frow + q) != 0);
    return any;
  };
  for (int64_t base = 0; base < total; base += (int64_t)gridDim.x * NT) {
    const int nw = collect_tiles(base, total, list, &count, flagged);
    for (int w = 0; w < nw; ++w) {
      log_bwd_a_tile<true>(TileCoord(list[w], tiles_r, tiles_c), sc, sg, sb, a, b, c, g, grad_a, M, K, N,
                           tiles_r, flags);
      __syncthreads();
    }
  }
}

// grad_b tile: rows k, columns n, reduction over m.
template <bool FLAGGED>
__device__ __forceinline__ void log_bwd_b_tile(const TileCoord& tc, float (&sa)[2][BK * LDR],
                                               float (&sc)[2][BK * LDC], float (&sg)[2][BK * LDC],
                                               const float* __restrict__ a, const float* __restrict__ b,
                                               const float* __restrict__ c, const float* __restrict__ g,
                                               float* __restrict__ grad_b, int M, int K, int N,
                                               const int* __restrict__ flags) {
  const Micro8x4 mt;
  const float* ab = a + (int64_t)tc.bt * M * K;
  const float* bb = b + (int64_t)tc.bt * K * N;
  const float* cb = c + (int64_t)tc.bt * M * N;
  const float* gb = g + (int64_t)tc.bt * M * N;
  const bool vec_a = (K % 4 == 0) && aligned16(ab);
  const bool vec_c = (N % 4 == 0) && aligned16(cb), vec_g = (N % 4 == 0) && aligned16(gb);
  const int nt = (M + BK - 1) / BK;
  constexpr int GRP = 128 / BK;
  const int ngrp = FLAGGED ? (M + 127) / 128 : 1;
  const int fpitch = (N + 127) / 128;
  const int* fcol = FLAGGED ? flags + (int64_t)tc.bt * ngrp * fpitch + tc.c0 / 128 : nullptr;

  float acc[8][4], bv[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = tc.r0 + mt.row(i), n = tc.c0 + mt.col(j);
      acc[i][j] = 0.f;
      bv[i][j] = (k < K && n < N) ? __ldg(bb + (int64_t)k * N + n) : 0.f;
    }

  TileLoader<BR, BK, NT, false> la;
  TileLoader<BC, BK, NT, false> lc, lg;
  for (int grp = 0; grp < ngrp; ++grp) {
    if (FLAGGED && __ldg(fcol + (int64_t)grp * fpitch) == 0) continue;
    const int t_begin = FLAGGED ? grp * GRP : 0;
    const int t_end = FLAGGED ? min(nt, t_begin + GRP) : nt;
    if (t_begin >= t_end) continue;
    la.load(ab, 1, K, tc.r0, t_begin * BK, K, M, vec_a, 0.f);
    lc.load(cb, 1, N, tc.c0, t_begin * BK, N, M, vec_c, pinf_f());
    lg.load(gb, 1, N, tc.c0, t_begin * BK, N, M, vec_g, 0.f);
    __syncthreads();
    la.store(sa[0], LDR);
    lc.store_scaled(sc[0], LDC, -kLog2e);
    lg.store(sg[0], LDC);
    __syncthreads();
    for (int t = t_begin; t < t_end; ++t) {
      const int cur = (t - t_begin) & 1;
      if (t + 1 < t_end) {
        la.load(ab, 1, K, tc.r0, (t + 1) * BK, K, M, vec_a, 0.f);
        lc.load(cb, 1, N, tc.c0, (t + 1) * BK, N, M, vec_c, pinf_f());
        lg.load(gb, 1, N, tc.c0, (t + 1) * BK, N, M, vec_g, 0.f);
      }
#pragma unroll
      for (int kk = 0; kk < BK; ++kk) {
        float xa[8], cv[4], gv[4];
        mt.load_x(sa[cur] + kk * LDR, LDR, xa);
        mt.load_y(sc[cur] + kk * LDC, cv);
        mt.load_y(sg[cur] + kk * LDC, gv);
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            acc[i][j] = fmaf(ex2_approx(fmaf(xa[i] + bv[i][j], kLog2e, cv[j])), gv[j], acc[i][j]);
      }
      if (t + 1 < t_end) {
        la.store(sa[cur ^ 1], LDR);
        lc.store_scaled(sc[cur ^ 1], LDC, -kLog2e);
        lg.store(sg[cur ^ 1], LDC);
      }
      __syncthreads();
    }
  }
  store_tile<FLAGGED>(grad_b + (int64_t)tc.bt * K * N, N, K, N, tc, mt, acc);
}

template <bool FLAGGED>
__global__ void __launch_bounds__(NT) dense_log_bwd_b_kernel(const float* __restrict__ a,
                                                             const float* __restrict__ b,
                                                             const float* __restrict__ c,
                                                             const float* __restrict__ g,
                                                             float* __restrict__ grad_b, int M, int K, int N,
                                                             int tiles_r, int tiles_c,
                                                             const int* __restrict__ flags, int64_t total,
                                                             const int* error, int64_t out_count) {
  __shared__ __align__(16) float sa[2][BK * LDR];
  __shared__ __align__(16) float sc[2][BK * LDC];
  __shared__ __align__(16) float sg[2][BK * LDC];
  if (!FLAGGED) {
    log_bwd_b_tile<false>(TileCoord(blockIdx.x, tiles_r, tiles_c), sa, sc, sg, a, b, c, g, grad_b, M, K, N, flags);
    return;
  }
  if (poison_if_failed(error, grad_b, out_count)) return;
  __shared__ int list[NT];
  __shared__ int count;
  const int ngrp = (M + 127) / 128, fpitch = (N + 127) / 128;
  auto flagged = [&](int64_t id) {
    const TileCoord t(id, tiles_r, tiles_c);
    const int* fcol = flags + (int64_t)t.bt * ngrp * fpitch + t.c0 / 128;
    bool any = false;
    for (int q = 0; q < ngrp; ++q) any |= (__ldg(fcol + (int64_t)q * fpitch) != 0);
    return any;
  };
  for (int64_t base = 0; base < total; base += (int64_t)gridDim.x * NT) {
    const int nw = collect_tiles(base, total, list, &count, flagged);
    for (int w = 0; w < nw; ++w) {
      log_bwd_b_tile<true>(TileCoord(list[w], tiles_r, tiles_c), sa, sc, sg, a, b, c, g, grad_b, M, K, N, flags);
      __syncthreads();
    }
  }
}

// ------------------------------------------------------------------ index routing
constexpr int ROUTE_WARPS = 8;

// grad_a: one warp per (batch, m) row.  hist holds KT buckets per warp; K larger than KT is
// covered in passes.  Lanes take 32 consecutive n at a time; lanes that target the same bucket
// add one after another in lane (= n) order so the sum is the reference's ascending-n sum.
constexpr int RU = 8;
template <bool MUL>
__global__ void __launch_bounds__(ROUTE_WARPS * 32) route_grad_a_kernel(const float* __restrict__ b,
                                                                         const int* __restrict__ idx,
                                                                         const float* __restrict__ g,
                                                                         float* __restrict__ grad_a,
                                                                         int64_t rows, int M, int K, int N,
                                                                         int KT) {
  extern __shared__ float hist_all[];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int64_t row = (int64_t)blockIdx.x * ROUTE_WARPS + warp;
  if (row >= rows) return;  // whole warp leaves together
  float* hist = hist_all + warp * KT;
  const int bt = (int)(row / M);
  const int* irow = idx + row * N;
  const float* grow = g + row * N;
  const float* bb = b + (int64_t)bt * K * N;
  for (int kbase = 0; kbase < K; kbase += KT) {
    const int kend = min(kbase + KT, K);
    for (int k = lane; k < kend - kbase; k += 32) hist[k] = 0.f;
    __syncwarp();
    // RU groups of 32 cells are fetched together: the walk is otherwise one global-load latency per group
    for (int n0 = 0; n0 < N; n0 += 32 * RU) {
      int kk[RU];
      float gg[RU];
#pragma unroll
      for (int u = 0; u < RU; ++u) {
        const int n = n0 + u * 32 + lane;
        kk[u] = -1;
        gg[u] = 0.f;
        if (n < N) {
          kk[u] = __ldg(irow + n);
          gg[u] = __ldg(grow + n);
        }
      }
#pragma unroll
      for (int u = 0; u < RU; ++u) {
        const int n = n0 + u * 32 + lane;
        const bool hit = kk[u] >= kbase && kk[u] < kend;
        if (MUL && hit) gg[u] = __fmul_rn(__ldg(bb + (int64_t)kk[u] * N + n), gg[u]);
      }
#pragma unroll
      for (int u = 0; u < RU; ++u) {
        if (n0 + u * 32 >= N) break;
        const int k = kk[u];
        const float gv = gg[u];
        const bool hit = k >= kbase && k < kend;
        // lanes without a target get distinct negative keys so they group with nobody
        const unsigned peers = __match_any_sync(0xffffffffu, hit ? k : -1 - lane);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        const int last = __reduce_max_sync(0xffffffffu, hit ? rank : 0);
        for (int r = 0; r <= last; ++r) {
          if (hit && rank == r) hist[k - kbase] = __fadd_rn(hist[k - kbase], gv);
          __syncwarp();
        }
      }
    }
    for (int k = lane; k < kend - kbase; k += 32) grad_a[row * K + kbase + k] = hist[k];
    __syncwarp();
  }
}

// grad_b: one CTA of 32 warps per (batch, 32 consecutive n).  Rows of idx / g are read 32 at a time
// as coalesced 32x32 tiles and turned through shared memory, after which warp w owns column n0 + w:
// its lanes hold 32 consecutive m, and lanes that target the same bucket add one after another in
// lane (= m) order, so every bucket is the reference's ascending-m sum.  hist: [32 columns][KB + 1].
constexpr int RB_WARPS = 32, RD = 4;
template <bool MUL>
__global__ void __launch_bounds__(RB_WARPS * 32) route_grad_b_kernel(const float* __restrict__ a,
                                                                     const int* __restrict__ idx,
                                                                     const float* __restrict__ g,
                                                                     float* __restrict__ grad_b, int M, int K, int N,
                                                                     int tiles_n, int KB) {
  extern __shared__ float hist_all[];
  __shared__ int si[2][32][33];
  __shared__ float sg[2][32][33];
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  const int n0 = (blockIdx.x % tiles_n) * 32;
  const int bt = blockIdx.x / tiles_n;
  const int* ib = idx + (int64_t)bt * M * N;
  const float* gb = g + (int64_t)bt * M * N;
  const float* ab = a + (int64_t)bt * M * K;
  float* ob = grad_b + (int64_t)bt * K * N;
  float* hist = hist_all + warp * (KB + 1);
  const int nl = n0 + lane;  // column this thread loads; warp = row offset within the tile
  for (int kbase = 0; kbase < K; kbase += KB) {
    const int kend = min(kbase + KB, K);
    for (int k = lane; k < kend - kbase; k += 32) hist[k] = 0.f;
    // RD tiles are in flight in registers: the walk is otherwise one global-load latency per tile
    int kq[RD];
    float gq[RD];
    auto fetch = [&](int m, int& kn, float& gn) {
      kn = -1;
      gn = 0.f;
      if (m < M && nl < N) {
        kn = __ldg(ib + (int64_t)m * N + nl);
        gn = __ldg(gb + (int64_t)m * N + nl);
        if (kn < kbase || kn >= kend) kn = -1;
        if (MUL && kn >= 0) gn = __fmul_rn(__ldg(ab + (int64_t)m * K + kn), gn);
      }
    };
#pragma unroll
    for (int u = 0; u < RD; ++u) fetch(u * 32 + warp, kq[u], gq[u]);
    for (int mb = 0; mb < M; mb += 32 * RD) {
#pragma unroll
      for (int u = 0; u < RD; ++u) {
        const int m0 = mb + u * 32;
        if (m0 >= M) break;
        // buffer u & 1 was last read two tiles ago, before the previous tile's barrier
        si[u & 1][warp][lane] = kq[u];
        sg[u & 1][warp][lane] = gq[u];
        fetch(m0 + 32 * RD + warp, kq[u], gq[u]);
        __syncthreads();
        const int k = si[u & 1][lane][warp];  // lane = m offset, warp = column
        const float gv = sg[u & 1][lane][warp];
        const bool hit = k >= 0;
        // lanes without a target get distinct negative keys so they group with nobody
        const unsigned peers = __match_any_sync(0xffffffffu, hit ? k : -1 - lane);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        const int last = __reduce_max_sync(0xffffffffu, hit ? rank : 0);
        for (int r = 0; r <= last; ++r) {
          if (hit && rank == r) hist[k - kbase] = __fadd_rn(hist[k - kbase], gv);
          __syncwarp();
        }
      }
    }
    __syncthreads();
    // bucket k of all 32 columns is one 128-byte row of grad_b
    if (nl < N)
      for (int k = warp; k < kend - kbase; k += RB_WARPS)
        ob[(int64_t)(kbase + k) * N + nl] = hist_all[lane * (KB + 1) + k];
    __syncthreads();
  }
}

// grad_b for short reductions (K floats of shared memory per thread): one THREAD per column (batch, n).  It walks
// m upwards — the lanes of a warp are consecutive n, so every step is one coalesced read of idx and of g — and adds
// each cotangent to the bucket its index names in a private K-bucket histogram (odd pitch): ascending-m sums
// with no ranking of lanes that share a bucket, which is what the kernel above spends its time on.  Eight steps
// are fetched together and the next eight requested before these are added up.
constexpr int RC_T = 128;   // threads per CTA at most; fewer when K is longer (K floats of shared memory each)
template <bool MUL>
__global__ void __launch_bounds__(RC_T) route_grad_b_cols_kernel(const float* __restrict__ a,
                                                                 const int* __restrict__ idx,
                                                                 const float* __restrict__ g,
                                                                 float* __restrict__ grad_b, int M, int K, int N,
                                                                 int64_t cols) {
  extern __shared__ float hist_all[];
  const int pitch = K | 1;
  float* hist = hist_all + threadIdx.x * pitch;
  for (int k = 0; k < K; ++k) hist[k] = 0.f;
  const int64_t col = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = col < cols;
  const int64_t bt = live ? col / N : 0;
  const int n = live ? (int)(col % N) : 0;
  const int* ip = idx + bt * M * N + n;
  const float* gp = g + bt * M * N + n;
  const float* ab = a + bt * M * K;
  constexpr int U = 8;
  int kq[2][U];
  float gq[2][U];
  auto fetch = [&](int m0, int (&kd)[U], float (&gd)[U]) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int m = m0 + u;
      const bool ok = live && m < M;
      kd[u] = ok ? __ldg(ip + (int64_t)m * N) : -1;
      gd[u] = ok ? __ldg(gp + (int64_t)m * N) : 0.f;
    }
    if (MUL) {
#pragma unroll
      for (int u = 0; u < U; ++u)
        if ((unsigned)kd[u] < (unsigned)K) gd[u] = __fmul_rn(__ldg(ab + (int64_t)(m0 + u) * K + kd[u]), gd[u]);
    }
  };
  auto add_up = [&](const int (&kd)[U], const float (&gd)[U]) {
#pragma unroll
    for (int u = 0; u < U; ++u)
      if ((unsigned)kd[u] < (unsigned)K) hist[kd[u]] = __fadd_rn(hist[kd[u]], gd[u]);
  };
  fetch(0, kq[0], gq[0]);
  for (int m0 = 0; m0 < M; m0 += 2 * U) {
    fetch(m0 + U, kq[1], gq[1]);
    add_up(kq[0], gq[0]);
    fetch(m0 + 2 * U, kq[0], gq[0]);
    add_up(kq[1], gq[1]);
  }
  if (live) {
    float* ob = grad_b + bt * K * N + n;
    for (int k = 0; k < K; ++k) ob[(int64_t)k * N] = hist[k];
  }
}

}  // namespace
}  // namespace gbmm

namespace gbmm {
// Exact recomputation of the gradient terms of the result tiles marked in `flags`, added to
// grad_a / grad_b (see dense.cuh).
int launch_log_bwd_flagged(const float* a, const float* b, const float* c, const float* g, float* grad_a,
                           float* grad_b, const int* flags, int64_t B, int64_t M, int64_t K, int64_t N,
                           cudaStream_t st, const int* error) {
  const int m = (int)M, k = (int)K, n = (int)N;
  if (grad_a) {
    const int64_t tr = ceil_div(M, BR), tcn = ceil_div(K, BC), blocks = B * tr * tcn;
    if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
    unsigned grid = 0;
    if (int rc = capped_grid(blocks, &grid)) return rc;
    dense_log_bwd_a_kernel<true><<<grid, NT, 0, st>>>(a, b, c, g, grad_a, m, k, n, (int)tr, (int)tcn, flags, blocks,
                                                      error, B * M * K);
    if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
  }
  if (grad_b) {
    const int64_t tr = ceil_div(K, BR), tcn = ceil_div(N, BC), blocks = B * tr * tcn;
    if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
    unsigned grid = 0;
    if (int rc = capped_grid(blocks, &grid)) return rc;
    dense_log_bwd_b_kernel<true><<<grid, NT, 0, st>>>(a, b, c, g, grad_b, m, k, n, (int)tr, (int)tcn, flags, blocks,
                                                      error, B * K * N);
  }
  return launch_status();
}
}  // namespace gbmm

using namespace gbmm;

extern "C" int gbmm_dense_backward_f32(int mode, const float* a, const float* b, const float* grad_out,
                                       const float* part, const void* aux, float* grad_a, float* grad_b,
                                       int64_t B, int64_t M, int64_t K, int64_t N, void* stream) {
  if (mode < 0 || mode > 3) return GBMM_ERR_INVALID_ARG;
  if (B < 0 || M < 0 || K < 0 || N < 0) return GBMM_ERR_INVALID_ARG;
  if (B == 0 || K == 0) return GBMM_OK;  // both gradients are empty
  if (M >= (1LL << 31) - BR || K >= (1LL << 31) - BR || N >= (1LL << 31) - BR) return GBMM_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (M == 0 || N == 0) {
    // empty reduction: the non-empty gradient is all zeros
    if (grad_a && M > 0 && cudaMemsetAsync(grad_a, 0, sizeof(float) * B * M * K, st) != cudaSuccess)
      return GBMM_ERR_LAUNCH;
    if (grad_b && N > 0 && cudaMemsetAsync(grad_b, 0, sizeof(float) * B * K * N, st) != cudaSuccess)
      return GBMM_ERR_LAUNCH;
    return GBMM_OK;
  }
  if (!a || !b || !grad_out) return GBMM_ERR_INVALID_ARG;
  const int m = (int)M, k = (int)K, n = (int)N;
  if (mode == GBMM_MODE_LOG) {
    if (!part) return GBMM_ERR_INVALID_ARG;
    {  // small problems: 32x32 tiles, both gradients in one launch (dense_small.cu)
      const int64_t big_a = B * ceil_div(M, BR) * ceil_div(K, BC), big_b = B * ceil_div(K, BR) * ceil_div(N, BC);
      if (small_log_wanted(big_a > big_b ? big_a : big_b))
        return launch_small_log_bwd(a, b, part, grad_out, grad_a, grad_b, B, M, K, N, st);
    }
    if (grad_a) {
      const int64_t tr = ceil_div(M, BR), tcn = ceil_div(K, BC), blocks = B * tr * tcn;
      if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
      dense_log_bwd_a_kernel<false><<<(unsigned)blocks, NT, 0, st>>>(a, b, part, grad_out, grad_a, m, k, n,
                                                                     (int)tr, (int)tcn, nullptr, blocks, nullptr, 0);
      if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
    }
    if (grad_b) {
      const int64_t tr = ceil_div(K, BR), tcn = ceil_div(N, BC), blocks = B * tr * tcn;
      if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
      dense_log_bwd_b_kernel<false><<<(unsigned)blocks, NT, 0, st>>>(a, b, part, grad_out, grad_b, m, k, n,
                                                                     (int)tr, (int)tcn, nullptr, blocks, nullptr, 0);
    }
    return launch_status();
  }
  if (!aux) return GBMM_ERR_INVALID_ARG;
  const int* idx = static_cast<const int*>(aux);
  const bool mul = (mode == GBMM_MODE_PRODMAX);
  if (grad_a) {
    const int KT = (int)(K < 2048 ? K : 2048);
    const int64_t rows = B * M, blocks = ceil_div(rows, ROUTE_WARPS);
    if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
    const size_t smem = sizeof(float) * ROUTE_WARPS * KT;
    if (mul) {
      cudaFuncSetAttribute(route_grad_a_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      route_grad_a_kernel<true><<<(unsigned)blocks, ROUTE_WARPS * 32, smem, st>>>(b, idx, grad_out, grad_a, rows,
                                                                                 m, k, n, KT);
    } else {
      cudaFuncSetAttribute(route_grad_a_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      route_grad_a_kernel<false><<<(unsigned)blocks, ROUTE_WARPS * 32, smem, st>>>(b, idx, grad_out, grad_a,
                                                                                  rows, m, k, n, KT);
    }
    if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
  }
  if (grad_b) {
    // up to 1024 buckets per column (131 KB of shared memory) per pass
    const int KB = (int)(K < 1024 ? K : 1024);
    const int64_t tiles_n = ceil_div(N, 32), blocks = B * tiles_n;
    if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
    const size_t smem = sizeof(float) * 32 * (KB + 1);
    // short reductions: one thread per column with a private histogram (GENBMM_B200_ROUTE_B=w keeps the kernel below)
    int ct = RC_T;   // 128, 64 or 32 threads per CTA, so that a CTA's histograms stay below 100 KB
    while (ct > 32 && sizeof(float) * ct * (size_t)(K | 1) > (size_t)100 * 1024) ct /= 2;
    const size_t smem_cols = sizeof(float) * ct * (size_t)(K | 1);
    const char* eb = getenv("GENBMM_B200_ROUTE_B");
    if (smem_cols <= (size_t)100 * 1024 && !(eb && eb[0] == 'w')) {
      const int64_t cols = B * N, cblocks = ceil_div(cols, ct);
      if (cblocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
      if (mul) {
        cudaFuncSetAttribute(route_grad_b_cols_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_cols);
        route_grad_b_cols_kernel<true><<<(unsigned)cblocks, ct, smem_cols, st>>>(a, idx, grad_out, grad_b, m, k, n, cols);
      } else {
        cudaFuncSetAttribute(route_grad_b_cols_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_cols);
        route_grad_b_cols_kernel<false><<<(unsigned)cblocks, ct, smem_cols, st>>>(a, idx, grad_out, grad_b, m, k, n, cols);
      }
      return launch_status();
    }
    if (mul) {
      cudaFuncSetAttribute(route_grad_b_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      route_grad_b_kernel<true><<<(unsigned)blocks, RB_WARPS * 32, smem, st>>>(a, idx, grad_out, grad_b, m, k, n,
                                                                              (int)tiles_n, KB);
    } else {
      cudaFuncSetAttribute(route_grad_b_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      route_grad_b_kernel<false><<<(unsigned)blocks, RB_WARPS * 32, smem, st>>>(a, idx, grad_out, grad_b, m, k, n,
                                                                               (int)tiles_n, KB);
    }
  }
  return launch_status();
}
