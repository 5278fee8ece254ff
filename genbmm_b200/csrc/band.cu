// Banded semiring products in the reference's diagonal storage:
//   data:(B,n,W), W = lu+ld+1, data[b,i,j] = Dense[b, i+j-lu, i].
//
// Index algebra (banded_cuda_kernel.cu:28-36,48-49,123,132-133), with Wa, Wb the operand
// widths, r_lu = a_lu+b_ld, Wo = Wa+Wb-1: a triple (i, ja, jo) couples
//   a[i][ja],  b[o][k2],  out[i][jo]   with  o = i+jo-r_lu,  k2 = ja-jo+Wb-1,
// and exists when 0 <= o < n, 0 <= k2 < Wb and the shared dense index p = i+ja-a_lu lies in
// [0,n).  Forward reduces over ja, grad_a over jo, grad_b (cell (o,k2)) over i.
//
// Replaces banded_cuda_forward_kernel_mul / banded_cuda_backward_kernel_mul
// (banded_cuda_kernel.cu:13-152), which map lanes to rows (every load strided by W) and get
// grad_b from a second launch on band-transposed copies.  Here lanes run along the contiguous
// band axis, a CTA stages the rows it needs in shared memory (the b rows with an even pitch,
// so that the skewed access b[o(j)][k2(j)] of consecutive lanes hits distinct banks), only
// the outputs a mode needs are written, and grad_b is computed directly.
// When the rows of a CTA do not fit in shared memory the same code reads global memory.
#include "band.cuh"

namespace gbmm {
namespace {

constexpr int NT = 256;
constexpr int kSmemBudget = 200 * 1024;

// A window of consecutive matrix rows, either staged in shared memory or the tensor itself.
template <typename T>
struct Rows {
  const T* p;
  int pitch;
  int64_t row0;
  __device__ __forceinline__ T at(int64_t row, int col) const { return p[(row - row0) * pitch + col]; }
};

// Cooperative copy of rows [row0, row0+cnt) of a (n, W) matrix into shared memory with the
// given pitch; rows outside [0,n) are zero-filled.  One warp per row, lanes along the row.
template <typename T>
__device__ __forceinline__ void stage_rows(T* dst, int pitch, const T* src, int W, int64_t row0, int cnt,
                                           int64_t n) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  for (int r = warp; r < cnt; r += NT / 32) {
    const int64_t row = row0 + r;
    const bool ok = row >= 0 && row < n;
    for (int c = lane; c < W; c += 32) dst[r * pitch + c] = ok ? __ldg(src + row * W + c) : T(0);
  }
}

// even pitch for b rows: consecutive lanes step by pitch-1 floats, which must be odd
__host__ __device__ inline int b_pitch(int Wb) { return (Wb & 1) ? Wb + 1 : Wb; }

// ------------------------------------------------------------------ forward
template <int MODE>
__device__ __forceinline__ void band_fwd_tile(const int64_t tile_id, const float* __restrict__ a, const float* __restrict__ b,
                                                      float* __restrict__ out, int* __restrict__ idx,
                                                      float* __restrict__ maxes, BandDims d, int TI,
                                                      int tiles_i, int staged, const int* __restrict__ flags) {
  extern __shared__ float smem[];
  const int Wa = d.Wa(), Wb = d.Wb(), Wo = d.Wo(), r_lu = d.r_lu();
  const int64_t n = d.n;
  const int64_t bt = tile_id / tiles_i;
  const int64_t i0 = (int64_t)(tile_id % tiles_i) * TI;
  // behind the block-banded fast path only the flagged 64-row blocks are recomputed
  if (flags && __ldg(flags + bt * ((n + 63) / 64) + i0 / 64) == 0) return;
  const float* ab = a + bt * n * Wa;
  const float* bb = b + bt * n * Wb;
  Rows<float> va{ab, Wa, 0}, vb{bb, Wb, 0};
  if (staged) {
    float* sa = smem;
    float* sb = smem + TI * Wa;
    const int ldb = b_pitch(Wb);
    stage_rows(sa, Wa, ab, Wa, i0, TI, n);
    stage_rows(sb, ldb, bb, Wb, i0 - r_lu, TI + Wo - 1, n);
    __syncthreads();
    va = Rows<float>{sa, Wa, i0};
    vb = Rows<float>{sb, ldb, i0 - r_lu};
  }
  const int total = TI * Wo;
  for (int e = threadIdx.x; e < total; e += NT) {
    const int il = e / Wo, jo = e - il * Wo;
    const int64_t i = i0 + il;
    if (i >= n) break;
    const int64_t oi = (bt * n + i) * Wo + jo;
    const int64_t o = i + jo - r_lu;
    if (o < 0 || o >= n) {  // outside the matrix: the reference leaves its zero fill
      out[oi] = 0.f;
      if (MODE == GBMM_BAND_MAX && idx) idx[oi] = 0;
      if (MODE == GBMM_BAND_LOG && maxes) maxes[oi] = 0.f;
      continue;
    }
    // valid ja: k2 = ja-jo+Wb-1 in [0,Wb) and p = i+ja-a_lu in [0,n)
    int lo = max(0, jo - (Wb - 1));
    int hi = min(Wa - 1, jo);
    lo = (int)max((int64_t)lo, (int64_t)d.a_lu - i);
    hi = (int)min((int64_t)hi, n - 1 - i + d.a_lu);
    const int kofs = Wb - 1 - jo;
    if (MODE == GBMM_BAND_MUL) {
      float val = 0.f;
#pragma unroll 8
      for (int ja = lo; ja <= hi; ++ja) val = fmaf(va.at(i, ja), vb.at(o, ja + kofs), val);
      out[oi] = val;
    } else if (MODE == GBMM_BAND_MAX) {
      float m = kFloor;
      int ind = -1;
#pragma unroll 8
      for (int ja = lo; ja <= hi; ++ja) {
        const float v = __fadd_rn(va.at(i, ja), vb.at(o, ja + kofs));
        if (v > m) {
          m = v;
          ind = ja;
        }
      }
      out[oi] = m;
      if (idx) idx[oi] = ind;
    } else {
      float m = kFloor;
#pragma unroll 8
      for (int ja = lo; ja <= hi; ++ja) m = fmaxf(m, va.at(i, ja) + vb.at(o, ja + kofs));
      float s = 0.f;
#pragma unroll 8
      for (int ja = lo; ja <= hi; ++ja) s += exp_sfu((va.at(i, ja) + vb.at(o, ja + kofs)) - m);
      out[oi] = logf(s) + m;
      if (maxes) maxes[oi] = m;
    }
  }
}

// LISTED false: one tile per CTA (grid = `total` tiles).  LISTED true (behind a fast path, flags != nullptr):
// a capped grid whose CTAs gather the tiles that have flagged rows and work through them.
template <int MODE, bool LISTED>
__global__ void __launch_bounds__(NT) band_fwd_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                                                      int* __restrict__ idx, float* __restrict__ maxes, BandDims d, int TI,
                                                      int tiles_i, int staged, const int* __restrict__ flags, int64_t total) {
  if (!LISTED) {
    band_fwd_tile<MODE>(blockIdx.x, a, b, out, idx, maxes, d, TI, tiles_i, staged, flags);
    return;
  }
  __shared__ int list[NT];
  __shared__ int count;
  const int64_t fb = (d.n + 63) / 64;
  auto flagged = [&](int64_t id) {
    return __ldg(flags + (id / tiles_i) * fb + ((id % tiles_i) * TI) / 64) != 0;
  };
  for (int64_t base = 0; base < total; base += (int64_t)gridDim.x * NT) {
    const int nw = collect_tiles(base, total, list, &count, flagged);
    for (int w = 0; w < nw; ++w) {
      band_fwd_tile<MODE>(list[w], a, b, out, idx, maxes, d, TI, tiles_i, staged, flags);
      __syncthreads();
    }
  }
}

// ------------------------------------------------------------------ grad_a
template <int MODE>
__device__ __forceinline__ void band_bwd_a_tile(const int64_t tile_id, const float* __restrict__ a, const float* __restrict__ b,
                                                        const float* __restrict__ g, const void* __restrict__ part,
                                                        float* __restrict__ grad_a, BandDims d, int TI,
                                                        int tiles_i, int staged, const int* __restrict__ flags) {
  extern __shared__ float smem[];
  const int Wa = d.Wa(), Wb = d.Wb(), Wo = d.Wo(), r_lu = d.r_lu();
  const int64_t n = d.n;
  const int64_t bt = tile_id / tiles_i;
  const int64_t i0 = (int64_t)(tile_id % tiles_i) * TI;
  if (flags && __ldg(flags + bt * ((n + 63) / 64) + i0 / 64) == 0) return;  // rows of flagged blocks only
  const float* ab = a + bt * n * Wa;
  const float* bb = b + bt * n * Wb;
  const float* gb = g + bt * n * Wo;
  const float* pf = (MODE == GBMM_BAND_LOG) ? static_cast<const float*>(part) + bt * n * Wo : nullptr;
  const int* pi = (MODE == GBMM_BAND_MAX) ? static_cast<const int*>(part) + bt * n * Wo : nullptr;
  Rows<float> vb{bb, Wb, 0}, vg{gb, Wo, 0}, vpf{pf, Wo, 0};
  Rows<int> vpi{pi, Wo, 0};
  if (staged) {
    const int ldb = b_pitch(Wb);
    float* sb = smem;
    float* sg = sb + (TI + Wo - 1) * ldb;
    float* sp = sg + TI * Wo;
    stage_rows(sb, ldb, bb, Wb, i0 - r_lu, TI + Wo - 1, n);
    stage_rows(sg, Wo, gb, Wo, i0, TI, n);
    if (MODE == GBMM_BAND_LOG) stage_rows(sp, Wo, pf, Wo, i0, TI, n);
    if (MODE == GBMM_BAND_MAX) stage_rows(reinterpret_cast<int*>(sp), Wo, pi, Wo, i0, TI, n);
    __syncthreads();
    vb = Rows<float>{sb, ldb, i0 - r_lu};
    vg = Rows<float>{sg, Wo, i0};
    vpf = Rows<float>{sp, Wo, i0};
    vpi = Rows<int>{reinterpret_cast<int*>(sp), Wo, i0};
  }
  const int total = TI * Wa;
  for (int e = threadIdx.x; e < total; e += NT) {
    const int il = e / Wa, ja = e - il * Wa;
    const int64_t i = i0 + il;
    if (i >= n) break;
    const int64_t ai = (bt * n + i) * Wa + ja;
    const int64_t p = i + ja - d.a_lu;
    float val = 0.f;
    if (p >= 0 && p < n) {
      // valid jo: k2 = ja-jo+Wb-1 in [0,Wb) and o = i+jo-r_lu in [0,n)
      int lo = ja, hi = min(Wo - 1, ja + Wb - 1);
      lo = (int)max((int64_t)lo, (int64_t)r_lu - i);
      hi = (int)min((int64_t)hi, n - 1 - i + r_lu);
      const float av = (MODE == GBMM_BAND_LOG) ? __ldg(ab + (i * Wa + ja)) : 0.f;
#pragma unroll 8
      for (int jo = lo; jo <= hi; ++jo) {
        const int64_t o = i + jo - r_lu;
        const int k2 = ja - jo + Wb - 1;
        if (MODE == GBMM_BAND_MUL) {
          val = fmaf(vb.at(o, k2), vg.at(i, jo), val);
        } else if (MODE == GBMM_BAND_MAX) {
          if (vpi.at(i, jo) == ja) val = __fadd_rn(val, vg.at(i, jo));
        } else {
          val = fmaf(exp_sfu((av + vb.at(o, k2)) - vpf.at(i, jo)), vg.at(i, jo), val);
        }
      }
    }
    grad_a[ai] = val;
  }
}

// LISTED false: one tile per CTA (grid = `total` tiles).  LISTED true (behind a fast path, flags != nullptr):
// a capped grid whose CTAs gather the tiles that have flagged rows and work through them.
template <int MODE, bool LISTED>
__global__ void __launch_bounds__(NT) band_bwd_a_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                        const float* __restrict__ g, const void* __restrict__ part,
                                                        float* __restrict__ grad_a, BandDims d, int TI, int tiles_i,
                                                        int staged, const int* __restrict__ flags, int64_t total) {
  if (!LISTED) {
    band_bwd_a_tile<MODE>(blockIdx.x, a, b, g, part, grad_a, d, TI, tiles_i, staged, flags);
    return;
  }
  __shared__ int list[NT];
  __shared__ int count;
  const int64_t fb = (d.n + 63) / 64;
  auto flagged = [&](int64_t id) {
    return __ldg(flags + (id / tiles_i) * fb + ((id % tiles_i) * TI) / 64) != 0;
  };
  for (int64_t base = 0; base < total; base += (int64_t)gridDim.x * NT) {
    const int nw = collect_tiles(base, total, list, &count, flagged);
    for (int w = 0; w < nw; ++w) {
      band_bwd_a_tile<MODE>(list[w], a, b, g, part, grad_a, d, TI, tiles_i, staged, flags);
      __syncthreads();
    }
  }
}

// ------------------------------------------------------------------ grad_b
// CTA owns TO consecutive rows o of b; the contributing rows i = o-jo+r_lu span
// [o0-(Wo-1-r_lu), o0+TO-1+r_lu] and are walked in ascending chunks of TI rows.
template <int MODE>
__device__ __forceinline__ void band_bwd_b_tile(const int64_t tile_id, const float* __restrict__ a, const float* __restrict__ b,
                                                        const float* __restrict__ g, const void* __restrict__ part,
                                                        float* __restrict__ grad_b, BandDims d, int TO, int TI,
                                                        int tiles_o, int staged, const int* __restrict__ flags) {
  extern __shared__ float smem[];
  const int Wa = d.Wa(), Wb = d.Wb(), Wo = d.Wo(), r_lu = d.r_lu();
  const int r_ld = Wo - 1 - r_lu;
  const int64_t n = d.n;
  const int64_t bt = tile_id / tiles_o;
  const int64_t o0 = (int64_t)(tile_id % tiles_o) * TO;
  const float* ab = a + bt * n * Wa;
  const float* bb = b + bt * n * Wb;
  const float* gb = g + bt * n * Wo;
  const float* pf = (MODE == GBMM_BAND_LOG) ? static_cast<const float*>(part) + bt * n * Wo : nullptr;
  const int* pi = (MODE == GBMM_BAND_MAX) ? static_cast<const int*>(part) + bt * n * Wo : nullptr;
  float* ob = grad_b + bt * n * Wb;

  const int64_t i_begin = max((int64_t)0, o0 - r_ld);
  const int64_t i_end = min(n, o0 + TO + r_lu);  // exclusive
  const int total = TO * Wb;
  // With flags (behind the block-banded fast path) only rows i of flagged 64-row blocks
  // contribute and the sums are added to what the fast kernel wrote.
  const int* frow = flags ? flags + bt * ((n + 63) / 64) : nullptr;
  if (frow) {
    bool any = false;
    for (int64_t q = i_begin / 64; q <= (i_end - 1) / 64; ++q) any |= (__ldg(frow + q) != 0);
    if (!any) return;
  }

  float* acc = smem;             // [TO*Wb], staged mode only
  float* sa = acc + TO * Wb;     // [TI*Wa]
  float* sg = sa + TI * Wa;      // [TI*Wo]
  float* sp = sg + TI * Wo;      // [TI*Wo]
  if (staged) {
    for (int e = threadIdx.x; e < total; e += NT) acc[e] = 0.f;
  }
  const int64_t step = staged ? TI : (i_end - i_begin > 0 ? i_end - i_begin : 1);
  for (int64_t c0 = i_begin; c0 < i_end; c0 += step) {
    const int64_t c1 = min(i_end, c0 + step);
    Rows<float> va{ab, Wa, 0}, vg{gb, Wo, 0}, vpf{pf, Wo, 0};
    Rows<int> vpi{pi, Wo, 0};
    if (staged) {
      __syncthreads();  // previous chunk fully consumed
      stage_rows(sa, Wa, ab, Wa, c0, (int)(c1 - c0), n);
      stage_rows(sg, Wo, gb, Wo, c0, (int)(c1 - c0), n);
      if (MODE == GBMM_BAND_LOG) stage_rows(sp, Wo, pf, Wo, c0, (int)(c1 - c0), n);
      if (MODE == GBMM_BAND_MAX) stage_rows(reinterpret_cast<int*>(sp), Wo, pi, Wo, c0, (int)(c1 - c0), n);
      __syncthreads();
      va = Rows<float>{sa, Wa, c0};
      vg = Rows<float>{sg, Wo, c0};
      vpf = Rows<float>{sp, Wo, c0};
      vpi = Rows<int>{reinterpret_cast<int*>(sp), Wo, c0};
    }
    for (int e = threadIdx.x; e < total; e += NT) {
      const int ol = e / Wb, k2 = e - ol * Wb;
      const int64_t o = o0 + ol;
      if (o >= n) break;
      const int64_t p = o + k2 - d.b_lu;
      float val = staged ? acc[e] : 0.f;
      if (p >= 0 && p < n) {
        // i = o - jo + r_lu with jo in [0,Wo) and ja = k2+jo-(Wb-1) in [0,Wa)
        //   => jo in [Wb-1-k2, Wb-1-k2+Wa-1]  =>  i in [o+r_lu-(Wb-1-k2+Wa-1), o+r_lu-(Wb-1-k2)]
        int64_t lo = o + r_lu - (Wb - 1 - k2 + Wa - 1);
        int64_t hi = o + r_lu - (Wb - 1 - k2);
        lo = max(lo, c0);
        hi = min(hi, c1 - 1);
        const float bv = (MODE == GBMM_BAND_LOG) ? __ldg(bb + (o * Wb + k2)) : 0.f;
#pragma unroll 4
        for (int64_t i = lo; i <= hi; ++i) {
          if (frow && __ldg(frow + i / 64) == 0) continue;
          const int jo = (int)(o - i + r_lu);
          const int ja = k2 + jo - (Wb - 1);
          if (MODE == GBMM_BAND_MUL) {
            val = fmaf(va.at(i, ja), vg.at(i, jo), val);
          } else if (MODE == GBMM_BAND_MAX) {
            if (vpi.at(i, jo) == ja) val = __fadd_rn(val, vg.at(i, jo));
          } else {
            val = fmaf(exp_sfu((va.at(i, ja) + bv) - vpf.at(i, jo)), vg.at(i, jo), val);
          }
        }
      }
      if (staged)
        acc[e] = val;
      else
        ob[o * Wb + k2] = frow ? ob[o * Wb + k2] + val : val;
    }
  }
  if (staged) {
    // each thread re-reads only the slots it wrote itself
    for (int e = threadIdx.x; e < total; e += NT) {
      const int ol = e / Wb;
      if (o0 + ol >= n) break;
      float* dst = ob + (o0 + ol) * Wb + (e - ol * Wb);
      *dst = frow ? *dst + acc[e] : acc[e];
    }
  } else if (i_begin >= i_end && !frow) {
    for (int e = threadIdx.x; e < total; e += NT) {
      const int ol = e / Wb;
      if (o0 + ol >= n) break;
      ob[(o0 + ol) * Wb + (e - ol * Wb)] = 0.f;
    }
  }
}

// LISTED false: one tile per CTA (grid = `total` tiles).  LISTED true (behind a fast path, flags != nullptr):
// a capped grid whose CTAs gather the tiles that have flagged rows and work through them.
template <int MODE, bool LISTED>
__global__ void __launch_bounds__(NT) band_bwd_b_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                        const float* __restrict__ g, const void* __restrict__ part,
                                                        float* __restrict__ grad_b, BandDims d, int TO, int TI,
                                                        int tiles_o, int staged, const int* __restrict__ flags, int64_t total) {
  if (!LISTED) {
    band_bwd_b_tile<MODE>(blockIdx.x, a, b, g, part, grad_b, d, TO, TI, tiles_o, staged, flags);
    return;
  }
  __shared__ int list[NT];
  __shared__ int count;
  const int64_t fb = (d.n + 63) / 64;
  const int r_lu = d.r_lu(), r_ld = d.Wo() - 1 - r_lu;
  auto flagged = [&](int64_t id) {
    const int64_t o0 = (id % tiles_o) * TO;
    const int64_t i_begin = max((int64_t)0, o0 - r_ld), i_end = min(d.n, o0 + TO + r_lu);
    const int* frow = flags + (id / tiles_o) * fb;
    bool any = false;
    for (int64_t q = i_begin / 64; q <= (i_end - 1) / 64; ++q) any |= (__ldg(frow + q) != 0);
    return any;
  };
  for (int64_t base = 0; base < total; base += (int64_t)gridDim.x * NT) {
    const int nw = collect_tiles(base, total, list, &count, flagged);
    for (int w = 0; w < nw; ++w) {
      band_bwd_b_tile<MODE>(list[w], a, b, g, part, grad_b, d, TO, TI, tiles_o, staged, flags);
      __syncthreads();
    }
  }
}

// ------------------------------------------------------------------ max semiring: index routing
// Each result cell (i, jo) hands its cotangent to exactly one cell of each operand, the one its
// saved argmax names: grad_a[i][ja] with ja = idx[i][jo], and grad_b[o][k2] with o = i+jo-r_lu,
// k2 = ja-jo+Wb-1.  O(n*Wo) work instead of the O(n*Wa*Wb) comparisons of
// banded_cuda_kernel.cu:139-141; sums run in ascending jo (grad_a) and ascending i (grad_b), the
// order of the reference's loops (its grad_b comes from the operand-swapped call, which walks
// the same cells in ascending i).

// grad_a: one warp per row i; lanes take 32 consecutive jo, same-target lanes add in lane order.
constexpr int RUB = 9;
__global__ void __launch_bounds__(256) band_route_a_kernel(const int* __restrict__ idx, const float* __restrict__ g,
                                                           float* __restrict__ grad_a, int64_t rows, BandDims d) {
  extern __shared__ float hist_all[];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;
  if (row >= rows) return;
  const int Wa = d.Wa(), Wb = d.Wb(), Wo = d.Wo(), r_lu = d.r_lu();
  const int64_t n = d.n, i = row % n;
  float* hist = hist_all + warp * Wa;
  for (int k = lane; k < Wa; k += 32) hist[k] = 0.f;
  __syncwarp();
  // RUB groups of 32 cells are fetched together (a 257-wide result band is one batch): the walk is
  // otherwise one global-load latency per group
  for (int j0 = 0; j0 < Wo; j0 += 32 * RUB) {
    int kk[RUB];
    float gg[RUB];
#pragma unroll
    for (int u = 0; u < RUB; ++u) {
      const int jo = j0 + u * 32 + lane;
      kk[u] = -1;
      gg[u] = 0.f;
      if (jo < Wo) {
        kk[u] = __ldg(idx + row * Wo + jo);
        gg[u] = __ldg(g + row * Wo + jo);
      }
    }
#pragma unroll
    for (int u = 0; u < RUB; ++u) {
      if (j0 + u * 32 >= Wo) break;
      const int jo = j0 + u * 32 + lane;
      const int k = kk[u];
      const float gv = gg[u];
      bool hit = false;
      if (jo < Wo) {
        const int64_t o = i + jo - r_lu;
        const int k2 = k - jo + Wb - 1;
        const int64_t p = i + k - d.a_lu;
        hit = o >= 0 && o < n && k >= 0 && k < Wa && k2 >= 0 && k2 < Wb && p >= 0 && p < n;
      }
      const unsigned peers = __match_any_sync(0xffffffffu, hit ? k : -1 - lane);
      const int rank = __popc(peers & ((1u << lane) - 1u));
      const int last = __reduce_max_sync(0xffffffffu, hit ? rank : 0);
      for (int r = 0; r <= last; ++r) {
        if (hit && rank == r) hist[k] = __fadd_rn(hist[k], gv);
        __syncwarp();
      }
    }
  }
  for (int k = lane; k < Wa; k += 32) grad_a[row * Wa + k] = hist[k];
}

// grad_b: one CTA of 32 warps per 32 consecutive rows o of b.  The cells (i, jo = o - i + r_lu) that feed
// row o lie on an anti-diagonal of idx / g, so rows i are taken 32 at a time as coalesced 32 x 63 tiles and
// turned through shared memory: warp w then owns o = o0 + w, its lanes 32 consecutive i, and lanes that
// target the same bucket k2 add one after another in lane (= i) order — the ascending-i sum a sequential
// walk would give.  hist: [32 rows o][Wb + 1].
constexpr int PD = 2;
__global__ void __launch_bounds__(1024) band_route_b_kernel(const int* __restrict__ idx, const float* __restrict__ g,
                                                            float* __restrict__ grad_b, BandDims d, int tiles_o) {
  extern __shared__ float hist_all[];
  __shared__ int si[32][66];
  __shared__ float sg[32][66];
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  const int Wa = d.Wa(), Wb = d.Wb(), Wo = d.Wo(), r_lu = d.r_lu(), r_ld = Wo - 1 - r_lu;
  const int64_t n = d.n;
  const int64_t bt = blockIdx.x / tiles_o;
  const int64_t o0 = (int64_t)(blockIdx.x % tiles_o) * 32, o = o0 + warp;
  const int* ib = idx + bt * n * Wo;
  const float* gb = g + bt * n * Wo;
  float* hist = hist_all + warp * (Wb + 1);
  for (int k = lane; k < Wb; k += 32) hist[k] = 0.f;
  const int64_t i_lo = max((int64_t)0, o0 - r_ld), i_hi = min(n - 1, o0 + 31 + r_lu);
  // tile row = warp (i = i0 + warp), tile column c <-> jo = jbase + c, c in [0, 63); PD tiles are in flight
  // in registers, the walk is otherwise one global-load latency per tile
  int kq[PD][2];
  float gq[PD][2];
  auto fetch = [&](int64_t i0, int (&kv)[2], float (&gv)[2]) {
    const int64_t jbase = o0 - i0 - 31 + r_lu, ii = i0 + warp;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int c = lane + 32 * h;
      const int64_t jo = jbase + c;
      const bool ok = c < 63 && ii <= i_hi && jo >= 0 && jo < Wo;
      kv[h] = ok ? __ldg(ib + ii * Wo + jo) : -1;
      gv[h] = ok ? __ldg(gb + ii * Wo + jo) : 0.f;
    }
  };
#pragma unroll
  for (int u = 0; u < PD; ++u) fetch(i_lo + 32 * u, kq[u], gq[u]);
  for (int64_t ib0 = i_lo; ib0 <= i_hi; ib0 += 32 * PD) {
#pragma unroll
    for (int u = 0; u < PD; ++u) {
      const int64_t i0 = ib0 + 32 * u;
      if (i0 > i_hi) break;
      __syncthreads();  // the previous tile has been consumed
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        si[warp][lane + 32 * h] = kq[u][h];
        sg[warp][lane + 32 * h] = gq[u][h];
      }
      fetch(i0 + 32 * PD, kq[u], gq[u]);
      __syncthreads();
      // lane = row of the tile; this warp's o meets it at column warp + 31 - lane
      const int ja = si[lane][warp + 31 - lane];
      const float gv = sg[lane][warp + 31 - lane];
      const int64_t i = i0 + lane, jo = o - i + r_lu;
      const int k2 = ja - (int)jo + Wb - 1;
      const int64_t p = i + ja - d.a_lu;
      const bool hit = o < n && ja >= 0 && ja < Wa && k2 >= 0 && k2 < Wb && p >= 0 && p < n;
      // lanes without a target get distinct negative keys so they group with nobody
      const unsigned peers = __match_any_sync(0xffffffffu, hit ? k2 : -1 - lane);
      const int rank = __popc(peers & ((1u << lane) - 1u));
      const int last = __reduce_max_sync(0xffffffffu, hit ? rank : 0);
      for (int r = 0; r <= last; ++r) {
        if (hit && rank == r) hist[k2] = __fadd_rn(hist[k2], gv);
        __syncwarp();
      }
    }
  }
  __syncwarp();
  if (o < n)
    for (int k = lane; k < Wb; k += 32) grad_b[(bt * n + o) * Wb + k] = hist[k];
}

// (One thread per row for grad_a as well was measured twice and lost both times against the warp-per-row kernel's
// 0.37 ms at 32 x 8192 x 129 diagonals: 0.75 ms with the cells of 32 rows turned through shared memory first, 0.64
// ms with every thread walking its own contiguous row by 128-bit loads, whose 32 lanes touch 32 different lines.)
// grad_b, one THREAD per row o of b (RB_T rows per CTA), each with its own Wb-bucket histogram in shared memory
// (odd pitch: the threads of a warp hit 32 different banks for the same bucket).  A warp walks the rows i that
// reach any of its 32 rows o in ascending order; at a given i its lanes read the cells (i, jo = o - i + r_lu),
// which are consecutive in memory, and every lane adds its cell's cotangent to the bucket its index names.  A
// thread therefore accumulates its row's buckets in ascending i — the order of a sequential walk, with no
// ordering work between lanes (the kernel above spends most of its time ranking lanes that share a bucket).
constexpr int RB_T = 128;
__global__ void __launch_bounds__(RB_T) band_route_b_rows_kernel(const int* __restrict__ idx,
                                                                 const float* __restrict__ g,
                                                                 float* __restrict__ grad_b, BandDims d,
                                                                 int64_t rows) {
  extern __shared__ float hist_all[];
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  const int Wa = d.Wa(), Wb = d.Wb(), Wo = d.Wo(), r_lu = d.r_lu(), r_ld = Wo - 1 - r_lu;
  const int pitch = Wb | 1;
  const int64_t n = d.n;
  float* hist = hist_all + threadIdx.x * pitch;
  for (int k = 0; k < Wb; ++k) hist[k] = 0.f;
  // this warp's rows: row0 .. row0 + 31 of the flattened (batch, o) index; a warp may straddle two batch
  // elements, so every lane keeps its own batch element and row
  const int64_t row = (int64_t)blockIdx.x * RB_T + threadIdx.x;
  const bool live = row < rows;
  const int64_t bt = live ? row / n : 0, o = live ? row % n : 0;
  const int* ib = idx + bt * n * Wo;
  const float* gb = g + bt * n * Wo;
  // steps s = 0 .. 31 + Wo - 1: lane l looks at i = o - r_ld - l' ... every lane walks ITS OWN ascending i range
  // [o - r_ld, o + r_lu], offset so that the lanes of a warp are at the same i (hence at consecutive cells)
  // whenever their rows are consecutive: i = (o - lane) - r_ld + s
  const int steps = 31 + Wo;
  // 32-bit walk (n < 2^30): at step s this thread is at i = i0 + s, jo = jo0 - s, i.e. Wo - 1 elements further
  // on in idx / g per step; the steps at which that cell exists are [s_lo, s_hi)
  const int n32 = (int)n, i0 = (int)o - lane - r_ld, jo0 = lane + Wo - 1;
  const int s_lo = max(max(0, -i0), jo0 - Wo + 1), s_hi = live ? min(min(steps, n32 - i0), jo0 + 1) : 0;
  const int* ip = ib + (int64_t)i0 * Wo + jo0;
  const float* gp = gb + (int64_t)i0 * Wo + jo0;
  const int stride = Wo - 1;
  // U cells are fetched together and the next U are requested before this group is added up, so that the walk
  // costs one global-load latency per 2U steps overlapped with the additions (the histogram updates of a group
  // are a dependent chain through shared memory: the compiler cannot tell that two cells name different buckets).
  constexpr int U = 16;
  int ja[2][U];
  float gv[2][U];
  auto fetch = [&](int s0, int (&jd)[U], float (&gd)[U]) {
    const int* ips = ip + (int64_t)s0 * stride;
    const float* gps = gp + (int64_t)s0 * stride;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool ok = s0 + u >= s_lo && s0 + u < s_hi;
      jd[u] = ok ? __ldg(ips + u * stride) : -1;
      gd[u] = ok ? __ldg(gps + u * stride) : 0.f;
    }
  };
  auto add_up = [&](int s0, const int (&jd)[U], const float (&gd)[U]) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int s = s0 + u;
      const int k2 = jd[u] - (jo0 - s) + Wb - 1, p = i0 + s + jd[u] - d.a_lu;
      if ((unsigned)jd[u] < (unsigned)Wa && (unsigned)k2 < (unsigned)Wb && (unsigned)p < (unsigned)n32)
        hist[k2] = __fadd_rn(hist[k2], gd[u]);
    }
  };
  fetch(0, ja[0], gv[0]);
  for (int s0 = 0; s0 < steps; s0 += 2 * U) {
    fetch(s0 + U, ja[1], gv[1]);
    add_up(s0, ja[0], gv[0]);
    fetch(s0 + 2 * U, ja[0], gv[0]);
    add_up(s0 + U, ja[1], gv[1]);
  }
  __syncthreads();
  for (int r = warp; r < RB_T; r += RB_T / 32) {
    const int64_t grow = (int64_t)blockIdx.x * RB_T + r;
    if (grow >= rows) break;
    for (int k = lane; k < Wb; k += 32) grad_b[grow * Wb + k] = hist_all[r * pitch + k];
  }
}

// ------------------------------------------------------------------ log semiring, second order
// With the weight s = exp(a[i][ja] + b[o][k2] - out[i][jo]) of a triple, cotangents h_a, h_b of
// the first-order gradients, H = h_a[i][ja] + h_b[o][k2] and t[i][jo] = sum_ja s H:
//   d/da[i][ja] = sum_jo g s (H - t),   d/db[o][k2] = sum_i g s (H - t),   d/dg[i][jo] = t.
// Two passes of O(n*Wa*Wb) replace banded_cuda_backbackward_kernel_A/B/C
// (banded_cuda_kernel.cu:154-350), whose A and B are O(n*Wa*Wo*Wa).  One thread per band cell,
// operands read from global memory (this is not a hot path).
__global__ void __launch_bounds__(NT) band_bwd2_t_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                         const float* __restrict__ out, const float* __restrict__ ha,
                                                         const float* __restrict__ hb, float* __restrict__ t,
                                                         BandDims d, int64_t cells) {
  const int64_t e = (int64_t)blockIdx.x * NT + threadIdx.x;
  if (e >= cells) return;
  const int Wa = d.Wa(), Wb = d.Wb(), Wo = d.Wo(), r_lu = d.r_lu();
  const int64_t n = d.n;
  const int jo = (int)(e % Wo);
  const int64_t i = (e / Wo) % n, bt = e / (Wo * n);
  const int64_t o = i + jo - r_lu;
  float val = 0.f;
  if (o >= 0 && o < n) {
    int lo = max(0, jo - (Wb - 1)), hi = min(Wa - 1, jo);
    lo = (int)max((int64_t)lo, (int64_t)d.a_lu - i);
    hi = (int)min((int64_t)hi, n - 1 - i + d.a_lu);
    const float c = __ldg(out + e);
    const int64_t ar = (bt * n + i) * Wa, br = (bt * n + o) * Wb;
    const int kofs = Wb - 1 - jo;
    for (int ja = lo; ja <= hi; ++ja) {
      const float s = exp_sfu((__ldg(a + ar + ja) + __ldg(b + br + ja + kofs)) - c);
      val = fmaf(s, __ldg(ha + ar + ja) + __ldg(hb + br + ja + kofs), val);
    }
  }
  t[e] = val;
}

__global__ void __launch_bounds__(NT) band_bwd2_a_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                         const float* __restrict__ out, const float* __restrict__ g,
                                                         const float* __restrict__ t, const float* __restrict__ ha,
                                                         const float* __restrict__ hb, float* __restrict__ da,
                                                         BandDims d, int64_t cells) {
  const int64_t e = (int64_t)blockIdx.x * NT + threadIdx.x;
  if (e >= cells) return;
  const int Wa = d.Wa(), Wb = d.Wb(), Wo = d.Wo(), r_lu = d.r_lu();
  const int64_t n = d.n;
  const int ja = (int)(e % Wa);
  const int64_t i = (e / Wa) % n, bt = e / (Wa * n);
  const int64_t p = i + ja - d.a_lu;
  float val = 0.f;
  if (p >= 0 && p < n) {
    int lo = ja, hi = min(Wo - 1, ja + Wb - 1);
    lo = (int)max((int64_t)lo, (int64_t)r_lu - i);
    hi = (int)min((int64_t)hi, n - 1 - i + r_lu);
    const float av = __ldg(a + e), hv = __ldg(ha + e);
    const int64_t orow = (bt * n + i) * Wo;
    for (int jo = lo; jo <= hi; ++jo) {
      const int64_t o = i + jo - r_lu;
      const int64_t bi = (bt * n + o) * Wb + (ja - jo + Wb - 1);
      const float w = exp_sfu((av + __ldg(b + bi)) - __ldg(out + orow + jo)) * __ldg(g + orow + jo);
      val = fmaf(w, (hv + __ldg(hb + bi)) - __ldg(t + orow + jo), val);
    }
  }
  da[e] = val;
}

__global__ void __launch_bounds__(NT) band_bwd2_b_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                         const float* __restrict__ out, const float* __restrict__ g,
                                                         const float* __restrict__ t, const float* __restrict__ ha,
                                                         const float* __restrict__ hb, float* __restrict__ db,
                                                         BandDims d, int64_t cells) {
  const int64_t e = (int64_t)blockIdx.x * NT + threadIdx.x;
  if (e >= cells) return;
  const int Wa = d.Wa(), Wb = d.Wb(), Wo = d.Wo(), r_lu = d.r_lu();
  const int64_t n = d.n;
  const int k2 = (int)(e % Wb);
  const int64_t o = (e / Wb) % n, bt = e / (Wb * n);
  const int64_t p = o + k2 - d.b_lu;
  float val = 0.f;
  if (p >= 0 && p < n) {
    // i = o - jo + r_lu with ja = k2 + jo - (Wb-1) in [0, Wa)
    int64_t lo = o + r_lu - (Wb - 1 - k2 + Wa - 1), hi = o + r_lu - (Wb - 1 - k2);
    lo = max(lo, (int64_t)0);
    hi = min(hi, n - 1);
    const float bv = __ldg(b + e), hv = __ldg(hb + e);
    for (int64_t i = lo; i <= hi; ++i) {
      const int jo = (int)(o - i + r_lu), ja = k2 + jo - (Wb - 1);
      const int64_t ai = (bt * n + i) * Wa + ja, oi = (bt * n + i) * Wo + jo;
      const float w = exp_sfu((__ldg(a + ai) + bv) - __ldg(out + oi)) * __ldg(g + oi);
      val = fmaf(w, (__ldg(ha + ai) + hv) - __ldg(t + oi), val);
    }
  }
  db[e] = val;
}

int pick_rows(size_t fixed_floats, size_t per_row_floats) {
  for (int t = 32; t >= 1; t >>= 1)
    if ((fixed_floats + per_row_floats * t) * sizeof(float) <= (size_t)kSmemBudget) return t;
  return 0;
}

template <typename KernelT>
bool allow_smem(KernelT kernel, size_t bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) == cudaSuccess;
}

int check_band(int mode, int64_t B, int64_t n, int a_lu, int a_ld, int b_lu, int b_ld) {
  if (mode != GBMM_BAND_LOG && mode != GBMM_BAND_MAX && mode != GBMM_BAND_MUL) return GBMM_ERR_INVALID_ARG;
  if (B < 0 || n < 0 || a_lu < 0 || a_ld < 0 || b_lu < 0 || b_ld < 0) return GBMM_ERR_INVALID_ARG;
  const int64_t Wo = (int64_t)a_lu + a_ld + b_lu + b_ld + 1;
  if (Wo >= (1 << 24) || n >= (1LL << 31) - 64) return GBMM_ERR_UNSUPPORTED;
  return GBMM_OK;
}

}  // namespace
}  // namespace gbmm

using namespace gbmm;

// The direct kernels above on every row (flags == nullptr) or on the flagged 64-row blocks only.
static int exact_forward(int mode, const float* a, const float* b, float* out, int32_t* idx, float* maxes,
                         const BandDims& d, int64_t B, const int* flags, cudaStream_t st) {
  const int64_t n = d.n;
  const int Wa = d.Wa(), Wb = d.Wb(), Wo = d.Wo();
  const size_t ldb = b_pitch(Wb);
  int TI = pick_rows((size_t)(Wo - 1) * ldb, (size_t)Wa + ldb);
  const int staged = TI > 0;
  if (!staged) TI = 8;
  const size_t smem = staged ? ((size_t)TI * Wa + (size_t)(TI + Wo - 1) * ldb) * sizeof(float) : 0;
  const int64_t tiles = ceil_div(n, TI), blocks = B * tiles;
  if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  unsigned grid = 0;
  if (int rc = capped_grid(blocks, &grid)) return rc;
#define GBMM_LAUNCH_BAND_FWD(MODE)                                                                      \
  do {                                                                                                  \
    if (flags) {                                                                                        \
      if (smem + 2048 > 48 * 1024 && !allow_smem(band_fwd_kernel<MODE, true>, smem)) return GBMM_ERR_LAUNCH; \
      band_fwd_kernel<MODE, true><<<grid, NT, smem, st>>>(a, b, out, idx, maxes, d, TI, (int)tiles, staged, \
                                                          flags, blocks);                               \
    } else {                                                                                            \
      if (smem > 48 * 1024 && !allow_smem(band_fwd_kernel<MODE, false>, smem)) return GBMM_ERR_LAUNCH;  \
      band_fwd_kernel<MODE, false><<<(unsigned)blocks, NT, smem, st>>>(a, b, out, idx, maxes, d, TI,    \
                                                                       (int)tiles, staged, flags, blocks); \
    }                                                                                                   \
  } while (0)
  if (mode == GBMM_BAND_MUL) GBMM_LAUNCH_BAND_FWD(GBMM_BAND_MUL);
  else if (mode == GBMM_BAND_MAX) GBMM_LAUNCH_BAND_FWD(GBMM_BAND_MAX);
  else GBMM_LAUNCH_BAND_FWD(GBMM_BAND_LOG);
#undef GBMM_LAUNCH_BAND_FWD
  return launch_status();
}

static int route_max_backward(const float* grad_out, const int* idx, float* grad_a, float* grad_b,
                              const BandDims& d, int64_t B, cudaStream_t st, bool* handled) {
  const size_t smem_a = sizeof(float) * 8 * d.Wa(), smem_b = sizeof(float) * 32 * (d.Wb() + 1);
  *handled = smem_a <= (size_t)kSmemBudget && smem_b + 17 * 1024 <= (size_t)kSmemBudget;
  if (!*handled) return GBMM_OK;  // bands too wide for the histograms: the scanning kernels take over
  if (grad_a) {
    const int64_t rows = B * d.n, blocks = ceil_div(rows, 8);
    if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
    if (smem_a > 48 * 1024 && !allow_smem(band_route_a_kernel, smem_a)) return GBMM_ERR_LAUNCH;
    band_route_a_kernel<<<(unsigned)blocks, 256, smem_a, st>>>(idx, grad_out, grad_a, rows, d);
    if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
  }
  if (grad_b) {
    const int64_t tiles = ceil_div(d.n, 32), blocks = B * tiles;
    if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
    const size_t smem_rows = sizeof(float) * RB_T * (d.Wb() | 1);
    const char* eb = getenv("GENBMM_B200_BAND_ROUTE_B");   // "w": the warp-per-row kernel
    const bool by_rows = !(eb && eb[0] == 'w');
    if (by_rows && smem_rows <= (size_t)100 * 1024 && d.n < (1LL << 30)) {   // at least two CTAs per SM; 32-bit walk
      const int64_t rows = B * d.n, rblocks = ceil_div(rows, RB_T);
      if (rblocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
      if (smem_rows > 48 * 1024 && !allow_smem(band_route_b_rows_kernel, smem_rows)) return GBMM_ERR_LAUNCH;
      band_route_b_rows_kernel<<<(unsigned)rblocks, RB_T, smem_rows, st>>>(idx, grad_out, grad_b, d, rows);
      return launch_status();
    }
    // the kernel also holds 16.5 KB of static tiles; together they may pass the 48 KB default
    if (smem_b + 17 * 1024 > 48 * 1024 && !allow_smem(band_route_b_kernel, smem_b)) return GBMM_ERR_LAUNCH;
    band_route_b_kernel<<<(unsigned)blocks, 1024, smem_b, st>>>(idx, grad_out, grad_b, d, (int)tiles);
  }
  return launch_status();
}

static int exact_backward(int mode, const float* a, const float* b, const float* grad_out, const void* part,
                          float* grad_a, float* grad_b, const BandDims& d, int64_t B, const int* flags,
                          cudaStream_t st) {
  const int64_t n = d.n;
  if (mode == GBMM_BAND_MAX) {
    bool handled = false;
    const int rc = route_max_backward(grad_out, static_cast<const int*>(part), grad_a, grad_b, d, B, st, &handled);
    if (rc != GBMM_OK || handled) return rc;
  }
  const int Wa = d.Wa(), Wb = d.Wb(), Wo = d.Wo();
  const size_t ldb = b_pitch(Wb);
  if (grad_a) {
    int TI = pick_rows((size_t)(Wo - 1) * ldb, ldb + 2 * (size_t)Wo);
    const int staged = TI > 0;
    if (!staged) TI = 8;
    const size_t smem = staged ? ((size_t)(TI + Wo - 1) * ldb + 2 * (size_t)TI * Wo) * sizeof(float) : 0;
    const int64_t tiles = ceil_div(n, TI), blocks = B * tiles;
    if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
    unsigned grid = 0;
    if (int rc = capped_grid(blocks, &grid)) return rc;
#define GBMM_LAUNCH_BAND_BWD_A(MODE)                                                                      \
  do {                                                                                                    \
    if (flags) {                                                                                          \
      if (smem + 2048 > 48 * 1024 && !allow_smem(band_bwd_a_kernel<MODE, true>, smem)) return GBMM_ERR_LAUNCH; \
      band_bwd_a_kernel<MODE, true><<<grid, NT, smem, st>>>(a, b, grad_out, part, grad_a, d, TI, (int)tiles, \
                                                            staged, flags, blocks);                       \
    } else {                                                                                              \
      if (smem > 48 * 1024 && !allow_smem(band_bwd_a_kernel<MODE, false>, smem)) return GBMM_ERR_LAUNCH;  \
      band_bwd_a_kernel<MODE, false><<<(unsigned)blocks, NT, smem, st>>>(a, b, grad_out, part, grad_a, d, TI, \
                                                                         (int)tiles, staged, flags, blocks); \
    }                                                                                                     \
  } while (0)
    if (mode == GBMM_BAND_MUL) GBMM_LAUNCH_BAND_BWD_A(GBMM_BAND_MUL);
    else if (mode == GBMM_BAND_MAX) GBMM_LAUNCH_BAND_BWD_A(GBMM_BAND_MAX);
    else GBMM_LAUNCH_BAND_BWD_A(GBMM_BAND_LOG);
#undef GBMM_LAUNCH_BAND_BWD_A
    if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
  }
  if (grad_b) {
    int TO = 32, TI = 0;
    for (; TO >= 1 && TI == 0; TO >>= 1) {
      TI = pick_rows((size_t)TO * Wb, (size_t)Wa + 2 * (size_t)Wo);
      if (TI) break;
    }
    const int staged = TI > 0;
    if (!staged) {
      TO = 8;
      TI = 1;
    }
    const size_t smem = staged ? ((size_t)TO * Wb + (size_t)TI * (Wa + 2 * (size_t)Wo)) * sizeof(float) : 0;
    const int64_t tiles = ceil_div(n, TO), blocks = B * tiles;
    if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
    unsigned grid = 0;
    if (int rc = capped_grid(blocks, &grid)) return rc;
#define GBMM_LAUNCH_BAND_BWD_B(MODE)                                                                      \
  do {                                                                                                    \
    if (flags) {                                                                                          \
      if (smem + 2048 > 48 * 1024 && !allow_smem(band_bwd_b_kernel<MODE, true>, smem)) return GBMM_ERR_LAUNCH; \
      band_bwd_b_kernel<MODE, true><<<grid, NT, smem, st>>>(a, b, grad_out, part, grad_b, d, TO, TI,      \
                                                            (int)tiles, staged, flags, blocks);           \
    } else {                                                                                              \
      if (smem > 48 * 1024 && !allow_smem(band_bwd_b_kernel<MODE, false>, smem)) return GBMM_ERR_LAUNCH;  \
      band_bwd_b_kernel<MODE, false><<<(unsigned)blocks, NT, smem, st>>>(a, b, grad_out, part, grad_b, d, TO, TI, \
                                                                         (int)tiles, staged, flags, blocks); \
    }                                                                                                     \
  } while (0)
    if (mode == GBMM_BAND_MUL) GBMM_LAUNCH_BAND_BWD_B(GBMM_BAND_MUL);
    else if (mode == GBMM_BAND_MAX) GBMM_LAUNCH_BAND_BWD_B(GBMM_BAND_MAX);
    else GBMM_LAUNCH_BAND_BWD_B(GBMM_BAND_LOG);
#undef GBMM_LAUNCH_BAND_BWD_B
  }
  return launch_status();
}

// Bands this narrow leave too few in-band cells per 64x64 block for the block-banded kernels
// to pay off; the direct kernels take them.
static bool use_block_path(const BandDims& d) { return (int64_t)d.Wa() * d.Wb() >= 64; }

extern "C" int64_t gbmm_band_workspace_bytes(int64_t B, int64_t n) {
  if (B < 0 || n < 0) return -1;
  return band_fast_workspace_bytes(B, n);
}

extern "C" int gbmm_band_forward_f32(int mode, const float* a, int a_lu, int a_ld, const float* b, int b_lu,
                                     int b_ld, float* out, int32_t* idx, float* maxes, int64_t B, int64_t n,
                                     void* workspace, int64_t workspace_bytes, void* stream) {
  const int st0 = check_band(mode, B, n, a_lu, a_ld, b_lu, b_ld);
  if (st0 != GBMM_OK) return st0;
  if (B == 0 || n == 0) return GBMM_OK;
  if (!a || !b || !out) return GBMM_ERR_INVALID_ARG;
  if (mode == GBMM_BAND_MAX && !idx) return GBMM_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const BandDims d{n, a_lu, a_ld, b_lu, b_ld};
  const bool have_ws = workspace && workspace_bytes >= band_fast_workspace_bytes(B, n) &&
                       (reinterpret_cast<uintptr_t>(workspace) & 255) == 0;
  const bool fast = use_block_path(d) && (mode != GBMM_BAND_LOG || (have_ws && !maxes));
  if (!fast) return exact_forward(mode, a, b, out, idx, maxes, d, B, nullptr, st);
  int* flags = nullptr;
  const int rc = band_fast_forward(mode, a, b, out, idx, d, B, workspace, &flags, st);
  if (rc != GBMM_OK || mode != GBMM_BAND_LOG) return rc;
  return exact_forward(mode, a, b, out, nullptr, nullptr, d, B, flags, st);
}

extern "C" int gbmm_band_backward_f32(int mode, const float* a, int a_lu, int a_ld, const float* b, int b_lu,
                                      int b_ld, const float* grad_out, const void* part, float* grad_a,
                                      float* grad_b, int64_t B, int64_t n, void* workspace,
                                      int64_t workspace_bytes, void* stream) {
  const int st0 = check_band(mode, B, n, a_lu, a_ld, b_lu, b_ld);
  if (st0 != GBMM_OK) return st0;
  if (B == 0 || n == 0) return GBMM_OK;
  if (!a || !b || !grad_out) return GBMM_ERR_INVALID_ARG;
  if (mode != GBMM_BAND_MUL && !part) return GBMM_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const BandDims d{n, a_lu, a_ld, b_lu, b_ld};
  const bool have_ws = workspace && workspace_bytes >= band_fast_workspace_bytes(B, n) &&
                       (reinterpret_cast<uintptr_t>(workspace) & 255) == 0;
  const bool fast = use_block_path(d) && mode != GBMM_BAND_MAX && (mode != GBMM_BAND_LOG || have_ws);
  if (!fast) return exact_backward(mode, a, b, grad_out, part, grad_a, grad_b, d, B, nullptr, st);
  int* flags = nullptr;
  const int rc = band_fast_backward(mode, a, b, grad_out, static_cast<const float*>(part), grad_a, grad_b, d, B,
                                    workspace, &flags, st);
  if (rc != GBMM_OK || mode != GBMM_BAND_LOG) return rc;
  return exact_backward(mode, a, b, grad_out, part, grad_a, grad_b, d, B, flags, st);
}

extern "C" int gbmm_band_tc_eligible(int mode, int64_t n, int a_lu, int a_ld, int b_lu, int b_ld) {
  if (a_lu < 0 || a_ld < 0 || b_lu < 0 || b_ld < 0 || n < 0) return 0;
  return band_tc_eligible(mode, BandDims{n, a_lu, a_ld, b_lu, b_ld}) ? 1 : 0;
}

extern "C" int64_t gbmm_band_tc_workspace_bytes(int backward, int64_t B, int64_t n, int a_lu, int a_ld, int b_lu,
                                                int b_ld) {
  if (B < 0 || n < 0 || a_lu < 0 || a_ld < 0 || b_lu < 0 || b_ld < 0) return -1;
  return band_tc_workspace_bytes(backward, B, BandDims{n, a_lu, a_ld, b_lu, b_ld});
}

extern "C" int gbmm_band_tc_workspace_init(void* workspace, int64_t workspace_bytes, void* stream) {
  if (!workspace || workspace_bytes < 0) return GBMM_ERR_INVALID_ARG;
  return cudaMemsetAsync(workspace, 0, (size_t)workspace_bytes, static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? GBMM_OK
             : GBMM_ERR_LAUNCH;
}

extern "C" int gbmm_band_tc_forward_f32(int mode, const float* a, int a_lu, int a_ld, const float* b, int b_lu,
                                        int b_ld, float* out, int64_t B, int64_t n, void* workspace,
                                        int64_t workspace_bytes, void* stream) {
  const int st0 = check_band(mode, B, n, a_lu, a_ld, b_lu, b_ld);
  if (st0 != GBMM_OK) return st0;
  if (B == 0 || n == 0) return GBMM_OK;
  if (!a || !b || !out || !workspace) return GBMM_ERR_INVALID_ARG;
  const BandDims d{n, a_lu, a_ld, b_lu, b_ld};
  if (!band_tc_eligible(mode, d)) return GBMM_ERR_UNSUPPORTED;
  if (workspace_bytes < band_tc_workspace_bytes(0, B, d) || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return GBMM_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int* flags = nullptr;
  const int rc = band_tc_forward(mode, a, b, out, d, B, workspace, &flags, st);
  if (rc != GBMM_OK || mode != GBMM_BAND_LOG) return rc;
  return exact_forward(mode, a, b, out, nullptr, nullptr, d, B, flags, st);
}

extern "C" int gbmm_band_tc_backward_f32(int mode, const float* a, int a_lu, int a_ld, const float* b, int b_lu,
                                         int b_ld, const float* grad_out, const float* part, float* grad_a,
                                         float* grad_b, int64_t B, int64_t n, void* workspace,
                                         int64_t workspace_bytes, int operands_ready, void* stream) {
  const int st0 = check_band(mode, B, n, a_lu, a_ld, b_lu, b_ld);
  if (st0 != GBMM_OK) return st0;
  if (B == 0 || n == 0) return GBMM_OK;
  if (!a || !b || !grad_out || !workspace) return GBMM_ERR_INVALID_ARG;
  if (mode == GBMM_BAND_LOG && !part) return GBMM_ERR_INVALID_ARG;
  const BandDims d{n, a_lu, a_ld, b_lu, b_ld};
  if (!band_tc_eligible(mode, d)) return GBMM_ERR_UNSUPPORTED;
  if (workspace_bytes < band_tc_workspace_bytes(1, B, d) || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return GBMM_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int* flags = nullptr;
  const int rc = band_tc_backward(mode, a, b, grad_out, part, grad_a, grad_b, d, B, workspace, operands_ready, &flags,
                                  st);
  if (rc != GBMM_OK || mode != GBMM_BAND_LOG) return rc;
  return exact_backward(mode, a, b, grad_out, part, grad_a, grad_b, d, B, flags, st);
}

extern "C" int gbmm_band_max_eligible(int64_t n, int a_lu, int a_ld, int b_lu, int b_ld) {
  if (a_lu < 0 || a_ld < 0 || b_lu < 0 || b_ld < 0 || n < 0) return 0;
  return band_max_fast_eligible(BandDims{n, a_lu, a_ld, b_lu, b_ld}) ? 1 : 0;
}

extern "C" int64_t gbmm_band_max_workspace_bytes(int64_t B, int64_t n, int a_lu, int a_ld, int b_lu, int b_ld) {
  if (B < 0 || n < 0 || a_lu < 0 || a_ld < 0 || b_lu < 0 || b_ld < 0) return -1;
  return band_max_workspace_bytes(B, BandDims{n, a_lu, a_ld, b_lu, b_ld});
}

extern "C" int gbmm_band_max_workspace_init(void* workspace, int64_t workspace_bytes, void* stream) {
  if (!workspace || workspace_bytes < 0 || (reinterpret_cast<uintptr_t>(workspace) & 15)) return GBMM_ERR_INVALID_ARG;
  return band_max_workspace_init(workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int gbmm_band_max_forward_f32(const float* a, int a_lu, int a_ld, const float* b, int b_lu, int b_ld,
                                         float* out, int32_t* idx, int64_t B, int64_t n, void* workspace,
                                         int64_t workspace_bytes, void* stream) {
  const int st0 = check_band(GBMM_BAND_MAX, B, n, a_lu, a_ld, b_lu, b_ld);
  if (st0 != GBMM_OK) return st0;
  if (B == 0 || n == 0) return GBMM_OK;
  if (!a || !b || !out || !idx || !workspace) return GBMM_ERR_INVALID_ARG;
  const BandDims d{n, a_lu, a_ld, b_lu, b_ld};
  if (!band_max_fast_eligible(d)) return GBMM_ERR_UNSUPPORTED;
  if (workspace_bytes < band_max_workspace_bytes(B, d) || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return GBMM_ERR_INVALID_ARG;
  return band_max_forward(a, b, out, idx, d, B, workspace, static_cast<cudaStream_t>(stream));
}

extern "C" int gbmm_band_backbackward_f32(const float* a, int a_lu, int a_ld, const float* b, int b_lu, int b_ld,
                                          const float* grad_out, const float* part, const float* h_a,
                                          const float* h_b, float* d_a, float* d_b, float* d_grad_out, int64_t B,
                                          int64_t n, void* stream) {
  const int st0 = check_band(GBMM_BAND_LOG, B, n, a_lu, a_ld, b_lu, b_ld);
  if (st0 != GBMM_OK) return st0;
  if (B == 0 || n == 0) return GBMM_OK;
  if (!a || !b || !grad_out || !part || !h_a || !h_b || !d_a || !d_b || !d_grad_out) return GBMM_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const BandDims d{n, a_lu, a_ld, b_lu, b_ld};
  const int64_t co = B * n * d.Wo(), ca = B * n * d.Wa(), cb = B * n * d.Wb();
  if (ceil_div(co, NT) >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  band_bwd2_t_kernel<<<(unsigned)ceil_div(co, NT), NT, 0, st>>>(a, b, part, h_a, h_b, d_grad_out, d, co);
  if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
  band_bwd2_a_kernel<<<(unsigned)ceil_div(ca, NT), NT, 0, st>>>(a, b, part, grad_out, d_grad_out, h_a, h_b, d_a, d,
                                                                ca);
  if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
  band_bwd2_b_kernel<<<(unsigned)ceil_div(cb, NT), NT, 0, st>>>(a, b, part, grad_out, d_grad_out, h_a, h_b, d_b, d,
                                                                cb);
  return launch_status();
}
