// Banded products as block-banded FP32 products (the fast path of the banded operators).
//
// In dense terms a band tensor data:(n,W) with `lu` is a matrix X[r,c] = data[r][c-r+lu]
// (X is the transpose of the matrix the reference calls Dense; see band.cu).  With Xa, Xb the
// operands and G the cotangent of the result,
//   forward  out[i,o] = sum_p Xa[i,p] Xb[o,p]
//   grad_a   dXa[i,p] = sum_o G[i,o]  Xb[o,p]
//   grad_b   dXb[o,p] = sum_i G[i,o]  Xa[i,p]
// are three products between band matrices whose result is again a band.  A CTA owns a 64x64
// block (r-block, c-block) of the result that intersects the result band, walks the reduction
// index s over the range where both operand bands are populated for that block, in chunks of 16,
// and in every chunk rebuilds two small dense tiles in shared memory from the band storage
// (zero outside the band or the matrix).  The inner loop is then an ordinary register-tiled
// product: 4x4 results per thread, two 128-bit LDS and 16 FFMA per reduction step.  About 45 % of
// the FFMAs of a 64x64 block hit band cells for 129-wide bands; the rest multiply zeros.
//
// Semirings.  sum: as above.  log: factorised as in dense_fast.cu — operands exponentiated
// against their row maxima while the tiles are built, out = log(S) + ra[i] + rb[o]; a 64-row
// block whose S underflows anywhere is flagged and recomputed by the exact kernels of band.cu
// (forward), and in the backward its rows contribute through those exact kernels only.
// max (forward only): v = x + y with -inf outside the band, strict `>` in ascending p, which is
// ascending ja for a fixed row, so the lowest-index tie rule of banded_cuda_kernel.cu:52-59 holds.
#include "band.cuh"

namespace gbmm {
namespace {

constexpr int TB = 64, SK = 32, NTB = 256, LDT = TB + 4;
constexpr float kTinyLog = -62.383246f;  // log(2^-90)

enum { F_FWD = 0, F_DA = 1, F_DB = 2 };
enum { S_MUL = 0, S_LOG = 1, S_MAX = 2 };

struct BandView {
  const float* p;  // this batch element's (n, W) data
  int lu, W;
};

// Is (row, col) a stored cell of the band matrix, and where?  Rows, columns and band offsets
// fit in 32 bits (n < 2^31); only the element index is 64-bit.
__device__ __forceinline__ bool band_cell(const BandView& m, int n, int row, int col, int64_t* idx) {
  const int j = col - row + m.lu;
  if ((unsigned)row >= (unsigned)n || (unsigned)col >= (unsigned)n || (unsigned)j >= (unsigned)m.W) return false;
  *idx = (int64_t)row * m.W + j;
  return true;
}

struct BlockArgs {
  const float* a;
  const float* b;
  const float* g;      // cotangent (backward)
  const float* part;   // forward output (log backward)
  const float* ra;     // (B, n) row maxima of a (log)
  const float* rb;     // (B, n) row maxima of b (log)
  int* flags;          // (B, ceil(n/64)) log: row blocks that need the exact kernels
  float* out;          // result band (forward: out; backward: the gradient)
  int* idx;            // forward max: argmax in a's band coordinate
  BandDims d;
  int ncb;             // c-blocks per r-block
};

template <int FORM, int SEMI>
__global__ void __launch_bounds__(NTB) band_block_kernel(BlockArgs g) {
  __shared__ __align__(16) float xt[SK * LDT];
  __shared__ __align__(16) float yt[SK * LDT];
  const BandDims& d = g.d;
  const int n = (int)d.n;
  const int Wa = d.Wa(), Wb = d.Wb(), Wo = d.Wo(), r_lu = d.r_lu(), r_ld = Wo - 1 - r_lu;
  const int nrb = (n + TB - 1) / TB;
  const int64_t id = blockIdx.x;
  const int cbi = (int)(id % g.ncb);
  const int rbk = (int)((id / g.ncb) % nrb);
  const int64_t bt = id / ((int64_t)g.ncb * nrb);
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;

  const BandView A{g.a + bt * n * (int64_t)Wa, d.a_lu, Wa};
  const BandView Bm{g.b + bt * n * (int64_t)Wb, d.b_lu, Wb};
  const BandView G{g.g ? g.g + bt * n * (int64_t)Wo : nullptr, r_lu, Wo};
  const BandView P{g.part ? g.part + bt * n * (int64_t)Wo : nullptr, r_lu, Wo};
  const float* ra = g.ra ? g.ra + bt * n : nullptr;
  const float* rb = g.rb ? g.rb + bt * n : nullptr;
  const int* flags = g.flags ? g.flags + bt * nrb : nullptr;

  // result band (lu_out), operand supports s - r in [-xl, xu], s - c in [-yl, yu]
  int lu_out, w_out, xl, xu, yl, yu;
  if (FORM == F_FWD) { lu_out = r_lu; w_out = Wo; xl = d.a_lu; xu = d.a_ld; yl = d.b_lu; yu = d.b_ld; }
  if (FORM == F_DA)  { lu_out = d.a_lu; w_out = Wa; xl = r_lu; xu = r_ld; yl = d.b_ld; yu = d.b_lu; }
  if (FORM == F_DB)  { lu_out = d.b_lu; w_out = Wb; xl = r_ld; xu = r_lu; yl = d.a_ld; yu = d.a_lu; }
  const int r0 = rbk * TB;
  // first c-block that can meet the band of rows r0..: floor((r0 - lu_out) / TB)
  const int cfirst = (r0 - lu_out >= 0) ? (r0 - lu_out) / TB : -((lu_out - r0 + TB - 1) / TB);
  const int c0 = (cfirst + cbi) * TB;
  if (c0 - (r0 + TB - 1) > (w_out - 1 - lu_out)) return;  // wholly beyond the band

  // value of X at (r, s) and of Y at (c, s), transformed for the semiring
  auto xval = [&](int r, int s) -> float {
    int64_t q;
    if (FORM == F_FWD) {
      if (!band_cell(A, n, r, s, &q)) return SEMI == S_MAX ? __int_as_float(0xff800000) : 0.f;
      const float v = __ldg(A.p + q);
      return SEMI == S_LOG ? exp_sfu(v - __ldg(ra + r)) : v;
    }
    // backward: G at (i, o); F_DA: (r, s) = (i, o); F_DB: (r, s) = (o, i)
    const int i = FORM == F_DA ? r : s, o = FORM == F_DA ? s : r;
    if (!band_cell(G, n, i, o, &q)) return 0.f;
    const float gv = __ldg(G.p + q);
    if (SEMI != S_LOG) return gv;
    if (__ldg(flags + i / TB)) return 0.f;  // this row goes through the exact kernels
    return gv * exp_sfu((__ldg(ra + i) + __ldg(rb + o)) - __ldg(P.p + q));
  };
  // (max semiring: a missing cell of either operand is -inf, so the sum never wins)
  constexpr float kPadY = 0.f;
  auto yval = [&](int c, int s) -> float {
    int64_t q;
    if (FORM == F_DB) {  // A at (i, p) = (s, c)
      if (!band_cell(A, n, s, c, &q)) return 0.f;
      const float v = __ldg(A.p + q);
      return SEMI == S_LOG ? exp_sfu(v - __ldg(ra + s)) : v;
    }
    // Bm at (o, p): F_FWD: (c, s) = (o, p); F_DA: (c, s) = (p, o)
    const int o = FORM == F_FWD ? c : s, p = FORM == F_FWD ? s : c;
    if (!band_cell(Bm, n, o, p, &q)) return SEMI == S_MAX ? __int_as_float(0xff800000) : kPadY;
    const float v = __ldg(Bm.p + q);
    return SEMI == S_LOG ? exp_sfu(v - __ldg(rb + o)) : v;
  };
  // which logical index runs along memory for each operand tile
  constexpr bool X_S_FAST = (FORM != F_DB);   // F_DB reads G[i][..o..]: r (= o) is contiguous
  constexpr bool Y_S_FAST = (FORM == F_FWD);  // F_DA reads Bm[o][..p..] and F_DB A[i][..p..]: c contiguous

  float acc[4][4];
  int best[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[i][j] = SEMI == S_MAX ? kFloor : 0.f;
      best[i][j] = -1;
    }

  const int s_lo = max(max(r0 - xl, c0 - yl), 0);
  const int s_hi = min(min(r0 + TB - 1 + xu, c0 + TB - 1 + yu), n - 1);
  constexpr int NE = TB * SK / NTB;  // tile elements per thread and operand
  constexpr float kPadX = SEMI == S_MAX ? -__builtin_huge_valf() : 0.f;
  float xr[NE], yr[NE];
  // fetch one chunk of both operand tiles into registers (issued before the previous chunk is
  // multiplied, so the global-memory latency overlaps the FFMAs)
  auto fetch = [&](int s0) {
#pragma unroll
    for (int q = 0; q < NE; ++q) {
      const int e = tid + q * NTB;
      {
        const int sl = X_S_FAST ? e % SK : e / TB, rl = X_S_FAST ? e / SK : e % TB;
        xr[q] = (s0 + sl <= s_hi) ? xval(r0 + rl, s0 + sl) : kPadX;
      }
      {
        const int sl = Y_S_FAST ? e % SK : e / TB, cl = Y_S_FAST ? e / SK : e % TB;
        yr[q] = (s0 + sl <= s_hi) ? yval(c0 + cl, s0 + sl) : kPadX;
      }
    }
  };
  // The log semiring's tile values cost extra loads and an exponential each; prefetching them a
  // chunk ahead costs more in registers than it hides (measured), so those fetch in place.
  constexpr bool PREFETCH = SEMI != S_LOG;
  if (PREFETCH && s_lo <= s_hi) fetch(s_lo);
  for (int s0 = s_lo; s0 <= s_hi; s0 += SK) {
    __syncthreads();  // the previous chunk's tiles are fully consumed
    if (!PREFETCH) fetch(s0);
#pragma unroll
    for (int q = 0; q < NE; ++q) {
      const int e = tid + q * NTB;
      xt[(X_S_FAST ? e % SK : e / TB) * LDT + (X_S_FAST ? e / SK : e % TB)] = xr[q];
      yt[(Y_S_FAST ? e % SK : e / TB) * LDT + (Y_S_FAST ? e / SK : e % TB)] = yr[q];
    }
    __syncthreads();
    if (PREFETCH && s0 + SK <= s_hi) fetch(s0 + SK);
#pragma unroll
    for (int sl = 0; sl < SK; ++sl) {
      const float4 xv = *reinterpret_cast<const float4*>(xt + sl * LDT + ty * 4);
      const float4 yv = *reinterpret_cast<const float4*>(yt + sl * LDT + tx * 4);
      const float x[4] = {xv.x, xv.y, xv.z, xv.w}, y[4] = {yv.x, yv.y, yv.z, yv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (SEMI == S_MAX) {
            const float v = __fadd_rn(x[i], y[j]);
            if (v > acc[i][j]) {
              acc[i][j] = v;
              best[i][j] = s0 + sl;
            }
          } else {
            acc[i][j] = fmaf(x[i], y[j], acc[i][j]);
          }
        }
    }
  }

  // epilogue: scatter the block's band cells into band storage
  bool bad = false;
  float* ob = g.out + bt * n * (int64_t)w_out;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + ty * 4 + i;
    if (r >= n) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = c0 + tx * 4 + j;
      const int cell = c - r + lu_out;
      if (cell < 0 || cell >= w_out) continue;
      const int64_t q = (int64_t)r * w_out + cell;
      const bool inside = c >= 0 && c < n;
      float v = acc[i][j];
      if (FORM == F_FWD) {
        if (SEMI == S_LOG) {
          const float sh = inside ? __ldg(ra + r) + __ldg(rb + c) : 0.f;
          bad |= inside && (!(v >= 8.0779356694631609e-28f) || !(v <= 3.0e38f) || sh < kFloor);
          v = logf(v) + sh;
        }
        if (SEMI == S_MAX)
          g.idx[bt * n * (int64_t)w_out + q] = (inside && best[i][j] >= 0) ? best[i][j] - r + d.a_lu
                                                                            : (inside ? -1 : 0);
        ob[q] = inside ? v : 0.f;  // cells outside the matrix stay zero (banded_cuda_kernel.cu:38)
      } else {
        if (SEMI == S_LOG && inside) {
          const float src = FORM == F_DA ? __ldg(A.p + q) : __ldg(Bm.p + q);
          v *= exp_sfu(src - (FORM == F_DA ? __ldg(ra + r) : __ldg(rb + r)));
        }
        ob[q] = inside ? v : 0.f;
      }
    }
  }
  if (FORM == F_FWD && SEMI == S_LOG) {
    if (__syncthreads_or(bad) && tid == 0) g.flags[bt * nrb + rbk] = 1;
  }
}

// Row maxima over the in-matrix cells of a band tensor: one warp per row; rows without a
// finite entry get 0 (their exponentials become 0 and the row block is flagged).
__global__ void __launch_bounds__(256) band_rowmax_kernel(const float* __restrict__ x, float* __restrict__ r,
                                                          int64_t rows, int64_t n, int lu, int W) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;
  if (row >= rows) return;
  const int64_t i = row % n;
  float m = __int_as_float(0xff800000);
  for (int j = lane; j < W; j += 32) {
    const int64_t c = i + j - lu;
    if (c >= 0 && c < n) m = fmaxf(m, __ldg(x + row * W + j));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) r[row] = (m == __int_as_float(0xff800000)) ? 0.f : m;
}

// Backward: which 64-row blocks did (or would) the forward flag?  S = exp(out - ra - rb) is
// recovered from the saved output; one warp per row, one flag per row block.
__global__ void __launch_bounds__(256) band_flags_kernel(const float* __restrict__ out, const float* __restrict__ ra,
                                                         const float* __restrict__ rb, int* __restrict__ flags,
                                                         int64_t rows, int64_t n, int r_lu, int Wo) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;
  if (row >= rows) return;
  const int64_t bt = row / n, i = row % n;
  bool bad = false;
  const float rai = __ldg(ra + row);
  for (int j = lane; j < Wo; j += 32) {
    const int64_t o = i + j - r_lu;
    if (o < 0 || o >= n) continue;
    const float sh = rai + __ldg(rb + bt * n + o);
    const float ls = __ldg(out + row * Wo + j) - sh;
    bad |= !(ls >= kTinyLog) || sh < kFloor;
  }
  if (__any_sync(0xffffffffu, bad) && lane == 0) flags[bt * ((n + TB - 1) / TB) + i / TB] = 1;
}

template <int FORM, int SEMI>
int launch_block(const BlockArgs& args0, int64_t B, cudaStream_t st) {
  BlockArgs args = args0;
  const BandDims& d = args.d;
  const int w_out = FORM == F_FWD ? d.Wo() : (FORM == F_DA ? d.Wa() : d.Wb());
  args.ncb = (TB + w_out - 2) / TB + 2;
  const int64_t nrb = ceil_div(d.n, TB), blocks = B * nrb * args.ncb;
  if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  band_block_kernel<FORM, SEMI><<<(unsigned)blocks, NTB, 0, st>>>(args);
  return launch_status();
}

}  // namespace

// shared with band_tc.cu
int band_saved_flags(const float* out, const float* ra, const float* rb, int* flags, int64_t B, int64_t n, int r_lu,
                     int Wo, cudaStream_t st) {
  band_flags_kernel<<<(unsigned)ceil_div(B * n, 8), 256, 0, st>>>(out, ra, rb, flags, B * n, n, r_lu, Wo);
  return launch_status();
}

int64_t band_fast_workspace_bytes(int64_t B, int64_t n) {
  return (int64_t)sizeof(float) * (2 * ((B * n + 63) / 64 * 64) + (B * ceil_div(n, TB) + 63) / 64 * 64);
}

static void carve_band(void* ws, int64_t B, int64_t n, float** ra, float** rb, int** flags) {
  float* p = static_cast<float*>(ws);
  *ra = p;
  p += (B * n + 63) / 64 * 64;
  *rb = p;
  p += (B * n + 63) / 64 * 64;
  *flags = reinterpret_cast<int*>(p);
}

int band_fast_forward(int mode, const float* a, const float* b, float* out, int* idx, const BandDims& d, int64_t B,
                      void* ws, int** flags_out, cudaStream_t st) {
  BlockArgs args{a, b, nullptr, nullptr, nullptr, nullptr, nullptr, out, idx, d, 0};
  if (mode == GBMM_BAND_MUL) return launch_block<F_FWD, S_MUL>(args, B, st);
  if (mode == GBMM_BAND_MAX) return launch_block<F_FWD, S_MAX>(args, B, st);
  float *ra, *rb;
  int* flags;
  carve_band(ws, B, d.n, &ra, &rb, &flags);
  if (cudaMemsetAsync(flags, 0, sizeof(int) * B * ceil_div(d.n, TB), st) != cudaSuccess) return GBMM_ERR_LAUNCH;
  const unsigned rows_blocks = (unsigned)ceil_div(B * d.n, 8);
  band_rowmax_kernel<<<rows_blocks, 256, 0, st>>>(a, ra, B * d.n, d.n, d.a_lu, d.Wa());
  band_rowmax_kernel<<<rows_blocks, 256, 0, st>>>(b, rb, B * d.n, d.n, d.b_lu, d.Wb());
  if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
  args.ra = ra;
  args.rb = rb;
  args.flags = flags;
  *flags_out = flags;
  return launch_block<F_FWD, S_LOG>(args, B, st);
}

int band_fast_backward(int mode, const float* a, const float* b, const float* g, const float* part, float* grad_a,
                       float* grad_b, const BandDims& d, int64_t B, void* ws, int** flags_out, cudaStream_t st) {
  BlockArgs args{a, b, g, part, nullptr, nullptr, nullptr, nullptr, nullptr, d, 0};
  if (mode == GBMM_BAND_LOG) {
    float *ra, *rb;
    int* flags;
    carve_band(ws, B, d.n, &ra, &rb, &flags);
    if (cudaMemsetAsync(flags, 0, sizeof(int) * B * ceil_div(d.n, TB), st) != cudaSuccess) return GBMM_ERR_LAUNCH;
    const unsigned rows_blocks = (unsigned)ceil_div(B * d.n, 8);
    band_rowmax_kernel<<<rows_blocks, 256, 0, st>>>(a, ra, B * d.n, d.n, d.a_lu, d.Wa());
    band_rowmax_kernel<<<rows_blocks, 256, 0, st>>>(b, rb, B * d.n, d.n, d.b_lu, d.Wb());
    band_flags_kernel<<<rows_blocks, 256, 0, st>>>(part, ra, rb, flags, B * d.n, d.n, d.r_lu(), d.Wo());
    if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
    args.ra = ra;
    args.rb = rb;
    args.flags = flags;
    *flags_out = flags;
  }
  int rc = GBMM_OK;
  if (grad_a) {
    args.out = grad_a;
    rc = mode == GBMM_BAND_LOG ? launch_block<F_DA, S_LOG>(args, B, st) : launch_block<F_DA, S_MUL>(args, B, st);
    if (rc != GBMM_OK) return rc;
  }
  if (grad_b) {
    args.out = grad_b;
    rc = mode == GBMM_BAND_LOG ? launch_block<F_DB, S_LOG>(args, B, st) : launch_block<F_DB, S_MUL>(args, B, st);
  }
  return rc;
}

}  // namespace gbmm
