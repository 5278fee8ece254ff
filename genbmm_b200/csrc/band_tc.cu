// Banded sum / log products on the tensor cores (3xTF32 on tcgen05), for bands at least 32 wide.
//
// In dense terms a band tensor data:(n,W) with `lu` is a matrix X[r,c] = data[r][c-r+lu], and the
// forward product and both gradients are products between band matrices (see band_block.cu):
//   forward  out[i,o] = sum_p Xa[i,p] Xb[o,p]
//   grad_a   dXa[i,p] = sum_o G[i,o]  Xb[o,p]
//   grad_b   dXb[o,p] = sum_i G[i,o]  Xa[i,p]
// A dense tile of X is a *strided view* of band storage: X[r,c] sits r*(W-1) + c + lu elements
// after the start, i.e. rows W-1 elements apart and columns contiguous — except that cells outside
// the band alias the neighbouring rows.  So every operand is first copied (exponentiated for the
// log semiring, split into tf32 hi + lo) into a "skewed" layout with zero padding after each row:
// pitch = off + W + 192 (pitch % 4 == 1, off zero columns in front so that lu + off is a multiple
// of 32).  With 192 zeros between consecutive rows' bands, any 128 x 32 box of the view (pitch - 1
// elements between rows) that touches the band reads the band cells where they are and zeros
// elsewhere, and TMA can fetch it: as a K-major tile (reduction index contiguous) through a 3-D map,
// or as an MN-major tile (result index contiguous) through a 4-D map, exactly the two operand forms
// of the dense kernel (dense_tc.cu).  The padding is written once (gbmm_band_tc_workspace_init) and
// never again: the per-call copy only rewrites the W band columns.
//
// band_tc_kernel is the persistent single-CTA tcgen05 kernel of dense_tc.cu with three changes:
// tiles are enumerated over the 128x128 blocks that meet the result band, each with its own
// reduction range (where both operand bands are populated); the two operands take separate TMA
// coordinates; and the epilogue scatters a tile's band cells into band storage (each tile row is a
// contiguous run of a band row).  A chunk accumulates in a pair of TMEM buffers (hi*hi products in one, the
// two correction products in the other).  Log semiring: factorised like the dense path (row maxima, guard
// flags per 64-row block, flagged blocks redone by the exact kernels of band.cu).
#include <algorithm>

#include "band.cuh"
#include "tc.cuh"

namespace gbmm {
namespace {

// Zero columns after every row of a skewed copy.  TMA fetches an operand tile as 128 / BOX boxes: BOX result
// indices x 32 reduction steps of a K-major tile, or the same number of cells of an MN-major one (BOX <= 32:
// 32 result indices x BOX reduction steps; 64: 64 x 32), each a whole number of 1 KB swizzle groups of the tile.
// Across such a box the band offset varies by at most BOX - 1 + 31, so a box that meets the band reads, outside
// it, fewer than BOX + 31 cells to either side of a row's band cells: zeros, with a pad of BOX + 32.  (A box
// that does not meet the band at all is fetched from an out-of-range coordinate instead, which TMA fills with
// zeros.)  With whole 128-row boxes the pad was 192 and the copies 2.5 times the band at 129 diagonals.
#ifndef GBMM_BAND_BOX
#define GBMM_BAND_BOX 32
#endif
constexpr int BOX = GBMM_BAND_BOX;
static_assert(BOX == 8 || BOX == 16 || BOX == 32 || BOX == 64 || BOX == 128, "box rows");
constexpr int SKEW_PAD = BOX + 32;
constexpr int NBOX = TM / BOX;                       // boxes per operand tile
constexpr int MN_KB = BOX <= 32 ? BOX : 32;          // MN-major box: reduction rows ...
constexpr int MN_NBLK = BOX <= 32 ? 1 : BOX / 32;    // ... and 32-index blocks

struct Skew {
  int off, pitch, kofs;   // zero columns in front, floats per row, lu + off (a multiple of 4)
  int64_t bstride;        // floats per batch element (a multiple of 4)
};
Skew make_skew(int lu, int W, int64_t n) {
  Skew s;
  s.off = (4 - lu % 4) % 4;
  s.pitch = s.off + W + SKEW_PAD;
  s.pitch += (1 - s.pitch % 4 + 4) % 4;
  s.kofs = lu + s.off;
  s.bstride = (n * s.pitch + 3) & ~int64_t(3);
  return s;
}
int64_t skew_floats(const Skew& s, int64_t B) { return pad64(B * s.bstride + 64); }

// One warp per band row.  KIND 0: v = x.  KIND 1: v = exp(x - m), m = the row's maximum over its in-matrix
// cells (0 when there is none), also written to ra_out[row].  KIND 2: v = g * exp(ra[row] + rb[col] - x), x
// the saved output, 0 in flagged 64-row blocks.  Cells outside the matrix become 0.  Rows of up to 32 * NV
// cells are held in registers (all loads of a row in flight at once); wider rows are walked twice.
template <int KIND, int NV>
__global__ void __launch_bounds__(256) band_skew_kernel(const float* __restrict__ x, const float* __restrict__ g,
                                                        const float* __restrict__ ra, const float* __restrict__ rb,
                                                        const int* __restrict__ flags, float* __restrict__ ra_out,
                                                        float* __restrict__ hi, float* __restrict__ lo, int64_t rows,
                                                        int n, int lu, int W, int off, int pitch, int64_t bstride) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;
  if (row >= rows) return;
  const int i = (int)(row % n);
  const int64_t bt = row / n;
  const float* xr = x + row * W;
  // in-matrix cells of this row: j in [jlo, jhi)
  const int jlo = max(0, lu - i), jhi = min(W, n - i + lu);
  float* hr = hi + bt * bstride + (int64_t)i * pitch + off;
  float* lr = lo + bt * bstride + (int64_t)i * pitch + off;
  const float* gr = KIND == 2 ? g + row * W : nullptr;
  const float* rbb = KIND == 2 ? rb + bt * n + (i - lu) : nullptr;  // rbb[j] = rb of column i + j - lu
  float shift = 0.f;
  bool dead = false;
  if (KIND == 2) {
    shift = __ldg(ra + row);
    dead = __ldg(flags + bt * ((n + 63) / 64) + i / 64) != 0;
  }
  if (W <= 32 * NV) {
    float xv[NV], gv[NV], cv[NV];
#pragma unroll
    for (int q = 0; q < NV; ++q) {
      const int j = lane + 32 * q;
      const bool in = j >= jlo && j < jhi;
      xv[q] = in ? __ldg(xr + j) : __int_as_float(0xff800000);
      gv[q] = (KIND == 2 && in) ? __ldg(gr + j) : 0.f;
      cv[q] = (KIND == 2 && in) ? __ldg(rbb + j) : 0.f;
    }
    if (KIND == 1) {
      float m = xv[0];
#pragma unroll
      for (int q = 1; q < NV; ++q) m = fmaxf(m, xv[q]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      shift = (m == __int_as_float(0xff800000)) ? 0.f : m;
      if (lane == 0) ra_out[row] = shift;
    }
#pragma unroll
    for (int q = 0; q < NV; ++q) {
      const int j = lane + 32 * q;
      if (j >= W) break;
      float v = 0.f;
      if (j >= jlo && j < jhi) {
        if (KIND == 0) v = xv[q];
        if (KIND == 1) v = exp_sfu(xv[q] - shift);
        if (KIND == 2) v = dead ? 0.f : gv[q] * exp_sfu((shift + cv[q]) - xv[q]);
      }
      if (lo == nullptr) {   // one unsplit copy: the product kernel splits it in shared memory
        hr[j] = v;
      } else {
        const float h = tf32_round(v);
        hr[j] = h;
        lr[j] = v - h;
      }
    }
    return;
  }
  if (KIND == 1) {
    float m = __int_as_float(0xff800000);
    for (int j = jlo + lane; j < jhi; j += 32) m = fmaxf(m, __ldg(xr + j));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    shift = (m == __int_as_float(0xff800000)) ? 0.f : m;
    if (lane == 0) ra_out[row] = shift;
  }
  for (int j = lane; j < W; j += 32) {
    float v = 0.f;
    if (j >= jlo && j < jhi) {
      const float xv = __ldg(xr + j);
      if (KIND == 0) v = xv;
      if (KIND == 1) v = exp_sfu(xv - shift);
      if (KIND == 2) v = dead ? 0.f : __ldg(gr + j) * exp_sfu((shift + __ldg(rbb + j)) - xv);
    }
    if (lo == nullptr) {
      hr[j] = v;
    } else {
      const float h = tf32_round(v);
      hr[j] = h;
      lr[j] = v - h;
    }
  }
}

template <int KIND>
int launch_skew(const float* x, const float* g, const float* ra, const float* rb, const int* flags, float* ra_out,
                float* hi, float* lo, int64_t B, int64_t n, int lu, int W, const Skew& s, cudaStream_t st) {
  const int64_t rows = B * n, blocks = ceil_div(rows, 8);
  if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  if (W <= 256)
    band_skew_kernel<KIND, 8><<<(unsigned)blocks, 256, 0, st>>>(x, g, ra, rb, flags, ra_out, hi, lo, rows, (int)n, lu,
                                                               W, s.off, s.pitch, s.bstride);
  else
    band_skew_kernel<KIND, 16><<<(unsigned)blocks, 256, 0, st>>>(x, g, ra, rb, flags, ra_out, hi, lo, rows, (int)n, lu,
                                                                W, s.off, s.pitch, s.bstride);
  return launch_status();
}

// Tensor maps over a skewed copy.  !MN: contiguous index = reduction (coordinate s + kofs), rows = result
// index.  MN: contiguous index = result (32-blocks (r + kofs) / 32), rows = reduction.
template <bool MN>
bool make_skew_map(CUtensorMap* map, const float* base, int64_t B, int64_t n, const Skew& s) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  if (reinterpret_cast<uintptr_t>(base) & 15) return false;
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const cuuint64_t rstride = (cuuint64_t)(s.pitch - 1) * sizeof(float), bstride = (cuuint64_t)s.bstride * sizeof(float);
  if (MN) {
    // contiguous index = result index + kofs, cut into (index % 32, index / 32); the map starts kofs % 32 floats
    // into the copy so that result index r sits in block (r + kofs - kofs % 32) / 32
    const cuuint64_t dims[4] = {32, (cuuint64_t)n, (cuuint64_t)(n + s.kofs + 128 + 63) / 32, (cuuint64_t)B};
    const cuuint64_t strides[3] = {rstride, 32 * sizeof(float), bstride};
    const cuuint32_t box[4] = {32, MN_KB, MN_NBLK, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base + s.kofs % 32), dims, strides, box,
              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  const cuuint64_t dims[3] = {(cuuint64_t)(n + s.kofs + 32), (cuuint64_t)n, (cuuint64_t)B};
  const cuuint64_t strides[2] = {rstride, bstride};
  const cuuint32_t box[3] = {TK, BOX, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

enum { E_SUM = 0, E_LOG = 1, E_GRADLOG = 2 };   // E_GRADLOG: out = sum * exp(src - ra[row]), src laid out like out

struct BandTcArgs {
  int n, lu_out, w_out;      // result band
  int xl, xu, yl, yu;        // operand supports: s - r in [-xl, xu], s - c in [-yl, yu]
  int kofs_x, kofs_y;        // lu + off of the two skewed operands
  int nrb, ncb;              // 128-row blocks, candidate column tiles per row block
  int64_t total;             // batch * nrb * ncb
  float* out;                // (batch, n, w_out)
  const float* ra;           // E_LOG: row maxima of a; E_GRADLOG: row maxima of the operand the gradient is for
  const float* rb;           // E_LOG: row maxima of b
  const float* src;          // E_GRADLOG: that operand, (batch, n, w_out)
  int* flags;                // E_LOG: (batch, ceil(n / 64))
  int* error;
};

// Tile `tile` -> batch element, first row / column, first reduction index (a multiple of 32) and number of
// 32-step stages.  false: the tile lies beyond the result band and owns no cell.  nt == 0: the tile owns band
// cells but no term reaches them (outside the matrix, or no common support): zeros are written.
__device__ __forceinline__ bool band_tile(const BandTcArgs& g, int64_t tile, int& bt, int& r0, int& c0, int& s0,
                                          int& nt) {
  const int cbi = (int)(tile % g.ncb);
  const int rbk = (int)((tile / g.ncb) % g.nrb);
  bt = (int)(tile / ((int64_t)g.ncb * g.nrb));
  r0 = rbk * TM;
  const int lo = r0 - g.lu_out;
  const int cfirst = lo >= 0 ? lo / TN : -((-lo + TN - 1) / TN);
  c0 = (cfirst + cbi) * TN;
  if (c0 > r0 + TM - 1 + (g.w_out - 1 - g.lu_out)) return false;
  const int s_lo = max(max(r0 - g.xl, c0 - g.yl), 0);
  int s_hi = min(min(r0 + TM - 1 + g.xu, c0 + TN - 1 + g.yu), g.n - 1);
  if (c0 >= g.n || c0 + TN - 1 < 0) s_hi = s_lo - 1;
  s0 = s_lo & ~31;
  nt = s_hi >= s_lo ? (s_hi - s0) / TK + 1 : 0;
  return true;
}

// One warp's 32 rows x TEC columns of a tile: band cells (col - row + lu_out in [0, w_out)) go to band
// storage; lanes run along columns, so a tile row is written as one contiguous run.  The epilogue reads nothing
// large from global memory: every load it issues queues behind the SM's TMA traffic for microseconds, so the log
// gradients' factor exp(a - ra) is applied by a separate pass (band_scale_kernel).  E_GRADLOG is the fused form
// (one load per cell, from the operand's own band storage at the offset the result is written to), selectable
// and measured slower (see band_fused_scale).
template <int EPI>
__device__ __forceinline__ void store_band32(const float (&sum)[32], float* blk, const BandTcArgs& g, int bt, int row0,
                                             int col0, int lane, float rshift, bool& bad) {
  float* ob = g.out + (int64_t)bt * g.n * g.w_out;
  const int rows = min(32, g.n - row0);
  __syncwarp();
#pragma unroll
  for (int q = 0; q < 32; ++q) blk[lane * 33 + q] = sum[q];
  __syncwarp();
  const int c = col0 + lane;
  const bool inside = c >= 0 && c < g.n;
  float cshift = 0.f;
  if (EPI == E_LOG && inside) cshift = __ldg(g.rb + (int64_t)bt * g.n + c);
  // cell of (row0 + rr, c) = c - row0 - rr + lu_out: valid rr in [rr_lo, rr_hi); consecutive rows of this
  // lane's column are w_out - 1 elements apart in band storage
  const int top = c - row0 + g.lu_out;  // cell at rr = 0
  const int rr_lo = max(0, top - (g.w_out - 1)), rr_hi = min(rows, top + 1);
  float* op = ob + (int64_t)row0 * g.w_out + top;
  const int step = g.w_out - 1;
  if (EPI == E_GRADLOG) {
    // the factor exp(src - shift[row]) of this lane's 32 cells, multiplied into the block in shared memory: all
    // 32 loads are issued before the first is used (one round trip to memory per block instead of eight)
    const float* sp = g.src + (int64_t)bt * g.n * g.w_out + (int64_t)row0 * g.w_out + top;
    float sv[32];
#pragma unroll
    for (int rr = 0; rr < 32; ++rr)
      sv[rr] = (inside && rr >= rr_lo && rr < rr_hi) ? __ldg(sp + rr * step) : 0.f;
#pragma unroll
    for (int rr = 0; rr < 32; ++rr) {
      const float rs = __shfl_sync(0xffffffffu, rshift, rr);
      blk[rr * 33 + lane] *= exp_sfu(sv[rr] - rs);
    }
  }
  // (not fully unrolled: 64 copies of this body do not fit the instruction cache)
#pragma unroll 4
  for (int rr = 0; rr < 32; ++rr) {
    const float rs = EPI == E_LOG ? __shfl_sync(0xffffffffu, rshift, rr) : 0.f;
    if (rr >= rr_lo && rr < rr_hi) {
      const float v = blk[rr * 33 + lane];
      float o = 0.f;
      if (inside) {
        if (EPI != E_LOG) o = v;
        if (EPI == E_LOG) {
          const float sh = rs + cshift;
          bad |= !(v >= kTiny) || !(v <= 3.0e38f) || (sh < kFloor);
          o = __logf(v) + sh;
        }
      }
      op[rr * step] = o;  // cells outside the matrix stay zero (banded_cuda_kernel.cu:38)
    }
  }
}

template <int EPI>
__device__ __forceinline__ void store_band(const float (&sum)[TEC], float* blk, const BandTcArgs& g, int bt, int row0,
                                           int col0, int lane, bool& bad) {
  // shift of row row0 + lane, handed round by shuffles
  float rshift = 0.f;
  if (EPI != E_SUM && row0 + lane < g.n) rshift = __ldg(g.ra + (int64_t)bt * g.n + row0 + lane);
#pragma unroll
  for (int pass = 0; pass < TEC / 32; ++pass) {
    float part[32];
#pragma unroll
    for (int q = 0; q < 32; ++q) part[q] = sum[pass * 32 + q];
    store_band32<EPI>(part, blk, g, bt, row0, col0 + pass * 32, lane, rshift, bad);
  }
}

// grad[row][j] *= exp(src[row][j] - shift[row]) over the in-matrix cells of a band tensor (the others hold 0).
__global__ void __launch_bounds__(256) band_scale_kernel(float* __restrict__ grad, const float* __restrict__ src,
                                                         const float* __restrict__ shift, int64_t rows, int n, int lu,
                                                         int W) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;
  if (row >= rows) return;
  const int i = (int)(row % n);
  const int jlo = max(0, lu - i), jhi = min(W, n - i + lu);
  const float sh = __ldg(shift + row);
  for (int j = jlo + lane; j < jhi; j += 32)
    grad[row * W + j] *= exp_sfu(__ldg(src + row * W + j) - sh);
}

template <int EPI, bool X_MN, bool Y_MN>
__global__ void __launch_bounds__(TNT, 1) band_tc_kernel(const __grid_constant__ CUtensorMap mx_hi,
                                                         const __grid_constant__ CUtensorMap mx_lo,
                                                         const __grid_constant__ CUtensorMap my_hi,
                                                         const __grid_constant__ CUtensorMap my_lo, BandTcArgs g) {
  extern __shared__ unsigned char smem_raw[];
  TcSmem& sm = *reinterpret_cast<TcSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < TST; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
#pragma unroll
    for (int q = 0; q < TNB; ++q) {
      mbar_init(&sm.chunk_full[q], 1);
      mbar_init(&sm.chunk_empty[q], TEW);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  bool fail = false;

  if (warp == 0) {
    // Lane 0 waits for the stage and announces its bytes; lanes 0 .. NBOX-1 then fetch one box of each of the four
    // tiles: box `lane` of a K-major tile is its rows BOX * lane .. + BOX - 1; of an MN-major tile, the matching
    // group of reduction rows of a 32-index block.  A box that lies wholly outside the operand's band is read from
    // a row coordinate beyond the matrix (zero fill) — its true coordinates would alias other rows' band cells.
    uint32_t it = 0;
    const int oob = g.n + BOX;
    for (int64_t tile = blockIdx.x; tile < g.total && !fail; tile += gridDim.x) {
      int bt, r0, c0, s0, nt;
      if (!band_tile(g, tile, bt, r0, c0, s0, nt)) continue;
      for (int t = 0; t < nt; ++t, ++it) {
        const int s = it % TST, sr = s0 + t * TK;
        int ok = 1;
        if (lane == 0) {
          if (it >= TST && !mbar_wait_bounded(&sm.empty[s], ((it / TST) - 1) & 1)) ok = 0;
          if (ok) mbar_arrive_expect_tx(&sm.full[s], 4 * kTileBytes);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          fail = true;
          break;
        }
        if (lane < NBOX) {
          // MN-major box `lane`: first block and first reduction row, offset in the tile (floats)
          const int mblk = BOX <= 32 ? lane / (32 / MN_KB) : lane * MN_NBLK;
          const int mk = BOX <= 32 ? MN_KB * (lane % (32 / MN_KB)) : 0;
          const int mat = mblk * 1024 + mk * 32;
          if (X_MN) {
            const int rho = r0 + 32 * mblk, k = sr + mk;
            const bool hit = (k + MN_KB - 1 - rho) >= -g.xl && (k - (rho + 32 * MN_NBLK - 1)) <= g.xu;
            const int blk = (rho + g.kofs_x - g.kofs_x % 32) / 32;
            tma_load_4d(sm.a_hi[s] + mat, &mx_hi, &sm.full[s], 0, hit ? k : oob, blk, bt);
            tma_load_4d(sm.a_lo[s] + mat, &mx_lo, &sm.full[s], 0, hit ? k : oob, blk, bt);
          } else {
            const int r = r0 + BOX * lane;
            const bool hit = (sr + TK - 1 - r) >= -g.xl && (sr - (r + BOX - 1)) <= g.xu;
            tma_load_3d(sm.a_hi[s] + lane * BOX * 32, &mx_hi, &sm.full[s], sr + g.kofs_x, hit ? r : oob, bt);
            tma_load_3d(sm.a_lo[s] + lane * BOX * 32, &mx_lo, &sm.full[s], sr + g.kofs_x, hit ? r : oob, bt);
          }
          if (Y_MN) {
            const int rho = c0 + 32 * mblk, k = sr + mk;
            const bool hit = (k + MN_KB - 1 - rho) >= -g.yl && (k - (rho + 32 * MN_NBLK - 1)) <= g.yu;
            const int blk = (rho + g.kofs_y - g.kofs_y % 32) / 32;
            tma_load_4d(sm.b_hi[s] + mat, &my_hi, &sm.full[s], 0, hit ? k : oob, blk, bt);
            tma_load_4d(sm.b_lo[s] + mat, &my_lo, &sm.full[s], 0, hit ? k : oob, blk, bt);
          } else {
            const int r = c0 + BOX * lane;
            const bool hit = (sr + TK - 1 - r) >= -g.yl && (sr - (r + BOX - 1)) <= g.yu;
            tma_load_3d(sm.b_hi[s] + lane * BOX * 32, &my_hi, &sm.full[s], sr + g.kofs_y, hit ? r : oob, bt);
            tma_load_3d(sm.b_lo[s] + lane * BOX * 32, &my_lo, &sm.full[s], sr + g.kofs_y, hit ? r : oob, bt);
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = kIdesc | (X_MN ? 1u << 15 : 0u) | (Y_MN ? 1u << 16 : 0u);
      uint32_t it = 0, gc = 0;
      for (int64_t tile = blockIdx.x; tile < g.total && !fail; tile += gridDim.x) {
        int bt, r0, c0, s0, nt;
        if (!band_tile(g, tile, bt, r0, c0, s0, nt)) continue;
        for (int t = 0; t < nt; ++t, ++it) {
          // a chunk accumulates in a pair of TMEM buffers: the hi*hi products in one, the two correction
          // products (2^-11 of their size) in the other, so the large sum is truncated once per reduction
          // step of 8 instead of three times
          const int s = it % TST, buf = gc % (TNB / 2);
          const bool chunk_start = (t % TCH) == 0;
          if (chunk_start && gc >= TNB / 2 &&
              !mbar_wait_bounded(&sm.chunk_empty[buf], ((gc / (TNB / 2)) - 1) & 1)) {
            fail = true;
            break;
          }
          if (!mbar_wait_bounded(&sm.full[s], (it / TST) & 1)) {
            fail = true;
            break;
          }
          tc_fence_after();
          const uint32_t acc = tmem + (uint32_t)(2 * buf * TN), acc_c = acc + TN;
#pragma unroll
          for (int kk = 0; kk < TK / 8; ++kk) {
            const int ko = kk * 8 * (int)sizeof(float);
            const uint64_t ah = X_MN ? umma_desc_mn(sm.a_hi[s], kk) : umma_desc(sm.a_hi[s], ko);
            const uint64_t al = X_MN ? umma_desc_mn(sm.a_lo[s], kk) : umma_desc(sm.a_lo[s], ko);
            const uint64_t bh = Y_MN ? umma_desc_mn(sm.b_hi[s], kk) : umma_desc(sm.b_hi[s], ko);
            const uint64_t bl = Y_MN ? umma_desc_mn(sm.b_lo[s], kk) : umma_desc(sm.b_lo[s], ko);
            const uint32_t more = (!chunk_start || kk > 0) ? 1u : 0u;
            umma_tf32(acc_c, al, bh, idesc, more);
            umma_tf32(acc_c, ah, bl, idesc, 1u);
            umma_tf32(acc, ah, bh, idesc, more);
          }
          umma_commit(&sm.empty[s]);
          if ((t % TCH) == TCH - 1 || t == nt - 1) {
            umma_commit(&sm.chunk_full[buf]);
            ++gc;
          }
        }
      }
    }
    __syncwarp();
  } else {
    const int quad = warp % 4;
    const int cbase = ((warp - 2) / 4) * TEC;
    float* blk = sm.epi[warp - 2];
    uint32_t gc = 0;
    for (int64_t tile = blockIdx.x; tile < g.total && !fail; tile += gridDim.x) {
      int bt, r0, c0, s0, nt;
      if (!band_tile(g, tile, bt, r0, c0, s0, nt)) continue;
      const int nchunks = (nt + TCH - 1) / TCH;
      float sum[TEC];
#pragma unroll
      for (int q = 0; q < TEC; ++q) sum[q] = 0.f;
      for (int chunk = 0; chunk < nchunks; ++chunk, ++gc) {
        const int buf = gc % (TNB / 2);
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&sm.chunk_full[buf], (gc / (TNB / 2)) & 1))) {
          fail = true;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < TEC / 32; ++c) {
          float v[32], w[32];
          const uint32_t col = (uint32_t)(2 * buf * TN + cbase + c * 32);
          tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + col, v);
          tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + col + TN, w);
#pragma unroll
          for (int q = 0; q < 32; ++q) sum[c * 32 + q] += v[q] + w[q];
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0)
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.chunk_empty[buf])) : "memory");
      }
      if (fail) break;
      bool bad = false;
      store_band<EPI>(sum, blk, g, bt, r0 + quad * 32, c0 + cbase, lane, bad);
      if (EPI == E_LOG) {
        const int row0 = r0 + quad * 32;
        if (__any_sync(0xffffffffu, bad) && lane == 0 && row0 < g.n)
          atomicExch(g.flags + (int64_t)bt * ((g.n + 63) / 64) + row0 / 64, 1);
      }
    }
  }
  if (__any_sync(0xffffffffu, fail) && lane == 0) atomicExch(g.error, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

struct SkewOperand {
  const float* hi;
  const float* lo;
  Skew s;
};

template <int EPI, bool X_MN, bool Y_MN>
int launch_band_tc(const SkewOperand& X, const SkewOperand& Y, BandTcArgs args, int64_t B, cudaStream_t st) {
  CUtensorMap m0, m1, m2, m3;
  if (!make_skew_map<X_MN>(&m0, X.hi, B, args.n, X.s) || !make_skew_map<X_MN>(&m1, X.lo, B, args.n, X.s) ||
      !make_skew_map<Y_MN>(&m2, Y.hi, B, args.n, Y.s) || !make_skew_map<Y_MN>(&m3, Y.lo, B, args.n, Y.s))
    return GBMM_ERR_LAUNCH;
  args.kofs_x = X.s.kofs;
  args.kofs_y = Y.s.kofs;
  args.nrb = (int)ceil_div((int64_t)args.n, TM);
  args.ncb = (args.w_out + 2 * TN - 2) / TN + 1;
  args.total = B * args.nrb * args.ncb;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return GBMM_ERR_DEVICE;
  const unsigned blocks = (unsigned)(args.total < sms ? args.total : sms);
  const size_t smem = sizeof(TcSmem) + 1024;
  if (cudaFuncSetAttribute(band_tc_kernel<EPI, X_MN, Y_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return GBMM_ERR_LAUNCH;
  band_tc_kernel<EPI, X_MN, Y_MN><<<blocks, TNT, smem, st>>>(m0, m1, m2, m3, args);
  return launch_status();
}

// ------------------------------------------------------------------------------------------------------------
// Converter-fed variant: no operand copies at all.
//
// The kernel above streams padded hi/lo copies of its operands: 5 bytes of HBM traffic per band byte, written by
// one pass and read back by the next, which is what bounds it.  Here the operand tiles are built where they
// are consumed.  Eight converter warps read the band tensors themselves (coalesced along the band row), apply
// everything the copy pass did — zero outside band and matrix, exp(x - row maximum) for the log semiring, the
// tf32 hi / lo split — and write the four tiles of a stage straight into shared memory in the layout
// tcgen05.mma reads (K-major rows of 128 bytes, 128-byte swizzle: 16-byte chunk c of row r sits at chunk
// c ^ (r & 7)).  Both operand forms become K-major tiles, so no MN-major descriptor is needed:
//   ROW  element (r, s) = data[r][s - r + lu]   lanes run along s: one row of the tile per warp-wide load
//   COL  element (r, s) = data[s][r - s + lu]   lanes run along r: four warp-wide loads (s .. s+3) make one
//                                               16-byte chunk per lane, stored with one 128-bit store
// A stage is handed to the MMA warp through `full` (one arrival per converter warp, after a
// fence.proxy.async: the tensor core reads shared memory through the async proxy) and comes back through `empty`
// (tcgen05.commit).  The MMA warp and the eight epilogue warps are those of the kernel above; every tile's
// reduction fits one accumulation chunk here (band_cv_fits), so the epilogue reads each TMEM buffer pair once.
// DRAM traffic per product: the operands once (neighbouring tiles share rows through L2) and the result.
constexpr int CVW = 8;                          // converter warps
constexpr int CV_NT = (CVW + 1 + TEW) * 32;     // + MMA warp + epilogue warps

struct CvOperand {
  const float* data;    // (batch, n, W) band tensor
  const float* shift;   // log semiring: (batch, n) maximum of each storage row, else null
  int W, lu;
};

struct BandCvArgs {
  BandTcArgs g;
  CvOperand x, y;
};

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Loads the 16 values a thread contributes to one operand tile; bit q of `mask` says whether value q is a cell
// of the band inside the matrix (the others are 0).  `sh` is this lane's share of the shifts (log semiring).
template <bool COL>
__device__ __forceinline__ void cv_load(float (&v)[16], uint32_t& mask, float& sh, const CvOperand& op, int64_t bt,
                                        int n, int r0, int s0, int cw, int lane) {
  const float* base = op.data + bt * (int64_t)n * op.W;
  mask = 0;
  if (!COL) {
#pragma unroll
    for (int q = 0; q < 16; ++q) {
      const int r = r0 + cw * 16 + q, sc = s0 + lane, j = sc - r + op.lu;
      const bool ok = r >= 0 && r < n && sc < n && j >= 0 && j < op.W;
      v[q] = ok ? __ldg(base + (int64_t)r * op.W + j) : 0.f;
      mask |= ok ? (1u << q) : 0u;
    }
    // shift of row cw * 16 + (lane & 15), handed round by shuffles
    const int rr = r0 + cw * 16 + (lane & 15);
    sh = (op.shift && rr >= 0 && rr < n) ? __ldg(op.shift + bt * n + rr) : 0.f;
  } else {
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int u = cw * 4 + t, r = r0 + (u >> 3) * 32 + lane, c = u & 7;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int sc = s0 + 4 * c + e, j = r - sc + op.lu;
        const bool ok = r >= 0 && r < n && sc < n && j >= 0 && j < op.W;
        v[t * 4 + e] = ok ? __ldg(base + (int64_t)sc * op.W + j) : 0.f;
        mask |= ok ? (1u << (t * 4 + e)) : 0u;
      }
    }
    // shift of storage row s0 + lane
    sh = (op.shift && s0 + lane < n) ? __ldg(op.shift + bt * n + s0 + lane) : 0.f;
  }
}

template <bool COL>
__device__ __forceinline__ void cv_store(const float (&v)[16], uint32_t mask, float sh, bool has_shift, float* hi,
                                         float* lo, int cw, int lane) {
  if (!COL) {
#pragma unroll
    for (int q = 0; q < 16; ++q) {
      const int rl = cw * 16 + q;
      float x = v[q];
      if (has_shift) {
        const float e = exp_sfu(x - __shfl_sync(0xffffffffu, sh, q));
        x = ((mask >> q) & 1u) ? e : 0.f;
      }
      const float h = tf32_round(x);
      const int at = rl * 32 + ((((lane >> 2) ^ (rl & 7)) << 2) | (lane & 3));
      hi[at] = h;
      lo[at] = x - h;
    }
  } else {
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int u = cw * 4 + t, rl = (u >> 3) * 32 + lane, c = u & 7;
      float h[4], l[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float x = v[t * 4 + e];
        if (has_shift) {
          const float ex = exp_sfu(x - __shfl_sync(0xffffffffu, sh, 4 * c + e));
          x = ((mask >> (t * 4 + e)) & 1u) ? ex : 0.f;
        }
        h[e] = tf32_round(x);
        l[e] = x - h[e];
      }
      const int at = rl * 32 + ((c ^ (rl & 7)) << 2);
      *reinterpret_cast<float4*>(hi + at) = make_float4(h[0], h[1], h[2], h[3]);
      *reinterpret_cast<float4*>(lo + at) = make_float4(l[0], l[1], l[2], l[3]);
    }
  }
}

template <int EPI, bool X_COL, bool Y_COL>
__global__ void __launch_bounds__(CV_NT, 1) band_cv_kernel(BandCvArgs p) {
  extern __shared__ unsigned char smem_raw[];
  TcSmem& sm = *reinterpret_cast<TcSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const BandTcArgs& g = p.g;
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < TST; ++s) {
      mbar_init(&sm.full[s], CVW);
      mbar_init(&sm.empty[s], 1);
    }
#pragma unroll
    for (int q = 0; q < TNB; ++q) {
      mbar_init(&sm.chunk_full[q], 1);
      mbar_init(&sm.chunk_empty[q], TEW);
    }
    fence_barrier_init();
  }
  if (warp == CVW) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  bool fail = false;

  if (warp < CVW) {
    // ---- converters: band storage -> the four operand tiles of a stage
    uint32_t it = 0;
    for (int64_t tile = blockIdx.x; tile < g.total && !fail; tile += gridDim.x) {
      int bt, r0, c0, s0, nt;
      if (!band_tile(g, tile, bt, r0, c0, s0, nt)) continue;
      for (int t = 0; t < nt; ++t, ++it) {
        const int s = it % TST, sr = s0 + t * TK;
        float xv[16], yv[16], xs, ys;
        uint32_t xm, ym;
        // the loads of this stage are in flight while the stage's buffers are still being read
        cv_load<X_COL>(xv, xm, xs, p.x, bt, g.n, r0, sr, warp, lane);
        cv_load<Y_COL>(yv, ym, ys, p.y, bt, g.n, c0, sr, warp, lane);
        if (it >= TST && !__all_sync(0xffffffffu, mbar_wait_bounded(&sm.empty[s], ((it / TST) - 1) & 1))) {
          fail = true;
          break;
        }
        cv_store<X_COL>(xv, xm, xs, p.x.shift != nullptr, sm.a_hi[s], sm.a_lo[s], warp, lane);
        cv_store<Y_COL>(yv, ym, ys, p.y.shift != nullptr, sm.b_hi[s], sm.b_lo[s], warp, lane);
        fence_async_smem();   // these generic-proxy stores, before the tensor core's async-proxy reads
        __syncwarp();
        if (lane == 0)
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.full[s])) : "memory");
      }
    }
  } else if (warp == CVW) {
    if (lane == 0) {
      uint32_t it = 0, gc = 0;
      for (int64_t tile = blockIdx.x; tile < g.total && !fail; tile += gridDim.x) {
        int bt, r0, c0, s0, nt;
        if (!band_tile(g, tile, bt, r0, c0, s0, nt)) continue;
        if (nt == 0) continue;
        const int buf = gc % (TNB / 2);
        if (gc >= TNB / 2 && !mbar_wait_bounded(&sm.chunk_empty[buf], ((gc / (TNB / 2)) - 1) & 1)) {
          fail = true;
          break;
        }
        const uint32_t acc = tmem + (uint32_t)(2 * buf * TN), acc_c = acc + TN;
        for (int t = 0; t < nt; ++t, ++it) {
          const int s = it % TST;
          if (!mbar_wait_bounded(&sm.full[s], (it / TST) & 1)) {
            fail = true;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < TK / 8; ++kk) {
            const int ko = kk * 8 * (int)sizeof(float);
            const uint64_t ah = umma_desc(sm.a_hi[s], ko), al = umma_desc(sm.a_lo[s], ko);
            const uint64_t bh = umma_desc(sm.b_hi[s], ko), bl = umma_desc(sm.b_lo[s], ko);
            const uint32_t more = (t > 0 || kk > 0) ? 1u : 0u;
            umma_tf32(acc_c, al, bh, kIdesc, more);
            umma_tf32(acc_c, ah, bl, kIdesc, 1u);
            umma_tf32(acc, ah, bh, kIdesc, more);
          }
          umma_commit(&sm.empty[s]);
        }
        if (fail) break;
        umma_commit(&sm.chunk_full[buf]);
        ++gc;
      }
    }
    __syncwarp();
  } else {
    // ---- epilogue: TMEM -> band storage, 32 columns at a time (one accumulation chunk per tile)
    const int ew = warp - (CVW + 1), quad = warp % 4;
    const int cbase = (ew / 4) * TEC;
    float* blk = sm.epi[ew];
    uint32_t gc = 0;
    for (int64_t tile = blockIdx.x; tile < g.total && !fail; tile += gridDim.x) {
      int bt, r0, c0, s0, nt;
      if (!band_tile(g, tile, bt, r0, c0, s0, nt)) continue;
      const int row0 = r0 + quad * 32;
      float rshift = 0.f;
      if (EPI != E_SUM && row0 + lane < g.n) rshift = __ldg(g.ra + (int64_t)bt * g.n + row0 + lane);
      bool bad = false;
      if (nt == 0) {
        // the tile owns band cells that no term reaches: zeros outside the matrix; inside it (log semiring) the
        // log of an empty sum, which marks the row block for the exact kernels like any underflow
        float zero[32];
#pragma unroll
        for (int q = 0; q < 32; ++q) zero[q] = 0.f;
#pragma unroll
        for (int c = 0; c < TEC / 32; ++c)
          store_band32<EPI>(zero, blk, g, bt, row0, c0 + cbase + c * 32, lane, rshift, bad);
        if (EPI == E_LOG && __any_sync(0xffffffffu, bad) && lane == 0 && row0 < g.n)
          atomicExch(g.flags + (int64_t)bt * ((g.n + 63) / 64) + row0 / 64, 1);
        continue;
      }
      const int buf = gc % (TNB / 2);
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(&sm.chunk_full[buf], (gc / (TNB / 2)) & 1))) {
        fail = true;
        break;
      }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < TEC / 32; ++c) {
        float v[32], w[32];
        const uint32_t col = (uint32_t)(2 * buf * TN + cbase + c * 32);
        tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + col, v);
        tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + col + TN, w);
#pragma unroll
        for (int q = 0; q < 32; ++q) v[q] += w[q];
        store_band32<EPI>(v, blk, g, bt, row0, c0 + cbase + c * 32, lane, rshift, bad);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0)
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.chunk_empty[buf])) : "memory");
      ++gc;
      if (EPI == E_LOG) {
        if (__any_sync(0xffffffffu, bad) && lane == 0 && row0 < g.n)
          atomicExch(g.flags + (int64_t)bt * ((g.n + 63) / 64) + row0 / 64, 1);
      }
    }
  }
  if (__any_sync(0xffffffffu, fail) && lane == 0) atomicExch(g.error, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == CVW) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------------------
// Split-in-shared-memory variant: ONE unsplit fp32 skewed copy per operand instead of a hi and a lo copy.
//
// TMA fetches the raw fp32 tile (same boxes, same zero padding, K-major or MN-major) into the stage's `hi` buffer;
// eight splitter warps then rewrite it in place — hi = tf32(x) back where x was, lo = x - hi at the same offset of
// the `lo` buffer — with 128-bit shared-memory accesses and no address arithmetic (the split does not care which
// layout the tile has), and hand the stage to the MMA warp (fence.proxy.async, then one arrival per splitter warp
// on `full`).  Halves the bytes the copy pass writes and the products read; costs 96 KB of shared-memory traffic
// per stage next to the 96 KB the twelve MMAs read.  Tiles fit one accumulation chunk (band_max_stages <= TCH),
// so the epilogue reads each TMEM buffer pair once, 32 columns at a time, as in band_cv_kernel.
constexpr int SPW = 8;                               // splitter warps
constexpr int SP_NT = (SPW + 1 + TEW + 1) * 32;      // + MMA warp + epilogue warps + TMA warp
constexpr int SP_TMA_WARP = SPW + 1 + TEW;

template <int EPI, bool X_MN, bool Y_MN>
__global__ void __launch_bounds__(SP_NT, 1) band_sp_kernel(const __grid_constant__ CUtensorMap mx,
                                                           const __grid_constant__ CUtensorMap my, BandTcArgs g) {
  extern __shared__ unsigned char smem_raw[];
  TcSmem& sm = *reinterpret_cast<TcSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < TST; ++s) {
      mbar_init(&sm.raw_full[s], 1);
      mbar_init(&sm.full[s], SPW);
      mbar_init(&sm.empty[s], 1);
    }
#pragma unroll
    for (int q = 0; q < TNB; ++q) {
      mbar_init(&sm.chunk_full[q], 1);
      mbar_init(&sm.chunk_empty[q], TEW);
    }
    fence_barrier_init();
  }
  if (warp == SPW) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  bool fail = false;

  if (warp == SP_TMA_WARP) {
    // ---- producer: raw fp32 tiles into the `hi` buffers (boxes as in band_tc_kernel)
    uint32_t it = 0;
    const int oob = g.n + BOX;
    for (int64_t tile = blockIdx.x; tile < g.total && !fail; tile += gridDim.x) {
      int bt, r0, c0, s0, nt;
      if (!band_tile(g, tile, bt, r0, c0, s0, nt)) continue;
      for (int t = 0; t < nt; ++t, ++it) {
        const int s = it % TST, sr = s0 + t * TK;
        int ok = 1;
        if (lane == 0) {
          if (it >= TST && !mbar_wait_bounded(&sm.empty[s], ((it / TST) - 1) & 1)) ok = 0;
          if (ok) mbar_arrive_expect_tx(&sm.raw_full[s], 2 * kTileBytes);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          fail = true;
          break;
        }
        if (lane < NBOX) {
          const int mblk = BOX <= 32 ? lane / (32 / MN_KB) : lane * MN_NBLK;
          const int mk = BOX <= 32 ? MN_KB * (lane % (32 / MN_KB)) : 0;
          const int mat = mblk * 1024 + mk * 32;
          if (X_MN) {
            const int rho = r0 + 32 * mblk, k = sr + mk;
            const bool hit = (k + MN_KB - 1 - rho) >= -g.xl && (k - (rho + 32 * MN_NBLK - 1)) <= g.xu;
            tma_load_4d(sm.a_hi[s] + mat, &mx, &sm.raw_full[s], 0, hit ? k : oob,
                        (rho + g.kofs_x - g.kofs_x % 32) / 32, bt);
          } else {
            const int r = r0 + BOX * lane;
            const bool hit = (sr + TK - 1 - r) >= -g.xl && (sr - (r + BOX - 1)) <= g.xu;
            tma_load_3d(sm.a_hi[s] + lane * BOX * 32, &mx, &sm.raw_full[s], sr + g.kofs_x, hit ? r : oob, bt);
          }
          if (Y_MN) {
            const int rho = c0 + 32 * mblk, k = sr + mk;
            const bool hit = (k + MN_KB - 1 - rho) >= -g.yl && (k - (rho + 32 * MN_NBLK - 1)) <= g.yu;
            tma_load_4d(sm.b_hi[s] + mat, &my, &sm.raw_full[s], 0, hit ? k : oob,
                        (rho + g.kofs_y - g.kofs_y % 32) / 32, bt);
          } else {
            const int r = c0 + BOX * lane;
            const bool hit = (sr + TK - 1 - r) >= -g.yl && (sr - (r + BOX - 1)) <= g.yu;
            tma_load_3d(sm.b_hi[s] + lane * BOX * 32, &my, &sm.raw_full[s], sr + g.kofs_y, hit ? r : oob, bt);
          }
        }
        __syncwarp();
      }
    }
  } else if (warp < SPW) {
    // ---- splitters: x -> (tf32(x), x - tf32(x)), in place
    uint32_t it = 0;
    for (int64_t tile = blockIdx.x; tile < g.total && !fail; tile += gridDim.x) {
      int bt, r0, c0, s0, nt;
      if (!band_tile(g, tile, bt, r0, c0, s0, nt)) continue;
      for (int t = 0; t < nt; ++t, ++it) {
        const int s = it % TST;
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&sm.raw_full[s], (it / TST) & 1))) {
          fail = true;
          break;
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float4* hi = reinterpret_cast<float4*>(half ? sm.b_hi[s] : sm.a_hi[s]);
          float4* lo = reinterpret_cast<float4*>(half ? sm.b_lo[s] : sm.a_lo[s]);
          float4 x[TM * TK / 4 / (SPW * 32)];
#pragma unroll
          for (int q = 0; q < TM * TK / 4 / (SPW * 32); ++q) x[q] = hi[tid + q * SPW * 32];
#pragma unroll
          for (int q = 0; q < TM * TK / 4 / (SPW * 32); ++q) {
            const float4 h = make_float4(tf32_round(x[q].x), tf32_round(x[q].y), tf32_round(x[q].z),
                                         tf32_round(x[q].w));
            hi[tid + q * SPW * 32] = h;
            lo[tid + q * SPW * 32] = make_float4(x[q].x - h.x, x[q].y - h.y, x[q].z - h.z, x[q].w - h.w);
          }
        }
        fence_async_smem();   // these generic-proxy stores, before the tensor core's async-proxy reads
        __syncwarp();
        if (lane == 0)
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.full[s])) : "memory");
      }
    }
  } else if (warp == SPW) {
    if (lane == 0) {
      constexpr uint32_t idesc = kIdesc | (X_MN ? 1u << 15 : 0u) | (Y_MN ? 1u << 16 : 0u);
      uint32_t it = 0, gc = 0;
      for (int64_t tile = blockIdx.x; tile < g.total && !fail; tile += gridDim.x) {
        int bt, r0, c0, s0, nt;
        if (!band_tile(g, tile, bt, r0, c0, s0, nt)) continue;
        if (nt == 0) continue;
        const int buf = gc % (TNB / 2);
        if (gc >= TNB / 2 && !mbar_wait_bounded(&sm.chunk_empty[buf], ((gc / (TNB / 2)) - 1) & 1)) {
          fail = true;
          break;
        }
        const uint32_t acc = tmem + (uint32_t)(2 * buf * TN), acc_c = acc + TN;
        for (int t = 0; t < nt; ++t, ++it) {
          const int s = it % TST;
          if (!mbar_wait_bounded(&sm.full[s], (it / TST) & 1)) {
            fail = true;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < TK / 8; ++kk) {
            const int ko = kk * 8 * (int)sizeof(float);
            const uint64_t ah = X_MN ? umma_desc_mn(sm.a_hi[s], kk) : umma_desc(sm.a_hi[s], ko);
            const uint64_t al = X_MN ? umma_desc_mn(sm.a_lo[s], kk) : umma_desc(sm.a_lo[s], ko);
            const uint64_t bh = Y_MN ? umma_desc_mn(sm.b_hi[s], kk) : umma_desc(sm.b_hi[s], ko);
            const uint64_t bl = Y_MN ? umma_desc_mn(sm.b_lo[s], kk) : umma_desc(sm.b_lo[s], ko);
            const uint32_t more = (t > 0 || kk > 0) ? 1u : 0u;
            umma_tf32(acc_c, al, bh, idesc, more);
            umma_tf32(acc_c, ah, bl, idesc, 1u);
            umma_tf32(acc, ah, bh, idesc, more);
          }
          umma_commit(&sm.empty[s]);
        }
        if (fail) break;
        umma_commit(&sm.chunk_full[buf]);
        ++gc;
      }
    }
    __syncwarp();
  } else {
    // ---- epilogue: TMEM -> band storage, 32 columns at a time (one accumulation chunk per tile)
    const int ew = warp - (SPW + 1), quad = warp % 4;
    const int cbase = (ew / 4) * TEC;
    float* blk = sm.epi[ew];
    uint32_t gc = 0;
    for (int64_t tile = blockIdx.x; tile < g.total && !fail; tile += gridDim.x) {
      int bt, r0, c0, s0, nt;
      if (!band_tile(g, tile, bt, r0, c0, s0, nt)) continue;
      const int row0 = r0 + quad * 32;
      float rshift = 0.f;
      if (EPI != E_SUM && row0 + lane < g.n) rshift = __ldg(g.ra + (int64_t)bt * g.n + row0 + lane);
      bool bad = false;
      if (nt == 0) {
        // the tile owns band cells that no term reaches: zeros outside the matrix; inside it (log semiring) the
        // log of an empty sum, which marks the row block for the exact kernels like any underflow
        float zero[32];
#pragma unroll
        for (int q = 0; q < 32; ++q) zero[q] = 0.f;
#pragma unroll
        for (int c = 0; c < TEC / 32; ++c)
          store_band32<EPI>(zero, blk, g, bt, row0, c0 + cbase + c * 32, lane, rshift, bad);
        if (EPI == E_LOG && __any_sync(0xffffffffu, bad) && lane == 0 && row0 < g.n)
          atomicExch(g.flags + (int64_t)bt * ((g.n + 63) / 64) + row0 / 64, 1);
        continue;
      }
      const int buf = gc % (TNB / 2);
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(&sm.chunk_full[buf], (gc / (TNB / 2)) & 1))) {
        fail = true;
        break;
      }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < TEC / 32; ++c) {
        float v[32], w[32];
        const uint32_t col = (uint32_t)(2 * buf * TN + cbase + c * 32);
        tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + col, v);
        tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + col + TN, w);
        if (c == TEC / 32 - 1) {
          // the last of this warp's columns is in registers: the MMA warp may have the buffers back while
          // these cells are still on their way to band storage
          tc_fence_before();
          __syncwarp();
          if (lane == 0)
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.chunk_empty[buf])) : "memory");
        }
#pragma unroll
        for (int q = 0; q < 32; ++q) v[q] += w[q];
        store_band32<EPI>(v, blk, g, bt, row0, c0 + cbase + c * 32, lane, rshift, bad);
      }
      ++gc;
      if (EPI == E_LOG) {
        if (__any_sync(0xffffffffu, bad) && lane == 0 && row0 < g.n)
          atomicExch(g.flags + (int64_t)bt * ((g.n + 63) / 64) + row0 / 64, 1);
      }
    }
  }
  if (__any_sync(0xffffffffu, fail) && lane == 0) atomicExch(g.error, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == SPW) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// Host-side copy of band_tile's reduction range: the largest number of 32-step stages any tile of this product
// has.  The converter-fed kernel takes products whose tiles all fit one accumulation chunk (TCH stages).
int band_max_stages(const BandTcArgs& g) {
  const int nrb = (int)ceil_div((int64_t)g.n, TM), ncb = (g.w_out + 2 * TN - 2) / TN + 1;
  int most = 0;
  for (int rbk = 0; rbk < nrb; ++rbk) {
    const int r0 = rbk * TM, lo = r0 - g.lu_out;
    const int cfirst = lo >= 0 ? lo / TN : -((-lo + TN - 1) / TN);
    for (int cbi = 0; cbi < ncb; ++cbi) {
      const int c0 = (cfirst + cbi) * TN;
      if (c0 > r0 + TM - 1 + (g.w_out - 1 - g.lu_out)) continue;
      const int s_lo = std::max(std::max(r0 - g.xl, c0 - g.yl), 0);
      int s_hi = std::min(std::min(r0 + TM - 1 + g.xu, c0 + TN - 1 + g.yu), g.n - 1);
      if (c0 >= g.n || c0 + TN - 1 < 0) s_hi = s_lo - 1;
      const int s0 = s_lo & ~31;
      most = std::max(most, s_hi >= s_lo ? (s_hi - s0) / TK + 1 : 0);
    }
    if (rbk == 2 && nrb > 6) rbk = nrb - 4;   // interior row blocks repeat: the first and last three suffice
  }
  return most;
}

template <int EPI, bool X_COL, bool Y_COL>
int launch_band_cv(const CvOperand& X, const CvOperand& Y, BandTcArgs args, int64_t B, cudaStream_t st) {
  args.kofs_x = args.kofs_y = 0;
  args.nrb = (int)ceil_div((int64_t)args.n, TM);
  args.ncb = (args.w_out + 2 * TN - 2) / TN + 1;
  args.total = B * args.nrb * args.ncb;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return GBMM_ERR_DEVICE;
  const unsigned blocks = (unsigned)(args.total < sms ? args.total : sms);
  const size_t smem = sizeof(TcSmem) + 1024;
  if (cudaFuncSetAttribute(band_cv_kernel<EPI, X_COL, Y_COL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return GBMM_ERR_LAUNCH;
  BandCvArgs p{args, X, Y};
  band_cv_kernel<EPI, X_COL, Y_COL><<<blocks, CV_NT, smem, st>>>(p);
  return launch_status();
}

template <int EPI, bool X_MN, bool Y_MN>
int launch_band_sp(const SkewOperand& X, const SkewOperand& Y, BandTcArgs args, int64_t B, cudaStream_t st) {
  CUtensorMap m0, m1;
  if (!make_skew_map<X_MN>(&m0, X.hi, B, args.n, X.s) || !make_skew_map<Y_MN>(&m1, Y.hi, B, args.n, Y.s))
    return GBMM_ERR_LAUNCH;
  args.kofs_x = X.s.kofs;
  args.kofs_y = Y.s.kofs;
  args.nrb = (int)ceil_div((int64_t)args.n, TM);
  args.ncb = (args.w_out + 2 * TN - 2) / TN + 1;
  args.total = B * args.nrb * args.ncb;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return GBMM_ERR_DEVICE;
  const unsigned blocks = (unsigned)(args.total < sms ? args.total : sms);
  const size_t smem = sizeof(TcSmem) + 1024;
  if (cudaFuncSetAttribute(band_sp_kernel<EPI, X_MN, Y_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return GBMM_ERR_LAUNCH;
  band_sp_kernel<EPI, X_MN, Y_MN><<<blocks, SP_NT, smem, st>>>(m0, m1, args);
  return launch_status();
}

// rmax[row] = maximum of the row's in-matrix cells, 0 when it has none (the shift of the log semiring)
__global__ void __launch_bounds__(256) band_rowmax_cv_kernel(const float* __restrict__ x, float* __restrict__ rmax,
                                                             int64_t rows, int n, int lu, int W) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;
  if (row >= rows) return;
  const int i = (int)(row % n);
  const int jlo = max(0, lu - i), jhi = min(W, n - i + lu);
  float m = __int_as_float(0xff800000);
  for (int j = jlo + lane; j < jhi; j += 32) m = fmaxf(m, __ldg(x + row * W + j));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) rmax[row] = (m == __int_as_float(0xff800000)) ? 0.f : m;
}

// gp[row][j] = g * exp(ra[row] + rb[col] - out) over the in-matrix cells of the result band, 0 elsewhere and
// in flagged 64-row blocks (whose terms the exact kernels add): the cotangent of the factorised sum
__global__ void __launch_bounds__(256) band_gprime_kernel(const float* __restrict__ out, const float* __restrict__ g,
                                                          const float* __restrict__ ra, const float* __restrict__ rb,
                                                          const int* __restrict__ flags, float* __restrict__ gp,
                                                          int64_t rows, int n, int lu, int W) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;
  if (row >= rows) return;
  const int i = (int)(row % n);
  const int64_t bt = row / n;
  const int jlo = max(0, lu - i), jhi = min(W, n - i + lu);
  const float shift = __ldg(ra + row);
  const bool dead = __ldg(flags + bt * ((n + 63) / 64) + i / 64) != 0;
  const float* rbb = rb + bt * n + (i - lu);
  for (int j = lane; j < W; j += 32) {
    float v = 0.f;
    if (!dead && j >= jlo && j < jhi)
      v = __ldg(g + row * W + j) * exp_sfu((shift + __ldg(rbb + j)) - __ldg(out + row * W + j));
    gp[row * W + j] = v;
  }
}

struct BandWs {
  int* error;
  float *ra, *rb;
  int* flags;
  SkewOperand A, Bm, G;
};

BandWs carve_ws(void* ws, int64_t B, const BandDims& d, bool backward) {
  BandWs w;
  float* p = static_cast<float*>(ws);
  auto take = [&](int64_t floats) {
    float* q = p;
    p += pad64(floats);
    return q;
  };
  w.error = reinterpret_cast<int*>(take(64));
  w.ra = take(B * d.n);
  w.rb = take(B * d.n);
  w.flags = reinterpret_cast<int*>(take(B * ceil_div(d.n, 64)));
  w.A.s = make_skew(d.a_lu, d.Wa(), d.n);
  w.Bm.s = make_skew(d.b_lu, d.Wb(), d.n);
  w.G.s = make_skew(d.r_lu(), d.Wo(), d.n);
  w.A.hi = take(skew_floats(w.A.s, B));
  w.A.lo = take(skew_floats(w.A.s, B));
  w.Bm.hi = take(skew_floats(w.Bm.s, B));
  w.Bm.lo = take(skew_floats(w.Bm.s, B));
  w.G.hi = w.G.lo = nullptr;
  if (backward) {
    w.G.hi = take(skew_floats(w.G.s, B));
    w.G.lo = take(skew_floats(w.G.s, B));
  }
  return w;
}

}  // namespace

// declared in band.cuh
bool band_tc_eligible(int mode, const BandDims& d) {
  if (mode != GBMM_BAND_MUL && mode != GBMM_BAND_LOG) return false;
  return d.Wa() >= 32 && d.Wb() >= 32 && d.n >= 128 && d.n < (1LL << 30);
}

int64_t band_tc_workspace_bytes(int backward, int64_t B, const BandDims& d) {
  const Skew sa = make_skew(d.a_lu, d.Wa(), d.n), sb = make_skew(d.b_lu, d.Wb(), d.n),
             sg = make_skew(d.r_lu(), d.Wo(), d.n);
  int64_t floats = 64 + 2 * pad64(B * d.n) + pad64(B * ceil_div(d.n, 64)) + 2 * skew_floats(sa, B) +
                   2 * skew_floats(sb, B);
  if (backward) floats += 2 * skew_floats(sg, B);
  return floats * (int64_t)sizeof(float);
}

// the guard flags of a saved output come from band_block.cu
int band_saved_flags(const float* out, const float* ra, const float* rb, int* flags, int64_t B, int64_t n, int r_lu,
                     int Wo, cudaStream_t st);

// The three products of a banded multiply as BandTcArgs (result band and operand supports; see band_tile).
static BandTcArgs product_args(int which, const BandDims& d) {   // 0 forward, 1 grad_a, 2 grad_b
  BandTcArgs args{};
  const int r_lu = d.r_lu(), r_ld = d.Wo() - 1 - r_lu;
  args.n = (int)d.n;
  if (which == 0) {
    args.lu_out = r_lu; args.w_out = d.Wo();
    args.xl = d.a_lu; args.xu = d.a_ld; args.yl = d.b_lu; args.yu = d.b_ld;
  } else if (which == 1) {
    args.lu_out = d.a_lu; args.w_out = d.Wa();
    args.xl = r_lu; args.xu = r_ld; args.yl = d.b_ld; args.yu = d.b_lu;
  } else {
    args.lu_out = d.b_lu; args.w_out = d.Wb();
    args.xl = r_ld; args.xu = r_lu; args.yl = d.a_ld; args.yu = d.a_lu;
  }
  return args;
}

// The converter-fed kernel takes a banded multiply when every tile of its three products fits one accumulation
// chunk (bands up to about 129 wide at aligned offsets) AND GENBMM_B200_BAND_CV=1 asks for it: it moves a fifth of
// the bytes of the copy-fed kernel but measured slower (the conversion in shared memory, not DRAM, bounds it).
static bool band_cv_fits(const BandDims& d) {
  const char* e = getenv("GENBMM_B200_BAND_CV");
  if (!(e && e[0] == '1')) return false;
  for (int which = 0; which < 3; ++which)
    if (band_max_stages(product_args(which, d)) > TCH) return false;
  return true;
}

// One unsplit copy per operand, split in shared memory by band_sp_kernel (the default), when every tile of the
// three products fits one accumulation chunk; GENBMM_B200_BAND_SPLIT=0 keeps the hi / lo copies of band_tc_kernel,
// which also takes the wider bands.
static bool band_sp_fits(const BandDims& d) {
  const char* e = getenv("GENBMM_B200_BAND_SPLIT");
  if (e && e[0] == '0') return false;
  for (int which = 0; which < 3; ++which)
    if (band_max_stages(product_args(which, d)) > TCH) return false;
  return true;
}

static int band_cv_forward(int mode, const float* a, const float* b, float* out, const BandDims& d, int64_t B,
                    const BandWs& w, int** flags_out, cudaStream_t st) {
  const bool lg = mode == GBMM_BAND_LOG;
  const int64_t rows = B * d.n;
  if (lg) {
    if (cudaMemsetAsync(w.flags, 0, sizeof(int) * B * ceil_div(d.n, 64), st) != cudaSuccess) return GBMM_ERR_LAUNCH;
    band_rowmax_cv_kernel<<<(unsigned)ceil_div(rows, 8), 256, 0, st>>>(a, w.ra, rows, (int)d.n, d.a_lu, d.Wa());
    band_rowmax_cv_kernel<<<(unsigned)ceil_div(rows, 8), 256, 0, st>>>(b, w.rb, rows, (int)d.n, d.b_lu, d.Wb());
    if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
  }
  BandTcArgs args = product_args(0, d);
  args.out = out;
  args.ra = w.ra;
  args.rb = w.rb;
  args.flags = w.flags;
  args.error = w.error;
  *flags_out = lg ? w.flags : nullptr;
  const CvOperand X{a, lg ? w.ra : nullptr, d.Wa(), d.a_lu}, Y{b, lg ? w.rb : nullptr, d.Wb(), d.b_lu};
  const int rc = lg ? launch_band_cv<E_LOG, false, false>(X, Y, args, B, st)
                    : launch_band_cv<E_SUM, false, false>(X, Y, args, B, st);
  if (rc != GBMM_OK) return rc;
  return launch_poison_on_error(w.error, out, B * d.n * d.Wo(), nullptr, 0, st);
}

static int band_cv_backward(int mode, const float* a, const float* b, const float* g, const float* part, float* grad_a,
                     float* grad_b, const BandDims& d, int64_t B, const BandWs& w, int operands_ready,
                     int** flags_out, cudaStream_t st) {
  const bool lg = mode == GBMM_BAND_LOG;
  const int64_t rows = B * d.n;
  const unsigned rblocks = (unsigned)ceil_div(rows, 8);
  const float* gsrc = g;
  int rc = GBMM_OK;
  if (lg) {
    if (!operands_ready) {   // the forward's row maxima and guard flags are not in the workspace: rebuild them
      if (cudaMemsetAsync(w.flags, 0, sizeof(int) * B * ceil_div(d.n, 64), st) != cudaSuccess) return GBMM_ERR_LAUNCH;
      band_rowmax_cv_kernel<<<rblocks, 256, 0, st>>>(a, w.ra, rows, (int)d.n, d.a_lu, d.Wa());
      band_rowmax_cv_kernel<<<rblocks, 256, 0, st>>>(b, w.rb, rows, (int)d.n, d.b_lu, d.Wb());
      if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
      rc = band_saved_flags(part, w.ra, w.rb, w.flags, B, d.n, d.r_lu(), d.Wo(), st);
      if (rc != GBMM_OK) return rc;
    }
    // G' = g exp(ra + rb - out), compact, in the space of the copy-fed kernel's cotangent copies
    float* gp = const_cast<float*>(w.G.hi);
    band_gprime_kernel<<<rblocks, 256, 0, st>>>(part, g, w.ra, w.rb, w.flags, gp, rows, (int)d.n, d.r_lu(), d.Wo());
    if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
    gsrc = gp;
  }
  *flags_out = lg ? w.flags : nullptr;
  const CvOperand G{gsrc, nullptr, d.Wo(), d.r_lu()};
  const CvOperand XA{a, lg ? w.ra : nullptr, d.Wa(), d.a_lu}, XB{b, lg ? w.rb : nullptr, d.Wb(), d.b_lu};
  if (grad_a) {
    // dXa[i,p] = sum_o G[i,o] Xb[o,p]: X = G by rows, Y = Xb by columns
    BandTcArgs args = product_args(1, d);
    args.out = grad_a;
    args.error = w.error;
    rc = launch_band_cv<E_SUM, false, true>(G, XB, args, B, st);
    if (rc != GBMM_OK) return rc;
    if (lg) {  // log: dXa = EA (.) sum
      band_scale_kernel<<<rblocks, 256, 0, st>>>(grad_a, a, w.ra, rows, (int)d.n, d.a_lu, d.Wa());
      if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
    }
  }
  if (grad_b) {
    // dXb[o,p] = sum_i G[i,o] Xa[i,p]: both by columns
    BandTcArgs args = product_args(2, d);
    args.out = grad_b;
    args.error = w.error;
    rc = launch_band_cv<E_SUM, true, true>(G, XA, args, B, st);
    if (rc != GBMM_OK) return rc;
    if (lg) {
      band_scale_kernel<<<rblocks, 256, 0, st>>>(grad_b, b, w.rb, rows, (int)d.n, d.b_lu, d.Wb());
      if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
    }
  }
  return launch_poison_on_error(w.error, grad_a, B * d.n * d.Wa(), grad_b, B * d.n * d.Wb(), st);
}

int band_tc_forward(int mode, const float* a, const float* b, float* out, const BandDims& d, int64_t B, void* ws,
                    int** flags_out, cudaStream_t st) {
  const BandWs w = carve_ws(ws, B, d, false);
  const bool lg = mode == GBMM_BAND_LOG;
  if (cudaMemsetAsync(w.error, 0, sizeof(int), st) != cudaSuccess) return GBMM_ERR_LAUNCH;
  if (band_cv_fits(d)) return band_cv_forward(mode, a, b, out, d, B, w, flags_out, st);
  const bool sp = band_sp_fits(d);   // one unsplit copy per operand (lo pointer null), split in shared memory
  float* a_lo = sp ? nullptr : const_cast<float*>(w.A.lo);
  float* b_lo = sp ? nullptr : const_cast<float*>(w.Bm.lo);
  int rc = GBMM_OK;
  if (lg) {
    if (cudaMemsetAsync(w.flags, 0, sizeof(int) * B * ceil_div(d.n, 64), st) != cudaSuccess) return GBMM_ERR_LAUNCH;
    // the row maxima come out of the same pass that exponentiates (and splits) the operands
    rc = launch_skew<1>(a, nullptr, nullptr, nullptr, nullptr, w.ra, const_cast<float*>(w.A.hi), a_lo, B, d.n,
                        d.a_lu, d.Wa(), w.A.s, st);
    if (rc != GBMM_OK) return rc;
    rc = launch_skew<1>(b, nullptr, nullptr, nullptr, nullptr, w.rb, const_cast<float*>(w.Bm.hi), b_lo, B, d.n,
                        d.b_lu, d.Wb(), w.Bm.s, st);
  } else {
    rc = launch_skew<0>(a, nullptr, nullptr, nullptr, nullptr, nullptr, const_cast<float*>(w.A.hi), a_lo, B, d.n,
                        d.a_lu, d.Wa(), w.A.s, st);
    if (rc != GBMM_OK) return rc;
    rc = launch_skew<0>(b, nullptr, nullptr, nullptr, nullptr, nullptr, const_cast<float*>(w.Bm.hi), b_lo, B, d.n,
                        d.b_lu, d.Wb(), w.Bm.s, st);
  }
  if (rc != GBMM_OK) return rc;
  // out[i,o] = sum_p Xa[i,p] Xb[o,p]: both operands K-major
  BandTcArgs args{};
  args.n = (int)d.n;
  args.lu_out = d.r_lu();
  args.w_out = d.Wo();
  args.xl = d.a_lu; args.xu = d.a_ld; args.yl = d.b_lu; args.yu = d.b_ld;
  args.out = out;
  args.ra = w.ra;
  args.rb = w.rb;
  args.flags = w.flags;
  args.error = w.error;
  *flags_out = lg ? w.flags : nullptr;
  if (sp)
    rc = lg ? launch_band_sp<E_LOG, false, false>(w.A, w.Bm, args, B, st)
            : launch_band_sp<E_SUM, false, false>(w.A, w.Bm, args, B, st);
  else
    rc = lg ? launch_band_tc<E_LOG, false, false>(w.A, w.Bm, args, B, st)
            : launch_band_tc<E_SUM, false, false>(w.A, w.Bm, args, B, st);
  if (rc != GBMM_OK) return rc;
  // a product kernel that gave up on a bounded wait set the error word: the result becomes NaN
  return launch_poison_on_error(w.error, out, B * d.n * d.Wo(), nullptr, 0, st);
}

// GENBMM_B200_BAND_SCALE=fused applies the log gradients' factor in band_sp_kernel's epilogue instead of a pass of
// its own.  Measured at 32 x 8192 x 129 diagonals: backward 1.30 ms against 1.20 ms with the pass (2.10 ms while
// the epilogue's loads went out four at a time): the loads still wait behind the SM's TMA traffic, and the tile's
// accumulators are held for as long.
static bool band_fused_scale() {
  const char* e = getenv("GENBMM_B200_BAND_SCALE");
  return e && e[0] == 'f';
}

int band_tc_backward(int mode, const float* a, const float* b, const float* g, const float* part, float* grad_a,
                     float* grad_b, const BandDims& d, int64_t B, void* ws, int operands_ready, int** flags_out,
                     cudaStream_t st) {
  const BandWs w = carve_ws(ws, B, d, true);
  const bool lg = mode == GBMM_BAND_LOG;
  if (cudaMemsetAsync(w.error, 0, sizeof(int), st) != cudaSuccess) return GBMM_ERR_LAUNCH;
  if (band_cv_fits(d))
    return band_cv_backward(mode, a, b, g, part, grad_a, grad_b, d, B, w, operands_ready, flags_out, st);
  int rc = GBMM_OK;
  const bool sp = band_sp_fits(d);   // unsplit copies (lo pointers null), split in shared memory
  float *ah = const_cast<float*>(w.A.hi), *al = sp ? nullptr : const_cast<float*>(w.A.lo),
        *bh = const_cast<float*>(w.Bm.hi), *bl = sp ? nullptr : const_cast<float*>(w.Bm.lo),
        *gh = const_cast<float*>(w.G.hi), *gl = sp ? nullptr : const_cast<float*>(w.G.lo);
  if (lg) {
    if (!operands_ready) {
      if (cudaMemsetAsync(w.flags, 0, sizeof(int) * B * ceil_div(d.n, 64), st) != cudaSuccess) return GBMM_ERR_LAUNCH;
      // both row maxima are needed whichever gradient is asked for (G' uses ra and rb)
      rc = launch_skew<1>(a, nullptr, nullptr, nullptr, nullptr, w.ra, ah, al, B, d.n, d.a_lu, d.Wa(), w.A.s, st);
      if (rc != GBMM_OK) return rc;
      rc = launch_skew<1>(b, nullptr, nullptr, nullptr, nullptr, w.rb, bh, bl, B, d.n, d.b_lu, d.Wb(), w.Bm.s, st);
      if (rc != GBMM_OK) return rc;
      rc = band_saved_flags(part, w.ra, w.rb, w.flags, B, d.n, d.r_lu(), d.Wo(), st);
      if (rc != GBMM_OK) return rc;
    }
    rc = launch_skew<2>(part, g, w.ra, w.rb, w.flags, nullptr, gh, gl, B, d.n, d.r_lu(), d.Wo(), w.G.s, st);
  } else {
    if (grad_b && !operands_ready)
      rc = launch_skew<0>(a, nullptr, nullptr, nullptr, nullptr, nullptr, ah, al, B, d.n, d.a_lu, d.Wa(), w.A.s, st);
    if (rc != GBMM_OK) return rc;
    if (grad_a && !operands_ready)
      rc = launch_skew<0>(b, nullptr, nullptr, nullptr, nullptr, nullptr, bh, bl, B, d.n, d.b_lu, d.Wb(), w.Bm.s, st);
    if (rc != GBMM_OK) return rc;
    rc = launch_skew<0>(g, nullptr, nullptr, nullptr, nullptr, nullptr, gh, gl, B, d.n, d.r_lu(), d.Wo(), w.G.s, st);
  }
  if (rc != GBMM_OK) return rc;
  *flags_out = lg ? w.flags : nullptr;
  const int r_lu = d.r_lu(), r_ld = d.Wo() - 1 - r_lu;
  if (grad_a) {
    // dXa[i,p] = sum_o G[i,o] Xb[o,p]: X = G K-major (o contiguous), Y = Xb MN-major (p contiguous)
    BandTcArgs args{};
    args.n = (int)d.n;
    args.lu_out = d.a_lu;
    args.w_out = d.Wa();
    args.xl = r_lu; args.xu = r_ld; args.yl = d.b_ld; args.yu = d.b_lu;
    args.out = grad_a;
    args.error = w.error;
    const bool fused_scale = lg && sp && band_fused_scale();
    if (fused_scale) {   // log: dXa = EA (.) sum, the factor applied by the product's epilogue
      args.ra = w.ra;
      args.src = a;
    }
    rc = fused_scale ? launch_band_sp<E_GRADLOG, false, true>(w.G, w.Bm, args, B, st)
         : sp        ? launch_band_sp<E_SUM, false, true>(w.G, w.Bm, args, B, st)
                     : launch_band_tc<E_SUM, false, true>(w.G, w.Bm, args, B, st);
    if (rc != GBMM_OK) return rc;
    if (lg && !fused_scale) {  // log: dXa = EA (.) sum
      band_scale_kernel<<<(unsigned)ceil_div(B * d.n, 8), 256, 0, st>>>(grad_a, a, w.ra, B * d.n, (int)d.n, d.a_lu,
                                                                      d.Wa());
      if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
    }
  }
  if (grad_b) {
    // dXb[o,p] = sum_i G[i,o] Xa[i,p]: X = G MN-major (o contiguous), Y = Xa MN-major (p contiguous)
    BandTcArgs args{};
    args.n = (int)d.n;
    args.lu_out = d.b_lu;
    args.w_out = d.Wb();
    args.xl = r_ld; args.xu = r_lu; args.yl = d.a_ld; args.yu = d.a_lu;
    args.out = grad_b;
    args.error = w.error;
    const bool fused_scale = lg && sp && band_fused_scale();
    if (fused_scale) {
      args.ra = w.rb;
      args.src = b;
    }
    rc = fused_scale ? launch_band_sp<E_GRADLOG, true, true>(w.G, w.A, args, B, st)
         : sp        ? launch_band_sp<E_SUM, true, true>(w.G, w.A, args, B, st)
                     : launch_band_tc<E_SUM, true, true>(w.G, w.A, args, B, st);
    if (rc != GBMM_OK) return rc;
    if (lg && !fused_scale) {
      band_scale_kernel<<<(unsigned)ceil_div(B * d.n, 8), 256, 0, st>>>(grad_b, b, w.rb, B * d.n, (int)d.n, d.b_lu,
                                                                      d.Wb());
      rc = launch_status();
      if (rc != GBMM_OK) return rc;
    }
  }
  // a product kernel that gave up on a bounded wait set the error word: both gradients become NaN
  return launch_poison_on_error(w.error, grad_a, B * d.n * d.Wa(), grad_b, B * d.n * d.Wb(), st);
}

}  // namespace gbmm
