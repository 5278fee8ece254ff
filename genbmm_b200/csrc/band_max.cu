// Banded max-plus forward (multiply_max) for bands at least 32 wide: the dense max kernel's inner loop
// (dense_fwd.cu) fed from skewed copies of the band tensors.
//
// As in band_tc.cu, X[r,c] = data[r][c-r+lu] is a strided view of band storage once every row is followed
// by enough padding: rows pitch-1 apart, columns contiguous.  Here the padding (and every out-of-matrix
// cell) holds -inf, so a term that involves a cell outside either band is -inf and never exceeds the
// running maximum, which starts at -1e9 like the reference's (banded_cuda_kernel.cu:45-60).
// A CTA owns a 128 x 64 block of the result that meets the result band and walks the reduction index over
// the range where both operand bands are populated, 16 steps at a time: (k, k+1) pairs side by side in
// shared memory, one packed add and one 3-input max per two terms, two alternating sets of running maxima,
// the first 16-step tile that reached the maximum remembered in a byte.  A block's reduction range is short
// (at most 63 + Wb or 127 + Wa steps), so all of it is loaded into shared memory up front (one CTA per SM,
// up to 218 KB); the winning tile of each result is then searched there for the first p whose term equals
// the maximum, with no second trip to global memory.  Ascending p is ascending index in a's band for a fixed
// row, so this is the reference's lowest-index tie rule; the stored index is p - i + a_lu.
#include <cstdlib>
#include <type_traits>
#include <algorithm>

#include "band.cuh"
#include "tile.cuh"
#include "tma.cuh"

namespace gbmm {
namespace {

constexpr int BM = 128, BN = 64, BK = 16, NT = 256;
constexpr int LDX = BM + 4, LDY = BN + 4;
constexpr int MAX_PAD = 192;  // >= 127 (tile rows) + 2 * 15 (reduction range rounded to tiles of 16)

__device__ __forceinline__ float nan_f() { return __int_as_float(0x7fc00000); }
__device__ __forceinline__ float ninf_f() { return __int_as_float(0xff800000); }
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

struct MaxSkew {
  int off, pitch, kofs;
  int64_t bstride;
};
MaxSkew make_max_skew(int lu, int W, int64_t n) {
  MaxSkew s;
  s.off = (4 - lu % 4) % 4;  // 128-bit loads along the reduction index: lu + off a multiple of 4
  s.pitch = s.off + W + MAX_PAD;
  s.pitch += (1 - s.pitch % 4 + 4) % 4;
  s.kofs = lu + s.off;
  s.bstride = (n * s.pitch + 3) & ~int64_t(3);
  return s;
}
int64_t max_skew_floats(const MaxSkew& s, int64_t B) { return (B * s.bstride + 64 + 63) & ~int64_t(63); }

// band rows into the skewed layout; cells outside the matrix become -inf (one warp per row)
__global__ void __launch_bounds__(256) band_max_skew_kernel(const float* __restrict__ x, float* __restrict__ dst,
                                                            int64_t rows, int n, int lu, int W, int off, int pitch,
                                                            int64_t bstride) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;
  if (row >= rows) return;
  const int i = (int)(row % n);
  const int64_t bt = row / n;
  const int jlo = max(0, lu - i), jhi = min(W, n - i + lu);
  float* dr = dst + bt * bstride + (int64_t)i * pitch + off;
  for (int j = lane; j < W; j += 32) dr[j] = (j >= jlo && j < jhi) ? __ldg(x + row * W + j) : ninf_f();
}

__global__ void fill_ninf_kernel(float* p, int64_t count) {
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (int64_t)gridDim.x * blockDim.x)
    p[e] = ninf_f();
}

struct MaxArgs {
  const float* xs;  // skewed a
  const float* ys;  // skewed b
  int64_t x_bstride, y_bstride;
  int x_rstride, y_rstride;  // pitch - 1
  int x_kofs, y_kofs;
  int n, a_lu, a_ld, b_lu, b_ld, r_lu, Wo;
  int nrb, ncb;
  float* out;
  int* idx;
  int x_ninf, y_ninf;  // offset (from a batch element's base) of 16 bytes of -inf padding
  int* error;          // set when a bounded wait ran out (band_max_w_kernel)
};

// Dynamic shared memory: the operand tiles of the block's whole reduction range (at most kMaxSteps tiles of
// 16 steps), pair layout: x element (k, m) at ((k/2) * LDX + m) * 2 + (k & 1), y likewise with LDY.
// Tiles are 4 floats further apart than their size: results of one warp search different tiles, and with a
// stride that is a multiple of 32 banks all those reads would hit the same bank.
constexpr int XS = (BK / 2) * LDX * 2 + 4, YS = (BK / 2) * LDY * 2 + 4;  // floats per x / y tile
constexpr int kMaxSteps = 17;  // 272 reduction steps: 17 * (XS + YS) * 4 bytes = 213 KB
__host__ __device__ constexpr size_t max_smem_bytes(int steps) { return (size_t)steps * (XS + YS) * sizeof(float); }

template <bool SKIP>
__global__ void __launch_bounds__(NT, 1) band_max_kernel(MaxArgs g) {
  extern __shared__ __align__(16) float smem_dyn[];
  const Micro8x4 mt;
  const int tid = threadIdx.x, lane = tid & 31;
  const int64_t id = blockIdx.x;
  const int cbi = (int)(id % g.ncb), rbk = (int)((id / g.ncb) % g.nrb);
  const int64_t bt = id / ((int64_t)g.ncb * g.nrb);
  const int r0 = rbk * BM;
  const int lo = r0 - g.r_lu;
  const int cfirst = lo >= 0 ? lo / BN : -((-lo + BN - 1) / BN);
  const int c0 = (cfirst + cbi) * BN;
  const int r_ld = g.Wo - 1 - g.r_lu;
  if (c0 > r0 + BM - 1 + r_ld) return;  // beyond the band: owns no cell
  const int s_lo = max(max(r0 - g.a_lu, c0 - g.b_lu), 0);
  int s_hi = min(min(r0 + BM - 1 + g.a_ld, c0 + BN - 1 + g.b_ld), g.n - 1);
  if (c0 >= g.n || c0 + BN - 1 < 0) s_hi = s_lo - 1;  // outside the matrix: only zeros to write
  const int s0 = s_lo & ~(BK - 1);
  const int nt = s_hi >= s_lo ? (s_hi - s0) / BK + 1 : 0;  // <= kMaxSteps by the eligibility rule
  float* sx = smem_dyn;
  float* sy = smem_dyn + (size_t)nt * XS;

  const float* xb = g.xs + bt * g.x_bstride + g.x_kofs;
  const float* yb = g.ys + bt * g.y_bstride + g.y_kofs;

  // Tile loads: 4 consecutive reduction indices per 128-bit load (always aligned: row stride, kofs and the
  // reduction start are multiples of 4); rows outside the matrix give NaN terms, which the maximum ignores.
  // Tile t + 1 is fetched into registers while tile t is multiplied and stored behind it; every tile stays
  // in shared memory for the index search at the end.
  float4 xa[2], ya;
  auto fetch = [&](int t) {
    const int s = s0 + t * BK;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int f = tid + q * NT, o = f / (BK / 4), r = (f % (BK / 4)) * 4;
      const int i = r0 + o;
      xa[q] = (i < g.n) ? __ldg(reinterpret_cast<const float4*>(xb + (int64_t)i * g.x_rstride + s + r))
                        : make_float4(nan_f(), nan_f(), nan_f(), nan_f());
    }
    const int o = tid / (BK / 4), r = (tid % (BK / 4)) * 4;
    const int c = c0 + o;
    ya = (c >= 0 && c < g.n) ? __ldg(reinterpret_cast<const float4*>(yb + (int64_t)c * g.y_rstride + s + r))
                             : make_float4(nan_f(), nan_f(), nan_f(), nan_f());
  };
  auto stage = [&](int t) {
    float* dx = sx + (size_t)t * XS;
    float* dy = sy + (size_t)t * YS;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int f = tid + q * NT, o = f / (BK / 4), r = (f % (BK / 4)) * 4;
      *reinterpret_cast<float2*>(dx + ((r / 2) * LDX + o) * 2) = make_float2(xa[q].x, xa[q].y);
      *reinterpret_cast<float2*>(dx + ((r / 2 + 1) * LDX + o) * 2) = make_float2(xa[q].z, xa[q].w);
    }
    const int o = tid / (BK / 4), r = (tid % (BK / 4)) * 4;
    *reinterpret_cast<float2*>(dy + ((r / 2) * LDY + o) * 2) = make_float2(ya.x, ya.y);
    *reinterpret_cast<float2*>(dy + ((r / 2 + 1) * LDY + o) * 2) = make_float2(ya.z, ya.w);
  };
  if (nt > 0) {
    fetch(0);
    stage(0);
  }
  __syncthreads();

  float X[8][4], Y[8][4];
  unsigned cidp[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    cidp[i] = 0xffffffffu;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      X[i][j] = kFloor;
      Y[i][j] = kFloor;
    }
  }

  // A warp owns rows 8w..8w+7 and 64+8w..64+8w+7 of the block.  Row r meets reduction steps r - a_lu .. r + a_ld
  // only, so for a 16-step tile near either end of the block's range one or both of the warp's row groups
  // hold nothing but -inf terms; with SKIP those halves of the micro-tile are carried over instead of
  // multiplied.  The barrier per tile still waits for the warps that are live in it, so the gain is what the
  // idle warps leave to the pipes: 6 % at 129 x 129 diagonals; where the range is short next to a's band no
  // warp is ever idle and the launcher takes the plain kernel.
  const int rw = r0 + (tid >> 5) * 8;
  auto half_live = [&](int t, int first_row) {
    const int s = s0 + t * BK;
    return s <= first_row + 7 + g.a_ld && s + BK - 1 >= first_row - g.a_lu;
  };
  auto tile_body = [&](auto UP, auto LOW, int t, float (&acc)[8][4], const float (&prev)[8][4]) {
    constexpr bool kUp = decltype(UP)::value, kLow = decltype(LOW)::value;
    const float* tx_ = sx + (size_t)t * XS;
    const float* ty_ = sy + (size_t)t * YS;
    if (!kUp) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = prev[i][j];
    }
    if (!kLow) {
#pragma unroll
      for (int i = 4; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = prev[i][j];
    }
    if (kUp || kLow) {
#pragma unroll
      for (int kp2 = 0; kp2 < BK / 2; ++kp2) {
        const float* xs = tx_ + (kp2 * LDX + mt.ty * 4) * 2;
        const float* ys = ty_ + (kp2 * LDY + mt.tx * 4) * 2;
        const ulonglong2 y01 = *reinterpret_cast<const ulonglong2*>(ys);
        const ulonglong2 y23 = *reinterpret_cast<const ulonglong2*>(ys + 4);
        const unsigned long long yp[4] = {y01.x, y01.y, y23.x, y23.y};
        unsigned long long xp[8];
        if (kUp) {
          const ulonglong2 x01 = *reinterpret_cast<const ulonglong2*>(xs);
          const ulonglong2 x23 = *reinterpret_cast<const ulonglong2*>(xs + 4);
          xp[0] = x01.x; xp[1] = x01.y; xp[2] = x23.x; xp[3] = x23.y;
        }
        if (kLow) {
          const ulonglong2 x45 = *reinterpret_cast<const ulonglong2*>(xs + 128);
          const ulonglong2 x67 = *reinterpret_cast<const ulonglong2*>(xs + 132);
          xp[4] = x45.x; xp[5] = x45.y; xp[6] = x67.x; xp[7] = x67.y;
        }
#pragma unroll
        for (int i = kUp ? 0 : 4; i < (kLow ? 8 : 4); ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float v0, v1;
            unpack2(add2(xp[i], yp[j]), v0, v1);
            acc[i][j] = max3(kp2 == 0 ? prev[i][j] : acc[i][j], v0, v1);
          }
      }
#pragma unroll
      for (int i = kUp ? 0 : 4; i < (kLow ? 8 : 4); ++i) {  // strict `>`: an equal maximum in a later tile keeps the index
        if (acc[i][0] > prev[i][0]) cidp[i] = __byte_perm(cidp[i], (unsigned)t, 0x3214);
        if (acc[i][1] > prev[i][1]) cidp[i] = __byte_perm(cidp[i], (unsigned)t, 0x3240);
        if (acc[i][2] > prev[i][2]) cidp[i] = __byte_perm(cidp[i], (unsigned)t, 0x3410);
        if (acc[i][3] > prev[i][3]) cidp[i] = __byte_perm(cidp[i], (unsigned)t, 0x4210);
      }
    }
  };
  auto tile_step = [&](int t, float (&acc)[8][4], const float (&prev)[8][4]) {
    if (t + 1 < nt) fetch(t + 1);
    const bool up = !SKIP || half_live(t, rw), low = !SKIP || half_live(t, rw + 64);
    using T = std::true_type;
    using F = std::false_type;
    if (up && low) tile_body(T{}, T{}, t, acc, prev);
    else if (up) tile_body(T{}, F{}, t, acc, prev);
    else if (low) tile_body(F{}, T{}, t, acc, prev);
    else tile_body(F{}, F{}, t, acc, prev);
    if (t + 1 < nt) stage(t + 1);
    __syncthreads();
  };
  int t = 0;
  for (; t + 1 < nt; t += 2) {
    tile_step(t, X, Y);
    tile_step(t + 1, Y, X);
  }
  if (t < nt) {
    tile_step(t, X, Y);
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) Y[i][j] = X[i][j];
  }
  // from here on Y holds the maxima.  The winning tile of every result is still in shared memory: search it
  // from the last step down, so the lowest matching p is the assignment that sticks; the stored value is that
  // term itself (a zero keeps the sign the reference would keep).
  float* ob = g.out + bt * g.n * (int64_t)g.Wo;
  int* ib = g.idx + bt * g.n * (int64_t)g.Wo;
  (void)lane;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int ml = mt.row(i), m = r0 + ml;
    if (m >= g.n) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int cl = mt.col(j), c = c0 + cl;
      const int cell = c - m + g.r_lu;
      if (cell < 0 || cell >= g.Wo) continue;
      const bool inside = c >= 0 && c < g.n;
      const unsigned c8 = (cidp[i] >> (8 * j)) & 0xffu;
      float val = Y[i][j];
      int p = -1;
      if (inside && c8 != 0xffu) {
        const float* tx_ = sx + (size_t)c8 * XS + ml * 2;
        const float* ty_ = sy + (size_t)c8 * YS + cl * 2;
#pragma unroll
        for (int kp2 = BK / 2 - 1; kp2 >= 0; --kp2) {
          float v0, v1;
          unpack2(add2(*reinterpret_cast<const unsigned long long*>(tx_ + kp2 * LDX * 2),
                       *reinterpret_cast<const unsigned long long*>(ty_ + kp2 * LDY * 2)),
                  v0, v1);
          if (v1 == Y[i][j]) p = 2 * kp2 + 1;
          if (v0 == Y[i][j]) p = 2 * kp2;
        }
        // the stored value is the matching term itself: only for a zero can it differ from the maximum
        // (in sign), so that is the one case that reads the term again
        if (val == 0.f && p >= 0) {
          const float2 xv = *reinterpret_cast<const float2*>(tx_ + (p / 2) * LDX * 2);
          const float2 yv = *reinterpret_cast<const float2*>(ty_ + (p / 2) * LDY * 2);
          val = (p & 1) ? __fadd_rn(xv.y, yv.y) : __fadd_rn(xv.x, yv.x);
        }
        if (p >= 0) p += s0 + (int)c8 * BK;
      }
      const int64_t e = (int64_t)m * g.Wo + cell;
      ob[e] = inside ? val : 0.f;  // cells outside the matrix stay zero (banded_cuda_kernel.cu:38)
      ib[e] = inside ? (p >= 0 ? p - m + g.a_lu : -1) : 0;
    }
  }
}


// ---- 64 x 64 blocks, one 16 x 32 sub-block per warp, each warp on its own reduction range ----
//
// A term (i, o, p) is a band term only for |p - i| and |p - o| within the bands, so the smaller the sub-block
// that shares one reduction range, the fewer padded terms it executes: 128 x 64 blocks in lockstep execute 49 000
// terms per row of the result at 129 x 129 diagonals for 16 600 band terms; 16 x 32 sub-blocks, each walking only
// the 16-step tiles that meet both of ITS bands, execute 28 000.  For that the warps of a CTA must not wait for
// one another per tile: every thread requests all tiles of the block's range at once with 16-byte cp.async
// copies and makes one deferred arrival per tile on that tile's mbarrier, and a warp waits only for the tiles it
// reads.  At most 107 KB of tiles at 129 diagonals: two CTAs per SM, so one CTA's copies land while the other
// multiplies.  Measured at 32 x 8192 x 129 diagonals: 1.33 ms against 1.78 ms for the lockstep kernel.  With
// 8 x 4 results per thread (4 warps per CTA, 8 per SM) the same scheme took 1.76 ms: too few warps to cover the
// shared-memory and pipe latencies; with 4 x 4 the CTA has 8 warps, and with 4 x 2 on 64 x 32 blocks three CTAs
// fit an SM (24 warps): 1.23 ms.
//
// Shared-memory layout of a 16-step tile: [quad of steps][row][4 steps], one 128-bit load per row and quad; a
// thread's rows are ty + 4 i and its columns tx + 8 j, so the lanes of a warp read consecutive 16-byte cells
// (no bank conflicts), and the two halves of a loaded quad are the (k, k+1) pairs of the packed add.
constexpr int WB = 64;               // rows of a block
constexpr int WT = 4 * WB * 4 + 4;   // floats per tile of a; + 4: the search reads the same cell of different tiles
constexpr int kMaxTilesW = 26;       // 26 tiles of a and b at 64 columns = 214 KB
__host__ __device__ constexpr int w_tile_y(int wc) { return 4 * wc * 4 + 4; }  // floats per tile of b, wc columns
__host__ __device__ constexpr size_t w_smem_bytes(int tiles, int wc) {
  return (size_t)tiles * (WT + w_tile_y(wc)) * sizeof(float);
}

__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
// one arrival on `bar` once every cp.async this thread has issued so far has landed (counted in the barrier's
// initial count: .noinc)
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// IR x JC results per thread: rows ty + 4 i, columns tx + 8 j; a warp's sub-block is 4 IR rows x 8 JC columns, a
// block 64 rows x 16 JC columns (two warps across).  8 x 4: 4 warps of 32 x 32; 4 x 4: 8 warps of 16 x 32;
// 4 x 2: 64 x 32 blocks, 8 warps of 16 x 16 (less shared memory and fewer registers: three CTAs per SM).
template <int IR, int JC, int UQ>
__global__ void __launch_bounds__(1024 / IR, JC == 2 ? 3 : 2) band_max_w_kernel(MaxArgs g) {
  constexpr int WNT = 1024 / IR, WROWS = 4 * IR, WCOLS = 8 * JC, WC = 2 * WCOLS, WTY = w_tile_y(WC);
  static_assert(WNT == 256 || JC == 4, "the staging below gives every thread at most one chunk of b per tile");
  extern __shared__ __align__(16) float smem_dyn[];
  __shared__ __align__(8) uint64_t landed[kMaxTilesW];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ty = lane >> 3, tx = lane & 7;
  const int64_t id = blockIdx.x;
  const int cbi = (int)(id % g.ncb), rbk = (int)((id / g.ncb) % g.nrb);
  const int64_t bt = id / ((int64_t)g.ncb * g.nrb);
  const int r0 = rbk * WB;
  const int lo = r0 - g.r_lu;
  const int cfirst = lo >= 0 ? lo / WC : -((-lo + WC - 1) / WC);
  const int c0 = (cfirst + cbi) * WC;
  const int r_ld = g.Wo - 1 - g.r_lu;
  if (c0 > r0 + WB - 1 + r_ld) return;  // beyond the band: owns no cell
  const int s_lo = max(max(r0 - g.a_lu, c0 - g.b_lu), 0);
  int s_hi = min(min(r0 + WB - 1 + g.a_ld, c0 + WC - 1 + g.b_ld), g.n - 1);
  if (c0 >= g.n || c0 + WC - 1 < 0) s_hi = s_lo - 1;  // outside the matrix: only zeros to write
  const int s0 = s_lo & ~(BK - 1);
  const int nt = s_hi >= s_lo ? (s_hi - s0) / BK + 1 : 0;  // <= the launch's tile count by the eligibility rule
  float* sx = smem_dyn;
  float* sy = smem_dyn + (size_t)nt * WT;

  if (tid == 0) {
    for (int t = 0; t < nt; ++t) mbar_init(&landed[t], WNT);
    fence_barrier_init();
  }
  __syncthreads();

  // Requests, in tile order.  A tile of a is 256 chunks of 16 bytes (64 rows x 4 quads), a tile of b 4 WC; 8 lanes
  // take the same quad of 8 consecutive rows: 128 contiguous bytes of shared memory per quarter warp, 64
  // contiguous bytes of a row per four quads.  Rows and columns outside the matrix read 16 bytes of -inf padding.
  {
    const float* xbase = g.xs + bt * g.x_bstride;
    const float* ybase = g.ys + bt * g.y_bstride;
    constexpr int NQ = 256 / WNT;
    const float* xsrc[NQ];
    const float* ysrc[NQ];
    int xofs[NQ], yofs[NQ];
    bool yown[NQ];
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
      const int f = tid + q * WNT, row = (f >> 5) * 8 + (f & 7), quad = (f >> 3) & 3;
      const int i = r0 + row, c = c0 + row;
      xofs[q] = (quad * WB + row) * 4;
      yofs[q] = (quad * WC + row) * 4;
      yown[q] = row < WC;
      xsrc[q] = i < g.n ? xbase + g.x_kofs + (int64_t)i * g.x_rstride + s0 + 4 * quad : nullptr;
      ysrc[q] = (c >= 0 && c < g.n) ? ybase + g.y_kofs + (int64_t)c * g.y_rstride + s0 + 4 * quad : nullptr;
    }
    for (int t = 0; t < nt; ++t) {
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        cp_async16(sx + (size_t)t * WT + xofs[q], xsrc[q] ? xsrc[q] + t * BK : xbase + g.x_ninf);
        if (yown[q]) cp_async16(sy + (size_t)t * WTY + yofs[q], ysrc[q] ? ysrc[q] + t * BK : ybase + g.y_ninf);
      }
      cp_async_arrive(&landed[t]);
    }
  }

  // this warp's sub-block and the tiles that meet both of its bands
  const int rl0 = (warp >> 1) * WROWS, cl0 = (warp & 1) * WCOLS;
  const int w_lo = max(max(r0 + rl0 - g.a_lu, c0 + cl0 - g.b_lu), s_lo);
  const int w_hi = min(min(r0 + rl0 + WROWS - 1 + g.a_ld, c0 + cl0 + WCOLS - 1 + g.b_ld), s_hi);
  const int t_lo = w_hi >= w_lo ? (w_lo - s0) / BK : 0;
  const int t_hi = w_hi >= w_lo ? (w_hi - s0) / BK : -1;

  // The warps of a CTA are at different tiles at any moment and two CTAs share the SM, so the code must stay
  // small enough for the instruction cache: one copy of the tile body (the maxima before the tile are copied
  // aside for the "did this tile raise it" test instead of alternating two register sets) and a rolled search
  // loop (with 8 x 4 results per thread, everything unrolled and two alternating sets, the schedulers sat
  // without instructions five cycles for every one they issued).
  float Y[IR][JC];
  unsigned cidp[IR];
#pragma unroll
  for (int i = 0; i < IR; ++i) {
    cidp[i] = 0xffffffffu;
#pragma unroll
    for (int j = 0; j < JC; ++j) Y[i][j] = kFloor;
  }
  bool fail = false;
#pragma unroll 1
  for (int t = t_lo; t <= t_hi; ++t) {
    if (!mbar_wait_bounded(&landed[t], 0)) fail = true;
    const float* xt = sx + (size_t)t * WT + (rl0 + ty) * 4;
    const float* yt = sy + (size_t)t * WTY + (cl0 + tx) * 4;
    float P[IR][JC];
#pragma unroll
    for (int i = 0; i < IR; ++i)
#pragma unroll
      for (int j = 0; j < JC; ++j) P[i][j] = Y[i][j];
    auto quad = [&](int q) {
      ulonglong2 xq[IR], yq[JC];
#pragma unroll
      for (int i = 0; i < IR; ++i) xq[i] = *reinterpret_cast<const ulonglong2*>(xt + (q * WB + 4 * i) * 4);
#pragma unroll
      for (int j = 0; j < JC; ++j) yq[j] = *reinterpret_cast<const ulonglong2*>(yt + (q * WC + 8 * j) * 4);
#pragma unroll
      for (int i = 0; i < IR; ++i)
#pragma unroll
        for (int j = 0; j < JC; ++j) {
          float v0, v1, v2, v3;
          unpack2(add2(xq[i].x, yq[j].x), v0, v1);
          unpack2(add2(xq[i].y, yq[j].y), v2, v3);
          Y[i][j] = max3(max3(Y[i][j], v0, v1), v2, v3);
        }
    };
    if (t > t_lo && t < t_hi) {
#pragma unroll UQ
      for (int q = 0; q < BK / 4; ++q) quad(q);
    } else {  // the first and the last tile of the warp's range: only the quads that meet it
      const int qa = t == t_lo ? ((w_lo - s0) & (BK - 1)) >> 2 : 0;
      const int qb = t == t_hi ? ((w_hi - s0) & (BK - 1)) >> 2 : BK / 4 - 1;
#pragma unroll 1
      for (int q = qa; q <= qb; ++q) quad(q);
    }
#pragma unroll
    for (int i = 0; i < IR; ++i) {  // strict `>`: an equal maximum in a later tile keeps the index
      if (Y[i][0] > P[i][0]) cidp[i] = __byte_perm(cidp[i], (unsigned)t, 0x3214);
      if (Y[i][1] > P[i][1]) cidp[i] = __byte_perm(cidp[i], (unsigned)t, 0x3240);
      if (JC > 2) {
        if (Y[i][JC - 2] > P[i][JC - 2]) cidp[i] = __byte_perm(cidp[i], (unsigned)t, 0x3410);
        if (Y[i][JC - 1] > P[i][JC - 1]) cidp[i] = __byte_perm(cidp[i], (unsigned)t, 0x4210);
      }
    }
  }
  if (__any_sync(0xffffffffu, fail) && lane == 0) atomicExch(g.error, 1);

  // Y holds the maxima; the winning tile of every result is still in shared memory: search it from the last
  // step down, so the lowest matching p is the assignment that sticks; the stored value is that term itself.
  float* ob = g.out + bt * g.n * (int64_t)g.Wo;
  int* ib = g.idx + bt * g.n * (int64_t)g.Wo;
  // The four results of a row are searched side by side (one rolled loop over the quads, eight independent
  // loads in flight): one result at a time, the loop ran at the latency of a shared-memory load per quad.
#pragma unroll
  for (int i = 0; i < IR; ++i) {
    const int ml = rl0 + ty + 4 * i, m = r0 + ml;
    if (m >= g.n) continue;
    const float* xt[JC];
    const float* yt[JC];
    int p[JC], cell[JC];
    bool hunt[JC], inside[JC];
#pragma unroll
    for (int j = 0; j < JC; ++j) {
      const int cl = cl0 + tx + 8 * j, c = c0 + cl;
      cell[j] = c - m + g.r_lu;
      inside[j] = c >= 0 && c < g.n;
      const unsigned c8 = (cidp[i] >> (8 * j)) & 0xffu;
      hunt[j] = cell[j] >= 0 && cell[j] < g.Wo && inside[j] && c8 != 0xffu;
      const unsigned tile = hunt[j] ? c8 : 0u;  // a result with nothing to find reads tile 0 and ignores it
      xt[j] = sx + (size_t)tile * WT + ml * 4;
      yt[j] = sy + (size_t)tile * WTY + cl * 4;
      p[j] = -1;
    }
    bool any = false;
#pragma unroll
    for (int j = 0; j < JC; ++j) any |= hunt[j];
    if (any) {
#pragma unroll 1
      for (int q = BK / 4 - 1; q >= 0; --q) {
#pragma unroll
        for (int j = 0; j < JC; ++j) {
          const ulonglong2 xv = *reinterpret_cast<const ulonglong2*>(xt[j] + q * WB * 4);
          const ulonglong2 yv = *reinterpret_cast<const ulonglong2*>(yt[j] + q * WC * 4);
          float v0, v1, v2, v3;
          unpack2(add2(xv.x, yv.x), v0, v1);
          unpack2(add2(xv.y, yv.y), v2, v3);
          if (v3 == Y[i][j]) p[j] = 4 * q + 3;
          if (v2 == Y[i][j]) p[j] = 4 * q + 2;
          if (v1 == Y[i][j]) p[j] = 4 * q + 1;
          if (v0 == Y[i][j]) p[j] = 4 * q;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < JC; ++j) {
      if (cell[j] < 0 || cell[j] >= g.Wo) continue;
      float val = Y[i][j];
      int pj = hunt[j] ? p[j] : -1;
      if (pj >= 0) {
        // the stored value is the matching term itself: only for a zero can it differ from the maximum (in
        // sign), so that is the one case that reads the term again
        if (val == 0.f)
          val = __fadd_rn(xt[j][(pj >> 2) * WB * 4 + (pj & 3)], yt[j][(pj >> 2) * WC * 4 + (pj & 3)]);
        pj += s0 + (int)((cidp[i] >> (8 * j)) & 0xffu) * BK;
      }
      const int64_t e = (int64_t)m * g.Wo + cell[j];
      ob[e] = inside[j] ? val : 0.f;  // cells outside the matrix stay zero (banded_cuda_kernel.cu:38)
      ib[e] = inside[j] ? (pj >= 0 ? pj - m + g.a_lu : -1) : 0;
    }
  }
}

// tiles of 16 steps in the longest reduction range of a 64 x wc block
int w_tiles(const BandDims& d, int wc = 64) {
  const int64_t range = std::min<int64_t>(WB - 1 + d.Wa(), wc - 1 + d.Wb()) + (BK - 1);
  return (int)ceil_div(range, BK);
}

}  // namespace

// declared in band.cuh
static bool lockstep_blocks_wanted() {  // GENBMM_B200_BAND_MAX=block keeps the 128 x 64 blocks in lockstep
  const char* mode = getenv("GENBMM_B200_BAND_MAX");
  return mode && mode[0] == 'b';
}

bool band_max_fast_eligible(const BandDims& d) {
  // a block's whole reduction range stays in shared memory: at most kMaxTilesW tiles of 16 steps for the 64 x 64
  // blocks (the narrower band up to 338 wide), kMaxSteps for the 128 x 64 blocks
  if (d.Wa() < 32 || d.Wb() < 32 || d.n < 128 || d.n >= (1LL << 30)) return false;
  if (!lockstep_blocks_wanted()) return w_tiles(d) <= kMaxTilesW;
  const int64_t range = std::min<int64_t>(BM - 1 + d.Wa(), BN - 1 + d.Wb()) + 2 * (BK - 1);
  return range <= kMaxSteps * BK;
}

int64_t band_max_workspace_bytes(int64_t B, const BandDims& d) {
  const MaxSkew sa = make_max_skew(d.a_lu, d.Wa(), d.n), sb = make_max_skew(d.b_lu, d.Wb(), d.n);
  return (int64_t)sizeof(float) * (max_skew_floats(sa, B) + max_skew_floats(sb, B) + 64);  // + the error word
}

int band_max_workspace_init(void* ws, int64_t bytes, cudaStream_t st) {
  fill_ninf_kernel<<<1184, 256, 0, st>>>(static_cast<float*>(ws), bytes / (int64_t)sizeof(float));
  return launch_status();
}

int band_max_forward(const float* a, const float* b, float* out, int* idx, const BandDims& d, int64_t B, void* ws,
                     cudaStream_t st) {
  const MaxSkew sa = make_max_skew(d.a_lu, d.Wa(), d.n), sb = make_max_skew(d.b_lu, d.Wb(), d.n);
  float* xs = static_cast<float*>(ws);
  float* ys = xs + max_skew_floats(sa, B);
  const int64_t rows = B * d.n, rblocks = ceil_div(rows, 8);
  if (rblocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  band_max_skew_kernel<<<(unsigned)rblocks, 256, 0, st>>>(a, xs, rows, (int)d.n, d.a_lu, d.Wa(), sa.off, sa.pitch,
                                                         sa.bstride);
  band_max_skew_kernel<<<(unsigned)rblocks, 256, 0, st>>>(b, ys, rows, (int)d.n, d.b_lu, d.Wb(), sb.off, sb.pitch,
                                                         sb.bstride);
  if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
  MaxArgs g{};
  g.xs = xs;
  g.ys = ys;
  g.x_bstride = sa.bstride;
  g.y_bstride = sb.bstride;
  g.x_rstride = sa.pitch - 1;
  g.y_rstride = sb.pitch - 1;
  g.x_kofs = sa.kofs;
  g.y_kofs = sb.kofs;
  g.n = (int)d.n;
  g.a_lu = d.a_lu; g.a_ld = d.a_ld; g.b_lu = d.b_lu; g.b_ld = d.b_ld;
  g.r_lu = d.r_lu();
  g.Wo = d.Wo();
  g.nrb = (int)ceil_div(d.n, BM);
  g.ncb = (g.Wo + BM - 1 + BN - 1) / BN + 1;
  g.out = out;
  g.idx = idx;
  if (!lockstep_blocks_wanted()) {
    g.x_ninf = (sa.off + d.Wa() + 3) & ~3;  // the first whole 16 bytes of a row's padding
    g.y_ninf = (sb.off + d.Wb() + 3) & ~3;
    g.error = reinterpret_cast<int*>(ys + max_skew_floats(sb, B));
    // 64 x 32 blocks (4 x 2 results per thread, 79 registers, 68 KB of tiles at 129 diagonals: three CTAs per SM)
    // unless GENBMM_B200_BAND_MAX_COLS=64 asks for 64 x 64 blocks (4 x 4 per thread, two CTAs per SM):
    // 1.23 against 1.31 ms at 32 x 8192 x 129 diagonals
    const char* shape = getenv("GENBMM_B200_BAND_MAX_COLS");
    const int wc = (shape && atoi(shape) == 64) ? 64 : 32;
    g.nrb = (int)ceil_div(d.n, WB);
    g.ncb = (g.Wo + (WB - 1) + (wc - 1)) / wc + 1;
    const int64_t wblocks = B * g.nrb * g.ncb;
    if (wblocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
    const size_t wsmem = w_smem_bytes(w_tiles(d, wc), wc);
    if (cudaMemsetAsync(g.error, 0, sizeof(int), st) != cudaSuccess) return GBMM_ERR_LAUNCH;
    auto go = [&](auto kern) {
      // several CTAs per SM need the largest shared-memory carveout
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)w_smem_bytes(kMaxTilesW, 64)) != cudaSuccess ||
          cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                               cudaSharedmemCarveoutMaxShared) != cudaSuccess)
        return false;
      kern<<<(unsigned)wblocks, 256, wsmem, st>>>(g);
      return true;
    };
    if (!(wc == 32 ? go(band_max_w_kernel<4, 2, 4>) : go(band_max_w_kernel<4, 4, 4>))) return GBMM_ERR_LAUNCH;
    if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
    return launch_poison_on_error(g.error, out, B * d.n * d.Wo(), nullptr, 0, st);
  }
  const int64_t blocks = B * g.nrb * g.ncb;
  if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  const size_t smem = max_smem_bytes(kMaxSteps);
  if (cudaFuncSetAttribute(band_max_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
          cudaSuccess ||
      cudaFuncSetAttribute(band_max_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
          cudaSuccess)
    return GBMM_ERR_LAUNCH;
  // every block gets the size of the longest range (the sizes differ by block, the launch has one)
  const int64_t range = std::min<int64_t>(BM - 1 + d.Wa(), BN - 1 + d.Wb()) + 2 * (BK - 1);
  const int steps = (int)std::min<int64_t>(kMaxSteps, ceil_div(range, BK));
  // a warp's 8 rows are live in about Wa + 23 of the block's steps: skipping pays when that leaves a good part
  // of the range idle
  if ((d.Wa() + 23) * 20 < range * 17)
    band_max_kernel<true><<<(unsigned)blocks, NT, max_smem_bytes(steps), st>>>(g);
  else
    band_max_kernel<false><<<(unsigned)blocks, NT, max_smem_bytes(steps), st>>>(g);
  return launch_status();
}

}  // namespace gbmm
