// Dense semiring forward kernels: c[b,m,n] = (+)_k a[b,m,k] (x) b[b,k,n].
//
// Replaces the reference's one-thread-per-output kernels (matmul_cuda_kernel.cu:13-152) with
// shared-memory tiled kernels: a CTA of 256 threads owns a 128x64 tile of the result, each
// thread an 8x4 micro-tile; operand tiles of 16 reduction steps are double-buffered through
// registers into shared memory.
//
//   max-plus / prod-max : per reduction tile only the tile maximum is tracked (FADD|FMUL + one
//       3-input FMNMX per two terms); a strict `>` against the running maximum, taken in tile
//       order, remembers the first tile that reached it, and that one tile is rescanned at the
//       end for the first k attaining the maximum.  This reproduces the reference's
//       `if (v > m) { m = v; ind = i; }` (lowest k on ties, -1 and -1e9 when nothing exceeds
//       -1e9) bit for bit, including the sign of a zero maximum.
//   log : per tile, the exact tile maximum first, one rescale of the running sum when it
//       grows, then exp(v - m) on the SFU.  The running maximum starts at -1e9 as in the
//       reference.
//   sample : the log kernel followed by an inverse-CDF pass that keeps the reference's fp32
//       running sum in ascending k and its strict double inequality.
#include "dense.cuh"
#include "tile.cuh"
#include "tma.cuh"

namespace gbmm {
namespace {

constexpr int BM = 128, BN = 64, BK = 16, NT = 256;
constexpr int LDX = BM + 4, LDY = BN + 4;

struct TileCoord {
  int bt, m0, n0;
  __device__ __forceinline__ TileCoord(int64_t id, int tiles_m, int tiles_n) {
    n0 = (int)(id % tiles_n) * BN;
    m0 = (int)((id / tiles_n) % tiles_m) * BM;
    bt = (int)(id / ((int64_t)tiles_n * tiles_m));
  }
};

__device__ __forceinline__ float nan_f() { return __int_as_float(0x7fc00000); }
__device__ __forceinline__ float ninf_f() { return __int_as_float(0xff800000); }
// ------------------------------------------------------------------ max-plus / prod-max
// Packed pairs (sm_100): the two terms of a reduction-step pair are formed by one add.f32x2 /
// mul.f32x2 and folded into the tile maximum by one 3-input max, i.e. one FP32-pipe and one ALU
// instruction per two terms.  The shared tiles therefore hold (k, k+1) pairs side by side:
// element (k, m) at ((k/2) * LD + m) * 2 + (k & 1).
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// a tile (k contiguous in global memory): float4 = 4 consecutive k of one row -> two pairs
__device__ __forceinline__ void store_pairs_a(float* s, const TileLoader<BM, BK, NT, true>& l) {
#pragma unroll
  for (int q = 0; q < TileLoader<BM, BK, NT, true>::NV; ++q) {
    const int f = threadIdx.x + q * NT;
    const int o = f / (BK / 4), r = (f % (BK / 4)) * 4;
    *reinterpret_cast<float2*>(s + ((r / 2) * LDX + o) * 2) = make_float2(l.v[q].x, l.v[q].y);
    *reinterpret_cast<float2*>(s + ((r / 2 + 1) * LDX + o) * 2) = make_float2(l.v[q].z, l.v[q].w);
  }
}
// b tile (n contiguous in global memory): float4 = 4 consecutive columns at one k
__device__ __forceinline__ void store_pairs_b(float* s, const TileLoader<BN, BK, NT, false>& l) {
#pragma unroll
  for (int q = 0; q < TileLoader<BN, BK, NT, false>::NV; ++q) {
    const int f = threadIdx.x + q * NT;
    const int r = f / (BN / 4), o = (f % (BN / 4)) * 4;
    float* p = s + ((r / 2) * LDY + o) * 2 + (r & 1);
    p[0] = l.v[q].x;
    p[2] = l.v[q].y;
    p[4] = l.v[q].z;
    p[6] = l.v[q].w;
  }
}

// PACK: the index of the winning reduction tile is kept in one byte (4 results per register), which
// needs at most 255 tiles (K <= 4080) and lets two CTAs share an SM; otherwise one int per result.
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void cp_async8(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// waits until at most `pending` of this thread's committed groups are still in flight (pending < 8)
__device__ __forceinline__ void cp_async_wait(int pending) {
  switch (pending) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
  }
}

// RESIDENT (reductions of at most kResidentTiles tiles, dynamic shared memory): every reduction tile stays in
// shared memory, so the final search for the first k that attains the maximum reads shared memory instead of
// going back to global memory — for short reductions that search costs more than the reduction itself
// (K = 128: 1 MB of search reads per CTA against 100 KB of operands).  All tiles are requested at once with
// cp.async straight into the pair layout (one group per tile, waited for in order), so the latency of global
// memory is paid once per CTA instead of once per 16-step tile.
constexpr int kResidentTiles = 8;
constexpr int kTileX = BK * LDX, kTileY = BK * LDY;
// Resident tiles are 4 floats further apart than their size (both sizes are multiples of 32 floats): in the
// final search the lanes of a warp read the same cell of DIFFERENT tiles, which would otherwise all fall on
// one bank.
constexpr int kTileXr = kTileX + 4, kTileYr = kTileY + 4;

template <bool MUL, bool PACK, bool RESIDENT>
__global__ void __launch_bounds__(NT, PACK ? 2 : 1) dense_max_fwd_kernel(const float* __restrict__ a,
                                                                         const float* __restrict__ b,
                                                                         float* __restrict__ out,
                                                                         int* __restrict__ idx, int M, int K, int N,
                                                                         int tiles_m, int tiles_n,
                                                                         const float* __restrict__ b_t, int kp) {
  __shared__ __align__(16) float sx_two[RESIDENT ? 1 : 2][RESIDENT ? 4 : kTileX];
  __shared__ __align__(16) float sy_two[RESIDENT ? 1 : 2][RESIDENT ? 4 : kTileY];
  extern __shared__ __align__(16) float resident_smem[];   // RESIDENT: nt x tiles, then nt y tiles
  const int nt_all = (K + BK - 1) / BK;
  float* const sx_base = RESIDENT ? resident_smem : &sx_two[0][0];
  float* const sy_base = RESIDENT ? resident_smem + (size_t)nt_all * kTileXr : &sy_two[0][0];
  auto sx = [&](int t) -> float* { return sx_base + (RESIDENT ? t * kTileXr : (t & 1) * kTileX); };
  auto sy = [&](int t) -> float* { return sy_base + (RESIDENT ? t * kTileYr : (t & 1) * kTileY); };
  const TileCoord tc(blockIdx.x, tiles_m, tiles_n);
  const Micro8x4 mt;
  const float* ab = a + (int64_t)tc.bt * M * K;
  const float* bb = b + (int64_t)tc.bt * K * N;
  const bool vec_a = aligned16(ab) && (K % 4 == 0);
  const bool vec_b = aligned16(bb) && (N % 4 == 0);

  // Two sets of running maxima: a reduction tile folds its terms into one set starting from the
  // other (the first 3-input max of the tile reads the old maximum), so "this tile raised the
  // maximum" is one comparison of the two sets afterwards, and the roles swap for the next tile.
  float X[8][4], Y[8][4];
  int cid[PACK ? 1 : 8][4];
  unsigned cidp[PACK ? 8 : 1];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (PACK) cidp[i] = 0xffffffffu;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      X[i][j] = kFloor;
      Y[i][j] = kFloor;
      if (!PACK) cid[i][j] = -1;
    }
  }

  TileLoader<BM, BK, NT, true> la;
  TileLoader<BN, BK, NT, false> lb;
  const int nt = (K + BK - 1) / BK;
  // a NaN in the padded reduction steps makes the term a NaN, which the maximum ignores
  if (RESIDENT) {
    const bool pair_ok = (K % 2 == 0) && ((reinterpret_cast<uintptr_t>(ab) & 7) == 0);
    for (int t = 0; t < nt; ++t) {
#pragma unroll
      for (int q = 0; q < TileLoader<BM, BK, NT, true>::NV; ++q) {   // a: 4 consecutive k of one row -> two pairs
        const int f = threadIdx.x + q * NT, o = f / (BK / 4), r = (f % (BK / 4)) * 4;
        const int m = tc.m0 + o, k = t * BK + r;
        float* d0 = sx(t) + ((r / 2) * LDX + o) * 2;
        float* d1 = sx(t) + ((r / 2 + 1) * LDX + o) * 2;
        const float* src = ab + (int64_t)m * K + k;
        if (pair_ok && m < M && k + 3 < K) {
          cp_async8(d0, src);
          cp_async8(d1, src + 2);
        } else {
          const bool ok = m < M;
          d0[0] = (ok && k + 0 < K) ? __ldg(src + 0) : nan_f();
          d0[1] = (ok && k + 1 < K) ? __ldg(src + 1) : nan_f();
          d1[0] = (ok && k + 2 < K) ? __ldg(src + 2) : nan_f();
          d1[1] = (ok && k + 3 < K) ? __ldg(src + 3) : nan_f();
        }
      }
#pragma unroll
      for (int q = 0; q < TileLoader<BN, BK, NT, false>::NV; ++q) {  // b: 4 consecutive columns at one k
        const int f = threadIdx.x + q * NT, r = f / (BN / 4), o = (f % (BN / 4)) * 4;
        const int k = t * BK + r, n = tc.n0 + o;
        float* d = sy(t) + ((r / 2) * LDY + o) * 2 + (r & 1);
        const float* src = bb + (int64_t)k * N + n;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (k < K && n + e < N)
            cp_async4(d + 2 * e, src + e);
          else
            d[2 * e] = 0.f;
        }
      }
      cp_async_commit();
    }
  } else {
    la.load(ab, K, 1, tc.m0, 0, M, K, vec_a, nan_f());
    lb.load(bb, 1, N, tc.n0, 0, N, K, vec_b, 0.f);
    store_pairs_a(sx(0), la);
    store_pairs_b(sy(0), lb);
    __syncthreads();
  }

  auto tile_step = [&](int t, float (&acc)[8][4], const float (&prev)[8][4]) {
    if (RESIDENT) {   // tile t has landed (this thread's copies, then everyone's)
      cp_async_wait(nt - 1 - t);
      __syncthreads();
    } else if (t + 1 < nt) {
      la.load(ab, K, 1, tc.m0, (t + 1) * BK, M, K, vec_a, nan_f());
      lb.load(bb, 1, N, tc.n0, (t + 1) * BK, N, K, vec_b, 0.f);
    }
#pragma unroll
    for (int kp2 = 0; kp2 < BK / 2; ++kp2) {
      const float* xs = sx(t) + (kp2 * LDX + mt.ty * 4) * 2;
      const float* ys = sy(t) + (kp2 * LDY + mt.tx * 4) * 2;
      const ulonglong2 x01 = *reinterpret_cast<const ulonglong2*>(xs);
      const ulonglong2 x23 = *reinterpret_cast<const ulonglong2*>(xs + 4);
      const ulonglong2 x45 = *reinterpret_cast<const ulonglong2*>(xs + 128);
      const ulonglong2 x67 = *reinterpret_cast<const ulonglong2*>(xs + 132);
      const ulonglong2 y01 = *reinterpret_cast<const ulonglong2*>(ys);
      const ulonglong2 y23 = *reinterpret_cast<const ulonglong2*>(ys + 4);
      const unsigned long long xp[8] = {x01.x, x01.y, x23.x, x23.y, x45.x, x45.y, x67.x, x67.y};
      const unsigned long long yp[4] = {y01.x, y01.y, y23.x, y23.y};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float v0, v1;
          unpack2(MUL ? mul2(xp[i], yp[j]) : add2(xp[i], yp[j]), v0, v1);
          acc[i][j] = max3(kp2 == 0 ? prev[i][j] : acc[i][j], v0, v1);
        }
    }
    // strict `>`: an equal maximum in a later tile does not move the index
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (PACK) {
        if (acc[i][0] > prev[i][0]) cidp[i] = __byte_perm(cidp[i], (unsigned)t, 0x3214);
        if (acc[i][1] > prev[i][1]) cidp[i] = __byte_perm(cidp[i], (unsigned)t, 0x3240);
        if (acc[i][2] > prev[i][2]) cidp[i] = __byte_perm(cidp[i], (unsigned)t, 0x3410);
        if (acc[i][3] > prev[i][3]) cidp[i] = __byte_perm(cidp[i], (unsigned)t, 0x4210);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (acc[i][j] > prev[i][j]) cid[i][j] = t;
      }
    }
    if (!RESIDENT) {
      if (t + 1 < nt) {
        store_pairs_a(sx(t + 1), la);
        store_pairs_b(sy(t + 1), lb);
      }
      __syncthreads();
    }
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
  // from here on Y holds the maxima
  auto tile_of = [&](int i, int j) -> int {
    if (!PACK) return cid[PACK ? 0 : i][j];
    const unsigned c = (cidp[PACK ? i : 0] >> (8 * j)) & 0xffu;
    return c == 0xffu ? -1 : (int)c;
  };

  // Rescan the winning tile of every result for the first k that attains the maximum; the
  // stored value is that term itself, so a zero keeps the sign the reference would keep.
  float* ob = out + (int64_t)tc.bt * M * N;
  int* ib = idx + (int64_t)tc.bt * M * N;
  const bool vec_o = aligned16(ob) && aligned16(ib) && (N % 4 == 0);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = tc.m0 + mt.row(i);  // the same row for the four lanes of a quad
    float val[4];
    int ind[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      val[j] = Y[i][j];
      ind[j] = -1;
    }
    if (RESIDENT) {
      // every tile is still in shared memory: each thread searches the winning tile of its own results, from
      // the last pair down so that the lowest matching k is the assignment that sticks; a NaN (padding beyond
      // K) never equals the maximum
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int ct = tile_of(i, j);
        if (ct < 0) continue;
        const float* xs = sx(ct) + mt.row(i) * 2;
        const float* ys = sy(ct) + mt.col(j) * 2;
#pragma unroll
        for (int kp2 = BK / 2 - 1; kp2 >= 0; --kp2) {
          const float2 xv = *reinterpret_cast<const float2*>(xs + kp2 * LDX * 2);
          const float2 yv = *reinterpret_cast<const float2*>(ys + kp2 * LDY * 2);
          const float t1 = MUL ? __fmul_rn(xv.y, yv.y) : __fadd_rn(xv.y, yv.y);
          const float t0 = MUL ? __fmul_rn(xv.x, yv.x) : __fadd_rn(xv.x, yv.x);
          if (t1 == Y[i][j]) {
            val[j] = t1;
            ind[j] = ct * BK + 2 * kp2 + 1;
          }
          if (t0 == Y[i][j]) {
            val[j] = t0;
            ind[j] = ct * BK + 2 * kp2;
          }
        }
      }
    } else if (b_t) {
      // Quad-cooperative scan: the four lanes of a quad take the quad's results one owner at a
      // time; each lane loads a quarter (16 bytes of a, 16 of b_t) of the winning tile's two
      // 64-byte segments, so one warp-wide load touches 8 segments instead of 32, and the lowest
      // matching k is found by a minimum over the quad.
      const unsigned full = 0xffffffffu;
      const int lane = threadIdx.x & 31, q = lane & 3;
      const int tx_quad = mt.tx & ~3;
#pragma unroll
      for (int o = 0; o < 4; ++o) {
        const int src = (lane & ~3) | o;
        float bo[4], av[4][4], bv[4][4];
        int ct[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          bo[j] = __shfl_sync(full, Y[i][j], src);
          ct[j] = __shfl_sync(full, tile_of(i, j), src);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = tc.n0 + (tx_quad + o) * 4 + j;
          const int k0 = ct[j] * BK + 4 * q;
          const bool ok = ct[j] >= 0 && m < M && n < N;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            av[j][kk] = nan_f();
            bv[j][kk] = 0.f;
          }
          if (ok) {
            const float* ap = ab + (int64_t)m * K + k0;
            if (vec_a && k0 + 3 < K) {
              const float4 t4 = __ldg(reinterpret_cast<const float4*>(ap));
              av[j][0] = t4.x; av[j][1] = t4.y; av[j][2] = t4.z; av[j][3] = t4.w;
            } else {
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                if (k0 + kk < K) av[j][kk] = __ldg(ap + kk);
            }
            const float4 u4 = __ldg(reinterpret_cast<const float4*>(b_t + ((int64_t)tc.bt * N + n) * kp + k0));
            bv[j][0] = u4.x; bv[j][1] = u4.y; bv[j][2] = u4.z; bv[j][3] = u4.w;
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          int loc = 99;
          float vm = 0.f;
#pragma unroll
          for (int kk = 3; kk >= 0; --kk) {
            // a NaN (padding beyond K, or no winner) never equals the maximum
            const float t = MUL ? __fmul_rn(av[j][kk], bv[j][kk]) : __fadd_rn(av[j][kk], bv[j][kk]);
            if (t == bo[j]) {
              loc = 4 * q + kk;
              vm = t;
            }
          }
#pragma unroll
          for (int d = 1; d <= 2; d <<= 1) {
            const int oloc = __shfl_xor_sync(full, loc, d);
            const float ovm = __shfl_xor_sync(full, vm, d);
            if (oloc < loc) {
              loc = oloc;
              vm = ovm;
            }
          }
          if (q == o && loc != 99) {
            ind[j] = ct[j] * BK + loc;
            val[j] = vm;
          }
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = tc.n0 + mt.col(j);
        val[j] = Y[i][j];
        ind[j] = -1;
        const int ct = tile_of(i, j);
        if (m < M && n < N && ct >= 0) {
          // all loads of the tile are issued before any is used; the scan runs from the last k
          // down, so the lowest matching k is the assignment that sticks.  With a transposed copy
          // of b (b_t: (batch, N, kp), kp a multiple of 16) both 16-term segments are contiguous:
          // 8 128-bit loads and 4 sectors per result instead of 32 loads and 18 sectors.
          const int k0 = ct * BK;
          const float* ap = ab + (int64_t)m * K + k0;
          float xv[BK], yv[BK], v[BK];
          if (vec_a && k0 + BK <= K) {
  #pragma unroll
            for (int q = 0; q < BK / 4; ++q) {
              const float4 t4 = __ldg(reinterpret_cast<const float4*>(ap) + q);
              xv[4 * q] = t4.x; xv[4 * q + 1] = t4.y; xv[4 * q + 2] = t4.z; xv[4 * q + 3] = t4.w;
            }
          } else {
  #pragma unroll
            for (int kk = 0; kk < BK; ++kk) xv[kk] = (k0 + kk < K) ? __ldg(ap + kk) : nan_f();
          }
          if (b_t) {
            const float4* bp = reinterpret_cast<const float4*>(b_t + ((int64_t)tc.bt * N + n) * kp + k0);
  #pragma unroll
            for (int q = 0; q < BK / 4; ++q) {
              const float4 t4 = __ldg(bp + q);
              yv[4 * q] = t4.x; yv[4 * q + 1] = t4.y; yv[4 * q + 2] = t4.z; yv[4 * q + 3] = t4.w;
            }
          } else {
            const float* bp = bb + (int64_t)k0 * N + n;
  #pragma unroll
            for (int kk = 0; kk < BK; ++kk) yv[kk] = (k0 + kk < K) ? __ldg(bp + (int64_t)kk * N) : 0.f;
          }
  #pragma unroll
          for (int kk = 0; kk < BK; ++kk) {
            const float t = MUL ? __fmul_rn(xv[kk], yv[kk]) : __fadd_rn(xv[kk], yv[kk]);
            v[kk] = (k0 + kk < K) ? t : nan_f();
          }
  #pragma unroll
          for (int kk = BK - 1; kk >= 0; --kk)
            if (v[kk] == Y[i][j]) {
              val[j] = v[kk];
              ind[j] = k0 + kk;
            }
        }
      }
    }
    if (m >= M) continue;
    const int nb = tc.n0 + mt.col(0);
    if (vec_o && nb + 3 < N) {
      *reinterpret_cast<float4*>(ob + (int64_t)m * N + nb) = make_float4(val[0], val[1], val[2], val[3]);
      *reinterpret_cast<int4*>(ib + (int64_t)m * N + nb) = make_int4(ind[0], ind[1], ind[2], ind[3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (nb + j < N) {
          ob[(int64_t)m * N + nb + j] = val[j];
          ib[(int64_t)m * N + nb + j] = ind[j];
        }
    }
  }
}

// ------------------------------------------------------------------ max-plus / prod-max, TMA-staged
// The same reduction with the operand tiles brought in by TMA instead of through registers.  A 32-step stage of the
// four-stage shared-memory ring is eight boxes of a (4 steps x 128 rows) and eight of the transposed copy of b
// (4 steps x 64 rows): a box lands as [row][4 steps], so a stage is [quad of steps][row][4] — one 128-bit load
// per row and quad, adjacent rows in adjacent 16-byte cells, the two halves of a loaded quad being the (k, k+1)
// pairs of the packed add: as many shared-memory loads as the pair layout of the kernel above, and none of its
// staging instructions.  `full` barriers carry the byte counts, `empty` barriers one arrival per warp.  Thread 0
// issues the copies: after its warp has finished a stage it waits for the other warps' arrivals on that stage
// and refills the slot with the tile four stages ahead (the other warps never wait for anything but data).
// Reduction steps beyond K read as NaN (the tensor map's out-of-bounds fill), a term the maximum ignores, exactly
// like the padding of the kernel above.  A thread's eight rows are ty + 16 i and its four columns tx + 16 j.
constexpr int XS_STAGES = 4, XS_K = 32;
struct alignas(1024) MaxTmaSmem {
  float a[XS_STAGES][BM * XS_K];
  float b[XS_STAGES][BN * XS_K];
  uint64_t full[XS_STAGES];
  uint64_t empty[XS_STAGES];
};

template <bool MUL>
__global__ void __launch_bounds__(NT, 2) dense_max_tma_kernel(const __grid_constant__ CUtensorMap map_a,
                                                              const __grid_constant__ CUtensorMap map_bt,
                                                              const float* __restrict__ a,
                                                              const float* __restrict__ b_t, float* __restrict__ out,
                                                              int* __restrict__ idx, int M, int K, int N, int tiles_m,
                                                              int tiles_n, int kp, int* __restrict__ error) {
  extern __shared__ unsigned char smem_raw[];
  MaxTmaSmem& sm = *reinterpret_cast<MaxTmaSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const TileCoord tc(blockIdx.x, tiles_m, tiles_n);
  const int tid = threadIdx.x, lane = tid & 31, tx = tid % 16, ty = tid / 16;
  const int nst = (K + XS_K - 1) / XS_K;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < XS_STAGES; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], NT / 32);
    }
    fence_barrier_init();
  }
  __syncthreads();
  auto issue = [&](int t) {
    const int s = t % XS_STAGES;
    mbar_arrive_expect_tx(&sm.full[s], (BM + BN) * XS_K * sizeof(float));
#pragma unroll
    for (int q = 0; q < XS_K / 4; ++q) {   // one box per quad of steps: [row][4 steps], 16 bytes per row
      tma_load_3d(sm.a[s] + q * BM * 4, &map_a, &sm.full[s], t * XS_K + 4 * q, tc.m0, tc.bt);
      tma_load_3d(sm.b[s] + q * BN * 4, &map_bt, &sm.full[s], t * XS_K + 4 * q, tc.n0, tc.bt);
    }
  };
  if (tid == 0)
    for (int t = 0; t < XS_STAGES && t < nst; ++t) issue(t);

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
  bool fail = false;

  // one 16-step sub-tile: quads q0 .. q0 + 3 of the stage; u = its index among all 16-step tiles
  auto sub_tile = [&](const float* xs, const float* ys, int q0, int u, float (&acc)[8][4], const float (&prev)[8][4]) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      ulonglong2 xq[8], yq[4];
#pragma unroll
      for (int i = 0; i < 8; ++i) xq[i] = *reinterpret_cast<const ulonglong2*>(xs + ((q0 + c) * BM + 16 * i) * 4);
#pragma unroll
      for (int j = 0; j < 4; ++j) yq[j] = *reinterpret_cast<const ulonglong2*>(ys + ((q0 + c) * BN + 16 * j) * 4);
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float v0, v1, v2, v3;
          unpack2(MUL ? mul2(xq[i].x, yq[j].x) : add2(xq[i].x, yq[j].x), v0, v1);
          unpack2(MUL ? mul2(xq[i].y, yq[j].y) : add2(xq[i].y, yq[j].y), v2, v3);
          acc[i][j] = max3(max3(c == 0 ? prev[i][j] : acc[i][j], v0, v1), v2, v3);
        }
    }
    // strict `>`: an equal maximum in a later tile does not move the index
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (acc[i][0] > prev[i][0]) cidp[i] = __byte_perm(cidp[i], (unsigned)u, 0x3214);
      if (acc[i][1] > prev[i][1]) cidp[i] = __byte_perm(cidp[i], (unsigned)u, 0x3240);
      if (acc[i][2] > prev[i][2]) cidp[i] = __byte_perm(cidp[i], (unsigned)u, 0x3410);
      if (acc[i][3] > prev[i][3]) cidp[i] = __byte_perm(cidp[i], (unsigned)u, 0x4210);
    }
  };

  for (int t = 0; t < nst; ++t) {
    const int s = t % XS_STAGES;
    if (!mbar_wait_bounded(&sm.full[s], (t / XS_STAGES) & 1)) fail = true;
    if (__any_sync(0xffffffffu, fail)) {
      fail = true;
      break;
    }
    const float* xs = sm.a[s] + ty * 4;
    const float* ys = sm.b[s] + tx * 4;
    sub_tile(xs, ys, 0, 2 * t, X, Y);
    sub_tile(xs, ys, 4, 2 * t + 1, Y, X);
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.empty[s])) : "memory");
    if (tid == 0 && t + XS_STAGES < nst) {
      // every warp is done with this slot: refill it with the tile four stages ahead
      if (!mbar_wait_bounded(&sm.empty[s], (t / XS_STAGES) & 1)) {
        fail = true;
      } else {
        issue(t + XS_STAGES);
      }
    }
  }
  if (__syncthreads_or(fail)) {
    // a wait gave up: record it (the caller's next kernel turns the result into NaN) and write nothing.  The
    // copies still in flight get a bounded chance to land before the shared memory is released.
    if (tid == 0) {
      for (int t2 = 0; t2 < XS_STAGES; ++t2) mbar_wait_bounded(&sm.full[t2], 0);
      if (error) atomicExch(error, 1);
    }
    return;
  }
  // from here on Y holds the maxima (two sub-tiles per stage: the roles are back where they started)
  auto tile_of = [&](int i, int j) -> int {
    const unsigned c = (cidp[i] >> (8 * j)) & 0xffu;
    return c == 0xffu ? -1 : (int)c;
  };
  const float* ab = a + (int64_t)tc.bt * M * K;
  float* ob = out + (int64_t)tc.bt * M * N;
  int* ib = idx + (int64_t)tc.bt * M * N;
  // Quad-cooperative search of the winning 16-step tile, as in the kernel above: the four lanes of a quad share
  // their rows (same ty) and own four consecutive columns; they take the quad's results one owner at a time, each
  // lane loading a quarter (16 bytes of a, 16 of b_t) of the tile's two 64-byte segments.
  const unsigned full = 0xffffffffu;
  const int q = lane & 3, tx_quad = tx & ~3;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = tc.m0 + ty + 16 * i;
    float val[4];
    int ind[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      val[j] = Y[i][j];
      ind[j] = -1;
    }
#pragma unroll
    for (int o = 0; o < 4; ++o) {
      const int src = (lane & ~3) | o;
      float bo[4], av[4][4], bv[4][4];
      int ct[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        bo[j] = __shfl_sync(full, Y[i][j], src);
        ct[j] = __shfl_sync(full, tile_of(i, j), src);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = tc.n0 + tx_quad + o + 16 * j;
        const int k0 = ct[j] * BK + 4 * q;
        const bool ok = ct[j] >= 0 && m < M && n < N;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          av[j][kk] = nan_f();
          bv[j][kk] = 0.f;
        }
        if (ok) {
          if (k0 + 3 < K) {   // K is a multiple of 4 on this path
            const float4 t4 = __ldg(reinterpret_cast<const float4*>(ab + (int64_t)m * K + k0));
            av[j][0] = t4.x; av[j][1] = t4.y; av[j][2] = t4.z; av[j][3] = t4.w;
          }
          const float4 u4 = __ldg(reinterpret_cast<const float4*>(b_t + ((int64_t)tc.bt * N + n) * kp + k0));
          bv[j][0] = u4.x; bv[j][1] = u4.y; bv[j][2] = u4.z; bv[j][3] = u4.w;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int loc = 99;
        float vm = 0.f;
#pragma unroll
        for (int kk = 3; kk >= 0; --kk) {
          // a NaN (padding beyond K, or no winner) never equals the maximum
          const float t = MUL ? __fmul_rn(av[j][kk], bv[j][kk]) : __fadd_rn(av[j][kk], bv[j][kk]);
          if (t == bo[j]) {
            loc = 4 * q + kk;
            vm = t;
          }
        }
#pragma unroll
        for (int d = 1; d <= 2; d <<= 1) {
          const int oloc = __shfl_xor_sync(full, loc, d);
          const float ovm = __shfl_xor_sync(full, vm, d);
          if (oloc < loc) {
            loc = oloc;
            vm = ovm;
          }
        }
        if (q == o && loc != 99) {
          ind[j] = ct[j] * BK + loc;
          val[j] = vm;
        }
      }
    }
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = tc.n0 + tx + 16 * j;
      if (n < N) {
        ob[(int64_t)m * N + n] = val[j];
        ib[(int64_t)m * N + n] = ind[j];
      }
    }
  }
}

// Tensor map of a (batch, rows, cols) fp32 array with rows `pitch` apart, fetched as boxes of box_rows rows x 4
// columns (16 bytes per row, no swizzle); elements outside [0, rows) x [0, cols) read as NaN.
bool make_max_map(CUtensorMap* map, const float* base, uint64_t batch, uint64_t rows, uint64_t cols, uint64_t pitch,
                  uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || (reinterpret_cast<uintptr_t>(base) & 15) || (pitch & 3)) return false;
  const cuuint64_t dims[3] = {cols, rows, batch};
  const cuuint64_t strides[2] = {pitch * sizeof(float), rows * pitch * sizeof(float)};
  const cuuint32_t box[3] = {4, box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NAN_REQUEST_ZERO_FMA) == CUDA_SUCCESS;
}

// b:(batch, K, N) -> b_t:(batch, N, kp) for the rescan of the max kernels (plain 32x32 tile transpose)
__global__ void __launch_bounds__(256) transpose_b_kernel(const float* __restrict__ b, float* __restrict__ b_t,
                                                          int K, int N, int kp, int tiles_k, int tiles_n) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
  const int64_t id = blockIdx.x;
  const int n0 = (int)(id % tiles_n) * 32, k0 = (int)((id / tiles_n) % tiles_k) * 32;
  const int64_t bt = id / ((int64_t)tiles_n * tiles_k);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int k = k0 + ty + q * 8, n = n0 + tx;
    tile[ty + q * 8][tx] = (k < K && n < N) ? __ldg(b + (bt * K + k) * N + n) : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int n = n0 + ty + q * 8, k = k0 + tx;
    if (n < N && k < kp) b_t[(bt * N + n) * kp + k] = tile[tx][ty + q * 8];
  }
}

// ------------------------------------------------------------------ log-sum-exp
__device__ __forceinline__ void log_fwd_tile(const TileCoord& tc, float (&sx)[2][BK * LDX],
                                             float (&sy)[2][BK * LDY], const float* __restrict__ a,
                                             const float* __restrict__ b, float* __restrict__ out,
                                             float* __restrict__ maxes, int M, int K, int N) {
  const Micro8x4 mt;
  const float* ab = a + (int64_t)tc.bt * M * K;
  const float* bb = b + (int64_t)tc.bt * K * N;
  const bool vec_a = aligned16(ab) && (K % 4 == 0);
  const bool vec_b = aligned16(bb) && (N % 4 == 0);

  float mx[8][4], sum[8][4], tmx[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      mx[i][j] = kFloor;
      sum[i][j] = 0.f;
    }

  TileLoader<BM, BK, NT, true> la;
  TileLoader<BN, BK, NT, false> lb;
  const int nt = (K + BK - 1) / BK;
  // padded reduction steps carry -inf: ignored by the maximum, exp(-inf - m) = 0 in the sum
  la.load(ab, K, 1, tc.m0, 0, M, K, vec_a, ninf_f());
  lb.load(bb, 1, N, tc.n0, 0, N, K, vec_b, 0.f);
  la.store(sx[0], LDX);
  lb.store(sy[0], LDY);
  __syncthreads();

  for (int t = 0; t < nt; ++t) {
    const int cur = t & 1;
    if (t + 1 < nt) {
      la.load(ab, K, 1, tc.m0, (t + 1) * BK, M, K, vec_a, ninf_f());
      lb.load(bb, 1, N, tc.n0, (t + 1) * BK, N, K, vec_b, 0.f);
    }
    // pass 1: exact maximum of this tile's terms
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) tmx[i][j] = ninf_f();
#pragma unroll 2
    for (int kk = 0; kk < BK; kk += 2) {
      float x0[8], x1[8], y0[4], y1[4];
      mt.load_x(sx[cur] + kk * LDX, LDX, x0);
      mt.load_y(sy[cur] + kk * LDY, y0);
      mt.load_x(sx[cur] + (kk + 1) * LDX, LDX, x1);
      mt.load_y(sy[cur] + (kk + 1) * LDY, y1);
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) tmx[i][j] = max3(tmx[i][j], x0[i] + y0[j], x1[i] + y1[j]);
    }
    // rescale the running sum where the maximum grew
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (tmx[i][j] > mx[i][j]) {
          sum[i][j] *= exp_sfu(mx[i][j] - tmx[i][j]);
          mx[i][j] = tmx[i][j];
        }
    // The sums of pass 1 are recomputed, not kept: the barrier stops the compiler from
    // carrying BK*32 of them in registers across the two passes.
    asm volatile("" ::: "memory");
    // pass 2: accumulate exp(v - m)
    // exp(v - m) = 2^(v*log2e - m*log2e): one FADD, one FFMA, one MUFU and one FADD per term
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) tmx[i][j] = -mx[i][j] * kLog2e;
#pragma unroll 4
    for (int kk = 0; kk < BK; ++kk) {
      float x[8], y[4];
      mt.load_x(sx[cur] + kk * LDX, LDX, x);
      mt.load_y(sy[cur] + kk * LDY, y);
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) sum[i][j] += ex2_approx(fmaf(x[i] + y[j], kLog2e, tmx[i][j]));
    }
    if (t + 1 < nt) {
      la.store(sx[cur ^ 1], LDX);
      lb.store(sy[cur ^ 1], LDY);
    }
    __syncthreads();
  }

  float* ob = out + (int64_t)tc.bt * M * N;
  float* mb = maxes ? maxes + (int64_t)tc.bt * M * N : nullptr;
  const bool vec_o = aligned16(ob) && (!mb || aligned16(mb)) && (N % 4 == 0);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = tc.m0 + mt.row(i);
    if (m >= M) continue;
    float val[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) val[j] = logf(sum[i][j]) + mx[i][j];
    const int nb = tc.n0 + mt.col(0);
    if (vec_o && nb + 3 < N) {
      *reinterpret_cast<float4*>(ob + (int64_t)m * N + nb) = make_float4(val[0], val[1], val[2], val[3]);
      if (mb)
        *reinterpret_cast<float4*>(mb + (int64_t)m * N + nb) =
            make_float4(mx[i][0], mx[i][1], mx[i][2], mx[i][3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (nb + j < N) {
          ob[(int64_t)m * N + nb + j] = val[j];
          if (mb) mb[(int64_t)m * N + nb + j] = mx[i][j];
        }
    }
  }
}

// One tile per CTA (FLAGGED false: grid = all tiles).  Behind the factorised fast path (FLAGGED) only the
// 128x128 result tiles it marked are recomputed: a capped grid whose CTAs gather the marked tiles among
// their share of the `total` tiles and work through them.
template <bool FLAGGED>
__global__ void __launch_bounds__(NT) dense_log_fwd_kernel(const float* __restrict__ a,
                                                           const float* __restrict__ b,
                                                           float* __restrict__ out,
                                                           float* __restrict__ maxes, int M, int K, int N,
                                                           int tiles_m, int tiles_n,
                                                           const int* __restrict__ flags, int64_t total,
                                                           const int* error, int64_t out_count) {
  __shared__ __align__(16) float sx[2][BK * LDX];
  __shared__ __align__(16) float sy[2][BK * LDY];
  if (!FLAGGED) {
    log_fwd_tile(TileCoord(blockIdx.x, tiles_m, tiles_n), sx, sy, a, b, out, maxes, M, K, N);
    return;
  }
  // the product kernel before this one gave up on a bounded wait: the whole result becomes NaN
  if (poison_if_failed(error, out, out_count)) return;
  __shared__ int list[NT];
  __shared__ int count;
  const int fm = (M + 127) / 128, fn = (N + 127) / 128;
  auto flagged = [&](int64_t id) {
    const TileCoord t(id, tiles_m, tiles_n);
    return __ldg(flags + ((int64_t)t.bt * fm + t.m0 / 128) * fn + t.n0 / 128) != 0;
  };
  for (int64_t base = 0; base < total; base += (int64_t)gridDim.x * NT) {
    const int nw = collect_tiles(base, total, list, &count, flagged);
    for (int w = 0; w < nw; ++w) {
      log_fwd_tile(TileCoord(list[w], tiles_m, tiles_n), sx, sy, a, b, out, maxes, M, K, N);
      __syncthreads();
    }
  }
}

// ------------------------------------------------------------------ inverse-CDF sampling pass
// Follows matmul_cuda_kernel.cu:109-118: with p_k = exp(a+b-out) and `total` the fp32 running
// sum in ascending k, the sample is the first k with total < u and total + p_k > u; 0 if none.
// total never decreases, so the condition can hold for one k only and no early exit is needed.
__global__ void __launch_bounds__(NT) dense_sample_pick_kernel(const float* __restrict__ a,
                                                               const float* __restrict__ b,
                                                               const float* __restrict__ u,
                                                               const float* __restrict__ out,
                                                               int* __restrict__ idx, int M, int K, int N,
                                                               int tiles_m, int tiles_n) {
  __shared__ __align__(16) float sx[2][BK * LDX];
  __shared__ __align__(16) float sy[2][BK * LDY];
  const TileCoord tc(blockIdx.x, tiles_m, tiles_n);
  const Micro8x4 mt;
  const float* ab = a + (int64_t)tc.bt * M * K;
  const float* bb = b + (int64_t)tc.bt * K * N;
  const float* ub = u + (int64_t)tc.bt * M * N;
  const float* ob = out + (int64_t)tc.bt * M * N;
  const bool vec_a = aligned16(ab) && (K % 4 == 0);
  const bool vec_b = aligned16(bb) && (N % 4 == 0);

  float total[8][4], lse[8][4], r[8][4];
  int pick[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = tc.m0 + mt.row(i), n = tc.n0 + mt.col(j);
      const bool ok = m < M && n < N;
      total[i][j] = 0.f;
      pick[i][j] = 0;
      lse[i][j] = ok ? -kLog2e * __ldg(ob + (int64_t)m * N + n) : 0.f;  // -out * log2(e)
      r[i][j] = ok ? __ldg(ub + (int64_t)m * N + n) : 0.f;
    }

  TileLoader<BM, BK, NT, true> la;
  TileLoader<BN, BK, NT, false> lb;
  const int nt = (K + BK - 1) / BK;
  la.load(ab, K, 1, tc.m0, 0, M, K, vec_a, ninf_f());
  lb.load(bb, 1, N, tc.n0, 0, N, K, vec_b, 0.f);
  la.store(sx[0], LDX);
  lb.store(sy[0], LDY);
  __syncthreads();

  for (int t = 0; t < nt; ++t) {
    const int cur = t & 1;
    if (t + 1 < nt) {
      la.load(ab, K, 1, tc.m0, (t + 1) * BK, M, K, vec_a, ninf_f());
      lb.load(bb, 1, N, tc.n0, (t + 1) * BK, N, K, vec_b, 0.f);
    }
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float x[8], y[4];
      mt.load_x(sx[cur] + kk * LDX, LDX, x);
      mt.load_y(sy[cur] + kk * LDY, y);
      const int k = t * BK + kk;
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float e = ex2_approx(fmaf(x[i] + y[j], kLog2e, lse[i][j]));  // exp(a + b - out)
          const float nxt = total[i][j] + e;
          if (total[i][j] < r[i][j] && nxt > r[i][j]) pick[i][j] = k;
          total[i][j] = nxt;
        }
    }
    if (t + 1 < nt) {
      la.store(sx[cur ^ 1], LDX);
      lb.store(sy[cur ^ 1], LDY);
    }
    __syncthreads();
  }

  int* ib = idx + (int64_t)tc.bt * M * N;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = tc.m0 + mt.row(i);
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = tc.n0 + mt.col(j);
      if (n < N) ib[(int64_t)m * N + n] = pick[i][j];
    }
  }
}

}  // namespace
}  // namespace gbmm

namespace gbmm {
// Exact log-sum-exp of the result tiles marked in `flags` (all tiles when flags is null).
int launch_log_fwd_flagged(const float* a, const float* b, float* out, const int* flags, int64_t B, int64_t M,
                           int64_t K, int64_t N, cudaStream_t st, const int* error) {
  const int64_t tiles_m = ceil_div(M, BM), tiles_n = ceil_div(N, BN), blocks = B * tiles_m * tiles_n;
  if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  if (!flags) {
    dense_log_fwd_kernel<false><<<(unsigned)blocks, NT, 0, st>>>(a, b, out, nullptr, (int)M, (int)K, (int)N,
                                                                 (int)tiles_m, (int)tiles_n, nullptr, blocks,
                                                                 nullptr, 0);
    return launch_status();
  }
  unsigned grid = 0;
  if (int rc = capped_grid(blocks, &grid)) return rc;
  dense_log_fwd_kernel<true><<<grid, NT, 0, st>>>(a, b, out, nullptr, (int)M, (int)K, (int)N, (int)tiles_m,
                                                  (int)tiles_n, flags, blocks, error, B * M * N);
  return launch_status();
}
}  // namespace gbmm

using namespace gbmm;

extern "C" int gbmm_dense_sample_pick_f32(const float* a, const float* b, const float* u, const float* out,
                                          int32_t* idx, int64_t B, int64_t M, int64_t K, int64_t N, void* stream) {
  if (B < 0 || M < 0 || K < 0 || N < 0) return GBMM_ERR_INVALID_ARG;
  if (B == 0 || M == 0 || N == 0) return GBMM_OK;
  if ((K > 0 && (!a || !b)) || !u || !out || !idx) return GBMM_ERR_INVALID_ARG;
  if (M >= (1LL << 31) - BM || K >= (1LL << 31) - BK || N >= (1LL << 31) - BN) return GBMM_ERR_UNSUPPORTED;
  const int64_t tiles_m = ceil_div(M, BM), tiles_n = ceil_div(N, BN), blocks = B * tiles_m * tiles_n;
  if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  dense_sample_pick_kernel<<<(unsigned)blocks, NT, 0, static_cast<cudaStream_t>(stream)>>>(
      a, b, u, const_cast<float*>(out), idx, (int)M, (int)K, (int)N, (int)tiles_m, (int)tiles_n);
  return launch_status();
}

extern "C" int64_t gbmm_dense_forward_workspace_bytes(int mode, int64_t B, int64_t M, int64_t K, int64_t N) {
  if (B < 0 || M < 0 || K < 0 || N < 0) return -1;
  if (mode != GBMM_MODE_MAX && mode != GBMM_MODE_PRODMAX) return 0;
  if ((K + BK - 1) / BK <= kResidentTiles) return 0;   // short reductions search shared memory, no copy of b
  if (dense_max_w_eligible(nullptr, K)) return 0;        // as does dense_max_w_kernel (a misaligned `a` falls back to
                                                         // the plain index search of the kernel below)
  return (int64_t)sizeof(float) * B * N * ((K + 15) / 16 * 16);
}

extern "C" int gbmm_dense_forward_f32(int mode, const float* a, const float* b, const float* u, float* out,
                                      void* aux, int64_t B, int64_t M, int64_t K, int64_t N, void* workspace,
                                      int64_t workspace_bytes, void* stream) {
  if (mode < 0 || mode > 3) return GBMM_ERR_INVALID_ARG;
  if (B < 0 || M < 0 || K < 0 || N < 0) return GBMM_ERR_INVALID_ARG;
  if (B == 0 || M == 0 || N == 0) return GBMM_OK;
  if (!a && K > 0) return GBMM_ERR_INVALID_ARG;
  if (!b && K > 0) return GBMM_ERR_INVALID_ARG;
  if (!out) return GBMM_ERR_INVALID_ARG;
  if (mode != GBMM_MODE_LOG && !aux) return GBMM_ERR_INVALID_ARG;
  if (mode == GBMM_MODE_SAMPLE && !u) return GBMM_ERR_INVALID_ARG;
  if (M >= (1LL << 31) - BM || K >= (1LL << 31) - BK || N >= (1LL << 31) - BN) return GBMM_ERR_UNSUPPORTED;
  const int64_t tiles_m = ceil_div(M, BM), tiles_n = ceil_div(N, BN);
  const int64_t blocks = B * tiles_m * tiles_n;
  if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid((unsigned)blocks), block(NT);
  const int m = (int)M, k = (int)K, n = (int)N, tm = (int)tiles_m, tn = (int)tiles_n;
  switch (mode) {
    case GBMM_MODE_LOG:
      if (small_log_wanted(blocks)) return launch_small_log_fwd(a, b, out, static_cast<float*>(aux), B, M, K, N, st);
      dense_log_fwd_kernel<false><<<grid, block, 0, st>>>(a, b, out, static_cast<float*>(aux), m, k, n, tm, tn, nullptr,
                                                          blocks, nullptr, 0);
      break;
    case GBMM_MODE_MAX:
    case GBMM_MODE_PRODMAX: {
      const bool pack = ceil_div(K, BK) <= 255;
      int* ix = static_cast<int*>(aux);
      const bool mul = mode == GBMM_MODE_PRODMAX;
      if (dense_max_w_eligible(a, K)) {   // short reductions: warps that do not wait for one another
        if (int rc = launch_dense_max_w(mul, a, b, out, ix, B, M, K, N, st)) return rc;
        break;
      }
      if (K > 0 && ceil_div(K, BK) <= kResidentTiles) {
        // short reductions: every tile stays in shared memory and the index search reads it there
        const size_t dyn = (size_t)ceil_div(K, BK) * (kTileXr + kTileYr) * sizeof(float);
        auto kernel = mul ? dense_max_fwd_kernel<true, true, true> : dense_max_fwd_kernel<false, true, true>;
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn) != cudaSuccess)
          return GBMM_ERR_LAUNCH;
        kernel<<<grid, block, dyn, st>>>(a, b, out, ix, m, k, n, tm, tn, nullptr, 0);
        break;
      }
      // with scratch for a transposed copy of b the final index search reads contiguous segments
      float* b_t = nullptr;
      const int kp = (int)((K + 15) / 16 * 16);
      if (workspace && K > 0 && workspace_bytes >= gbmm_dense_forward_workspace_bytes(mode, B, M, K, N) &&
          (reinterpret_cast<uintptr_t>(workspace) & 63) == 0) {
        b_t = static_cast<float*>(workspace);
        const int64_t tk = ceil_div(kp, 32), tnn = ceil_div(N, 32), tb = B * tk * tnn;
        if (tb >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
        transpose_b_kernel<<<(unsigned)tb, 256, 0, st>>>(b, b_t, k, n, kp, (int)tk, (int)tnn);
        if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
      }
      {
        // TMA-staged kernel (GENBMM_B200_MAX_TMA=1): a's rows must be 16-byte multiples and the transposed copy of
        // b is its B operand.  Same results; measured 3.11 ms against 3.03 ms for the register-staged kernel at
        // 32 x 1024^3 (3.09 ms in an earlier form with k-major 128-byte-swizzled tiles and 64-bit loads): the packed
        // adds and 3-input maxima bound both, so it is not the default.
        const char* e = getenv("GENBMM_B200_MAX_TMA");
        CUtensorMap ma, mb;
        if ((e && e[0] == '1') && b_t && pack && K % 4 == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 &&
            make_max_map(&ma, a, B, M, K, K, BM) && make_max_map(&mb, b_t, B, N, kp, kp, BN)) {
          const size_t dyn = sizeof(MaxTmaSmem) + 1024;
          auto kernel = mul ? dense_max_tma_kernel<true> : dense_max_tma_kernel<false>;
          if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn) != cudaSuccess)
            return GBMM_ERR_LAUNCH;
          kernel<<<grid, block, dyn, st>>>(ma, mb, a, b_t, out, ix, m, k, n, tm, tn, kp, nullptr);
          break;
        }
      }
      if (!mul) {
        if (pack)
          dense_max_fwd_kernel<false, true, false><<<grid, block, 0, st>>>(a, b, out, ix, m, k, n, tm, tn, b_t, kp);
        else
          dense_max_fwd_kernel<false, false, false><<<grid, block, 0, st>>>(a, b, out, ix, m, k, n, tm, tn, b_t, kp);
      } else {
        if (pack)
          dense_max_fwd_kernel<true, true, false><<<grid, block, 0, st>>>(a, b, out, ix, m, k, n, tm, tn, b_t, kp);
        else
          dense_max_fwd_kernel<true, false, false><<<grid, block, 0, st>>>(a, b, out, ix, m, k, n, tm, tn, b_t, kp);
      }
      break;
    }
    case GBMM_MODE_SAMPLE:
      if (small_log_wanted(blocks)) {
        if (int rc = launch_small_log_fwd(a, b, out, nullptr, B, M, K, N, st)) return rc;
      } else {
        dense_log_fwd_kernel<false><<<grid, block, 0, st>>>(a, b, out, nullptr, m, k, n, tm, tn, nullptr, blocks,
                                                            nullptr, 0);
      }
      if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
      dense_sample_pick_kernel<<<grid, block, 0, st>>>(a, b, u, out, static_cast<int*>(aux), m, k, n, tm, tn);
      break;
  }
  return launch_status();
}
