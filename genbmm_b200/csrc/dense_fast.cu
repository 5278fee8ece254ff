// Factorised log-semiring product: the fast path of logbmm.
//
// With row maxima ra[m] = max_k a[m,k] and column maxima rb[n] = max_k b[k,n],
//   c[m,n] = log sum_k exp(a[m,k] + b[k,n]) = ra[m] + rb[n] + log S[m,n],
//   S = EA @ EB,  EA[m,k] = exp(a[m,k] - ra[m]) in (0,1],  EB[k,n] = exp(b[k,n] - rb[n]) in (0,1]
// (the factorisation the reference sketches in a commented einsum, genmul.py:45-47).  All
// exponentials move out of the inner loop: S is an ordinary fp32 matrix product, one FFMA per
// (m,k,n) triple instead of one MUFU.EX2, which lifts the bound of the kernel from the SFU
// (16/clk/SM) to the FP32 pipe (128/clk/SM).  The gradients factorise the same way, with
// w = exp(a+b-c) = EA[m,k] * EB[k,n] / S[m,n] and G' = g / S = g * exp(ra + rb - c):
//   grad_a = EA (.) (G' @ EB^T),      grad_b = EB (.) (EA^T @ G').
//
// Guard.  The shift ra[m] + rb[n] is an upper bound of max_k(a+b), not the maximum itself.
// When the true maximum lies far below it S underflows and the factorisation loses the
// result.  Every 128x128 result tile therefore records a flag if any of its S is below 2^-90
// (or not finite), or if ra+rb is below the reference's -1e9 floor; flagged tiles are
// recomputed by the exact SFU kernels (dense_fwd.cu / dense_bwd.cu), forward and backward,
// and contribute nothing to the factorised gradients (their G' is zero).  A term that matters
// to an unflagged result has EA*EB >= 2^-90 * 2^-24, far above the underflow threshold of
// either factor, so unflagged results carry ordinary fp32 rounding only.
//
// Scratch.  The exponentiated operands are written once by small HBM-bound kernels into
// caller-provided scratch, in the orientation the product wants (reduction index outermost,
// row pitch padded to 4 floats), and fetched by TMA (cp.async.bulk.tensor, zero-filled at the
// edges) into a 4-stage shared-memory ring; one elected thread issues the copies, all threads
// wait on the stage's mbarrier with a bounded wait.
#include "dense.cuh"
#include "tma.cuh"

namespace gbmm {
namespace {

constexpr int GI = 128, GJ = 128, GK = 32, GS = 3, GNT = 256;
constexpr float kTiny = 8.0779356694631609e-28f;  // 2^-90

__host__ __device__ inline int64_t pad4(int64_t x) { return (x + 3) & ~int64_t(3); }
__host__ __device__ inline int64_t pad64(int64_t x) { return (x + 63) & ~int64_t(63); }

// ------------------------------------------------------------------ row / column maxima
// ra[b,m] = max_k a[b,m,k]; one warp per row.  A row with no finite-or-+inf entry (all -inf,
// or NaN-only) gets 0 so that EA becomes 0 rather than NaN and the tile is flagged.
__global__ void __launch_bounds__(256) rowmax_kernel(const float* __restrict__ a, float* __restrict__ ra,
                                                     int64_t rows, int K) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;
  if (row >= rows) return;
  const float* p = a + row * K;
  float m = __int_as_float(0xff800000);
  for (int k = lane; k < K; k += 32) m = fmaxf(m, __ldg(p + k));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) ra[row] = (m == __int_as_float(0xff800000)) ? 0.f : m;
}

// rb[b,n] = max_k b[b,k,n]; CTA = 32 columns x 8 k-slices, reduced through shared memory.
__global__ void __launch_bounds__(256) colmax_kernel(const float* __restrict__ b, float* __restrict__ rb, int K,
                                                     int N, int tiles_n) {
  __shared__ float part[8][33];
  const int lane = threadIdx.x % 32, slice = threadIdx.x / 32;
  const int bt = blockIdx.x / tiles_n;
  const int n = (blockIdx.x % tiles_n) * 32 + lane;
  float m = __int_as_float(0xff800000);
  if (n < N) {
    const float* p = b + (int64_t)bt * K * N + n;
    for (int k = slice; k < K; k += 8) m = fmaxf(m, __ldg(p + (int64_t)k * N));
  }
  part[slice][lane] = m;
  __syncthreads();
  if (slice == 0 && n < N) {
#pragma unroll
    for (int s = 1; s < 8; ++s) m = fmaxf(m, part[s][lane]);
    rb[(int64_t)bt * N + n] = (m == __int_as_float(0xff800000)) ? 0.f : m;
  }
}

// ------------------------------------------------------------------ exponentiated operands
// Reads a (batch, R, C) tensor in 32x32 tiles, applies the transform and writes it in the
// same orientation (dst_n, pitch pad4(C)) and/or transposed (dst_t: (batch, C, R), pitch
// pad4(R)); either destination may be null.
//   KIND 0: exp(src[r,c] - shift[r])      (a with its row maxima)
//   KIND 1: exp(src[r,c] - shift[c])      (b with its column maxima)
//   KIND 2: g[r,c] * exp(ra[r] + rb[c] - src[r,c]), zero inside flagged tiles   (G' = g / S)
template <int KIND>
__global__ void __launch_bounds__(256) transform_kernel(const float* __restrict__ src,
                                                        const float* __restrict__ shift,
                                                        const float* __restrict__ shift2,
                                                        const float* __restrict__ g,
                                                        const int* __restrict__ flags, float* __restrict__ dst_n,
                                                        float* __restrict__ dst_t, int R, int C, int tiles_r,
                                                        int tiles_c) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
  const int64_t id = blockIdx.x;
  const int c0 = (int)(id % tiles_c) * 32, r0 = (int)((id / tiles_c) % tiles_r) * 32;
  const int64_t bt = id / ((int64_t)tiles_c * tiles_r);
  const float* sb = src + bt * R * C;
  const int64_t pc = pad4(C), pr = pad4(R);
  bool dead = false;
  if (KIND == 2) dead = __ldg(flags + (bt * ((R + 127) / 128) + r0 / 128) * ((C + 127) / 128) + c0 / 128) != 0;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int r = r0 + ty + q * 8, c = c0 + tx;
    float v = 0.f;
    if (r < R && c < C) {
      const float x = __ldg(sb + (int64_t)r * C + c);
      if (KIND == 0) v = exp_sfu(x - __ldg(shift + bt * R + r));
      if (KIND == 1) v = exp_sfu(x - __ldg(shift + bt * C + c));
      if (KIND == 2)
        v = dead ? 0.f
                 : __ldg(g + bt * R * C + (int64_t)r * C + c) *
                       exp_sfu((__ldg(shift + bt * R + r) + __ldg(shift2 + bt * C + c)) - x);
      if (dst_n) dst_n[(bt * R + r) * pc + c] = v;
    }
    tile[ty + q * 8][tx] = v;
  }
  if (dst_t) {
    __syncthreads();
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int c = c0 + ty + q * 8, r = r0 + tx;
      if (c < C && r < R) dst_t[(bt * C + c) * pr + r] = tile[tx][ty + q * 8];
    }
  }
}

// The same transforms on 64x64 tiles with 128-bit loads and stores, for tensors whose rows are a
// multiple of 4 floats and 16-byte aligned (the common case); about twice the bandwidth of the
// scalar kernel above.  Flags are per 128x128 tile, so a 64x64 tile has one flag.
template <int KIND>
__global__ void __launch_bounds__(256) transform4_kernel(const float* __restrict__ src,
                                                         const float* __restrict__ shift,
                                                         const float* __restrict__ shift2,
                                                         const float* __restrict__ g,
                                                         const int* __restrict__ flags, float* __restrict__ dst_n,
                                                         float* __restrict__ dst_t, int R, int C, int tiles_r,
                                                         int tiles_c) {
  __shared__ float tile[64][65];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int64_t id = blockIdx.x;
  const int c0 = (int)(id % tiles_c) * 64, r0 = (int)((id / tiles_c) % tiles_r) * 64;
  const int64_t bt = id / ((int64_t)tiles_c * tiles_r);
  const float* sb = src + bt * R * C;
  const int64_t pc = pad4(C), pr = pad4(R);
  bool dead = false;
  if (KIND == 2) dead = __ldg(flags + (bt * ((R + 127) / 128) + r0 / 128) * ((C + 127) / 128) + c0 / 128) != 0;
  const int c = c0 + tx * 4;
  float4 cs = make_float4(0.f, 0.f, 0.f, 0.f);  // per-column shifts of this thread's 4 columns
  if (c < C) {
    if (KIND == 1) cs = __ldg(reinterpret_cast<const float4*>(shift + bt * C + c));
    if (KIND == 2) cs = __ldg(reinterpret_cast<const float4*>(shift2 + bt * C + c));
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int rl = ty + q * 16, r = r0 + rl;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < R && c < C) {  // C % 4 == 0: the whole group is inside
      const float4 x = __ldg(reinterpret_cast<const float4*>(sb + (int64_t)r * C + c));
      if (KIND == 0) {
        const float sh = __ldg(shift + bt * R + r);
        v = make_float4(exp_sfu(x.x - sh), exp_sfu(x.y - sh), exp_sfu(x.z - sh), exp_sfu(x.w - sh));
      }
      if (KIND == 1) v = make_float4(exp_sfu(x.x - cs.x), exp_sfu(x.y - cs.y), exp_sfu(x.z - cs.z), exp_sfu(x.w - cs.w));
      if (KIND == 2 && !dead) {
        const float sh = __ldg(shift + bt * R + r);
        const float4 gv = __ldg(reinterpret_cast<const float4*>(g + bt * R * C + (int64_t)r * C + c));
        v = make_float4(gv.x * exp_sfu((sh + cs.x) - x.x), gv.y * exp_sfu((sh + cs.y) - x.y),
                        gv.z * exp_sfu((sh + cs.z) - x.z), gv.w * exp_sfu((sh + cs.w) - x.w));
      }
      if (dst_n) *reinterpret_cast<float4*>(dst_n + (bt * R + r) * pc + c) = v;
    }
    tile[rl][tx * 4 + 0] = v.x;
    tile[rl][tx * 4 + 1] = v.y;
    tile[rl][tx * 4 + 2] = v.z;
    tile[rl][tx * 4 + 3] = v.w;
  }
  if (dst_t) {
    __syncthreads();
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int cl = ty + q * 16, cc = c0 + cl, r = r0 + tx * 4;
      if (cc < C && r < R) {  // pad4(R) pitch: a group that straddles R still lands in the row's padding
        const float4 v = make_float4(tile[tx * 4 + 0][cl], tile[tx * 4 + 1][cl], tile[tx * 4 + 2][cl],
                                     tile[tx * 4 + 3][cl]);
        *reinterpret_cast<float4*>(dst_t + (bt * C + cc) * pr + r) = v;
      }
    }
  }
}

// ------------------------------------------------------------------ TMA-fed FP32 product
// C[i,j] = sum_r X[r,i] * Y[r,j] for X:(batch,R,I) and Y:(batch,R,J), both with the reduction
// index outermost.  CTA = 256 threads, 128x128 result tile, 8x8 per thread, reduction tiles of
// 16 rows in a 4-stage ring.  PACKED uses sm_100's two-wide FP32 FMA (fma.rn.f32x2): half the
// issue slots per FMA (measured 0.644 ms against 0.738 ms for the scalar form on the
// 16x1024^3 product); the scalar form is kept for comparison.
struct alignas(128) GemmSmem {
  float x[GS][GK * GI];
  float y[GS][GK * GJ];
  uint64_t full[GS];
};

enum { EPI_LOG = 0, EPI_GRAD = 1 };

struct EpiParams {
  float* out;          // EPI_LOG: c (batch,I,J);  EPI_GRAD: the gradient (batch,I,J)
  const float* row_v;  // EPI_LOG: ra (batch,I);   EPI_GRAD: shift by row (or null)
  const float* col_v;  // EPI_LOG: rb (batch,J);   EPI_GRAD: shift by column (or null)
  const float* src;    // EPI_GRAD: the operand whose exponential multiplies the sum (batch,I,J)
  int* flags;          // EPI_LOG: one flag per CTA
  int* error;          // set to 1 if a bounded wait gave up
};

__device__ __forceinline__ void ffma2(unsigned long long& d, unsigned long long a, unsigned long long b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

template <int EPI, bool PACKED>
__global__ void __launch_bounds__(GNT, 2) sgemm_tn_kernel(const __grid_constant__ CUtensorMap mx,
                                                          const __grid_constant__ CUtensorMap my, EpiParams ep,
                                                          int R, int I, int J, int tiles_i, int tiles_j) {
  extern __shared__ unsigned char smem_raw[];
  GemmSmem& sm = *reinterpret_cast<GemmSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int64_t id = blockIdx.x;
  const int j0 = (int)(id % tiles_j) * GJ, i0 = (int)((id / tiles_j) % tiles_i) * GI;
  const int bt = (int)(id / ((int64_t)tiles_j * tiles_i));
  const int nt = (R + GK - 1) / GK;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < GS; ++s) mbar_init(&sm.full[s], 1);
    fence_barrier_init();
  }
  __syncthreads();
  auto issue = [&](int stage, int tile) {
    mbar_arrive_expect_tx(&sm.full[stage], (GI + GJ) * GK * sizeof(float));
    tma_load_3d(sm.x[stage], &mx, &sm.full[stage], i0, tile * GK, bt);
    tma_load_3d(sm.y[stage], &my, &sm.full[stage], j0, tile * GK, bt);
  };
  if (tid == 0)
    for (int s = 0; s < GS && s < nt; ++s) issue(s, s);

  float acc[8][8];
  unsigned long long acc2[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) acc2[i][j] = 0ull;
  }

  bool fail = false;
  int t = 0;
  for (; t < nt; ++t) {
    const int s = t % GS;
    if (!mbar_wait_bounded(&sm.full[s], (t / GS) & 1)) fail = true;
    const float* xs = sm.x[s];
    const float* ys = sm.y[s];
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      const float4 xa = *reinterpret_cast<const float4*>(xs + kk * GI + ty * 4);
      const float4 xb = *reinterpret_cast<const float4*>(xs + kk * GI + 64 + ty * 4);
      const float x[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
      if (PACKED) {
        // two FMAs per instruction (fma.rn.f32x2): results paired along j, x broadcast to both halves
        const ulonglong2 ya = *reinterpret_cast<const ulonglong2*>(ys + kk * GJ + tx * 4);
        const ulonglong2 yb = *reinterpret_cast<const ulonglong2*>(ys + kk * GJ + 64 + tx * 4);
        const unsigned long long y2[4] = {ya.x, ya.y, yb.x, yb.y};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const unsigned long long xx = pack2(x[i], x[i]);
#pragma unroll
          for (int j = 0; j < 4; ++j) ffma2(acc2[i][j], xx, y2[j]);
        }
      } else {
        const float4 ya = *reinterpret_cast<const float4*>(ys + kk * GJ + tx * 4);
        const float4 yb = *reinterpret_cast<const float4*>(ys + kk * GJ + 64 + tx * 4);
        const float y[8] = {ya.x, ya.y, ya.z, ya.w, yb.x, yb.y, yb.z, yb.w};
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(x[i], y[j], acc[i][j]);
      }
    }
    // everyone is done with stage s (and agrees on whether a wait gave up) before it is refilled
    if (__syncthreads_or(fail)) {
      fail = true;
      break;
    }
    if (tid == 0 && t + GS < nt) issue(s, t + GS);
  }
  if (fail) {
    // give the copies still in flight a bounded chance to land before the CTA's shared memory
    // is released, record the failure, write no result
    for (int u = t + 1; u < nt && u < t + GS; ++u) mbar_wait_bounded(&sm.full[u % GS], (u / GS) & 1);
    // the fix-up kernel that follows sees the word and turns the whole result into NaN; the tile's guard
    // flag is still written so that nothing downstream ever reads a stale one
    if (tid == 0) {
      atomicExch(ep.error, 1);
      if (EPI == EPI_LOG) ep.flags[blockIdx.x] = 0;
    }
    return;
  }

  if (PACKED) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) unpack2(acc2[i][j], acc[i][2 * j], acc[i][2 * j + 1]);
  }
  bool bad = false;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int ii = i0 + (i < 4 ? 0 : 64) + ty * 4 + (i & 3);
    if (ii >= I) continue;
    const float rv = ep.row_v ? __ldg(ep.row_v + (int64_t)bt * I + ii) : 0.f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int jb = j0 + h * 64 + tx * 4;
      float v[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int jj = jb + q;
        const float s = acc[i][h * 4 + q];
        v[q] = 0.f;
        if (jj < J) {
          const float cv = ep.col_v ? __ldg(ep.col_v + (int64_t)bt * J + jj) : 0.f;
          if (EPI == EPI_LOG) {
            const float shift = rv + cv;
            v[q] = logf(s) + shift;
            bad |= !(s >= kTiny) || !(s <= 3.0e38f) || (shift < kFloor);
          } else {
            const float x = __ldg(ep.src + ((int64_t)bt * I + ii) * J + jj);
            v[q] = exp_sfu(x - (rv + cv)) * s;
          }
        }
      }
      float* op = ep.out + ((int64_t)bt * I + ii) * J + jb;
      if ((J % 4 == 0) && jb + 3 < J && ((reinterpret_cast<uintptr_t>(op) & 15) == 0)) {
        *reinterpret_cast<float4*>(op) = make_float4(v[0], v[1], v[2], v[3]);
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q)
          if (jb + q < J) op[q] = v[q];
      }
    }
  }
  if (EPI == EPI_LOG) {
    const int any = __syncthreads_or(bad);
    if (tid == 0) ep.flags[blockIdx.x] = any;
  }
}

template <int EPI>
int launch_gemm(const float* x, int64_t x_pitch, const float* y, int64_t y_pitch, const EpiParams& ep, int64_t B,
                int64_t R, int64_t I, int64_t J, cudaStream_t st, int slot) {
  CUtensorMap mx, my;
  if (!make_map_3d(&mx, x, B, R, I, x_pitch, GK, GI) || !make_map_3d(&my, y, B, R, J, y_pitch, GK, GJ))
    return GBMM_ERR_LAUNCH;
  const int64_t ti = ceil_div(I, GI), tj = ceil_div(J, GJ), blocks = B * ti * tj;
  if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  const size_t smem = sizeof(GemmSmem) + 128;
  auto kernel = sgemm_tn_kernel<EPI, true>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return GBMM_ERR_LAUNCH;
  const bool timed = profile_begin(slot, st);
  kernel<<<(unsigned)blocks, GNT, smem, st>>>(mx, my, ep, (int)R, (int)I, (int)J, (int)ti, (int)tj);
  if (timed) profile_end(slot, st);
  return launch_status();
}

template <int KIND>
int launch_transform(const float* src, const float* shift, const float* shift2, const float* g, const int* flags,
                     float* dst_n, float* dst_t, int64_t B, int64_t R, int64_t C, cudaStream_t st) {
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = (C % 4 == 0) && al16(src) && (!g || al16(g)) && (KIND == 0 || al16(KIND == 1 ? shift : shift2)) &&
                   (!dst_n || al16(dst_n)) && (!dst_t || al16(dst_t));
  if (vec) {
    const int64_t tr = ceil_div(R, 64), tcn = ceil_div(C, 64), blocks = B * tr * tcn;
    if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
    transform4_kernel<KIND><<<(unsigned)blocks, 256, 0, st>>>(src, shift, shift2, g, flags, dst_n, dst_t, (int)R,
                                                             (int)C, (int)tr, (int)tcn);
    return launch_status();
  }
  const int64_t tr = ceil_div(R, 32), tcn = ceil_div(C, 32), blocks = B * tr * tcn;
  if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  transform_kernel<KIND><<<(unsigned)blocks, 256, 0, st>>>(src, shift, shift2, g, flags, dst_n, dst_t, (int)R,
                                                          (int)C, (int)tr, (int)tcn);
  return launch_status();
}

// carve `floats` floats (rounded up to 256 bytes) from the workspace
float* carve(float*& cursor, int64_t floats) {
  float* p = cursor;
  cursor += pad64(floats);
  return p;
}

bool bad_dims(int64_t B, int64_t M, int64_t K, int64_t N) {
  return B < 0 || M < 0 || K < 0 || N < 0;
}
bool big_dims(int64_t M, int64_t K, int64_t N) {
  const int64_t lim = (1LL << 31) - 256;
  return M >= lim || K >= lim || N >= lim;
}

}  // namespace
}  // namespace gbmm

using namespace gbmm;

namespace gbmm {
int rowmax_only(const float* a, float* rowmax, int64_t B, int64_t M, int64_t K, cudaStream_t st) {
  rowmax_kernel<<<(unsigned)ceil_div(B * M, 8), 256, 0, st>>>(a, rowmax, B * M, (int)K);
  return launch_status();
}

// rowmax:(B,M) = max_k a, colmax:(B,N) = max_k b (0 for rows/columns without a finite entry)
int launch_rowcol_max(const float* a, const float* b, float* rowmax, float* colmax, int64_t B, int64_t M, int64_t K,
                      int64_t N, cudaStream_t st) {
  rowmax_kernel<<<(unsigned)ceil_div(B * M, 8), 256, 0, st>>>(a, rowmax, B * M, (int)K);
  const int64_t tn = ceil_div(N, 32);
  colmax_kernel<<<(unsigned)(B * tn), 256, 0, st>>>(b, colmax, (int)K, (int)N, (int)tn);
  return launch_status();
}
}  // namespace gbmm

extern "C" int64_t gbmm_logbmm_workspace_bytes(int backward, int64_t B, int64_t M, int64_t K, int64_t N) {
  if (bad_dims(B, M, K, N)) return -1;
  int64_t floats = 64;  // error word
  if (!backward)
    floats += pad64(B * K * pad4(M)) + pad64(B * K * pad4(N));
  else
    floats += pad64(B * M * pad4(K)) + pad64(B * N * pad4(K)) + pad64(B * M * pad4(N)) + pad64(B * N * pad4(M));
  return floats * (int64_t)sizeof(float);
}

extern "C" int64_t gbmm_logbmm_flag_count(int64_t B, int64_t M, int64_t N) {
  if (B < 0 || M < 0 || N < 0) return -1;
  return B * ceil_div(M, GI) * ceil_div(N, GJ);
}

extern "C" int gbmm_logbmm_forward_f32(const float* a, const float* b, float* out, float* rowmax, float* colmax,
                                       int32_t* flags, void* workspace, int64_t workspace_bytes, int64_t B,
                                       int64_t M, int64_t K, int64_t N, void* stream) {
  if (bad_dims(B, M, K, N)) return GBMM_ERR_INVALID_ARG;
  if (B == 0 || M == 0 || N == 0) return GBMM_OK;
  if (K == 0) return GBMM_ERR_UNSUPPORTED;  // empty reduction: use gbmm_dense_forward_f32
  if (!a || !b || !out || !rowmax || !colmax || !flags || !workspace) return GBMM_ERR_INVALID_ARG;
  if (big_dims(M, K, N)) return GBMM_ERR_UNSUPPORTED;
  if (workspace_bytes < gbmm_logbmm_workspace_bytes(0, B, M, K, N)) return GBMM_ERR_INVALID_ARG;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return GBMM_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* cur = static_cast<float*>(workspace);
  int* error = reinterpret_cast<int*>(carve(cur, 64));
  float* eat = carve(cur, B * K * pad4(M));  // EA^T : (B, K, pad4(M))
  float* eb = carve(cur, B * K * pad4(N));   // EB   : (B, K, pad4(N))
  if (cudaMemsetAsync(error, 0, sizeof(int), st) != cudaSuccess) return GBMM_ERR_LAUNCH;

  rowmax_kernel<<<(unsigned)ceil_div(B * M, 8), 256, 0, st>>>(a, rowmax, B * M, (int)K);
  const int64_t tn = ceil_div(N, 32);
  colmax_kernel<<<(unsigned)(B * tn), 256, 0, st>>>(b, colmax, (int)K, (int)N, (int)tn);
  if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
  int rc = launch_transform<0>(a, rowmax, nullptr, nullptr, nullptr, nullptr, eat, B, M, K, st);
  if (rc != GBMM_OK) return rc;
  rc = launch_transform<1>(b, colmax, nullptr, nullptr, nullptr, eb, nullptr, B, K, N, st);
  if (rc != GBMM_OK) return rc;
  EpiParams ep{out, rowmax, colmax, nullptr, flags, error};
  rc = launch_gemm<EPI_LOG>(eat, pad4(M), eb, pad4(N), ep, B, K, M, N, st, 0);
  if (rc != GBMM_OK) return rc;
  return launch_log_fwd_flagged(a, b, out, flags, B, M, K, N, st, error);
}

extern "C" int gbmm_logbmm_backward_f32(const float* a, const float* b, const float* grad_out, const float* out,
                                        const float* rowmax, const float* colmax, const int32_t* flags,
                                        float* grad_a, float* grad_b, void* workspace, int64_t workspace_bytes,
                                        int64_t B, int64_t M, int64_t K, int64_t N, void* stream) {
  if (bad_dims(B, M, K, N)) return GBMM_ERR_INVALID_ARG;
  if (B == 0 || K == 0) return GBMM_OK;
  if (M == 0 || N == 0) return GBMM_ERR_UNSUPPORTED;  // use gbmm_dense_backward_f32
  if (!a || !b || !grad_out || !out || !rowmax || !colmax || !flags || !workspace) return GBMM_ERR_INVALID_ARG;
  if (big_dims(M, K, N)) return GBMM_ERR_UNSUPPORTED;
  if (workspace_bytes < gbmm_logbmm_workspace_bytes(1, B, M, K, N)) return GBMM_ERR_INVALID_ARG;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return GBMM_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* cur = static_cast<float*>(workspace);
  int* error = reinterpret_cast<int*>(carve(cur, 64));
  float* ea = carve(cur, B * M * pad4(K));   // EA   : (B, M, pad4(K))
  float* ebt = carve(cur, B * N * pad4(K));  // EB^T : (B, N, pad4(K))
  float* gp = carve(cur, B * M * pad4(N));   // G'   : (B, M, pad4(N))
  float* gt = carve(cur, B * N * pad4(M));   // G'^T : (B, N, pad4(M))
  if (cudaMemsetAsync(error, 0, sizeof(int), st) != cudaSuccess) return GBMM_ERR_LAUNCH;

  int rc = launch_transform<0>(a, rowmax, nullptr, nullptr, nullptr, ea, nullptr, B, M, K, st);
  if (rc != GBMM_OK) return rc;
  rc = launch_transform<1>(b, colmax, nullptr, nullptr, nullptr, nullptr, ebt, B, K, N, st);
  if (rc != GBMM_OK) return rc;
  rc = launch_transform<2>(out, rowmax, colmax, grad_out, flags, gp, gt, B, M, N, st);
  if (rc != GBMM_OK) return rc;
  if (grad_a) {
    // grad_a[m,k] = EA[m,k] * sum_n G'[m,n] EB[k,n]:  X = G'^T (r=n, i=m),  Y = EB^T (r=n, j=k)
    EpiParams ep{grad_a, rowmax, nullptr, a, nullptr, error};
    rc = launch_gemm<EPI_GRAD>(gt, pad4(M), ebt, pad4(K), ep, B, N, M, K, st, 1);
    if (rc != GBMM_OK) return rc;
  }
  if (grad_b) {
    // grad_b[k,n] = EB[k,n] * sum_m EA[m,k] G'[m,n]:  X = EA (r=m, i=k),  Y = G' (r=m, j=n)
    EpiParams ep{grad_b, nullptr, colmax, b, nullptr, error};
    rc = launch_gemm<EPI_GRAD>(ea, pad4(K), gp, pad4(N), ep, B, M, K, N, st, 2);
    if (rc != GBMM_OK) return rc;
  }
  return launch_log_bwd_flagged(a, b, out, grad_out, grad_a, grad_b, flags, B, M, K, N, st, error);
}

// Blocks until the stream's work is done and returns GBMM_ERR_LAUNCH if a kernel of the fast
// path recorded that a bounded wait gave up (its outputs are then invalid), GBMM_OK otherwise.
extern "C" int gbmm_logbmm_check(const void* workspace, void* stream) {
  int err = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(&err, workspace, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess)
    return GBMM_ERR_LAUNCH;
  if (cudaStreamSynchronize(st) != cudaSuccess) return GBMM_ERR_LAUNCH;
  return err ? GBMM_ERR_LAUNCH : GBMM_OK;
}

// ------------------------------------------------------------------ forward without allocation
// Some callers may not allocate device memory at the point where they need a product: code
// running inside a memory-pool region whose owner forbids new reservations, a real-time loop
// that must not touch the driver's allocator because its latency is unbounded, or a host
// framework that hands the operator fixed input/output buffers and nothing else.  For them the
// scratch of the factorised forward lives in this fixed device array instead of a
// caller-provided workspace.  It costs kNoAllocBytes of device memory on every GPU that loads
// the library, until the process exits, so it is kept small; problems that need more are
// rejected.
constexpr int64_t kNoAllocBytes = 32LL << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

namespace {
constexpr int kMaxDevices = 64;
void* g_noalloc_ptr[kMaxDevices] = {nullptr};

// Device address of g_noalloc_scratch on the current device.  In host code the array's name
// is only a handle for the runtime, not an address a kernel can use, so the address is asked
// for once per device (with that device current) and remembered.
int noalloc_scratch(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return GBMM_ERR_DEVICE;
  void* p = g_noalloc_ptr[dev];
  if (!p) {
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) return GBMM_ERR_DEVICE;
    g_noalloc_ptr[dev] = p;
  }
  *out = p;
  return GBMM_OK;
}
}  // namespace

extern "C" int64_t gbmm_logbmm_forward_noalloc_max_bytes(void) { return kNoAllocBytes; }

extern "C" int64_t gbmm_logbmm_forward_noalloc_need_bytes(int64_t B, int64_t M, int64_t K, int64_t N) {
  if (bad_dims(B, M, K, N)) return -1;
  const int64_t floats = 64 + pad64(B * K * pad4(M)) + pad64(B * K * pad4(N)) + pad64(B * M) + pad64(B * N) +
                         pad64(B * ceil_div(M, GI) * ceil_div(N, GJ));
  return floats * (int64_t)sizeof(float);
}

extern "C" int gbmm_logbmm_forward_noalloc_f32(const float* a, const float* b, float* out, int64_t B, int64_t M,
                                               int64_t K, int64_t N, void* stream) {
  if (bad_dims(B, M, K, N)) return GBMM_ERR_INVALID_ARG;
  if (B == 0 || M == 0 || N == 0) return GBMM_OK;
  if (K == 0) return GBMM_ERR_UNSUPPORTED;
  if (!a || !b || !out) return GBMM_ERR_INVALID_ARG;
  if (big_dims(M, K, N)) return GBMM_ERR_UNSUPPORTED;
  if (gbmm_logbmm_forward_noalloc_need_bytes(B, M, K, N) > kNoAllocBytes) return GBMM_ERR_SCRATCH_LIMIT;
  void* base = nullptr;
  int rc = noalloc_scratch(&base);
  if (rc != GBMM_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* cur = static_cast<float*>(base);
  int* error = reinterpret_cast<int*>(carve(cur, 64));
  float* eat = carve(cur, B * K * pad4(M));
  float* eb = carve(cur, B * K * pad4(N));
  float* rowmax = carve(cur, B * M);
  float* colmax = carve(cur, B * N);
  int* flags = reinterpret_cast<int*>(carve(cur, B * ceil_div(M, GI) * ceil_div(N, GJ)));
  // the array keeps whatever the previous call left: the error word is the one thing that
  // must start at zero; everything else is fully rewritten before it is read
  if (cudaMemsetAsync(error, 0, sizeof(int), st) != cudaSuccess) return GBMM_ERR_LAUNCH;

  rowmax_kernel<<<(unsigned)ceil_div(B * M, 8), 256, 0, st>>>(a, rowmax, B * M, (int)K);
  const int64_t tn = ceil_div(N, 32);
  colmax_kernel<<<(unsigned)(B * tn), 256, 0, st>>>(b, colmax, (int)K, (int)N, (int)tn);
  if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
  rc = launch_transform<0>(a, rowmax, nullptr, nullptr, nullptr, nullptr, eat, B, M, K, st);
  if (rc != GBMM_OK) return rc;
  rc = launch_transform<1>(b, colmax, nullptr, nullptr, nullptr, eb, nullptr, B, K, N, st);
  if (rc != GBMM_OK) return rc;

  CUtensorMap mx, my;
  if (!make_map_3d(&mx, eat, B, K, M, pad4(M), GK, GI) || !make_map_3d(&my, eb, B, K, N, pad4(N), GK, GJ))
    return GBMM_ERR_LAUNCH;
  const int64_t ti = ceil_div(M, GI), tj = ceil_div(N, GJ), blocks = B * ti * tj;
  if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  const size_t smem = sizeof(GemmSmem) + 128;
  if (cudaFuncSetAttribute(sgemm_tn_kernel<EPI_LOG, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem) != cudaSuccess)
    return GBMM_ERR_LAUNCH;
  EpiParams ep{out, rowmax, colmax, nullptr, flags, error};
  sgemm_tn_kernel<EPI_LOG, true><<<(unsigned)blocks, GNT, smem, st>>>(mx, my, ep, (int)K, (int)M, (int)N,
                                                                      (int)ti, (int)tj);
  if (cudaGetLastError() != cudaSuccess) return GBMM_ERR_LAUNCH;
  return launch_log_fwd_flagged(a, b, out, flags, B, M, K, N, st, error);
}

extern "C" int gbmm_logbmm_forward_noalloc_check(void* stream) {
  void* base = nullptr;
  int rc = noalloc_scratch(&base);
  if (rc != GBMM_OK) return rc;
  return gbmm_logbmm_check(base, stream);  // the error word is the first word of the array
}
