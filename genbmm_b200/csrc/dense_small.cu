// Exact log-semiring kernels for small problems: 32x32 result tiles.
//
// The 128x64-tile kernels of dense_fwd.cu / dense_bwd.cu put one CTA on a whole 64x64 product (half of its
// rows padding) and leave most of the GPU idle when the batch is small: benchmark configuration 1 (32 products
// of 64x64x64) is 32 CTAs on 148 SMs, three times over (forward, grad_a, grad_b).  Here a CTA of 256 threads
// owns a 32x32 tile of its result (2x2 results per thread) and walks the reduction in chunks of 64 staged in
// shared memory, and the two gradients are ONE launch: the first CTAs of the grid take the tiles of grad_a,
// the rest the tiles of grad_b.  Same arithmetic per term as the large-tile kernels
// (matmul_cuda_kernel.cu:13-45 forward, :159-217 backward are what they restate):
//   forward   out[m,n] = log sum_k exp(a[m,k] + b[k,n] - mx) + mx, running maximum from -1e9, per chunk: exact
//             maximum first, the running sum rescaled when it grows, then one FADD, one FFMA, one MUFU.EX2 and
//             one FADD per term;
//   backward  w = exp(a[m,k] + b[k,n] - c[m,n]); grad_a[m,k] = sum_n w g[m,n]; grad_b[k,n] = sum_m w g[m,n].
// Every tile has the shape  result[i,j] = sum_r term(i, j, r)  with two shared arrays indexed [r][i] / [r][j]
// (pitch 33: conflict-free both for the transposing stores and for the reads):
//   forward  i=m j=n r=k:  X[r][i] = a[m,k] (transposed on the way in), Y[r][j] = b[k,n]
//   grad_a   i=m j=k r=n:  C[r][i] = -c[m,n] log2e, G[r][i] = g[m,n], Y[r][j] = b[k,n] (all transposed), a[m,k] in registers
//   grad_b   i=k j=n r=m:  X[r][i] = a[m,k], C[r][j] = -c[m,n] log2e, G[r][j] = g[m,n] (as stored), b[k,n] in registers
#include <cstdlib>

#include "dense.cuh"

namespace gbmm {
namespace {

constexpr int ST = 32;    // tile side
constexpr int SR = 64;    // reduction steps per chunk
constexpr int SP = 33;    // shared pitch
constexpr int SNT = 256;  // threads

__device__ __forceinline__ float ninf() { return __int_as_float(0xff800000); }

// dst[r][o] = scale * src[(o0 + o) * ld + r0 + r]  (o < ST outer indices, r < SR reduction steps; the source is
// contiguous along r): lanes run along r, so the loads are coalesced and the stores hit 32 banks.
__device__ __forceinline__ void stage_transposed(float* dst, const float* __restrict__ src, int64_t ld, int o0,
                                                 int o_ext, int r0, int r_ext, float scale, float fill) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = warp; o < ST; o += SNT / 32) {
    const bool row_ok = o0 + o < o_ext;
    const float* p = src + (int64_t)(o0 + o) * ld + r0;
#pragma unroll
    for (int r = lane; r < SR; r += 32) dst[r * SP + o] = (row_ok && r0 + r < r_ext) ? __ldg(p + r) * scale : fill;
  }
}

// dst[r][o] = scale * src[(r0 + r) * ld + o0 + o]  (the source is contiguous along o)
__device__ __forceinline__ void stage_natural(float* dst, const float* __restrict__ src, int64_t ld, int o0, int o_ext,
                                              int r0, int r_ext, float scale, float fill) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool col_ok = o0 + lane < o_ext;
#pragma unroll
  for (int r = warp; r < SR; r += SNT / 32)
    dst[r * SP + lane] = (col_ok && r0 + r < r_ext) ? __ldg(src + (int64_t)(r0 + r) * ld + o0 + lane) * scale : fill;
}

struct Micro2x2 {
  int i, j;  // first of the thread's two rows / columns inside the tile
  __device__ __forceinline__ Micro2x2() : i(2 * (threadIdx.x / 16)), j(2 * (threadIdx.x % 16)) {}
};

__device__ __forceinline__ void store2x2(float* __restrict__ dst, int64_t ld, int i0, int i_ext, int j0, int j_ext,
                                         const Micro2x2& mt, const float (&v)[2][2]) {
#pragma unroll
  for (int di = 0; di < 2; ++di) {
    const int i = i0 + mt.i + di;
    if (i >= i_ext) continue;
#pragma unroll
    for (int dj = 0; dj < 2; ++dj)
      if (j0 + mt.j + dj < j_ext) dst[(int64_t)i * ld + j0 + mt.j + dj] = v[di][dj];
  }
}

__global__ void __launch_bounds__(SNT) small_log_fwd_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                            float* __restrict__ out, float* __restrict__ maxes, int M,
                                                            int K, int N, int tiles_m, int tiles_n) {
  __shared__ float sx[SR * SP], sy[SR * SP];
  const int64_t id = blockIdx.x;
  const int n0 = (int)(id % tiles_n) * ST, m0 = (int)((id / tiles_n) % tiles_m) * ST;
  const int64_t bt = id / ((int64_t)tiles_n * tiles_m);
  const float* ab = a + bt * M * K;
  const float* bb = b + bt * K * N;
  const Micro2x2 mt;
  float mx[2][2], sum[2][2];
#pragma unroll
  for (int di = 0; di < 2; ++di)
#pragma unroll
    for (int dj = 0; dj < 2; ++dj) {
      mx[di][dj] = kFloor;
      sum[di][dj] = 0.f;
    }
  for (int k0 = 0; k0 < K; k0 += SR) {
    // padded steps carry -inf in a: ignored by the maximum, exp(-inf - m) = 0 in the sum
    stage_transposed(sx, ab, K, m0, M, k0, K, 1.f, ninf());
    stage_natural(sy, bb, N, n0, N, k0, K, 1.f, 0.f);
    __syncthreads();
    float tm[2][2];
#pragma unroll
    for (int di = 0; di < 2; ++di)
#pragma unroll
      for (int dj = 0; dj < 2; ++dj) tm[di][dj] = ninf();
#pragma unroll 8
    for (int r = 0; r < SR; ++r) {
      const float x0 = sx[r * SP + mt.i], x1 = sx[r * SP + mt.i + 1];
      const float y0 = sy[r * SP + mt.j], y1 = sy[r * SP + mt.j + 1];
      tm[0][0] = fmaxf(tm[0][0], x0 + y0);
      tm[0][1] = fmaxf(tm[0][1], x0 + y1);
      tm[1][0] = fmaxf(tm[1][0], x1 + y0);
      tm[1][1] = fmaxf(tm[1][1], x1 + y1);
    }
    float nm[2][2];
#pragma unroll
    for (int di = 0; di < 2; ++di)
#pragma unroll
      for (int dj = 0; dj < 2; ++dj) {
        if (tm[di][dj] > mx[di][dj]) {
          sum[di][dj] *= exp_sfu(mx[di][dj] - tm[di][dj]);
          mx[di][dj] = tm[di][dj];
        }
        nm[di][dj] = -mx[di][dj] * kLog2e;
      }
#pragma unroll 8
    for (int r = 0; r < SR; ++r) {
      const float x0 = sx[r * SP + mt.i], x1 = sx[r * SP + mt.i + 1];
      const float y0 = sy[r * SP + mt.j], y1 = sy[r * SP + mt.j + 1];
      sum[0][0] += ex2_approx(fmaf(x0 + y0, kLog2e, nm[0][0]));
      sum[0][1] += ex2_approx(fmaf(x0 + y1, kLog2e, nm[0][1]));
      sum[1][0] += ex2_approx(fmaf(x1 + y0, kLog2e, nm[1][0]));
      sum[1][1] += ex2_approx(fmaf(x1 + y1, kLog2e, nm[1][1]));
    }
    __syncthreads();
  }
  float v[2][2];
#pragma unroll
  for (int di = 0; di < 2; ++di)
#pragma unroll
    for (int dj = 0; dj < 2; ++dj) v[di][dj] = logf(sum[di][dj]) + mx[di][dj];
  store2x2(out + bt * M * N, N, m0, M, n0, N, mt, v);
  if (maxes) store2x2(maxes + bt * M * N, N, m0, M, n0, N, mt, mx);
}

// One launch for both gradients: CTAs [0, tiles_a) own the 32x32 tiles of grad_a (rows m, columns k, reduction
// over n), the others the tiles of grad_b (rows k, columns n, reduction over m).  Either output may be null.
__global__ void __launch_bounds__(SNT) small_log_bwd_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                            const float* __restrict__ c, const float* __restrict__ g,
                                                            float* __restrict__ grad_a, float* __restrict__ grad_b,
                                                            int M, int K, int N, int tm, int tk, int tn,
                                                            int64_t tiles_a) {
  __shared__ float s0[SR * SP], s1[SR * SP], s2[SR * SP];
  const Micro2x2 mt;
  float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, fix[2][2];
  if ((int64_t)blockIdx.x < tiles_a) {
    const int64_t id = blockIdx.x;
    const int k0 = (int)(id % tk) * ST, m0 = (int)((id / tk) % tm) * ST;
    const int64_t bt = id / ((int64_t)tk * tm);
    const float* ab = a + bt * M * K;
    const float* bb = b + bt * K * N;
    const float* cb = c + bt * M * N;
    const float* gb = g + bt * M * N;
#pragma unroll
    for (int di = 0; di < 2; ++di)
#pragma unroll
      for (int dj = 0; dj < 2; ++dj) {
        const int m = m0 + mt.i + di, k = k0 + mt.j + dj;
        fix[di][dj] = (m < M && k < K) ? __ldg(ab + (int64_t)m * K + k) : 0.f;
      }
    for (int n0 = 0; n0 < N; n0 += SR) {
      // padding: -c log2e = -inf makes the weight 0, g = 0 removes the term
      stage_transposed(s0, cb, N, m0, M, n0, N, -kLog2e, ninf());
      stage_transposed(s1, gb, N, m0, M, n0, N, 1.f, 0.f);
      stage_transposed(s2, bb, N, k0, K, n0, N, 1.f, 0.f);
      __syncthreads();
#pragma unroll 8
      for (int r = 0; r < SR; ++r) {
        const float c0 = s0[r * SP + mt.i], c1 = s0[r * SP + mt.i + 1];
        const float g0 = s1[r * SP + mt.i], g1 = s1[r * SP + mt.i + 1];
        const float b0 = s2[r * SP + mt.j], b1 = s2[r * SP + mt.j + 1];
        acc[0][0] = fmaf(ex2_approx(fmaf(fix[0][0] + b0, kLog2e, c0)), g0, acc[0][0]);
        acc[0][1] = fmaf(ex2_approx(fmaf(fix[0][1] + b1, kLog2e, c0)), g0, acc[0][1]);
        acc[1][0] = fmaf(ex2_approx(fmaf(fix[1][0] + b0, kLog2e, c1)), g1, acc[1][0]);
        acc[1][1] = fmaf(ex2_approx(fmaf(fix[1][1] + b1, kLog2e, c1)), g1, acc[1][1]);
      }
      __syncthreads();
    }
    if (grad_a) store2x2(grad_a + bt * M * K, K, m0, M, k0, K, mt, acc);
    return;
  }
  const int64_t id = blockIdx.x - tiles_a;
  const int n0 = (int)(id % tn) * ST, k0 = (int)((id / tn) % tk) * ST;
  const int64_t bt = id / ((int64_t)tn * tk);
  const float* ab = a + bt * M * K;
  const float* bb = b + bt * K * N;
  const float* cb = c + bt * M * N;
  const float* gb = g + bt * M * N;
#pragma unroll
  for (int di = 0; di < 2; ++di)
#pragma unroll
    for (int dj = 0; dj < 2; ++dj) {
      const int k = k0 + mt.i + di, n = n0 + mt.j + dj;
      fix[di][dj] = (k < K && n < N) ? __ldg(bb + (int64_t)k * N + n) : 0.f;
    }
  for (int m0 = 0; m0 < M; m0 += SR) {
    stage_natural(s0, ab, K, k0, K, m0, M, 1.f, 0.f);
    stage_natural(s1, cb, N, n0, N, m0, M, -kLog2e, ninf());
    stage_natural(s2, gb, N, n0, N, m0, M, 1.f, 0.f);
    __syncthreads();
#pragma unroll 8
    for (int r = 0; r < SR; ++r) {
      const float a0 = s0[r * SP + mt.i], a1 = s0[r * SP + mt.i + 1];
      const float c0 = s1[r * SP + mt.j], c1 = s1[r * SP + mt.j + 1];
      const float g0 = s2[r * SP + mt.j], g1 = s2[r * SP + mt.j + 1];
      acc[0][0] = fmaf(ex2_approx(fmaf(a0 + fix[0][0], kLog2e, c0)), g0, acc[0][0]);
      acc[0][1] = fmaf(ex2_approx(fmaf(a0 + fix[0][1], kLog2e, c1)), g1, acc[0][1]);
      acc[1][0] = fmaf(ex2_approx(fmaf(a1 + fix[1][0], kLog2e, c0)), g0, acc[1][0]);
      acc[1][1] = fmaf(ex2_approx(fmaf(a1 + fix[1][1], kLog2e, c1)), g1, acc[1][1]);
    }
    __syncthreads();
  }
  if (grad_b) store2x2(grad_b + bt * K * N, N, k0, K, n0, N, mt, acc);
}

}  // namespace

// The large-tile kernels fill the GPU once their grids reach two CTAs per SM; below that the 32x32 tiles of
// this file give 8 to 16 times as many CTAs for the same work.
bool small_log_wanted(int64_t large_tile_ctas) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return false;
  const char* e = getenv("GENBMM_B200_SMALL");  // 0: large tiles always, 1: small tiles always (tests)
  if (e && e[0] == '0') return false;
  if (e && e[0] == '1') return true;
  return large_tile_ctas < 2LL * sms;
}

int launch_small_log_fwd(const float* a, const float* b, float* out, float* maxes, int64_t B, int64_t M, int64_t K,
                         int64_t N, cudaStream_t st) {
  const int64_t tm = ceil_div(M, ST), tn = ceil_div(N, ST), blocks = B * tm * tn;
  if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  small_log_fwd_kernel<<<(unsigned)blocks, SNT, 0, st>>>(a, b, out, maxes, (int)M, (int)K, (int)N, (int)tm, (int)tn);
  return launch_status();
}

int launch_small_log_bwd(const float* a, const float* b, const float* c, const float* g, float* grad_a, float* grad_b,
                         int64_t B, int64_t M, int64_t K, int64_t N, cudaStream_t st) {
  const int64_t tm = ceil_div(M, ST), tk = ceil_div(K, ST), tn = ceil_div(N, ST);
  const int64_t tiles_a = grad_a ? B * tm * tk : 0, tiles_b = grad_b ? B * tk * tn : 0;
  if (tiles_a + tiles_b >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  if (tiles_a + tiles_b == 0) return GBMM_OK;
  small_log_bwd_kernel<<<(unsigned)(tiles_a + tiles_b), SNT, 0, st>>>(a, b, c, g, grad_a, grad_b, (int)M, (int)K,
                                                                     (int)N, (int)tm, (int)tk, (int)tn, tiles_a);
  return launch_status();
}

}  // namespace gbmm
