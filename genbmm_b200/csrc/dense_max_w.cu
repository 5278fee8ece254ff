// Max-plus / prod-max forward for reductions of up to 288 steps (K a multiple of 4): the whole reduction of a
// 64 x 32 block of the result stays in shared memory, and the warps of a CTA do not wait for one another.
//
// This is the structure of the banded max kernel (band_max.cu, band_max_w_kernel) on dense operands.  Every thread
// requests all 16-step tiles of its block at once — 16-byte cp.async copies of a's rows, 4-byte copies of b's
// (b is (K, N): four consecutive steps of a column are N floats apart, and reading it this way saves the
// transposed copy the long-reduction kernel needs) — and makes one deferred arrival per tile on that tile's
// mbarrier; a warp then walks the tiles with its 16 x 16 sub-block (4 x 2 results per thread), waiting only for
// data.  Layout of a tile: [quad of steps][row][4 steps], one 128-bit load per row and quad, lanes on
// consecutive 16-byte cells; the two halves of a loaded quad are the (k, k+1) pairs of the packed add / multiply.
// The first 16-step tile that reached a result's maximum is remembered in a byte and searched at the end, in
// shared memory, for the first k whose term equals the maximum — `if (v > m) { m = v; ind = i; }` from m = -1e9,
// ind = -1 (matmul_cuda_kernel.cu:60-73, :137-150) bit for bit: lowest k on ties, -1 / -1e9 when nothing exceeds
// -1e9, NaN terms never selected, the stored value is the winning term itself (sign of a zero preserved).
// Steps beyond K and rows / columns beyond the matrices are copied from four NaNs in device memory: a NaN term is
// ignored by the maximum under both semirings.
// 80 registers and 6 KB of tiles per 16 steps: three CTAs (24 warps) per SM up to 176 steps.  Against the kernel
// it replaces for K <= 128 (128 x 64 blocks in lockstep, tiles resident as well): 99 -> 79 us at 256 x 128^3;
// at 32 x 1024 x K x 1024: 0.57 against 0.65 ms (K = 128), 1.04 against 1.20 ms (K = 256), and 1.99 against 1.57
// ms at K = 416, where only one CTA fits an SM — hence the limit of 288 steps.
// GENBMM_B200_MAX_SHORT=block keeps the lockstep kernels.
#include <cstdlib>

#include "dense.cuh"
#include "tma.cuh"

namespace gbmm {
namespace {

constexpr int WB = 64, WC = 32, WNT = 256, BK = 16;
constexpr int WTX = 4 * WB * 4 + 4, WTY = 4 * WC * 4 + 4;   // floats per tile of a / of b; + 4: see the search
constexpr int kMaxTiles = 18;   // two CTAs per SM; with one (up to 26 tiles fit) the lockstep kernel is faster

// four NaNs: the source of every copy that has nothing to copy
__device__ __align__(16) unsigned g_nan4[4] = {0x7fc00000u, 0x7fc00000u, 0x7fc00000u, 0x7fc00000u};
// set when a warp's bounded wait for its own copies ran out; that warp's results are then NaN / -1
__device__ int g_gave_up = 0;

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
__device__ __forceinline__ void cp_async16(float* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(float* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
// one arrival on `bar` once every cp.async this thread has issued so far has landed (counted in the barrier's
// initial count: .noinc)
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <bool MUL>
__global__ void __launch_bounds__(WNT, 3) dense_max_w_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                             float* __restrict__ out, int* __restrict__ idx, int M,
                                                             int K, int N, int tiles_m, int tiles_n,
                                                             int* __restrict__ error) {
  extern __shared__ __align__(16) float smem_dyn[];
  __shared__ __align__(8) uint64_t landed[kMaxTiles];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ty = lane >> 3, tx = lane & 7;
  const int64_t id = blockIdx.x;
  const int c0 = (int)(id % tiles_n) * WC, r0 = (int)((id / tiles_n) % tiles_m) * WB;
  const int64_t bt = id / ((int64_t)tiles_n * tiles_m);
  const int nt = (K + BK - 1) / BK;
  float* sx = smem_dyn;
  float* sy = smem_dyn + (size_t)nt * WTX;
  const float* ab = a + bt * M * K;
  const float* bb = b + bt * K * N;

  if (tid == 0) {
    for (int t = 0; t < nt; ++t) mbar_init(&landed[t], WNT);
    fence_barrier_init();
  }
  __syncthreads();

  // Requests, in tile order.  a: 256 chunks of 16 bytes per tile (64 rows x 4 quads), one per thread; 8 lanes
  // take the same quad of 8 consecutive rows (128 contiguous bytes of shared memory per quarter warp), the four
  // quads of a row are 64 contiguous bytes of a.  b: 512 floats per tile (16 steps x 32 columns), two per thread,
  // a warp on 32 consecutive columns of one step.
  {
    const int row = (tid >> 5) * 8 + (tid & 7), quad = (tid >> 3) & 3;
    const int i = r0 + row;
    const int xofs = (quad * WB + row) * 4;
    const float* xrow = i < M ? ab + (int64_t)i * K + 4 * quad : nullptr;
    const int col = tid & 31, kk0 = tid >> 5;   // steps kk0 and kk0 + 8 of the tile
    const int c = c0 + col;
    const bool cin = c < N;
    for (int t = 0; t < nt; ++t) {
      const int k0 = t * BK;
      cp_async16(sx + (size_t)t * WTX + xofs,
                 (xrow && k0 + 4 * quad + 3 < K) ? static_cast<const void*>(xrow + k0) : static_cast<const void*>(g_nan4));
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int kk = kk0 + 8 * q, k = k0 + kk;
        cp_async4(sy + (size_t)t * WTY + ((kk >> 2) * WC + col) * 4 + (kk & 3),
                  (cin && k < K) ? static_cast<const void*>(bb + (int64_t)k * N + c) : static_cast<const void*>(g_nan4));
      }
      cp_async_arrive(&landed[t]);
    }
  }

  const int rl0 = (warp >> 1) * 16, cl0 = (warp & 1) * 16;
  float Y[4][2];
  unsigned cidp[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    cidp[i] = 0xffffffffu;
    Y[i][0] = kFloor;
    Y[i][1] = kFloor;
  }
  bool fail = false;
  // one copy of the tile body (the maxima before the tile are copied aside for the "did this tile raise it" test):
  // the warps of the CTAs on an SM are at different tiles, and their code has to fit the instruction cache
#pragma unroll 1
  for (int t = 0; t < nt; ++t) {
    if (!mbar_wait_bounded(&landed[t], 0)) fail = true;
    const float* xt = sx + (size_t)t * WTX + (rl0 + ty) * 4;
    const float* yt = sy + (size_t)t * WTY + (cl0 + tx) * 4;
    float P[4][2];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      P[i][0] = Y[i][0];
      P[i][1] = Y[i][1];
    }
#pragma unroll
    for (int q = 0; q < BK / 4; ++q) {
      ulonglong2 xq[4], yq[2];
#pragma unroll
      for (int i = 0; i < 4; ++i) xq[i] = *reinterpret_cast<const ulonglong2*>(xt + (q * WB + 4 * i) * 4);
#pragma unroll
      for (int j = 0; j < 2; ++j) yq[j] = *reinterpret_cast<const ulonglong2*>(yt + (q * WC + 8 * j) * 4);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          float v0, v1, v2, v3;
          unpack2(MUL ? mul2(xq[i].x, yq[j].x) : add2(xq[i].x, yq[j].x), v0, v1);
          unpack2(MUL ? mul2(xq[i].y, yq[j].y) : add2(xq[i].y, yq[j].y), v2, v3);
          Y[i][j] = max3(max3(Y[i][j], v0, v1), v2, v3);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // strict `>`: an equal maximum in a later tile keeps the index
      if (Y[i][0] > P[i][0]) cidp[i] = __byte_perm(cidp[i], (unsigned)t, 0x3214);
      if (Y[i][1] > P[i][1]) cidp[i] = __byte_perm(cidp[i], (unsigned)t, 0x3240);
    }
  }
  fail = __any_sync(0xffffffffu, fail);
  if (fail && lane == 0) {
    atomicExch(&g_gave_up, 1);
    if (error) atomicExch(error, 1);
  }

  // The winning tile of every result is still in shared memory: search it from the last step down, so the lowest
  // matching k is the assignment that sticks.  The two results of a row side by side, one rolled loop over the
  // quads.  Tiles are 4 floats further apart than their size: the lanes of a warp search different tiles, and with
  // a stride that is a multiple of 32 banks all those reads would hit the same bank.
  float* ob = out + bt * M * N;
  int* ib = idx + bt * M * N;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int ml = rl0 + ty + 4 * i, m = r0 + ml;
    if (m >= M) continue;
    const float* xs[2];
    const float* ys[2];
    int p[2], cc[2];
    bool hunt[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int cl = cl0 + tx + 8 * j;
      cc[j] = c0 + cl;
      const unsigned c8 = (cidp[i] >> (8 * j)) & 0xffu;
      hunt[j] = cc[j] < N && c8 != 0xffu;
      const unsigned tile = hunt[j] ? c8 : 0u;  // a result with nothing to find reads tile 0 and ignores it
      xs[j] = sx + (size_t)tile * WTX + ml * 4;
      ys[j] = sy + (size_t)tile * WTY + cl * 4;
      p[j] = -1;
    }
    if (hunt[0] || hunt[1]) {
#pragma unroll 1
      for (int q = BK / 4 - 1; q >= 0; --q) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const ulonglong2 xv = *reinterpret_cast<const ulonglong2*>(xs[j] + q * WB * 4);
          const ulonglong2 yv = *reinterpret_cast<const ulonglong2*>(ys[j] + q * WC * 4);
          float v0, v1, v2, v3;
          unpack2(MUL ? mul2(xv.x, yv.x) : add2(xv.x, yv.x), v0, v1);
          unpack2(MUL ? mul2(xv.y, yv.y) : add2(xv.y, yv.y), v2, v3);
          if (v3 == Y[i][j]) p[j] = 4 * q + 3;
          if (v2 == Y[i][j]) p[j] = 4 * q + 2;
          if (v1 == Y[i][j]) p[j] = 4 * q + 1;
          if (v0 == Y[i][j]) p[j] = 4 * q;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      if (cc[j] >= N) continue;
      float val = Y[i][j];
      int pj = hunt[j] ? p[j] : -1;
      if (pj >= 0) {
        // the stored value is the matching term itself: only for a zero can it differ from the maximum (in
        // sign), so that is the one case that reads the term again
        if (val == 0.f) {
          const float xv = xs[j][(pj >> 2) * WB * 4 + (pj & 3)], yv = ys[j][(pj >> 2) * WC * 4 + (pj & 3)];
          val = MUL ? __fmul_rn(xv, yv) : __fadd_rn(xv, yv);
        }
        pj += (int)((cidp[i] >> (8 * j)) & 0xffu) * BK;
      }
      const int64_t e = (int64_t)m * N + cc[j];
      ob[e] = fail ? __int_as_float(0x7fc00000) : val;   // a give-up cannot pass for a result
      ib[e] = fail ? -1 : pj;
    }
  }
}


}  // namespace

// declared in dense.cuh
bool dense_max_w_eligible(const float* a, int64_t K) {
  const char* e = getenv("GENBMM_B200_MAX_SHORT");   // "block": the lockstep kernels take short reductions too
  if (e && e[0] == 'b') return false;
  return K > 0 && K % 4 == 0 && K <= (int64_t)kMaxTiles * BK && (reinterpret_cast<uintptr_t>(a) & 15) == 0;
}

int launch_dense_max_w(bool mul, const float* a, const float* b, float* out, int* idx, int64_t B, int64_t M, int64_t K,
                       int64_t N, cudaStream_t st) {
  const int64_t tiles_m = ceil_div(M, WB), tiles_n = ceil_div(N, WC), blocks = B * tiles_m * tiles_n;
  if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  const int nt = (int)ceil_div(K, BK);
  const size_t smem = (size_t)nt * (WTX + WTY) * sizeof(float);
  auto kernel = mul ? dense_max_w_kernel<true> : dense_max_w_kernel<false>;
  // several CTAs per SM need the largest shared-memory carveout
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)((size_t)kMaxTiles * (WTX + WTY) * sizeof(float))) != cudaSuccess ||
      cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) !=
          cudaSuccess)
    return GBMM_ERR_LAUNCH;
  kernel<<<(unsigned)blocks, WNT, smem, st>>>(a, b, out, idx, (int)M, (int)K, (int)N, (int)tiles_m, (int)tiles_n,
                                              nullptr);
  return launch_status();
}

}  // namespace gbmm
