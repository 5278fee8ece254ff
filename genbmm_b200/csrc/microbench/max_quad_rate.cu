// Micro-benchmark of the [quad of steps][row][4 steps] layout of band_max_w_kernel / dense_max_w_kernel: packed add +
// 3-input maximum with the per-tile tracking, IR x JC results per thread, operands static in shared memory, no
// global traffic.  Not part of the library.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o max_quad_rate max_quad_rate.cu && ./max_quad_rate
//
// Measured on a B200 (terms per clock and SM at 1.965 GHz): 4 x 2 results per thread 54.4 (24 warps per SM) and
// 56.1 (32 warps), 4 x 4: 58.0 / 58.6 (16 warps), 8 x 4: 58.1 / 57.8 (8 warps).
#include <cstdio>
#include <cuda_runtime.h>
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ float max3(float a, float b, float c) { return fmaxf(fmaxf(a, b), c); }
template <int IR, int JC, int NT, int MINB>
__global__ void __launch_bounds__(NT, MINB) k(float* out, int iters) {
  constexpr int ROWS = 64, COLS = 16 * JC;
  __shared__ __align__(16) float sx[4 * ROWS * 4], sy[4 * 64 * 4];
  for (int i = threadIdx.x; i < 4 * ROWS * 4; i += NT) sx[i] = i * 0.001f;
  for (int i = threadIdx.x; i < 4 * 64 * 4; i += NT) sy[i] = i * 0.002f;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, ty = lane >> 3, tx = lane & 7;
  const int rl0 = ((warp >> 1) * 4 * IR) % ROWS, cl0 = (warp & 1) * 8 * JC;
  float Y[IR][JC]; unsigned cid[IR];
  for (int i = 0; i < IR; ++i) { cid[i] = 0; for (int j = 0; j < JC; ++j) Y[i][j] = -1e9f; }
  for (int it = 0; it < iters; ++it) {
    float P[IR][JC];
#pragma unroll
    for (int i = 0; i < IR; ++i)
#pragma unroll
      for (int j = 0; j < JC; ++j) P[i][j] = Y[i][j];
    const float* xt = sx + (rl0 + ty) * 4;
    const float* yt = sy + (cl0 + tx) * 4;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      asm volatile("" ::: "memory");
      ulonglong2 xq[IR], yq[JC];
#pragma unroll
      for (int i = 0; i < IR; ++i) xq[i] = *reinterpret_cast<const ulonglong2*>(xt + (q * ROWS + 4 * i) * 4);
#pragma unroll
      for (int j = 0; j < JC; ++j) yq[j] = *reinterpret_cast<const ulonglong2*>(yt + (q * COLS + 8 * j) * 4);
#pragma unroll
      for (int i = 0; i < IR; ++i)
#pragma unroll
        for (int j = 0; j < JC; ++j) {
          float v0, v1, v2, v3;
          unpack2(add2(xq[i].x, yq[j].x), v0, v1);
          unpack2(add2(xq[i].y, yq[j].y), v2, v3);
          Y[i][j] = max3(max3(Y[i][j], v0, v1), v2, v3);
        }
    }
#pragma unroll
    for (int i = 0; i < IR; ++i) {
      if (Y[i][0] > P[i][0]) cid[i] = __byte_perm(cid[i], (unsigned)it, 0x3214);
      if (Y[i][1] > P[i][1]) cid[i] = __byte_perm(cid[i], (unsigned)it, 0x3240);
      if (JC > 2) {
        if (Y[i][JC - 2] > P[i][JC - 2]) cid[i] = __byte_perm(cid[i], (unsigned)it, 0x3410);
        if (Y[i][JC - 1] > P[i][JC - 1]) cid[i] = __byte_perm(cid[i], (unsigned)it, 0x4210);
      }
    }
  }
  float s = 0; for (int i = 0; i < IR; ++i) { s += __uint_as_float(cid[i]); for (int j = 0; j < JC; ++j) s += Y[i][j]; }
  out[blockIdx.x * NT + threadIdx.x] = s;
}
template <int IR, int JC, int NT, int MINB>
void run(float* out, const char* name) {
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  const int iters = 40000, blocks = 148 * MINB;
  for (int rep = 0; rep < 2; ++rep) {
    cudaEventRecord(e0);
    k<IR, JC, NT, MINB><<<blocks, NT>>>(out, iters);
    cudaEventRecord(e1); cudaEventSynchronize(e1);
    float ms; cudaEventElapsedTime(&ms, e0, e1);
    const double terms = (double)blocks * NT * IR * JC * 16.0 * iters;
    if (rep) printf("%s: %.3f ms, %.1f terms/clk/SM at 1.965 GHz\n", name, ms, terms / (ms * 1e-3) / 148 / 1.965e9);
  }
}
int main() {
  float* out; cudaMalloc(&out, 148 * 8 * 1024 * 4);
  run<4, 2, 256, 3>(out, "4x2, 256 thr x 3 CTAs (24 warps)");
  run<4, 2, 256, 4>(out, "4x2, 256 thr x 4 CTAs (32 warps)");
  run<4, 4, 256, 2>(out, "4x4, 256 thr x 2 CTAs (16 warps)");
  run<4, 4, 512, 1>(out, "4x4, 512 thr x 1 CTA  (16 warps)");
  run<8, 4, 128, 2>(out, "8x4, 128 thr x 2 CTAs (8 warps)");
  run<8, 4, 256, 1>(out, "8x4, 256 thr x 1 CTA (8 warps)");
  printf("%s\n", cudaGetErrorString(cudaGetLastError()));
  return 0;
}
