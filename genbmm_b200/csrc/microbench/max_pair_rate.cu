// Micro-benchmark behind the max-plus kernels' bound: the inner loop of dense_max_fwd_kernel alone (packed add +
// 3-input maximum, 8 x 4 results per thread, (k, k+1) pair layout, operands static in shared memory, no global
// traffic), 16 warps per SM.  Not part of the library.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o max_pair_rate max_pair_rate.cu && ./max_pair_rate
//
// Measured on a B200 (terms per clock and SM at 1.965 GHz): mode 0 (the loop itself) 65.4, mode 1 (an integer op in
// place of the packed add) 42.0, mode 2 (packed add + FFMA, no maximum) 66.0, mode 3 (mode 0 + the per-tile
// tracking: copy of the maxima, compare, byte insert) 58.9, mode 4 (mode 3 + a CTA barrier per tile) 56.3.
#include <cstdio>
#include <cuda_runtime.h>
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ float max3(float a, float b, float c) { return fmaxf(fmaxf(a, b), c); }
template <int MODE>   // 0: add2 + max3, 1: max3 only (operands reused), 2: add2 only
__global__ void __launch_bounds__(256, 2) k(float* out, int iters) {
  __shared__ __align__(16) float sx[8 * 132 * 2], sy[8 * 68 * 2];
  for (int i = threadIdx.x; i < 8 * 132 * 2; i += 256) sx[i] = i * 0.001f;
  for (int i = threadIdx.x; i < 8 * 68 * 2; i += 256) sy[i] = i * 0.002f;
  __syncthreads();
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[8][4];
  for (int i = 0; i < 8; ++i) for (int j = 0; j < 4; ++j) acc[i][j] = -1e9f;
  unsigned cid[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int it = 0; it < iters; ++it) {
    float prev[8][4];
    if (MODE >= 3)
      for (int i = 0; i < 8; ++i) for (int j = 0; j < 4; ++j) prev[i][j] = acc[i][j];
    if (MODE == 4) __syncthreads();
#pragma unroll
    for (int kp = 0; kp < 8; ++kp) {
      asm volatile("" ::: "memory");
      const float* xs = sx + (kp * 132 + ty * 4) * 2;
      const float* ys = sy + (kp * 68 + tx * 4) * 2;
      const ulonglong2 x01 = *reinterpret_cast<const ulonglong2*>(xs), x23 = *reinterpret_cast<const ulonglong2*>(xs + 4);
      const ulonglong2 x45 = *reinterpret_cast<const ulonglong2*>(xs + 128), x67 = *reinterpret_cast<const ulonglong2*>(xs + 132);
      const ulonglong2 y01 = *reinterpret_cast<const ulonglong2*>(ys), y23 = *reinterpret_cast<const ulonglong2*>(ys + 4);
      const unsigned long long xp[8] = {x01.x, x01.y, x23.x, x23.y, x45.x, x45.y, x67.x, x67.y};
      const unsigned long long yp[4] = {y01.x, y01.y, y23.x, y23.y};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float v0, v1;
          if (MODE == 0 || MODE >= 3) { unpack2(add2(xp[i], yp[j]), v0, v1); acc[i][j] = max3(acc[i][j], v0, v1); }
          if (MODE == 1) { unpack2(xp[i] ^ yp[j], v0, v1); acc[i][j] = max3(acc[i][j], v0, v1); }
          if (MODE == 2) { unpack2(add2(xp[i], yp[j]), v0, v1); acc[i][j] += v0 * v1; }
        }
    }
    if (MODE >= 3) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (acc[i][0] > prev[i][0]) cid[i] = __byte_perm(cid[i], (unsigned)it, 0x3214);
        if (acc[i][1] > prev[i][1]) cid[i] = __byte_perm(cid[i], (unsigned)it, 0x3240);
        if (acc[i][2] > prev[i][2]) cid[i] = __byte_perm(cid[i], (unsigned)it, 0x3410);
        if (acc[i][3] > prev[i][3]) cid[i] = __byte_perm(cid[i], (unsigned)it, 0x4210);
      }
    }
  }
  float s = 0; for (int i = 0; i < 8; ++i) { s += __uint_as_float(cid[i]); for (int j = 0; j < 4; ++j) s += acc[i][j]; }
  out[blockIdx.x * 256 + threadIdx.x] = s;
}
int main() {
  float* out; cudaMalloc(&out, 296 * 256 * 4);
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  const int iters = 20000;
  for (int mode = 0; mode < 5; ++mode) {
    for (int rep = 0; rep < 2; ++rep) {
      cudaEventRecord(e0);
      if (mode == 0) k<0><<<296, 256>>>(out, iters);
      if (mode == 1) k<1><<<296, 256>>>(out, iters);
      if (mode == 2) k<2><<<296, 256>>>(out, iters);
      if (mode == 3) k<3><<<296, 256>>>(out, iters);
      if (mode == 4) k<4><<<296, 256>>>(out, iters);
      cudaEventRecord(e1); cudaEventSynchronize(e1);
      float ms; cudaEventElapsedTime(&ms, e0, e1);
      const double terms = 296.0 * 256 * 32 * 16.0 * iters;
      if (rep) printf("mode %d: %.3f ms, %.1f terms/clk/SM at 1.965 GHz\n", mode, ms, terms / (ms * 1e-3) / 148 / 1.965e9);
    }
  }
  printf("%s\n", cudaGetErrorString(cudaGetLastError()));
  return 0;
}
