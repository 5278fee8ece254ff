// Shared device helpers for the genbmm_b200 kernels (sm_100a only).
#pragma once
#include <cstdlib>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/genbmm_b200.h"

namespace gbmm {

// The reference starts every running maximum at -1e9 rather than -inf
// (matmul_cuda_kernel.cu:31,62,93,139; banded_cuda_kernel.cu:44,79).
constexpr float kFloor = -1e9f;
constexpr float kLog2e = 1.4426950408889634f;

// One MUFU.EX2.  The .ftz form flushes results below 2^-126 to zero instead of spending
// extra instructions on denormals; every use here adds the result to a sum whose other
// terms are at least 2^-126 times larger in the cases that matter.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// exp(x) on the SFU: one FMUL + one MUFU.EX2.
__device__ __forceinline__ float exp_sfu(float x) { return ex2_approx(x * kLog2e); }

// 3-input maximum (one FMNMX3 on sm_100).  NaN operands are ignored, as with the
// reference's `if (v > m)` which never selects a NaN.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__host__ __device__ __forceinline__ int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Optional CUDA-event bracket around a product launch (capi.cu; see gbmm_profile_enable).
bool profile_begin(int slot, cudaStream_t st);
void profile_end(int slot, cudaStream_t st);

// What a give-up looks like to the caller.  A product kernel whose bounded wait for a TMA copy or a tensor-core
// commit ran out sets its call's error word and leaves an unknown part of its output unwritten.  The kernel that
// follows it on the stream (the exact fix-up kernel where there is one, else poison_on_error_kernel) looks at
// the word first and, when it is set, overwrites the WHOLE output with NaN, so the failure cannot be taken for
// a result and no host synchronisation is needed to find out.  Returns true when it did (the caller returns).
__device__ __forceinline__ bool poison_if_failed(const int* error, float* out, int64_t count) {
  if (error == nullptr || *reinterpret_cast<const volatile int*>(error) == 0) return false;
  const float nan = __int_as_float(0x7fc00000);
  if (out != nullptr)
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x)
      out[i] = nan;
  return true;
}
// The stand-alone form (capi.cu): up to two outputs, either may be null.
int launch_poison_on_error(const int* error, float* out0, int64_t count0, float* out1, int64_t count1,
                           cudaStream_t st);

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? GBMM_OK : GBMM_ERR_LAUNCH; }

// Work list of a fix-up kernel launched with a capped grid.  CTA c of G = gridDim.x looks at the tile ids
// c, c + G, c + 2G, ...: in the round starting at `base` thread t tests id base + c + t * G, and the ids for
// which `flagged` holds are appended to `list` (one entry per thread of the CTA) in shared memory, in no
// particular order.  Returns how many there are; every thread of the CTA gets the same count.
template <class Pred>
__device__ __forceinline__ int collect_tiles(int64_t base, int64_t total, int* list, int* count, Pred flagged) {
  __syncthreads();  // the previous round's list is no longer read
  if (threadIdx.x == 0) *count = 0;
  __syncthreads();
  const int64_t id = base + blockIdx.x + (int64_t)threadIdx.x * gridDim.x;
  if (id < total && flagged(id)) list[atomicAdd(count, 1)] = (int)id;
  __syncthreads();
  return *count;
}

// Grid of such a kernel: one CTA per SM (a step without flagged tiles, the usual one, pays for launching and
// retiring the grid: 1.167 ms per 32 x 1024^3 step with four CTAs per SM, 1.156 ms with one), never more than
// there are tiles.
// GENBMM_B200_FIXUP_CTAS=<n> replaces the cap (tests use a tiny one to drive a CTA through several rounds).
inline int capped_grid(int64_t tiles, unsigned* grid) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return GBMM_ERR_DEVICE;
  static const int64_t forced = [] {
    const char* e = getenv("GENBMM_B200_FIXUP_CTAS");
    return e ? (int64_t)atoll(e) : (int64_t)0;
  }();
  const int64_t cap = forced > 0 ? forced : (int64_t)sms;
  *grid = (unsigned)(tiles < cap ? tiles : cap);
  return GBMM_OK;
}

}  // namespace gbmm
