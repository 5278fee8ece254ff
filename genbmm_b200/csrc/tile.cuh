// Global -> register -> shared staging of operand tiles for the dense semiring kernels.
//
// A tile covers BO "outer" indices (rows or columns of the result) times BK reduction
// indices and is stored reduction-major in shared memory: element (r, o) at s[r * LD + o],
// so the compute loop reads 4 consecutive outer indices with one 128-bit LDS.
// The operand's element (o, r) lives at base[o * so + r * sr] with exactly one of the two
// strides equal to 1:
//   RED_CONTIG  (sr == 1): e.g. a[m][k] reduced over k; 128-bit loads along r, transposed on
//                the way into shared memory.
//   !RED_CONTIG (so == 1): e.g. b[k][n] reduced over k; 128-bit loads along o, stored as is.
// Each float4 group is loaded with one LDG.128 when the operand is 16-byte aligned with a
// pitch that is a multiple of 4 elements and the group lies inside the matrix; otherwise it
// is assembled from guarded scalar loads, out-of-range elements taking `pad`.
#pragma once
#include "common.cuh"

namespace gbmm {

template <int BO, int BK, int NTHREADS, bool RED_CONTIG>
struct TileLoader {
  static_assert((BO * BK) % (4 * NTHREADS) == 0, "tile must split into whole float4 per thread");
  static constexpr int NV = BO * BK / 4 / NTHREADS;
  float4 v[NV];

  __device__ __forceinline__ void load(const float* __restrict__ base, int64_t so, int64_t sr,
                                       int o0, int r0, int o_ext, int r_ext, bool vec, float pad) {
#pragma unroll
    for (int q = 0; q < NV; ++q) {
      const int f = threadIdx.x + q * NTHREADS;
      if (RED_CONTIG) {
        const int o = o0 + f / (BK / 4);
        const int r = r0 + (f % (BK / 4)) * 4;
        const float* p = base + (int64_t)o * so + r;
        if (vec && o < o_ext && r + 3 < r_ext) {
          v[q] = __ldg(reinterpret_cast<const float4*>(p));
        } else {
          const bool ok = o < o_ext;
          v[q].x = (ok && r + 0 < r_ext) ? __ldg(p + 0) : pad;
          v[q].y = (ok && r + 1 < r_ext) ? __ldg(p + 1) : pad;
          v[q].z = (ok && r + 2 < r_ext) ? __ldg(p + 2) : pad;
          v[q].w = (ok && r + 3 < r_ext) ? __ldg(p + 3) : pad;
        }
      } else {
        const int r = r0 + f / (BO / 4);
        const int o = o0 + (f % (BO / 4)) * 4;
        const float* p = base + (int64_t)r * sr + o;
        if (vec && r < r_ext && o + 3 < o_ext) {
          v[q] = __ldg(reinterpret_cast<const float4*>(p));
        } else {
          const bool ok = r < r_ext;
          v[q].x = (ok && o + 0 < o_ext) ? __ldg(p + 0) : pad;
          v[q].y = (ok && o + 1 < o_ext) ? __ldg(p + 1) : pad;
          v[q].z = (ok && o + 2 < o_ext) ? __ldg(p + 2) : pad;
          v[q].w = (ok && o + 3 < o_ext) ? __ldg(p + 3) : pad;
        }
      }
    }
  }

  // store() after multiplying every element by `scale`
  __device__ __forceinline__ void store_scaled(float* __restrict__ s, int LD, float scale) {
#pragma unroll
    for (int q = 0; q < NV; ++q) {
      v[q].x *= scale;
      v[q].y *= scale;
      v[q].z *= scale;
      v[q].w *= scale;
    }
    store(s, LD);
  }

  // LD = pitch of the shared tile in floats (a multiple of 4).
  __device__ __forceinline__ void store(float* __restrict__ s, int LD) const {
#pragma unroll
    for (int q = 0; q < NV; ++q) {
      const int f = threadIdx.x + q * NTHREADS;
      if (RED_CONTIG) {
        const int o = f / (BK / 4);
        const int r = (f % (BK / 4)) * 4;
        s[(r + 0) * LD + o] = v[q].x;
        s[(r + 1) * LD + o] = v[q].y;
        s[(r + 2) * LD + o] = v[q].z;
        s[(r + 3) * LD + o] = v[q].w;
      } else {
        const int r = f / (BO / 4);
        const int o = (f % (BO / 4)) * 4;
        *reinterpret_cast<float4*>(s + r * LD + o) = v[q];
      }
    }
  }
};

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Thread -> micro-tile mapping shared by the 128x64 kernels (256 threads, 8x4 results each):
// rows ty*4+{0..3} and 64+ty*4+{0..3}; columns tx*4+{0..3}.
struct Micro8x4 {
  int tx, ty;
  __device__ __forceinline__ Micro8x4() : tx(threadIdx.x % 16), ty(threadIdx.x / 16) {}
  __device__ __forceinline__ int row(int i) const { return (i < 4 ? 0 : 64) + ty * 4 + (i & 3); }
  __device__ __forceinline__ int col(int j) const { return tx * 4 + j; }
  // operands of one reduction step from the shared tiles
  __device__ __forceinline__ void load_x(const float* sx, int LDX, float (&x)[8]) const {
    const float4 lo = *reinterpret_cast<const float4*>(sx + ty * 4);
    const float4 hi = *reinterpret_cast<const float4*>(sx + 64 + ty * 4);
    x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w;
    x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
  }
  __device__ __forceinline__ void load_y(const float* sy, float (&y)[4]) const {
    const float4 t = *reinterpret_cast<const float4*>(sy + tx * 4);
    y[0] = t.x; y[1] = t.y; y[2] = t.z; y[3] = t.w;
  }
};

}  // namespace gbmm
