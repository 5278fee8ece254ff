// Shared declarations of the banded kernels.
#pragma once
#include "common.cuh"

namespace gbmm {

struct BandDims {
  int64_t n;
  int a_lu, a_ld, b_lu, b_ld;
  __host__ __device__ int Wa() const { return a_lu + a_ld + 1; }
  __host__ __device__ int Wb() const { return b_lu + b_ld + 1; }
  __host__ __device__ int r_lu() const { return a_lu + b_ld; }
  __host__ __device__ int Wo() const { return Wa() + Wb() - 1; }
};

// Block-banded fast path (band_block.cu).  `ws` is the caller's workspace of at least
// band_fast_workspace_bytes(B, n) bytes (log semiring only; may be null otherwise); for the log
// semiring *flags_out receives the device array (B, ceil(n/64)) of row blocks that the exact
// kernels must redo.
int64_t band_fast_workspace_bytes(int64_t B, int64_t n);
int band_fast_forward(int mode, const float* a, const float* b, float* out, int* idx, const BandDims& d, int64_t B,
                      void* ws, int** flags_out, cudaStream_t st);
int band_fast_backward(int mode, const float* a, const float* b, const float* g, const float* part, float* grad_a,
                       float* grad_b, const BandDims& d, int64_t B, void* ws, int** flags_out, cudaStream_t st);

// Tensor-core path (band_tc.cu) for the sum and log semirings with bands at least 32 wide.  `ws` holds at
// least band_tc_workspace_bytes and was zero-filled once before its first use with these dimensions (the
// zero padding between the rows of the skewed operand copies is never rewritten).
bool band_tc_eligible(int mode, const BandDims& d);
int64_t band_tc_workspace_bytes(int backward, int64_t B, const BandDims& d);
int band_tc_forward(int mode, const float* a, const float* b, float* out, const BandDims& d, int64_t B, void* ws,
                    int** flags_out, cudaStream_t st);
int band_tc_backward(int mode, const float* a, const float* b, const float* g, const float* part, float* grad_a,
                     float* grad_b, const BandDims& d, int64_t B, void* ws, int operands_ready, int** flags_out,
                     cudaStream_t st);

// Max-plus forward from skewed copies (band_max.cu), bands at least 32 wide.  `ws` holds at least
// band_max_workspace_bytes and was filled with -inf once (band_max_workspace_init) before its first use with
// these dimensions; the kernels rewrite the band cells of the copies, never the padding.
bool band_max_fast_eligible(const BandDims& d);
int64_t band_max_workspace_bytes(int64_t B, const BandDims& d);
int band_max_workspace_init(void* ws, int64_t bytes, cudaStream_t st);
int band_max_forward(const float* a, const float* b, float* out, int* idx, const BandDims& d, int64_t B, void* ws,
                     cudaStream_t st);

}  // namespace gbmm
