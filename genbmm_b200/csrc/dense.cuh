// Launchers shared between the dense translation units.
#pragma once
#include "common.cuh"

namespace gbmm {

// Exact (SFU) log-sum-exp forward restricted to the 128x128 result tiles whose entry in
// flags[batch][ceil(M/128)][ceil(N/128)] is non-zero; flags == nullptr means every tile.
// `error` (with flags): the error word of the product kernel that ran before; when it is set the whole of `out`
// is overwritten with NaN instead (poison_if_failed, common.cuh).
int launch_log_fwd_flagged(const float* a, const float* b, float* out, const int* flags, int64_t B, int64_t M,
                           int64_t K, int64_t N, cudaStream_t st, const int* error = nullptr);

// Exact log backward restricted to the terms of flagged result tiles, ADDED to grad_a and
// grad_b (either may be null).  `error`: as above, for both gradients.
int launch_log_bwd_flagged(const float* a, const float* b, const float* c, const float* g, float* grad_a,
                           float* grad_b, const int* flags, int64_t B, int64_t M, int64_t K, int64_t N,
                           cudaStream_t st, const int* error = nullptr);

// Row maxima of a and column maxima of b for the factorised logbmm (dense_fast.cu).
int launch_rowcol_max(const float* a, const float* b, float* rowmax, float* colmax, int64_t B, int64_t M, int64_t K,
                      int64_t N, cudaStream_t st);

// 32x32-tile exact log kernels for small problems (dense_small.cu); `small_log_wanted` says whether a grid of
// `large_tile_ctas` CTAs of the 128x64-tile kernels would leave the GPU underfilled.
bool small_log_wanted(int64_t large_tile_ctas);
int launch_small_log_fwd(const float* a, const float* b, float* out, float* maxes, int64_t B, int64_t M, int64_t K,
                         int64_t N, cudaStream_t st);
int launch_small_log_bwd(const float* a, const float* b, const float* c, const float* g, float* grad_a, float* grad_b,
                         int64_t B, int64_t M, int64_t K, int64_t N, cudaStream_t st);

int rowmax_only(const float* a, float* rowmax, int64_t B, int64_t M, int64_t K, cudaStream_t st);

// Max-plus / prod-max forward for short reductions (dense_max_w.cu): K a multiple of 4, at most 288, a 16-byte
// aligned; values and int32 indices as the reference's kernels give them.
bool dense_max_w_eligible(const float* a, int64_t K);
int launch_dense_max_w(bool mul, const float* a, const float* b, float* out, int* idx, int64_t B, int64_t M, int64_t K,
                       int64_t N, cudaStream_t st);

}  // namespace gbmm
