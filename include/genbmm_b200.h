/*
 * genbmm_b200 — C ABI of the B200 (sm_100a) semiring batched-matmul library.
 *
 * Every entry point takes raw device pointers, plain sizes and a CUDA stream
 * (a cudaStream_t passed as void*; NULL = the legacy default stream), launches
 * asynchronously on that stream and returns a status code (0 = ok).  Nothing
 * here allocates, frees or synchronises unless a comment says otherwise.
 * All tensors are fp32 (indices int32), row-major and contiguous.
 *
 * The entry points replace, one for one, the functions of the reference's
 * pybind11 module `_genbmm` (harvardnlp/genbmm, matmul_cuda.cpp:165-172); the
 * comment on each declaration names the reference function it stands in for.
 * The difference in shape is deliberate: the reference functions allocate and
 * return torch tensors, these fill caller-provided buffers.
 */
#ifndef GENBMM_B200_H
#define GENBMM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define GBMM_OK 0
#define GBMM_ERR_INVALID_ARG 1  /* null pointer, negative size, unknown mode */
#define GBMM_ERR_UNSUPPORTED 2  /* size beyond what the kernels index (e.g. a dimension >= 2^31) */
#define GBMM_ERR_LAUNCH 3       /* the CUDA runtime refused a launch (see cudaGetLastError) */
#define GBMM_ERR_DEVICE 4       /* not an sm_100 device, or no device */
#define GBMM_ERR_SCRATCH_LIMIT 5 /* problem needs more than the built-in scratch of a no-allocation entry point */

/* semiring selectors — the integer `mode` of the reference
 * (dense: matmul_cuda_kernel.cu:487-542; banded: banded_cuda_kernel.cu:42-98) */
#define GBMM_MODE_LOG 0
#define GBMM_MODE_MAX 1
#define GBMM_MODE_SAMPLE 2   /* dense only */
#define GBMM_MODE_PRODMAX 3  /* dense only */
#define GBMM_BAND_LOG 0
#define GBMM_BAND_MAX 1
#define GBMM_BAND_MUL 3

/* Human-readable text for a status code (static storage). */
const char* gbmm_status_string(int status);

/* ABI version of this header. */
int gbmm_abi_version(void);

/*
 * Dense forward.  Replaces `_genbmm.forward(a, b, mode)` — matmul_forward,
 * matmul_cuda.cpp:69-77 -> matmul_cuda_forward, matmul_cuda_kernel.cu:465-543.
 *   a:(B,M,K) b:(B,K,N) -> out:(B,M,N)
 *   mode LOG:     out = log sum_k exp(a+b); aux (float*, may be NULL) receives the
 *                 running maximum `maxes` the reference returns as its second output.
 *   mode MAX:     out = max_k a+b; aux (int32*) = argmax, lowest k on ties, -1 if no
 *                 term exceeds -1e9.
 *   mode PRODMAX: out = max_k a*b; aux as for MAX.
 *   mode SAMPLE:  out = log sum_k exp(a+b); aux (int32*) = first k with
 *                 cdf(k-1) < u < cdf(k) of softmax_k(a+b), 0 if none; `u`:(B,M,N) are the
 *                 uniforms, which the reference draws itself (matmul_cuda_kernel.cu:517)
 *                 and this ABI takes from the caller.  `u` is ignored by other modes.
 * workspace: optional scratch of gbmm_dense_forward_workspace_bytes(mode, B, M, K, N) bytes
 * (64-byte aligned; 0 for the modes that need none).  Modes MAX and PRODMAX keep a transposed
 * copy of b there, which makes their final index search read contiguous memory (about 3x
 * faster at K = 1024); without it they read b in place.  Results are identical either way.
 */
int64_t gbmm_dense_forward_workspace_bytes(int mode, int64_t B, int64_t M, int64_t K, int64_t N);
int gbmm_dense_forward_f32(int mode, const float* a, const float* b, const float* u,
                           float* out, void* aux,
                           int64_t B, int64_t M, int64_t K, int64_t N,
                           void* workspace, int64_t workspace_bytes, void* stream);

/*
 * The second half of mode SAMPLE on its own: given out = logsumexp_k(a + b) from any of the log forward
 * entry points, draws idx (matmul_cuda_kernel.cu:109-118: fp32 running sum of exp(a + b - out) in ascending
 * k, strict double inequality against u, default 0).  Lets the caller take the logsumexp from the factorised
 * / tensor-core forward instead of the exact kernel.
 */
int gbmm_dense_sample_pick_f32(const float* a, const float* b, const float* u, const float* out, int32_t* idx,
                               int64_t B, int64_t M, int64_t K, int64_t N, void* stream);

/*
 * Dense backward.  Replaces `_genbmm.backward(a, b, grad_output, part, maxes, mode)`
 * — matmul_backward, matmul_cuda.cpp:79-92 -> matmul_cuda_backward,
 * matmul_cuda_kernel.cu:625-720.  Fills grad_a:(B,M,K) and grad_b:(B,K,N); either
 * may be NULL to skip it.  Unlike the reference, mode LOG fills grad_b too (the
 * reference leaves it zero and obtains it from a second call on transposed copies,
 * genmul.py:38-41).
 *   mode LOG:  part = the forward's out (float*); aux unused (may be NULL).
 *   other modes: aux = the forward's int32 indices; part unused (may be NULL).
 */
int gbmm_dense_backward_f32(int mode, const float* a, const float* b, const float* grad_out,
                            const float* part, const void* aux,
                            float* grad_a, float* grad_b,
                            int64_t B, int64_t M, int64_t K, int64_t N, void* stream);

/*
 * Dense log-semiring second-order terms.  Replaces `_genbmm.backbackward(a, b, grad_output, part,
 * maxes, grad_out_a, 0)` — matmul_backbackward, matmul_cuda.cpp:94-110 -> matmul_cuda_backbackward,
 * matmul_cuda_kernel.cu:547-622 — extended to the cotangents of both first-order gradients:
 * for L = <grad_a, h_a> + <grad_b, h_b> it fills d_a = dL/da:(B,M,K), d_b = dL/db:(B,K,N) and
 * d_grad_out = dL/dgrad_output:(B,M,N).  part = the forward's out.  (The reference's entry takes
 * h_a only and reaches h_b through a second call on transposed copies; pass zeros for an absent
 * cotangent.)  All sizes must be > 0.
 */
int gbmm_dense_backbackward_f32(const float* a, const float* b, const float* grad_out, const float* part,
                                const float* h_a, const float* h_b,
                                float* d_a, float* d_b, float* d_grad_out,
                                int64_t B, int64_t M, int64_t K, int64_t N, void* stream);

/*
 * Banded forward.  Replaces `_genbmm.forward_band(a, a_lu, a_lb, b, b_lu, b_lb, mode)`
 * — banded_forward, matmul_cuda.cpp:112-123 -> banded_cuda_forward,
 * banded_cuda_kernel.cu:354-402.
 *   a:(B,n,a_lu+a_ld+1) b:(B,n,b_lu+b_ld+1) -> out:(B,n,Wo), Wo = Wa+Wb-1, with result
 *   bands lu = a_lu+b_ld, ld = a_ld+b_lu.  Cells outside the matrix are written as 0.
 *   idx (int32*, required for mode MAX; argmax in a's band coordinate, -1 if none) and maxes
 *   (float*, mode LOG, optional) are written in full (0 outside the matrix) when given.
 * workspace: optional scratch of gbmm_band_workspace_bytes(B, n) bytes, 256-byte aligned.  With
 * it (and maxes == NULL) mode LOG runs the block-banded fast kernels with the exact kernels as
 * guard; without it mode LOG runs the exact kernels only.  Other modes ignore it.
 */
int64_t gbmm_band_workspace_bytes(int64_t B, int64_t n);
int gbmm_band_forward_f32(int mode, const float* a, int a_lu, int a_ld,
                          const float* b, int b_lu, int b_ld,
                          float* out, int32_t* idx, float* maxes,
                          int64_t B, int64_t n, void* workspace, int64_t workspace_bytes, void* stream);

/*
 * Banded backward.  Replaces `_genbmm.backward_band(a, a_lu, a_lb, b, b_lu, b_lb,
 * grad_output, part, mode)` — banded_backward, matmul_cuda.cpp:125-143 ->
 * banded_cuda_backward, banded_cuda_kernel.cu:404-450 — which yields grad_a only; the
 * reference gets grad_b from a second call with operands swapped and band-transposed
 * cotangents (sparse.py:436-446, 540-544, 625-635).  Here grad_b:(B,n,Wb) is computed
 * directly; grad_a or grad_b may be NULL to skip it.
 *   mode MUL: part unused.  mode LOG: part = forward out (float*).
 *   mode MAX: part = forward idx (int32*, a's band coordinate).
 * workspace: as for the forward (mode LOG).
 */
int gbmm_band_backward_f32(int mode, const float* a, int a_lu, int a_ld,
                           const float* b, int b_lu, int b_ld,
                           const float* grad_out, const void* part,
                           float* grad_a, float* grad_b,
                           int64_t B, int64_t n, void* workspace, int64_t workspace_bytes, void* stream);

/*
 * Tensor-core variants of gbmm_band_forward_f32 / gbmm_band_backward_f32 for modes 3 (sum) and 0 (log)
 * when both bands are at least 32 wide and n >= 128 (gbmm_band_tc_eligible): the three banded products run
 * as 3xTF32 on tcgen05 over zero-padded, skewed copies of the operands kept in the workspace.  Same
 * results as the plain entry points (log mode: same guard, flagged 64-row blocks are redone exactly).
 * Workspace contract: at least gbmm_band_tc_workspace_bytes bytes, 256-byte aligned, zero-filled ONCE with
 * gbmm_band_tc_workspace_init before its first use and afterwards only passed to these two functions with
 * the same B, n and band widths (they rewrite the band cells of the copies, never the zero padding).  A
 * backward workspace may also serve the forward.  Calls sharing a workspace must not overlap on the GPU.
 * `maxes` and `idx` are not produced (mode 0 needs neither for its backward).
 * operands_ready != 0 tells the backward that the workspace still holds what the last
 * gbmm_band_tc_forward_f32 call of the same mode left for exactly these a and b (unchanged since): their
 * skewed copies, row maxima and guard flags are then reused instead of rebuilt.
 */
int gbmm_band_tc_eligible(int mode, int64_t n, int a_lu, int a_ld, int b_lu, int b_ld);
int64_t gbmm_band_tc_workspace_bytes(int backward, int64_t B, int64_t n, int a_lu, int a_ld, int b_lu, int b_ld);
int gbmm_band_tc_workspace_init(void* workspace, int64_t workspace_bytes, void* stream);
int gbmm_band_tc_forward_f32(int mode, const float* a, int a_lu, int a_ld, const float* b, int b_lu, int b_ld,
                             float* out, int64_t B, int64_t n, void* workspace, int64_t workspace_bytes,
                             void* stream);
int gbmm_band_tc_backward_f32(int mode, const float* a, int a_lu, int a_ld, const float* b, int b_lu, int b_ld,
                              const float* grad_out, const float* part, float* grad_a, float* grad_b,
                              int64_t B, int64_t n, void* workspace, int64_t workspace_bytes,
                              int operands_ready, void* stream);

/*
 * Fast max-plus forward (mode 1 of gbmm_band_forward_f32: values and int32 indices in a's band coordinate,
 * bit-identical to it) for bands at least 32 wide and n >= 128 (gbmm_band_max_eligible).  It works from
 * skewed copies of the operands kept in the workspace, whose padding holds -inf: fill the workspace ONCE
 * with gbmm_band_max_workspace_init and afterwards pass it only to this function with the same B, n and
 * band widths.  Calls sharing a workspace must not overlap on the GPU.  The workspace's last 256 bytes hold the
 * call's error word: a kernel whose bounded wait for its own copies ran out sets it, and the result is then
 * overwritten with NaN before the call's work on the stream ends.
 */
int gbmm_band_max_eligible(int64_t n, int a_lu, int a_ld, int b_lu, int b_ld);
int64_t gbmm_band_max_workspace_bytes(int64_t B, int64_t n, int a_lu, int a_ld, int b_lu, int b_ld);
int gbmm_band_max_workspace_init(void* workspace, int64_t workspace_bytes, void* stream);
int gbmm_band_max_forward_f32(const float* a, int a_lu, int a_ld, const float* b, int b_lu, int b_ld,
                              float* out, int32_t* idx, int64_t B, int64_t n,
                              void* workspace, int64_t workspace_bytes, void* stream);

/*
 * Banded log-semiring second-order terms.  Replaces `_genbmm.backbackward_band(a, a_lu, a_lb, b,
 * b_lu, b_lb, grad_output, part, maxes, grad_out_a, 0)` — banded_backbackward,
 * matmul_cuda.cpp:145-161 -> banded_cuda_backbackward, banded_cuda_kernel.cu:453-546 — extended to
 * the cotangents of both first-order gradients: for L = <grad_a, h_a> + <grad_b, h_b> it fills
 * d_a:(B,n,Wa), d_b:(B,n,Wb) and d_grad_out:(B,n,Wo).  part = the forward's out.  Pass zeros for
 * an absent cotangent.
 */
int gbmm_band_backbackward_f32(const float* a, int a_lu, int a_ld, const float* b, int b_lu, int b_ld,
                               const float* grad_out, const float* part, const float* h_a, const float* h_b,
                               float* d_a, float* d_b, float* d_grad_out,
                               int64_t B, int64_t n, void* stream);

/*
 * Double-precision entry points: the reference dispatches every kernel over float, double and half
 * (AT_DISPATCH_FLOATING_TYPES_AND_HALF, matmul_cuda_kernel.cu:489; AT_DISPATCH_FLOATING_TYPES,
 * banded_cuda_kernel.cu:389).  Same arguments and semantics as the _f32 functions with double data (indices stay
 * int32); no workspace.  Half and bfloat16 inputs are widened to float by the Python layer, as nothing in the
 * path is bound by their storage.
 */
int gbmm_dense_forward_f64(int mode, const double* a, const double* b, const double* u, double* out, void* aux,
                           int64_t B, int64_t M, int64_t K, int64_t N, void* stream);
int gbmm_dense_backward_f64(int mode, const double* a, const double* b, const double* grad_out, const double* part,
                            const void* aux, double* grad_a, double* grad_b,
                            int64_t B, int64_t M, int64_t K, int64_t N, void* stream);
int gbmm_band_forward_f64(int mode, const double* a, int a_lu, int a_ld, const double* b, int b_lu, int b_ld,
                          double* out, int32_t* idx, double* maxes, int64_t B, int64_t n, void* stream);
int gbmm_band_backward_f64(int mode, const double* a, int a_lu, int a_ld, const double* b, int b_lu, int b_ld,
                           const double* grad_out, const void* part, double* grad_a, double* grad_b,
                           int64_t B, int64_t n, void* stream);

/*
 * Factorised log-semiring product (fast path of logbmm).  Same result as
 * gbmm_dense_forward_f32(GBMM_MODE_LOG, ...) / gbmm_dense_backward_f32 within fp32 rounding,
 * computed as ordinary fp32 matrix products of exponentiated operands
 * (c = rowmax + colmax + log(exp(a - rowmax) @ exp(b - colmax)), the formulation sketched in
 * the reference's commented einsum, genmul.py:45-47), with the exact kernels re-run on the
 * 128x128 result tiles where the factorisation would underflow.  They stand in for the same
 * reference functions as the dense entry points above (matmul_cuda.cpp:69-92).
 *
 * Scratch: the caller provides `workspace` (256-byte aligned, at least
 * gbmm_logbmm_workspace_bytes(backward, B, M, K, N) bytes; contents need not be preserved
 * between calls) and three small tensors that forward fills and backward reads:
 * rowmax:(B,M), colmax:(B,N) and flags: gbmm_logbmm_flag_count(B, M, N) int32.
 * K must be > 0 (and M, N > 0 for backward); use the dense entry points otherwise.
 */
int64_t gbmm_logbmm_workspace_bytes(int backward, int64_t B, int64_t M, int64_t K, int64_t N);
int64_t gbmm_logbmm_flag_count(int64_t B, int64_t M, int64_t N);
int gbmm_logbmm_forward_f32(const float* a, const float* b, float* out, float* rowmax, float* colmax,
                            int32_t* flags, void* workspace, int64_t workspace_bytes,
                            int64_t B, int64_t M, int64_t K, int64_t N, void* stream);
int gbmm_logbmm_backward_f32(const float* a, const float* b, const float* grad_out, const float* out,
                             const float* rowmax, const float* colmax, const int32_t* flags,
                             float* grad_a, float* grad_b, void* workspace, int64_t workspace_bytes,
                             int64_t B, int64_t M, int64_t K, int64_t N, void* stream);
/* What happens when a kernel of a fast path gives up.  Every wait inside the TMA / tcgen05 product kernels
 * (dense and banded) is bounded; a wait that runs out sets the first word of the call's workspace, and the kernel
 * that follows on the stream then overwrites the WHOLE output of that product with NaN.  A caller therefore never
 * receives a partly written result that looks valid, and needs no host synchronisation to be safe.
 * gbmm_logbmm_check is the diagnostic on top of that: it synchronises the stream and returns GBMM_ERR_LAUNCH when
 * the word is set.  `workspace` is the one passed to the call being checked (gbmm_logbmm_*_f32,
 * gbmm_logbmm_tc_*_f32 or gbmm_band_tc_*_f32). */
int gbmm_logbmm_check(const void* workspace, void* stream);

/* The NaN fill described above as a call of its own: if *error_word (device memory) is non-zero when the kernel
 * runs, out[0..count) becomes NaN, otherwise nothing is written.  The fast paths apply it themselves; it is
 * exported for callers that chain their own kernels behind a workspace's error word, and for tests. */
int gbmm_poison_on_error(const int32_t* error_word, float* out, int64_t count, void* stream);

/* Number of kernel launches this library has issued in this process (all entry points, all threads).  The
 * library's link step routes every launch through the counter, so the difference between two reads is the exact
 * number of kernels launched in between.  No counterpart in the reference. */
uint64_t gbmm_launch_count(void);

/*
 * Tensor-core variants of gbmm_logbmm_forward_f32 / _backward_f32: the same factorised products computed as
 * 3xTF32 on tcgen05 (each exponentiated operand split into tf32 hi + lo parts; accumulators in
 * TMEM).  Same arguments and outputs; its own, larger workspace
 * (gbmm_logbmm_tc_workspace_bytes).  rowmax / colmax / flags are interchangeable with the ones of
 * gbmm_logbmm_forward_f32 for the purposes of gbmm_logbmm_backward_f32.
 * The forward leaves the split operands exp(a - rowmax), exp(b - colmax) in its workspace; passed
 * unmodified to the backward of the same (a, b) as `factors`, they are reused instead of rebuilt
 * (null = rebuild them; the backward workspace is sized for that case either way).
 */
int64_t gbmm_logbmm_tc_workspace_bytes(int backward, int64_t B, int64_t M, int64_t K, int64_t N);
int gbmm_logbmm_tc_forward_f32(const float* a, const float* b, float* out, float* rowmax, float* colmax,
                               int32_t* flags, void* workspace, int64_t workspace_bytes,
                               int64_t B, int64_t M, int64_t K, int64_t N, void* stream);
int gbmm_logbmm_tc_backward_f32(const float* a, const float* b, const float* grad_out, const float* out,
                                const float* rowmax, const float* colmax, const int32_t* flags,
                                float* grad_a, float* grad_b, const void* factors,
                                void* workspace, int64_t workspace_bytes,
                                int64_t B, int64_t M, int64_t K, int64_t N, void* stream);

/*
 * logbmm forward for callers that cannot allocate device memory.  (No counterpart in the
 * reference, whose every entry point allocates its outputs with torch.)
 *
 * Who needs it: a caller that must not call cudaMalloc where it needs the product — e.g. it
 * runs inside a region whose memory owner forbids new reservations, it sits in a latency-bound
 * loop where the allocator's unbounded cost is unacceptable, or its host framework gives an
 * operator fixed input and output buffers and no workspace.  Such a caller cannot provide the
 * workspace, rowmax, colmax and flags that gbmm_logbmm_forward_f32 asks for.
 *
 * What it does: the same computation and result as gbmm_logbmm_forward_f32 (out = log sum_k
 * exp(a + b)); the caller passes only a, b and out.  All scratch lives in one fixed device
 * array inside the library, gbmm_logbmm_forward_noalloc_max_bytes() = 32 MiB, which every GPU
 * that loads the library holds until the process exits.  The call allocates and frees
 * nothing, on the device or through any library.
 *
 * Limits and rules:
 *  - gbmm_logbmm_forward_noalloc_need_bytes(B, M, K, N) must not exceed the maximum, else the
 *    call returns GBMM_ERR_SCRATCH_LIMIT and launches nothing (roughly 4*B*K*(M+N) bytes:
 *    e.g. up to three 1024x1024x1024 products per call).  K must be > 0.
 *  - The first call on each device looks up the array's device address (with that device
 *    current); make that first call outside any stream capture.
 *  - All calls on a device share the array.  It keeps the previous call's contents; the call
 *    clears the one word that must start at zero and rewrites the rest before reading it.
 *    Two calls whose kernels can overlap on the GPU (different streams, no ordering between
 *    them) race on the array and give wrong results: order them.
 */
int64_t gbmm_logbmm_forward_noalloc_max_bytes(void);
int64_t gbmm_logbmm_forward_noalloc_need_bytes(int64_t B, int64_t M, int64_t K, int64_t N);
int gbmm_logbmm_forward_noalloc_f32(const float* a, const float* b, float* out,
                                    int64_t B, int64_t M, int64_t K, int64_t N, void* stream);
/* gbmm_logbmm_check for the built-in scratch (the caller has no workspace pointer to pass): synchronises the
 * stream, returns GBMM_ERR_LAUNCH if the last no-allocation call on the current device gave up on a bounded
 * wait (its `out` is then all NaN, see gbmm_logbmm_check).  Allocates nothing. */
int gbmm_logbmm_forward_noalloc_check(void* stream);

/*
 * Layout helper of the chain (CRF) driver, no counterpart in the reference: dst block d <- src block map[d],
 * a block being `elems` contiguous floats (elems % 4 == 0, both pointers 16-byte aligned, map on the device);
 * map[d] < 0 fills block d with the log semiring's identity matrix of side `side` (0 on the diagonal, -1e9
 * elsewhere).  Used to put a chain of C x C matrices into the chain-major, bit-reversed order in which every
 * level of the pairwise tree multiplies the first half of the buffer by the second, and to undo it.
 */
int gbmm_gather_blocks_f32(const float* src, float* dst, const int64_t* map, int64_t blocks, int64_t elems,
                           int side, void* stream);

/* Diagnostic timing of the fast path's product kernels (no counterpart in the reference).
 * While enabled, each gbmm_logbmm_* call brackets its product launch with CUDA events on its
 * stream; gbmm_profile_last_ms(which) waits for the latest bracket (which = 0 forward product,
 * 1 grad_a product, 2 grad_b product) and returns milliseconds, or -1.  Not thread-safe. */
void gbmm_profile_enable(int on);
float gbmm_profile_last_ms(int which);

#ifdef __cplusplus
}
#endif
#endif /* GENBMM_B200_H */
