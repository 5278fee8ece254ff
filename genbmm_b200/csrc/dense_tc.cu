// Tensor-core variant of the factorised logbmm products: 3xTF32 on tcgen05 with TMEM accumulators.
//
// The factorised path (dense_fast.cu) turns logbmm and its gradients into ordinary fp32 matrix
// products of exponentiated operands.  Here those products run on the 5th-generation tensor
// cores.  TF32 keeps 11 significand bits, too few for the 1e-5 tolerance, so each operand is
// split once, while it is exponentiated, into hi = tf32(x) and lo = x - hi, and the product is
// accumulated as  A_lo*B_hi + A_hi*B_lo + A_hi*B_hi  in one fp32 TMEM accumulator (the dropped
// lo*lo term is below 2^-22 relative).  Per 128x128 result tile and 32-wide reduction stage:
// four TMA loads (A_hi, A_lo, B_hi, B_lo: 16 KB each, 128-byte swizzle) and
// 12 tcgen05.mma.kind::tf32 instructions (M=128, N=128, K=8).
// Either operand may be stored with the reduction index contiguous ("K-major": 128 rows of 128
// bytes) or with the result index contiguous ("MN-major": 4 blocks of 32 reduction rows x 32
// result indices), so the three products of a step all read EA, EB and G' in the layout a, b and
// grad_out already have and no transposed copy is made.
//
// Two kernels share this scheme.  tc_gemm_kernel: one persistent CTA per SM on 128x128 tiles (cta_group::1).
// tc_pair_gemm_kernel: a cluster of two CTAs on a 256x256 tile (cta_group::2 loads and MMAs; the only
// cluster-multicast instruction is the tcgen05.commit barrier arrive, never a load).  In both, warp 0 issues
// the TMA loads, warp 1 owns the TMEM allocation and issues the MMAs (one elected lane each), the remaining
// warps read the accumulator back with tcgen05.ld (each its own 32-lane quarter) and write log(S) + ra + rb
// (or the gradient) to global memory.
// The tensor core adds into its fp32 accumulator with truncation, an error that grows with the
// length of the sum; so the reduction is cut into chunks of 256 steps, each accumulated in one of
// two TMEM buffers and then added, in round-to-nearest fp32, to per-thread register sums by the
// epilogue warps while the MMAs fill the other buffer.
// Stages are handed over with mbarriers (full: TMA -> MMA; empty: tcgen05.commit -> TMA;
// chunk_full: commit -> epilogue; chunk_empty: epilogue -> MMA).  Every wait is bounded; a wait that gives up sets the error
// word, and all paths meet at the final barrier so that the TMEM columns are always released.  Every load reads
// this GPU's own memory; no TMA load uses cluster multicast.
#include <cstdlib>

#include "dense.cuh"
#include "tc.cuh"

namespace gbmm {
namespace {

enum { TC_LOG = 0, TC_GRAD = 1 };

struct TcEpi {
  float* out;          // (batch, I, J)
  const float* row_v;  // TC_LOG: ra (batch, I);  TC_GRAD: shift by row or null
  const float* col_v;  // TC_LOG: rb (batch, J);  TC_GRAD: shift by column or null
  const float* src;    // TC_GRAD: operand whose exponential multiplies the sum
  int* flags;          // TC_LOG
  int* error;
};

// Pulls the part of `src` that store_sums will read for this warp (32 rows x NSUM columns) into L2
// while the tile is still being accumulated; lane = row, one request per 128-byte line.
template <int NSUM>
__device__ __forceinline__ void prefetch_src(const float* src, int bt, int row0, int col0, int I, int J, int lane) {
  const int ii = row0 + lane;
  if (!src || ii >= I) return;
  const float* p = src + ((int64_t)bt * I + ii) * J + col0;
#pragma unroll
  for (int q = 0; q < NSUM; q += 32)
    if (col0 + q < J) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + q));
}

// Epilogue of one warp: its NSUM sums per lane (lane = result row row0 + lane, columns col0 ..
// col0 + NSUM - 1) become log(S) + shifts (TC_LOG) or exp(src - shift) * S (TC_GRAD) in global memory.
template <int EPI, int NSUM>
__device__ __forceinline__ void store_sums(const float (&sum)[NSUM], float* blk, const TcEpi& ep, int bt, int row0,
                                           int col0, int I, int J, int lane, bool& bad) {
  // Hand the sums over through shared memory so that global memory is touched along rows:
  // lane = row when writing the warp's private 32x32 block, 8 lanes x 4 columns per row when
  // reading it back; one pass per 32 of the warp's columns.  All global loads of a pass are issued
  // before any is used (the registers of the sums just handed over hold them).
  const int hl = lane % 8, hr = lane / 8;
  const bool vec = (J % 4 == 0) && ((reinterpret_cast<uintptr_t>(ep.out) & 15) == 0) &&
                   (!ep.src || (reinterpret_cast<uintptr_t>(ep.src) & 15) == 0) &&
                   (!ep.col_v || (reinterpret_cast<uintptr_t>(ep.col_v) & 15) == 0);
#pragma unroll
  for (int pass = 0; pass < NSUM / 32; ++pass) {
    __syncwarp();
#pragma unroll
    for (int q = 0; q < 32; ++q) blk[lane * 33 + q] = sum[pass * 32 + q];
    __syncwarp();
    const int jj = col0 + pass * 32 + hl * 4;
    if (jj >= J) continue;
    const bool full4 = vec && jj + 3 < J;
    float cv[4] = {0.f, 0.f, 0.f, 0.f};
    if (ep.col_v) {
      if (full4) {
        const float4 t4 = __ldg(reinterpret_cast<const float4*>(ep.col_v + (int64_t)bt * J + jj));
        cv[0] = t4.x; cv[1] = t4.y; cv[2] = t4.z; cv[3] = t4.w;
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (jj + k < J) cv[k] = __ldg(ep.col_v + (int64_t)bt * J + jj + k);
      }
    }
    float x[8][4], rv[8];
#pragma unroll
    for (int itr = 0; itr < 8; ++itr) {
      const int ii = row0 + itr * 4 + hr;
      rv[itr] = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) x[itr][k] = 0.f;
      if (ii >= I) continue;
      if (ep.row_v) rv[itr] = __ldg(ep.row_v + (int64_t)bt * I + ii);
      if (EPI == TC_GRAD) {
        const float* sp = ep.src + ((int64_t)bt * I + ii) * J + jj;
        if (full4) {
          const float4 t4 = __ldg(reinterpret_cast<const float4*>(sp));
          x[itr][0] = t4.x; x[itr][1] = t4.y; x[itr][2] = t4.z; x[itr][3] = t4.w;
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            if (jj + k < J) x[itr][k] = __ldg(sp + k);
        }
      }
    }
#pragma unroll
    for (int itr = 0; itr < 8; ++itr) {
      const int r = itr * 4 + hr;
      const int ii = row0 + r;
      if (ii >= I) continue;
      float o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float v = blk[r * 33 + hl * 4 + k];
        if (EPI == TC_LOG) {
          const float shift = rv[itr] + cv[k];
          if (jj + k < J) bad |= !(v >= kTiny) || !(v <= 3.0e38f) || (shift < kFloor);
          o[k] = __logf(v) + shift;  // lg2.approx: absolute error below 2e-7 on the logarithm
        } else {
          o[k] = exp_sfu(x[itr][k] - (rv[itr] + cv[k])) * v;
        }
      }
      float* op = ep.out + ((int64_t)bt * I + ii) * J + jj;
      if (full4) {
        *reinterpret_cast<float4*>(op) = make_float4(o[0], o[1], o[2], o[3]);
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (jj + k < J) op[k] = o[k];
      }
    }
  }
}

// D[i,j] = sum_r A[i,r] B[j,r].  A is stored (batch,I,R) when !A_MN and (batch,R,I) when A_MN; B
// likewise (batch,J,R) or (batch,R,J).
// Persistent: the grid has one CTA per SM and CTA c takes tiles c, c + gridDim.x, ...; the three
// roles keep running stage and chunk counters across tiles, so the loads and MMAs of the next tile
// proceed (up to TNB chunks ahead) while the epilogue warps are still writing the previous one.
template <int EPI, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(TNT, 1) tc_gemm_kernel(const __grid_constant__ CUtensorMap ma_hi,
                                                         const __grid_constant__ CUtensorMap ma_lo,
                                                         const __grid_constant__ CUtensorMap mb_hi,
                                                         const __grid_constant__ CUtensorMap mb_lo, TcEpi ep, int R,
                                                         int I, int J, int tiles_i, int tiles_j,
                                                         int64_t total_tiles) {
  extern __shared__ unsigned char smem_raw[];
  TcSmem& sm = *reinterpret_cast<TcSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int nt = (R + TK - 1) / TK;
  const int nchunks = (nt + TCH - 1) / TCH;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < TST; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
#pragma unroll
    for (int q = 0; q < TNB; ++q) {
      mbar_init(&sm.chunk_full[q], 1);
      mbar_init(&sm.chunk_empty[q], TEW);  // one arrival per epilogue warp
    }
    fence_barrier_init();
  }
  if (warp == 1) {  // the whole warp allocates; the same warp frees at the end
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  bool fail = false;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;  // stages issued so far, over all tiles of this CTA
      for (int64_t tile = blockIdx.x; tile < total_tiles && !fail; tile += gridDim.x) {
        const int j0 = (int)(tile % tiles_j) * TN, i0 = (int)((tile / tiles_j) % tiles_i) * TM;
        const int bt = (int)(tile / ((int64_t)tiles_j * tiles_i));
        for (int t = 0; t < nt; ++t, ++it) {
          const int s = it % TST;
          if (it >= TST && !mbar_wait_bounded(&sm.empty[s], ((it / TST) - 1) & 1)) {
            fail = true;
            break;
          }
          mbar_arrive_expect_tx(&sm.full[s], 4 * kTileBytes);
          tma_tile<A_MN>(sm.a_hi[s], &ma_hi, &sm.full[s], t * TK, i0, bt);
          tma_tile<A_MN>(sm.a_lo[s], &ma_lo, &sm.full[s], t * TK, i0, bt);
          tma_tile<B_MN>(sm.b_hi[s], &mb_hi, &sm.full[s], t * TK, j0, bt);
          tma_tile<B_MN>(sm.b_lo[s], &mb_lo, &sm.full[s], t * TK, j0, bt);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = kIdesc | (A_MN ? 1u << 15 : 0u) | (B_MN ? 1u << 16 : 0u);
      uint32_t it = 0, gc = 0;  // stages and chunks consumed so far
      for (int64_t tile = blockIdx.x; tile < total_tiles && !fail; tile += gridDim.x) {
        for (int t = 0; t < nt; ++t, ++it) {
          const int s = it % TST, buf = gc % TNB;
          const bool chunk_start = (t % TCH) == 0;
          if (chunk_start && gc >= TNB && !mbar_wait_bounded(&sm.chunk_empty[buf], ((gc / TNB) - 1) & 1)) {
            fail = true;
            break;
          }
          if (!mbar_wait_bounded(&sm.full[s], (it / TST) & 1)) {
            fail = true;
            break;
          }
          tc_fence_after();
          const uint32_t acc = tmem + (uint32_t)(buf * TN);
#pragma unroll
          for (int kk = 0; kk < TK / 8; ++kk) {
            const int ko = kk * 8 * (int)sizeof(float);  // 32 bytes per K=8 step inside the 128-byte row
            const uint64_t ah = A_MN ? umma_desc_mn(sm.a_hi[s], kk) : umma_desc(sm.a_hi[s], ko);
            const uint64_t al = A_MN ? umma_desc_mn(sm.a_lo[s], kk) : umma_desc(sm.a_lo[s], ko);
            const uint64_t bh = B_MN ? umma_desc_mn(sm.b_hi[s], kk) : umma_desc(sm.b_hi[s], ko);
            const uint64_t bl = B_MN ? umma_desc_mn(sm.b_lo[s], kk) : umma_desc(sm.b_lo[s], ko);
            umma_tf32(acc, al, bh, idesc, (!chunk_start || kk > 0) ? 1u : 0u);
            umma_tf32(acc, ah, bl, idesc, 1u);
            umma_tf32(acc, ah, bh, idesc, 1u);
          }
          umma_commit(&sm.empty[s]);  // stage s may be refilled once these MMAs have read it
          if ((t % TCH) == TCH - 1 || t == nt - 1) {
            umma_commit(&sm.chunk_full[buf]);
            ++gc;
          }
        }
      }
    }
    __syncwarp();
  } else {
    const int quad = warp % 4;                 // TMEM lanes this warp may read: 32*quad .. 32*quad+31
    const int cbase = ((warp - 2) / 4) * TEC;  // first of this warp's columns
    float* blk = sm.epi[warp - 2];
    uint32_t gc = 0;
    bool bad_any = false;
    for (int64_t tile = blockIdx.x; tile < total_tiles && !fail; tile += gridDim.x) {
      const int j0 = (int)(tile % tiles_j) * TN, i0 = (int)((tile / tiles_j) % tiles_i) * TM;
      const int bt = (int)(tile / ((int64_t)tiles_j * tiles_i));
      float sum[TEC];
#pragma unroll
      for (int q = 0; q < TEC; ++q) sum[q] = 0.f;
      if (EPI == TC_GRAD) prefetch_src<TEC>(ep.src, bt, i0 + quad * 32, j0 + cbase, I, J, lane);
      for (int chunk = 0; chunk < nchunks; ++chunk, ++gc) {
        const int buf = gc % TNB;
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&sm.chunk_full[buf], (gc / TNB) & 1))) {
          fail = true;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < TEC / 32; ++c) {
          float v[32];
          tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * TN + cbase + c * 32), v);
#pragma unroll
          for (int q = 0; q < 32; ++q) sum[c * 32 + q] += v[q];
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0)
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.chunk_empty[buf])) : "memory");
      }
      if (fail) break;
      bool bad = false;
      store_sums<EPI, TEC>(sum, blk, ep, bt, i0 + quad * 32, j0 + cbase, I, J, lane, bad);
      if (EPI == TC_LOG) {
        // flags were zeroed before the launch; any epilogue warp that saw a bad sum raises the tile's
        if (__any_sync(0xffffffffu, bad) && lane == 0) atomicExch(ep.flags + tile, 1);
      }
      bad_any |= bad;
    }
    (void)bad_any;
  }
  if (__any_sync(0xffffffffu, fail) && lane == 0) atomicExch(ep.error, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ---- split-in-shared-memory variant -------------------------------------------------------------
// The same product from ONE unsplit fp32 copy per operand (the split passes write half the bytes, the product
// reads half): a TMA warp lands the raw tile in the stage's `hi` buffer, eight splitter warps rewrite it in place
// (hi = tf32(x) where x was, lo = x - hi at the same offset of the `lo` buffer; the split does not care which
// layout the tile has) and hand the stage to the MMA warp (fence.proxy.async, one arrival per splitter warp on
// `full`).  Selected by GENBMM_B200_TC_SPLIT=1 (see unsplit_mode for what was measured).
// Roles: warps 0-7 split, 8 issues the MMAs, 9-16 are the epilogue, 17 is the TMA producer.
constexpr int DSPW = 8;
constexpr int DSP_NT = (DSPW + 1 + TEW + 1) * 32;
constexpr int DSP_TMA_WARP = DSPW + 1 + TEW;
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int EPI, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(DSP_NT, 1) tc_gemm_sp_kernel(const __grid_constant__ CUtensorMap ma,
                                                               const __grid_constant__ CUtensorMap mb, TcEpi ep, int R,
                                                               int I, int J, int tiles_i, int tiles_j,
                                                               int64_t total_tiles) {
  extern __shared__ unsigned char smem_raw[];
  TcSmem& sm = *reinterpret_cast<TcSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int nt = (R + TK - 1) / TK;
  const int nchunks = (nt + TCH - 1) / TCH;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < TST; ++s) {
      mbar_init(&sm.raw_full[s], 1);
      mbar_init(&sm.full[s], DSPW);
      mbar_init(&sm.empty[s], 1);
    }
#pragma unroll
    for (int q = 0; q < TNB; ++q) {
      mbar_init(&sm.chunk_full[q], 1);
      mbar_init(&sm.chunk_empty[q], TEW);
    }
    fence_barrier_init();
  }
  if (warp == DSPW) {  // the whole warp allocates; the same warp frees at the end
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  bool fail = false;

  if (warp == DSP_TMA_WARP) {
    if (lane == 0) {
      uint32_t it = 0;
      for (int64_t tile = blockIdx.x; tile < total_tiles && !fail; tile += gridDim.x) {
        const int j0 = (int)(tile % tiles_j) * TN, i0 = (int)((tile / tiles_j) % tiles_i) * TM;
        const int bt = (int)(tile / ((int64_t)tiles_j * tiles_i));
        for (int t = 0; t < nt; ++t, ++it) {
          const int s = it % TST;
          if (it >= TST && !mbar_wait_bounded(&sm.empty[s], ((it / TST) - 1) & 1)) {
            fail = true;
            break;
          }
          mbar_arrive_expect_tx(&sm.raw_full[s], 2 * kTileBytes);
          tma_tile<A_MN>(sm.a_hi[s], &ma, &sm.raw_full[s], t * TK, i0, bt);
          tma_tile<B_MN>(sm.b_hi[s], &mb, &sm.raw_full[s], t * TK, j0, bt);
        }
      }
    }
    __syncwarp();
  } else if (warp < DSPW) {
    uint32_t it = 0;
    for (int64_t tile = blockIdx.x; tile < total_tiles && !fail; tile += gridDim.x) {
      for (int t = 0; t < nt; ++t, ++it) {
        const int s = it % TST;
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&sm.raw_full[s], (it / TST) & 1))) {
          fail = true;
          break;
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float4* hi = reinterpret_cast<float4*>(half ? sm.b_hi[s] : sm.a_hi[s]);
          float4* lo = reinterpret_cast<float4*>(half ? sm.b_lo[s] : sm.a_lo[s]);
          constexpr int NQ = TM * TK / 4 / (DSPW * 32);
          float4 x[NQ];
#pragma unroll
          for (int q = 0; q < NQ; ++q) x[q] = hi[tid + q * DSPW * 32];
#pragma unroll
          for (int q = 0; q < NQ; ++q) {
            const float4 h = make_float4(tf32_round(x[q].x), tf32_round(x[q].y), tf32_round(x[q].z),
                                         tf32_round(x[q].w));
            hi[tid + q * DSPW * 32] = h;
            lo[tid + q * DSPW * 32] = make_float4(x[q].x - h.x, x[q].y - h.y, x[q].z - h.z, x[q].w - h.w);
          }
        }
        fence_async_shared();  // these generic-proxy stores, before the tensor core's async-proxy reads
        __syncwarp();
        if (lane == 0)
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.full[s])) : "memory");
      }
    }
  } else if (warp == DSPW) {
    if (lane == 0) {
      constexpr uint32_t idesc = kIdesc | (A_MN ? 1u << 15 : 0u) | (B_MN ? 1u << 16 : 0u);
      uint32_t it = 0, gc = 0;
      for (int64_t tile = blockIdx.x; tile < total_tiles && !fail; tile += gridDim.x) {
        for (int t = 0; t < nt; ++t, ++it) {
          const int s = it % TST, buf = gc % TNB;
          const bool chunk_start = (t % TCH) == 0;
          if (chunk_start && gc >= TNB && !mbar_wait_bounded(&sm.chunk_empty[buf], ((gc / TNB) - 1) & 1)) {
            fail = true;
            break;
          }
          if (!mbar_wait_bounded(&sm.full[s], (it / TST) & 1)) {
            fail = true;
            break;
          }
          tc_fence_after();
          const uint32_t acc = tmem + (uint32_t)(buf * TN);
#pragma unroll
          for (int kk = 0; kk < TK / 8; ++kk) {
            const int ko = kk * 8 * (int)sizeof(float);
            const uint64_t ah = A_MN ? umma_desc_mn(sm.a_hi[s], kk) : umma_desc(sm.a_hi[s], ko);
            const uint64_t al = A_MN ? umma_desc_mn(sm.a_lo[s], kk) : umma_desc(sm.a_lo[s], ko);
            const uint64_t bh = B_MN ? umma_desc_mn(sm.b_hi[s], kk) : umma_desc(sm.b_hi[s], ko);
            const uint64_t bl = B_MN ? umma_desc_mn(sm.b_lo[s], kk) : umma_desc(sm.b_lo[s], ko);
            umma_tf32(acc, al, bh, idesc, (!chunk_start || kk > 0) ? 1u : 0u);
            umma_tf32(acc, ah, bl, idesc, 1u);
            umma_tf32(acc, ah, bh, idesc, 1u);
          }
          umma_commit(&sm.empty[s]);
          if ((t % TCH) == TCH - 1 || t == nt - 1) {
            umma_commit(&sm.chunk_full[buf]);
            ++gc;
          }
        }
      }
    }
    __syncwarp();
  } else {
    const int ew = warp - (DSPW + 1), quad = warp % 4;  // TMEM lanes this warp may read: 32*quad .. 32*quad+31
    const int cbase = (ew / 4) * TEC;
    float* blk = sm.epi[ew];
    uint32_t gc = 0;
    for (int64_t tile = blockIdx.x; tile < total_tiles && !fail; tile += gridDim.x) {
      const int j0 = (int)(tile % tiles_j) * TN, i0 = (int)((tile / tiles_j) % tiles_i) * TM;
      const int bt = (int)(tile / ((int64_t)tiles_j * tiles_i));
      float sum[TEC];
#pragma unroll
      for (int q = 0; q < TEC; ++q) sum[q] = 0.f;
      if (EPI == TC_GRAD) prefetch_src<TEC>(ep.src, bt, i0 + quad * 32, j0 + cbase, I, J, lane);
      for (int chunk = 0; chunk < nchunks; ++chunk, ++gc) {
        const int buf = gc % TNB;
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&sm.chunk_full[buf], (gc / TNB) & 1))) {
          fail = true;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < TEC / 32; ++c) {
          float v[32];
          tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * TN + cbase + c * 32), v);
#pragma unroll
          for (int q = 0; q < 32; ++q) sum[c * 32 + q] += v[q];
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0)
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.chunk_empty[buf])) : "memory");
      }
      if (fail) break;
      bool bad = false;
      store_sums<EPI, TEC>(sum, blk, ep, bt, i0 + quad * 32, j0 + cbase, I, J, lane, bad);
      if (EPI == TC_LOG) {
        if (__any_sync(0xffffffffu, bad) && lane == 0) atomicExch(ep.flags + tile, 1);
      }
    }
  }
  if (__any_sync(0xffffffffu, fail) && lane == 0) atomicExch(ep.error, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == DSPW) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ---- CTA-pair variant ------------------------------------------------------------------------
// The same product with tcgen05.mma.cta_group::2: a cluster of two CTAs (two SMs) owns a 256x256
// result tile.  Each CTA loads 128 rows of A and 128 of the 256 columns of B; one thread of the
// leader CTA (cluster rank 0) issues M=256, N=256, K=8 instructions that read A from each CTA's own
// shared memory and the two halves of B from both, and leave rows 128*rank .. 128*rank+127 of the
// tile in that CTA's TMEM.  Per multiply-add each SM reads half as many operand bytes from shared
// memory as with 128x128 tiles, which is what bounds the single-CTA kernel.
//   full[s]       (leader)   : the leader's producer arrives with the byte count of both CTAs' loads;
//                              both CTAs' TMA loads report to it
//   empty[s]      (each CTA) : tcgen05.commit from the leader, multicast to both CTAs
//   chunk_full[q] (each CTA) : tcgen05.commit multicast; wakes that CTA's epilogue warps
//   chunk_empty[q](leader)   : one arrival per epilogue warp of both CTAs
// TMEM holds two accumulation buffers of 256 columns.  The cluster barrier at the start orders the
// barrier initialisation before any remote arrival, the one at the end keeps both CTAs resident until
// neither can signal the other any more.  No multicast loads; every wait is bounded.
constexpr int PN = 256;           // columns of the pair tile = accumulator columns per buffer
constexpr int PNB = 2;            // TMEM buffers
constexpr int PEC = PN * 4 / TEW; // columns per epilogue warp (128)
constexpr uint32_t kIdescPair = (1u << 4) | (2u << 7) | (2u << 10) | ((PN >> 3) << 17) | ((256 >> 4) << 24);

__device__ __forceinline__ void umma_pair_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// one arrival on the barrier at this shared-memory offset in both CTAs of the pair, once every MMA
// issued so far by this thread has finished
__device__ __forceinline__ void umma_pair_commit(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"((uint16_t)3)
      : "memory");
}

template <bool MN>
__device__ __forceinline__ void tma_pair_tile(void* dst, const CUtensorMap* map, uint32_t bar, int k, int row,
                                              int bt) {
  if (MN)
    tma_pair_load_4d(dst, map, bar, 0, k, row / 32, bt);
  else
    tma_pair_load_3d(dst, map, bar, k, row, bt);
}

template <int EPI, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TNT, 1)
    tc_pair_gemm_kernel(const __grid_constant__ CUtensorMap ma_hi, const __grid_constant__ CUtensorMap ma_lo,
                        const __grid_constant__ CUtensorMap mb_hi, const __grid_constant__ CUtensorMap mb_lo, TcEpi ep,
                        int R, int I, int J, int tiles_i, int tiles_j, int64_t total_tiles) {
  extern __shared__ unsigned char smem_raw[];
  TcSmem& sm = *reinterpret_cast<TcSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const uint32_t rank = cluster_ctarank();
  const int64_t pair = blockIdx.x / 2, npairs = gridDim.x / 2;
  const int nt = (R + TK - 1) / TK;
  const int nchunks = (nt + TCH - 1) / TCH;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < TST; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
#pragma unroll
    for (int q = 0; q < PNB; ++q) {
      mbar_init(&sm.chunk_full[q], 1);
      mbar_init(&sm.chunk_empty[q], 2 * TEW);  // the epilogue warps of both CTAs
    }
    fence_barrier_init();
  }
  if (warp == 1) {  // the same warp of both CTAs allocates, and frees at the end
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  bool fail = false;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t full_addr[TST];
#pragma unroll
      for (int s = 0; s < TST; ++s) full_addr[s] = cluster_map(smem_u32(&sm.full[s]), 0);
      uint32_t it = 0;
      for (int64_t tile = pair; tile < total_tiles && !fail; tile += npairs) {
        const int j0 = (int)(tile % tiles_j) * PN + (int)rank * TN;   // this CTA's half of the B columns
        const int i0 = (int)((tile / tiles_j) % tiles_i) * (2 * TM) + (int)rank * TM;
        const int bt = (int)(tile / ((int64_t)tiles_j * tiles_i));
        for (int t = 0; t < nt; ++t, ++it) {
          const int s = it % TST;
          if (it >= TST && !mbar_wait_bounded_cluster(&sm.empty[s], ((it / TST) - 1) & 1)) {
            fail = true;
            break;
          }
          if (rank == 0) mbar_arrive_expect_tx(&sm.full[s], 8 * kTileBytes);
          tma_pair_tile<A_MN>(sm.a_hi[s], &ma_hi, full_addr[s], t * TK, i0, bt);
          tma_pair_tile<A_MN>(sm.a_lo[s], &ma_lo, full_addr[s], t * TK, i0, bt);
          tma_pair_tile<B_MN>(sm.b_hi[s], &mb_hi, full_addr[s], t * TK, j0, bt);
          tma_pair_tile<B_MN>(sm.b_lo[s], &mb_lo, full_addr[s], t * TK, j0, bt);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = kIdescPair | (A_MN ? 1u << 15 : 0u) | (B_MN ? 1u << 16 : 0u);
      uint32_t it = 0, gc = 0;
      for (int64_t tile = pair; tile < total_tiles && !fail; tile += npairs) {
        for (int t = 0; t < nt; ++t, ++it) {
          const int s = it % TST, buf = gc % PNB;
          const bool chunk_start = (t % TCH) == 0;
          if (chunk_start && gc >= PNB && !mbar_wait_bounded_cluster(&sm.chunk_empty[buf], ((gc / PNB) - 1) & 1)) {
            fail = true;
            break;
          }
          if (!mbar_wait_bounded_cluster(&sm.full[s], (it / TST) & 1)) {
            fail = true;
            break;
          }
          tc_fence_after();
          const uint32_t acc = tmem + (uint32_t)(buf * PN);
#pragma unroll
          for (int kk = 0; kk < TK / 8; ++kk) {
            const int ko = kk * 8 * (int)sizeof(float);
            const uint64_t ah = A_MN ? umma_desc_mn(sm.a_hi[s], kk) : umma_desc(sm.a_hi[s], ko);
            const uint64_t al = A_MN ? umma_desc_mn(sm.a_lo[s], kk) : umma_desc(sm.a_lo[s], ko);
            const uint64_t bh = B_MN ? umma_desc_mn(sm.b_hi[s], kk) : umma_desc(sm.b_hi[s], ko);
            const uint64_t bl = B_MN ? umma_desc_mn(sm.b_lo[s], kk) : umma_desc(sm.b_lo[s], ko);
            umma_pair_tf32(acc, al, bh, idesc, (!chunk_start || kk > 0) ? 1u : 0u);
            umma_pair_tf32(acc, ah, bl, idesc, 1u);
            umma_pair_tf32(acc, ah, bh, idesc, 1u);
          }
          umma_pair_commit(&sm.empty[s]);
          if ((t % TCH) == TCH - 1 || t == nt - 1) {
            umma_pair_commit(&sm.chunk_full[buf]);
            ++gc;
          }
        }
      }
    }
    __syncwarp();
  } else {
    const int quad = warp % 4;
    const int cbase = ((warp - 2) / 4) * PEC;
    float* blk = sm.epi[warp - 2];
    uint32_t empty_addr[PNB];
#pragma unroll
    for (int q = 0; q < PNB; ++q) empty_addr[q] = cluster_map(smem_u32(&sm.chunk_empty[q]), 0);
    uint32_t gc = 0;
    for (int64_t tile = pair; tile < total_tiles && !fail; tile += npairs) {
      const int j0 = (int)(tile % tiles_j) * PN;
      const int i0 = (int)((tile / tiles_j) % tiles_i) * (2 * TM) + (int)rank * TM;
      const int bt = (int)(tile / ((int64_t)tiles_j * tiles_i));
      float sum[PEC];
#pragma unroll
      for (int q = 0; q < PEC; ++q) sum[q] = 0.f;
      if (EPI == TC_GRAD) prefetch_src<PEC>(ep.src, bt, i0 + quad * 32, j0 + cbase, I, J, lane);
      for (int chunk = 0; chunk < nchunks; ++chunk, ++gc) {
        const int buf = gc % PNB;
        if (!__all_sync(0xffffffffu, mbar_wait_bounded_cluster(&sm.chunk_full[buf], (gc / PNB) & 1))) {
          fail = true;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < PEC / 32; ++c) {
          float v[32];
          tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * PN + cbase + c * 32), v);
#pragma unroll
          for (int q = 0; q < 32; ++q) sum[c * 32 + q] += v[q];
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(empty_addr[buf]);
      }
      if (fail) break;
      bool bad = false;
      store_sums<EPI, PEC>(sum, blk, ep, bt, i0 + quad * 32, j0 + cbase, I, J, lane, bad);
      if (EPI == TC_LOG) {
        // one flag per 128x128 block of the result: this warp's 128 columns lie in one of them
        const int fi = i0 / TM, fj = (j0 + cbase) / TN;
        if (__any_sync(0xffffffffu, bad) && lane == 0 && fi < (I + TM - 1) / TM && fj < (J + TN - 1) / TN)
          atomicExch(ep.flags + ((int64_t)bt * ((I + TM - 1) / TM) + fi) * ((J + TN - 1) / TN) + fj, 1);
      }
    }
  }
  if (__any_sync(0xffffffffu, fail) && lane == 0) atomicExch(ep.error, 1);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ---- exponentiate + split ------------------------------------------------------------------

// v = transform(src) over a (batch, R, C) tensor, then hi = tf32(v), lo = v - hi written in the same
// orientation with rows `pitch` (a multiple of 32) floats apart; the padding columns are never
// written: as reduction steps the tensor map cuts them off, as result indices they only reach
// results the epilogue does not store.  KIND as in dense_fast.cu:
//   0: exp(src - shift[r])   1: exp(src - shift[c])   2: g * exp(shift[r] + shift2[c] - src), 0 if flagged
// One thread per 4 consecutive columns; VEC: C % 4 == 0 and src, g 16-byte aligned -> 128-bit loads.
template <int KIND, bool VEC>
__global__ void __launch_bounds__(256) split_transform_kernel(const float* __restrict__ src,
                                                              const float* __restrict__ shift,
                                                              const float* __restrict__ shift2,
                                                              const float* __restrict__ g,
                                                              const int* __restrict__ flags, float* __restrict__ hi_out,
                                                              float* __restrict__ lo_out, int R, int C, int64_t pitch,
                                                              int64_t groups) {
  const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= groups) return;
  const int gpr = (C + 3) / 4;  // groups per row
  const int c = (int)(e % gpr) * 4;
  const int64_t row = e / gpr;  // bt * R + r
  const int r = (int)(row % R);
  const int64_t bt = row / R;
  float x[4] = {0.f, 0.f, 0.f, 0.f}, gv[4] = {0.f, 0.f, 0.f, 0.f}, sc[4] = {0.f, 0.f, 0.f, 0.f};
  const float* sp = src + row * C + c;
  const bool full = c + 3 < C;
  if (VEC) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(sp));
    x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w;
    if (KIND == 2) {
      const float4 u = __ldg(reinterpret_cast<const float4*>(g + row * C + c));
      gv[0] = u.x; gv[1] = u.y; gv[2] = u.z; gv[3] = u.w;
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (c + k < C) {
        x[k] = __ldg(sp + k);
        if (KIND == 2) gv[k] = __ldg(g + row * C + c + k);
      }
  }
  if (KIND != 0) {
    const float* cs = (KIND == 1 ? shift : shift2) + bt * C + c;
    if (VEC) {  // C % 4 == 0: bt * C + c is a multiple of 4; the shift vectors are 16-byte aligned
      const float4 t = __ldg(reinterpret_cast<const float4*>(cs));
      sc[0] = t.x; sc[1] = t.y; sc[2] = t.z; sc[3] = t.w;
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (c + k < C) sc[k] = __ldg(cs + k);
    }
  }
  const float sr = KIND != 1 ? __ldg(shift + row) : 0.f;
  bool dead = false;
  if (KIND == 2) dead = __ldg(flags + (bt * ((R + 127) / 128) + r / 128) * ((C + 127) / 128) + c / 128) != 0;
  float hi[4], lo[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float v;
    if (KIND == 0) v = exp_sfu(x[k] - sr);
    if (KIND == 1) v = exp_sfu(x[k] - sc[k]);
    if (KIND == 2) v = dead ? 0.f : gv[k] * exp_sfu((sr + sc[k]) - x[k]);
    if (!full && c + k >= C) v = 0.f;
    hi[k] = lo_out ? tf32_round(v) : v;   // lo_out == nullptr: one unsplit copy (split in shared memory later)
    lo[k] = v - hi[k];
  }
  // pitch % 32 == 0 and c % 4 == 0: the group is 16-byte aligned and lies inside the row's pitch
  *reinterpret_cast<float4*>(hi_out + row * pitch + c) = make_float4(hi[0], hi[1], hi[2], hi[3]);
  if (lo_out) *reinterpret_cast<float4*>(lo_out + row * pitch + c) = make_float4(lo[0], lo[1], lo[2], lo[3]);
}

template <int KIND>
int launch_split(const float* src, const float* shift, const float* shift2, const float* g, const int* flags,
                 float* hi, float* lo, int64_t B, int64_t R, int64_t C, cudaStream_t st) {
  const int64_t groups = B * R * ceil_div(C, 4), blocks = ceil_div(groups, 256);
  if (blocks >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = (C % 4 == 0) && al16(src) && (!g || al16(g)) && (KIND == 0 || al16(KIND == 1 ? shift : shift2));
  if (vec)
    split_transform_kernel<KIND, true><<<(unsigned)blocks, 256, 0, st>>>(src, shift, shift2, g, flags, hi, lo, (int)R,
                                                                        (int)C, pad32(C), groups);
  else
    split_transform_kernel<KIND, false><<<(unsigned)blocks, 256, 0, st>>>(src, shift, shift2, g, flags, hi, lo,
                                                                         (int)R, (int)C, pad32(C), groups);
  return launch_status();
}

// Fused operand preparation of the forward: the maximum and the exponentiated, split operand in one pass.
// rowsplit: one warp per row of a (rows of up to 128 * NV floats held in registers): ra = row maximum (0 for
// a row without a finite-or-+inf entry, like rowmax_kernel), EA = exp(a - ra) as hi + lo.
template <int NV>
__global__ void __launch_bounds__(256) rowsplit_kernel(const float* __restrict__ src, float* __restrict__ rowmax,
                                                       float* __restrict__ hi_out, float* __restrict__ lo_out,
                                                       int64_t rows, int C, int64_t pitch) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;
  if (row >= rows) return;
  const float4* sp = reinterpret_cast<const float4*>(src + row * C);
  const int groups = C / 4;  // C % 4 == 0 on this path
  float4 x[NV];
  float m = __int_as_float(0xff800000);
#pragma unroll
  for (int q = 0; q < NV; ++q) {
    const int gq = lane + 32 * q;
    if (gq < groups) {
      x[q] = __ldg(sp + gq);
      m = fmaxf(fmaxf(m, fmaxf(x[q].x, x[q].y)), fmaxf(x[q].z, x[q].w));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const float sh = (m == __int_as_float(0xff800000)) ? 0.f : m;
  if (lane == 0) rowmax[row] = sh;
  float4* hp = reinterpret_cast<float4*>(hi_out + row * pitch);
  float4* lp = reinterpret_cast<float4*>(lo_out + row * pitch);
#pragma unroll
  for (int q = 0; q < NV; ++q) {
    const int gq = lane + 32 * q;
    if (gq < groups) {
      const float v[4] = {exp_sfu(x[q].x - sh), exp_sfu(x[q].y - sh), exp_sfu(x[q].z - sh), exp_sfu(x[q].w - sh)};
      float h[4], l[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        h[k] = lo_out ? tf32_round(v[k]) : v[k];
        l[k] = v[k] - h[k];
      }
      hp[gq] = make_float4(h[0], h[1], h[2], h[3]);
      if (lo_out) lp[gq] = make_float4(l[0], l[1], l[2], l[3]);
    }
  }
}

// colsplit: one CTA per (batch element, 32 columns of b), 32 columns x 8 row slices: first the column maxima
// (rb, 0 for a column without a finite-or-+inf entry, like colmax_kernel), then the same elements again — from
// L1 / L2 — as EB = exp(b - rb), hi + lo.
__global__ void __launch_bounds__(256) colsplit_kernel(const float* __restrict__ src, float* __restrict__ colmax,
                                                       float* __restrict__ hi_out, float* __restrict__ lo_out, int R,
                                                       int C, int64_t pitch, int tiles_c) {
  __shared__ float part[8][33];
  const int lane = threadIdx.x % 32, slice = threadIdx.x / 32;
  const int64_t bt = blockIdx.x / tiles_c;
  const int c = (blockIdx.x % tiles_c) * 32 + lane;
  const float* sp = src + bt * R * C + c;
  float m = __int_as_float(0xff800000);
  if (c < C) {
#pragma unroll 4
    for (int r = slice; r < R; r += 8) m = fmaxf(m, __ldg(sp + (int64_t)r * C));
  }
  part[slice][lane] = m;
  __syncthreads();
#pragma unroll
  for (int s2 = 0; s2 < 8; ++s2) m = fmaxf(m, part[s2][lane]);
  const float sh = (m == __int_as_float(0xff800000)) ? 0.f : m;
  if (c >= C) return;
  if (slice == 0) colmax[bt * C + c] = sh;
  float* hp = hi_out + bt * R * pitch + c;
  float* lp = lo_out + bt * R * pitch + c;
#pragma unroll 4
  for (int r = slice; r < R; r += 8) {
    const float v = exp_sfu(__ldg(sp + (int64_t)r * C) - sh);
    const float h = lo_out ? tf32_round(v) : v;
    hp[(int64_t)r * pitch] = h;
    if (lo_out) lp[(int64_t)r * pitch] = v - h;
  }
}

// colsplit for reductions of up to 32 * NV rows: one CTA of 32 warps per (batch element, 32 columns) holds the
// whole strip in registers (thread = column lane x row slice, NV rows each), so b is read once and every
// load of the strip is in flight together; measured 76 us against 92 us for the two-pass kernel at
// 32 x 1024 x 1024.
template <int NV, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) colsplit_reg_kernel(const float* __restrict__ src, float* __restrict__ colmax,
                                                       float* __restrict__ hi_out, float* __restrict__ lo_out, int R,
                                                       int C, int64_t pitch, int tiles_c) {
  __shared__ float part[WARPS][33];
  const int lane = threadIdx.x % 32, slice = threadIdx.x / 32;
  const int64_t bt = blockIdx.x / tiles_c;
  const int c = (blockIdx.x % tiles_c) * 32 + lane;
  const float* sp = src + bt * R * C + c;
  const float ninf = __int_as_float(0xff800000);
  float v[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int r = slice + WARPS * i;
    v[i] = (c < C && r < R) ? __ldg(sp + (int64_t)r * C) : ninf;
  }
  float m = ninf;
#pragma unroll
  for (int i = 0; i < NV; ++i) m = fmaxf(m, v[i]);
  part[slice][lane] = m;
  __syncthreads();
#pragma unroll
  for (int s2 = 0; s2 < WARPS; ++s2) m = fmaxf(m, part[s2][lane]);
  const float sh = (m == ninf) ? 0.f : m;
  if (c >= C) return;
  if (slice == 0) colmax[bt * C + c] = sh;
  float* hp = hi_out + bt * R * pitch + c;
  float* lp = lo_out + bt * R * pitch + c;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int r = slice + WARPS * i;
    if (r < R) {
      const float e = exp_sfu(v[i] - sh);
      const float h = lo_out ? tf32_round(e) : e;
      hp[(int64_t)r * pitch] = h;
      if (lo_out) lp[(int64_t)r * pitch] = e - h;
    }
  }
}

// Tensor map over a (batch, rows, cols) fp32 array with rows `pitch` (a multiple of 32) apart, 128-byte
// swizzle (16-byte atoms for !MN, 32-byte atoms for MN).  !MN: the columns are the reduction index; boxes of 128 rows x 32 columns.  MN: the rows are
// the reduction index; dimensions (col % 32, row, col / 32, batch), boxes of 32 x 32 rows x 4 blocks.
// Reduction steps outside the array read as zero.
template <bool MN>
bool make_map_sw128(CUtensorMap* map, const float* base, uint64_t batch, uint64_t rows, uint64_t cols,
                    uint64_t pitch) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch & 31)) return false;
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  if (MN) {
    const cuuint64_t dims[4] = {32, rows, pitch / 32, batch};
    const cuuint64_t strides[3] = {pitch * sizeof(float), 32 * sizeof(float), rows * pitch * sizeof(float)};
    const cuuint32_t box[4] = {32, TK, TM / 32, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  const cuuint64_t dims[3] = {cols, rows, batch};
  const cuuint64_t strides[2] = {pitch * sizeof(float), rows * pitch * sizeof(float)};
  const cuuint32_t box[3] = {TK, TM, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// the products that take the CTA-pair kernel (long reductions over large results)
bool pair_wanted(int64_t R, int64_t I, int64_t J) {
  return I > TM && J > TN && R * (I < J ? I : J) >= 512 * 1024;
}

// One operand of a product: hi/lo arrays of shape (batch, rows, cols) with the given pitch.
struct TcOperand {
  const float* hi;
  const float* lo;
  int64_t rows, cols, pitch;
};

// D:(batch,I,J) = A B^T over R reduction steps.  !A_MN: A is (batch, I, R); A_MN: (batch, R, I); B likewise.
template <int EPI, bool A_MN, bool B_MN>
int launch_tc(const TcOperand& A, const TcOperand& Bo, const TcEpi& ep, int64_t B, int64_t R, int64_t I, int64_t J,
              cudaStream_t st, int slot) {
  if (!A.lo || !Bo.lo) {  // single unsplit copies: split in shared memory (never the pair kernel, see unsplit_mode)
    if (A.lo || Bo.lo) return GBMM_ERR_INVALID_ARG;
    CUtensorMap ua, ub;
    if (!make_map_sw128<A_MN>(&ua, A.hi, B, A.rows, A.cols, A.pitch) ||
        !make_map_sw128<B_MN>(&ub, Bo.hi, B, Bo.rows, Bo.cols, Bo.pitch))
      return GBMM_ERR_LAUNCH;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      return GBMM_ERR_DEVICE;
    const size_t smem = sizeof(TcSmem) + 1024;
    const int64_t ti = ceil_div(I, TM), tj = ceil_div(J, TN), tiles = B * ti * tj;
    const unsigned blocks = (unsigned)(tiles < sms ? tiles : sms);
    if (cudaFuncSetAttribute(tc_gemm_sp_kernel<EPI, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return GBMM_ERR_LAUNCH;
    const bool timed = profile_begin(slot, st);
    tc_gemm_sp_kernel<EPI, A_MN, B_MN><<<blocks, DSP_NT, smem, st>>>(ua, ub, ep, (int)R, (int)I, (int)J, (int)ti,
                                                                    (int)tj, tiles);
    if (timed) profile_end(slot, st);
    return launch_status();
  }
  CUtensorMap m0, m1, m2, m3;
  if (!make_map_sw128<A_MN>(&m0, A.hi, B, A.rows, A.cols, A.pitch) ||
      !make_map_sw128<A_MN>(&m1, A.lo, B, A.rows, A.cols, A.pitch) ||
      !make_map_sw128<B_MN>(&m2, Bo.hi, B, Bo.rows, Bo.cols, Bo.pitch) ||
      !make_map_sw128<B_MN>(&m3, Bo.lo, B, Bo.rows, Bo.cols, Bo.pitch))
    return GBMM_ERR_LAUNCH;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return GBMM_ERR_DEVICE;
  const size_t smem = sizeof(TcSmem) + 1024;
  // 256x256 tiles on CTA pairs for long reductions over large results: a short reduction leaves a pair tile's
  // epilogue (twice the columns per warp, two TMEM buffers) too little main loop to hide behind, and the
  // single-CTA kernel with its four buffers is faster (measured crossover: 512 steps x 1024 rows).
  // GENBMM_B200_TC_PAIR=0 keeps the single-CTA kernel everywhere.
  static const bool pair_ok = [] {
    const char* e = getenv("GENBMM_B200_TC_PAIR");
    return !(e && e[0] == '0');
  }();
  if (pair_ok && sms >= 2 && pair_wanted(R, I, J)) {
    const int64_t ti = ceil_div(I, 2 * TM), tj = ceil_div(J, PN), tiles = B * ti * tj;
    const int64_t pairs = tiles < sms / 2 ? tiles : sms / 2;
    if (cudaFuncSetAttribute(tc_pair_gemm_kernel<EPI, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return GBMM_ERR_LAUNCH;
    const bool timed = profile_begin(slot, st);
    tc_pair_gemm_kernel<EPI, A_MN, B_MN><<<(unsigned)(2 * pairs), TNT, smem, st>>>(m0, m1, m2, m3, ep, (int)R, (int)I,
                                                                                  (int)J, (int)ti, (int)tj, tiles);
    if (timed) profile_end(slot, st);
    return launch_status();
  }
  const int64_t ti = ceil_div(I, TM), tj = ceil_div(J, TN), tiles = B * ti * tj;
  const unsigned blocks = (unsigned)(tiles < sms ? tiles : sms);  // one persistent CTA per SM
  if (cudaFuncSetAttribute(tc_gemm_kernel<EPI, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem) != cudaSuccess)
    return GBMM_ERR_LAUNCH;
  const bool timed = profile_begin(slot, st);
  tc_gemm_kernel<EPI, A_MN, B_MN><<<blocks, TNT, smem, st>>>(m0, m1, m2, m3, ep, (int)R, (int)I, (int)J, (int)ti,
                                                            (int)tj, tiles);
  if (timed) profile_end(slot, st);
  return launch_status();
}

float* carve(float*& cursor, int64_t floats) {
  float* p = cursor;
  cursor += pad64(floats);
  return p;
}

// The exponentiated, split operands EA:(B,M,pad32(K)) and EB:(B,K,pad32(N)); the forward writes them
// behind the 64-float header of its workspace, the backward reads them from there or rebuilds them.
struct Factors {
  float *ea_hi, *ea_lo, *eb_hi, *eb_lo;   // unsplit mode: ea_hi / eb_hi hold the one copy, the lo pointers are null
};
// GENBMM_B200_TC_SPLIT=1: one unsplit copy per operand and tc_gemm_sp_kernel for every problem none of whose three
// products would take the CTA-pair kernel (one rule for the forward and both gradients, so that they can share
// the copies).  Half the workspace and half the operand bytes — and not the default: the chain driver's
// 16 x 511 x 256 x 256 step takes 11.8 ms this way against 10.6 ms with hi + lo copies.  The 128 x 128 tile is
// already at the shared-memory bandwidth (96 KB of operand reads per 32-step stage for 768 clocks of MMAs); the
// in-place split adds another 96 KB per stage, which costs more than the HBM bytes it saves.
bool unsplit_mode(int64_t M, int64_t K, int64_t N) {
  const char* e = getenv("GENBMM_B200_TC_SPLIT");   // read per call: a forward and its backward must agree, so
  if (!e || e[0] != '1') return false;              // change it only between problems
  return !(pair_wanted(K, M, N) || pair_wanted(N, M, K) || pair_wanted(M, K, N));
}
int64_t factor_floats(int64_t B, int64_t M, int64_t K, int64_t N) {
  const int copies = unsplit_mode(M, K, N) ? 1 : 2;
  return copies * (pad64(B * M * pad32(K)) + pad64(B * K * pad32(N)));
}
Factors carve_factors(float*& cur, int64_t B, int64_t M, int64_t K, int64_t N) {
  const bool one = unsplit_mode(M, K, N);
  Factors f;
  f.ea_hi = carve(cur, B * M * pad32(K));
  f.ea_lo = one ? nullptr : carve(cur, B * M * pad32(K));
  f.eb_hi = carve(cur, B * K * pad32(N));
  f.eb_lo = one ? nullptr : carve(cur, B * K * pad32(N));
  return f;
}
// forward: maxima and split operands together (one read of a and of b from HBM each)
int build_factors_with_maxima(const float* a, const float* b, float* rowmax, float* colmax, const Factors& f, int64_t B,
                              int64_t M, int64_t K, int64_t N, cudaStream_t st) {
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  int rc = GBMM_OK;
  const int64_t rblocks = ceil_div(B * M, 8);
  if (K % 4 == 0 && K <= 1024 && al16(a) && rblocks < (1LL << 31)) {
    rowsplit_kernel<8><<<(unsigned)rblocks, 256, 0, st>>>(a, rowmax, f.ea_hi, f.ea_lo, B * M, (int)K, pad32(K));
    rc = launch_status();
  } else {
    rowmax_only(a, rowmax, B, M, K, st);
    rc = launch_split<0>(a, rowmax, nullptr, nullptr, nullptr, f.ea_hi, f.ea_lo, B, M, K, st);
  }
  if (rc != GBMM_OK) return rc;
  const int64_t tn = ceil_div(N, 32);
  if (B * tn >= (1LL << 31)) return GBMM_ERR_UNSUPPORTED;
  const unsigned cblocks = (unsigned)(B * tn);
  const int k = (int)K, n = (int)N;
  if (K <= 256)
    colsplit_reg_kernel<32, 8><<<cblocks, 256, 0, st>>>(b, colmax, f.eb_hi, f.eb_lo, k, n, pad32(N), (int)tn);
  else if (K <= 512)
    colsplit_reg_kernel<32, 16><<<cblocks, 512, 0, st>>>(b, colmax, f.eb_hi, f.eb_lo, k, n, pad32(N), (int)tn);
  else if (K <= 1024)
    colsplit_reg_kernel<32, 32><<<cblocks, 1024, 0, st>>>(b, colmax, f.eb_hi, f.eb_lo, k, n, pad32(N), (int)tn);
  else
    colsplit_kernel<<<cblocks, 256, 0, st>>>(b, colmax, f.eb_hi, f.eb_lo, k, n, pad32(N), (int)tn);
  return launch_status();
}

int build_factors(const float* a, const float* b, const float* rowmax, const float* colmax, const Factors& f,
                  int64_t B, int64_t M, int64_t K, int64_t N, cudaStream_t st) {
  int rc = launch_split<0>(a, rowmax, nullptr, nullptr, nullptr, f.ea_hi, f.ea_lo, B, M, K, st);
  if (rc != GBMM_OK) return rc;
  return launch_split<1>(b, colmax, nullptr, nullptr, nullptr, f.eb_hi, f.eb_lo, B, K, N, st);
}

}  // namespace
}  // namespace gbmm

using namespace gbmm;

extern "C" int64_t gbmm_logbmm_tc_workspace_bytes(int backward, int64_t B, int64_t M, int64_t K, int64_t N) {
  if (B < 0 || M < 0 || K < 0 || N < 0) return -1;
  int64_t floats = 64 + factor_floats(B, M, K, N);
  if (backward) floats += (unsplit_mode(M, K, N) ? 1 : 2) * pad64(B * M * pad32(N));
  return floats * (int64_t)sizeof(float);
}

extern "C" int gbmm_logbmm_tc_forward_f32(const float* a, const float* b, float* out, float* rowmax, float* colmax,
                                          int32_t* flags, void* workspace, int64_t workspace_bytes, int64_t B,
                                          int64_t M, int64_t K, int64_t N, void* stream) {
  if (B < 0 || M < 0 || K < 0 || N < 0) return GBMM_ERR_INVALID_ARG;
  if (B == 0 || M == 0 || N == 0) return GBMM_OK;
  if (K == 0) return GBMM_ERR_UNSUPPORTED;
  if (!a || !b || !out || !rowmax || !colmax || !flags || !workspace) return GBMM_ERR_INVALID_ARG;
  const int64_t lim = (1LL << 31) - 256;
  if (M >= lim || K >= lim || N >= lim) return GBMM_ERR_UNSUPPORTED;
  if (workspace_bytes < gbmm_logbmm_tc_workspace_bytes(0, B, M, K, N)) return GBMM_ERR_INVALID_ARG;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return GBMM_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* cur = static_cast<float*>(workspace);
  int* error = reinterpret_cast<int*>(carve(cur, 64));
  const Factors f = carve_factors(cur, B, M, K, N);
  if (cudaMemsetAsync(error, 0, sizeof(int), st) != cudaSuccess) return GBMM_ERR_LAUNCH;
  int rc = build_factors_with_maxima(a, b, rowmax, colmax, f, B, M, K, N, st);
  if (rc != GBMM_OK) return rc;
  if (cudaMemsetAsync(flags, 0, sizeof(int) * B * ceil_div(M, TM) * ceil_div(N, TN), st) != cudaSuccess)
    return GBMM_ERR_LAUNCH;
  // out[m,n] = ra[m] + rb[n] + log sum_k EA[m,k] EB[k,n]
  TcEpi ep{out, rowmax, colmax, nullptr, flags, error};
  rc = launch_tc<TC_LOG, false, true>(TcOperand{f.ea_hi, f.ea_lo, M, K, pad32(K)},
                                      TcOperand{f.eb_hi, f.eb_lo, K, N, pad32(N)}, ep, B, K, M, N, st, 0);
  if (rc != GBMM_OK) return rc;
  return launch_log_fwd_flagged(a, b, out, flags, B, M, K, N, st, error);
}

extern "C" int gbmm_logbmm_tc_backward_f32(const float* a, const float* b, const float* grad_out, const float* out,
                                           const float* rowmax, const float* colmax, const int32_t* flags,
                                           float* grad_a, float* grad_b, const void* factors, void* workspace,
                                           int64_t workspace_bytes, int64_t B, int64_t M, int64_t K, int64_t N,
                                           void* stream) {
  if (B < 0 || M < 0 || K < 0 || N < 0) return GBMM_ERR_INVALID_ARG;
  if (B == 0 || K == 0) return GBMM_OK;
  if (M == 0 || N == 0) return GBMM_ERR_UNSUPPORTED;
  if (!a || !b || !grad_out || !out || !rowmax || !colmax || !flags || !workspace) return GBMM_ERR_INVALID_ARG;
  const int64_t lim = (1LL << 31) - 256;
  if (M >= lim || K >= lim || N >= lim) return GBMM_ERR_UNSUPPORTED;
  if (workspace_bytes < gbmm_logbmm_tc_workspace_bytes(1, B, M, K, N)) return GBMM_ERR_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) || (reinterpret_cast<uintptr_t>(factors) & 255))
    return GBMM_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* cur = static_cast<float*>(workspace);
  int* error = reinterpret_cast<int*>(carve(cur, 64));
  Factors f = carve_factors(cur, B, M, K, N);
  float* gp_hi = carve(cur, B * M * pad32(N));  // G' : (B, M, pad32(N))
  float* gp_lo = unsplit_mode(M, K, N) ? nullptr : carve(cur, B * M * pad32(N));
  if (cudaMemsetAsync(error, 0, sizeof(int), st) != cudaSuccess) return GBMM_ERR_LAUNCH;
  int rc = GBMM_OK;
  if (factors) {  // the forward's workspace: same header, same carving
    float* fc = const_cast<float*>(static_cast<const float*>(factors)) + 64;
    f = carve_factors(fc, B, M, K, N);
  } else {
    rc = build_factors(a, b, rowmax, colmax, f, B, M, K, N, st);
    if (rc != GBMM_OK) return rc;
  }
  rc = launch_split<2>(out, rowmax, colmax, grad_out, flags, gp_hi, gp_lo, B, M, N, st);
  if (rc != GBMM_OK) return rc;
  const TcOperand EA{f.ea_hi, f.ea_lo, M, K, pad32(K)}, EB{f.eb_hi, f.eb_lo, K, N, pad32(N)};
  const TcOperand GP{gp_hi, gp_lo, M, N, pad32(N)};
  if (grad_a) {
    // grad_a[m,k] = EA[m,k] * sum_n G'[m,n] EB[k,n]
    TcEpi ep{grad_a, rowmax, nullptr, a, nullptr, error};
    rc = launch_tc<TC_GRAD, false, false>(GP, EB, ep, B, N, M, K, st, 1);
    if (rc != GBMM_OK) return rc;
  }
  if (grad_b) {
    // grad_b[k,n] = EB[k,n] * sum_m EA[m,k] G'[m,n]
    TcEpi ep{grad_b, nullptr, colmax, b, nullptr, error};
    rc = launch_tc<TC_GRAD, true, true>(EA, GP, ep, B, M, K, N, st, 2);
    if (rc != GBMM_OK) return rc;
  }
  return launch_log_bwd_flagged(a, b, out, grad_out, grad_a, grad_b, flags, B, M, K, N, st, error);
}
