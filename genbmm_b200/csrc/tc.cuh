// Building blocks shared by the tcgen05 (3xTF32) kernels: tile geometry, the shared-memory ring,
// shared-memory and instruction descriptors, MMA / commit / TMEM-load wrappers and TMA tile loads.
// Everything here is cta_group::1; the CTA-pair forms live beside the kernel that uses them.
#pragma once
#include "tma.cuh"

namespace gbmm {
namespace {

constexpr int TM = 128, TN = 128, TK = 32, TST = 3;
constexpr int TEW = 8;                 // epilogue warps: two per TMEM lane quarter, 64 columns each
constexpr int TNT = (2 + TEW) * 32;
constexpr int TEC = TN * 4 / TEW;      // columns per epilogue warp
constexpr float kTiny = 8.0779356694631609e-28f;  // 2^-90
constexpr uint32_t kTileBytes = TM * TK * sizeof(float);  // 16 KB per operand tile
constexpr int TNB = 4;                 // TMEM accumulation buffers of 128 columns
constexpr uint32_t kTmemCols = TNB * 128;
constexpr int TCH = 8;                // stages per accumulation chunk (256 reduction steps)

__host__ __device__ inline int64_t pad32(int64_t x) { return (x + 31) & ~int64_t(31); }
__host__ __device__ inline int64_t pad64(int64_t x) { return (x + 63) & ~int64_t(63); }

struct alignas(1024) TcSmem {
  float a_hi[TST][TM * TK];
  float a_lo[TST][TM * TK];
  float b_hi[TST][TN * TK];
  float b_lo[TST][TN * TK];
  float epi[TEW][32 * 33];  // per epilogue warp: a 32x32 block on its way to global memory
  uint64_t full[TST];
  uint64_t empty[TST];
  uint64_t chunk_full[TNB];
  uint64_t chunk_empty[TNB];
  uint64_t raw_full[TST];   // band_sp_kernel: TMA -> splitter warps (fits the alignment slack of this struct)
  uint32_t tmem_base;
};
static_assert(sizeof(TcSmem) + 1024 <= 232448, "the ring must fit the 227 KB a CTA can have");

// ---- descriptors -------------------------------------------------------------------------
// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the
// 128-byte swizzle (what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B): start address / 16 in
// bits 0-13, leading byte offset (unused for this layout, 1) in bits 16-29, stride between
// 8-row groups (1024 B) / 16 in bits 32-45, descriptor version 1 in bits 46-47, layout type
// 2 (128-byte swizzle) in bits 61-63.
__device__ __forceinline__ uint64_t umma_desc(const void* smem_tile, int k_byte_offset) {
  const uint32_t addr = smem_u32(smem_tile) + k_byte_offset;
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Descriptor of an MN-major tile.  For 32-bit operands the tensor core reads MN-major tiles only in
// the "128-byte swizzle with 32-byte atoms" layout (layout type 1; TMA writes it with
// CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B): 32 result indices (128 bytes) contiguous per reduction row,
// 4 reduction rows per 512-byte swizzle atom.  Here the atoms of one 32-index block are stacked along
// the reduction (32 rows = 4 KB) and the four blocks of the 128 result indices follow one another:
// leading byte offset = distance between blocks (4096 B), stride byte offset = distance between
// 4-row groups (512 B); one K=8 instruction reads two groups, the next starts 1 KB further on.
__device__ __forceinline__ uint64_t umma_desc_mn(const void* smem_tile, int k_step) {
  const uint32_t addr = smem_u32(smem_tile) + k_step * 1024;
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(4096 >> 4) << 16;
  d |= (uint64_t)(512 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)1 << 61;
  return d;
}

// Instruction descriptor for kind::tf32, fp32 accumulate, M=128, N=128: c_format F32 (1) at bit 4,
// a/b format TF32 (2) at bits 7 and 10, a/b MN-major at bits 15 and 16, N/8 at bit 17, M/16 at bit 24.
constexpr uint32_t kIdesc = (1u << 4) | (2u << 7) | (2u << 10) | ((TN >> 3) << 17) | ((TM >> 4) << 24);

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// the mbarrier receives one arrival when every MMA issued so far by this thread has finished
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
      "%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

// TMA load of one operand tile (128 result indices from `row`, 32 reduction steps from `k`).
// K-major: one (128 rows x 32 fp32) box of a 3-D map.  MN-major: one (4 blocks x 32 rows x 32 fp32)
// box of a 4-D map whose dimensions are (index % 32, reduction row, index / 32, batch).
template <bool MN>
__device__ __forceinline__ void tma_tile(void* dst, const CUtensorMap* map, uint64_t* bar, int k, int row, int bt) {
  if (MN)
    tma_load_4d(dst, map, bar, 0, k, row / 32, bt);
  else
    tma_load_3d(dst, map, bar, k, row, bt);
}

__device__ __forceinline__ float tf32_round(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

}  // namespace
}  // namespace gbmm
