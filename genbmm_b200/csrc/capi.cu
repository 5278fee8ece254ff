// Status text and ABI version of the C interface declared in include/genbmm_b200.h.
#include "common.cuh"

extern "C" const char* gbmm_status_string(int status) {
  switch (status) {
    case GBMM_OK: return "ok";
    case GBMM_ERR_INVALID_ARG: return "invalid argument";
    case GBMM_ERR_UNSUPPORTED: return "size not supported";
    case GBMM_ERR_LAUNCH: return "CUDA launch failed";
    case GBMM_ERR_DEVICE: return "no usable CUDA device";
    case GBMM_ERR_SCRATCH_LIMIT: return "problem exceeds the built-in scratch of the no-allocation entry point";
    default: return "unknown status";
  }
}

extern "C" int gbmm_abi_version(void) { return 1; }

// Diagnostic timing of the product kernels of the factorised logbmm (FP32-pipe and tensor-core
// variants).  While enabled, every gbmm_logbmm_* call brackets its product launch with CUDA
// events on the call's stream; gbmm_profile_last_ms(which) waits for the latest bracket of
// which = 0 (forward product), 1 (grad_a product), 2 (grad_b product) and returns its duration
// in milliseconds, or -1 if there is none.  Not thread-safe; off by default.
namespace gbmm {
namespace {
bool g_profile = false;
cudaEvent_t g_events[3][2];
bool g_event_made[3] = {false, false, false};
bool g_event_used[3] = {false, false, false};
}  // namespace

bool profile_begin(int slot, cudaStream_t st) {
  if (!g_profile || slot < 0 || slot > 2) return false;
  if (!g_event_made[slot]) {
    if (cudaEventCreate(&g_events[slot][0]) != cudaSuccess || cudaEventCreate(&g_events[slot][1]) != cudaSuccess)
      return false;
    g_event_made[slot] = true;
  }
  return cudaEventRecord(g_events[slot][0], st) == cudaSuccess;
}

void profile_end(int slot, cudaStream_t st) {
  if (cudaEventRecord(g_events[slot][1], st) == cudaSuccess) g_event_used[slot] = true;
}
}  // namespace gbmm

extern "C" void gbmm_profile_enable(int on) { gbmm::g_profile = on != 0; }

extern "C" float gbmm_profile_last_ms(int which) {
  using namespace gbmm;
  if (which < 0 || which > 2 || !g_event_used[which]) return -1.f;
  float ms = -1.f;
  if (cudaEventSynchronize(g_events[which][1]) != cudaSuccess) return -1.f;
  if (cudaEventElapsedTime(&ms, g_events[which][0], g_events[which][1]) != cudaSuccess) return -1.f;
  return ms;
}

// ---- block gather: the chain driver's layout changes ---------------------------------------------
namespace gbmm {
namespace {
// dst block d <- src block map[d] (a block = `elems` contiguous floats, elems % 4 == 0, both 16-byte
// aligned); map[d] < 0 fills the block with the log semiring's identity matrix (0 on the diagonal of a
// side x side block, -1e9 elsewhere).  One CTA per (block, 16 KB slice).
__global__ void __launch_bounds__(256) gather_blocks_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                            const int64_t* __restrict__ map, int64_t elems, int side,
                                                            int slices) {
  const int64_t d = blockIdx.x / slices;
  const int sl = blockIdx.x % slices;
  const int64_t m = map[d];
  const int64_t lo = (int64_t)sl * 4096, hi = min(elems, lo + 4096);
  float4* dp = reinterpret_cast<float4*>(dst + d * elems);
  if (m >= 0) {
    const float4* sp = reinterpret_cast<const float4*>(src + m * elems);
    for (int64_t e = lo / 4 + threadIdx.x; e < hi / 4; e += 256) dp[e] = __ldg(sp + e);
  } else {
    for (int64_t e = lo / 4 + threadIdx.x; e < hi / 4; e += 256) {
      float v[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int64_t f = 4 * e + q;
        v[q] = (side > 0 && f / side == f % side) ? 0.f : -1e9f;
      }
      dp[e] = make_float4(v[0], v[1], v[2], v[3]);
    }
  }
}
}  // namespace
}  // namespace gbmm

extern "C" int gbmm_gather_blocks_f32(const float* src, float* dst, const int64_t* map, int64_t blocks, int64_t elems,
                                      int side, void* stream) {
  if (blocks < 0 || elems < 0 || (elems & 3)) return GBMM_ERR_INVALID_ARG;
  if (blocks == 0 || elems == 0) return GBMM_OK;
  if (!src || !dst || !map || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15))
    return GBMM_ERR_INVALID_ARG;
  const int64_t slices = (elems + 4095) / 4096;
  if (blocks * slices >= (1LL << 31) || slices >= (1LL << 30)) return GBMM_ERR_UNSUPPORTED;
  gbmm::gather_blocks_kernel<<<(unsigned)(blocks * slices), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, dst, map, elems, side, (int)slices);
  return gbmm::launch_status();
}
