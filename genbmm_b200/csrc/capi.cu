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

extern "C" int gbmm_abi_version(void) { return 2; }

// ---- launch counter ------------------------------------------------------------------------------
// Every `kernel<<<...>>>(...)` in this library compiles to a call of the runtime's launch-configuration push
// followed by the launch itself.  The library is linked with `--wrap` on that symbol (genbmm_b200/build.py), so
// every kernel launch any entry point makes passes through the function below exactly once: the count is of
// launches actually issued, not an estimate kept beside them.  Memsets and copies are not kernels and are not
// counted.
#include <atomic>
namespace gbmm {
namespace {
std::atomic<unsigned long long> g_launches{0};
}
}  // namespace gbmm
extern "C" unsigned __real___cudaPushCallConfiguration(dim3 grid, dim3 block, size_t shared, struct CUstream_st* st);
extern "C" unsigned __wrap___cudaPushCallConfiguration(dim3 grid, dim3 block, size_t shared, struct CUstream_st* st) {
  gbmm::g_launches.fetch_add(1, std::memory_order_relaxed);
  return __real___cudaPushCallConfiguration(grid, block, shared, st);
}
extern "C" uint64_t gbmm_launch_count(void) { return gbmm::g_launches.load(std::memory_order_relaxed); }

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

// ---- NaN fill of an output whose product kernel gave up (see poison_if_failed in common.cuh) -------
namespace gbmm {
namespace {
__global__ void __launch_bounds__(256) poison_on_error_kernel(const int* __restrict__ error, float* out0,
                                                              int64_t count0, float* out1, int64_t count1) {
  if (!poison_if_failed(error, out0, count0)) return;
  poison_if_failed(error, out1, count1);
}
}  // namespace

int launch_poison_on_error(const int* error, float* out0, int64_t count0, float* out1, int64_t count1,
                           cudaStream_t st) {
  unsigned grid = 0;
  if (int rc = capped_grid(1LL << 20, &grid)) return rc;
  poison_on_error_kernel<<<grid, 256, 0, st>>>(error, out0, count0, out1, count1);
  return launch_status();
}
}  // namespace gbmm

extern "C" int gbmm_poison_on_error(const int32_t* error_word, float* out, int64_t count, void* stream) {
  if (!error_word || count < 0 || (count > 0 && !out)) return GBMM_ERR_INVALID_ARG;
  return gbmm::launch_poison_on_error(error_word, out, count, nullptr, 0, static_cast<cudaStream_t>(stream));
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
    if (hi - lo == 4096) {  // a whole slice: the thread's four loads are in flight together
      const int64_t e = lo / 4 + threadIdx.x;
      const float4 v0 = __ldg(sp + e), v1 = __ldg(sp + e + 256), v2 = __ldg(sp + e + 512), v3 = __ldg(sp + e + 768);
      dp[e] = v0;
      dp[e + 256] = v1;
      dp[e + 512] = v2;
      dp[e + 768] = v3;
    } else {
      for (int64_t e = lo / 4 + threadIdx.x; e < hi / 4; e += 256) dp[e] = __ldg(sp + e);
    }
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
