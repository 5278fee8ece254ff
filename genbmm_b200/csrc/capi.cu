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
