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
