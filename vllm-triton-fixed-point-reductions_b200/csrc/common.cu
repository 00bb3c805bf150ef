// Status strings, per-thread error text and launch checking for the C ABI.
#include <cstdlib>
#include <stdio.h>
#include <string.h>

#include "fxp_common.cuh"

namespace fxpr {

static thread_local char g_last_error[512] = {0};

void set_last_error(const char* what, cudaError_t err) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", what,
           cudaGetErrorString(err), cudaGetErrorName(err));
}

void set_last_error_text(const char* text) {
  snprintf(g_last_error, sizeof(g_last_error), "%s", text);
}

// Launch errors are reported without synchronising: only configuration errors
// (bad grid, too much shared memory, no kernel image) surface here, which is what
// a caller inside a CUDA-graph capture can still act on.
int check_launch(const char* what) {
  cudaError_t err = cudaPeekAtLastError();
  if (err != cudaSuccess) {
    set_last_error(what, err);
    cudaGetLastError();  // clear the sticky launch-config error
    return FXPR_ERR_CUDA;
  }
  return FXPR_OK;
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("FXPR_NO_PDL");
    return !(v && v[0] == '1');
  }();
  return on;
}

}  // namespace fxpr

extern "C" int fxpr_version(void) { return 100; }

extern "C" const char* fxpr_last_error(void) { return fxpr::g_last_error; }

extern "C" const char* fxpr_status_string(int status) {
  switch (status) {
    case FXPR_OK: return "ok";
    case FXPR_ERR_BAD_ARG: return "bad argument";
    case FXPR_ERR_UNSUPPORTED: return "unsupported dtype or layout";
    case FXPR_ERR_SCRATCH: return "scratch buffer missing or too small";
    case FXPR_ERR_CUDA: return "CUDA call failed";
    case FXPR_ERR_TIMEOUT: return "device-side wait timed out";
    case FXPR_ERR_ARCH: return "device is not compute capability 10.x";
  }
  return "unknown status";
}
