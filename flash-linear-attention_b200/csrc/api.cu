// Error reporting and version entry points of the C ABI.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace flab {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int check_launch(const char *what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: launch failed: %s", what, cudaGetErrorString(e));
    return FLAB_E_LAUNCH;
  }
  return FLAB_OK;
}

}  // namespace flab

extern "C" {
int flab_abi_version(void) { return FLAB_ABI_VERSION; }
const char *flab_last_error(void) { return flab::g_err; }
}
