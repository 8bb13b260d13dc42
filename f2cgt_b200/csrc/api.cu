// Error plumbing and version of the C ABI (include/f2cgt_b200.h).
#include "common.cuh"

namespace f2c {

static thread_local char g_error[512] = "";

int set_error(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return status;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return F2C_OK;
}

}  // namespace f2c

extern "C" const char* f2c_last_error(void) { return f2c::g_error; }
extern "C" int f2c_version(void) { return 100; }
