// Error plumbing and version of the C ABI (include/f2cgt_b200.h).
#include <mutex>

#include "common.cuh"
#include "stream_pipe.cuh"

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

int sm_count(int device) {
  static std::mutex mu;
  static int cached[64] = {};
  if (device < 0 || device >= 64) return kSmCount;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n < 1) {
      (void)cudaGetLastError();
      n = kSmCount;
    }
    cached[device] = n;
  }
  return cached[device];
}

int current_sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
  return sm_count(dev);
}

// Word that kernels with bounded waits raise when a wait runs out; one per device (it lives in the device image).
static __device__ int g_wait_expired;

int* stream_error_word() {
  static std::mutex mu;
  static int* word_of_device[64] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (word_of_device[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_wait_expired) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    word_of_device[dev] = (int*)ptr;
  }
  return word_of_device[dev];
}

}  // namespace f2c

extern "C" int f2c_device_status(int32_t* code_host, void* stream) {
  using namespace f2c;
  F2C_REQUIRE(code_host != nullptr, F2C_ERR_INVALID, "device_status: null pointer");
  int* word = stream_error_word();
  F2C_REQUIRE(word != nullptr, F2C_ERR_CUDA, "device_status: the status word of this device is not reachable");
  cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaMemcpy(code_host, word, sizeof(int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && *code_host != 0) e = cudaMemset(word, 0, sizeof(int));
  if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
  return F2C_OK;
}

extern "C" const char* f2c_last_error(void) { return f2c::g_error; }
extern "C" int f2c_version(void) { return 100; }
