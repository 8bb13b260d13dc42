// Memory of a row-sharded table that other processes on the same box can map (no counterpart in the reference,
// which keeps one host replica per machine: examples/load_dataset.py:63-85).
//
// A shard is one cudaMalloc allocation of its own, exported with cudaIpcGetMemHandle; a consumer opens the
// handle WHILE ITS OWN GPU IS THE CURRENT DEVICE with cudaIpcMemLazyEnablePeerAccess, which is what maps the
// memory into that GPU's address space and enables peer access from it to the owner.  (A mapping opened while
// the owner's ordinal is current belongs to the owner's context in the consumer process and is not readable by
// kernels of the consumer's GPU.)  One allocation per shard also keeps every handle distinct, so the rule that
// a handle can be opened once per process is never met.
//
// These are the only entry points of the library that allocate or free device memory.
#include <string.h>

#include "common.cuh"
#include "vq_params.cuh"

namespace f2c {
#define F2C_IPC_CUDA(call)                                                                        \
  do {                                                                                            \
    cudaError_t e_ = (call);                                                                      \
    if (e_ != cudaSuccess) {                                                                      \
      (void)cudaGetLastError();                                                                   \
      return set_error(F2C_ERR_CUDA, "%s: %s failed: %s", op, #call, cudaGetErrorString(e_));   \
    }                                                                                             \
  } while (0)
int ensure_readable_from_current_device(const void* ptr, const char* op, const char* what, int index) {
  int here = 0;
  F2C_IPC_CUDA(cudaGetDevice(&here));
  F2C_REQUIRE(ptr != nullptr, F2C_ERR_INVALID, "%s: %s shard %d is null", op, what, index);
  cudaPointerAttributes attr{};
  F2C_IPC_CUDA(cudaPointerGetAttributes(&attr, ptr));
  F2C_REQUIRE(attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged, F2C_ERR_INVALID,
              "%s: %s shard %d is not device memory", op, what, index);
  if (attr.type == cudaMemoryTypeDevice && attr.device != here) {
    int can = 0;
    F2C_IPC_CUDA(cudaDeviceCanAccessPeer(&can, here, attr.device));
    F2C_REQUIRE(can, F2C_ERR_UNSUPPORTED, "%s: GPU %d cannot read %s shard %d on GPU %d (no peer access)", op, here, what, index,
                attr.device);
    cudaError_t e = cudaDeviceEnablePeerAccess(attr.device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
      (void)cudaGetLastError();
    } else {
      F2C_IPC_CUDA(e);
    }
  }
  return F2C_OK;
}

}  // namespace f2c

using namespace f2c;

static_assert(sizeof(cudaIpcMemHandle_t) == F2C_SHARD_HANDLE_BYTES, "handle size");

extern "C" int f2c_shard_create(const void* rows, int64_t bytes, void** shard, unsigned char* handle, void* stream) {
  const char* op = "shard_create";
  F2C_REQUIRE(bytes > 0 && rows != nullptr && shard != nullptr && handle != nullptr, F2C_ERR_INVALID,
              "%s: null pointer or empty shard", op);
  void* p = nullptr;
  F2C_IPC_CUDA(cudaMalloc(&p, (size_t)bytes));
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemcpyAsync(p, rows, (size_t)bytes, cudaMemcpyDeviceToDevice, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    (void)cudaFree(p);
    return set_error(F2C_ERR_CUDA, "%s: %s", op, cudaGetErrorString(e));
  }
  memcpy(handle, &h, sizeof(h));
  *shard = p;
  return F2C_OK;
}

extern "C" int f2c_shard_free(void* shard) {
  const char* op = "shard_free";
  if (shard == nullptr) return F2C_OK;
  F2C_IPC_CUDA(cudaFree(shard));
  return F2C_OK;
}

extern "C" int f2c_shard_open(const unsigned char* handle, void** shard) {
  const char* op = "shard_open";
  F2C_REQUIRE(handle != nullptr && shard != nullptr, F2C_ERR_INVALID, "%s: null pointer", op);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  F2C_IPC_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *shard = p;
  return F2C_OK;
}

extern "C" int f2c_shard_close(void* shard) {
  const char* op = "shard_close";
  if (shard == nullptr) return F2C_OK;
  F2C_IPC_CUDA(cudaIpcCloseMemHandle(shard));
  return F2C_OK;
}

extern "C" int f2c_shard_copy(void* dst, const void* src, int64_t bytes, void* stream) {
  const char* op = "shard_copy";
  F2C_REQUIRE(bytes >= 0 && (bytes == 0 || (dst != nullptr && src != nullptr)), F2C_ERR_INVALID, "%s: bad arguments", op);
  if (bytes == 0) return F2C_OK;
  F2C_IPC_CUDA(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, (cudaStream_t)stream));
  return F2C_OK;
}
