// Launch parameters shared by the fused VQ / two-level aggregation kernels.
#pragma once
#include "common.cuh"

namespace f2c {

// Row-sharded tables (PEER kernels): node row r (VQ codes, slot) lives on shard r / rps_nodes, hot row h on shard
// h / rps_hot; every shard is mapped into this process (own memory or CUDA-IPC peer mappings).
struct VqPeer {
  const uint8_t* code[8];
  const int32_t* slot[8];   // all null = hot-first numbering
  const uint8_t* hot[8];
  uint32_t rps_nodes, rps_hot;
  unsigned long long magic_nodes, magic_hot;  // floor(2^64 / rps) + 1: exact 32-bit division by one multiply-high
};

struct VqParams {
  const void* codes;       // [n_src, n_cb]
  const float* codebooks;  // [n_cb, K, cs]
  const void* indptr;
  const void* indices;
  float* out;
  int64_t n_dst;
  int n_cb, cs, feat_dim;
  uint32_t K;
  int code_kind;           // 0 u8, 1 i8, 2 i16
  int cb_per_part;         // codebooks (subspaces) handled by one blockIdx.y
  int reduce;
  int vec_store;
  DropoutArgs drop;
  // two-level extension
  const uint8_t* sq_codes;  // [n_hot, sq_row_bytes]
  const float* sq_codebooks;
  const int32_t* slot;      // [n_src] row of the SQ table or -1; nullptr = hot-first numbering: source s is hot iff s < n_hot, row s
  int64_t n_hot;
  int64_t sq_row_bytes;
  int sq_cs, sq_n_cb, sq_signed;
  // geometry of the codebooks staged by the pipelined kernel (fused_vq_fast.cu)
  int fast_stride;    // bytes between consecutive codes of one subspace in shared memory
  int fast_spq;       // subspaces interleaved per 128-byte line (1 = natural layout)
  int fast_cb_bytes;  // staged bytes per column part
  VqPeer peer;        // only read by PEER kernels
};

// Streamed (fused_vq_stream.cu) or register-prefetch (fused_vq_fast.cu) kernel for the common shapes, by `variant`
// (an f2c_kernel value); sets *served = false (and launches nothing) when the shape is not one of theirs.
int launch_vq_fast(VqParams& p, int hot_bits, int index_dtype, int variant, cudaStream_t st, const char* op, bool* served,
                   bool peer = false);

// Make sure the current device can read `ptr` (device memory of this or another GPU of the box): peer access is
// one-directional and is requested here when needed (idempotent).  Returns a status with the error text set.
int ensure_readable_from_current_device(const void* ptr, const char* op, const char* what, int index);

// Hot-row slot of source node `id`: looked up, or - with hot-first numbering (no slot array) - the id itself.
__device__ __forceinline__ int hot_slot_of(const VqParams& p, int64_t id) {
  if (p.slot != nullptr) return __ldg(p.slot + id);
  return id < p.n_hot ? (int)id : -1;
}

}  // namespace f2c
