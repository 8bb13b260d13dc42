// Launch parameters shared by the fused VQ / two-level aggregation kernels.
#pragma once
#include "common.cuh"

namespace f2c {

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
};

// Streamed (fused_vq_stream.cu) or register-prefetch (fused_vq_fast.cu) kernel for the common shapes, by `variant`
// (an f2c_kernel value); sets *served = false (and launches nothing) when the shape is not one of theirs.
int launch_vq_fast(VqParams& p, int hot_bits, int index_dtype, int variant, cudaStream_t st, const char* op, bool* served);

// Hot-row slot of source node `id`: looked up, or - with hot-first numbering (no slot array) - the id itself.
__device__ __forceinline__ int hot_slot_of(const VqParams& p, int64_t id) {
  if (p.slot != nullptr) return __ldg(p.slot + id);
  return id < p.n_hot ? (int)id : -1;
}

}  // namespace f2c
