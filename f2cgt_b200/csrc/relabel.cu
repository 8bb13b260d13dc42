// Relabelling of a minibatch's node ids - the GPU stand-in for the `tensor_relabel([seeds, sub_indices])`
// operator the reference imports from its (absent) ShmTensor submodule (call sites
// examples/dataloader.py:176-177,289-290): the distinct ids of the concatenation become 0..n_unique-1 IN ORDER OF
// FIRST OCCURRENCE, so the seeds (which come first and are distinct) keep positions 0..len(seeds)-1 - the
// model slices h[:num_dst] (examples/conv.py:48-49) - and every id is replaced by its new number.
//
// An open-addressing hash table (64-bit keys, linear probing, capacity >= 2 n, so chains stay short) records for
// every distinct id the smallest position at which it occurs (atomicMin): that makes the numbering independent
// of thread scheduling.  Two launches around a prefix sum the caller owns, like the sampler:
//   f2c_relabel_mark    builds the table and writes first[i] = 1 where position i is a first occurrence;
//   (caller)            rank = exclusive prefix sum of first; n_unique = its total;
//   f2c_relabel_assign  writes unique[rank[i]] = keys[i] for first occurrences and relabelled[i] = rank[first position of keys[i]].
#include "block_build.cuh"

namespace f2c {

template <typename IdxT>
__global__ void __launch_bounds__(256) relabel_insert_kernel(const IdxT* __restrict__ keys, int64_t n, unsigned long long* tab_keys,
                                                             int32_t* tab_pos, int64_t cap_mask, int32_t* error) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t key = (int64_t)keys[i];
  // ids must be >= 0: -1 (the padding value of some samplers) is the table's empty marker and would share a slot with
  // whatever key claims it next; a negative id is reported instead of being numbered wrongly
  if (key < 0) { atomicExch(error, 2); return; }
  const int64_t slot = find_or_insert(tab_keys, cap_mask, (unsigned long long)key);
  if (slot < 0) { atomicExch(error, 1); return; }
  atomicMin(tab_pos + slot, (int32_t)i);
}

template <typename IdxT>
__global__ void __launch_bounds__(256) relabel_first_kernel(const IdxT* __restrict__ keys, int64_t n, const unsigned long long* tab_keys,
                                                            const int32_t* tab_pos, int64_t cap_mask, int32_t* first) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t slot = find(tab_keys, cap_mask, (unsigned long long)(int64_t)keys[i]);
  first[i] = (slot >= 0 && tab_pos[slot] == (int32_t)i) ? 1 : 0;
}

template <typename IdxT>
__global__ void __launch_bounds__(256) relabel_assign_kernel(const IdxT* __restrict__ keys, int64_t n, const unsigned long long* tab_keys,
                                                             const int32_t* tab_pos, int64_t cap_mask, const int32_t* __restrict__ first,
                                                             const IdxT* __restrict__ rank, IdxT* __restrict__ unique,
                                                             IdxT* __restrict__ relabelled) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const IdxT key = keys[i];
  const int64_t slot = find(tab_keys, cap_mask, (unsigned long long)(int64_t)key);
  const int32_t p = slot >= 0 ? tab_pos[slot] : (int32_t)i;
  relabelled[i] = rank[p];
  if (first[i]) unique[(int64_t)rank[i]] = key;
}

}  // namespace f2c

using namespace f2c;

extern "C" int64_t f2c_relabel_capacity(int64_t n_keys) {
  int64_t cap = 1024;
  while (cap < 2 * n_keys) cap <<= 1;
  return cap;
}

extern "C" int f2c_relabel_mark(const void* keys, int index_dtype, int64_t n_keys, void* table_keys, void* table_pos,
                                int64_t capacity, int32_t* first, int32_t* error_flag, void* stream) {
  const char* op = "relabel_mark";
  F2C_REQUIRE(is_index_dtype(index_dtype), F2C_ERR_UNSUPPORTED, "%s: ids must be int32 or int64", op);
  F2C_REQUIRE(n_keys >= 0 && n_keys < (1ll << 31), F2C_ERR_LIMIT, "%s: at most 2^31 - 1 ids", op);
  F2C_REQUIRE(capacity >= 2 * n_keys && capacity >= 2 && (capacity & (capacity - 1)) == 0, F2C_ERR_INVALID,
              "%s: capacity must be a power of two >= 2 n (use f2c_relabel_capacity)", op);
  F2C_REQUIRE(table_keys && table_pos && error_flag && (n_keys == 0 || (keys && first)), F2C_ERR_INVALID, "%s: null pointer", op);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(table_keys, 0xFF, (size_t)capacity * 8, st);
  if (e == cudaSuccess) e = cudaMemsetAsync(table_pos, 0x7F, (size_t)capacity * 4, st);
  if (e == cudaSuccess) e = cudaMemsetAsync(error_flag, 0, 4, st);
  if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "%s: %s", op, cudaGetErrorString(e));
  if (n_keys == 0) return F2C_OK;
  const unsigned grid = (unsigned)ceil_div(n_keys, 256);
  if (index_dtype == F2C_I32) {
    relabel_insert_kernel<int32_t><<<grid, 256, 0, st>>>((const int32_t*)keys, n_keys, (unsigned long long*)table_keys, (int32_t*)table_pos, capacity - 1, error_flag);
    relabel_first_kernel<int32_t><<<grid, 256, 0, st>>>((const int32_t*)keys, n_keys, (const unsigned long long*)table_keys, (const int32_t*)table_pos, capacity - 1, first);
  } else {
    relabel_insert_kernel<int64_t><<<grid, 256, 0, st>>>((const int64_t*)keys, n_keys, (unsigned long long*)table_keys, (int32_t*)table_pos, capacity - 1, error_flag);
    relabel_first_kernel<int64_t><<<grid, 256, 0, st>>>((const int64_t*)keys, n_keys, (const unsigned long long*)table_keys, (const int32_t*)table_pos, capacity - 1, first);
  }
  return check_launch(op);
}

extern "C" int f2c_relabel_assign(const void* keys, int index_dtype, int64_t n_keys, const void* table_keys, const void* table_pos,
                                  int64_t capacity, const int32_t* first, const void* rank, void* unique, void* relabelled,
                                  void* stream) {
  const char* op = "relabel_assign";
  F2C_REQUIRE(is_index_dtype(index_dtype), F2C_ERR_UNSUPPORTED, "%s: ids must be int32 or int64", op);
  F2C_REQUIRE(n_keys >= 0 && n_keys < (1ll << 31) && capacity >= 2 && (capacity & (capacity - 1)) == 0, F2C_ERR_INVALID,
              "%s: bad sizes", op);
  if (n_keys == 0) return F2C_OK;
  F2C_REQUIRE(keys && table_keys && table_pos && first && rank && unique && relabelled, F2C_ERR_INVALID, "%s: null pointer", op);
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = (unsigned)ceil_div(n_keys, 256);
  if (index_dtype == F2C_I32)
    relabel_assign_kernel<int32_t><<<grid, 256, 0, st>>>((const int32_t*)keys, n_keys, (const unsigned long long*)table_keys, (const int32_t*)table_pos,
                                                         capacity - 1, first, (const int32_t*)rank, (int32_t*)unique, (int32_t*)relabelled);
  else
    relabel_assign_kernel<int64_t><<<grid, 256, 0, st>>>((const int64_t*)keys, n_keys, (const unsigned long long*)table_keys, (const int32_t*)table_pos,
                                                         capacity - 1, first, (const int64_t*)rank, (int64_t*)unique, (int64_t*)relabelled);
  return check_launch(op);
}
