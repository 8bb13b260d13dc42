// Uniform neighbour sampling without replacement over a CSC graph - the GPU stand-in for the
// `csr_sampling(indptr, indices, seeds, num_pick, replace=False)` operator the reference imports from
// its (absent) ShmTensor submodule (call sites examples/dataloader.py:174-175,287-288): for every seed,
// all in-neighbours when it has at most num_pick of them, otherwise num_pick distinct ones, each subset
// equally likely.  Output is a CSC over the seeds holding GLOBAL neighbour ids.
//
// Two launches around a prefix sum the caller owns: `f2c_sample_degrees` writes min(deg, num_pick) per
// seed, `f2c_sample_neighbors` fills the indices at the offsets of the scanned degrees.  One thread
// per seed runs Floyd's subset algorithm (num_pick <= 64 draws, chosen positions kept in registers /
// local memory); draws come from Philox4x32-10 keyed by the caller's seed with the seed node's
// position as counter, so a sample is reproducible and independent of launch geometry.
#include "block_build.cuh"

namespace f2c {

template <typename IdxT>
__global__ void __launch_bounds__(256) sample_degrees_kernel(const IdxT* __restrict__ indptr, const IdxT* __restrict__ seeds,
                                                             IdxT* __restrict__ out_deg, int64_t n_seeds, int num_pick) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_seeds) return;
  int64_t v = (int64_t)seeds[i];
  int64_t d = (int64_t)indptr[v + 1] - (int64_t)indptr[v];
  out_deg[i] = (IdxT)(d < num_pick ? d : num_pick);
}

template <typename IdxT>
__global__ void __launch_bounds__(256) sample_neighbors_kernel(const IdxT* __restrict__ indptr, const IdxT* __restrict__ indices,
                                                               const IdxT* __restrict__ seeds, const IdxT* __restrict__ out_indptr,
                                                               IdxT* __restrict__ out_indices, int64_t n_seeds, int num_pick,
                                                               uint64_t rng_seed, uint64_t rng_offset) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_seeds) return;
  sample_one_seed(indptr, indices, (int64_t)seeds[i], i, out_indices + (int64_t)out_indptr[i], num_pick, rng_seed, rng_offset);
}

// Entries [out_indptr[n_seeds], capacity) of an over-allocated index buffer get the id of the first seed: a valid,
// already present id, so that relabelling the whole buffer gives the same numbering as relabelling its used part.
template <typename IdxT>
__global__ void __launch_bounds__(256) sample_fill_tail_kernel(const IdxT* __restrict__ seeds, const IdxT* __restrict__ out_indptr,
                                                               IdxT* __restrict__ out_indices, int64_t n_seeds, int64_t capacity) {
  const int64_t used = (int64_t)out_indptr[n_seeds];
  const IdxT fill = seeds[0];
  for (int64_t j = used + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < capacity; j += (int64_t)gridDim.x * blockDim.x)
    out_indices[j] = fill;
}

}  // namespace f2c

using namespace f2c;

extern "C" int f2c_sample_degrees(const void* indptr, const void* seeds, void* out_deg, int index_dtype, int64_t n_seeds,
                                  int num_pick, void* stream) {
  F2C_REQUIRE(is_index_dtype(index_dtype), F2C_ERR_UNSUPPORTED, "sample_degrees: ids must be int32 or int64");
  F2C_REQUIRE(n_seeds >= 0 && num_pick >= 1 && num_pick <= kMaxPick, F2C_ERR_LIMIT, "sample_degrees: num_pick must be in [1, %d]", kMaxPick);
  if (n_seeds == 0) return F2C_OK;
  F2C_REQUIRE(indptr && seeds && out_deg, F2C_ERR_INVALID, "sample_degrees: null pointer");
  unsigned grid = (unsigned)ceil_div(n_seeds, 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (index_dtype == F2C_I32)
    sample_degrees_kernel<int32_t><<<grid, 256, 0, st>>>((const int32_t*)indptr, (const int32_t*)seeds, (int32_t*)out_deg, n_seeds, num_pick);
  else
    sample_degrees_kernel<int64_t><<<grid, 256, 0, st>>>((const int64_t*)indptr, (const int64_t*)seeds, (int64_t*)out_deg, n_seeds, num_pick);
  return check_launch("sample_degrees");
}

extern "C" int f2c_sample_neighbors(const void* indptr, const void* indices, const void* seeds, const void* out_indptr,
                                    void* out_indices, int64_t out_capacity, int index_dtype, int64_t n_seeds, int num_pick,
                                    uint64_t rng_seed, uint64_t rng_offset, void* stream) {
  F2C_REQUIRE(is_index_dtype(index_dtype), F2C_ERR_UNSUPPORTED, "sample_neighbors: ids must be int32 or int64");
  F2C_REQUIRE(n_seeds >= 0 && num_pick >= 1 && num_pick <= kMaxPick, F2C_ERR_LIMIT, "sample_neighbors: num_pick must be in [1, %d]", kMaxPick);
  if (n_seeds == 0) return F2C_OK;
  F2C_REQUIRE(indptr && seeds && out_indptr && out_capacity >= 0, F2C_ERR_INVALID, "sample_neighbors: null pointer or negative capacity");
  unsigned grid = (unsigned)ceil_div(n_seeds, 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (index_dtype == F2C_I32)
    sample_neighbors_kernel<int32_t><<<grid, 256, 0, st>>>((const int32_t*)indptr, (const int32_t*)indices, (const int32_t*)seeds,
                                                           (const int32_t*)out_indptr, (int32_t*)out_indices, n_seeds, num_pick,
                                                           rng_seed, rng_offset);
  else
    sample_neighbors_kernel<int64_t><<<grid, 256, 0, st>>>((const int64_t*)indptr, (const int64_t*)indices, (const int64_t*)seeds,
                                                           (const int64_t*)out_indptr, (int64_t*)out_indices, n_seeds, num_pick,
                                                           rng_seed, rng_offset);
  int rc = check_launch("sample_neighbors");
  if (rc || out_capacity <= 0) return rc;
  // the caller sized out_indices for the worst case (n_seeds * num_pick) instead of reading the edge count back
  unsigned tail_grid = (unsigned)ceil_div(out_capacity, 256 * 8);
  if (tail_grid > 1024u) tail_grid = 1024u;
  if (index_dtype == F2C_I32)
    sample_fill_tail_kernel<int32_t><<<tail_grid, 256, 0, st>>>((const int32_t*)seeds, (const int32_t*)out_indptr, (int32_t*)out_indices, n_seeds, out_capacity);
  else
    sample_fill_tail_kernel<int64_t><<<tail_grid, 256, 0, st>>>((const int64_t*)seeds, (const int64_t*)out_indptr, (int64_t*)out_indices, n_seeds, out_capacity);
  return check_launch("sample_neighbors (tail)");
}
