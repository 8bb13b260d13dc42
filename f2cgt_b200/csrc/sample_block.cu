// One hop of a minibatch block in ONE library call: neighbour sampling + relabelling, i.e. what the reference's loader does
// per hop with csr_sampling followed by tensor_relabel([seeds, sub_indices]) (examples/dataloader.py:167-182; both
// operators live in its absent ShmTensor submodule).  The pieces are the library's own sampler and relabel kernels
// (sampler.cu, relabel.cu) and two prefix sums; doing the sequence here instead of from the host language removes
// ~15 host-side tensor operations and two of three host synchronisations per hop - the training step is bound by
// exactly that overhead.
//
// Sizes the host does not know yet are replaced by upper bounds: the sampled ids go to keys[n_seeds ...] with capacity
// n_seeds * num_pick (the unused tail holds copies of seeds[0], a valid id that changes nothing in the numbering), and
// `unique` has room for every key.  The three numbers the host needs afterwards (edges sampled, distinct nodes, error
// flag) are written to a small device header that the caller reads once.
#include <cub/device/device_scan.cuh>

#include "common.cuh"

namespace f2c {

template <typename IdxT>
__global__ void sample_block_copy_seeds_kernel(const IdxT* __restrict__ seeds, IdxT* __restrict__ keys, IdxT* __restrict__ deg_tail,
                                               int64_t n_seeds) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_seeds) keys[i] = seeds[i];
  if (i == 0) *deg_tail = 0;  // the scan runs over n_seeds + 1 degrees; the last one is zero
}

template <typename IdxT>
__global__ void sample_block_finish_kernel(const IdxT* __restrict__ sub_indptr, const IdxT* __restrict__ rank,
                                           const int32_t* __restrict__ first, const int32_t* __restrict__ error, int64_t n_seeds,
                                           int64_t n_keys, int64_t* __restrict__ header) {
  header[0] = (int64_t)sub_indptr[n_seeds];
  header[1] = (int64_t)rank[n_keys - 1] + first[n_keys - 1];
  header[2] = (int64_t)*error;
  header[3] = 0;
}

struct BlockWorkspace {
  size_t table_keys, table_pos, first, rank, deg, error, scan, scan_bytes, total;
};

static BlockWorkspace plan_block_workspace(int64_t n_seeds, int num_pick, int index_dtype) {
  const int64_t n_keys = n_seeds + n_seeds * num_pick;
  const size_t idx = (size_t)dtype_size(index_dtype);
  const size_t cap = (size_t)f2c_relabel_capacity(n_keys);
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  BlockWorkspace w{};
  size_t at = 0;
  w.table_keys = at; at += up(cap * 8);
  w.table_pos = at; at += up(cap * 4);
  w.first = at; at += up((size_t)n_keys * 4);
  w.rank = at; at += up((size_t)n_keys * idx);
  w.deg = at; at += up((size_t)(n_seeds + 1) * idx);
  w.error = at; at += 256;
  size_t a = 0, b = 0;
  if (index_dtype == F2C_I32) {
    cub::DeviceScan::ExclusiveSum(nullptr, a, (const int32_t*)nullptr, (int32_t*)nullptr, (int)(n_seeds + 1));
    cub::DeviceScan::ExclusiveSum(nullptr, b, (const int32_t*)nullptr, (int32_t*)nullptr, (int)n_keys);
  } else {
    cub::DeviceScan::ExclusiveSum(nullptr, a, (const int64_t*)nullptr, (int64_t*)nullptr, (int)(n_seeds + 1));
    cub::DeviceScan::ExclusiveSum(nullptr, b, (const int32_t*)nullptr, (int64_t*)nullptr, (int)n_keys);
  }
  w.scan = at;
  w.scan_bytes = a > b ? a : b;
  at += up(w.scan_bytes + 1);
  w.total = at;
  return w;
}

template <typename IdxT>
static int run_sample_block(const void* indptr, const void* indices, const void* seeds, int index_dtype, int64_t n_seeds, int num_pick,
                            uint64_t rng_seed, uint64_t rng_offset, void* sub_indptr, void* keys, void* unique, void* relabelled,
                            int64_t* header, unsigned char* ws, const BlockWorkspace& w, cudaStream_t st) {
  const char* op = "sample_block";
  const int64_t cap_edges = n_seeds * num_pick, n_keys = n_seeds + cap_edges;
  IdxT* deg = reinterpret_cast<IdxT*>(ws + w.deg);
  int32_t* first = reinterpret_cast<int32_t*>(ws + w.first);
  IdxT* rank = reinterpret_cast<IdxT*>(ws + w.rank);
  int32_t* error = reinterpret_cast<int32_t*>(ws + w.error);
  IdxT* keys_t = reinterpret_cast<IdxT*>(keys);
  // 1. degrees, seeds into the head of the key buffer
  int rc = f2c_sample_degrees(indptr, seeds, deg, index_dtype, n_seeds, num_pick, st);
  if (rc) return rc;
  sample_block_copy_seeds_kernel<IdxT><<<(unsigned)ceil_div(n_seeds, 256), 256, 0, st>>>((const IdxT*)seeds, keys_t, deg + n_seeds, n_seeds);
  // 2. CSC offsets of the block
  size_t scan_bytes = w.scan_bytes;
  cudaError_t e = cub::DeviceScan::ExclusiveSum(ws + w.scan, scan_bytes, (const IdxT*)deg, (IdxT*)sub_indptr, (int)(n_seeds + 1), st);
  if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "%s: scan of the degrees: %s", op, cudaGetErrorString(e));
  // 3. sampled neighbour ids behind the seeds (tail padded with seeds[0])
  rc = f2c_sample_neighbors(indptr, indices, seeds, sub_indptr, keys_t + n_seeds, cap_edges, index_dtype, n_seeds, num_pick, rng_seed,
                            rng_offset, st);
  if (rc) return rc;
  // 4. relabel [seeds, sampled ids]: first occurrences, their ranks, new numbers
  const int64_t capacity = f2c_relabel_capacity(n_keys);
  rc = f2c_relabel_mark(keys, index_dtype, n_keys, ws + w.table_keys, ws + w.table_pos, capacity, first, error, st);
  if (rc) return rc;
  scan_bytes = w.scan_bytes;
  e = cub::DeviceScan::ExclusiveSum(ws + w.scan, scan_bytes, (const int32_t*)first, rank, (int)n_keys, st);
  if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "%s: scan of the first occurrences: %s", op, cudaGetErrorString(e));
  rc = f2c_relabel_assign(keys, index_dtype, n_keys, ws + w.table_keys, ws + w.table_pos, capacity, first, rank, unique, relabelled, st);
  if (rc) return rc;
  sample_block_finish_kernel<IdxT><<<1, 1, 0, st>>>((const IdxT*)sub_indptr, rank, first, error, n_seeds, n_keys, header);
  return check_launch(op);
}

}  // namespace f2c

using namespace f2c;

extern "C" int64_t f2c_sample_block_workspace(int64_t n_seeds, int num_pick, int index_dtype) {
  if (n_seeds <= 0 || num_pick < 1 || !is_index_dtype(index_dtype)) return 0;
  return (int64_t)plan_block_workspace(n_seeds, num_pick, index_dtype).total;
}

extern "C" int f2c_sample_block(const void* indptr, const void* indices, const void* seeds, int index_dtype, int64_t n_seeds,
                                int num_pick, uint64_t rng_seed, uint64_t rng_offset, void* sub_indptr, void* keys, void* unique,
                                void* relabelled, int64_t* header_device, void* workspace, int64_t workspace_bytes, void* stream) {
  const char* op = "sample_block";
  F2C_REQUIRE(is_index_dtype(index_dtype), F2C_ERR_UNSUPPORTED, "%s: ids must be int32 or int64", op);
  F2C_REQUIRE(n_seeds >= 1 && num_pick >= 1 && num_pick <= 64, F2C_ERR_LIMIT, "%s: needs at least one seed and num_pick in [1, 64]", op);
  F2C_REQUIRE(n_seeds * (int64_t)(num_pick + 1) < (1ll << 31), F2C_ERR_LIMIT, "%s: at most 2^31 - 1 ids per hop", op);
  F2C_REQUIRE(indptr && seeds && sub_indptr && keys && unique && relabelled && header_device && workspace, F2C_ERR_INVALID,
              "%s: null pointer", op);
  const BlockWorkspace w = plan_block_workspace(n_seeds, num_pick, index_dtype);
  F2C_REQUIRE(workspace_bytes >= (int64_t)w.total && aligned(workspace, 256), F2C_ERR_INVALID,
              "%s: the workspace must hold f2c_sample_block_workspace() bytes and be 256-byte aligned", op);
  cudaStream_t st = (cudaStream_t)stream;
  if (index_dtype == F2C_I32)
    return run_sample_block<int32_t>(indptr, indices, seeds, index_dtype, n_seeds, num_pick, rng_seed, rng_offset, sub_indptr, keys, unique,
                                     relabelled, header_device, (unsigned char*)workspace, w, st);
  return run_sample_block<int64_t>(indptr, indices, seeds, index_dtype, n_seeds, num_pick, rng_seed, rng_offset, sub_indptr, keys, unique,
                                   relabelled, header_device, (unsigned char*)workspace, w, st);
}
