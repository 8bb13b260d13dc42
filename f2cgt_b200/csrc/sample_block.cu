// One hop of a minibatch block in ONE kernel: neighbour sampling + relabelling, i.e. what the reference's loader does per hop
// with csr_sampling followed by tensor_relabel([seeds, sub_indices]) (examples/dataloader.py:167-182; both operators live
// in its absent ShmTensor submodule).  Same draws and same numbering as the separate entry points (sampler.cu,
// relabel.cu: the device code is shared through block_build.cuh); what changes is the launch count.  Built from those
// entry points a hop is 12 small dependent kernels, three memsets and two host-visible sizes; a training step is bound by
// the host's launch rate, and three hops were 40 % of all launches of a step.  Here a hop is one cooperative kernel whose
// phases are separated by grid-wide barriers:
//
//   A  clear the hash table; per seed: degree = min(in-degree, num_pick); seeds -> keys[0 .. n_seeds)
//      every CTA owns a contiguous run of seeds: exclusive scan of its degrees, its total to cta_sum[]
//   B  CSC offsets = local scan + sum of the totals of the CTAs before; sampled ids -> keys[n_seeds + offset ...];
//      the unused tail of keys (the buffers are sized for num_pick neighbours per seed) = seeds[0]
//   C  insert keys[0 .. n_used) into the table, atomicMin of the position per distinct id
//   D  every CTA owns a contiguous run of keys: flag first occurrences, exclusive scan, total to cta_sum2[]
//   E  new number of a first occurrence = local scan + totals before; unique[number] = id; relabelled[i] = number of the
//      first occurrence of keys[i]; header = {edges, distinct ids, error}
//
// Sizes the host does not know yet are replaced by upper bounds: `keys`, `unique` and `relabelled` hold n_seeds *
// (num_pick + 1) entries; the three numbers the host needs afterwards are written to a small device header that the
// caller reads once.  The grid is what the device keeps resident (cooperative launch), so the barriers cannot starve.
#include <cooperative_groups.h>
#include <cub/block/block_scan.cuh>

#include <mutex>

#include "block_build.cuh"

namespace cg = cooperative_groups;

namespace f2c {

constexpr int kHopThreads = 256;
constexpr int kHopMaxCtas = 1024;  // cta_sum[] entries scanned in shared memory by every CTA

template <typename IdxT>
struct HopParams {
  const IdxT* indptr;
  const IdxT* indices;
  const IdxT* seeds;
  IdxT* sub_indptr;    // [n_seeds + 1]
  IdxT* keys;          // [n_keys]
  IdxT* unique;        // [n_keys]
  IdxT* relabelled;    // [n_keys]
  int64_t* header;     // [4]
  unsigned long long* tab_keys;  // [capacity]
  int32_t* tab_pos;              // [capacity]
  int32_t* local_rank;           // [n_keys]  scan of the first-occurrence flags inside the owning CTA's run
  int64_t* cta_sum;              // [2 * kHopMaxCtas]
  int32_t* error;
  int64_t n_seeds, n_keys, capacity;
  int num_pick;
  uint64_t rng_seed, rng_offset;
};

// exclusive prefix of cta_sum[0 .. n) into shared memory (n <= kHopMaxCtas), returns the grand total; all threads call
__device__ __forceinline__ int64_t scan_cta_sums(const int64_t* __restrict__ sums, int n, int64_t* __restrict__ prefix_smem) {
  using Scan = cub::BlockScan<int64_t, kHopThreads>;
  __shared__ typename Scan::TempStorage tmp;
  __shared__ int64_t carry_smem;
  if (threadIdx.x == 0) carry_smem = 0;
  __syncthreads();
  for (int base = 0; base < n; base += kHopThreads) {
    const int i = base + (int)threadIdx.x;
    const int64_t v = i < n ? sums[i] : 0;
    int64_t ex, total;
    Scan(tmp).ExclusiveSum(v, ex, total);
    const int64_t carry = carry_smem;
    if (i < n) prefix_smem[i] = carry + ex;
    __syncthreads();
    if (threadIdx.x == 0) carry_smem = carry + total;
    __syncthreads();
  }
  return carry_smem;
}

template <typename IdxT>
__global__ void __launch_bounds__(kHopThreads) sample_block_kernel(const HopParams<IdxT> p) {
  cg::grid_group grid = cg::this_grid();
  using Scan = cub::BlockScan<int64_t, kHopThreads>;
  __shared__ typename Scan::TempStorage scan_tmp;
  __shared__ int64_t prefix[kHopMaxCtas];
  __shared__ int64_t run_carry;
  const int tid = (int)threadIdx.x, cta = (int)blockIdx.x, n_cta = (int)gridDim.x;
  const int64_t gtid = (int64_t)cta * kHopThreads + tid, gthreads = (int64_t)n_cta * kHopThreads;

  // ---- A: clear the table, degrees, local scan of the degrees
  for (int64_t s = gtid; s < p.capacity; s += gthreads) {
    p.tab_keys[s] = kEmptyKey;
    p.tab_pos[s] = 0x7fffffff;
  }
  if (gtid == 0) *p.error = 0;
  const int64_t seeds_per_cta = (p.n_seeds + n_cta - 1) / n_cta;
  const int64_t seed_lo = min((int64_t)cta * seeds_per_cta, p.n_seeds), seed_hi = min(seed_lo + seeds_per_cta, p.n_seeds);
  if (tid == 0) run_carry = 0;
  __syncthreads();
  for (int64_t base = seed_lo; base < seed_hi; base += kHopThreads) {
    const int64_t i = base + tid;
    int64_t deg = 0;
    if (i < seed_hi) {
      const IdxT v = p.seeds[i];
      p.keys[i] = v;
      const int64_t d = (int64_t)p.indptr[(int64_t)v + 1] - (int64_t)p.indptr[(int64_t)v];
      deg = d < p.num_pick ? d : p.num_pick;
    }
    int64_t ex, total;
    Scan(scan_tmp).ExclusiveSum(deg, ex, total);
    const int64_t carry = run_carry;
    if (i < seed_hi) p.sub_indptr[i] = (IdxT)(carry + ex);  // relative to this CTA's run until phase B
    __syncthreads();
    if (tid == 0) run_carry = carry + total;
    __syncthreads();
  }
  if (tid == 0) p.cta_sum[cta] = run_carry;
  grid.sync();

  // ---- B: global offsets, the draws, the tail
  const int64_t n_edges = scan_cta_sums(p.cta_sum, n_cta, prefix);
  const int64_t n_used = p.n_seeds + n_edges;
  {
    const int64_t mine = prefix[cta];
    for (int64_t i = seed_lo + tid; i < seed_hi; i += kHopThreads) {
      const int64_t off = (int64_t)p.sub_indptr[i] + mine;
      p.sub_indptr[i] = (IdxT)off;
      sample_one_seed(p.indptr, p.indices, (int64_t)p.seeds[i], i, p.keys + p.n_seeds + off, p.num_pick, p.rng_seed, p.rng_offset);
    }
    if (gtid == 0) p.sub_indptr[p.n_seeds] = (IdxT)n_edges;
    const IdxT fill = p.seeds[0];
    for (int64_t j = n_used + gtid; j < p.n_keys; j += gthreads) {
      p.keys[j] = fill;
      p.relabelled[j] = 0;  // seeds[0] is the first key, so its new number is 0
    }
  }
  grid.sync();

  // ---- C: every distinct id remembers the smallest position at which it occurs
  const int64_t cap_mask = p.capacity - 1;
  for (int64_t i = gtid; i < n_used; i += gthreads) {
    const int64_t key = (int64_t)p.keys[i];
    // ids must be >= 0: -1 is the table's empty marker
    if (key < 0) { atomicExch(p.error, 2); continue; }
    const int64_t slot = find_or_insert(p.tab_keys, cap_mask, (unsigned long long)key);
    if (slot < 0) { atomicExch(p.error, 1); continue; }
    atomicMin(p.tab_pos + slot, (int32_t)i);
  }
  grid.sync();

  // ---- D: first occurrences, scanned inside every CTA's run of keys
  const int64_t keys_per_cta = (n_used + n_cta - 1) / n_cta;
  const int64_t key_lo = min((int64_t)cta * keys_per_cta, n_used), key_hi = min(key_lo + keys_per_cta, n_used);
  if (tid == 0) run_carry = 0;
  __syncthreads();
  for (int64_t base = key_lo; base < key_hi; base += kHopThreads) {
    const int64_t i = base + tid;
    int64_t first = 0;
    if (i < key_hi) {
      const int64_t slot = find(p.tab_keys, cap_mask, (unsigned long long)(int64_t)p.keys[i]);
      first = (slot >= 0 && p.tab_pos[slot] == (int32_t)i) ? 1 : 0;
    }
    int64_t ex, total;
    Scan(scan_tmp).ExclusiveSum(first, ex, total);
    const int64_t carry = run_carry;
    if (i < key_hi) p.local_rank[i] = (int32_t)(carry + ex);
    __syncthreads();
    if (tid == 0) run_carry = carry + total;
    __syncthreads();
  }
  if (tid == 0) p.cta_sum[kHopMaxCtas + cta] = run_carry;
  grid.sync();

  // ---- E: numbers
  const int64_t n_unique = scan_cta_sums(p.cta_sum + kHopMaxCtas, n_cta, prefix);
  for (int64_t i = gtid; i < n_used; i += gthreads) {
    const IdxT key = p.keys[i];
    const int64_t slot = find(p.tab_keys, cap_mask, (unsigned long long)(int64_t)key);
    const int64_t pos = slot >= 0 ? (int64_t)p.tab_pos[slot] : i;  // slot < 0 only after an error that phase C has flagged
    const int64_t number = (int64_t)p.local_rank[pos] + prefix[pos / keys_per_cta];
    p.relabelled[i] = (IdxT)number;
    if (pos == i) p.unique[number] = key;
  }
  if (gtid == 0) {
    p.header[0] = n_edges;
    p.header[1] = n_unique;
    p.header[2] = (int64_t)*p.error;
    p.header[3] = 0;
  }
}

struct HopWorkspace {
  size_t table_keys, table_pos, local_rank, cta_sum, error, total;
};

static HopWorkspace plan_hop_workspace(int64_t n_seeds, int num_pick) {
  const int64_t n_keys = n_seeds + n_seeds * num_pick;
  const size_t cap = (size_t)f2c_relabel_capacity(n_keys);
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  HopWorkspace w{};
  size_t at = 0;
  w.table_keys = at; at += up(cap * 8);
  w.table_pos = at; at += up(cap * 4);
  w.local_rank = at; at += up((size_t)n_keys * 4);
  w.cta_sum = at; at += up((size_t)2 * kHopMaxCtas * 8);
  w.error = at; at += 256;
  w.total = at;
  return w;
}

// CTAs of the hop kernel the device keeps resident, per device (one occupancy query each)
template <typename IdxT>
static int resident_hop_ctas(int dev) {
  static std::mutex m;
  static int cached[64] = {};
  std::lock_guard<std::mutex> lock(m);
  int& slot = cached[dev & 63];
  if (slot == 0) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sample_block_kernel<IdxT>, kHopThreads, 0) != cudaSuccess || per_sm < 1)
      per_sm = 1;
    // two CTAs per SM are enough to cover the memory latency of the table probes, and leave room for the kernels of
    // the training stream this hop usually runs beside
    if (per_sm > 2) per_sm = 2;
    int n = per_sm * sm_count(dev);
    slot = n > kHopMaxCtas ? kHopMaxCtas : n;
  }
  return slot;
}

template <typename IdxT>
static int run_sample_block(const void* indptr, const void* indices, const void* seeds, int64_t n_seeds, int num_pick, uint64_t rng_seed,
                            uint64_t rng_offset, void* sub_indptr, void* keys, void* unique, void* relabelled, int64_t* header,
                            unsigned char* ws, const HopWorkspace& w, cudaStream_t st) {
  const char* op = "sample_block";
  HopParams<IdxT> p;
  p.indptr = (const IdxT*)indptr; p.indices = (const IdxT*)indices; p.seeds = (const IdxT*)seeds;
  p.sub_indptr = (IdxT*)sub_indptr; p.keys = (IdxT*)keys; p.unique = (IdxT*)unique; p.relabelled = (IdxT*)relabelled;
  p.header = header;
  p.tab_keys = reinterpret_cast<unsigned long long*>(ws + w.table_keys);
  p.tab_pos = reinterpret_cast<int32_t*>(ws + w.table_pos);
  p.local_rank = reinterpret_cast<int32_t*>(ws + w.local_rank);
  p.cta_sum = reinterpret_cast<int64_t*>(ws + w.cta_sum);
  p.error = reinterpret_cast<int32_t*>(ws + w.error);
  p.n_seeds = n_seeds; p.n_keys = n_seeds + n_seeds * num_pick; p.capacity = f2c_relabel_capacity(p.n_keys);
  p.num_pick = num_pick; p.rng_seed = rng_seed; p.rng_offset = rng_offset;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
  int grid = resident_hop_ctas<IdxT>(dev);
  // no more CTAs than there are tiles of keys (every CTA still takes part in every barrier)
  const int64_t tiles = ceil_div(p.n_keys, kHopThreads);
  if ((int64_t)grid > tiles) grid = (int)tiles;
  void* args[] = {(void*)&p};
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)sample_block_kernel<IdxT>, dim3((unsigned)grid), dim3(kHopThreads), args, 0, st);
  if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "%s: cooperative launch: %s", op, cudaGetErrorString(e));
  return check_launch(op);
}

}  // namespace f2c

using namespace f2c;

extern "C" int64_t f2c_sample_block_workspace(int64_t n_seeds, int num_pick, int index_dtype) {
  if (n_seeds <= 0 || num_pick < 1 || num_pick > kMaxPick || !is_index_dtype(index_dtype)) return 0;
  return (int64_t)plan_hop_workspace(n_seeds, num_pick).total;
}

extern "C" int f2c_sample_block(const void* indptr, const void* indices, const void* seeds, int index_dtype, int64_t n_seeds,
                                int num_pick, uint64_t rng_seed, uint64_t rng_offset, void* sub_indptr, void* keys, void* unique,
                                void* relabelled, int64_t* header_device, void* workspace, int64_t workspace_bytes, void* stream) {
  const char* op = "sample_block";
  F2C_REQUIRE(is_index_dtype(index_dtype), F2C_ERR_UNSUPPORTED, "%s: ids must be int32 or int64", op);
  F2C_REQUIRE(n_seeds >= 1 && num_pick >= 1 && num_pick <= kMaxPick, F2C_ERR_LIMIT, "%s: needs at least one seed and num_pick in [1, %d]",
              op, kMaxPick);
  F2C_REQUIRE(n_seeds * (int64_t)(num_pick + 1) < (1ll << 31), F2C_ERR_LIMIT, "%s: at most 2^31 - 1 ids per hop", op);
  F2C_REQUIRE(indptr && seeds && sub_indptr && keys && unique && relabelled && header_device && workspace, F2C_ERR_INVALID,
              "%s: null pointer", op);
  // the workspace may be larger (sized for a bigger hop); the layout is that of THIS hop
  const HopWorkspace w = plan_hop_workspace(n_seeds, num_pick);
  F2C_REQUIRE(workspace_bytes >= (int64_t)w.total && aligned(workspace, 256), F2C_ERR_INVALID,
              "%s: the workspace must hold f2c_sample_block_workspace() bytes and be 256-byte aligned", op);
  cudaStream_t st = (cudaStream_t)stream;
  if (index_dtype == F2C_I32)
    return run_sample_block<int32_t>(indptr, indices, seeds, n_seeds, num_pick, rng_seed, rng_offset, sub_indptr, keys, unique, relabelled,
                                     header_device, (unsigned char*)workspace, w, st);
  return run_sample_block<int64_t>(indptr, indices, seeds, n_seeds, num_pick, rng_seed, rng_offset, sub_indptr, keys, unique, relabelled,
                                   header_device, (unsigned char*)workspace, w, st);
}
