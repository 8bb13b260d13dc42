// Device pieces shared by the minibatch builders: the per-seed neighbour draw (sampler.cu, sample_block.cu) and the
// hash table behind the first-occurrence numbering (relabel.cu, sample_block.cu).  One definition each, so the one-call
// hop and the separate entry points cannot drift apart.
#pragma once
#include "common.cuh"

namespace f2c {

constexpr int kMaxPick = 64;

// All in-neighbours of `v` when it has at most num_pick of them, else num_pick distinct ones (Floyd's subset algorithm:
// for j = d-k .. d-1: t = U{0..j}; take t unless already taken, then take j).  Draws: Philox4x32-10 keyed by the
// caller's seed with the seed node's POSITION as counter, so a sample does not depend on launch geometry.
template <typename IdxT>
__device__ __forceinline__ void sample_one_seed(const IdxT* __restrict__ indptr, const IdxT* __restrict__ indices, int64_t v,
                                                int64_t position, IdxT* __restrict__ out, int num_pick, uint64_t rng_seed,
                                                uint64_t rng_offset) {
  const int64_t begin = (int64_t)indptr[v];
  const int64_t d = (int64_t)indptr[v + 1] - begin;
  if (d <= num_pick) {
    for (int64_t t = 0; t < d; ++t) out[t] = indices[begin + t];
    return;
  }
  Philox ph(rng_seed, rng_offset);
  int64_t chosen[kMaxPick];
  uint4 r = make_uint4(0, 0, 0, 0);
  for (int s = 0; s < num_pick; ++s) {
    if ((s & 1) == 0) r = ph((uint64_t)position * (kMaxPick / 2) + (uint64_t)(s >> 1));
    const uint64_t bits = (s & 1) == 0 ? ((uint64_t)r.x << 32 | r.y) : ((uint64_t)r.z << 32 | r.w);
    const int64_t j = d - num_pick + s;
    // multiply-shift maps 64 random bits to [0, j]; the bias is below 2^-32 for any graph that fits in memory
    int64_t t = (int64_t)__umul64hi(bits, (uint64_t)(j + 1));
    bool taken = false;
    for (int q = 0; q < s; ++q) taken |= chosen[q] == t;
    chosen[s] = taken ? j : t;
  }
  for (int s = 0; s < num_pick; ++s) out[s] = indices[begin + chosen[s]];
}

// ---- open-addressing table: 64-bit keys, linear probing, capacity a power of two >= 2 n ----
constexpr unsigned long long kEmptyKey = ~0ull;

__device__ __forceinline__ uint64_t hash64(uint64_t x) {  // murmur3 finaliser
  x ^= x >> 33; x *= 0xff51afd7ed558ccdull; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ull; x ^= x >> 33;
  return x;
}

// slot of `key` in the table (inserting it when absent); -1 if no slot was found within `cap` probes (cannot
// happen with cap >= 2 n unless the table is corrupted; the caller flags it)
__device__ __forceinline__ int64_t find_or_insert(unsigned long long* tab_keys, int64_t cap_mask, unsigned long long key) {
  int64_t slot = (int64_t)(hash64(key) & (uint64_t)cap_mask);
  for (int64_t probe = 0; probe <= cap_mask; ++probe) {
    const unsigned long long prev = atomicCAS(tab_keys + slot, kEmptyKey, key);
    if (prev == kEmptyKey || prev == key) return slot;
    slot = (slot + 1) & cap_mask;
  }
  return -1;
}
__device__ __forceinline__ int64_t find(const unsigned long long* tab_keys, int64_t cap_mask, unsigned long long key) {
  int64_t slot = (int64_t)(hash64(key) & (uint64_t)cap_mask);
  for (int64_t probe = 0; probe <= cap_mask; ++probe) {
    const unsigned long long k = tab_keys[slot];
    if (k == key) return slot;
    if (k == kEmptyKey) return -1;
    slot = (slot + 1) & cap_mask;
  }
  return -1;
}

}  // namespace f2c
