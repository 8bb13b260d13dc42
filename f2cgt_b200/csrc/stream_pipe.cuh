// Building blocks of the streamed fused kernels (fused_sq_stream.cu, fused_vq_stream.cu).
//
// A CTA owns a contiguous range of destination rows ("chunk"), hence a contiguous range of the block's edges.
// A few PRODUCER warps walk that edge range in batches (each warp a contiguous share of every batch) and copy, with
// cp.async, first the neighbour ids and then what each edge needs (its compressed row, or its code row and hot-row
// slot) into shared-memory rings indexed by edge number.  CONSUMER warps aggregate destination rows out of the rings.
// Several producer warps are needed because one warp keeps only ~100 cache lines of cp.async requests in flight
// (measured on B200: one warp gathers ~90 random 64-byte rows per microsecond, four warps ~270, which is what the SM
// sustains).  The two sides only share two watermarks in shared memory:
//   staged       edges [0, staged) of the chunk are complete in the rings           (producer -> consumers)
//   progress[w]  first edge consumer warp w still needs; kDone when it has finished   (consumers -> producer)
// The producer may overwrite ring position e % cap only when e - min(progress) <= cap.  Nothing else synchronises
// the warps inside a chunk, so the dependent chain indptr -> ids -> rows is paid once per CTA, not once per row.
//
// Every wait is a bounded poll: when the limit runs out the warp raises the CTA's abort flag and the kernel's
// global error word, all warps leave their loops, and the kernel returns (no trap, no endless spin).
#pragma once
#include "common.cuh"

namespace f2c {
namespace strm {

// Batches are small (a producer warp's share is 32..128 edges) and several are in flight, so that the ring holds,
// besides what is in flight, a full round of consumer work that is already published: with a ring barely larger than
// the in-flight window the two sides would alternate instead of overlapping.
constexpr int kIdLead = 6;   // the ids of batch i + kIdLead are requested while the rows of batch i are requested
constexpr int kRowLag = 4;   // batch i is published once the rows of batch i + kRowLag have been requested
constexpr uint32_t kDone = 0xFFFFFFFFu;
constexpr int kSpinLimit = 1 << 20;   // polls (each followed by a sleep of kPollSleepNs) before a wait gives up (~0.2 s)
constexpr unsigned kPollSleepNs = 200;
constexpr int kMaxChunkRows = 1024;   // destination rows whose indptr slice is staged at once
constexpr uint32_t kSmemTotal = 227u * 1024u;

struct Sync {
  uint32_t staged;
  uint32_t abort;
  uint32_t pad[2];
  uint32_t progress[28];
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

template <int BYTES> __device__ __forceinline__ void cp_async(uint32_t dst, const void* src);
template <> __device__ __forceinline__ void cp_async<4>(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
template <> __device__ __forceinline__ void cp_async<8>(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
template <> __device__ __forceinline__ void cp_async<16>(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}

// barrier over the P producer warps only
template <int P> __device__ __forceinline__ void producer_barrier() { asm volatile("bar.sync 2, %0;" ::"n"(P * 32) : "memory"); }

__device__ __forceinline__ void raise_abort(Sync* sync, int* error, int code) {
  st_release(&sync->abort, 1u);
  if (error != nullptr) atomicExch(error, code);
}

// Consumer side (all 32 lanes call it): wait until edges [0, need) are staged.  `seen` caches the lowest value any lane
// has read (warp-uniform, monotone inside a chunk).  Every lane performs its own acquire load, so each lane may read the
// ring once the warp-wide minimum covers `need`.  Returns false (uniformly) when the CTA is aborting.
__device__ __forceinline__ bool wait_staged(Sync* sync, uint32_t need, uint32_t& seen, int* error) {
  if (seen >= need) return true;
  int spins = 0;
  for (;;) {
    seen = __reduce_min_sync(0xffffffffu, ld_acquire(&sync->staged));
    if (seen >= need) return true;
    // a waiting warp must leave the issue slots to the producer warps: sleep long between polls
    __nanosleep(kPollSleepNs);
    if ((++spins & 15) == 0) {
      if (__any_sync(0xffffffffu, ld_acquire(&sync->abort) != 0u)) return false;
      if (spins > kSpinLimit) {
        raise_abort(sync, error, 1);
        return false;
      }
    }
  }
}

// Producer side (all 32 lanes call it): wait until ring positions up to edge `end_edge` may be written.
__device__ __forceinline__ bool wait_space(Sync* sync, int n_consumers, uint32_t end_edge, uint32_t cap, int lane, int* error) {
  int spins = 0;
  for (;;) {
    const uint32_t mine = lane < n_consumers ? ld_acquire(&sync->progress[lane]) : kDone;
    const uint32_t lowest = __reduce_min_sync(0xffffffffu, mine);
    if (lowest >= end_edge || end_edge - lowest <= cap) return true;
    __nanosleep(kPollSleepNs);
    if ((++spins & 15) == 0) {
      if (__any_sync(0xffffffffu, ld_acquire(&sync->abort) != 0u)) return false;
      if (spins > kSpinLimit) {
        raise_abort(sync, error, 2);
        return false;
      }
    }
  }
}

// Rows per chunk and number of chunks for a block of n_dst rows on `grid` CTAs: every CTA gets the same number of
// chunks (the last ones may be short or empty) and no chunk exceeds kMaxChunkRows.
static inline void plan_chunks(int64_t n_dst, int64_t grid, int* rows_per_chunk, int64_t* n_chunks) {
  const int64_t per_cta = ceil_div(n_dst, grid * kMaxChunkRows);
  *n_chunks = grid * per_cta;
  *rows_per_chunk = (int)ceil_div(n_dst, *n_chunks);
}

}  // namespace strm

// Non-zero when a streamed kernel gave up on a wait since the last query (see f2c_device_status).
int* stream_error_word();

}  // namespace f2c
