// Streamed fused SQ decode + mean/sum aggregation over a CSC block
// (reference operator sq_decompress_spmm_csr, src/fusion_spmm.cu:143-272).
//
//   out[d, :] = (sum_{k in N(d), CSC order} decode(codes[indices[k], :])) / max(deg(d), 1)
//
// Same arithmetic, same CSC summation order and same table decode as the register-prefetch kernel of
// fused_sq_spmm.cu (bit-identical results); what differs is how the neighbour rows reach the adders.
// A CTA owns a contiguous slice of the destination rows.  Four producer warps copy the slice's neighbour ids and
// then the neighbours' compressed rows (16-byte cp.async pieces, several lanes per row) into a shared-memory ring
// addressed by edge number (its first positions mirrored behind its end, so that a group's rows never wrap), a few batches of ids and rows ahead of what they publish; the consumer
// warps take their rows out of the ring with one LDS per lane and edge.  The dependent global-load chain
// indptr -> ids -> rows is therefore paid once per CTA instead of once per destination row, the consumers hold no
// prefetch registers, and their inner loop is [LDS row bytes, PRMT + LDS + FADD2 per code byte].
//
// Shared memory (227 KB): the 64 KB decode table sits on a 64 KB boundary of the shared window, so that a lookup
// address is the byte permute's result itself; everything below the table is the ring (plus the indptr slice and
// the id batches), everything above it the zero slab, the build scratch, the output staging area and the watermarks.
//
// Destination rows whose lane group spans more than 32 edges per row on average are not taken from the ring (their
// edges are still streamed, which costs bandwidth but keeps the ring arithmetic trivial): their group reads ids and
// rows from global memory directly.  This bounds the ring capacity a waiting consumer can pin and makes the
// producer/consumer pair deadlock-free for any degree distribution.
#include "sq_fused.cuh"
#include "stream_pipe.cuh"

namespace f2c {
namespace sqs {

using namespace strm;

template <int BITS> struct Geo {
  static constexpr int VEC = BITS <= 2 ? 4 : 8;     // bytes of a neighbour row per lane
  static constexpr int EPL = VEC * 8 / BITS;        // output columns per lane: 32, 16, 16, 8
  static constexpr int kConsumers = BITS == 1 ? 8 : 16;
  static constexpr int kProducers = BITS == 1 ? 8 : 4;   // 16-byte rows are request-rate bound: more warps in flight
  static constexpr int kThreads = (kConsumers + kProducers) * 32;
};

struct Params {
  const uint8_t* codes;
  const float* codebooks;
  const void* indptr;
  const void* indices;
  float* out;
  int64_t n_dst;
  uint32_t row_bytes;
  int feat_dim, column_slice, n_cb, logG, code_kind, reduce;
  int log_pieces;          // log2 of the lanes that copy one row (power of two >= row_bytes / 16)
  int rows_per_chunk;
  int64_t n_chunks;
  uint32_t b_need;         // bytes the region above the table must hold
  uint32_t off_stage, off_sync;  // offsets inside that region
  uint32_t share;          // edges per producer warp and batch
  int* error;
  const uint8_t* shard[8];       // PEER: row r lives on shard r / rows_per_shard
  uint32_t rows_per_shard;
  unsigned long long shard_magic;
  DropoutArgs drop;
};

template <int BITS, typename IdxT, bool PEER>
__global__ void __launch_bounds__(Geo<BITS>::kThreads, 1) sq_stream_kernel(const Params p) {
  using L = Lut<BITS>;
  constexpr int VEC = Geo<BITS>::VEC, EPL = Geo<BITS>::EPL, C = Geo<BITS>::kConsumers, kProducers = Geo<BITS>::kProducers;
  constexpr bool PACKED = BITS <= 4;
  extern __shared__ __align__(128) unsigned char smem_dyn[];

  // ---- shared-memory map (uniform over the CTA; depends on where the window places the dynamic area)
  const uint32_t win0 = smem_u32(smem_dyn);
  const uint32_t table_w = (win0 + kSmemTotal - 65536u - p.b_need) & ~0xFFFFu;  // >= win0: the host sized b_need for it
  unsigned char* const table_g = smem_dyn + (table_w - win0);
  unsigned char* const above = table_g + L::TABLE_BYTES;
  float* const values = reinterpret_cast<float*>(above + 256);
  float4* const stage_all = reinterpret_cast<float4*>(above + p.off_stage);
  Sync* const sync = reinterpret_cast<Sync*>(above + p.off_sync);
  uint32_t* const ptr_s = reinterpret_cast<uint32_t*>(smem_dyn);
  const uint32_t a_bytes = table_w - win0;
  const uint32_t ptr_bytes = ((uint32_t)(p.rows_per_chunk + 1) * 4u + 15u) & ~15u;
  const uint32_t rb = p.row_bytes;
  constexpr uint32_t ib = sizeof(IdxT);
  const int R = 32 >> p.logG;                  // destination rows per consumer warp pass
  const uint32_t gmax = (uint32_t)R * 32u;     // a lane group spanning more edges reads global memory directly
  // the first gmax ring positions are mirrored behind the ring's end, so a lane group's rows are contiguous
  // `share` = edges of one producer warp per batch (from the host); a batch is kProducers * share consecutive edges
  const uint32_t share = p.share;
  const uint32_t batch = share * kProducers;
  const uint32_t ids_bytes = (kIdLead + 1) * batch * ib;
  const uint32_t ids_w = win0 + ptr_bytes;
  const uint32_t ring_w = ids_w + ids_bytes;
  const uint32_t cap = (a_bytes - ptr_bytes - ids_bytes) / rb - gmax;   // must be >= (kRowLag + 1) * batch + gmax
  if (ptr_bytes + ids_bytes + ((kRowLag + 1) * batch + 2u * gmax) * rb > a_bytes) {
    // the shared window starts somewhere the host did not expect: a ring too small could stall, so do nothing
    if (threadIdx.x == 0 && p.error != nullptr) atomicExch(p.error, 3);
    return;
  }

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool is_producer = warp >= C;
  const int G = 1 << p.logG;
  const int lane_g = lane & (G - 1);
  const int sub = lane >> p.logG;
  const uint32_t byte0 = (uint32_t)lane_g * VEC;
  const bool lane_active = byte0 < rb;

  const IdxT* __restrict__ indptr = reinterpret_cast<const IdxT*>(p.indptr);
  const IdxT* __restrict__ indices = reinterpret_cast<const IdxT*>(p.indices);
  auto row_ptr = [&](uint32_t id) -> const uint8_t* {
    if (!PEER) return p.codes + (uint64_t)id * rb;
    const uint32_t owner = (uint32_t)__umul64hi((unsigned long long)id, p.shard_magic);
    const uint32_t local = id - owner * p.rows_per_shard;
    return p.shard[owner] + (uint64_t)local * rb;
  };

  // lane constants of the consumers
  uint32_t lane_off = L::lane_offset(lane) | table_w;  // the table's base rides in the upper half (its low 16 bits are 0)
  const uint32_t lane_off_zero = lane_off + L::TABLE_BYTES;
  int cb_row = (lane_g * EPL) / p.column_slice;
  if (cb_row >= p.n_cb) cb_row = p.n_cb - 1;
  const float emin = __ldg(p.codebooks + cb_row * kCodebookDim + 2);
  const float emax = __ldg(p.codebooks + cb_row * kCodebookDim + 3);
  const float mean = __ldg(p.codebooks + cb_row * kCodebookDim + 4);
  // sums are 0 or between 2^(emin-24) and deg * 2^emax in magnitude: when that is well inside the normal range the
  // mean can skip the per-element range check of the exact division
  const bool div_safe = __all_sync(0xffffffffu, BITS == 1 ? (mean > 1e-20f && mean < 1e20f) : (emin > -80.0f && emax < 80.0f));
  float4* const stage = stage_all + warp * (32 * (EPL / 4));

  bool table_built = false;
  for (int64_t chunk = blockIdx.x; chunk < p.n_chunks; chunk += gridDim.x) {
    const int64_t row0 = chunk * p.rows_per_chunk;
    if (row0 >= p.n_dst) break;
    const int nrows = (int)min((int64_t)p.rows_per_chunk, p.n_dst - row0);
    // ---- the chunk's indptr slice as 32-bit edge offsets relative to its first edge
    const int64_t e0 = (int64_t)indptr[row0];
    for (int i = tid; i <= nrows; i += Geo<BITS>::kThreads) ptr_s[i] = (uint32_t)((int64_t)indptr[row0 + i] - e0);
    if (tid == 0) sync->staged = 0u;
    if (tid < C) sync->progress[tid] = 0u;   // "needs everything" until the consumer publishes its first row
    if (tid == 0 && chunk == (int64_t)blockIdx.x) sync->abort = 0u;
    __syncthreads();
    const uint32_t ne = ptr_s[nrows];
    const IdxT* __restrict__ gids = indices + e0;

    if (is_producer) {
      // =========================================================== producer warps
      const uint32_t pw = (uint32_t)(warp - C);                 // this warp copies edges [pw * share, (pw + 1) * share) of every batch
      const uint32_t my_ids_w = ids_w + pw * (kIdLead + 1) * share * ib;
      const uint32_t nb = (ne + batch - 1) / batch;
      const uint32_t pieces = rb >> 4;                          // 16-byte pieces per row
      const uint32_t piece = (uint32_t)lane & ((1u << p.log_pieces) - 1u);
      const uint32_t e_lane = (uint32_t)lane >> p.log_pieces, e_step = 32u >> p.log_pieces;
      bool ok = true;
      for (uint32_t it = 0; it < nb + kIdLead + kRowLag; ++it) {
        // (a) neighbour ids of batch `it`
        if (it < nb) {
          const uint32_t b0 = it * batch + pw * share;
          const uint32_t n = b0 < ne ? min(share, ne - b0) : 0u;
          const uint32_t dst = my_ids_w + (it % (kIdLead + 1)) * share * ib;
          for (uint32_t j = lane; j < n; j += 32) cp_async<ib>(dst + j * ib, gids + b0 + j);
        }
        cp_async_commit();
        // (b) rows of batch it - kIdLead, whose ids have landed
        cp_async_wait<2 * kIdLead>();
        __syncwarp();
        if (ok && it >= (uint32_t)kIdLead && it - kIdLead < nb) {
          const uint32_t jb = it - kIdLead;
          const uint32_t b0 = jb * batch + pw * share;
          const uint32_t n = b0 < ne ? min(share, ne - b0) : 0u;
          ok = wait_space(sync, C, b0 + n, cap, lane, p.error);
          if (ok && piece < pieces) {
            const uint32_t src_ids = my_ids_w + (jb % (kIdLead + 1)) * share * ib;
            const uint32_t pos0 = b0 % cap;
#pragma unroll 4
            for (uint32_t e = e_lane; e < n; e += e_step) {
              const uint32_t id = lds_u32(src_ids + e * ib);
              uint32_t pos = pos0 + e;
              if (pos >= cap) pos -= cap;
              const uint8_t* src = row_ptr(id) + piece * 16u;
              cp_async<16>(ring_w + pos * rb + piece * 16u, src);
              if (pos < gmax) cp_async<16>(ring_w + (pos + cap) * rb + piece * 16u, src);
            }
          }
        }
        cp_async_commit();
        // (c) publish batch it - kIdLead - kRowLag, whose rows have landed
        cp_async_wait<2 * kRowLag>();
        producer_barrier<kProducers>();  // every producer warp's share of that batch has landed
        if (it >= (uint32_t)(kIdLead + kRowLag)) {
          const uint32_t jc = it - kIdLead - kRowLag;
          if (pw == 0 && lane == 0 && ld_acquire(&sync->abort) == 0u) st_release(&sync->staged, min((jc + 1) * batch, ne));
        }
      }
      cp_async_wait<0>();
    } else {
      // =========================================================== consumer warps
      if (!table_built) {
        build_sq_table<BITS, EPL>(table_g, values, p.codebooks, p.n_cb, p.column_slice, G, p.code_kind, tid, C * 32,
                                  [] { asm volatile("bar.sync 1, %0;" ::"n"(C * 32) : "memory"); });
        table_built = true;
      }
      const int n_groups = (nrows + R - 1) / R;
      if (lane == 0) st_release(&sync->progress[warp], warp < n_groups ? ptr_s[warp * R] : kDone);
      uint32_t seen = 0u;
      for (int g = warp; g < n_groups; g += C) {
        const int r_first = g * R;
        const int r_last = min(r_first + R, nrows);
        const uint32_t gbeg = ptr_s[r_first], gend = ptr_s[r_last];
        const int row = r_first + sub;
        uint32_t beg = 0u;
        int deg = 0;
        if (row < nrows) { beg = ptr_s[row]; deg = (int)(ptr_s[row + 1] - beg); }
        Acc<EPL, PACKED> acc;
        acc.clear();
        if (gend - gbeg > gmax) {
          // long rows: ids and rows straight from global memory (no wait on the producer)
          const int dmax = __reduce_max_sync(0xffffffffu, deg);
          for (int k = 0; k < dmax; ++k) {
            if (k < deg && lane_active) {
              VecLoad<VEC> d;
              d.load(row_ptr((uint32_t)gids[beg + k]) + byte0);
              sq_accumulate<BITS, VEC, DEC_LUT, true>(acc, d, 0u, lane_off, p.code_kind, 0.f, 0.f, 0.f);
            }
          }
        } else {
          if (!wait_staged(sync, gend, seen, p.error)) break;
          const int umax = __reduce_max_sync(0xffffffffu, deg);
          uint32_t addr = ring_w + (beg % cap) * rb + byte0;
#pragma unroll 2
          for (int u = 0; u < umax; ++u) {
            VecLoad<VEC> d;
            d.zero();
            const bool have = u < deg && lane_active;
            if (have) d.load_shared(addr);
            // slots beyond a row's degree look up slab 0 of the zero-filled copy: adding +0 changes nothing
            sq_accumulate<BITS, VEC, DEC_LUT, true>(acc, d, 0u, have ? lane_off : lane_off_zero, p.code_kind, 0.f, 0.f, 0.f);
            addr += rb;
          }
        }
        // the ring positions of this group are free again
        __syncwarp();
        if (lane == 0) st_release(&sync->progress[warp], g + C < n_groups ? ptr_s[(g + C) * R] : kDone);
        sq_store_rows<EPL>(acc, stage, lane, p.logG, deg, row < nrows && lane_active, row0 + r_first, (int64_t)(nrows - r_first),
                           p.feat_dim, p.reduce, div_safe, p.drop, p.out);
      }
      if (lane == 0) st_release(&sync->progress[warp], kDone);
    }
    __syncthreads();
  }
}

static int ilog2_ceil(int v) { int l = 0; while ((1 << l) < v) ++l; return l; }

}  // namespace sqs

// Launch the streamed kernel if it serves this shape: *served = false (nothing launched) otherwise.
// shards = nullptr for a whole table at `codes`; else `world` shard pointers of rows_per_shard rows each.
template <int BITS, typename IdxT>
static int launch_stream(const void* codes, int code_dtype, const float* codebooks, int64_t n_cb, const void* indptr, const void* indices,
                         float* out, int64_t n_dst, int64_t n_src, int64_t src_dim, int64_t D, int64_t cs, int reduce,
                         const DropoutArgs& drop, cudaStream_t st, const void* const* shards, int world, int64_t rows_per_shard,
                         bool* served) {
  using namespace sqs;
  using namespace strm;
  *served = false;
  if constexpr (BITS > 8) {
    return F2C_OK;
  } else {
    using G_ = Geo<BITS>;
    using L = Lut<BITS>;
    const int code_bytes = dtype_size(code_dtype);
    const int64_t row_bytes = src_dim * code_bytes;
    if (code_bytes != 1 || row_bytes % 16 != 0 || row_bytes > 32 * G_::VEC || D % 4 != 0 || !aligned(out, 16)) return F2C_OK;
    if (n_src >= (1ll << 32) || n_dst >= (1ll << 30)) return F2C_OK;
    if (shards == nullptr && !aligned(codes, 16)) return F2C_OK;
    for (int r = 0; shards != nullptr && r < world; ++r)
      if (!aligned(shards[r], 16)) return F2C_OK;
    const int G = 1 << ilog2_ceil((int)ceil_div(row_bytes, G_::VEC));
    if (!(n_cb == 1 || cs % G_::EPL == 0)) return F2C_OK;          // a lane's columns share one codebook row
    if (!(n_cb == 1 || L::COPIES % G == 0)) return F2C_OK;         // lanes sharing a table copy own the same columns
    Params p{};
    p.codes = (const uint8_t*)codes; p.codebooks = codebooks; p.indptr = indptr; p.indices = indices; p.out = out;
    p.n_dst = n_dst; p.row_bytes = (uint32_t)row_bytes; p.feat_dim = (int)D; p.column_slice = (int)cs; p.n_cb = (int)n_cb;
    p.logG = ilog2_ceil(G); p.code_kind = code_dtype == F2C_I8 ? CODE_I8 : CODE_U8; p.reduce = reduce; p.drop = drop;
    p.log_pieces = ilog2_ceil((int)(row_bytes / 16));
    const int R = 32 / G;
    int64_t grid = ceil_div(n_dst, (int64_t)G_::kConsumers * R);
    const int64_t sms = current_sm_count();
    if (grid > sms) grid = sms;
    plan_chunks(n_dst, grid, &p.rows_per_chunk, &p.n_chunks);
    const int n_rows = G < L::COPIES ? G : L::COPIES;
    const uint32_t values_bytes = ((uint32_t)n_rows * L::NCODE * 4u + 15u) & ~15u;
    p.off_stage = 256u + values_bytes;
    p.off_sync = p.off_stage + (uint32_t)G_::kConsumers * 32u * G_::EPL * 4u;
    p.b_need = p.off_sync + 256u;
    // edges per producer warp and batch: about 2 KB of rows, bounded by what the ring below the table holds (the table
    // sits on the highest 64 KB boundary that leaves b_need bytes above it; the window starts 1 KB into the SM's memory)
    {
      const uint32_t a_bytes = ((1024u + kSmemTotal - 65536u - p.b_need) & ~0xFFFFu) - 1024u;
      const uint32_t ptr_bytes = ((uint32_t)(p.rows_per_chunk + 1) * 4u + 15u) & ~15u;
      const uint32_t rb = (uint32_t)row_bytes, ib = (uint32_t)sizeof(IdxT), gmax = (uint32_t)R * 32u;
      uint32_t share = (a_bytes - ptr_bytes - 2u * gmax * rb) / (G_::kProducers * ((kIdLead + 1) * ib + (kRowLag + 1) * rb));
      uint32_t want = (uint32_t)(2048 / row_bytes);
      if (want < 32u) want = 32u;
      if (share > want) share = want;
      share &= ~7u;
      if (share < 8u) return F2C_OK;
      p.share = share;
    }
    p.error = stream_error_word();
    if (shards != nullptr) {
      for (int r = 0; r < 8; ++r) p.shard[r] = (const uint8_t*)shards[r < world ? r : 0];
      p.rows_per_shard = (uint32_t)rows_per_shard;
      p.shard_magic = ~0ull / (unsigned long long)rows_per_shard + 1ull;
    }
    auto launch = [&](auto kern) -> int {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTotal);
      if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "sq_decompress_spmm_csr: %s", cudaGetErrorString(e));
      kern<<<(unsigned)grid, G_::kThreads, kSmemTotal, st>>>(p);
      return check_launch("sq_decompress_spmm_csr");
    };
    *served = true;
    if (shards != nullptr) return launch(sq_stream_kernel<BITS, IdxT, true>);
    return launch(sq_stream_kernel<BITS, IdxT, false>);
  }
}

int launch_sq_stream(int bits, int index_dtype, const void* codes, int code_dtype, const float* codebooks, int64_t n_cb,
                     const void* indptr, const void* indices, float* out, int64_t n_dst, int64_t n_src, int64_t src_dim, int64_t D,
                     int64_t cs, int reduce, const DropoutArgs& drop, cudaStream_t st, const void* const* shards, int world,
                     int64_t rows_per_shard, bool* served) {
#define F2C_SQS(B)                                                                                                              \
  return index_dtype == F2C_I32                                                                                                  \
             ? launch_stream<B, int32_t>(codes, code_dtype, codebooks, n_cb, indptr, indices, out, n_dst, n_src, src_dim, D, cs, \
                                         reduce, drop, st, shards, world, rows_per_shard, served)                                \
             : launch_stream<B, int64_t>(codes, code_dtype, codebooks, n_cb, indptr, indices, out, n_dst, n_src, src_dim, D, cs, \
                                         reduce, drop, st, shards, world, rows_per_shard, served)
  switch (bits) {
    case 1: F2C_SQS(1);
    case 2: F2C_SQS(2);
    case 4: F2C_SQS(4);
    case 8: F2C_SQS(8);
    default: *served = false; return F2C_OK;
  }
#undef F2C_SQS
}

}  // namespace f2c
