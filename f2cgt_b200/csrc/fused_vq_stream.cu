// Streamed fused VQ decode + aggregation and the single-launch two-level (hot rows SQ, all other rows VQ)
// aggregation for the common shapes: uint8 codes, 256 centroids, 4/8/16 code bytes per row, column_slice in
// {4,...,128} dividing 128, hot rows 8- or 4-bit SQ.  Same arithmetic and CSC summation order as the other kernel
// families (reference: src/fusion_spmm.cu:72-141 for VQ, src/sq_quantization.cu:123-153 for the hot rows).
//
// A CTA owns a contiguous slice of the destination rows.  Its producer warps stage, per edge and in CSC order, the
// neighbour id (cp.async), then the neighbour's VQ code row (4..16 bytes) and - for the two-level op - its hot-row slot
// (plain loads, stored into shared-memory rings; stream_pipe.cuh has the watermarks).  Consumer warps own one destination row at a time; a lane owns
// four consecutive columns (one LDS.128 from the centroid its code selects, a coalesced 512-byte row store).  What is
// left of the dependent chain indptr -> ids -> (slot, codes) -> hot row for a consumer is its last link: the hot rows
// of a warp's NEXT destination row are requested (one coalesced 4-byte load per lane and hot edge, up to U per row)
// while the current row is aggregated, when the producer has already staged that row's slots.
//
//  * Codebooks are staged once per CTA; for column_slice < 32 the subspaces that one quarter-warp reads are
//    interleaved inside 128-byte lines, so that the eight lanes of a quarter-warp always hit eight different 16-byte
//    bank groups whatever the codes are.
//  * Hot rows are decoded through a byte-indexed table built with the same expression as the element-wise decode
//    (same bits), one private copy per lane and bank: a lookup never conflicts.
//  * The first kLongRow positions of the rings are mirrored behind their end, so a row's entries are contiguous and
//    the inner loop has no wrap test.  Rows with more than kLongRow neighbours bypass the rings (ids, slots and codes
//    from global memory, 32 edges at a time).
#include "stream_pipe.cuh"
#include "vq_params.cuh"

namespace f2c {
namespace vqs {

using namespace strm;

constexpr int kConsumers = 16;
constexpr int kProducers = 8;   // 4-byte requests (code row, slot) are request-rate bound: many warps in flight
constexpr int kThreads = (kConsumers + kProducers) * 32;
constexpr int U = 16;             // hot rows requested ahead per destination row
constexpr int kLongRow = 32;      // rows with more neighbours bypass the rings
constexpr int kLutBytes = 256 * 256;
constexpr int kPerLane = 2;       // edges per producer lane and batch (a warp's share of a batch is at most 64 edges)

struct Layout {  // byte offsets in dynamic shared memory, from the host
  uint32_t lut, ptr, ids, codes, slots, sync;
  uint32_t sub, cap;  // edges per producer warp and batch; ring capacity in edges
};

__device__ __forceinline__ uint32_t lds_u8(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ int lds_s32(uint32_t a) {
  int v;
  asm volatile("ld.shared.s32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ float4 lds_f4(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ float2 lds_f2(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ float lds_f1(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t ldg_nc_u16(const void* p) {
  uint16_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}

template <int ROWW> struct CodeRow { uint32_t w[ROWW]; };
template <int ROWW> __device__ __forceinline__ void load_code_row(CodeRow<ROWW>& c, const void* p) {
  if (ROWW == 1) c.w[0] = ldg_nc_u32(p);
  else if (ROWW == 2) { uint2 v = ldg_nc_u64(p); c.w[0] = v.x; c.w[1] = v.y; }
  else { uint4 v = ldg_nc_u128(p); c.w[0] = v.x; c.w[1] = v.y; c.w[ROWW > 2 ? 2 : 0] = v.z; c.w[ROWW > 3 ? 3 : 0] = v.w; }
}
template <int ROWW> __device__ __forceinline__ void store_code_row(uint32_t a, const CodeRow<ROWW>& c) {
  if (ROWW == 1) asm volatile("st.shared.b32 [%0], %1;" ::"r"(a), "r"(c.w[0]) : "memory");
  else if (ROWW == 2) asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(a), "r"(c.w[0]), "r"(c.w[ROWW > 1 ? 1 : 0]) : "memory");
  else asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(c.w[0]), "r"(c.w[ROWW > 1 ? 1 : 0]), "r"(c.w[ROWW > 2 ? 2 : 0]), "r"(c.w[ROWW > 3 ? 3 : 0]) : "memory");
}

// HB = 0: VQ only.  HB = 8 / 4: two-level with 8- / 4-bit hot rows.  ROWW = 32-bit words of one VQ code row.
template <int HB, typename IdxT, int ROWW>
__global__ void __launch_bounds__(kThreads, 1) vq_stream_kernel(const VqParams p, const Layout lay, const int rows_per_chunk,
                                                                const int64_t n_chunks, int* const error) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int C = kConsumers;
  constexpr uint32_t ROWB = ROWW * 4;
  constexpr uint32_t ib = sizeof(IdxT);
  unsigned char* const cb_s = smem;
  unsigned char* const lut_s = smem + lay.lut;
  uint32_t* const ptr_s = reinterpret_cast<uint32_t*>(smem + lay.ptr);
  Sync* const sync = reinterpret_cast<Sync*>(smem + lay.sync);
  const uint32_t ids_w = smem_u32(smem + lay.ids);
  const uint32_t codes_w = smem_u32(smem + lay.codes);
  const uint32_t slots_w = smem_u32(smem + lay.slots);
  const uint32_t sub = lay.sub, batch = lay.sub * kProducers, cap = lay.cap;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool is_producer = warp >= C;

  const int part = blockIdx.y;
  const int s_begin = part * p.cb_per_part;
  const int s_end = min(s_begin + p.cb_per_part, p.n_cb);
  const int col_begin = s_begin * p.cs;
  const int col_end = min(s_end * p.cs, p.feat_dim);
  const int cs = p.cs, spq = p.fast_spq;
  const uint32_t stride = (uint32_t)p.fast_stride;
  constexpr int K = 256;

  // ---- lane constants
  const int col = col_begin + 4 * lane;
  const bool active = col < col_end;
  const int colc = active ? col : col_begin;
  const int s = colc / cs, sl = s - s_begin, off = colc - s * cs;
  const uint32_t lane_base = spq > 1 ? (uint32_t)((sl / spq) * K * 128 + (sl % spq) * cs * 4 + off * 4)
                                     : (uint32_t)(sl * K) * stride + (uint32_t)off * 4u;
  const uint32_t cb_addr = smem_u32(cb_s) + lane_base;
  const uint32_t code_lane_w = codes_w + (uint32_t)s;  // byte s of every staged code row
  const uint8_t* const hot_base = HB != 0 ? p.sq_codes + (colc * (HB == 0 ? 8 : HB)) / 8 : nullptr;
  const uint32_t hot_row_bytes = (uint32_t)p.sq_row_bytes;
  const uint32_t lane_off = (uint32_t)lane * (HB == 4 ? 8u : 4u);  // < 256: fits the low byte of the permute result
  const uint32_t lut_base = smem_u32(lut_s);

  const IdxT* __restrict__ indptr = reinterpret_cast<const IdxT*>(p.indptr);
  const IdxT* __restrict__ indices = reinterpret_cast<const IdxT*>(p.indices);
  const uint8_t* __restrict__ codes = reinterpret_cast<const uint8_t*>(p.codes);

  float4 acc;
  auto add_vq = [&](uint32_t code) {
    const float4 v = lds_f4(cb_addr + code * stride);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  };
  auto add_hot = [&](uint32_t w) {
    if (HB == 8) {
      const float v0 = lds_f1(lut_base + __byte_perm(w, lane_off, 0x7704)), v1 = lds_f1(lut_base + __byte_perm(w, lane_off, 0x7714));
      const float v2 = lds_f1(lut_base + __byte_perm(w, lane_off, 0x7724)), v3 = lds_f1(lut_base + __byte_perm(w, lane_off, 0x7734));
      acc.x += v0; acc.y += v1; acc.z += v2; acc.w += v3;
    } else {
      const float2 a = lds_f2(lut_base + __byte_perm(w, lane_off, 0x7704)), b = lds_f2(lut_base + __byte_perm(w, lane_off, 0x7714));
      acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
    }
  };
  auto load_hot = [&](int sl_) -> uint32_t {
    const uint8_t* q = hot_base + (uint64_t)(uint32_t)sl_ * hot_row_bytes;
    return HB == 8 ? ldg_nc_u32(q) : ldg_nc_u16(q);
  };

  bool staged_tables = false;
  for (int64_t chunk = blockIdx.x; chunk < n_chunks; chunk += gridDim.x) {
    const int64_t row0 = chunk * rows_per_chunk;
    if (row0 >= p.n_dst) break;
    const int nrows = (int)min((int64_t)rows_per_chunk, p.n_dst - row0);
    const int64_t e0 = (int64_t)indptr[row0];
    for (int i = tid; i <= nrows; i += kThreads) ptr_s[i] = (uint32_t)((int64_t)indptr[row0 + i] - e0);
    if (tid == 0) sync->staged = 0u;
    if (tid < C) sync->progress[tid] = 0u;
    if (tid == 0 && chunk == (int64_t)blockIdx.x) sync->abort = 0u;
    __syncthreads();
    const uint32_t ne = ptr_s[nrows];
    const IdxT* __restrict__ gids = indices + e0;

    if (is_producer) {
      // =========================================================== producer warps
      // Warp pw stages edges [pw * sub, (pw + 1) * sub) of every batch: at most kPerLane edges per lane.  The neighbour ids
      // stream in with cp.async (coalesced, kIdLead batches ahead); code rows and slots are random 4..16-byte reads, which
      // cp.async handles badly (one L1 line per request, ~100 requests in flight per warp), so they are plain loads into
      // registers, one batch in flight while the previous one is stored into the rings and published.
      const uint32_t pw = (uint32_t)(warp - C);
      const uint32_t my_ids_w = ids_w + pw * (kIdLead + 1) * sub * ib;
      const uint32_t nb = (ne + batch - 1) / batch;
      bool ok = true;
      CodeRow<ROWW> code_r[2][kPerLane];
      int slot_r[2][kPerLane];
#pragma unroll
      for (int k = 0; k < kPerLane; ++k) { slot_r[0][k] = -1; slot_r[1][k] = -1; }
      auto share_of = [&](uint32_t j, uint32_t& b0, uint32_t& n) {
        b0 = j * batch + pw * sub;
        n = (j < nb && b0 < ne) ? min(sub, ne - b0) : 0u;
      };
      for (uint32_t it0 = 0; it0 < nb + kIdLead + 1; it0 += 2) {
#pragma unroll
        for (int P = 0; P < 2; ++P) {
          const uint32_t it = it0 + P;
          uint32_t b0, n;
          // (a) neighbour ids of batch `it`
          share_of(it, b0, n);
          {
            const uint32_t dst = my_ids_w + (it % (kIdLead + 1)) * sub * ib;
            for (uint32_t j = lane; j < n; j += 32) cp_async<ib>(dst + j * ib, gids + b0 + j);
          }
          cp_async_commit();
          cp_async_wait<kIdLead>();
          __syncwarp();
          // (b) request code rows and slots of batch it - kIdLead (its ids have landed) into register set P
          if (it >= (uint32_t)kIdLead) {
            const uint32_t jl = it - kIdLead;
            share_of(jl, b0, n);
            const uint32_t src_ids = my_ids_w + (jl % (kIdLead + 1)) * sub * ib;
#pragma unroll
            for (int k = 0; k < kPerLane; ++k) {
              const uint32_t e = lane + 32u * k;
              if (e < n) {
                const uint32_t id = lds_u32(src_ids + e * ib);
                load_code_row<ROWW>(code_r[P][k], codes + (uint64_t)id * ROWB);
                if (HB != 0) slot_r[P][k] = hot_slot_of(p, (int64_t)id);
              }
            }
          }
          // (c) store batch it - kIdLead - 1 (register set P ^ 1, requested one iteration ago) and publish it
          if (it >= (uint32_t)kIdLead + 1u) {
            const uint32_t js = it - kIdLead - 1;
            share_of(js, b0, n);
            if (ok && n > 0) ok = wait_space(sync, C, b0 + n, cap, lane, error);
            if (ok) {
              const uint32_t pos0 = b0 % cap;
#pragma unroll
              for (int k = 0; k < kPerLane; ++k) {
                const uint32_t e = lane + 32u * k;
                if (e < n) {
                  uint32_t pos = pos0 + e;
                  if (pos >= cap) pos -= cap;
                  store_code_row<ROWW>(codes_w + pos * ROWB, code_r[P ^ 1][k]);
                  if (HB != 0) asm volatile("st.shared.s32 [%0], %1;" ::"r"(slots_w + pos * 4u), "r"(slot_r[P ^ 1][k]) : "memory");
                  if (pos < (uint32_t)kLongRow) {  // mirror behind the ring's end: rows never wrap
                    store_code_row<ROWW>(codes_w + (pos + cap) * ROWB, code_r[P ^ 1][k]);
                    if (HB != 0) asm volatile("st.shared.s32 [%0], %1;" ::"r"(slots_w + (pos + cap) * 4u), "r"(slot_r[P ^ 1][k]) : "memory");
                  }
                }
              }
            }
            producer_barrier<kProducers>();  // every producer warp's share of that batch is in the rings
            if (js < nb && pw == 0 && lane == 0 && ld_acquire(&sync->abort) == 0u) st_release(&sync->staged, min((js + 1) * batch, ne));
          } else {
            producer_barrier<kProducers>();
          }
        }
      }
      cp_async_wait<0>();
    } else {
      // =========================================================== consumer warps
      if (!staged_tables) {
        constexpr int nthr = C * 32;
        // ---- this part's codebooks; column_slice is a power of two here.  Consecutive threads write consecutive
        //      16-byte pieces of shared memory (no bank conflicts while staging).
        {
          const int lg4 = 31 - __clz(cs >> 2);  // log2(float4 pieces per centroid)
          const int n_sub = s_end - s_begin;
          const float4* src = reinterpret_cast<const float4*>(p.codebooks + (int64_t)s_begin * K * cs);
          float4* dst = reinterpret_cast<float4*>(cb_s);
          if (spq > 1) {  // 128-byte line = the centroids `code` of spq consecutive subspaces
            const int n16 = ((n_sub + spq - 1) / spq) * K * 8;
            for (int i = tid; i < n16; i += nthr) {
              const int piece = i & 7, line = i >> 3;
              const int code = line % K, grp = line / K;
              const int ssub = grp * spq + (piece >> lg4), q = piece & ((1 << lg4) - 1);
              dst[i] = ssub < n_sub ? __ldg(src + ((ssub * K + code) << lg4) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
          } else {        // natural layout: the staged image equals the global one
            const int n16 = (n_sub * K) << lg4;
            for (int i = tid; i < n16; i += nthr) dst[i] = __ldg(src + i);
          }
        }
        // ---- hot-row decode table: entry (byte, lane) = the floats that `byte` decodes to with the codebook row of
        //      that lane's columns; slab `byte` starts at byte * 256, a lane's entry is 4 (8-bit) or 8 (4-bit) bytes
        if (HB != 0) {
          int lcol = col_begin + 4 * lane;
          if (lcol >= col_end) lcol = col_begin;
          int row = lcol / p.sq_cs;
          if (row >= p.sq_n_cb) row = p.sq_n_cb - 1;
          const float emin = __ldg(p.sq_codebooks + row * kCodebookDim + 2), emax = __ldg(p.sq_codebooks + row * kCodebookDim + 3);
          const float mean = __ldg(p.sq_codebooks + row * kCodebookDim + 4);
          for (int byte = warp; byte < 256; byte += C) {
            if (HB == 8) {
              const float c = p.sq_signed ? (float)(int8_t)byte : (float)byte;
              reinterpret_cast<float*>(lut_s + byte * 256)[lane] = sq_decode<8>(c, sq_scale<8>(emin, emax), emin, mean);
            } else {
              const float sc = sq_scale<4>(emin, emax);
              reinterpret_cast<float2*>(lut_s + byte * 256)[lane] =
                  make_float2(sq_decode<4>((float)(byte & 15), sc, emin, mean), sq_decode<4>((float)(byte >> 4), sc, emin, mean));
            }
          }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(C * 32) : "memory");
        staged_tables = true;
      }

      // ---- per-row state, two sets: set P is the row being aggregated, set P^1 the warp's next row
      uint32_t beg[2] = {0u, 0u};
      int deg[2] = {0, 0};
      uint32_t mask[2] = {0u, 0u};
      int slot_mine[2] = {-1, -1};
      bool ready[2] = {false, false};  // slots read and hot rows requested
      uint32_t hot[2][HB != 0 ? U : 1];
#pragma unroll
      for (int u = 0; u < (HB != 0 ? U : 1); ++u) { hot[0][u] = 0u; hot[1][u] = 0u; }
      uint32_t seen = 0u;
      bool alive = true;

      // read the row's extent; if it is a ring row whose entries are staged (or `block` is set: wait for them), read
      // its slots and request its hot rows
      auto prepare = [&](int P, int row, bool block) {
        beg[P] = ptr_s[row];
        deg[P] = (int)(ptr_s[row + 1] - beg[P]);
        mask[P] = 0u;
        slot_mine[P] = -1;
        ready[P] = true;
        if (deg[P] > kLongRow || deg[P] == 0) return;
        const uint32_t need = beg[P] + (uint32_t)deg[P];
        if (seen < need) {
          if (block) {
            if (!wait_staged(sync, need, seen, error)) { alive = false; return; }
          } else {
            seen = __reduce_min_sync(0xffffffffu, ld_acquire(&sync->staged));
            if (seen < need) { ready[P] = false; return; }
          }
        }
        if (HB != 0) {
          const uint32_t pos0 = beg[P] % cap;
          if (lane < deg[P]) slot_mine[P] = lds_s32(slots_w + (pos0 + (uint32_t)lane) * 4u);
          mask[P] = __ballot_sync(0xffffffffu, slot_mine[P] >= 0);
          if (mask[P] != 0u) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
              if ((mask[P] >> u) == 0u) break;
              if ((mask[P] >> u) & 1u) hot[P][u] = load_hot(__shfl_sync(0xffffffffu, slot_mine[P], u));
            }
          }
        }
      };

      int row = warp;
      if (lane == 0) st_release(&sync->progress[warp], row < nrows ? ptr_s[row] : kDone);
      if (row < nrows) prepare(0, row, true);
      while (row < nrows && alive) {
#pragma unroll
        for (int P = 0; P < 2; ++P) {
          if (row < nrows && alive) {  // warp uniform
            const int nxt = row + C;
            if (nxt < nrows) prepare(P ^ 1, nxt, false);
            // ---------------- aggregate row `row` (set P)
            acc = make_float4(0.f, 0.f, 0.f, 0.f);
            const int cnt = deg[P];
            if (cnt <= kLongRow) {
              const uint32_t pos0 = beg[P] % cap;
              const uint32_t cw = code_lane_w + pos0 * ROWB;
              if (HB != 0) {
                const uint32_t m = mask[P];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                  if (u >= cnt) break;
                  if ((m >> u) & 1u) add_hot(hot[P][u]);
                  else add_vq(lds_u8(cw + u * ROWB));
                }
                for (int u = U; u < cnt; ++u) {
                  const int sl_ = __shfl_sync(0xffffffffu, slot_mine[P], u);
                  if (sl_ >= 0) add_hot(load_hot(sl_));
                  else add_vq(lds_u8(cw + u * ROWB));
                }
              } else {
                int u = 0;
                for (; u + 4 <= cnt; u += 4) {
                  const uint32_t c0 = lds_u8(cw + u * ROWB), c1 = lds_u8(cw + (u + 1) * ROWB);
                  const uint32_t c2 = lds_u8(cw + (u + 2) * ROWB), c3 = lds_u8(cw + (u + 3) * ROWB);
                  const float4 v0 = lds_f4(cb_addr + c0 * stride), v1 = lds_f4(cb_addr + c1 * stride);
                  const float4 v2 = lds_f4(cb_addr + c2 * stride), v3 = lds_f4(cb_addr + c3 * stride);
                  acc.x += v0.x; acc.y += v0.y; acc.z += v0.z; acc.w += v0.w;
                  acc.x += v1.x; acc.y += v1.y; acc.z += v1.z; acc.w += v1.w;
                  acc.x += v2.x; acc.y += v2.y; acc.z += v2.z; acc.w += v2.w;
                  acc.x += v3.x; acc.y += v3.y; acc.z += v3.z; acc.w += v3.w;
                }
                for (; u < cnt; ++u) add_vq(lds_u8(cw + u * ROWB));
              }
            } else {
              // long row: 32 edges at a time, ids / slots / code bytes from global memory
              for (uint32_t k0 = 0; k0 < (uint32_t)cnt; k0 += 32) {
                const int n = min(32, cnt - (int)k0);
                int64_t id_mine = 0;
                int sl_mine = -1;
                if (lane < n) {
                  id_mine = (int64_t)gids[beg[P] + k0 + lane];
                  if (HB != 0) sl_mine = hot_slot_of(p, id_mine);
                }
                for (int u = 0; u < n; ++u) {
                  const int sl_ = HB != 0 ? __shfl_sync(0xffffffffu, sl_mine, u) : -1;
                  const int64_t id = __shfl_sync(0xffffffffu, id_mine, u);
                  if (HB != 0 && sl_ >= 0) add_hot(load_hot(sl_));
                  else add_vq((uint32_t)__ldg(codes + id * ROWB + s));
                }
              }
            }
            // the ring entries of this row are free again
            __syncwarp();
            if (lane == 0) st_release(&sync->progress[warp], nxt < nrows ? ptr_s[nxt] : kDone);
            if (active) {
              if (p.reduce == F2C_MEAN) {
                const float degf = cnt == 0 ? 1.0f : (float)cnt;
                acc.x = acc.x / degf; acc.y = acc.y / degf; acc.z = acc.z / degf; acc.w = acc.w / degf;
              }
              const int64_t flat = (row0 + row) * p.feat_dim + col;
              if (p.drop.enabled) acc = dropout_apply4(acc, (uint64_t)flat, p.drop);
              stg_cs_f4(p.out + flat, acc);
            }
            // the next row's slots were not staged when this row began: wait for them now
            if (nxt < nrows && !ready[P ^ 1]) prepare(P ^ 1, nxt, true);
            row = nxt;
          }
        }
      }
      if (lane == 0) st_release(&sync->progress[warp], kDone);
    }
    __syncthreads();
  }
}

}  // namespace vqs

template <int HB, typename IdxT>
static int launch_stream_rows(const VqParams& p, const vqs::Layout& lay, int roww, int rows_per_chunk, int64_t n_chunks, dim3 grid,
                              size_t smem, cudaStream_t st, const char* op) {
  int* error = stream_error_word();
#define F2C_VQS(RW)                                                                                      \
  {                                                                                                      \
    auto kern = vqs::vq_stream_kernel<HB, IdxT, RW>;                                                     \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "%s: %s", op, cudaGetErrorString(e));           \
    kern<<<grid, vqs::kThreads, smem, st>>>(p, lay, rows_per_chunk, n_chunks, error);                    \
    return check_launch(op);                                                                             \
  }
  if (roww == 1) F2C_VQS(1)
  if (roww == 2) F2C_VQS(2)
  F2C_VQS(4)
#undef F2C_VQS
}

// Streamed kernel for the common shapes; *served = false (nothing launched) when the shape is not one of them.
int launch_vq_stream(VqParams& p, int hot_bits, int index_dtype, cudaStream_t st, const char* op, bool* served) {
  using namespace vqs;
  using namespace strm;
  *served = false;
  const int cs = p.cs;
  const int64_t row_bytes = p.n_cb;  // uint8 codes
  if (p.code_kind != 0 || p.K != 256 || p.n_dst >= (1ll << 30)) return F2C_OK;
  if (!(row_bytes == 4 || row_bytes == 8 || row_bytes == 16) || !aligned(p.codes, (size_t)row_bytes)) return F2C_OK;
  if (cs < 4 || cs > 128 || (128 % cs) != 0 || p.feat_dim % 4 != 0 || !aligned(p.out, 16) || !aligned(p.codebooks, 16)) return F2C_OK;
  if (!(hot_bits == 0 || hot_bits == 8 || hot_bits == 4)) return F2C_OK;
  if (hot_bits != 0) {
    if (p.sq_n_cb > 1 && p.sq_cs % 4 != 0) return F2C_OK;
    const int align = hot_bits == 8 ? 4 : 2;
    if (p.sq_row_bytes % align != 0 || p.sq_row_bytes >= (1ll << 31) || !aligned(p.sq_codes, align)) return F2C_OK;
  }
  const int idx_bytes = index_dtype == F2C_I32 ? 4 : 8;
  // a column part = at most 128 columns
  const int sub_per_128 = 128 / cs;
  const int roww = (int)row_bytes / 4;
  const int spq = cs < 32 ? 32 / cs : 1;
  const int stride = cs < 32 ? 128 : cs * 4;
  const int per_part = sub_per_128 < p.n_cb ? sub_per_128 : p.n_cb;
  const size_t cb_bytes = spq > 1 ? (size_t)ceil_div(per_part, spq) * p.K * 128 : (size_t)per_part * p.K * cs * 4;
  p.cb_per_part = per_part;
  p.fast_spq = spq;
  p.fast_stride = stride;
  p.fast_cb_bytes = (int)cb_bytes;
  const int parts = (int)ceil_div(p.n_cb, per_part);
  int64_t grid_x = current_sm_count() / parts;
  if (grid_x < 1) grid_x = 1;
  const int64_t need = ceil_div(p.n_dst, kConsumers);
  if (grid_x > need) grid_x = need;
  int rows_per_chunk = 0;
  int64_t n_chunks = 0;
  plan_chunks(p.n_dst, grid_x, &rows_per_chunk, &n_chunks);
  // ---- shared-memory map: codebooks | table | indptr slice | id batches | code ring | slot ring | watermarks
  Layout lay{};
  uint32_t at = (uint32_t)cb_bytes;
  lay.lut = at;
  if (hot_bits != 0) at += kLutBytes;
  lay.ptr = at;
  at += (uint32_t)(((rows_per_chunk + 1) * 4 + 15) & ~15);
  const uint32_t sync_bytes = 256 + 16;  // the watermarks, 16-byte aligned
  if ((size_t)at + sync_bytes + 4096 > kSmemTotal) return F2C_OK;
  const uint32_t room = kSmemTotal - at - sync_bytes;
  const uint32_t per_edge = (uint32_t)row_bytes + (hot_bits != 0 ? 4u : 0u);
  // room >= (kIdLead + 1) * batch * idx + ((kRowLag + 1) * batch + 2 * kLongRow) * per_edge   (ring + its mirror),
  // batch = kProducers * sub
  uint32_t sub = (room - (2u * kLongRow + 4u) * per_edge) / (kProducers * ((kIdLead + 1) * idx_bytes + (kRowLag + 1) * per_edge));
  if (sub > 64u) sub = 64u;
  sub &= ~7u;
  if (sub < 8u) return F2C_OK;
  lay.sub = sub;
  const uint32_t batch = sub * kProducers;
  lay.ids = at;
  at += (kIdLead + 1) * batch * idx_bytes;
  const uint32_t cap = ((kSmemTotal - sync_bytes - at) / per_edge - kLongRow) & ~3u;  // >= (kRowLag + 1) * batch + kLongRow
  lay.cap = cap;
  lay.codes = at;
  at += (cap + kLongRow) * (uint32_t)row_bytes;
  lay.slots = at;
  if (hot_bits != 0) at += (cap + kLongRow) * 4u;
  lay.sync = (at + 15u) & ~15u;
  const size_t smem = lay.sync + 256;
  if (smem > kSmemTotal) return F2C_OK;
  dim3 grid((unsigned)grid_x, (unsigned)parts);
  *served = true;
#define F2C_VQS_IDX(HB)                                                                                                         \
  return index_dtype == F2C_I32 ? launch_stream_rows<HB, int32_t>(p, lay, roww, rows_per_chunk, n_chunks, grid, smem, st, op)   \
                                : launch_stream_rows<HB, int64_t>(p, lay, roww, rows_per_chunk, n_chunks, grid, smem, st, op)
  if (hot_bits == 0) F2C_VQS_IDX(0);
  if (hot_bits == 8) F2C_VQS_IDX(8);
  F2C_VQS_IDX(4);
#undef F2C_VQS_IDX
}

}  // namespace f2c
