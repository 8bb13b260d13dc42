// Pieces shared by the fused SQ decode + aggregation kernels (fused_sq_spmm.cu: rows prefetched into registers;
// fused_sq_stream.cu: rows streamed into a shared-memory ring by a producer warp): the byte-indexed decode table,
// the packed accumulators and the per-row accumulate step.  The decode expression is the reference's
// (src/fusion_spmm.cu:199-223), evaluated once per table entry.
#pragma once
#include "common.cuh"

namespace f2c {

enum { DEC_ARITH = 0, DEC_LUT = 1 };
enum { CODE_U8 = 0, CODE_I8 = 1, CODE_I16 = 2 };

template <int VEC> struct VecLoad;
template <> struct VecLoad<4> {
  uint32_t w[1];
  __device__ __forceinline__ void load(const void* p) { w[0] = ldg_nc_u32(p); }
  __device__ __forceinline__ void load_shared(uint32_t a) { asm volatile("ld.shared.b32 %0, [%1];" : "=r"(w[0]) : "r"(a)); }
  __device__ __forceinline__ void zero() { w[0] = 0u; }
};
template <> struct VecLoad<8> {
  uint32_t w[2];
  __device__ __forceinline__ void load(const void* p) { uint2 v = ldg_nc_u64(p); w[0] = v.x; w[1] = v.y; }
  __device__ __forceinline__ void load_shared(uint32_t a) {
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "r"(a));
  }
  __device__ __forceinline__ void zero() { w[0] = 0u; w[1] = 0u; }
};

// Decode table geometry: 256 slabs of 256 bytes (64 KB).  A slab holds COPIES copies of the FLOATS
// floats its byte encodes; one copy is one vector read (1-bit codes: two 16-byte halves kept 128 bytes
// apart so that eight lanes reading a half touch eight different bank groups).
template <int BITS> struct Lut {
  static constexpr int B = (BITS == 1 || BITS == 2 || BITS == 4) ? BITS : 8;
  static constexpr int FLOATS = 8 / B;                              // 8, 4, 2, 1
  static constexpr int COPY_BYTES = FLOATS >= 4 ? 16 : FLOATS * 4;
  static constexpr int HALVES = FLOATS == 8 ? 2 : 1;
  static constexpr int COPIES = 256 / (COPY_BYTES * HALVES) > 32 ? 32 : 256 / (COPY_BYTES * HALVES);  // 8, 16, 32, 32
  static constexpr int NCODE = 1 << B;
  static constexpr int TABLE_BYTES = 256 * 256;
  __device__ static __forceinline__ uint32_t lane_offset(int lane) { return (uint32_t)(lane & (COPIES - 1)) * COPY_BYTES; }
};

// Accumulators: fp32 pairs packed in 64-bit registers where the decode delivers pairs (table decode of
// 1/2/4-bit codes), so that every add is one add.f32x2 on operands that are already pairs; scalar
// fp32 registers otherwise.  Each half rounds to nearest exactly like a scalar add.
template <int EPL, bool PACKED> struct Acc;
template <int EPL> struct Acc<EPL, true> {
  unsigned long long v[EPL / 2];
  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int i = 0; i < EPL / 2; ++i) v[i] = 0ull;
  }
  __device__ __forceinline__ void add_pair(int i, unsigned long long x) { asm("add.rn.f32x2 %0, %0, %1;" : "+l"(v[i]) : "l"(x)); }
  __device__ __forceinline__ void add_one(int, float) {}
  __device__ __forceinline__ float4 chunk(int q) const {
    return make_float4(__uint_as_float((uint32_t)v[2 * q]), __uint_as_float((uint32_t)(v[2 * q] >> 32)),
                       __uint_as_float((uint32_t)v[2 * q + 1]), __uint_as_float((uint32_t)(v[2 * q + 1] >> 32)));
  }
  __device__ __forceinline__ float get(int e) const { return __uint_as_float((uint32_t)(v[e >> 1] >> (32 * (e & 1)))); }
};
template <int EPL> struct Acc<EPL, false> {
  float v[EPL];
  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int i = 0; i < EPL; ++i) v[i] = 0.0f;
  }
  __device__ __forceinline__ void add_pair(int, unsigned long long) {}
  __device__ __forceinline__ void add_one(int i, float x) { v[i] += x; }
  __device__ __forceinline__ float4 chunk(int q) const { return make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]); }
  __device__ __forceinline__ float get(int e) const { return v[e]; }
};

__device__ __forceinline__ unsigned long long lds_b64(uint32_t a) {
  unsigned long long v;
  asm volatile("ld.shared.b64 %0, [%1];" : "=l"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ void lds_b64x2(uint32_t a, unsigned long long& x, unsigned long long& y) {
  asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(x), "=l"(y) : "r"(a));
}
__device__ __forceinline__ float lds_f32(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}

// Add the decoded elements of one lane's share of a neighbour row to its accumulators.
// `table` = shared-window address of the decode table, lane_off = this lane's copy offset in a slab; aligned-table
// kernels pass table = 0 and the (64 KB aligned) address inside lane_off.
template <int BITS, int VEC, int DEC, bool ALIGNED, typename AccT>
__device__ __forceinline__ void sq_accumulate(AccT& acc, const VecLoad<VEC>& data, uint32_t table, uint32_t lane_off, int code_kind,
                                              float scale, float emin, float mean) {
  constexpr int NW = VEC / 4;
#pragma unroll
  for (int w = 0; w < NW; ++w) {
    const uint32_t word = data.w[w];
    if (DEC == DEC_LUT) {
      using L = Lut<BITS>;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        // result bytes [lane_off.b0, word.b_b, lane_off.b2, lane_off.b3]  ==  (byte << 8) | lane_off
        const uint32_t e = (ALIGNED ? 0u : table) + __byte_perm(word, lane_off, 0x7604u | (uint32_t)(b << 4));
        const int k = w * 4 + b;  // byte number inside the lane's slice
        if (L::FLOATS == 1) {
          acc.add_one(k, lds_f32(e));
        } else if (L::FLOATS == 2) {
          acc.add_pair(k, lds_b64(e));
        } else {
#pragma unroll
          for (int h = 0; h < L::HALVES; ++h) {
            unsigned long long x, y;
            lds_b64x2(e + 128 * h, x, y);
            acc.add_pair((k * L::HALVES + h) * 2, x);
            acc.add_pair((k * L::HALVES + h) * 2 + 1, y);
          }
        }
      }
    } else if (BITS == 16) {
      acc.add_one(w * 2 + 0, sq_decode<BITS>((float)(int16_t)(word & 0xFFFFu), scale, emin, mean));
      acc.add_one(w * 2 + 1, sq_decode<BITS>((float)(int16_t)(word >> 16), scale, emin, mean));
    } else if (BITS == 8) {
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        uint32_t byte = (word >> (8 * b)) & 0xFFu;
        float c = code_kind == CODE_I8 ? (float)(int8_t)byte : (float)byte;
        acc.add_one(w * 4 + b, sq_decode<BITS>(c, scale, emin, mean));
      }
    } else {  // 1-, 2- or 4-bit arithmetic decode
      constexpr int B = (BITS == 1 || BITS == 2 || BITS == 4) ? BITS : 4;
      constexpr int PER_WORD = 32 / B;
#pragma unroll
      for (int i = 0; i < PER_WORD; ++i)
        acc.add_one(w * PER_WORD + i, sq_decode<BITS>((float)((word >> (B * i)) & ((1u << B) - 1u)), scale, emin, mean));
    }
  }
}

// Build the decode table with threads tid = 0..nthr-1; `sync` is a barrier over exactly those threads.
//   table    256 slabs of 256 bytes, followed by a 256-byte zero slab (neighbour slots beyond a row's degree read it)
//   values   scratch of n_rows * NCODE floats, n_rows = min(G, COPIES)
// Copy c of a slab serves the lanes with lane % COPIES == c, whose lane group index is c % G.  Phase 1 decodes each code
// value once per distinct codebook row with the element-wise expression; phase 2 assembles the byte-indexed,
// bank-replicated table from those values, 16 bytes per store.
template <int BITS, int EPL, typename Sync>
__device__ __forceinline__ void build_sq_table(unsigned char* table, float* values, const float* __restrict__ codebooks, int n_cb,
                                               int column_slice, int G, int code_kind, int tid, int nthr, Sync sync) {
  using L = Lut<BITS>;
  const int n_rows = G < L::COPIES ? G : L::COPIES;
  for (int i = tid; i < n_rows * L::NCODE; i += nthr) {
    int code = i & (L::NCODE - 1), g = i / L::NCODE;
    int row = (g * EPL) / column_slice;
    if (row >= n_cb) row = n_cb - 1;
    float e0 = __ldg(codebooks + row * kCodebookDim + 2), e1 = __ldg(codebooks + row * kCodebookDim + 3);
    float m = __ldg(codebooks + row * kCodebookDim + 4);
    float c = (L::B == 8 && code_kind == CODE_I8) ? (float)(int8_t)code : (float)code;
    values[i] = sq_decode<BITS>(c, sq_scale<BITS>(e0, e1), e0, m);
  }
  sync();
  constexpr int SPAN = L::HALVES == 2 ? 128 : 256;
  for (int i = tid; i < 256 * 16; i += nthr) {
    const int byte = i >> 4, j = i & 15;
    float v[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int o = 16 * j + 4 * t;  // byte offset inside the slab
      const int h = L::HALVES == 2 ? o / 128 : 0;
      const int oo = o % SPAN;
      const int copy = oo / L::COPY_BYTES;
      const int f = (oo % L::COPY_BYTES) / 4 + 4 * h;
      const int g = copy & (n_rows - 1);
      v[t] = copy < L::COPIES ? values[g * L::NCODE + ((byte >> (L::B * f)) & (L::NCODE - 1))] : 0.0f;
    }
    *reinterpret_cast<float4*>(table + i * 16) = make_float4(v[0], v[1], v[2], v[3]);
  }
  for (int i = tid; i < 64; i += nthr) reinterpret_cast<float*>(table + L::TABLE_BYTES)[i] = 0.0f;
  sync();
}

// Mean / dropout / store of the R = 32 >> logG destination rows a warp has just summed: the sums are staged in the
// warp's shared-memory area (XOR-swizzled so that neither the writes nor the reads collide), read back row by row,
// divided by the degree (two FMA corrections reproduce the IEEE quotient) and written as whole rows.
//   stage      the warp's area of 32 * EPL floats
//   row_base   first destination row of the warp's group, n_rows_left = rows of the block from row_base on
template <int EPL, typename AccT>
__device__ __forceinline__ void sq_store_rows(const AccT& acc, float4* stage, int lane, int logG, int deg, bool have_row,
                                              int64_t row_base, int64_t n_rows_left, int feat_dim, int reduce, bool div_safe,
                                              const DropoutArgs& drop, float* __restrict__ out) {
  constexpr int Q = EPL / 4;                                    // chunks (float4) per lane
  constexpr int LQ = Q >= 8 ? 3 : Q == 4 ? 2 : Q == 2 ? 1 : 0;  // low chunk-index bits that only depend on q
  const int G = 1 << logG, lane_g = lane & (G - 1), sub = lane >> logG, rows_per_warp = 32 >> logG;
  const int NC = feat_dim >> 2;  // chunks per output row
  const int NCP = Q << logG;     // row stride of the staging area (>= NC)
  // chunk c of a row is kept at c ^ m, m = the lane bits that the low bits of c do not already spread
  // over the banks; m only touches the q part of the index, so a lane stays inside its own Q chunks
  if (have_row) {
    const int m = ((lane & 7) >> (3 - LQ)) & ((1 << LQ) - 1);
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      const int c4 = lane_g * Q + q;
      if (c4 < NC) stage[sub * NCP + (c4 ^ m)] = acc.chunk(q);
    }
  }
  // reciprocal of the row's degree, once per lane group (0 marks "do not divide")
  float my_rcp = 0.0f;
  if (reduce == F2C_MEAN && deg > 1) my_rcp = 1.0f / (float)deg;
  __syncwarp();
  for (int row = 0; row < rows_per_warp; ++row) {
    if (row >= n_rows_left) break;
    const int64_t dr = row_base + row;
    const float rcp = __shfl_sync(0xffffffffu, my_rcp, row << logG);
    const float degf = (float)__shfl_sync(0xffffffffu, deg, row << logG);
    for (int c = lane; c < NC; c += 32) {
      const int writer = (row << logG) + c / Q;  // lane that produced chunk c
      const int m = ((writer & 7) >> (3 - LQ)) & ((1 << LQ) - 1);
      float4 v = stage[row * NCP + (c ^ m)];
      if (rcp != 0.0f) {
        if (div_safe) {
          v.x = div_exact_fast(v.x, degf, rcp); v.y = div_exact_fast(v.y, degf, rcp);
          v.z = div_exact_fast(v.z, degf, rcp); v.w = div_exact_fast(v.w, degf, rcp);
        } else {
          v.x = div_exact(v.x, degf, rcp); v.y = div_exact(v.y, degf, rcp);
          v.z = div_exact(v.z, degf, rcp); v.w = div_exact(v.w, degf, rcp);
        }
      }
      if (drop.enabled) v = dropout_apply4(v, (uint64_t)(dr * feat_dim + 4 * c), drop);
      stg_cs_f4(out + dr * feat_dim + 4 * c, v);
    }
  }
  __syncwarp();
}

}  // namespace f2c
