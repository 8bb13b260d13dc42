// Fused SQ decode + aggregation, "one warp per destination row" layout (included by fused_sq_spmm.cu).
//
// A lane owns four consecutive output columns of each 128-column tile, i.e. 4*BITS/8 bytes of every
// neighbour row (half a byte for 1-bit codes).  Compared with giving a lane a long slice of the row
// this keeps the register footprint small enough for 48-64 resident warps per SM - the kernel lives
// on latency hiding, a sampled block offers ~10^5 independent rows but each one is a chain
// indptr -> indices -> rows - and the aggregated row leaves the warp as one coalesced 512-byte store,
// with no transposition.  Neighbour ids are fetched 32 at a time, coalesced, and broadcast by shuffle;
// the ids of the NEXT row and the indptr pair of the one after are prefetched while the current row is
// decoded.  Decode is the byte-indexed shared-memory table (Lut<>), arithmetic for 16-bit codes.
#pragma once

namespace f2c {

// Bytes of a neighbour row one lane consumes per 128-column tile, times two (1-bit: half a byte).
template <int BITS> struct RowWarp {
  static constexpr int HALF_BYTES = BITS;  // 2 * (4 columns * BITS / 8)
  // byte offset inside a 256-byte table slab for this lane (copy select + nibble half for 1-bit)
  __device__ static __forceinline__ uint32_t lane_offset(int lane) {
    if (BITS == 8) return (uint32_t)lane * 4u;            // 32 copies x 4 B
    if (BITS == 4) return (uint32_t)lane * 8u;            // 32 copies x 8 B
    if (BITS == 2) return (uint32_t)(lane & 15) * 16u;    // 16 copies x 16 B
    return (uint32_t)(lane & 7) * 16u + (uint32_t)(lane & 1) * 128u;  // 1 bit: 8 copies, odd lanes take floats 4..7
  }
  // table copy a lane reads -> lanes sharing a copy must share a codebook row
  static constexpr int COPIES = BITS >= 4 ? 32 : BITS == 2 ? 16 : 8;
};

template <int BITS>
__device__ __forceinline__ uint32_t rowwarp_load(const uint8_t* p) {
  // p already points at this lane's first byte of the row
  if (BITS == 16) return 0;  // handled separately (two words)
  if (BITS == 8) return ldg_nc_u32(p);
  if (BITS == 4) { uint16_t v; asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p)); return v; }
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u8 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

template <int BITS, typename IdxT, int DEC>
__global__ void __launch_bounds__(512) sq_spmm_rowwarp_kernel(const SqParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int U = 8;  // row loads in flight per lane
  const int lane = threadIdx.x & 31;

  if (DEC == DEC_LUT && !(p.ablate & 4)) {
    using L = Lut<BITS>;
    constexpr int COPIES = RowWarp<BITS>::COPIES;
    // phase 1: the 2^B code values of every codebook row a table copy can belong to
    float* base = reinterpret_cast<float*>(smem_raw + L::TABLE_BYTES);  // [COPIES][NCODE]
    for (int i = threadIdx.x; i < COPIES * L::NCODE; i += blockDim.x) {
      const int code = i & (L::NCODE - 1), copy = i / L::NCODE;
      // copy c serves lanes c, c + COPIES, ...; the host guarantees they share one codebook row
      const int col = BITS == 1 ? (copy >> 1) * 8 : copy * 4;  // first column of a lane that uses this copy
      int row = col / p.column_slice;
      if (row >= p.n_cb) row = p.n_cb - 1;
      const float e0 = __ldg(p.codebooks + row * kCodebookDim + 2), e1 = __ldg(p.codebooks + row * kCodebookDim + 3);
      const float m = __ldg(p.codebooks + row * kCodebookDim + 4);
      const float c = (L::B == 8 && p.code_kind == CODE_I8) ? (float)(int8_t)code : (float)code;
      base[i] = sq_decode<BITS>(c, sq_scale<BITS>(e0, e1), e0, m);
    }
    __syncthreads();
    // phase 2: slab `byte`, 16 bytes at a time
    constexpr int SPAN = L::HALVES == 2 ? 128 : 256;
    for (int i = threadIdx.x; i < 256 * 16; i += blockDim.x) {
      const int byte = i >> 4, j = i & 15;
      float v[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int o = 16 * j + 4 * t;
        const int h = L::HALVES == 2 ? o / 128 : 0;
        const int oo = o % SPAN;
        const int copy = oo / L::COPY_BYTES;
        const int f = (oo % L::COPY_BYTES) / 4 + 4 * h;
        v[t] = copy < COPIES ? base[copy * L::NCODE + ((byte >> (L::B * f)) & (L::NCODE - 1))] : 0.0f;
      }
      *reinterpret_cast<float4*>(smem_raw + i * 16) = make_float4(v[0], v[1], v[2], v[3]);
    }
    __syncthreads();
  }
  const uint32_t lane_off = RowWarp<BITS>::lane_offset(lane);

  const IdxT* __restrict__ indptr = reinterpret_cast<const IdxT*>(p.indptr);
  const IdxT* __restrict__ indices = reinterpret_cast<const IdxT*>(p.indices);
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int n_tiles = (p.feat_dim + 127) >> 7;
  const int tile_bytes = 16 * BITS;  // bytes of a code row per 128-column tile
  const int lane_byte = (lane * RowWarp<BITS>::HALF_BYTES) >> 1;

  // pipeline: row d (ids of its first 32 neighbours in `mine`), indptr pair of row d + n_warps
  int64_t d = warp;
  int64_t beg0 = 0, end0 = 0, beg1 = 0, end1 = 0;
  if (d < p.n_dst) { beg0 = (int64_t)indptr[d]; end0 = (int64_t)indptr[d + 1]; }
  if (d + n_warps < p.n_dst) { beg1 = (int64_t)indptr[d + n_warps]; end1 = (int64_t)indptr[d + n_warps + 1]; }
  uint32_t mine = beg0 + lane < end0 ? (uint32_t)indices[beg0 + lane] : 0u;

  for (; d < p.n_dst; d += n_warps) {
    // prefetch for the next two rows
    const uint32_t mine_next = beg1 + lane < end1 ? (uint32_t)indices[beg1 + lane] : 0u;
    int64_t beg2 = 0, end2 = 0;
    if (d + 2 * n_warps < p.n_dst) { beg2 = (int64_t)indptr[d + 2 * n_warps]; end2 = (int64_t)indptr[d + 2 * n_warps + 1]; }

    const int deg = (int)(end0 - beg0);
    const float degf = (float)(deg > 0 ? deg : 1);
    const float rcp = 1.0f / degf;

    for (int tile = 0; tile < n_tiles; ++tile) {
      const int col = tile * 128 + lane * 4;
      const bool active = col < p.feat_dim;
      const uint8_t* __restrict__ lane_codes = p.codes + (int64_t)tile * tile_bytes + lane_byte;
      float scale = 0.f, emin = 0.f, mean = 0.f;
      if (DEC == DEC_ARITH) {
        int row = (active ? col : 0) / p.column_slice;
        if (row >= p.n_cb) row = p.n_cb - 1;
        emin = __ldg(p.codebooks + row * kCodebookDim + 2);
        const float emax = __ldg(p.codebooks + row * kCodebookDim + 3);
        mean = __ldg(p.codebooks + row * kCodebookDim + 4);
        scale = sq_scale<BITS>(emin, emax);
      }
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;

      for (int k0 = 0; k0 < deg; k0 += 32) {
        const int cnt = deg - k0 < 32 ? deg - k0 : 32;
        const uint32_t ids = k0 == 0 ? mine : (k0 + lane < deg ? (uint32_t)indices[beg0 + k0 + lane] : 0u);
        for (int t0 = 0; t0 < cnt; t0 += U) {
          uint32_t w0[U], w1[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint32_t src = __shfl_sync(0xffffffffu, ids, (t0 + u) & 31);
            w0[u] = 0; w1[u] = 0;
            if (t0 + u < cnt && active && !(p.ablate & 8)) {
              const uint8_t* q = lane_codes + (int64_t)src * p.row_bytes;
              if (BITS == 16) { uint2 v = ldg_nc_u64(q); w0[u] = v.x; w1[u] = v.y; }
              else w0[u] = rowwarp_load<BITS>(q);
            }
          }
          if (!(p.ablate & 1)) {
#pragma unroll
          for (int u = 0; u < U; ++u) {
            if (t0 + u < cnt) {
              if (BITS == 16) {
                a0 += sq_decode<BITS>((float)(int16_t)(w0[u] & 0xFFFFu), scale, emin, mean);
                a1 += sq_decode<BITS>((float)(int16_t)(w0[u] >> 16), scale, emin, mean);
                a2 += sq_decode<BITS>((float)(int16_t)(w1[u] & 0xFFFFu), scale, emin, mean);
                a3 += sq_decode<BITS>((float)(int16_t)(w1[u] >> 16), scale, emin, mean);
              } else if (DEC == DEC_LUT) {
                if (BITS == 8) {
#pragma unroll
                  for (int b = 0; b < 4; ++b) {
                    const float v = *reinterpret_cast<const float*>(smem_raw + __byte_perm(w0[u], lane_off, 0x7604u | (uint32_t)(b << 4)));
                    if (b == 0) a0 += v; else if (b == 1) a1 += v; else if (b == 2) a2 += v; else a3 += v;
                  }
                } else if (BITS == 4) {
                  const float2 lo = *reinterpret_cast<const float2*>(smem_raw + __byte_perm(w0[u], lane_off, 0x7604u));
                  const float2 hi = *reinterpret_cast<const float2*>(smem_raw + __byte_perm(w0[u], lane_off, 0x7614u));
                  add2(a0, a1, lo.x, lo.y);
                  add2(a2, a3, hi.x, hi.y);
                } else {  // 2-bit: one byte = 4 columns; 1-bit: the lane's nibble of the byte (half selected by lane_off)
                  const float4 v = *reinterpret_cast<const float4*>(smem_raw + __byte_perm(w0[u], lane_off, 0x7604u));
                  add2(a0, a1, v.x, v.y);
                  add2(a2, a3, v.z, v.w);
                }
              } else {  // arithmetic decode of packed / 8-bit codes
                constexpr int B = BITS >= 8 ? 8 : BITS;
                uint32_t raw = w0[u];
                if (BITS == 1) raw >>= (lane & 1) * 4;
                float c[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const uint32_t code = (raw >> (B * e)) & ((1u << B) - 1u);
                  c[e] = (BITS == 8 && p.code_kind == CODE_I8) ? (float)(int8_t)code : (float)code;
                }
                a0 += sq_decode<BITS>(c[0], scale, emin, mean);
                a1 += sq_decode<BITS>(c[1], scale, emin, mean);
                a2 += sq_decode<BITS>(c[2], scale, emin, mean);
                a3 += sq_decode<BITS>(c[3], scale, emin, mean);
              }
            }
          }
          }
        }
      }

      if (active && !(p.ablate & 2)) {
        float4 v = make_float4(a0, a1, a2, a3);
        if (p.reduce == F2C_MEAN && deg > 1) {
          v.x = div_exact(v.x, degf, rcp); v.y = div_exact(v.y, degf, rcp);
          v.z = div_exact(v.z, degf, rcp); v.w = div_exact(v.w, degf, rcp);
        }
        if (p.drop.enabled) v = dropout_apply4(v, (uint64_t)(d * p.feat_dim + col), p.drop);
        stg_cs_f4(p.out + d * p.feat_dim + col, v);
      }
    }
    mine = mine_next;
    beg0 = beg1; end0 = end1; beg1 = beg2; end1 = end2;
  }
}

// Host side: can this layout serve the call, and with which decode?
template <int BITS, typename IdxT>
static int launch_rowwarp(SqParams p, bool lut, cudaStream_t st, bool* handled) {
  *handled = true;
  size_t smem = 0;
  int threads = 512;
  cudaError_t e = cudaSuccess;
  int resident = 1;
  if (lut) {
    auto kern = sq_spmm_rowwarp_kernel<BITS, IdxT, DEC_LUT>;
    smem = 65536 + (size_t)RowWarp<BITS>::COPIES * (BITS >= 8 ? 256 : (1 << BITS)) * sizeof(float);
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) {
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, threads, smem) != cudaSuccess || resident < 1) resident = 1;
      if (g_tune_ctas_per_sm > 0) resident = g_tune_ctas_per_sm;
      int64_t grid = ceil_div(p.n_dst, threads / 32);
      if (grid > (int64_t)kSmCount * resident) grid = (int64_t)kSmCount * resident;
      kern<<<(unsigned)grid, threads, smem, st>>>(p);
    }
  } else {
    auto kern = sq_spmm_rowwarp_kernel<BITS, IdxT, DEC_ARITH>;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, threads, 0) != cudaSuccess || resident < 1) resident = 1;
    if (g_tune_ctas_per_sm > 0) resident = g_tune_ctas_per_sm;
    int64_t grid = ceil_div(p.n_dst, threads / 32);
    if (grid > (int64_t)kSmCount * resident) grid = (int64_t)kSmCount * resident;
    kern<<<(unsigned)grid, threads, 0, st>>>(p);
  }
  if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "sq_decompress_spmm_csr: %s", cudaGetErrorString(e));
  return check_launch("sq_decompress_spmm_csr");
}

}  // namespace f2c
