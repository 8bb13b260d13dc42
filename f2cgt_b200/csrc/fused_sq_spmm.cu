// Fused SQ decode + mean/sum aggregation over a CSC block
// (reference operator sq_decompress_spmm_csr, src/fusion_spmm.cu:143-272).
//
//   out[d, :] = (sum_{k in N(d), CSC order} decode(codes[indices[k], :])) / max(deg(d), 1)
//
// The decoded fp32 rows never exist in memory: a neighbour's compressed row (16..256 B) is fetched
// with one 128-bit (or 64/32-bit) read-only load per lane, decoded in registers and added to fp32
// register accumulators in CSC order, which makes the result equal to decode-then-aggregate bit for
// bit and independent of launch geometry.
//
// Layout of work.  A destination row is owned by a group of G = row_bytes / VEC consecutive lanes
// (G a power of two, so a warp serves 32/G rows at once); lane g of the group owns bytes
// [g*VEC, (g+1)*VEC) of every neighbour row and the EPL = VEC*8/bits output columns they encode.
// Per step the group issues U independent row loads before it decodes any of them, so
// threads * U * VEC bytes are in flight per SM - what an HBM-latency-bound gather needs.
//
// Decode.  One MUFU.EX2 per element would cap the kernel below the HBM roofline for narrow codes, so
// 2/4/8-bit codes are decoded through a shared-memory table built at kernel start WITH THE SAME
// EXPRESSION as the element-wise decode (hence the same bits): the table is indexed by a whole code
// byte and returns the 4 / 2 / 1 floats the byte encodes, and it is replicated once per bank group
// (8 / 16 / 32 copies, 32 KB in all) so that a warp's lookups never collide.  1-bit codes are +-mean:
// the sign bit is injected into the constant with two integer ops.  16-bit codes (and tables that
// would need more than one codebook row per lane) use the arithmetic decode.
//
// Grid: persistent, a multiple of the SM count; each CTA builds its table once and walks row tiles
// with a grid stride.
#include "common.cuh"

namespace f2c {

int validate_sq(const char* op, int code_dtype, int64_t n_codebooks, int64_t src_dim, int64_t feat_dim, int bits,
                int64_t column_slice);

// tuning knobs (0 = heuristic); set through f2c_set_tuning for experiments
int g_tune_vec = 0, g_tune_u = 0, g_tune_lut = -1, g_tune_ctas_per_sm = 0;

template <int VEC> struct VecLoad;
template <> struct VecLoad<4> {
  uint32_t w[1];
  __device__ __forceinline__ void load(const void* p) { w[0] = ldg_nc_u32(p); }
};
template <> struct VecLoad<8> {
  uint32_t w[2];
  __device__ __forceinline__ void load(const void* p) { uint2 v = ldg_nc_u64(p); w[0] = v.x; w[1] = v.y; }
};
template <> struct VecLoad<16> {
  uint32_t w[4];
  __device__ __forceinline__ void load(const void* p) { uint4 v = ldg_nc_u128(p); w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; }
};

enum { DEC_ARITH = 0, DEC_LUT = 1 };
enum { CODE_U8 = 0, CODE_I8 = 1, CODE_I16 = 2 };

// Number of table copies for a given code width: one per shared-memory bank group of the lookup.
template <int BITS> struct LutGeom {
  static constexpr int FLOATS = 8 / BITS;             // floats returned per byte lookup: 1, 2, 4
  static constexpr int COPIES = 32 / FLOATS;          // 32, 16, 8
  static constexpr int BYTES = 256 * COPIES * FLOATS * 4;  // 32 KB
};

struct SqParams {
  const uint8_t* codes;
  const float* codebooks;
  const void* indptr;
  const void* indices;
  float* out;
  int64_t n_dst;
  int64_t row_bytes;
  int feat_dim;
  int column_slice;
  int n_cb;
  int logG;
  int code_kind;
  int reduce;
  int vec_store;
  DropoutArgs drop;
};

template <int BITS, int VEC, int U, typename IdxT, int DEC>
__global__ void __launch_bounds__(256) sq_spmm_kernel(const SqParams p) {
  constexpr int EPL = BITS == 16 ? VEC / 2 : VEC * 8 / BITS;  // output columns per lane
  constexpr int NW = VEC / 4;                                  // 32-bit words per lane per row
  extern __shared__ __align__(16) unsigned char smem_raw[];

  const int lane = threadIdx.x & 31;
  const int G = 1 << p.logG;
  const int lane_g = lane & (G - 1);
  const int sub = lane >> p.logG;
  const int rows_per_warp = 32 >> p.logG;
  const int byte0 = lane_g * VEC;
  const bool lane_active = byte0 < p.row_bytes;
  const int c0 = lane_g * EPL;

  // Codebook row of this lane's columns (the host guarantees they share one row on this path).
  int cb_row = c0 / p.column_slice;
  if (cb_row >= p.n_cb) cb_row = p.n_cb - 1;
  const float emin = __ldg(p.codebooks + cb_row * kCodebookDim + 2);
  const float emax = __ldg(p.codebooks + cb_row * kCodebookDim + 3);
  const float mean = __ldg(p.codebooks + cb_row * kCodebookDim + 4);
  const float scale = sq_scale<BITS>(emin, emax);
  (void)scale; (void)mean;

  if (DEC == DEC_LUT) {
    // table[byte][copy][FLOATS]; copy c serves lanes with lane % COPIES == c, whose lane_g is c % G
    constexpr int FLOATS = LutGeom<(BITS == 2 || BITS == 4 || BITS == 8) ? BITS : 8>::FLOATS;
    constexpr int COPIES = 32 / FLOATS;
    constexpr int B = (BITS == 2 || BITS == 4) ? BITS : 8;
    float* lut = reinterpret_cast<float*>(smem_raw);
    for (int i = threadIdx.x; i < 256 * COPIES * FLOATS; i += blockDim.x) {
      int f = i % FLOATS, copy = (i / FLOATS) % COPIES, byte = i / (FLOATS * COPIES);
      int row = ((copy & (G - 1)) * EPL) / p.column_slice;
      if (row >= p.n_cb) row = p.n_cb - 1;
      float e0 = __ldg(p.codebooks + row * kCodebookDim + 2), e1 = __ldg(p.codebooks + row * kCodebookDim + 3);
      float m = __ldg(p.codebooks + row * kCodebookDim + 4);
      float c;
      if (B == 8) c = p.code_kind == CODE_I8 ? (float)(int8_t)byte : (float)byte;
      else c = (float)((byte >> (B * f)) & ((1 << B) - 1));
      lut[i] = sq_decode<BITS>(c, sq_scale<BITS>(e0, e1), e0, m);
    }
    __syncthreads();
  }

  const IdxT* __restrict__ indptr = reinterpret_cast<const IdxT*>(p.indptr);
  const IdxT* __restrict__ indices = reinterpret_cast<const IdxT*>(p.indices);
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const uint8_t* __restrict__ my_codes = p.codes + byte0;

  for (int64_t row_base = warp * rows_per_warp; row_base < p.n_dst; row_base += n_warps * rows_per_warp) {
    const int64_t d = row_base + sub;
    const bool valid = d < p.n_dst && lane_active;
    int64_t begin = 0, end = 0;
    if (valid) { begin = (int64_t)indptr[d]; end = (int64_t)indptr[d + 1]; }
    float acc[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = 0.0f;

    for (int64_t k = begin; k < end; k += U) {
      VecLoad<VEC> data[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (k + u < end) {
          int64_t src = (int64_t)indices[k + u];
          data[u].load(my_codes + src * p.row_bytes);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (k + u < end) {
#pragma unroll
          for (int w = 0; w < NW; ++w) {
            const uint32_t word = data[u].w[w];
            if (BITS == 1) {
              const uint32_t negmean = __float_as_uint(-mean);
#pragma unroll
              for (int i = 0; i < 32; ++i)
                acc[w * 32 + i] += __uint_as_float(negmean ^ ((word << (31 - i)) & 0x80000000u));
            } else if (BITS == 16) {
              acc[w * 2 + 0] += sq_decode<BITS>((float)(int16_t)(word & 0xFFFFu), scale, emin, mean);
              acc[w * 2 + 1] += sq_decode<BITS>((float)(int16_t)(word >> 16), scale, emin, mean);
            } else if (DEC == DEC_LUT && BITS == 8) {
              const float* lut = reinterpret_cast<const float*>(smem_raw) + lane;
#pragma unroll
              for (int b = 0; b < 4; ++b) acc[w * 4 + b] += lut[((word >> (8 * b)) & 0xFFu) * 32];
            } else if (DEC == DEC_LUT && BITS == 4) {
              const float2* lut = reinterpret_cast<const float2*>(smem_raw) + (lane & 15);
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                float2 v = lut[((word >> (8 * b)) & 0xFFu) * 16];
                acc[w * 8 + 2 * b] += v.x;
                acc[w * 8 + 2 * b + 1] += v.y;
              }
            } else if (DEC == DEC_LUT && BITS == 2) {
              const float4* lut = reinterpret_cast<const float4*>(smem_raw) + (lane & 7);
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                float4 v = lut[((word >> (8 * b)) & 0xFFu) * 8];
                acc[w * 16 + 4 * b] += v.x;
                acc[w * 16 + 4 * b + 1] += v.y;
                acc[w * 16 + 4 * b + 2] += v.z;
                acc[w * 16 + 4 * b + 3] += v.w;
              }
            } else if (BITS == 8) {
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                uint32_t byte = (word >> (8 * b)) & 0xFFu;
                float c = p.code_kind == CODE_I8 ? (float)(int8_t)byte : (float)byte;
                acc[w * 4 + b] += sq_decode<BITS>(c, scale, emin, mean);
              }
            } else {  // 2- or 4-bit arithmetic decode
              constexpr int B = (BITS == 2 || BITS == 4) ? BITS : 4;
              constexpr int PER_WORD = 32 / B;
#pragma unroll
              for (int i = 0; i < PER_WORD; ++i)
                acc[w * PER_WORD + i] += sq_decode<BITS>((float)((word >> (B * i)) & ((1u << B) - 1u)), scale, emin, mean);
            }
          }
        }
      }
    }

    if (valid) {
      const float deg = end - begin == 0 ? 1.0f : (float)(end - begin);
      float* orow = p.out + d * p.feat_dim;
      if (p.reduce == F2C_MEAN) {
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[e] = acc[e] / deg;
      }
      if (p.vec_store) {
#pragma unroll
        for (int q = 0; q < EPL / 4; ++q) {
          int col = c0 + 4 * q;
          if (col < p.feat_dim) {  // feat_dim % 4 == 0 here
            float4 v = make_float4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
            if (p.drop.enabled) v = dropout_apply4(v, (uint64_t)(d * p.feat_dim + col), p.drop);
            stg_cs_f4(orow + col, v);
          }
        }
      } else {
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
          int col = c0 + e;
          if (col < p.feat_dim) {
            float v = acc[e];
            if (p.drop.enabled) v = dropout_apply1(v, (uint64_t)(d * p.feat_dim + col), p.drop);
            orow[col] = v;
          }
        }
      }
    }
  }
}

// Fallback for any shape / codebook layout: one warp per destination row, lane j walks code
// positions j, j+32, ... and keeps the (at most 8) columns of its current byte in registers.
template <int BITS, typename CodeT, typename IdxT>
__global__ void __launch_bounds__(256) sq_spmm_generic_kernel(const void* __restrict__ codes, const float* __restrict__ codebooks,
                                                              const IdxT* __restrict__ indptr, const IdxT* __restrict__ indices,
                                                              float* __restrict__ out, int64_t n_dst, int64_t src_dim, int feat_dim,
                                                              int column_slice, int reduce, DropoutArgs drop) {
  constexpr int PER = BITS >= 8 ? 1 : 8 / BITS;
  constexpr int B = BITS >= 8 ? 8 : BITS;
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int n_pos = (feat_dim + PER - 1) / PER;  // code positions that hold wanted columns
  for (int64_t d = warp; d < n_dst; d += n_warps) {
    const int64_t begin = (int64_t)indptr[d], end = (int64_t)indptr[d + 1];
    const float deg = end - begin == 0 ? 1.0f : (float)(end - begin);
    for (int j = lane; j < n_pos; j += 32) {
      float scale[PER], emin[PER], mean[PER], acc[PER];
#pragma unroll
      for (int e = 0; e < PER; ++e) {
        int col = j * PER + e;
        int row = (col < feat_dim ? col : feat_dim - 1) / column_slice;
        emin[e] = __ldg(codebooks + row * kCodebookDim + 2);
        float emax = __ldg(codebooks + row * kCodebookDim + 3);
        mean[e] = __ldg(codebooks + row * kCodebookDim + 4);
        scale[e] = sq_scale<BITS>(emin[e], emax);
        acc[e] = 0.0f;
      }
      for (int64_t k = begin; k < end; ++k) {
        int64_t src = (int64_t)indices[k];
        if (BITS >= 8) {
          float c = (float)reinterpret_cast<const CodeT*>(codes)[src * src_dim + j];
          acc[0] += sq_decode<BITS>(c, scale[0], emin[0], mean[0]);
        } else {
          uint32_t byte = reinterpret_cast<const uint8_t*>(codes)[src * src_dim + j];
#pragma unroll
          for (int e = 0; e < PER; ++e)
            acc[e] += sq_decode<BITS>((float)((byte >> (B * e)) & ((1u << B) - 1u)), scale[e], emin[e], mean[e]);
        }
      }
#pragma unroll
      for (int e = 0; e < PER; ++e) {
        int col = j * PER + e;
        if (col < feat_dim) {
          float v = reduce == F2C_MEAN ? acc[e] / deg : acc[e];
          if (drop.enabled) v = dropout_apply1(v, (uint64_t)(d * feat_dim + col), drop);
          out[d * feat_dim + col] = v;
        }
      }
    }
  }
}

static int ilog2(int v) { int l = 0; while ((1 << l) < v) ++l; return l; }

template <int BITS, int VEC, int U, typename IdxT, int DEC>
static int launch_fast(const SqParams& p, cudaStream_t st) {
  auto kern = sq_spmm_kernel<BITS, VEC, U, IdxT, DEC>;
  size_t smem = DEC == DEC_LUT ? 32768 : 0;  // below the 48 KB that needs no opt-in
  int rows_per_cta = 8 * (32 >> p.logG);
  int ctas_per_sm = g_tune_ctas_per_sm > 0 ? g_tune_ctas_per_sm : 4;
  int64_t grid = ceil_div(p.n_dst, rows_per_cta);
  if (grid > (int64_t)kSmCount * ctas_per_sm) grid = (int64_t)kSmCount * ctas_per_sm;
  kern<<<(unsigned)grid, 256, smem, st>>>(p);
  return check_launch("sq_decompress_spmm_csr");
}

template <int BITS, int VEC, typename IdxT, int DEC>
static int pick_u(const SqParams& p, cudaStream_t st) {
  int u = g_tune_u > 0 ? g_tune_u : 4;
  if (u >= 8) return launch_fast<BITS, VEC, 8, IdxT, DEC>(p, st);
  return launch_fast<BITS, VEC, 4, IdxT, DEC>(p, st);
}

template <int BITS, typename IdxT>
static int dispatch_fast(const SqParams& p, int vec, bool lut, cudaStream_t st) {
  constexpr int VMAX = BITS == 1 ? 4 : BITS == 2 ? 8 : 16;  // keeps EPL <= 32 accumulators
  constexpr bool CAN_LUT = BITS == 2 || BITS == 4 || BITS == 8;
  if (vec > VMAX) vec = VMAX;
  if constexpr (CAN_LUT) if (lut) {
    if (vec == 16) return pick_u<BITS, VMAX >= 16 ? 16 : VMAX, IdxT, DEC_LUT>(p, st);
    if (vec == 8) return pick_u<BITS, VMAX >= 8 ? 8 : VMAX, IdxT, DEC_LUT>(p, st);
    return pick_u<BITS, 4, IdxT, DEC_LUT>(p, st);
  }
  if (vec == 16) return pick_u<BITS, VMAX >= 16 ? 16 : VMAX, IdxT, DEC_ARITH>(p, st);
  if (vec == 8) return pick_u<BITS, VMAX >= 8 ? 8 : VMAX, IdxT, DEC_ARITH>(p, st);
  return pick_u<BITS, 4, IdxT, DEC_ARITH>(p, st);
}

template <int BITS, typename IdxT>
static int launch_sq_spmm(const void* codes, int code_dtype, const float* codebooks, int64_t n_cb, const void* indptr,
                          const void* indices, float* out, int64_t n_dst, int64_t src_dim, int64_t D, int64_t cs, int reduce,
                          const DropoutArgs& drop, cudaStream_t st) {
  if (n_dst == 0 || D == 0) return F2C_OK;
  const int code_bytes = dtype_size(code_dtype);
  const int64_t row_bytes = src_dim * code_bytes;
  // ---- can the vector kernel serve this shape? ----
  constexpr int VMAX = BITS == 1 ? 4 : BITS == 2 ? 8 : 16;
  int vec = 0;
  for (int v = VMAX; v >= 4; v >>= 1)
    if (row_bytes % v == 0 && aligned(codes, v) && row_bytes <= 32 * v) { vec = v; break; }
  if (g_tune_vec > 0 && vec > g_tune_vec && row_bytes <= 32 * g_tune_vec) vec = g_tune_vec;
  bool natural_dtype = BITS < 8 || (BITS == 8 && code_bytes == 1) || (BITS == 16 && code_bytes == 2);
  bool fast = vec != 0 && natural_dtype;
  int epl = 0, G = 0;
  if (fast) {
    epl = BITS == 16 ? vec / 2 : vec * 8 / BITS;
    G = 1 << ilog2((int)ceil_div(row_bytes, vec));
    // every lane's columns must share one codebook row
    fast = n_cb == 1 || cs % epl == 0;
  }
  if (fast) {
    SqParams p;
    p.codes = (const uint8_t*)codes; p.codebooks = codebooks; p.indptr = indptr; p.indices = indices; p.out = out;
    p.n_dst = n_dst; p.row_bytes = row_bytes; p.feat_dim = (int)D; p.column_slice = (int)cs; p.n_cb = (int)n_cb;
    p.logG = ilog2(G); p.code_kind = code_dtype == F2C_I8 ? CODE_I8 : code_dtype == F2C_U8 ? CODE_U8 : CODE_I16;
    p.reduce = reduce; p.vec_store = D % 4 == 0 && aligned(out, 16); p.drop = drop;
    // table copies are shared by lanes l and l + COPIES: they must own the same columns
    int copies = BITS == 8 ? 32 : BITS == 4 ? 16 : 8;
    bool lut = (n_cb == 1 || copies % G == 0) && g_tune_lut != 0;
    return dispatch_fast<BITS, IdxT>(p, vec, lut, st);
  }
  int64_t blocks = ceil_div(n_dst, 8);
  if (blocks > kSmCount * 32) blocks = kSmCount * 32;
#define F2C_GEN(T) sq_spmm_generic_kernel<BITS, T, IdxT><<<(unsigned)blocks, 256, 0, st>>>( \
      codes, codebooks, (const IdxT*)indptr, (const IdxT*)indices, out, n_dst, src_dim, (int)D, (int)cs, reduce, drop)
  if (code_dtype == F2C_I8) F2C_GEN(int8_t);
  else if (code_dtype == F2C_U8) F2C_GEN(uint8_t);
  else F2C_GEN(int16_t);
#undef F2C_GEN
  return check_launch("sq_decompress_spmm_csr");
}

}  // namespace f2c

using namespace f2c;

extern "C" int f2c_sq_spmm_csr(const void* codes, int code_dtype, const float* codebooks, int64_t n_codebooks,
                               const void* indptr, const void* indices, int index_dtype, float* out, int64_t n_dst,
                               int64_t src_dim, int64_t feat_dim, int bits, int64_t column_slice, int reduce,
                               const f2c_epilogue* epilogue, void* stream) {
  const char* op = "sq_decompress_spmm_csr";
  F2C_REQUIRE(n_dst >= 0, F2C_ERR_INVALID, "%s: negative size", op);
  int rc = validate_sq(op, code_dtype, n_codebooks, src_dim, feat_dim, bits, column_slice);
  if (rc) return rc;
  F2C_REQUIRE(is_index_dtype(index_dtype), F2C_ERR_UNSUPPORTED, "%s: indptr/indices must be int32 or int64", op);
  F2C_REQUIRE(reduce == F2C_MEAN || reduce == F2C_SUM, F2C_ERR_INVALID, "%s: reduce must be mean or sum", op);
  // The reference takes a packed byte's codebook row from its first element (src/fusion_spmm.cu:180);
  // that only equals the per-element rule of sq_decompress when a byte never straddles two rows.
  F2C_REQUIRE(bits >= 8 || n_codebooks == 1 || column_slice % (8 / bits) == 0, F2C_ERR_INVALID,
              "%s: column_slice (%lld) must be a multiple of %d for %d-bit codes", op, (long long)column_slice, 8 / bits, bits);
  F2C_REQUIRE(n_dst * feat_dim == 0 || (indptr && out && codebooks), F2C_ERR_INVALID, "%s: null pointer", op);
  DropoutArgs drop = make_dropout(epilogue);
  cudaStream_t st = (cudaStream_t)stream;
#define F2C_SQ(B)                                                                                                   \
  return index_dtype == F2C_I32                                                                                     \
             ? launch_sq_spmm<B, int32_t>(codes, code_dtype, codebooks, n_codebooks, indptr, indices, out, n_dst,   \
                                          src_dim, feat_dim, column_slice, reduce, drop, st)                       \
             : launch_sq_spmm<B, int64_t>(codes, code_dtype, codebooks, n_codebooks, indptr, indices, out, n_dst,   \
                                          src_dim, feat_dim, column_slice, reduce, drop, st)
  switch (bits) {
    case 1: F2C_SQ(1);
    case 2: F2C_SQ(2);
    case 4: F2C_SQ(4);
    case 8: F2C_SQ(8);
    default: F2C_SQ(16);
  }
#undef F2C_SQ
}

// Experiment knobs for the fused kernels (no counterpart in the reference).  key: 0 = bytes per lane
// per row load, 1 = rows in flight, 2 = table decode on/off, 3 = CTAs per SM.  value 0 (or -1 for
// key 2) restores the heuristic.
extern "C" int f2c_set_tuning(int key, int value) {
  switch (key) {
    case 0: g_tune_vec = value; break;
    case 1: g_tune_u = value; break;
    case 2: g_tune_lut = value; break;
    case 3: g_tune_ctas_per_sm = value; break;
    default: return set_error(F2C_ERR_INVALID, "set_tuning: unknown key %d", key);
  }
  return F2C_OK;
}
