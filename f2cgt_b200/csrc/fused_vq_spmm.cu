// Fused VQ decode + mean/sum aggregation (reference operator vq_decompress_spmm_csr,
// src/fusion_spmm.cu:72-141) and the single-launch two-level SQ+VQ aggregation.
//
//   out[d, j] = (sum_{k in N(d)} codebooks[s][codes[indices[k], s]][j - s*cs]) / max(deg(d), 1),  s = j / cs
//
// A VQ row is only n_codebooks code bytes (4..16 B), so HBM traffic per edge is tiny and the kernel
// lives on the on-chip gather: every edge pulls feat_dim floats out of the codebooks.  The codebooks
// (n_cb * K * cs * 4 bytes, 128 KB for 16x256x8 or 4x256x32) are therefore staged once per CTA in
// shared memory by a persistent grid; when they exceed one SM's shared memory the feature columns
// are split across blockIdx.y so that each CTA stages only the codebooks of its own column range,
// and a single codebook too large for that is served through the read-only L1/L2 path instead.
//
// One warp owns one destination row; a lane owns four consecutive columns of each 128-column tile
// (one LDS.128 from the centroid its code selects).  Neighbour indices are fetched 32 at a time and
// broadcast by shuffle; eight code loads / centroid reads are in flight per lane.  Accumulation is
// sequential in CSC order in fp32 registers (bit-identical to decode-then-aggregate).
//
// Two-level mode: slot[src] >= 0 redirects the edge to row slot[src] of the SQ table, whose bytes
// for the lane's four columns are decoded with the element-wise SQ expression; the branch is
// uniform across the warp because all lanes work on the same edge.
#include "common.cuh"
#include "vq_params.cuh"

namespace f2c {

int validate_vq(const char* op, int code_dtype, int64_t n_cb, int64_t length, int64_t cs, int64_t feat_dim);
int validate_sq(const char* op, int code_dtype, int64_t n_codebooks, int64_t src_dim, int64_t feat_dim, int bits,
                int64_t column_slice);

constexpr int kVqThreads = 1024;  // one CTA per SM: the staged codebooks leave room for one
constexpr size_t kVqSmemBudget = 200 * 1024;  // per CTA, leaves room for the static part and L1


__device__ __forceinline__ uint32_t vq_code(const void* codes, int kind, int64_t pos, uint32_t K) {
  int v;
  if (kind == 0) v = reinterpret_cast<const uint8_t*>(codes)[pos];
  else if (kind == 1) v = reinterpret_cast<const int8_t*>(codes)[pos];
  else v = reinterpret_cast<const int16_t*>(codes)[pos];
  uint32_t u = (uint32_t)v;
  return u < K ? u : K - 1;
}

// Decode the four SQ elements of columns [col, col+4) of one hot row.
template <int BITS>
__device__ __forceinline__ float4 sq_decode4(const uint8_t* __restrict__ row, int col, int is_signed, float scale, float emin,
                                             float mean) {
  float c[4];
  if (BITS == 16) {
    uint2 raw = ldg_nc_u64(row + 2 * col);
    c[0] = (float)(int16_t)(raw.x & 0xFFFFu); c[1] = (float)(int16_t)(raw.x >> 16);
    c[2] = (float)(int16_t)(raw.y & 0xFFFFu); c[3] = (float)(int16_t)(raw.y >> 16);
  } else if (BITS == 8) {
    uint32_t raw = ldg_nc_u32(row + col);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      uint32_t b = (raw >> (8 * e)) & 0xFFu;
      c[e] = is_signed ? (float)(int8_t)b : (float)b;
    }
  } else {
    constexpr int B = BITS >= 8 ? 4 : BITS;
    uint32_t raw;
    if (B == 4) raw = __ldg(reinterpret_cast<const uint16_t*>(row + col / 2));
    else if (B == 2) raw = __ldg(row + col / 4);
    else raw = (uint32_t)__ldg(row + col / 8) >> (col & 7);
#pragma unroll
    for (int e = 0; e < 4; ++e) c[e] = (float)((raw >> (B * e)) & ((1u << B) - 1u));
  }
  return make_float4(sq_decode<BITS>(c[0], scale, emin, mean), sq_decode<BITS>(c[1], scale, emin, mean),
                     sq_decode<BITS>(c[2], scale, emin, mean), sq_decode<BITS>(c[3], scale, emin, mean));
}

// HB = 0: pure VQ.  HB in {1,2,4,8,16}: two-level, SQ width HB.
template <int HB, typename IdxT, bool CB_SMEM>
__global__ void __launch_bounds__(kVqThreads) vq_spmm_kernel(const VqParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* cb_s = reinterpret_cast<float*>(smem_raw);
  const int part = blockIdx.y;
  const int s_begin = part * p.cb_per_part;
  const int s_end = min(s_begin + p.cb_per_part, p.n_cb);
  const int col_begin = s_begin * p.cs;
  const int col_end = min(s_end * p.cs, p.feat_dim);
  const float* __restrict__ cb_g = p.codebooks + (int64_t)s_begin * p.K * p.cs;
  if (CB_SMEM) {
    const int n4 = (s_end - s_begin) * (int)p.K * p.cs / 4;
    const float4* src = reinterpret_cast<const float4*>(cb_g);
    float4* dst = reinterpret_cast<float4*>(cb_s);
    for (int i = threadIdx.x; i < n4; i += blockDim.x) dst[i] = __ldg(src + i);
    __syncthreads();
  }
  const float* cb = CB_SMEM ? cb_s : cb_g;

  const IdxT* __restrict__ indptr = reinterpret_cast<const IdxT*>(p.indptr);
  const IdxT* __restrict__ indices = reinterpret_cast<const IdxT*>(p.indices);
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  constexpr int U = 8;

  for (int64_t d = warp; d < p.n_dst; d += n_warps) {
    const int64_t begin = (int64_t)indptr[d], end = (int64_t)indptr[d + 1];
    const float deg = end - begin == 0 ? 1.0f : (float)(end - begin);
    for (int col0 = col_begin; col0 < col_end; col0 += 128) {
      const int col = col0 + lane * 4;
      const bool active = col < col_end;
      const int s = active ? col / p.cs : s_begin;
      const int off = active ? col - s * p.cs : 0;
      const float* cb_lane = cb + ((int64_t)(s - s_begin) * p.K) * p.cs + off;
      float sq_scale_v = 0.f, sq_emin = 0.f, sq_mean = 0.f;
      if (HB != 0) {
        int row = (active ? col : col_begin) / p.sq_cs;
        if (row >= p.sq_n_cb) row = p.sq_n_cb - 1;
        sq_emin = __ldg(p.sq_codebooks + row * kCodebookDim + 2);
        float emax = __ldg(p.sq_codebooks + row * kCodebookDim + 3);
        sq_mean = __ldg(p.sq_codebooks + row * kCodebookDim + 4);
        sq_scale_v = sq_scale<HB == 0 ? 8 : HB>(sq_emin, emax);
      }
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int64_t k0 = begin; k0 < end; k0 += 32) {
        const int cnt = (int)(end - k0 < 32 ? end - k0 : 32);
        int64_t mine = lane < cnt ? (int64_t)indices[k0 + lane] : 0;
        int myslot = -1;
        if (HB != 0 && lane < cnt) myslot = hot_slot_of(p, (int64_t)mine);
        for (int t0 = 0; t0 < cnt; t0 += U) {
          float4 v[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int t = t0 + u;
            int64_t src = __shfl_sync(0xffffffffu, mine, t & 31);
            int sl = HB != 0 ? __shfl_sync(0xffffffffu, myslot, t & 31) : -1;
            v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < cnt && active) {
              if (HB != 0 && sl >= 0) {
                v[u] = sq_decode4<HB == 0 ? 8 : HB>(p.sq_codes + (int64_t)sl * p.sq_row_bytes, col, p.sq_signed, sq_scale_v,
                                                    sq_emin, sq_mean);
              } else {
                uint32_t code = vq_code(p.codes, p.code_kind, src * p.n_cb + s, p.K);
                const float4* c4 = reinterpret_cast<const float4*>(cb_lane + (int64_t)code * p.cs);
                v[u] = CB_SMEM ? *c4 : __ldg(c4);
              }
            }
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            if (t0 + u < cnt) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
          }
        }
      }
      if (active) {
        if (p.reduce == F2C_MEAN) { acc.x = acc.x / deg; acc.y = acc.y / deg; acc.z = acc.z / deg; acc.w = acc.w / deg; }
        float* o = p.out + d * p.feat_dim + col;
        if (p.vec_store) {
          if (p.drop.enabled) acc = dropout_apply4(acc, (uint64_t)(d * p.feat_dim + col), p.drop);
          stg_cs_f4(o, acc);
        } else {
          float a[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (col + e < col_end) {
              float x = a[e];
              if (p.drop.enabled) x = dropout_apply1(x, (uint64_t)(d * p.feat_dim + col + e), p.drop);
              o[e] = x;
            }
        }
      }
    }
  }
}

// Any shape (column_slice or feat_dim not a multiple of four, ...): lane j owns single columns
// j, j+32, ...; codebooks through the read-only cache.
template <typename IdxT>
__global__ void __launch_bounds__(256) vq_spmm_generic_kernel(const VqParams p) {
  const IdxT* __restrict__ indptr = reinterpret_cast<const IdxT*>(p.indptr);
  const IdxT* __restrict__ indices = reinterpret_cast<const IdxT*>(p.indices);
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t d = warp; d < p.n_dst; d += n_warps) {
    const int64_t begin = (int64_t)indptr[d], end = (int64_t)indptr[d + 1];
    const float deg = end - begin == 0 ? 1.0f : (float)(end - begin);
    for (int j = lane; j < p.feat_dim; j += 32) {
      const int s = j / p.cs, off = j - s * p.cs;
      float acc = 0.0f;
      for (int64_t k = begin; k < end; ++k) {
        int64_t src = (int64_t)indices[k];
        uint32_t code = vq_code(p.codes, p.code_kind, src * p.n_cb + s, p.K);
        acc += __ldg(p.codebooks + ((int64_t)s * p.K + code) * p.cs + off);
      }
      float v = p.reduce == F2C_MEAN ? acc / deg : acc;
      if (p.drop.enabled) v = dropout_apply1(v, (uint64_t)(d * p.feat_dim + j), p.drop);
      p.out[d * p.feat_dim + j] = v;
    }
  }
}

template <int HB, typename IdxT>
static int launch_vq(VqParams& p, cudaStream_t st, const char* op) {
  // split the subspaces over blockIdx.y until one part's codebooks fit in shared memory
  size_t one_cb = (size_t)p.K * p.cs * sizeof(float);
  bool use_smem = one_cb <= kVqSmemBudget;
  int parts = 1;
  if (use_smem) {
    while (ceil_div(p.n_cb, parts) * one_cb > kVqSmemBudget) ++parts;
    // a part must own whole 128-column tiles unless it is the only one (keeps lanes' float4 inside one part)
    p.cb_per_part = (int)ceil_div(p.n_cb, parts);
    parts = (int)ceil_div(p.n_cb, p.cb_per_part);
  } else {
    p.cb_per_part = p.n_cb;
  }
  size_t smem = use_smem ? (size_t)p.cb_per_part * one_cb : 0;
  int64_t rows_per_cta = kVqThreads / 32;
  int64_t grid_x = ceil_div(p.n_dst, rows_per_cta);
  int ctas_per_sm = 1;  // 1024 threads at <= 64 registers fill the register file
  int64_t cap = (int64_t)current_sm_count() * ctas_per_sm / parts;
  if (cap < 1) cap = 1;
  if (grid_x > cap) grid_x = cap;
  dim3 grid((unsigned)grid_x, (unsigned)parts);
  if (use_smem) {
    auto kern = vq_spmm_kernel<HB, IdxT, true>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "%s: %s", op, cudaGetErrorString(e));
    kern<<<grid, kVqThreads, smem, st>>>(p);
  } else {
    vq_spmm_kernel<HB, IdxT, false><<<grid, kVqThreads, 0, st>>>(p);
  }
  return check_launch(op);
}

}  // namespace f2c

using namespace f2c;

extern "C" int f2c_vq_spmm_csr(const void* codes, int code_dtype, const float* codebooks, const void* indptr,
                               const void* indices, int index_dtype, float* out, int64_t n_dst, int64_t n_codebooks,
                               int64_t length, int64_t column_slice, int64_t feat_dim, int reduce,
                               const f2c_epilogue* epilogue, void* stream) {
  const char* op = "vq_decompress_spmm_csr";
  F2C_REQUIRE(n_dst >= 0, F2C_ERR_INVALID, "%s: negative size", op);
  int rc = validate_vq(op, code_dtype, n_codebooks, length, column_slice, feat_dim);
  if (rc) return rc;
  F2C_REQUIRE(is_index_dtype(index_dtype), F2C_ERR_UNSUPPORTED, "%s: indptr/indices must be int32 or int64", op);
  F2C_REQUIRE(reduce == F2C_MEAN || reduce == F2C_SUM, F2C_ERR_INVALID, "%s: reduce must be mean or sum", op);
  F2C_REQUIRE(n_dst * feat_dim == 0 || (indptr && out && codebooks), F2C_ERR_INVALID, "%s: null pointer", op);
  if (n_dst == 0 || feat_dim == 0) return F2C_OK;
  VqParams p{};
  p.codes = codes; p.codebooks = codebooks; p.indptr = indptr; p.indices = indices; p.out = out; p.n_dst = n_dst;
  p.n_cb = (int)n_codebooks; p.cs = (int)column_slice; p.feat_dim = (int)feat_dim; p.K = (uint32_t)length;
  p.code_kind = code_dtype == F2C_U8 ? 0 : code_dtype == F2C_I8 ? 1 : 2;
  p.reduce = reduce; p.vec_store = feat_dim % 4 == 0 && aligned(out, 16); p.drop = make_dropout(epilogue);
  cudaStream_t st = (cudaStream_t)stream;
  bool fast = column_slice % 4 == 0 && aligned(codebooks, 16);
  if (!fast) {
    int64_t blocks = ceil_div(n_dst, 8);
    if (blocks > current_sm_count() * 32) blocks = current_sm_count() * 32;
    if (index_dtype == F2C_I32) vq_spmm_generic_kernel<int32_t><<<(unsigned)blocks, 256, 0, st>>>(p);
    else vq_spmm_generic_kernel<int64_t><<<(unsigned)blocks, 256, 0, st>>>(p);
    return check_launch(op);
  }
  const int variant = kernel_variant(epilogue);
  bool served = false;
  if (variant != F2C_KERNEL_GENERAL) {
    rc = launch_vq_fast(p, 0, index_dtype, variant, st, op, &served);
    if (served || rc) return rc;
    if (variant != F2C_KERNEL_AUTO) return set_error(F2C_ERR_UNSUPPORTED, "%s: shape not served by the requested kernel family", op);
  }
  return index_dtype == F2C_I32 ? launch_vq<0, int32_t>(p, st, op) : launch_vq<0, int64_t>(p, st, op);
}

extern "C" int f2c_hybrid_spmm_csr(const void* sq_codes, int sq_dtype, const float* sq_codebooks, int64_t sq_n_codebooks,
                                   int bits, int64_t sq_column_slice, int64_t sq_src_dim, const void* vq_codes,
                                   int vq_dtype, const float* vq_codebooks, int64_t vq_n_codebooks, int64_t length,
                                   int64_t vq_column_slice, const int32_t* slot, int64_t n_hot, const void* indptr, const void* indices,
                                   int index_dtype, float* out, int64_t n_dst, int64_t feat_dim, int reduce,
                                   const f2c_epilogue* epilogue, void* stream) {
  const char* op = "two_level_decompress_spmm_csr";
  F2C_REQUIRE(n_dst >= 0, F2C_ERR_INVALID, "%s: negative size", op);
  int rc = validate_vq(op, vq_dtype, vq_n_codebooks, length, vq_column_slice, feat_dim);
  if (rc) return rc;
  rc = validate_sq(op, sq_dtype, sq_n_codebooks, sq_src_dim, feat_dim, bits, sq_column_slice);
  if (rc) return rc;
  F2C_REQUIRE(is_index_dtype(index_dtype), F2C_ERR_UNSUPPORTED, "%s: indptr/indices must be int32 or int64", op);
  F2C_REQUIRE(reduce == F2C_MEAN || reduce == F2C_SUM, F2C_ERR_INVALID, "%s: reduce must be mean or sum", op);
  F2C_REQUIRE(n_dst * feat_dim == 0 || (indptr && out && vq_codebooks && sq_codebooks && (slot || n_hot >= 0)), F2C_ERR_INVALID,
              "%s: null pointer", op);
  const int sq_bytes = dtype_size(sq_dtype);
  F2C_REQUIRE((bits == 16) == (sq_bytes == 2), F2C_ERR_UNSUPPORTED,
              "%s: SQ codes must be int16 for 16 bits and uint8/int8 otherwise", op);
  F2C_REQUIRE(feat_dim % 4 == 0 && vq_column_slice % 4 == 0 && (sq_n_codebooks == 1 || sq_column_slice % 4 == 0),
              F2C_ERR_UNSUPPORTED, "%s: feat_dim and both column_slice values must be multiples of 4", op);
  const int64_t sq_row_bytes = sq_src_dim * sq_bytes;
  const int row_align = bits == 16 ? 8 : bits == 8 ? 4 : bits == 4 ? 2 : 1;
  F2C_REQUIRE(sq_row_bytes % row_align == 0 && aligned(sq_codes, row_align) && aligned(vq_codebooks, 16) && aligned(out, 16),
              F2C_ERR_UNSUPPORTED, "%s: tables are not aligned for vector access", op);
  if (n_dst == 0 || feat_dim == 0) return F2C_OK;
  VqParams p{};
  p.codes = vq_codes; p.codebooks = vq_codebooks; p.indptr = indptr; p.indices = indices; p.out = out; p.n_dst = n_dst;
  p.n_cb = (int)vq_n_codebooks; p.cs = (int)vq_column_slice; p.feat_dim = (int)feat_dim; p.K = (uint32_t)length;
  p.code_kind = vq_dtype == F2C_U8 ? 0 : vq_dtype == F2C_I8 ? 1 : 2;
  p.reduce = reduce; p.vec_store = 1; p.drop = make_dropout(epilogue);
  p.sq_codes = (const uint8_t*)sq_codes; p.sq_codebooks = sq_codebooks; p.slot = slot; p.n_hot = n_hot; p.sq_row_bytes = sq_row_bytes;
  p.sq_cs = (int)sq_column_slice; p.sq_n_cb = (int)sq_n_codebooks; p.sq_signed = sq_dtype == F2C_I8;
  cudaStream_t st = (cudaStream_t)stream;
  const int variant = kernel_variant(epilogue);
  bool served = false;
  if (variant != F2C_KERNEL_GENERAL) {
    rc = launch_vq_fast(p, bits, index_dtype, variant, st, op, &served);
    if (served || rc) return rc;
    if (variant != F2C_KERNEL_AUTO) return set_error(F2C_ERR_UNSUPPORTED, "%s: shape not served by the requested kernel family", op);
  }
#define F2C_HY(B) \
  return index_dtype == F2C_I32 ? launch_vq<B, int32_t>(p, st, op) : launch_vq<B, int64_t>(p, st, op)
  switch (bits) {
    case 1: F2C_HY(1);
    case 2: F2C_HY(2);
    case 4: F2C_HY(4);
    case 8: F2C_HY(8);
    default: F2C_HY(16);
  }
#undef F2C_HY
}

// The two-level (or, without an SQ table, the plain VQ) aggregation over tables that are row-sharded across the GPUs of one
// NVSwitch box: every shard pointer must be dereferenceable from the current device (own memory or a mapping made with
// f2c_shard_open).  One kernel reads remote code rows, slots and hot rows itself over NVLink.
extern "C" int f2c_hybrid_spmm_csr_peer(const void* const* sq_shards_host, const void* const* vq_shards_host,
                                        const int32_t* const* slot_shards_host, int world, int64_t rows_per_shard,
                                        int64_t hot_rows_per_shard, int64_t n_rows, int64_t n_hot, int sq_dtype,
                                        const float* sq_codebooks, int64_t sq_n_codebooks, int bits, int64_t sq_column_slice,
                                        int64_t sq_src_dim, int vq_dtype, const float* vq_codebooks, int64_t vq_n_codebooks,
                                        int64_t length, int64_t vq_column_slice, const void* indptr, const void* indices,
                                        int index_dtype, float* out, int64_t n_dst, int64_t feat_dim, int reduce,
                                        const f2c_epilogue* epilogue, void* stream) {
  const char* op = "two_level_decompress_spmm_csr_peer";
  const bool two_level = sq_shards_host != nullptr;
  F2C_REQUIRE(n_dst >= 0 && n_rows >= 0 && n_hot >= 0, F2C_ERR_INVALID, "%s: negative size", op);
  F2C_REQUIRE(world >= 1 && world <= 8, F2C_ERR_LIMIT, "%s: 1 to 8 shards (got %d)", op, world);
  F2C_REQUIRE(vq_shards_host != nullptr, F2C_ERR_INVALID, "%s: null pointer", op);
  F2C_REQUIRE(rows_per_shard >= 2 && rows_per_shard < (1ll << 32) && rows_per_shard * world >= n_rows, F2C_ERR_INVALID,
              "%s: %d shards of %lld rows do not cover %lld rows", op, world, (long long)rows_per_shard, (long long)n_rows);
  int rc = validate_vq(op, vq_dtype, vq_n_codebooks, length, vq_column_slice, feat_dim);
  if (rc) return rc;
  F2C_REQUIRE(is_index_dtype(index_dtype), F2C_ERR_UNSUPPORTED, "%s: indptr/indices must be int32 or int64", op);
  F2C_REQUIRE(reduce == F2C_MEAN || reduce == F2C_SUM, F2C_ERR_INVALID, "%s: reduce must be mean or sum", op);
  F2C_REQUIRE(n_dst * feat_dim == 0 || (indptr && out && vq_codebooks), F2C_ERR_INVALID, "%s: null pointer", op);
  VqParams p{};
  int64_t sq_row_bytes = 0;
  if (two_level) {
    rc = validate_sq(op, sq_dtype, sq_n_codebooks, sq_src_dim, feat_dim, bits, sq_column_slice);
    if (rc) return rc;
    F2C_REQUIRE(sq_codebooks != nullptr, F2C_ERR_INVALID, "%s: null pointer", op);
    F2C_REQUIRE(hot_rows_per_shard >= 2 && hot_rows_per_shard < (1ll << 32) && hot_rows_per_shard * world >= n_hot, F2C_ERR_INVALID,
                "%s: %d shards of %lld hot rows do not cover %lld", op, world, (long long)hot_rows_per_shard, (long long)n_hot);
    F2C_REQUIRE(feat_dim % 4 == 0 && vq_column_slice % 4 == 0 && (sq_n_codebooks == 1 || sq_column_slice % 4 == 0),
                F2C_ERR_UNSUPPORTED, "%s: feat_dim and both column_slice values must be multiples of 4", op);
    sq_row_bytes = sq_src_dim * dtype_size(sq_dtype);
  }
  if (n_dst == 0 || feat_dim == 0) return F2C_OK;
  for (int r = 0; r < world; ++r) {
    rc = ensure_readable_from_current_device(vq_shards_host[r], op, "VQ", r);
    if (rc) return rc;
    p.peer.code[r] = (const uint8_t*)vq_shards_host[r];
    if (two_level) {
      rc = ensure_readable_from_current_device(sq_shards_host[r], op, "SQ", r);
      if (rc) return rc;
      p.peer.hot[r] = (const uint8_t*)sq_shards_host[r];
      if (slot_shards_host != nullptr) {
        rc = ensure_readable_from_current_device(slot_shards_host[r], op, "slot", r);
        if (rc) return rc;
        p.peer.slot[r] = slot_shards_host[r];
      }
    }
  }
  for (int r = world; r < 8; ++r) { p.peer.code[r] = p.peer.code[0]; p.peer.hot[r] = p.peer.hot[0]; p.peer.slot[r] = p.peer.slot[0]; }
  p.peer.rps_nodes = (uint32_t)rows_per_shard;
  p.peer.magic_nodes = ~0ull / (unsigned long long)rows_per_shard + 1ull;
  p.peer.rps_hot = (uint32_t)(two_level ? hot_rows_per_shard : 2);
  p.peer.magic_hot = ~0ull / (unsigned long long)p.peer.rps_hot + 1ull;
  p.codes = p.peer.code[0]; p.codebooks = vq_codebooks; p.indptr = indptr; p.indices = indices; p.out = out; p.n_dst = n_dst;
  p.n_cb = (int)vq_n_codebooks; p.cs = (int)vq_column_slice; p.feat_dim = (int)feat_dim; p.K = (uint32_t)length;
  p.code_kind = vq_dtype == F2C_U8 ? 0 : vq_dtype == F2C_I8 ? 1 : 2;
  p.reduce = reduce; p.vec_store = 1; p.drop = make_dropout(epilogue);
  p.sq_codes = p.peer.hot[0]; p.sq_codebooks = sq_codebooks; p.slot = nullptr; p.n_hot = n_hot; p.sq_row_bytes = sq_row_bytes;
  p.sq_cs = (int)sq_column_slice; p.sq_n_cb = (int)sq_n_codebooks; p.sq_signed = sq_dtype == F2C_I8;
  bool served = false;
  rc = launch_vq_fast(p, two_level ? bits : 0, index_dtype, F2C_KERNEL_PREFETCH, (cudaStream_t)stream, op, &served, true);
  if (served || rc) return rc;
  return set_error(F2C_ERR_UNSUPPORTED, "%s: shape not served by the sharded kernel (uint8 codes, 4/8/16 code bytes per row, "
                                        "column_slice dividing 128, hot rows 8- or 4-bit)", op);
}
