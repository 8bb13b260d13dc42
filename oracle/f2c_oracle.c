/* TEST INFRASTRUCTURE ONLY - a CPU restatement of the arithmetic of gpzlx1/F2CGT's
 * compressed-feature hot path, used as the checker in tests/, in the smoke test and as the timed
 * CPU leg of the benchmark.  Nothing in the product package links, loads or calls this file.
 *
 * Every function cites the reference source (path inside the F2CGT project) it follows.  The code
 * is written from the reference's semantics, loop by loop in plain C; rows are independent, so the
 * outer row loops carry an OpenMP pragma, which never changes a result (each output element is
 * still produced by one thread in the reference's order).
 *
 * Parity pinning: the golden fixtures under tests/golden/ were produced by the reference's own CUDA
 * kernels on a B200 (oracle/build_ref.py + tests/golden/make_golden.py); tests/test_oracle_golden.py
 * holds this file to them - bit-exact for all integer/gather work and for the aggregation order,
 * and within 2 ulp for values that pass through exp2f/log2f, where the GPU's libdevice and the
 * host's libm legitimately differ in the last bits.
 *
 * Floating point: the reference is device code compiled with nvcc defaults, i.e. a*b+c contracts
 * to one fused multiply-add; the restatement therefore calls fmaf() where the reference writes
 * "x * s + e", and this file must be compiled with -ffp-contract=off so that nothing else fuses.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define CB_DIM 5 /* codebook row = [fmin, fmax, emin, emax, mean]  (src/sq_quantization.cu:17,36) */

/* ---- dtype tags shared with the tests (same numbering as include/f2cgt_b200.h) ---- */
enum { DT_U8 = 0, DT_I8 = 1, DT_I16 = 2, DT_I32 = 3, DT_I64 = 4, DT_F16 = 5, DT_F32 = 6, DT_F64 = 7 };

static inline int64_t load_idx(const void* p, int dt, int64_t i) {
  switch (dt) {
    case DT_U8: return ((const uint8_t*)p)[i];
    case DT_I8: return ((const int8_t*)p)[i];
    case DT_I16: return ((const int16_t*)p)[i];
    case DT_I32: return ((const int32_t*)p)[i];
    default: return ((const int64_t*)p)[i];
  }
}

/* ------------------------------------------------------------------------------------------
 * packbits: src/packbits.cu:24-41.  One output byte = OR of up to 8/bits input bytes, element i
 * of the byte at bit offset bits*i ("small end", :37-38); the last byte of a row may be ragged
 * (:30-32); pack_dim = ceil(unpack_dim / (8/bits)) (:46-47).
 * ------------------------------------------------------------------------------------------ */
void orc_packbits(const uint8_t* unpack, uint8_t* pack, int64_t rows, int64_t unpack_dim, int bits) {
  const int numel = 8 / bits;
  const uint8_t mask = (uint8_t)((1u << bits) - 1u);
  const int64_t pack_dim = (unpack_dim + numel - 1) / numel;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t b = 0; b < pack_dim; ++b) {
      int64_t begin = b * numel;
      int64_t end = begin + numel < unpack_dim ? begin + numel : unpack_dim;
      uint8_t v = 0;
      for (int64_t i = begin; i < end; ++i)
        v |= (uint8_t)((unpack[r * unpack_dim + i] & mask) << (bits * (i - begin)));
      pack[r * pack_dim + b] = v;
    }
  }
}

/* unpackbits: src/packbits.cu:84-94 with unpackbits_func src/cuda_utils.cuh:5-9. */
void orc_unpackbits(const uint8_t* pack, uint8_t* unpack, int64_t rows, int64_t unpack_dim,
                    int64_t pack_dim, int bits) {
  const int numel = 8 / bits;
  const uint8_t mask = (uint8_t)((1u << bits) - 1u);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t j = 0; j < unpack_dim; ++j)
      unpack[r * unpack_dim + j] = (pack[r * pack_dim + j / numel] >> (bits * (j % numel))) & mask;
}

/* ------------------------------------------------------------------------------------------
 * sq_compress: src/sq_quantization.cu:34-59.  Output is float-valued codes (:67); the caller
 * casts.  1 bit: x<=0 ? 0 : 1.  Otherwise log2-domain sign-magnitude with "zero counts as
 * negative" (:50) and an unsigned bias for widths below 8 (:57).
 * ------------------------------------------------------------------------------------------ */
void orc_sq_compress(const float* src, float* dst, const float* cb, int64_t rows, int64_t D, int bits,
                     int64_t column_slice) {
  const float drange = (float)(1 << (bits - 1));
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t j = 0; j < D; ++j) {
      float x = src[r * D + j];
      if (bits == 1) { dst[r * D + j] = x <= 0 ? 0.0f : 1.0f; continue; }
      const float* row = cb + (j / column_slice) * CB_DIM;
      float fmin = row[0], fmax = row[1], emin = row[2], emax = row[3];
      int neg = x <= 0;
      float v = fabsf(x);
      v = fminf(fmaxf(v, fmin), fmax);
      v = log2f(v);
      v = (v - emin) / (emax - emin) * drange;
      v = floorf(v);
      v = neg ? -1.0f - v : v;
      if (bits < 8) v += drange;
      dst[r * D + j] = v;
    }
  }
}

/* The value just before floorf() in sq_compress - lets a test tell a genuine mismatch from an
 * element that sits on a quantisation boundary where log2f implementations may round apart. */
void orc_sq_compress_prefloor(const float* src, float* dst, const float* cb, int64_t rows, int64_t D,
                              int bits, int64_t column_slice) {
  const float drange = (float)(1 << (bits - 1));
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t j = 0; j < D; ++j) {
      const float* row = cb + (j / column_slice) * CB_DIM;
      float v = fminf(fmaxf(fabsf(src[r * D + j]), row[0]), row[1]);
      dst[r * D + j] = (log2f(v) - row[2]) / (row[3] - row[2]) * drange;
    }
}

/* One SQ element: src/sq_quantization.cu:137-152 (identical maths at src/fusion_spmm.cu:199-223).
 * c is the raw code as float (unsigned for packed widths). */
static inline float sq_decode_one(float c, int bits, float drange, float emin, float emax, float mean) {
  if (bits == 1) return (c - 0.5f) * (2.0f * mean);
  if (bits < 8) c -= drange;
  c = c + 0.5f;
  float sign = c >= 0 ? 1.0f : -1.0f;
  float e = fmaf(fabsf(c), (emax - emin) / drange, emin); /* nvcc contracts |c|*s+emin */
  return exp2f(e) * sign;
}

static inline float sq_code_at(const void* codes, int code_dt, int64_t row, int64_t src_dim, int64_t j,
                               int bits) {
  if (bits >= 8) { /* src/sq_quantization.cu:127-128: value = (float)src_ptr[j] in the tensor's dtype */
    if (code_dt == DT_I16) return (float)((const int16_t*)codes)[row * src_dim + j];
    if (code_dt == DT_I8) return (float)((const int8_t*)codes)[row * src_dim + j];
    return (float)((const uint8_t*)codes)[row * src_dim + j];
  }
  const int pack = 8 / bits; /* :130-135, bytes are raw whatever the tensor's dtype says */
  uint8_t byte = ((const uint8_t*)codes)[row * src_dim + j / pack];
  return (float)((byte >> (bits * (j % pack))) & ((1u << bits) - 1u));
}

/* sq_decompress: src/sq_quantization.cu:119-155; codebook row of element j is j/column_slice. */
void orc_sq_decompress(const void* codes, int code_dt, float* out, const float* cb, int64_t rows,
                       int64_t src_dim, int64_t D, int bits, int64_t column_slice) {
  const float drange = (float)(1 << (bits - 1));
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t j = 0; j < D; ++j) {
      const float* row = cb + (j / column_slice) * CB_DIM;
      out[r * D + j] = sq_decode_one(sq_code_at(codes, code_dt, r, src_dim, j, bits), bits, drange,
                                     row[2], row[3], row[4]);
    }
}

/* ------------------------------------------------------------------------------------------
 * vq_decompress: src/vq_quantization.cu:18-31.  out[i,j] = codebooks[s][codes[i,s]][j - s*cs],
 * s = j / cs; codebooks contiguous [n_cb, K, cs], fp32 or fp16 (cb_dt).
 * ------------------------------------------------------------------------------------------ */
static inline float vq_at(const void* codes, int code_dt, const void* cbs, int cb_dt, int64_t row,
                          int64_t n_cb, int64_t K, int64_t cs, int64_t j) {
  int64_t s = j / cs, off = j % cs;
  int64_t idx = load_idx(codes, code_dt, row * n_cb + s);
  int64_t pos = s * K * cs + idx * cs + off;
  if (cb_dt == DT_F16) return (float)((const _Float16*)cbs)[pos];
  return ((const float*)cbs)[pos];
}

void orc_vq_decompress(const void* codes, int code_dt, const void* cbs, int cb_dt, float* out,
                       int64_t rows, int64_t n_cb, int64_t K, int64_t cs, int64_t D) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t j = 0; j < D; ++j) out[r * D + j] = vq_at(codes, code_dt, cbs, cb_dt, r, n_cb, K, cs, j);
}

/* ------------------------------------------------------------------------------------------
 * Mean aggregation over a CSC block: src/fusion_spmm.cu:24-42.  deg==0 divides by 1 (:28);
 * accumulate from 0 in CSC order k = begin..end-1 (:33-36); one division at the end (:37).
 * reduce: 0 = mean (the reference), 1 = sum (extension: the division is skipped).
 * The accumulator has the feature dtype, as in the reference (DType local_accum, :32).
 * ------------------------------------------------------------------------------------------ */
void orc_spmm_csr_f32(const float* feat, float* out, const void* indptr, const void* indices, int idx_dt,
                      int64_t n_dst, int64_t D, int reduce) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t d = 0; d < n_dst; ++d) {
    int64_t b = load_idx(indptr, idx_dt, d), e = load_idx(indptr, idx_dt, d + 1);
    float deg = e - b == 0 ? 1.0f : (float)(e - b);
    for (int64_t j = 0; j < D; ++j) {
      float acc = 0.0f;
      for (int64_t k = b; k < e; ++k) acc += feat[load_idx(indices, idx_dt, k) * D + j];
      out[d * D + j] = reduce == 0 ? acc / deg : acc;
    }
  }
}

void orc_spmm_csr_f64(const double* feat, double* out, const void* indptr, const void* indices,
                      int idx_dt, int64_t n_dst, int64_t D, int reduce) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t d = 0; d < n_dst; ++d) {
    int64_t b = load_idx(indptr, idx_dt, d), e = load_idx(indptr, idx_dt, d + 1);
    float deg = e - b == 0 ? 1.0f : (float)(e - b); /* "float deg" even for doubles (:28) */
    for (int64_t j = 0; j < D; ++j) {
      double acc = 0.0;
      for (int64_t k = b; k < e; ++k) acc += feat[load_idx(indices, idx_dt, k) * D + j];
      out[d * D + j] = reduce == 0 ? acc / deg : acc;
    }
  }
}

/* fp16 features: at::Half accumulates by converting to float, adding, and rounding back to half
 * at every step; the final division is half/float -> float -> half. */
void orc_spmm_csr_f16(const _Float16* feat, _Float16* out, const void* indptr, const void* indices,
                      int idx_dt, int64_t n_dst, int64_t D, int reduce) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t d = 0; d < n_dst; ++d) {
    int64_t b = load_idx(indptr, idx_dt, d), e = load_idx(indptr, idx_dt, d + 1);
    float deg = e - b == 0 ? 1.0f : (float)(e - b);
    for (int64_t j = 0; j < D; ++j) {
      _Float16 acc = (_Float16)0.0f;
      for (int64_t k = b; k < e; ++k)
        acc = (_Float16)((float)acc + (float)feat[load_idx(indices, idx_dt, k) * D + j]);
      out[d * D + j] = reduce == 0 ? (_Float16)((float)acc / deg) : acc;
    }
  }
}

/* ------------------------------------------------------------------------------------------
 * Fused SQ decode + mean: src/fusion_spmm.cu:173-236.  Same value as decode-then-aggregate.  The
 * reference takes the codebook row of a packed byte from its first element, j*pack/column_slice
 * (:180); callers keep column_slice a multiple of 8/bits, where that equals j/column_slice.
 * fp64 variant (acc64 != 0) accumulates the same decoded fp32 values in double - used to bound
 * the error of any summation order.
 * ------------------------------------------------------------------------------------------ */
void orc_sq_spmm_csr(const void* codes, int code_dt, const float* cb, const void* indptr,
                     const void* indices, int idx_dt, float* out, int64_t n_dst, int64_t src_dim,
                     int64_t D, int bits, int64_t column_slice, int reduce, int acc64) {
  const float drange = (float)(1 << (bits - 1));
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t d = 0; d < n_dst; ++d) {
    int64_t b = load_idx(indptr, idx_dt, d), e = load_idx(indptr, idx_dt, d + 1);
    float deg = e - b == 0 ? 1.0f : (float)(e - b);
    for (int64_t j = 0; j < D; ++j) {
      const float* row = cb + (j / column_slice) * CB_DIM;
      float acc = 0.0f;
      double acc_d = 0.0;
      for (int64_t k = b; k < e; ++k) {
        int64_t s = load_idx(indices, idx_dt, k);
        float v = sq_decode_one(sq_code_at(codes, code_dt, s, src_dim, j, bits), bits, drange, row[2],
                                row[3], row[4]);
        acc += v;
        acc_d += v;
      }
      if (acc64) out[d * D + j] = (float)(reduce == 0 ? acc_d / deg : acc_d);
      else out[d * D + j] = reduce == 0 ? acc / deg : acc;
    }
  }
}

/* Fused VQ decode + mean: src/fusion_spmm.cu:83-104 with vq_decompress_func src/cuda_utils.cuh:48-58. */
void orc_vq_spmm_csr(const void* codes, int code_dt, const float* cbs, const void* indptr,
                     const void* indices, int idx_dt, float* out, int64_t n_dst, int64_t n_cb, int64_t K,
                     int64_t cs, int64_t D, int reduce, int acc64) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t d = 0; d < n_dst; ++d) {
    int64_t b = load_idx(indptr, idx_dt, d), e = load_idx(indptr, idx_dt, d + 1);
    float deg = e - b == 0 ? 1.0f : (float)(e - b);
    for (int64_t j = 0; j < D; ++j) {
      float acc = 0.0f;
      double acc_d = 0.0;
      for (int64_t k = b; k < e; ++k) {
        float v = vq_at(codes, code_dt, cbs, DT_F32, load_idx(indices, idx_dt, k), n_cb, K, cs, j);
        acc += v;
        acc_d += v;
      }
      if (acc64) out[d * D + j] = (float)(reduce == 0 ? acc_d / deg : acc_d);
      else out[d * D + j] = reduce == 0 ? acc / deg : acc;
    }
  }
}

/* ------------------------------------------------------------------------------------------
 * Two-level hybrid.  The reference pins only the hybrid DECODE, as the concatenation
 * cat(sq_decompress(first rows), vq_decompress(rest)) (tests/test_fusion_decompress.py:32-43).
 * The single-launch hybrid aggregation is the composition "decode every source row with the
 * codec that owns it (reference decode above), then the reference mean": slot[s] >= 0 selects row
 * slot[s] of the SQ table, slot[s] < 0 selects row s of the VQ table.
 * ------------------------------------------------------------------------------------------ */
void orc_hybrid_decompress(const void* sq_codes, int sq_dt, const float* sq_cb, int bits,
                           int64_t column_slice, int64_t sq_rows, int64_t sq_src_dim, const void* vq_codes,
                           int vq_dt, const float* vq_cbs, int64_t vq_rows, int64_t n_cb, int64_t K,
                           int64_t cs, float* out, int64_t D) {
  orc_sq_decompress(sq_codes, sq_dt, out, sq_cb, sq_rows, sq_src_dim, D, bits, column_slice);
  orc_vq_decompress(vq_codes, vq_dt, vq_cbs, DT_F32, out + sq_rows * D, vq_rows, n_cb, K, cs, D);
}

void orc_hybrid_spmm_csr(const void* sq_codes, int sq_dt, const float* sq_cb, int bits,
                         int64_t column_slice, int64_t sq_src_dim, const void* vq_codes, int vq_dt,
                         const float* vq_cbs, int64_t n_cb, int64_t K, int64_t cs, const int32_t* slot,
                         const void* indptr, const void* indices, int idx_dt, float* out, int64_t n_dst,
                         int64_t D, int reduce, int acc64) {
  const float drange = (float)(1 << (bits - 1));
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t d = 0; d < n_dst; ++d) {
    int64_t b = load_idx(indptr, idx_dt, d), e = load_idx(indptr, idx_dt, d + 1);
    float deg = e - b == 0 ? 1.0f : (float)(e - b);
    for (int64_t j = 0; j < D; ++j) {
      const float* row = sq_cb + (j / column_slice) * CB_DIM;
      float acc = 0.0f;
      double acc_d = 0.0;
      for (int64_t k = b; k < e; ++k) {
        int64_t s = load_idx(indices, idx_dt, k);
        float v;
        if (slot[s] >= 0)
          v = sq_decode_one(sq_code_at(sq_codes, sq_dt, slot[s], sq_src_dim, j, bits), bits, drange,
                            row[2], row[3], row[4]);
        else
          v = vq_at(vq_codes, vq_dt, vq_cbs, DT_F32, s, n_cb, K, cs, j);
        acc += v;
        acc_d += v;
      }
      if (acc64) out[d * D + j] = (float)(reduce == 0 ? acc_d / deg : acc_d);
      else out[d * D + j] = reduce == 0 ? acc / deg : acc;
    }
  }
}

/* ------------------------------------------------------------------------------------------
 * Dropout: src/fusion_dropout.cu:11-17 zeroes an element with probability p when training and
 * never rescales survivors (:16).  The reference draws from a time-seeded XORWOW state per thread,
 * so only the statistics are comparable; the replacement is counter based (Philox4x32-10 keyed by
 * the caller's seed, counter = element index / 4, word = element index % 4) and this is its
 * restatement: element i is dropped iff its 32-bit draw is below floor(p * 2^32).
 * scale != 0 additionally multiplies survivors by 1/(1-p) (torch.nn.Dropout convention).
 * ------------------------------------------------------------------------------------------ */
static inline void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
  for (int r = 0; r < 10; ++r) {
    uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
    uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0, n1 = (uint32_t)p1;
    uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1, n3 = (uint32_t)p0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
}

uint32_t orc_dropout_threshold(float p) {
  double t = (double)p * 4294967296.0;
  if (t <= 0) return 0u;
  if (t >= 4294967295.0) return 4294967295u;
  return (uint32_t)t;
}

void orc_dropout(float* x, int64_t numel, float p, int training, uint64_t seed, uint64_t offset, int scale) {
  if (!training) return;
  const uint32_t thr = orc_dropout_threshold(p);
  const float keep_scale = scale ? 1.0f / (1.0f - p) : 1.0f;
  for (int64_t i = 0; i < numel; ++i) {
    uint64_t blk = (uint64_t)i / 4u;
    uint32_t c[4] = {(uint32_t)blk, (uint32_t)(blk >> 32), (uint32_t)offset, (uint32_t)(offset >> 32)};
    philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
    int drop = p >= 1.0f || c[i & 3] < thr;
    x[i] = drop ? 0.0f : (scale ? x[i] * keep_scale : x[i]);
  }
}

/* ------------------------------------------------------------------------------------------
 * K-means distance and assignment.  The arithmetic lives in RAFT 23.10 (rapidsai/raft,
 * branch-23.10), called at src/kmeans.cu:93-95,114-116; it is not part of the reference checkout,
 * so the operative definition is the reference's own torch restatement, examples/my_kmeans.py:
 * L2 = sum((a-b)^2) without a square root (:43-48), cosine = 1 - cos(a,b) (:51-55), labels =
 * argmin with the first minimum winning (:123-124).  metric: 0 = L2, 1 = cosine.
 * Distances are accumulated in double and rounded once, so that this is the reference VALUE to
 * within half an ulp and any fp32 evaluation order can be compared with a small tolerance.
 * ------------------------------------------------------------------------------------------ */
static inline double pair_dist(const float* a, const float* b, int64_t d, int metric) {
  if (metric == 0) {
    double s = 0;
    for (int64_t t = 0; t < d; ++t) { double df = (double)a[t] - (double)b[t]; s += df * df; }
    return s;
  }
  double ab = 0, aa = 0, bb = 0;
  for (int64_t t = 0; t < d; ++t) { ab += (double)a[t] * b[t]; aa += (double)a[t] * a[t]; bb += (double)b[t] * b[t]; }
  return 1.0 - ab / (sqrt(aa) * sqrt(bb));
}

void orc_pairwise_distance(const float* x, const float* y, float* dist, int64_t n, int64_t k, int64_t d,
                           int metric) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
    for (int64_t c = 0; c < k; ++c) dist[i * k + c] = (float)pair_dist(x + i * d, y + c * d, d, metric);
}

/* labels[i] = first argmin; best[i]/second[i] (optional) = the two smallest distances in double,
 * which lets a test excuse exact or near ties. */
void orc_kmeans_assign(const float* x, const float* centers, int64_t* labels, double* best, double* second,
                       int64_t n, int64_t k, int64_t d, int metric) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    double b1 = INFINITY, b2 = INFINITY;
    int64_t arg = 0;
    for (int64_t c = 0; c < k; ++c) {
      double v = pair_dist(x + i * d, centers + c * d, d, metric);
      if (v != v) v = 1.0; /* NaN distances are patched to 1 by the caller, examples/my_kmeans.py:92-94 */
      if (v < b1) { b2 = b1; b1 = v; arg = c; }
      else if (v < b2) b2 = v;
    }
    labels[i] = arg;
    if (best) best[i] = b1;
    if (second) second[i] = b2;
  }
}

/* ------------------------------------------------------------------------------------------
 * Neighbour sampling.  The reference's sampler lives in its ShmTensor submodule, whose source is
 * not part of the checkout (parity unpinned); the contract is read off the call sites
 * (examples/dataloader.py:167-182): per seed, all in-neighbours when there are at most num_pick,
 * else num_pick distinct ones chosen uniformly; output CSC over the seeds with global ids.  This
 * restates the library's own generator (Floyd's algorithm over Philox draws) so that the kernel can
 * be checked draw for draw; uniformity is checked statistically in the tests.
 * ------------------------------------------------------------------------------------------ */
void orc_sample_neighbors(const int64_t* indptr, const int64_t* indices, const int64_t* seeds,
                          const int64_t* out_indptr, int64_t* out_indices, int64_t n_seeds, int num_pick,
                          uint64_t rng_seed, uint64_t rng_offset) {
  for (int64_t i = 0; i < n_seeds; ++i) {
    int64_t v = seeds[i], begin = indptr[v], d = indptr[v + 1] - begin;
    int64_t* out = out_indices + out_indptr[i];
    if (d <= num_pick) { for (int64_t t = 0; t < d; ++t) out[t] = indices[begin + t]; continue; }
    int64_t chosen[64];
    uint32_t c[4] = {0, 0, 0, 0};
    for (int s = 0; s < num_pick; ++s) {
      if ((s & 1) == 0) {
        uint64_t ctr = (uint64_t)i * 32u + (uint64_t)(s >> 1);
        c[0] = (uint32_t)ctr; c[1] = (uint32_t)(ctr >> 32); c[2] = (uint32_t)rng_offset; c[3] = (uint32_t)(rng_offset >> 32);
        philox4x32_10(c, (uint32_t)rng_seed, (uint32_t)(rng_seed >> 32));
      }
      uint64_t bits = (s & 1) == 0 ? ((uint64_t)c[0] << 32 | c[1]) : ((uint64_t)c[2] << 32 | c[3]);
      int64_t j = d - num_pick + s;
      int64_t t = (int64_t)(((unsigned __int128)bits * (unsigned __int128)(uint64_t)(j + 1)) >> 64);
      int taken = 0;
      for (int q = 0; q < s; ++q) taken |= chosen[q] == t;
      chosen[s] = taken ? j : t;
    }
    for (int s = 0; s < num_pick; ++s) out[s] = indices[begin + chosen[s]];
  }
}
