// Scalar quantisation: log2-domain sign-magnitude codes of 1/2/4/8/16 bits
// (reference operators sq_compress / sq_decompress, src/sq_quantization.cu).
//
// Both are streaming element-wise kernels bound by HBM: compress moves 8 B per element
// (fp32 in, fp32-valued code out), decompress bits/8 + 4 B per element.  Each thread produces one
// 16-byte vector of outputs (two for 1-bit codes, so that it consumes a whole byte); ragged shapes
// fall back to one thread per element.  The arithmetic is the reference's expression compiled with
// the same math flags, so codes and decoded values carry the reference kernel's bits.
#include <type_traits>

#include "common.cuh"

namespace f2c {

// ---------------------------------------------------------------- compress
template <int BITS>
__device__ __forceinline__ float sq_encode(float x, const float* __restrict__ cb) {
  if (BITS == 1) return x <= 0.0f ? 0.0f : 1.0f;
  constexpr float drange = (float)(1 << (BITS - 1));
  float fmin = __ldg(cb + 0), fmax = __ldg(cb + 1), emin = __ldg(cb + 2), emax = __ldg(cb + 3);
  bool neg = x <= 0.0f;
  float v = fabsf(x);
  v = fminf(fmaxf(v, fmin), fmax);
  v = log2f(v);
  v = (v - emin) / (emax - emin) * drange;
  v = floorf(v);
  v = neg ? -1.0f - v : v;
  if (BITS < 8) v += drange;
  return v;
}

template <int BITS>
__global__ void __launch_bounds__(256) sq_compress_vec_kernel(const float4* __restrict__ src, float4* __restrict__ dst,
                                                              const float* __restrict__ codebooks, int64_t n_vec,
                                                              int vec_per_row, int column_slice) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  int c0 = (int)(i % vec_per_row) * 4;
  float4 x = src[i], y;
  y.x = sq_encode<BITS>(x.x, codebooks + (c0 + 0) / column_slice * kCodebookDim);
  y.y = sq_encode<BITS>(x.y, codebooks + (c0 + 1) / column_slice * kCodebookDim);
  y.z = sq_encode<BITS>(x.z, codebooks + (c0 + 2) / column_slice * kCodebookDim);
  y.w = sq_encode<BITS>(x.w, codebooks + (c0 + 3) / column_slice * kCodebookDim);
  dst[i] = y;
}

template <int BITS>
__global__ void __launch_bounds__(256) sq_compress_scalar_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                                 const float* __restrict__ codebooks, int64_t numel,
                                                                 int feat_dim, int column_slice) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= numel) return;
  int c = (int)(i % feat_dim);
  dst[i] = sq_encode<BITS>(src[i], codebooks + c / column_slice * kCodebookDim);
}

template <int BITS>
static int launch_compress(const float* src, float* dst, const float* cb, int64_t rows, int64_t D, int64_t cs,
                           cudaStream_t st) {
  int64_t numel = rows * D;
  if (numel == 0) return F2C_OK;
  if (D % 4 == 0 && aligned(src, 16) && aligned(dst, 16)) {
    int64_t n_vec = numel / 4;
    sq_compress_vec_kernel<BITS><<<(unsigned)ceil_div(n_vec, 256), 256, 0, st>>>(
        (const float4*)src, (float4*)dst, cb, n_vec, (int)(D / 4), (int)cs);
  } else {
    sq_compress_scalar_kernel<BITS><<<(unsigned)ceil_div(numel, 256), 256, 0, st>>>(src, dst, cb, numel, (int)D, (int)cs);
  }
  return check_launch("sq_compress");
}

// ---------------------------------------------------------------- decompress
template <typename CodeT>
__device__ __forceinline__ float code_as_float(const void* codes, int64_t pos) {
  return (float)reinterpret_cast<const CodeT*>(codes)[pos];
}

// One thread per output element: any shape, any alignment.
template <int BITS, typename CodeT>
__global__ void __launch_bounds__(256) sq_decompress_scalar_kernel(const void* __restrict__ codes, float* __restrict__ out,
                                                                   const float* __restrict__ codebooks, int64_t numel,
                                                                   int64_t src_dim, int feat_dim, int column_slice) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= numel) return;
  int64_t row = i / feat_dim;
  int j = (int)(i % feat_dim);
  const float* cb = codebooks + j / column_slice * kCodebookDim;
  float c;
  if (BITS >= 8) {
    c = code_as_float<CodeT>(codes, row * src_dim + j);
  } else {
    constexpr int PER = 8 / (BITS >= 8 ? 8 : BITS);
    constexpr uint32_t MASK = (1u << (BITS >= 8 ? 8 : BITS)) - 1u;
    uint32_t byte = reinterpret_cast<const uint8_t*>(codes)[row * src_dim + j / PER];
    c = (float)((byte >> (BITS * (j % PER))) & MASK);
  }
  float emin = __ldg(cb + 2), emax = __ldg(cb + 3), mean = __ldg(cb + 4);
  out[i] = sq_decode<BITS>(c, sq_scale<BITS>(emin, emax), emin, mean);
}

// Vector path: each thread decodes EPT consecutive columns of one row (EPT = 4, or 8 for 1-bit codes)
// from one aligned load of EPT*BITS/8 bytes and writes EPT/4 float4.
template <int BITS, typename CodeT>
__global__ void __launch_bounds__(256) sq_decompress_vec_kernel(const void* __restrict__ codes, float* __restrict__ out,
                                                                const float* __restrict__ codebooks, int64_t n_chunks,
                                                                int64_t src_dim, int feat_dim, int chunks_per_row,
                                                                int column_slice) {
  constexpr int EPT = BITS == 1 ? 8 : 4;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_chunks) return;
  int64_t row = i / chunks_per_row;
  int c0 = (int)(i % chunks_per_row) * EPT;
  float c[EPT];
  if (BITS >= 8 && sizeof(CodeT) == 2) {
    const CodeT* p = reinterpret_cast<const CodeT*>(codes) + row * src_dim + c0;
    uint2 raw = *reinterpret_cast<const uint2*>(p);
    CodeT tmp[4];
    *reinterpret_cast<uint2*>(tmp) = raw;
#pragma unroll
    for (int e = 0; e < 4; ++e) c[e] = (float)tmp[e];
  } else if (BITS >= 8) {
    const CodeT* p = reinterpret_cast<const CodeT*>(codes) + row * src_dim + c0;
    uint32_t raw = *reinterpret_cast<const uint32_t*>(p);
#pragma unroll
    for (int e = 0; e < 4; ++e) c[e] = (float)(CodeT)((raw >> (8 * e)) & 0xFFu);
  } else {
    constexpr int B = BITS >= 8 ? 1 : BITS;  // keeps shifts valid in dead instantiations
    constexpr uint32_t MASK = (1u << B) - 1u;
    const uint8_t* p = reinterpret_cast<const uint8_t*>(codes) + row * src_dim + c0 * B / 8;
    uint32_t raw;
    if (B == 4) raw = *reinterpret_cast<const uint16_t*>(p);
    else raw = *p;
#pragma unroll
    for (int e = 0; e < EPT; ++e) c[e] = (float)((raw >> (B * e)) & MASK);
  }
  int cb0 = c0 / column_slice, cb1 = (c0 + EPT - 1) / column_slice;
  float v[EPT];
  if (cb0 == cb1) {
    const float* cb = codebooks + cb0 * kCodebookDim;
    float emin = __ldg(cb + 2), emax = __ldg(cb + 3), mean = __ldg(cb + 4);
    float s = sq_scale<BITS>(emin, emax);
#pragma unroll
    for (int e = 0; e < EPT; ++e) v[e] = sq_decode<BITS>(c[e], s, emin, mean);
  } else {
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
      const float* cb = codebooks + (c0 + e) / column_slice * kCodebookDim;
      float emin = __ldg(cb + 2), emax = __ldg(cb + 3), mean = __ldg(cb + 4);
      v[e] = sq_decode<BITS>(c[e], sq_scale<BITS>(emin, emax), emin, mean);
    }
  }
  float4* o = reinterpret_cast<float4*>(out + row * feat_dim + c0);
#pragma unroll
  for (int q = 0; q < EPT / 4; ++q) stg_cs_f4(reinterpret_cast<float*>(o + q), make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
}

// Table variant of the vector path for 1..8-bit codes stored in bytes: a persistent grid whose CTAs first decode
// every code value once per codebook row WITH THE SAME EXPRESSION as the element-wise path (same bits) into shared
// memory - 2^BITS * n_codebooks exp2f per CTA instead of one per element - and then stream: a thread keeps one
// column position for its whole life, so its codebook row is fixed, row advance is an add, and an element costs a
// bit-field extract, a shift-add and one shared-memory read.  The table is replicated COPIES times (one copy per
// lane modulo COPIES) to spread the reads over the banks.
constexpr int kSqLutThreads = 256;
constexpr int kSqLutBytes = 64 * 1024;

template <int BITS>
__global__ void __launch_bounds__(kSqLutThreads) sq_decompress_lut_kernel(
    const uint8_t* __restrict__ codes, float* __restrict__ out, const float* __restrict__ codebooks, int64_t rows,
    int64_t row_bytes, int feat_dim, int chunks_per_row, int column_slice, int n_cb, int log_copies, int is_signed) {
  constexpr int EPT = BITS == 1 ? 8 : 4;
  constexpr int NCODE = 1 << BITS;
  constexpr uint32_t MASK = NCODE - 1;
  extern __shared__ float sq_tab[];
  const int copies = 1 << log_copies;
  {
    // a warp decodes 32 entries (one per lane), then hands them round by shuffle so that every store instruction
    // writes 32 consecutive words (entry-major, copy-minor): no bank conflicts while building
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_entries = n_cb * NCODE;
    const int per_store = 32 >> log_copies;  // entries covered by one store instruction
    for (int e0 = warp * 32; e0 < n_entries; e0 += (kSqLutThreads / 32) * 32) {
      const int i = e0 + lane;
      float v = 0.0f;
      if (i < n_entries) {
        const int row = i >> BITS, code = i & (int)MASK;
        const float emin = __ldg(codebooks + row * kCodebookDim + 2), emax = __ldg(codebooks + row * kCodebookDim + 3);
        const float mean = __ldg(codebooks + row * kCodebookDim + 4);
        const float c = (BITS == 8 && is_signed) ? (float)(int8_t)code : (float)code;
        v = sq_decode<BITS>(c, sq_scale<BITS>(emin, emax), emin, mean);
      }
      for (int j = 0; j < 32; j += per_store) {
        const int src = j + (lane >> log_copies);
        const float vv = __shfl_sync(0xffffffffu, v, src);
        if (e0 + src < n_entries) sq_tab[((e0 + src) << log_copies) + (lane & (copies - 1))] = vv;
      }
    }
  }
  __syncthreads();
  const int rows_per_cta = kSqLutThreads / chunks_per_row;
  const int c0 = (threadIdx.x % chunks_per_row) * EPT;
  int cb_row = c0 / column_slice;
  if (cb_row >= n_cb) cb_row = n_cb - 1;
  // byte address of entry (cb_row, code 0, this lane's copy); entry `code` is code << (log_copies + 2) further
  const uint32_t tab = (uint32_t)__cvta_generic_to_shared(sq_tab) + ((((uint32_t)cb_row << BITS) << log_copies) + (threadIdx.x & (copies - 1))) * 4u;
  const int sh = log_copies + 2;
  const int64_t step = (int64_t)gridDim.x * rows_per_cta;
  int64_t row = (int64_t)blockIdx.x * rows_per_cta + threadIdx.x / chunks_per_row;
  const uint8_t* cp = codes + row * row_bytes + (c0 * BITS) / 8;
  float* op = out + row * feat_dim + c0;
  const int64_t cstep = step * row_bytes, ostep = step * feat_dim;
  auto fetch = [&](const uint8_t* q) -> uint32_t {
    if (BITS == 8) return *reinterpret_cast<const uint32_t*>(q);
    if (BITS == 4) return *reinterpret_cast<const uint16_t*>(q);
    return *q;
  };
  auto emit = [&](uint32_t raw, float* o) {
    float v[EPT];
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
      const uint32_t code = (raw >> (BITS * e)) & MASK;
      asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v[e]) : "r"(tab + (code << sh)));
    }
#pragma unroll
    for (int q = 0; q < EPT / 4; ++q) stg_cs_f4(o + 4 * q, make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
  };
  constexpr int kInFlight = 8;  // rows in flight per thread
  for (; row + (kInFlight - 1) * step < rows; row += kInFlight * step, cp += kInFlight * cstep, op += kInFlight * ostep) {
    uint32_t raw[kInFlight];
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) raw[u] = fetch(cp + u * cstep);
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) emit(raw[u], op + u * ostep);
  }
  for (; row < rows; row += step, cp += cstep, op += ostep) emit(fetch(cp), op);
}

// Returns true when the table kernel was launched (shape served).
template <int BITS, typename CodeT>
static bool try_decompress_lut(const void* codes, float* out, const float* cb, int64_t rows, int64_t src_dim, int64_t D,
                               int64_t cs, cudaStream_t st) {
  if (BITS > 8 || sizeof(CodeT) != 1) return false;
  constexpr int EPT = BITS == 1 ? 8 : 4;
  constexpr int LOAD_BYTES = BITS == 8 ? 4 : (BITS == 4 ? 2 : 1);
  const int64_t n_cb = ceil_div(D, cs);
  if (D % EPT != 0 || rows < 4096 || !aligned(out, 16) || !aligned(codes, LOAD_BYTES) || src_dim % LOAD_BYTES != 0) return false;
  const int64_t cpr = D / EPT;
  if (cpr > kSqLutThreads || kSqLutThreads % cpr != 0) return false;
  if (n_cb > 1 && cs % EPT != 0) return false;  // a thread's columns must share one codebook row
  const int64_t entries = n_cb << BITS;
  if (entries * 4 > kSqLutBytes) return false;
  int log_copies = 0;
  while (log_copies < 5 && (entries << (log_copies + 1)) * 4 <= kSqLutBytes) ++log_copies;
  const size_t smem = (size_t)(entries << log_copies) * 4;
  auto kern = sq_decompress_lut_kernel<BITS <= 8 ? BITS : 8>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSqLutBytes) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  const int rows_per_cta = kSqLutThreads / (int)cpr;
  int64_t grid = ceil_div(rows, rows_per_cta);
  const int64_t cap = (int64_t)current_sm_count() * (smem > 32 * 1024 ? 3 : 6);
  if (grid > cap) grid = cap;
  kern<<<(unsigned)grid, kSqLutThreads, smem, st>>>((const uint8_t*)codes, out, cb, rows, src_dim, (int)D, (int)cpr, (int)cs,
                                                    (int)n_cb, log_copies, std::is_signed<CodeT>::value ? 1 : 0);
  return true;
}

template <int BITS, typename CodeT>
static int launch_decompress(const void* codes, float* out, const float* cb, int64_t rows, int64_t src_dim, int64_t D,
                             int64_t cs, cudaStream_t st) {
  int64_t numel = rows * D;
  if (numel == 0) return F2C_OK;
  constexpr int EPT = BITS == 1 ? 8 : 4;
  // bytes consumed per chunk and the alignment its single load needs
  constexpr int LOAD_BYTES = BITS >= 8 ? 4 * (int)sizeof(CodeT) : (BITS == 4 ? 2 : 1);
  int64_t row_bytes = src_dim * (int64_t)sizeof(CodeT);
  bool vec = D % EPT == 0 && aligned(out, 16) && aligned(codes, LOAD_BYTES) && row_bytes % LOAD_BYTES == 0;
  if (try_decompress_lut<BITS, CodeT>(codes, out, cb, rows, src_dim, D, cs, st)) return check_launch("sq_decompress");
  if (vec) {
    int64_t n_chunks = numel / EPT;
    sq_decompress_vec_kernel<BITS, CodeT><<<(unsigned)ceil_div(n_chunks, 256), 256, 0, st>>>(
        codes, out, cb, n_chunks, src_dim, (int)D, (int)(D / EPT), (int)cs);
  } else {
    sq_decompress_scalar_kernel<BITS, CodeT><<<(unsigned)ceil_div(numel, 256), 256, 0, st>>>(
        codes, out, cb, numel, src_dim, (int)D, (int)cs);
  }
  return check_launch("sq_decompress");
}

}  // namespace f2c

using namespace f2c;

extern "C" int f2c_sq_compress(const float* src, float* dst, const float* codebooks, int64_t n_codebooks,
                               int64_t rows, int64_t feat_dim, int bits, int64_t column_slice, void* stream) {
  F2C_REQUIRE(rows >= 0 && feat_dim >= 0, F2C_ERR_INVALID, "sq_compress: negative size");
  F2C_REQUIRE(is_sq_bits(bits), F2C_ERR_UNSUPPORTED, "sq_compress: target_bits must be 1, 2, 4, 8 or 16 (got %d)", bits);
  F2C_REQUIRE(column_slice >= 1, F2C_ERR_INVALID, "sq_compress: column_slice must be >= 1");
  F2C_REQUIRE(feat_dim < (1ll << 31) && column_slice < (1ll << 31), F2C_ERR_LIMIT, "sq_compress: feat_dim too large");
  F2C_REQUIRE(n_codebooks * column_slice >= feat_dim, F2C_ERR_INVALID,
              "sq_compress: %lld codebook rows of %lld columns do not cover feat_dim %lld", (long long)n_codebooks,
              (long long)column_slice, (long long)feat_dim);
  F2C_REQUIRE(rows * feat_dim == 0 || (src && dst && codebooks), F2C_ERR_INVALID, "sq_compress: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  switch (bits) {
    case 1: return launch_compress<1>(src, dst, codebooks, rows, feat_dim, column_slice, st);
    case 2: return launch_compress<2>(src, dst, codebooks, rows, feat_dim, column_slice, st);
    case 4: return launch_compress<4>(src, dst, codebooks, rows, feat_dim, column_slice, st);
    case 8: return launch_compress<8>(src, dst, codebooks, rows, feat_dim, column_slice, st);
    default: return launch_compress<16>(src, dst, codebooks, rows, feat_dim, column_slice, st);
  }
}

namespace f2c {
// Shared argument check of every SQ-decoding entry point.
int validate_sq(const char* op, int code_dtype, int64_t n_codebooks, int64_t src_dim, int64_t feat_dim, int bits,
                int64_t column_slice) {
  F2C_REQUIRE(is_sq_bits(bits), F2C_ERR_UNSUPPORTED, "%s: target_bits must be 1, 2, 4, 8 or 16 (got %d)", op, bits);
  F2C_REQUIRE(is_code_dtype(code_dtype), F2C_ERR_UNSUPPORTED, "%s: codes must be uint8, int8 or int16", op);
  F2C_REQUIRE(bits >= 8 || code_dtype != F2C_I16, F2C_ERR_UNSUPPORTED,
              "%s: packed %d-bit codes must be a uint8/int8 tensor", op, bits);
  F2C_REQUIRE(column_slice >= 1 && feat_dim >= 0 && src_dim >= 0, F2C_ERR_INVALID, "%s: bad column_slice/feat_dim", op);
  F2C_REQUIRE(feat_dim < (1ll << 24) && column_slice < (1ll << 31), F2C_ERR_LIMIT, "%s: feat_dim too large", op);
  int64_t capacity = bits >= 8 ? src_dim : src_dim * (8 / bits);
  F2C_REQUIRE(feat_dim <= capacity, F2C_ERR_INVALID, "%s: feat_dim %lld exceeds the %lld elements a code row holds", op,
              (long long)feat_dim, (long long)capacity);
  F2C_REQUIRE(n_codebooks * column_slice >= feat_dim, F2C_ERR_INVALID,
              "%s: %lld codebook rows of %lld columns do not cover feat_dim %lld", op, (long long)n_codebooks,
              (long long)column_slice, (long long)feat_dim);
  return F2C_OK;
}
}  // namespace f2c

extern "C" int f2c_sq_decompress(const void* codes, int code_dtype, const float* codebooks, int64_t n_codebooks,
                                 float* out, int64_t rows, int64_t src_dim, int64_t feat_dim, int bits,
                                 int64_t column_slice, void* stream) {
  F2C_REQUIRE(rows >= 0, F2C_ERR_INVALID, "sq_decompress: negative size");
  int rc = validate_sq("sq_decompress", code_dtype, n_codebooks, src_dim, feat_dim, bits, column_slice);
  if (rc) return rc;
  F2C_REQUIRE(rows * feat_dim == 0 || (codes && out && codebooks), F2C_ERR_INVALID, "sq_decompress: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
#define F2C_DEC(B, T) return launch_decompress<B, T>(codes, out, codebooks, rows, src_dim, feat_dim, column_slice, st)
  if (bits < 8) {
    switch (bits) {
      case 1: F2C_DEC(1, uint8_t);
      case 2: F2C_DEC(2, uint8_t);
      default: F2C_DEC(4, uint8_t);
    }
  }
  if (bits == 8) {
    if (code_dtype == F2C_I8) F2C_DEC(8, int8_t);
    if (code_dtype == F2C_U8) F2C_DEC(8, uint8_t);
    F2C_DEC(8, int16_t);
  }
  if (code_dtype == F2C_I16) F2C_DEC(16, int16_t);
  if (code_dtype == F2C_I8) F2C_DEC(16, int8_t);
  F2C_DEC(16, uint8_t);
#undef F2C_DEC
}
