// Vector (product) quantisation decode: out[i, j] = codebooks[s][codes[i, s]][j - s*cs], s = j / cs
// (reference operator vq_decompress, src/vq_quantization.cu:5-60).
//
// A pure gather bound by the fp32 output stream (4 B per element against 1/cs code bytes); the
// codebooks (<= a few hundred KB) are served by L1/L2 through the read-only path.  Each thread
// emits one float4 when the slice width and feat_dim are multiples of four.  A code outside
// [0, length) cannot be told from a valid one by the reference (it reads out of bounds); here it is
// clamped to the last centroid so that a bad table cannot fault the device.
#include <type_traits>

#include "common.cuh"

namespace f2c {

template <typename CodeT>
__device__ __forceinline__ uint32_t load_code(const void* codes, int64_t pos, uint32_t length) {
  int v = (int)reinterpret_cast<const CodeT*>(codes)[pos];
  uint32_t u = (uint32_t)v;
  return u < length ? u : length - 1;
}

__device__ __forceinline__ float4 load_cb4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 load_cb4(const __half* p) {
  uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
  __half2 a = *reinterpret_cast<__half2*>(&raw.x), b = *reinterpret_cast<__half2*>(&raw.y);
  float2 fa = __half22float2(a), fb = __half22float2(b);
  return make_float4(fa.x, fa.y, fb.x, fb.y);
}
__device__ __forceinline__ float load_cb1(const float* p) { return __ldg(p); }
__device__ __forceinline__ float load_cb1(const __half* p) { return __half2float(__ldg(p)); }

template <typename CodeT, typename CbT>
__global__ void __launch_bounds__(256) vq_decompress_vec_kernel(const void* __restrict__ codes, const CbT* __restrict__ cbs,
                                                                float* __restrict__ out, int64_t n_vec, int vec_per_row,
                                                                int n_cb, uint32_t length, int cs, int feat_dim) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  int64_t row = i / vec_per_row;
  int j = (int)(i % vec_per_row) * 4;
  int s = j / cs, off = j - s * cs;
  uint32_t code = load_code<CodeT>(codes, row * n_cb + s, length);
  float4 v = load_cb4(cbs + ((int64_t)s * length + code) * cs + off);
  stg_cs_f4(out + row * feat_dim + j, v);
}

template <typename CodeT, typename CbT>
__global__ void __launch_bounds__(256) vq_decompress_scalar_kernel(const void* __restrict__ codes, const CbT* __restrict__ cbs,
                                                                   float* __restrict__ out, int64_t numel, int n_cb,
                                                                   uint32_t length, int cs, int feat_dim) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= numel) return;
  int64_t row = i / feat_dim;
  int j = (int)(i % feat_dim);
  int s = j / cs, off = j - s * cs;
  uint32_t code = load_code<CodeT>(codes, row * n_cb + s, length);
  out[i] = load_cb1(cbs + ((int64_t)s * length + code) * cs + off);
}

// Streaming variant for the common shapes (uint8 codes, fp32 codebooks that fit in shared memory, vec_per_row
// dividing the CTA size): the codebooks are staged once per CTA of a persistent grid, a thread keeps one float4
// column position for its whole life (so its subspace and offset are computed once, and row advance is an add),
// and eight rows are in flight per thread.  Subspaces narrower than 32 columns are interleaved inside 128-byte
// lines, so that the eight lanes of a quarter-warp read eight different 16-byte bank groups whatever the codes.
constexpr int kVqStreamThreads = 1024;
constexpr size_t kVqStreamSmem = 200 * 1024;

__global__ void __launch_bounds__(kVqStreamThreads, 1) vq_decompress_stream_kernel(
    const uint8_t* __restrict__ codes, const float* __restrict__ cbs, float* __restrict__ out, int64_t rows, int vec_per_row,
    int n_cb, int K, int cs, int feat_dim, int spq, int stride) {
  extern __shared__ __align__(128) unsigned char vq_smem[];
  {  // consecutive threads write consecutive 16-byte pieces of shared memory (no bank conflicts while staging)
    const int lg4 = 31 - __clz(cs >> 2);
    const float4* src = reinterpret_cast<const float4*>(cbs);
    float4* dst = reinterpret_cast<float4*>(vq_smem);
    if (spq > 1) {  // 128-byte line = the centroids `code` of spq consecutive subspaces
      const int n16 = ((n_cb + spq - 1) / spq) * K * 8;
      for (int i = threadIdx.x; i < n16; i += kVqStreamThreads) {
        const int piece = i & 7, line = i >> 3;
        const int code = line % K, grp = line / K;
        const int sl = grp * spq + (piece >> lg4), q = piece & ((1 << lg4) - 1);
        dst[i] = sl < n_cb ? __ldg(src + ((sl * K + code) << lg4) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    } else {
      const int n16 = (n_cb * K) << lg4;
      for (int i = threadIdx.x; i < n16; i += kVqStreamThreads) dst[i] = __ldg(src + i);
    }
  }
  __syncthreads();
  const int rows_per_cta = kVqStreamThreads / vec_per_row;
  const int j = (threadIdx.x % vec_per_row) * 4;
  const int s = j / cs, off = j - s * cs;
  const uint32_t lane_base = (uint32_t)__cvta_generic_to_shared(vq_smem) +
                             (spq > 1 ? (uint32_t)((s / spq) * K * 128 + (s % spq) * cs * 4 + off * 4) : (uint32_t)(s * K * stride + off * 4));
  const int64_t step = (int64_t)gridDim.x * rows_per_cta;
  int64_t row = (int64_t)blockIdx.x * rows_per_cta + threadIdx.x / vec_per_row;
  const uint8_t* cp = codes + row * n_cb + s;
  float* op = out + row * feat_dim + j;
  const int64_t cstep = step * n_cb, ostep = step * feat_dim;
  const uint32_t kmax = (uint32_t)K - 1u;
  constexpr int kInFlight = 8;  // rows in flight per thread
  for (; row + (kInFlight - 1) * step < rows; row += kInFlight * step, cp += kInFlight * cstep, op += kInFlight * ostep) {
    uint32_t c[kInFlight];
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) c[u] = min((uint32_t)__ldg(cp + u * cstep), kmax);
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      float4 v;
      asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(lane_base + c[u] * (uint32_t)stride));
      stg_cs_f4(op + u * ostep, v);
    }
  }
  for (; row < rows; row += step, cp += cstep, op += ostep) {
    const uint32_t c = min((uint32_t)__ldg(cp), kmax);
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(lane_base + c * (uint32_t)stride));
    stg_cs_f4(op, v);
  }
}

// Returns true when the streaming kernel was launched.
static bool try_vq_decompress_stream(const void* codes, const float* cbs, float* out, int64_t rows, int64_t n_cb, int64_t K,
                                     int64_t cs, int64_t D, cudaStream_t st) {
  if (K > 256 || cs < 4 || (cs & (cs - 1)) != 0 || D % 4 != 0 || D / 4 > kVqStreamThreads || kVqStreamThreads % (D / 4) != 0) return false;
  if (!aligned(out, 16) || !aligned(cbs, 16) || rows < 4096) return false;
  const int spq = cs < 32 ? (int)(32 / cs) : 1;
  const int stride = cs < 32 ? 128 : (int)cs * 4;
  const size_t smem = spq > 1 ? (size_t)ceil_div(n_cb, spq) * K * 128 : (size_t)n_cb * K * cs * 4;
  if (smem > kVqStreamSmem) return false;
  if (cudaFuncSetAttribute(vq_decompress_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kVqStreamSmem) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  const int rows_per_cta = kVqStreamThreads / (int)(D / 4);
  int64_t grid = ceil_div(rows, rows_per_cta);
  if (grid > current_sm_count()) grid = current_sm_count();
  vq_decompress_stream_kernel<<<(unsigned)grid, kVqStreamThreads, smem, st>>>(
      (const uint8_t*)codes, cbs, out, rows, (int)(D / 4), (int)n_cb, (int)K, (int)cs, (int)D, spq, stride);
  return true;
}

template <typename CodeT, typename CbT>
static int launch_vq_decompress(const void* codes, const void* cbs, float* out, int64_t rows, int64_t n_cb, int64_t length,
                                int64_t cs, int64_t D, cudaStream_t st) {
  int64_t numel = rows * D;
  if (numel == 0) return F2C_OK;
  bool vec = cs % 4 == 0 && D % 4 == 0 && aligned(out, 16) && aligned(cbs, 4 * sizeof(CbT));
  if (sizeof(CodeT) == 1 && !std::is_signed<CodeT>::value && std::is_same<CbT, float>::value &&
      try_vq_decompress_stream(codes, (const float*)cbs, out, rows, n_cb, length, cs, D, st))
    return check_launch("vq_decompress");
  if (vec) {
    int64_t n_vec = numel / 4;
    vq_decompress_vec_kernel<CodeT, CbT><<<(unsigned)ceil_div(n_vec, 256), 256, 0, st>>>(
        codes, (const CbT*)cbs, out, n_vec, (int)(D / 4), (int)n_cb, (uint32_t)length, (int)cs, (int)D);
  } else {
    vq_decompress_scalar_kernel<CodeT, CbT><<<(unsigned)ceil_div(numel, 256), 256, 0, st>>>(
        codes, (const CbT*)cbs, out, numel, (int)n_cb, (uint32_t)length, (int)cs, (int)D);
  }
  return check_launch("vq_decompress");
}

int validate_vq(const char* op, int code_dtype, int64_t n_cb, int64_t length, int64_t cs, int64_t feat_dim) {
  F2C_REQUIRE(is_code_dtype(code_dtype), F2C_ERR_UNSUPPORTED, "%s: codes must be uint8, int8 or int16", op);
  F2C_REQUIRE(n_cb >= 1 && length >= 1 && cs >= 1 && feat_dim >= 0, F2C_ERR_INVALID, "%s: bad codebook shape", op);
  F2C_REQUIRE(feat_dim <= n_cb * cs, F2C_ERR_INVALID, "%s: feat_dim %lld exceeds n_codebooks*column_slice = %lld", op,
              (long long)feat_dim, (long long)(n_cb * cs));
  F2C_REQUIRE(feat_dim < (1ll << 24) && length < (1ll << 31) && cs < (1ll << 24) && n_cb < (1ll << 24), F2C_ERR_LIMIT,
              "%s: shape too large", op);
  return F2C_OK;
}

}  // namespace f2c

using namespace f2c;

extern "C" int f2c_vq_decompress(const void* codes, int code_dtype, const void* codebooks, int codebook_dtype, float* out,
                                 int64_t rows, int64_t n_codebooks, int64_t length, int64_t column_slice,
                                 int64_t feat_dim, void* stream) {
  F2C_REQUIRE(rows >= 0, F2C_ERR_INVALID, "vq_decompress: negative size");
  int rc = validate_vq("vq_decompress", code_dtype, n_codebooks, length, column_slice, feat_dim);
  if (rc) return rc;
  F2C_REQUIRE(codebook_dtype == F2C_F32 || codebook_dtype == F2C_F16, F2C_ERR_UNSUPPORTED,
              "vq_decompress: codebooks must be float32 or float16");
  F2C_REQUIRE(rows * feat_dim == 0 || (codes && out && codebooks), F2C_ERR_INVALID, "vq_decompress: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
#define F2C_VQ(T, C) return launch_vq_decompress<T, C>(codes, codebooks, out, rows, n_codebooks, length, column_slice, feat_dim, st)
  if (codebook_dtype == F2C_F32) {
    if (code_dtype == F2C_U8) F2C_VQ(uint8_t, float);
    if (code_dtype == F2C_I8) F2C_VQ(int8_t, float);
    F2C_VQ(int16_t, float);
  }
  if (code_dtype == F2C_U8) F2C_VQ(uint8_t, __half);
  if (code_dtype == F2C_I8) F2C_VQ(int8_t, __half);
  F2C_VQ(int16_t, __half);
#undef F2C_VQ
}
