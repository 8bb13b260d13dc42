// Mean / sum aggregation of dense feature rows over a CSC block (reference operator spmm_csr,
// src/fusion_spmm.cu:13-70): out[d,:] = (sum_{k in N(d)} feat[indices[k],:]) / max(deg,1).
//
// HBM-bound row gather (E * D * sizeof(T) bytes).  One warp per destination row; a lane owns one
// 16-byte vector of each 32-vector column tile, so a neighbour row is fetched with one coalesced
// 512-byte request per tile; neighbour indices are fetched 32 at a time and broadcast by shuffle;
// four row loads are kept in flight.  Accumulation is sequential in CSC order in the feature dtype,
// which reproduces the reference's result bit for bit (it is the comparator of the fused kernels).
#include "common.cuh"

namespace f2c {

template <typename T> struct Acc;
template <> struct Acc<float> {
  using type = float;
  static __device__ __forceinline__ float zero() { return 0.0f; }
  static __device__ __forceinline__ float add(float a, float b) { return a + b; }
  static __device__ __forceinline__ float div(float a, float deg) { return a / deg; }
};
template <> struct Acc<double> {
  using type = double;
  static __device__ __forceinline__ double zero() { return 0.0; }
  static __device__ __forceinline__ double add(double a, double b) { return a + b; }
  static __device__ __forceinline__ double div(double a, float deg) { return a / deg; }
};
template <> struct Acc<__half> {  // at::Half: float add / float divide, rounded to half after every step
  using type = __half;
  static __device__ __forceinline__ __half zero() { return __float2half_rn(0.0f); }
  static __device__ __forceinline__ __half add(__half a, __half b) { return __float2half_rn(__half2float(a) + __half2float(b)); }
  static __device__ __forceinline__ __half div(__half a, float deg) { return __float2half_rn(__half2float(a) / deg); }
};

// VEC = elements per 16-byte vector (or 1 for the unaligned/ragged path).
template <typename T, typename IdxT, int VEC>
__global__ void __launch_bounds__(256) spmm_csr_kernel(const T* __restrict__ feat, T* __restrict__ out,
                                                       const IdxT* __restrict__ indptr, const IdxT* __restrict__ indices,
                                                       int64_t n_dst, int feat_dim, int reduce) {
  using A = Acc<T>;
  struct alignas(sizeof(T) * VEC) Vec { T v[VEC]; };
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t d = warp; d < n_dst; d += n_warps) {
    const int64_t begin = (int64_t)indptr[d], end = (int64_t)indptr[d + 1];
    const float deg = end - begin == 0 ? 1.0f : (float)(end - begin);
    for (int col0 = 0; col0 < feat_dim; col0 += 32 * VEC) {
      const int col = col0 + lane * VEC;
      const bool active = col < feat_dim;
      T acc[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = A::zero();
      for (int64_t k0 = begin; k0 < end; k0 += 32) {
        int64_t mine = k0 + lane < end ? (int64_t)indices[k0 + lane] : 0;
        int cnt = (int)(end - k0 < 32 ? end - k0 : 32);
        for (int t0 = 0; t0 < cnt; t0 += 4) {
          Vec r[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            int64_t src = __shfl_sync(0xffffffffu, mine, (t0 + u) & 31);
            if (active && t0 + u < cnt) r[u] = *reinterpret_cast<const Vec*>(feat + src * feat_dim + col);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (active && t0 + u < cnt) {
#pragma unroll
              for (int e = 0; e < VEC; ++e) acc[e] = A::add(acc[e], r[u].v[e]);
            }
          }
        }
      }
      if (active) {
        Vec o;
#pragma unroll
        for (int e = 0; e < VEC; ++e) o.v[e] = reduce == F2C_MEAN ? A::div(acc[e], deg) : acc[e];
        *reinterpret_cast<Vec*>(out + d * feat_dim + col) = o;
      }
    }
  }
}

template <typename T, typename IdxT>
static int launch_spmm(const void* feat, const void* indptr, const void* indices, void* out, int64_t n_dst, int64_t D,
                       int reduce, cudaStream_t st) {
  if (n_dst == 0 || D == 0) return F2C_OK;
  constexpr int VEC = 16 / (int)sizeof(T);
  int64_t blocks = ceil_div(n_dst, 8);  // 8 warps per block, one row per warp per pass
  if (blocks > current_sm_count() * 64) blocks = current_sm_count() * 64;
  bool vec = D % VEC == 0 && aligned(feat, 16) && aligned(out, 16);
  if (vec)
    spmm_csr_kernel<T, IdxT, VEC><<<(unsigned)blocks, 256, 0, st>>>((const T*)feat, (T*)out, (const IdxT*)indptr,
                                                                     (const IdxT*)indices, n_dst, (int)D, reduce);
  else
    spmm_csr_kernel<T, IdxT, 1><<<(unsigned)blocks, 256, 0, st>>>((const T*)feat, (T*)out, (const IdxT*)indptr,
                                                                   (const IdxT*)indices, n_dst, (int)D, reduce);
  return check_launch("spmm_csr");
}

}  // namespace f2c

using namespace f2c;

extern "C" int f2c_spmm_csr(const void* feat, int feat_dtype, const void* indptr, const void* indices, int index_dtype,
                            void* out, int64_t n_dst, int64_t feat_dim, int reduce, void* stream) {
  F2C_REQUIRE(n_dst >= 0 && feat_dim >= 0, F2C_ERR_INVALID, "spmm_csr: negative size");
  F2C_REQUIRE(is_index_dtype(index_dtype), F2C_ERR_UNSUPPORTED, "spmm_csr: indptr/indices must be int32 or int64");
  F2C_REQUIRE(feat_dtype == F2C_F32 || feat_dtype == F2C_F16 || feat_dtype == F2C_F64, F2C_ERR_UNSUPPORTED,
              "spmm_csr: features must be float32, float16 or float64");
  F2C_REQUIRE(reduce == F2C_MEAN || reduce == F2C_SUM, F2C_ERR_INVALID, "spmm_csr: reduce must be mean or sum");
  F2C_REQUIRE(feat_dim < (1ll << 24), F2C_ERR_LIMIT, "spmm_csr: feat_dim too large");
  F2C_REQUIRE(n_dst * feat_dim == 0 || (indptr && out), F2C_ERR_INVALID, "spmm_csr: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
#define F2C_SP(T) \
  return index_dtype == F2C_I32 ? launch_spmm<T, int32_t>(feat, indptr, indices, out, n_dst, feat_dim, reduce, st) \
                                : launch_spmm<T, int64_t>(feat, indptr, indices, out, n_dst, feat_dim, reduce, st)
  if (feat_dtype == F2C_F32) F2C_SP(float);
  if (feat_dtype == F2C_F64) F2C_SP(double);
  F2C_SP(__half);
#undef F2C_SP
}

// ---------------------------------------------------------------- backward of the mean / sum aggregation
// grad_src[indices[k], :] += grad_out[d, :] * w(d) for every edge k of destination row d, w = 1 / max(deg, 1) for the
// mean.  This is what autograd needs for the hidden GraphSAGE layers (the reference gets it from DGL's SAGEConv,
// examples/models.py:31); the fused first layer has no gradient through its aggregation (its input is codes).
// One warp per destination row; a lane owns float4 pieces of the row and adds them with vector reductions
// (red.global.add.v4.f32), so the transposed block is never built.  Summation order over a source row's edges is
// whatever the reductions land in: results agree with the transposed-CSC form up to fp32 rounding.
namespace f2c {
__device__ __forceinline__ void red_add_f4(float* p, float4 v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

template <typename IdxT, bool VEC4>
__global__ void __launch_bounds__(256) spmm_backward_kernel(const float* __restrict__ grad_out, float* __restrict__ grad_src,
                                                            const IdxT* __restrict__ indptr, const IdxT* __restrict__ indices,
                                                            int64_t n_dst, int feat_dim, int reduce) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t d = warp; d < n_dst; d += n_warps) {
    const int64_t begin = (int64_t)indptr[d], end = (int64_t)indptr[d + 1];
    if (end == begin) continue;
    const float w = reduce == F2C_MEAN ? 1.0f / (float)(end - begin) : 1.0f;
    if (VEC4) {
      for (int c = lane * 4; c < feat_dim; c += 128) {
        float4 g = *reinterpret_cast<const float4*>(grad_out + d * feat_dim + c);
        g.x *= w; g.y *= w; g.z *= w; g.w *= w;
        for (int64_t k = begin; k < end; ++k) red_add_f4(grad_src + (int64_t)indices[k] * feat_dim + c, g);
      }
    } else {
      for (int c = lane; c < feat_dim; c += 32) {
        const float g = grad_out[d * feat_dim + c] * w;
        for (int64_t k = begin; k < end; ++k) atomicAdd(grad_src + (int64_t)indices[k] * feat_dim + c, g);
      }
    }
  }
}
}  // namespace f2c

extern "C" int f2c_spmm_csr_backward(const float* grad_out, const void* indptr, const void* indices, int index_dtype,
                                     float* grad_src, int64_t n_dst, int64_t n_src, int64_t feat_dim, int reduce, void* stream) {
  F2C_REQUIRE(n_dst >= 0 && n_src >= 0 && feat_dim >= 0, F2C_ERR_INVALID, "spmm_csr_backward: negative size");
  F2C_REQUIRE(is_index_dtype(index_dtype), F2C_ERR_UNSUPPORTED, "spmm_csr_backward: indptr/indices must be int32 or int64");
  F2C_REQUIRE(reduce == F2C_MEAN || reduce == F2C_SUM, F2C_ERR_INVALID, "spmm_csr_backward: reduce must be mean or sum");
  F2C_REQUIRE(feat_dim < (1ll << 24), F2C_ERR_LIMIT, "spmm_csr_backward: feat_dim too large");
  if (n_src * feat_dim == 0) return F2C_OK;
  F2C_REQUIRE(grad_src != nullptr && (n_dst * feat_dim == 0 || (grad_out && indptr)), F2C_ERR_INVALID, "spmm_csr_backward: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(grad_src, 0, (size_t)n_src * feat_dim * sizeof(float), st);
  if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "spmm_csr_backward: %s", cudaGetErrorString(e));
  if (n_dst == 0) return F2C_OK;
  int64_t blocks = ceil_div(n_dst, 8);
  if (blocks > current_sm_count() * 16) blocks = current_sm_count() * 16;
  const bool vec = feat_dim % 4 == 0 && aligned(grad_out, 16) && aligned(grad_src, 16);
#define F2C_BW(T, V) spmm_backward_kernel<T, V><<<(unsigned)blocks, 256, 0, st>>>(grad_out, grad_src, (const T*)indptr, (const T*)indices, n_dst, (int)feat_dim, reduce)
  if (index_dtype == F2C_I32) { if (vec) F2C_BW(int32_t, true); else F2C_BW(int32_t, false); }
  else { if (vec) F2C_BW(int64_t, true); else F2C_BW(int64_t, false); }
#undef F2C_BW
  return check_launch("spmm_csr_backward");
}

// ---------------------------------------------------------------- CSC sanity check (debug helper)
namespace f2c {
template <typename IdxT>
__global__ void __launch_bounds__(256) check_csc_kernel(const IdxT* __restrict__ indptr, const IdxT* __restrict__ indices,
                                                        int64_t n_dst, int64_t n_src, int32_t* __restrict__ flag) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (tid == 0 && (int64_t)indptr[0] != 0) atomicOr(flag, 1);
  for (int64_t d = tid; d < n_dst; d += stride)
    if ((int64_t)indptr[d + 1] < (int64_t)indptr[d]) atomicOr(flag, 2);
  const int64_t nnz = (int64_t)indptr[n_dst];
  for (int64_t e = tid; e < nnz; e += stride) {
    int64_t v = (int64_t)indices[e];
    if (v < 0 || v >= n_src) atomicOr(flag, 4);
  }
}
}  // namespace f2c

extern "C" int f2c_check_csc(const void* indptr, const void* indices, int index_dtype, int64_t n_dst, int64_t n_src,
                             int32_t* flag_device, void* stream) {
  F2C_REQUIRE(n_dst >= 0 && n_src >= 0, F2C_ERR_INVALID, "check_csc: negative size");
  F2C_REQUIRE(is_index_dtype(index_dtype), F2C_ERR_UNSUPPORTED, "check_csc: indptr/indices must be int32 or int64");
  F2C_REQUIRE(indptr && flag_device, F2C_ERR_INVALID, "check_csc: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(flag_device, 0, sizeof(int32_t), st);
  if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "check_csc: %s", cudaGetErrorString(e));
  unsigned grid = (unsigned)current_sm_count() * 8;
  if (index_dtype == F2C_I32)
    check_csc_kernel<int32_t><<<grid, 256, 0, st>>>((const int32_t*)indptr, (const int32_t*)indices, n_dst, n_src, flag_device);
  else
    check_csc_kernel<int64_t><<<grid, 256, 0, st>>>((const int64_t*)indptr, (const int64_t*)indices, n_dst, n_src, flag_device);
  return check_launch("check_csc");
}
