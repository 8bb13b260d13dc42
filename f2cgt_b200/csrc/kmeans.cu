// K-means distance matrix and assignment in fp32 CUDA cores
// (reference operators pairwise_distance / KMeans.predict, src/kmeans.cu:77-118, which wrap RAFT
// 23.10; semantics as restated by the reference in examples/my_kmeans.py:43-64,116-125):
//   L2      dist[i,c] = sum_t (x[i,t] - y[c,t])^2           (no square root)
//   cosine  dist[i,c] = 1 - <x_i, y_c> / (|x_i| |y_c|)      (1 when a norm is zero)
//   label[i] = first argmin_c dist[i,c]; a NaN distance counts as 1 (examples/my_kmeans.py:92-94)
//
// Two mappings:
//  * warp-per-point (any d, any k): lanes stride over the centres, x_i is broadcast; writes the
//    distance matrix with coalesced rows and/or reduces the argmin in the warp.  pairwise_distance is
//    bound by its n*k*4-byte output.
//  * thread-per-point (d <= 128): x_i lives in registers, centres are broadcast from shared memory
//    with 128-bit reads, four FMAs per read.  This is the exact fp32 scorer; the tensor-core kernel
//    (kmeans_tc.cu) uses it to re-score the points whose best two candidates are too close to call.
#include "common.cuh"

namespace f2c {

__device__ __forceinline__ float finish_cosine(float dot, float xx, float cc) {
  float den = sqrtf(xx) * sqrtf(cc);
  return den > 0.0f ? 1.0f - dot / den : 1.0f;
}

// ---------------------------------------------------------------- warp per point
template <int METRIC, bool WRITE_DIST, bool WRITE_LABEL>
__global__ void __launch_bounds__(256) kmeans_warp_kernel(const float* __restrict__ x, const float* __restrict__ y,
                                                          float* __restrict__ dist, int64_t* __restrict__ labels, int64_t n,
                                                          int k, int d) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t i = warp; i < n; i += n_warps) {
    const float* xi = x + i * d;
    float xx = 0.0f;
    if (METRIC == F2C_COSINE)
      for (int t = 0; t < d; ++t) { float a = __ldg(xi + t); xx = fmaf(a, a, xx); }
    float best = INFINITY;
    int best_c = 0x7fffffff;
    for (int c = lane; c < k; c += 32) {
      const float* yc = y + (int64_t)c * d;
      float v;
      if (METRIC == F2C_L2) {
        float acc = 0.0f;
        for (int t = 0; t < d; ++t) { float df = __ldg(xi + t) - __ldg(yc + t); acc = fmaf(df, df, acc); }
        v = acc;
      } else {
        float dot = 0.0f, cc = 0.0f;
        for (int t = 0; t < d; ++t) { float a = __ldg(xi + t), b = __ldg(yc + t); dot = fmaf(a, b, dot); cc = fmaf(b, b, cc); }
        v = finish_cosine(dot, xx, cc);
      }
      if (WRITE_DIST) dist[i * k + c] = v;
      if (WRITE_LABEL) {
        if (v != v) v = 1.0f;
        if (v < best) { best = v; best_c = c; }
      }
    }
    if (WRITE_LABEL) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        float ob = __shfl_xor_sync(0xffffffffu, best, o);
        int oc = __shfl_xor_sync(0xffffffffu, best_c, o);
        if (ob < best || (ob == best && oc < best_c)) { best = ob; best_c = oc; }
      }
      if (lane == 0) labels[i] = best_c == 0x7fffffff ? 0 : best_c;
    }
  }
}

// ---------------------------------------------------------------- thread per point
// Centres are staged KC at a time as [KC][DMAX] (zero padded) plus their squared norms.
template <int DMAX, int METRIC>
__global__ void __launch_bounds__(256) kmeans_thread_kernel(const float* __restrict__ x, const float* __restrict__ y,
                                                            int64_t* __restrict__ labels, const int32_t* __restrict__ subset,
                                                            const int32_t* __restrict__ count_dev, int64_t n, int k, int d, int kc) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // count_dev != nullptr: the number of listed points is only known on the device; a small grid walks the list
  if (count_dev != nullptr) {
    const int64_t cnt = *count_dev;
    n = cnt < n ? cnt : n;
  }
  float* yc_s = reinterpret_cast<float*>(smem_raw);  // [kc][DMAX]
  float* cc_s = yc_s + (size_t)kc * DMAX;            // [kc]
  for (int64_t base = (int64_t)blockIdx.x * blockDim.x; base < n; base += (int64_t)gridDim.x * blockDim.x) {
  const int64_t slot = base + threadIdx.x;
  const bool valid = slot < n;
  // subset != nullptr: only the listed points are (re)scored
  const int64_t i = valid ? (subset ? (int64_t)subset[slot] : slot) : 0;
  float xr[DMAX];
  float xx = 0.0f;
#pragma unroll
  for (int t = 0; t < DMAX; ++t) {
    xr[t] = (valid && t < d) ? __ldg(x + i * d + t) : 0.0f;
    if (METRIC == F2C_COSINE) xx = fmaf(xr[t], xr[t], xx);
  }
  float best = INFINITY;
  int best_c = 0;
  for (int c0 = 0; c0 < k; c0 += kc) {
    const int nc = min(kc, k - c0);
    __syncthreads();
    for (int e = threadIdx.x; e < nc * DMAX; e += blockDim.x) {
      int c = e / DMAX, t = e - c * DMAX;
      yc_s[e] = t < d ? __ldg(y + (int64_t)(c0 + c) * d + t) : 0.0f;
    }
    __syncthreads();
    if (METRIC == F2C_COSINE) {
      for (int c = threadIdx.x; c < nc; c += blockDim.x) {
        float cc = 0.0f;
        for (int t = 0; t < DMAX; ++t) cc = fmaf(yc_s[c * DMAX + t], yc_s[c * DMAX + t], cc);
        cc_s[c] = cc;
      }
      __syncthreads();
    }
    for (int c = 0; c < nc; ++c) {
      const float4* yc4 = reinterpret_cast<const float4*>(yc_s + (size_t)c * DMAX);
      float acc = 0.0f;
#pragma unroll
      for (int q = 0; q < DMAX / 4; ++q) {
        float4 b = yc4[q];
        if (METRIC == F2C_L2) {
          float d0 = xr[4 * q] - b.x, d1 = xr[4 * q + 1] - b.y, d2 = xr[4 * q + 2] - b.z, d3 = xr[4 * q + 3] - b.w;
          acc = fmaf(d0, d0, acc); acc = fmaf(d1, d1, acc); acc = fmaf(d2, d2, acc); acc = fmaf(d3, d3, acc);
        } else {
          acc = fmaf(xr[4 * q], b.x, acc); acc = fmaf(xr[4 * q + 1], b.y, acc);
          acc = fmaf(xr[4 * q + 2], b.z, acc); acc = fmaf(xr[4 * q + 3], b.w, acc);
        }
      }
      float v = METRIC == F2C_L2 ? acc : finish_cosine(acc, xx, cc_s[c]);
      if (v != v) v = 1.0f;
      if (v < best) { best = v; best_c = c0 + c; }
    }
  }
  if (valid) labels[i] = best_c;
  }
}

template <int DMAX>
static int launch_thread_assign(const float* x, const float* y, int64_t* labels, const int32_t* subset, int64_t n, int64_t k,
                                int64_t d, int metric, cudaStream_t st, const int32_t* count_dev = nullptr) {
  int kc = (int)k;
  const size_t budget = 96 * 1024;
  while ((size_t)kc * (DMAX + 1) * sizeof(float) > budget) kc = (kc + 1) / 2;
  size_t smem = (size_t)kc * (DMAX + 1) * sizeof(float);
  unsigned grid = (unsigned)ceil_div(n, 256);
  if (count_dev != nullptr && grid > 2u * current_sm_count()) grid = 2u * current_sm_count();  // the list is short: a small grid walks it
  cudaError_t e;
  if (metric == F2C_COSINE) {
    auto kern = kmeans_thread_kernel<DMAX, F2C_COSINE>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) kern<<<grid, 256, smem, st>>>(x, y, labels, subset, count_dev, n, (int)k, (int)d, kc);
  } else {
    auto kern = kmeans_thread_kernel<DMAX, F2C_L2>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) kern<<<grid, 256, smem, st>>>(x, y, labels, subset, count_dev, n, (int)k, (int)d, kc);
  }
  if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "kmeans_assign: %s", cudaGetErrorString(e));
  return check_launch("kmeans_assign");
}

// Exact fp32 assignment of all points (subset == nullptr) or of the listed ones.
int kmeans_assign_exact(const float* x, const float* y, int64_t* labels, const int32_t* subset, int64_t n, int64_t k,
                        int64_t d, int metric, cudaStream_t st) {
  if (n == 0) return F2C_OK;
  if (d <= 8) return launch_thread_assign<8>(x, y, labels, subset, n, k, d, metric, st);
  if (d <= 16) return launch_thread_assign<16>(x, y, labels, subset, n, k, d, metric, st);
  if (d <= 32) return launch_thread_assign<32>(x, y, labels, subset, n, k, d, metric, st);
  if (d <= 64) return launch_thread_assign<64>(x, y, labels, subset, n, k, d, metric, st);
  if (d <= 128) return launch_thread_assign<128>(x, y, labels, subset, n, k, d, metric, st);
  if (subset != nullptr) return set_error(F2C_ERR_UNSUPPORTED, "kmeans_assign: subset re-scoring needs d <= 128");
  int64_t blocks = ceil_div(n, 8);
  if (blocks > current_sm_count() * 32) blocks = current_sm_count() * 32;
  if (metric == F2C_COSINE)
    kmeans_warp_kernel<F2C_COSINE, false, true><<<(unsigned)blocks, 256, 0, st>>>(x, y, nullptr, labels, n, (int)k, (int)d);
  else
    kmeans_warp_kernel<F2C_L2, false, true><<<(unsigned)blocks, 256, 0, st>>>(x, y, nullptr, labels, n, (int)k, (int)d);
  return check_launch("kmeans_assign");
}

// Exact assignment of the points listed in `list`; their number sits in device memory (*count_dev <= max_count).
int kmeans_assign_exact_listed(const float* x, const float* y, int64_t* labels, const int32_t* list, const int32_t* count_dev,
                               int64_t max_count, int64_t k, int64_t d, int metric, cudaStream_t st) {
  if (max_count == 0) return F2C_OK;
  if (d <= 8) return launch_thread_assign<8>(x, y, labels, list, max_count, k, d, metric, st, count_dev);
  if (d <= 16) return launch_thread_assign<16>(x, y, labels, list, max_count, k, d, metric, st, count_dev);
  if (d <= 32) return launch_thread_assign<32>(x, y, labels, list, max_count, k, d, metric, st, count_dev);
  if (d <= 64) return launch_thread_assign<64>(x, y, labels, list, max_count, k, d, metric, st, count_dev);
  if (d <= 128) return launch_thread_assign<128>(x, y, labels, list, max_count, k, d, metric, st, count_dev);
  return set_error(F2C_ERR_UNSUPPORTED, "kmeans_assign: listed re-scoring needs d <= 128");
}

bool kmeans_tc_supported(int64_t n, int64_t k, int64_t d);
int64_t kmeans_tc_workspace(int64_t n);
int kmeans_assign_tc(const float* x, const float* y, int64_t* labels, int64_t n, int64_t k, int64_t d, int metric, void* workspace,
                     cudaStream_t st);

static int validate_km(const char* op, int64_t n, int64_t k, int64_t d, int metric) {
  F2C_REQUIRE(n >= 0 && k >= 1 && d >= 1, F2C_ERR_INVALID, "%s: bad shape n=%lld k=%lld d=%lld", op, (long long)n, (long long)k,
              (long long)d);
  F2C_REQUIRE(metric == F2C_L2 || metric == F2C_COSINE, F2C_ERR_INVALID, "%s: unknown metric", op);
  F2C_REQUIRE(k < (1ll << 24) && d < (1ll << 20), F2C_ERR_LIMIT, "%s: k or d too large", op);
  return F2C_OK;
}

}  // namespace f2c

using namespace f2c;

extern "C" int f2c_pairwise_distance(const float* x, const float* y, float* dist, int64_t n, int64_t k, int64_t d, int metric,
                                     void* stream) {
  int rc = validate_km("pairwise_distance", n, k, d, metric);
  if (rc) return rc;
  if (n == 0) return F2C_OK;
  F2C_REQUIRE(x && y && dist, F2C_ERR_INVALID, "pairwise_distance: null pointer");
  int64_t blocks = ceil_div(n, 8);
  if (blocks > current_sm_count() * 32) blocks = current_sm_count() * 32;
  cudaStream_t st = (cudaStream_t)stream;
  if (metric == F2C_COSINE)
    kmeans_warp_kernel<F2C_COSINE, true, false><<<(unsigned)blocks, 256, 0, st>>>(x, y, dist, nullptr, n, (int)k, (int)d);
  else
    kmeans_warp_kernel<F2C_L2, true, false><<<(unsigned)blocks, 256, 0, st>>>(x, y, dist, nullptr, n, (int)k, (int)d);
  return check_launch("pairwise_distance");
}

extern "C" int64_t f2c_kmeans_assign_workspace(int64_t n, int64_t k, int64_t d) {
  return kmeans_tc_supported(n, k, d) ? kmeans_tc_workspace(n) : 0;
}

extern "C" int f2c_kmeans_assign(const float* x, const float* centers, int64_t* labels, int64_t n, int64_t k, int64_t d,
                                 int metric, void* workspace, void* stream) {
  const int scorer = metric & (F2C_SCORER_EXACT | F2C_SCORER_TENSOR);  // per-call choice of the scorer (tests, benchmarks)
  metric &= ~(F2C_SCORER_EXACT | F2C_SCORER_TENSOR);
  int rc = validate_km("kmeans_assign", n, k, d, metric);
  if (rc) return rc;
  if (n == 0) return F2C_OK;
  F2C_REQUIRE(x && centers && labels, F2C_ERR_INVALID, "kmeans_assign: null pointer");
  // tensor-core path when a scratch buffer is supplied and the shape fits; the exact fp32 scorer otherwise
  // (measured on B200 with 256 centres: the tensor-core path is faster from d = 8 up for both metrics; below that
  //  the CUDA-core scorer reads so little per point that the 128-point tiles only add latency)
  const bool prefer_tc = d >= 8 || scorer == F2C_SCORER_TENSOR;
  if (workspace != nullptr && kmeans_tc_supported(n, k, d) && prefer_tc && scorer != F2C_SCORER_EXACT && aligned(workspace, 16))
    return kmeans_assign_tc(x, centers, labels, n, k, d, metric, workspace, (cudaStream_t)stream);
  return kmeans_assign_exact(x, centers, labels, nullptr, n, k, d, metric, (cudaStream_t)stream);
}
