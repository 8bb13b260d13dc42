// K-means assignment on the 5th-generation tensor cores (tcgen05, TMEM accumulators).
// Reference operator: KMeans.predict (src/kmeans.cu:77-98, RAFT kmeans_predict), i.e.
// labels[i] = first argmin_c dist(x_i, y_c) with dist = squared L2 or cosine distance.
//
// The n*k*d contraction S = X * Y^T is the only dense GEMM on the path, so it runs as
// tcgen05.mma.kind::tf32 with M = 128 points per tile, N = all (<= 256) centres, accumulators in TMEM
// (256 columns), operands in shared memory in the canonical no-swizzle K-major layout.  TF32 keeps 10
// mantissa bits, which would flip near ties, so both operands are split x = hi + lo (hi = top 19
// bits) and the products hi*hi + lo*hi + hi*lo are obtained in ONE GEMM by concatenating along K:
//     A' = [x_hi | x_lo | x_hi]   B' = [y_hi | y_hi | y_lo]      (K = 3d)
// which is fp32-accurate to ~2^-19.  For d > 32 (operands would not fit in shared memory) a single
// TF32 pass is used with a proportionally wider tolerance.  The epilogue reads the 128 x 256 scores
// with tcgen05.ld (one point per thread), forms  |y_c|^2 - 2 S  (L2)  or  -S / |y_c|  (cosine), and
// keeps the best and second best score.  A point whose two best scores are closer than the error
// bound of the split product is NOT decided here: its index is appended to a scratch list and the
// exact fp32 scorer (kmeans.cu) assigns it afterwards, so every label equals the label of the exact
// fp32 kernel.
//
// Shape of a CTA: 128 threads = 4 warps; thread t owns point t of the tile when loading / splitting
// the A tile and TMEM lane t in the epilogue; thread 0 issues the MMAs.  Centres are staged once per
// persistent CTA.  Every wait on the MMA-completion mbarrier is bounded; on expiry the CTA records
// an error code, frees its TMEM and returns.
#include <mutex>

#include "common.cuh"

namespace f2c {

int kmeans_assign_exact(const float* x, const float* y, int64_t* labels, const int32_t* subset, int64_t n, int64_t k, int64_t d,
                        int metric, cudaStream_t st);
int kmeans_assign_exact_listed(const float* x, const float* y, int64_t* labels, const int32_t* list, const int32_t* count_dev,
                               int64_t max_count, int64_t k, int64_t d, int metric, cudaStream_t st);

namespace tc {

constexpr int kTileM = 128;
constexpr int kMaxN = 256;
constexpr uint32_t kWaitLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Shared-memory matrix descriptor, K-major, no swizzle: element (row r, 16-byte K chunk c) lives at
// start + (r % 8) * 16 + (r / 8) * SBO + c * LBO.
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint32_t lo = ((addr & 0x3FFFFu) >> 4) | ((lbo >> 4) << 16);
  uint32_t hi = (sbo >> 4) | (1u << 14);  // bits 46-47: descriptor version 1 (sm_100); layout type 0 = no swizzle
  return ((uint64_t)hi << 32) | lo;
}

__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
      "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

struct Params {
  const float* x;
  const float* y;
  int64_t* labels;
  int32_t* amb_list;   // scratch: indices of undecided points
  int32_t* amb_count;  // scratch: their number
  int32_t* error;      // scratch: non-zero when a bounded wait expired
  int64_t n;
  int k, d;
  int dp;      // d padded to a multiple of 8
  int terms;   // 3: split product, 1: plain TF32
  int n_pad;   // k padded to a multiple of 16 (MMA N)
  int metric;
  float eps;   // relative error bound of one score
};

// Shared memory: [B tile][A tile][cnorm 256 floats][mbarrier 8 B][tmem slot 4 B]
__global__ void __launch_bounds__(128) kmeans_tc_kernel(const Params p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5;
  const int kc = p.terms * p.dp / 4;                 // 16-byte K chunks per operand row
  const uint32_t lbo_b = kMaxN * 16, lbo_a = kTileM * 16, sbo = 128;
  unsigned char* b_tile = smem;
  unsigned char* a_tile = smem + (size_t)kc * lbo_b;
  float* cnorm = reinterpret_cast<float*>(a_tile + (size_t)kc * lbo_a);
  uint64_t* mbar = reinterpret_cast<uint64_t*>(cnorm + kMaxN);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mbar + 1);

  // ---- one-time setup: TMEM, mbarrier, centre tile ----
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(mbar)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // centres: rows c = tid, tid + 128; padded rows / columns are zero; norm of padded rows = +inf (never chosen)
  for (int c = tid; c < kMaxN; c += 128) {
    float nrm = 0.0f;
    for (int g = 0; g < p.dp / 4; ++g) {
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int t = 4 * g + e;
        v[e] = (c < p.k && t < p.d) ? __ldg(p.y + (int64_t)c * p.d + t) : 0.0f;
        nrm = fmaf(v[e], v[e], nrm);
      }
      float4 hi, lo;
      hi.x = __uint_as_float(__float_as_uint(v[0]) & 0xFFFFE000u); lo.x = v[0] - hi.x;
      hi.y = __uint_as_float(__float_as_uint(v[1]) & 0xFFFFE000u); lo.y = v[1] - hi.y;
      hi.z = __uint_as_float(__float_as_uint(v[2]) & 0xFFFFE000u); lo.z = v[2] - hi.z;
      hi.w = __uint_as_float(__float_as_uint(v[3]) & 0xFFFFE000u); lo.w = v[3] - hi.w;
      const int G = p.dp / 4;
      if (p.terms == 3) {  // B' = [y_hi | y_hi | y_lo]
        *reinterpret_cast<float4*>(b_tile + (size_t)(g) * lbo_b + c * 16) = hi;
        *reinterpret_cast<float4*>(b_tile + (size_t)(G + g) * lbo_b + c * 16) = hi;
        *reinterpret_cast<float4*>(b_tile + (size_t)(2 * G + g) * lbo_b + c * 16) = lo;
      } else {
        *reinterpret_cast<float4*>(b_tile + (size_t)g * lbo_b + c * 16) = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
    if (p.metric == F2C_L2) cnorm[c] = c < p.k ? nrm : INFINITY;
    else cnorm[c] = c < p.k ? (nrm > 0.0f ? 1.0f / sqrtf(nrm) : 0.0f) : 0.0f;  // cosine: 1/|y_c|
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  // largest centre norm (tolerance of the L2 score)
  float cmax = 0.0f;
  if (p.metric == F2C_L2)
    for (int c = 0; c < p.k; ++c) cmax = fmaxf(cmax, cnorm[c]);
  cmax = sqrtf(cmax);

  const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p.n_pad >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
  const int ksteps = p.terms * p.dp / 8;  // one MMA consumes 8 tf32 = two 16-byte chunks of K
  uint32_t parity = 0;
  bool failed = false;

  const int64_t n_tiles = (p.n + kTileM - 1) / kTileM;
  for (int64_t tile = blockIdx.x; tile < n_tiles && !failed; tile += gridDim.x) {
    // ---- A tile: thread t loads, splits and stores point tile*128 + t ----
    const int64_t i = tile * kTileM + tid;
    float xx = 0.0f;
    for (int g = 0; g < p.dp / 4; ++g) {
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int t = 4 * g + e;
        v[e] = (i < p.n && t < p.d) ? __ldg(p.x + i * p.d + t) : 0.0f;
        xx = fmaf(v[e], v[e], xx);
      }
      float4 hi, lo;
      hi.x = __uint_as_float(__float_as_uint(v[0]) & 0xFFFFE000u); lo.x = v[0] - hi.x;
      hi.y = __uint_as_float(__float_as_uint(v[1]) & 0xFFFFE000u); lo.y = v[1] - hi.y;
      hi.z = __uint_as_float(__float_as_uint(v[2]) & 0xFFFFE000u); lo.z = v[2] - hi.z;
      hi.w = __uint_as_float(__float_as_uint(v[3]) & 0xFFFFE000u); lo.w = v[3] - hi.w;
      const int G = p.dp / 4;
      if (p.terms == 3) {  // A' = [x_hi | x_lo | x_hi]
        *reinterpret_cast<float4*>(a_tile + (size_t)(g) * lbo_a + tid * 16) = hi;
        *reinterpret_cast<float4*>(a_tile + (size_t)(G + g) * lbo_a + tid * 16) = lo;
        *reinterpret_cast<float4*>(a_tile + (size_t)(2 * G + g) * lbo_a + tid * 16) = hi;
      } else {
        *reinterpret_cast<float4*>(a_tile + (size_t)g * lbo_a + tid * 16) = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();  // A tile complete; every warp has finished reading the previous tile's accumulators
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // ---- S = A' * B'^T into TMEM ----
    if (tid == 0) {
      const uint32_t a_addr = smem_u32(a_tile), b_addr = smem_u32(b_tile);
      for (int s = 0; s < ksteps; ++s) {
        const uint64_t a_desc = make_desc(a_addr + (uint32_t)s * 2u * lbo_a, lbo_a, sbo);
        const uint64_t b_desc = make_desc(b_addr + (uint32_t)s * 2u * lbo_b, lbo_b, sbo);
        mma_tf32(tmem_base, a_desc, b_desc, idesc, s > 0 ? 1u : 0u);
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(mbar)) : "memory");
    }
    // ---- bounded wait for the MMAs ----
    uint32_t done = 0;
    for (uint32_t it = 0; it < kWaitLimit && !done; ++it) {
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}\n"
          : "=r"(done) : "r"(smem_u32(mbar)), "r"(parity) : "memory");
    }
    parity ^= 1u;
    if (__syncthreads_or(done == 0)) {  // somebody gave up: record it and leave through the common exit
      if (tid == 0) atomicExch(p.error, 1 + (int)((tile - blockIdx.x) / gridDim.x));  // 1 + how many tiles this CTA had finished
      failed = true;
      break;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // ---- epilogue: thread t = TMEM lane t = point i ----
    float best = INFINITY, second = INFINITY;
    int best_c = 0;
    bool odd = false;  // NaN seen: let the exact scorer decide
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
    for (int c0 = 0; c0 < p.n_pad; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(lane_addr + (uint32_t)c0, r);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int c = c0 + j;
        const float s = __uint_as_float(r[j]);
        const float score = p.metric == F2C_L2 ? fmaf(-2.0f, s, cnorm[c]) : -s * cnorm[c];
        if (c < p.k) {
          odd |= !(score == score);
          if (score < best) { second = best; best = score; best_c = c; }
          else if (score < second) second = score;
        }
      }
    }
    if (i < p.n) {
      const float xn = sqrtf(xx);
      // error bound of a score: L2  2*eps*|x||y|max ;  cosine  eps*|x|
      const float tol = p.metric == F2C_L2 ? 2.0f * p.eps * xn * cmax : p.eps * xn;
      if (odd || !(second - best > 2.0f * tol)) {
        const int slot = atomicAdd(p.amb_count, 1);
        p.amb_list[slot] = (int32_t)i;
      } else {
        p.labels[i] = best_c;
      }
    }
  }

  // ---- common exit: all TMEM reads retired, then the allocating warp frees the columns ----
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
  }
}

}  // namespace tc

// Eligibility and scratch size of the tensor-core path.
bool kmeans_tc_supported(int64_t n, int64_t k, int64_t d) { return n >= 1 && n < (1ll << 31) && k >= 1 && k <= tc::kMaxN && d >= 1 && d <= 64; }
int64_t kmeans_tc_workspace(int64_t n) { return 256 + 4 * n; }  // [count, error, pad][index list]

int kmeans_assign_tc(const float* x, const float* y, int64_t* labels, int64_t n, int64_t k, int64_t d, int metric, void* workspace,
                     cudaStream_t st) {
  tc::Params p{};
  p.x = x; p.y = y; p.labels = labels; p.n = n; p.k = (int)k; p.d = (int)d; p.metric = metric;
  p.dp = (int)((d + 7) / 8 * 8);
  p.terms = p.dp <= 32 ? 3 : 1;
  p.n_pad = (int)((k + 15) / 16 * 16);
  p.eps = p.terms == 3 ? 1.0f / 65536.0f : 1.0f / 256.0f;  // 2^-16 (split product, true error ~2^-18.4) or 2^-8 (plain TF32)
  int32_t* head = reinterpret_cast<int32_t*>(workspace);
  p.amb_count = head; p.error = head + 1; p.amb_list = head + 64;
  cudaError_t e = cudaMemsetAsync(head, 0, 256, st);
  if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "kmeans_assign: %s", cudaGetErrorString(e));
  const int kc = p.terms * p.dp / 4;
  size_t smem = (size_t)kc * (tc::kMaxN + tc::kTileM) * 16 + tc::kMaxN * 4 + 16;
  e = cudaFuncSetAttribute(tc::kmeans_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "kmeans_assign: %s", cudaGetErrorString(e));
  int64_t tiles = ceil_div(n, tc::kTileM);
  int per_sm = smem <= 100 * 1024 ? 2 : 1;  // two CTAs share the 512 TMEM columns of an SM
  int64_t grid = tiles < (int64_t)kSmCount * per_sm ? tiles : (int64_t)kSmCount * per_sm;
  tc::kmeans_tc_kernel<<<(unsigned)grid, 128, smem, st>>>(p);
  int rc = check_launch("kmeans_assign (tensor cores)");
  if (rc) return rc;
  // undecided points: exact fp32 scorer over the device-side list
  return kmeans_assign_exact_listed(x, y, labels, p.amb_list, p.amb_count, n, k, d, metric, st);
}

// ------------------------------------------------------------------------------------------------------
// K-means assignment for callers that cannot allocate device memory.
//
// f2c_kmeans_assign leaves the undecided-point list to the caller, which means one device allocation per
// call (or a buffer the caller has to carry around).  Some callers cannot do that: a data-loader or serving
// thread that lives inside a process whose framework allocator already owns almost all of HBM (a raw
// cudaMalloc there can fail, or make the framework drop its cache), and callers on a latency-critical
// path, where cudaMalloc / cudaFree would stall every stream of the device.  For them the scratch lives in
// a fixed array in the library's device image: 4 MiB + 256 B on every GPU that loads the library, held until
// the process exits, enough for kStaticMaxPoints points per call.
//
// The array's name below is only a host-side handle; the device address is obtained once per device with
// cudaGetSymbolAddress while that device is current.  That happens on the first call made on a device (a
// synchronising runtime query, once).  All calls on a device share the one array: the header is
// cleared at the start of every call, the list behind it keeps whatever the previous call left and is only
// read up to the new count.  Two calls that overlap on the GPU (different streams, or threads) would
// overwrite each other's list - serialise them.
namespace tc {
constexpr int64_t kStaticMaxPoints = 1 << 20;
static __device__ __align__(256) unsigned char g_static_scratch[256 + 4 * kStaticMaxPoints];
}  // namespace tc
}  // namespace f2c

extern "C" int f2c_kmeans_assign_static(const float* x, const float* centers, int64_t* labels, int64_t n, int64_t k,
                                        int64_t d, int metric, void* stream) {
  using namespace f2c;
  const char* op = "kmeans_assign_static";
  F2C_REQUIRE(n >= 0 && k >= 1 && d >= 1, F2C_ERR_INVALID, "%s: bad shape n=%lld k=%lld d=%lld", op, (long long)n, (long long)k,
              (long long)d);
  F2C_REQUIRE(metric == F2C_L2 || metric == F2C_COSINE, F2C_ERR_INVALID, "%s: unknown metric", op);
  F2C_REQUIRE(n <= tc::kStaticMaxPoints, F2C_ERR_LIMIT,
              "%s: %lld points exceed the %lld the built-in scratch holds; split the call or use kmeans_assign with a workspace", op,
              (long long)n, (long long)tc::kStaticMaxPoints);
  F2C_REQUIRE(k <= tc::kMaxN && d <= 64, F2C_ERR_LIMIT, "%s: at most %d centres of at most 64 dimensions", op, tc::kMaxN);
  if (n == 0) return F2C_OK;
  F2C_REQUIRE(x && centers && labels, F2C_ERR_INVALID, "%s: null pointer", op);

  // device address of the scratch array, looked up once per device (with that device current)
  static std::mutex mu;
  static void* scratch_of_device[64] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) return set_error(F2C_ERR_CUDA, "%s: cudaGetDevice: %s", op, cudaGetErrorString(e));
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (scratch_of_device[dev] == nullptr) {
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, tc::g_static_scratch);
      if (e != cudaSuccess || ptr == nullptr) return set_error(F2C_ERR_CUDA, "%s: cudaGetSymbolAddress: %s", op, cudaGetErrorString(e));
      scratch_of_device[dev] = ptr;
    }
    scratch = scratch_of_device[dev];
  }
  // same kernels as kmeans_assign; the header (count, error code) is cleared inside
  return kmeans_assign_tc(x, centers, labels, n, k, d, metric, scratch, (cudaStream_t)stream);
}

