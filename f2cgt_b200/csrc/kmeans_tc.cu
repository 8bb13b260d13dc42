// K-means assignment on the 5th-generation tensor cores (tcgen05, TMEM accumulators).
// Reference operator: KMeans.predict (src/kmeans.cu:77-98, RAFT kmeans_predict), i.e.
// labels[i] = first argmin_c dist(x_i, y_c) with dist = squared L2 or cosine distance.
//
// The n*k*d contraction S = X * Y^T is the only dense GEMM on the path, so it runs as
// tcgen05.mma.kind::tf32 with M = 128 points per tile, N = all (<= 256) centres, accumulators in TMEM,
// operands in shared memory in the canonical no-swizzle K-major layout.
//
//  * Accuracy.  TF32 keeps 10 mantissa bits, which would flip near ties, so both operands are split
//    x = hi + lo (hi = top 19 bits) and the products hi*hi + lo*hi + hi*lo are obtained in ONE GEMM by
//    concatenating along K:  A' = [x_hi | x_lo | x_hi],  B' = [y_hi | y_hi | y_lo]  (K = 3d), which is
//    fp32-accurate to ~2^-19.  For 32 < d <= 64 those operands would not fit in shared memory; there the split is
//    into bf16 pairs x = b1 + b2 (+ a rest below 2^-18 |x|) with the same concatenation on kind::f16
//    (half the bytes per value), accurate to ~2^-16.
//  * The whole score comes out of the GEMM.  argmin_c |y_c|^2 - 2 x.y_c = argmax_c (x.y_c - |y_c|^2 / 2): one
//    more K step carries [1, 1, 0...] on the point side and the split of -|y_c|^2/2 on the centre side
//    (cosine: the centre rows are pre-scaled by 1/|y_c| instead), so the epilogue is a pure running
//    arg-max - five instructions per (point, centre) - with no per-centre term to fetch.
//  * The epilogue reads the 128 x 256 scores with tcgen05.ld (one point per thread) and keeps the best and
//    second best score.  A point whose two best scores are closer than the error bound of the product is
//    NOT decided here: its index is appended to a scratch list and the exact fp32 scorer (kmeans.cu)
//    assigns it afterwards, so every label equals the label of the exact fp32 kernel.
//  * Overlap.  A CTA is two groups of eight warps that share the staged centre tile; each group has its own
//    point tile, mbarrier and 256 TMEM columns and runs load -> MMA -> epilogue on alternate tiles, so the
//    tensor pipe works on one group's tile while the other group is in its epilogue.  A point of the tile
//    belongs to two threads of its group (same TMEM lane, warps w and w + 4): they load and split alternate
//    chunks of its row and scan one half of the centres each - the epilogue, not the MMA, is what the kernel
//    spends its issue slots on, and twice the warps fill them better.  The group's first thread issues the
//    MMAs.  Every wait on an MMA-completion mbarrier is bounded; on expiry the group records an error code
//    and leaves, and the CTA frees its TMEM at the common exit.
#include <mutex>

#include <cuda_bf16.h>

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

__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
      "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

// x = b1 + b2 + (rest below 2^-18 |x|) with b1, b2 bf16 (round to nearest): eight values -> two 16-byte chunks
__device__ __forceinline__ void split8_bf16(const float (&v)[8], uint4& c1, uint4& c2) {
  uint32_t w1[4], w2[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const __nv_bfloat16 a1 = __float2bfloat16_rn(v[2 * e]), b1 = __float2bfloat16_rn(v[2 * e + 1]);
    const __nv_bfloat16 a2 = __float2bfloat16_rn(v[2 * e] - __bfloat162float(a1));
    const __nv_bfloat16 b2 = __float2bfloat16_rn(v[2 * e + 1] - __bfloat162float(b1));
    w1[e] = (uint32_t)__bfloat16_as_ushort(a1) | ((uint32_t)__bfloat16_as_ushort(b1) << 16);
    w2[e] = (uint32_t)__bfloat16_as_ushort(a2) | ((uint32_t)__bfloat16_as_ushort(b2) << 16);
  }
  c1 = make_uint4(w1[0], w1[1], w1[2], w1[3]);
  c2 = make_uint4(w2[0], w2[1], w2[2], w2[3]);
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

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
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
  int bf16;    // 1: operands are bf16 pairs (x = b1 + b2), A' = [x1 | x2 | x1], B' = [y1 | y1 | y2], kind::f16 (32 < d <= 64)
  int n_pad;   // k padded to a multiple of 32 (epilogue reads 32 columns at a time; MMA N needs 16)
  int metric;
  int vec4;    // rows of x can be read as float4
  float eps;   // relative error bound of one score
};

constexpr int kGroupThreads = 256;  // two threads per point of the tile
constexpr int kCtaThreads = 2 * kGroupThreads;

__device__ __forceinline__ void group_sync(int g) { asm volatile("bar.sync %0, 256;" ::"r"(g + 1) : "memory"); }

__device__ __forceinline__ void split4(const float (&v)[4], float4& hi, float4& lo) {
  hi.x = __uint_as_float(__float_as_uint(v[0]) & 0xFFFFE000u); lo.x = v[0] - hi.x;
  hi.y = __uint_as_float(__float_as_uint(v[1]) & 0xFFFFE000u); lo.y = v[1] - hi.y;
  hi.z = __uint_as_float(__float_as_uint(v[2]) & 0xFFFFE000u); lo.z = v[2] - hi.z;
  hi.w = __uint_as_float(__float_as_uint(v[3]) & 0xFFFFE000u); lo.w = v[3] - hi.w;
}

// running (best, second best, index of best) over a stream of scores, larger = better
struct Top2 {
  float best, second;
  int idx;
  __device__ __forceinline__ void init() { best = -INFINITY; second = -INFINITY; idx = 0; }
  __device__ __forceinline__ void push(float s, int c) {
    const bool gt = s > best;
    second = gt ? best : fmaxf(second, s);
    idx = gt ? c : idx;
    best = gt ? s : best;
  }
  __device__ __forceinline__ void merge(const Top2& o) {
    const bool gt = o.best > best || (o.best == best && o.idx < idx);
    second = gt ? fmaxf(best, o.second) : fmaxf(second, o.best);
    idx = gt ? o.idx : idx;
    best = gt ? o.best : best;
  }
};

// Shared memory: [B tile][A tile group 0][A tile group 1][scratch 256 floats][exchange 2 x 128 x 16 B][2 mbarriers]
// [tmem slot][2 fail flags][2 x 128 floats |x|^2]
template <bool BF16>
__global__ void __launch_bounds__(kCtaThreads, 1) kmeans_tc_kernel(const Params p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x;
  const int g = tid >> 8;            // group
  const int lt = tid & 255;          // thread within the group
  const int pt = lt & 127;           // its point of the tile = its TMEM lane
  const int half = lt >> 7;          // which half of the row's K chunks it loads and which half of the centres it scans
  const int lane_quarter = (lt >> 5) & 3;
  // 16-byte K chunks per operand row (the last two carry the norm term): 4 tf32 or 8 bf16 values per chunk
  const int kc_x = BF16 ? 3 * p.dp / 8 : p.terms * p.dp / 4;
  const int kc = kc_x + 2;
  const uint32_t lbo_b = kMaxN * 16, lbo_a = kTileM * 16, sbo = 128;
  unsigned char* b_tile = smem;
  unsigned char* a_tile = smem + (size_t)kc * lbo_b + (size_t)g * kc * lbo_a;
  float* scratch = reinterpret_cast<float*>(smem + (size_t)kc * lbo_b + (size_t)2 * kc * lbo_a);
  float4* exch = reinterpret_cast<float4*>(scratch + kMaxN) + g * kTileM;  // (best, second, index, |x|^2 part) of half 1
  uint64_t* mbar = reinterpret_cast<uint64_t*>(scratch + kMaxN + 2 * kTileM * 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mbar + 2);
  volatile uint32_t* fail = tmem_slot + 1;
  float* xx_s = reinterpret_cast<float*>(mbar + 8) + g * kTileM;  // |x|^2 of the tile's points (bf16 path)

  // ---- one-time setup: TMEM (all 512 columns: 256 per group), mbarriers, centre tile ----
  if (tid < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(mbar)) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(mbar + 1)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fail[0] = 0u; fail[1] = 0u;
  }
  // centre c = tid (first 256 threads, 256 rows); padded rows are zero with a norm term that never wins
  if (tid < kMaxN) {
    const int c = tid;
    const int G = p.dp / 4;
    float nrm = 0.0f;
    if (c < p.k)
      for (int t = 0; t < p.d; ++t) { const float v = __ldg(p.y + (int64_t)c * p.d + t); nrm = fmaf(v, v, nrm); }
    // cosine: rows are scaled to unit length (zero rows stay zero); L2: rows as they are
    const float row_scale = p.metric == F2C_COSINE ? (nrm > 0.0f ? 1.0f / sqrtf(nrm) : 0.0f) : 1.0f;
    if (BF16) {
      const int C = p.dp / 8;
      for (int cq = 0; cq < C; ++cq) {
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int t = 8 * cq + e;
          v[e] = (c < p.k && t < p.d) ? __ldg(p.y + (int64_t)c * p.d + t) * row_scale : 0.0f;
        }
        uint4 c1, c2;
        split8_bf16(v, c1, c2);  // B' = [y1 | y1 | y2]
        *reinterpret_cast<uint4*>(b_tile + (size_t)(cq) * lbo_b + c * 16) = c1;
        *reinterpret_cast<uint4*>(b_tile + (size_t)(C + cq) * lbo_b + c * 16) = c1;
        *reinterpret_cast<uint4*>(b_tile + (size_t)(2 * C + cq) * lbo_b + c * 16) = c2;
      }
    }
    for (int gq = 0; gq < (BF16 ? 0 : G); ++gq) {
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int t = 4 * gq + e;
        v[e] = (c < p.k && t < p.d) ? __ldg(p.y + (int64_t)c * p.d + t) * row_scale : 0.0f;
      }
      float4 hi, lo;
      split4(v, hi, lo);
      if (p.terms == 3) {  // B' = [y_hi | y_hi | y_lo]
        *reinterpret_cast<float4*>(b_tile + (size_t)(gq) * lbo_b + c * 16) = hi;
        *reinterpret_cast<float4*>(b_tile + (size_t)(G + gq) * lbo_b + c * 16) = hi;
        *reinterpret_cast<float4*>(b_tile + (size_t)(2 * G + gq) * lbo_b + c * 16) = lo;
      } else {
        *reinterpret_cast<float4*>(b_tile + (size_t)gq * lbo_b + c * 16) = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
    // norm term: -|y_c|^2 / 2 split in two TF32 values (L2), 0 (cosine), a value that never wins (padding)
    float h = c < p.k ? (p.metric == F2C_L2 ? -0.5f * nrm : 0.0f) : -1e30f;
    if (BF16) {  // three bf16 pieces of h against three ones on the point side
      const __nv_bfloat16 h1 = __float2bfloat16_rn(h);
      const __nv_bfloat16 h2 = __float2bfloat16_rn(h - __bfloat162float(h1));
      const __nv_bfloat16 h3 = __float2bfloat16_rn(h - __bfloat162float(h1) - __bfloat162float(h2));
      *reinterpret_cast<uint4*>(b_tile + (size_t)kc_x * lbo_b + c * 16) =
          make_uint4((uint32_t)__bfloat16_as_ushort(h1) | ((uint32_t)__bfloat16_as_ushort(h2) << 16), (uint32_t)__bfloat16_as_ushort(h3), 0u, 0u);
    } else {
      const float h_hi = __uint_as_float(__float_as_uint(h) & 0xFFFFE000u);
      *reinterpret_cast<float4*>(b_tile + (size_t)kc_x * lbo_b + c * 16) = make_float4(h_hi, h - h_hi, 0.0f, 0.0f);
    }
    *reinterpret_cast<float4*>(b_tile + (size_t)(kc_x + 1) * lbo_b + c * 16) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    scratch[c] = c < p.k ? nrm : 0.0f;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot + (uint32_t)g * 256u;
  // largest centre norm (tolerance of the L2 score); a non-finite centre sends every point to the exact scorer
  float cmax = 0.0f, poison = 0.0f;
  for (int c = 0; c < p.k; ++c) { cmax = fmaxf(cmax, scratch[c]); poison = fmaf(scratch[c], 0.0f, poison); }  // inf, NaN -> NaN
  const bool bad_centres = !(poison == 0.0f);
  cmax = sqrtf(cmax);

  // instruction descriptor: fp32 accumulate; A and B formats tf32 (2, kind::tf32) or bf16 (1, kind::f16); N / 8; M / 16
  const uint32_t fmt = BF16 ? 1u : 2u;
  const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(p.n_pad >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
  const int ksteps = kc / 2;  // one MMA consumes 8 tf32 = two 16-byte chunks of K
  const uint32_t mbar_addr = smem_u32(mbar + g);
  uint32_t parity = 0;

  const int64_t n_tiles = (p.n + kTileM - 1) / kTileM;
  const int64_t first = (int64_t)blockIdx.x * 2 + g, stride = (int64_t)gridDim.x * 2;
  // This thread's chunks of its point's row, fetched one tile ahead so that the global-load latency hides behind the
  // previous tile's MMA and epilogue: chunk q of the thread is 16-byte chunk half + 2q of the row (at most 8: d <= 64).
  constexpr int kMaxChunks = 8;
  float4 xv[kMaxChunks];
  // bf16 path (rows of 132 to 256 bytes): the tile's rows are fetched and split by a different thread mapping than the
  // one of the epilogue, so that a warp-wide load covers 8 rows x 128 contiguous bytes instead of 32 rows x 16 bytes
  // (the load queue was the limiter): lane = (row pl of 8, 32-byte chunk cl of 4), warp wq of the group, item
  // j = 0..3 -> row block 2 wq + (j >> 1), chunk cl + 4 (j & 1).  Shared-memory stores stay conflict-free (8 lanes =
  // 8 consecutive rows of one chunk), |x|^2 goes through shared memory to the epilogue thread of the point.
  const int wq = lt >> 5, pl = lt & 7, cl = (lt >> 3) & 3;
  auto fetch_row = [&](int64_t tile_) {
    const int64_t i_own = tile_ * kTileM + pt;
    const int G = p.dp / 4;
#pragma unroll
    for (int q = 0; q < kMaxChunks; ++q) {
      const int gq = BF16 ? 2 * (cl + 4 * ((q >> 1) & 1)) + (q & 1) : half + 2 * q;
      const int64_t i_ = BF16 ? tile_ * kTileM + (wq * 2 + (q >> 2)) * 8 + pl : i_own;
      xv[q] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (gq < G && tile_ < n_tiles && i_ < p.n) {
        if (p.vec4 && 4 * gq + 3 < p.d) {
          xv[q] = __ldg(reinterpret_cast<const float4*>(p.x + i_ * p.d) + gq);
        } else {
          float v[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int t = 4 * gq + e;
            v[e] = t < p.d ? __ldg(p.x + i_ * p.d + t) : 0.0f;
          }
          xv[q] = make_float4(v[0], v[1], v[2], v[3]);
        }
      }
    }
  };
  fetch_row(first);
  for (int64_t tile = first; tile < n_tiles; tile += stride) {
    // ---- A tile: the two threads of point tile*128 + pt split and store alternate 16-byte chunks of its row ----
    const int64_t i = tile * kTileM + pt;
    float xx = 0.0f;
    {
      const int G = p.dp / 4;
      if (BF16) {
        const int C = p.dp / 8;
        float part[2] = {0.0f, 0.0f};  // this thread's share of |x|^2 of its two rows
#pragma unroll
        for (int q2 = 0; q2 < kMaxChunks / 2; ++q2) {
          const int cq = cl + 4 * (q2 & 1);  // bf16 chunk = float4 chunks 2 cq, 2 cq + 1 = xv[2 q2], xv[2 q2 + 1]
          const int ptl = (wq * 2 + (q2 >> 1)) * 8 + pl;
          if (cq < C) {
            const float v[8] = {xv[2 * q2].x, xv[2 * q2].y, xv[2 * q2].z, xv[2 * q2].w,
                                xv[2 * q2 + 1].x, xv[2 * q2 + 1].y, xv[2 * q2 + 1].z, xv[2 * q2 + 1].w};
#pragma unroll
            for (int e = 0; e < 8; ++e) part[q2 >> 1] = fmaf(v[e], v[e], part[q2 >> 1]);
            uint4 c1, c2;
            split8_bf16(v, c1, c2);  // A' = [x1 | x2 | x1]
            *reinterpret_cast<uint4*>(a_tile + (size_t)(cq) * lbo_a + ptl * 16) = c1;
            *reinterpret_cast<uint4*>(a_tile + (size_t)(C + cq) * lbo_a + ptl * 16) = c2;
            *reinterpret_cast<uint4*>(a_tile + (size_t)(2 * C + cq) * lbo_a + ptl * 16) = c1;
          }
        }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          float v = part[b];
          v += __shfl_xor_sync(0xffffffffu, v, 8);
          v += __shfl_xor_sync(0xffffffffu, v, 16);
          if (cl == 0) xx_s[(wq * 2 + b) * 8 + pl] = v;
        }
      }
#pragma unroll
      for (int q = 0; q < (BF16 ? 0 : kMaxChunks); ++q) {
        const int gq = half + 2 * q;
        if (gq < G) {
          const float v[4] = {xv[q].x, xv[q].y, xv[q].z, xv[q].w};
          xx = fmaf(v[0], v[0], xx); xx = fmaf(v[1], v[1], xx); xx = fmaf(v[2], v[2], xx); xx = fmaf(v[3], v[3], xx);
          float4 hi, lo;
          split4(v, hi, lo);
          if (p.terms == 3) {  // A' = [x_hi | x_lo | x_hi]
            *reinterpret_cast<float4*>(a_tile + (size_t)(gq) * lbo_a + pt * 16) = hi;
            *reinterpret_cast<float4*>(a_tile + (size_t)(G + gq) * lbo_a + pt * 16) = lo;
            *reinterpret_cast<float4*>(a_tile + (size_t)(2 * G + gq) * lbo_a + pt * 16) = hi;
          } else {
            *reinterpret_cast<float4*>(a_tile + (size_t)gq * lbo_a + pt * 16) = xv[q];
          }
        }
      }
      // norm-term columns: ones against the pieces of -|y|^2 / 2 (two tf32 ones, or three bf16 ones = 0x3F80 each)
      *reinterpret_cast<uint4*>(a_tile + (size_t)(kc_x + half) * lbo_a + pt * 16) =
          half != 0 ? make_uint4(0u, 0u, 0u, 0u)
                    : (BF16 ? make_uint4(0x3F803F80u, 0x00003F80u, 0u, 0u) : make_uint4(0x3F800000u, 0x3F800000u, 0u, 0u));
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    group_sync(g);  // A tile complete; every warp of the group has finished reading the previous tile's accumulators
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (BF16) xx = half == 0 ? xx_s[pt] : 0.0f;  // read before the next tile's split overwrites it (two group syncs away)

    // ---- S = A' * B'^T into this group's TMEM columns ----
    if (lt == 0) {
      const uint32_t a_addr = smem_u32(a_tile), b_addr = smem_u32(b_tile);
      for (int s_ = 0; s_ < ksteps; ++s_) {
        const uint64_t a_desc = make_desc(a_addr + (uint32_t)s_ * 2u * lbo_a, lbo_a, sbo);
        const uint64_t b_desc = make_desc(b_addr + (uint32_t)s_ * 2u * lbo_b, lbo_b, sbo);
        if (BF16) mma_bf16(tmem_base, a_desc, b_desc, idesc, s_ > 0 ? 1u : 0u);
        else mma_tf32(tmem_base, a_desc, b_desc, idesc, s_ > 0 ? 1u : 0u);
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar_addr) : "memory");
    }
    fetch_row(tile + stride);  // next tile's row, in flight during this tile's MMA and epilogue
    // ---- bounded wait for the MMAs ----
    uint32_t done = 0;
    for (uint32_t it = 0; it < kWaitLimit && !done; ++it) {
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}\n"
          : "=r"(done) : "r"(mbar_addr), "r"(parity) : "memory");
    }
    parity ^= 1u;
    if (!done) fail[g] = 1u;
    group_sync(g);
    if (fail[g] != 0u) {  // somebody gave up: record it and leave through the common exit
      if (lt == 0) atomicExch(p.error, 1 + (int)((tile - first) / stride));  // 1 + how many tiles this group had finished
      break;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // ---- epilogue: TMEM lane pt = point i; its two threads scan one half of the centres each, with four
    //      independent trackers over interleaved columns; half 1 hands its result to half 0 through shared memory ----
    Top2 t0, t1, t2, t3;
    t0.init(); t1.init(); t2.init(); t3.init();
    const uint32_t lane_addr = tmem_base + ((uint32_t)(lane_quarter * 32) << 16);
    const int c_split = ((p.n_pad / 32 + 1) / 2) * 32;
    const int c_begin = half == 0 ? 0 : c_split, c_end = half == 0 ? c_split : p.n_pad;
    {
      uint32_t ra[16], rb[16];  // two 16-column loads alternate: one is consumed while the other is in flight
      auto scan = [&](const uint32_t (&r)[16], int c0) {
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
          t0.push(__uint_as_float(r[j]), c0 + j);
          t1.push(__uint_as_float(r[j + 1]), c0 + j + 1);
          t2.push(__uint_as_float(r[j + 2]), c0 + j + 2);
          t3.push(__uint_as_float(r[j + 3]), c0 + j + 3);
        }
      };
      if (c_begin < c_end) tmem_ld16(lane_addr + (uint32_t)c_begin, ra);
      for (int c0 = c_begin; c0 < c_end; c0 += 32) {  // c_end - c_begin is a multiple of 32
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        tmem_ld16(lane_addr + (uint32_t)(c0 + 16), rb);
        scan(ra, c0);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (c0 + 32 < c_end) tmem_ld16(lane_addr + (uint32_t)(c0 + 32), ra);
        scan(rb, c0 + 16);
      }
    }
    t0.merge(t1); t2.merge(t3); t0.merge(t2);
    if (half == 1) exch[pt] = make_float4(t0.best, t0.second, __int_as_float(t0.idx), xx);
    group_sync(g);
    if (half == 1) continue;
    {
      const float4 o = exch[pt];
      Top2 other;
      other.best = o.x; other.second = o.y; other.idx = __float_as_int(o.z);
      t0.merge(other);
      xx += o.w;
    }
    const float xn = sqrtf(xx);
    // error bound of a score: L2  eps*|x||y|max ;  cosine  eps*|x|
    const float tol = p.metric == F2C_L2 ? p.eps * xn * cmax : p.eps * xn;
    const bool odd = bad_centres || !(xx < INFINITY) || !(t0.best > -INFINITY);  // NaN / inf somewhere: exact scorer
    if (i < p.n) {
      if (odd || !(t0.best - t0.second > 2.0f * tol)) {  // undecided: the exact scorer assigns it afterwards
        const int slot = atomicAdd(p.amb_count, 1);
        p.amb_list[slot] = (int32_t)i;
      } else {
        p.labels[i] = t0.idx;
      }
    }
  }

  // ---- common exit: all TMEM reads retired, then the allocating warp frees the columns ----
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid < 32) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(*tmem_slot), "r"(512u) : "memory");
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
  p.bf16 = p.dp > 32 ? 1 : 0;  // 3 x tf32 does not fit in shared memory beyond d = 32; 3 x bf16 does up to d = 64
  if (p.bf16) p.dp = (int)((d + 15) / 16 * 16);  // one bf16 MMA consumes 16 values of K
  p.n_pad = (int)((k + 31) / 32 * 32);
  p.vec4 = d % 4 == 0 && aligned(x, 16);
  // relative error bound of one score: 2^-16 for the tf32 split (true error ~2^-18.4); 2^-14 for the bf16 split
  // (neglected terms x2.y2 + x.y3 + x3.y <= 3 * 2^-18 |x||y| = 2^-16.4)
  p.eps = p.bf16 ? 1.0f / 16384.0f : 1.0f / 65536.0f;
  int32_t* head = reinterpret_cast<int32_t*>(workspace);
  p.amb_count = head; p.error = head + 1; p.amb_list = head + 64;
  cudaError_t e = cudaMemsetAsync(head, 0, 256, st);
  if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "kmeans_assign: %s", cudaGetErrorString(e));
  const int kc = (p.bf16 ? 3 * p.dp / 8 : p.terms * p.dp / 4) + 2;
  size_t smem = (size_t)kc * (tc::kMaxN + 2 * tc::kTileM) * 16 + tc::kMaxN * 4 + 2 * tc::kTileM * 16 + 64 + 2 * tc::kTileM * 4;
  if (smem < 120 * 1024) smem = 120 * 1024;  // one CTA per SM: a second one would only wait for the TMEM columns
  auto kern = p.bf16 ? tc::kmeans_tc_kernel<true> : tc::kmeans_tc_kernel<false>;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "kmeans_assign: %s", cudaGetErrorString(e));
  int64_t tiles = ceil_div(n, tc::kTileM);
  int64_t grid = ceil_div(tiles, 2);  // one CTA per SM (it owns all 512 TMEM columns), two tiles in flight per CTA
  if (grid > current_sm_count()) grid = current_sm_count();
  kern<<<(unsigned)grid, tc::kCtaThreads, smem, st>>>(p);
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

// Device address of the scratch array on the current device, looked up once per device (with that device current).
static int static_scratch(const char* op, void** scratch) {
  static std::mutex mu;
  static void* scratch_of_device[64] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) return set_error(F2C_ERR_CUDA, "%s: cudaGetDevice: %s", op, cudaGetErrorString(e));
  std::lock_guard<std::mutex> lock(mu);
  if (scratch_of_device[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) return set_error(F2C_ERR_CUDA, "%s: cudaGetSymbolAddress: %s", op, cudaGetErrorString(e));
    scratch_of_device[dev] = ptr;
  }
  *scratch = scratch_of_device[dev];
  return F2C_OK;
}
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

  void* scratch = nullptr;
  int rc = tc::static_scratch(op, &scratch);
  if (rc) return rc;
  // same kernels as kmeans_assign; the header (count, error code) is cleared inside
  return kmeans_assign_tc(x, centers, labels, n, k, d, metric, scratch, (cudaStream_t)stream);
}

// What the last f2c_kmeans_assign_static call on the current device left in the header of the built-in array: the
// number of points the tensor-core pass handed to the exact scorer, and the code the kernel writes when one of its
// bounded barrier waits ran out (0 = none; labels of the unfinished tiles are then unwritten).  Waits for `stream`,
// copies the eight header bytes to the host, allocates nothing.  Returns F2C_ERR_CUDA when the code is non-zero.
extern "C" int f2c_kmeans_assign_static_status(int32_t* undecided_host, int32_t* error_host, void* stream) {
  using namespace f2c;
  const char* op = "kmeans_assign_static_status";
  void* scratch = nullptr;
  int rc = tc::static_scratch(op, &scratch);
  if (rc) return rc;
  cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "%s: %s", op, cudaGetErrorString(e));
  int32_t head[2] = {0, 0};
  e = cudaMemcpy(head, scratch, sizeof(head), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "%s: %s", op, cudaGetErrorString(e));
  if (undecided_host) *undecided_host = head[0];
  if (error_host) *error_host = head[1];
  if (head[1] != 0) return set_error(F2C_ERR_CUDA, "%s: the tensor-core kernel gave up on a bounded wait (code %d)", op, head[1]);
  return F2C_OK;
}
