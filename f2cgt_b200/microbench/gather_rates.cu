// Random-row gather ceilings of one B200 (and of NVLink from one peer): the rates the fused kernels' designs are
// argued from.  Stand-alone (CUDA runtime only); not part of libf2cgt_b200.so.
//
//   nvcc -O3 -gencode arch=compute_100a,code=sm_100a -o /tmp/gather_rates f2cgt_b200/microbench/gather_rates.cu
//   /tmp/gather_rates            # one GPU: local rows; two or more GPUs: also rows of GPU 1 read from GPU 0
//
// Rows of S = 16 / 32 / 64 / 128 bytes are picked by a hash out of a 2,449,029-row table (the benchmark's table), L2
// evicted before every launch.  Three ways to fetch them:
//   ldg     plain 16-byte loads into registers, many warps per SM (what the register-prefetch kernels do)
//   ldgsts  16-byte cp.async pieces into shared memory from P producer warps per SM (what the streamed kernels do)
//   bulk    one cp.async.bulk per row + mbarrier from P warps per SM (no multicast)
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <cuda_runtime.h>
#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e_), __LINE__); exit(1);} } while (0)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t hash_id(uint32_t e, uint32_t n_rows) {
  uint32_t x = e * 2654435761u; x ^= x >> 15; x *= 2246822519u; x ^= x >> 13;
  return x % n_rows;
}
// mode 0: cp.async 16B pieces, NB groups in flight per warp.  mode 1: bulk copy per row, NB mbarriers in flight per warp.
template <int MODE>
__global__ void __launch_bounds__(1024, 1) gather_kernel(const uint8_t* __restrict__ table, uint32_t n_rows, int S, int rows_per_cta,
                                                        int NB, unsigned long long* out_clk, int* err) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int P = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // per warp: NB slots of 32 rows
  const uint32_t slot_bytes = 32u * S;
  unsigned char* my = smem + (size_t)warp * NB * slot_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)P * NB * slot_bytes) + warp * NB;
  if (MODE == 1 && lane == 0) for (int i = 0; i < NB; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bars + i)));
  __syncthreads();
  const int per_warp = rows_per_cta / P;
  const uint32_t base_e = (blockIdx.x * P + warp) * per_warp;
  const int iters = per_warp / 32;
  unsigned long long t0 = clock64();
  if (MODE == 0) {
    const int pieces = S / 16, lg = pieces == 1 ? 0 : pieces == 2 ? 1 : pieces == 4 ? 2 : 3;
    // an iteration copies 32 rows: 32*pieces lane-ops = `pieces` instructions
    for (int it = 0; it < iters; ++it) {
      const uint32_t dst0 = smem_u32(my + (it % NB) * slot_bytes);
      for (int k = 0; k < pieces; ++k) {
        const int t = k * 32 + lane;
        const int r = t >> lg, c = t & (pieces - 1);
        const uint32_t id = hash_id(base_e + it * 32 + r, n_rows);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst0 + r * S + c * 16), "l"(table + (size_t)id * S + c * 16) : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      // keep NB-1 groups in flight
      switch (NB) {
        case 2: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
        case 4: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
        case 8: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 15;" ::: "memory"); break;
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else {
    for (int it = 0; it < iters; ++it) {
      const int slot = it % NB;
      const uint32_t bar = smem_u32(bars + slot);
      if (it >= NB) {
        const uint32_t parity = ((it / NB) - 1) & 1;
        uint32_t done = 0; int spins = 0;
        while (!done) {
          asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
          if (!done && ++spins > (1 << 20)) { *err = 1; return; }
        }
      }
      if (lane == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(slot_bytes) : "memory");
      __syncwarp();
      const uint32_t id = hash_id(base_e + it * 32 + lane, n_rows);
      const uint32_t dst = smem_u32(my + slot * slot_bytes + lane * S);
      asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(dst), "l"(table + (size_t)id * S), "r"(S), "r"(bar) : "memory");
    }
    // drain
    for (int k = 0; k < NB && k < iters; ++k) {
      const int it = iters - 1 - k;
      const uint32_t bar = smem_u32(bars + (it % NB));
      const uint32_t parity = (it / NB) & 1;
      uint32_t done = 0; int spins = 0;
      while (!done) {
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (!done && ++spins > (1 << 20)) { *err = 2; return; }
      }
    }
  }
  unsigned long long t1 = clock64();
  if (threadIdx.x == 0) out_clk[blockIdx.x] = t1 - t0;
}

// each lane group of (S/16) lanes reads one row per step; UNROLL rows in flight per lane
template <int UNROLL>
__global__ void __launch_bounds__(1024) peer_gather(const uint4* __restrict__ table, uint32_t n_rows, int S, int rows_per_cta, uint4* sink) {
  const int pieces = S / 16;
  const int lanes_total = blockDim.x;
  const int rows_per_step = lanes_total / pieces;
  const int piece = threadIdx.x % pieces, slot = threadIdx.x / pieces;
  uint4 acc = make_uint4(0, 0, 0, 0);
  const uint32_t base = blockIdx.x * rows_per_cta;
  for (int r0 = 0; r0 < rows_per_cta; r0 += rows_per_step * UNROLL) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const uint32_t id = hash_id(base + r0 + u * rows_per_step + slot, n_rows);
      v[u] = __ldg(table + (size_t)id * pieces + piece);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) { acc.x ^= v[u].x; acc.y ^= v[u].y; acc.z ^= v[u].z; acc.w ^= v[u].w; }
  }
  if (acc.x == 0x12345678u) sink[0] = acc;
}

static void run_ldg(const char* tag, const uint4* table, uint32_t n_rows, float* flush, uint4* sink, cudaEvent_t a, cudaEvent_t b) {
  const int rows_per_cta = 32768;
  for (int S : {16, 32, 64, 128})
    for (int threads : {512, 1024})
      for (int unroll : {4, 8, 16}) {
        float best = 1e9;
        for (int rep = 0; rep < 3; ++rep) {
          CK(cudaMemsetAsync(flush, rep, 256 << 20));
          CK(cudaEventRecord(a));
          if (unroll == 4) peer_gather<4><<<148, threads>>>(table, n_rows, S, rows_per_cta, sink);
          else if (unroll == 8) peer_gather<8><<<148, threads>>>(table, n_rows, S, rows_per_cta, sink);
          else peer_gather<16><<<148, threads>>>(table, n_rows, S, rows_per_cta, sink);
          CK(cudaEventRecord(b)); CK(cudaDeviceSynchronize());
          float ms; CK(cudaEventElapsedTime(&ms, a, b));
          if (ms < best) best = ms;
        }
        const double rows = 148.0 * rows_per_cta;
        printf("ldg %s S=%3d threads=%4d unroll=%2d  %8.1f us  %7.1f GB/s  %6.2f Grows/s\n", tag, S, threads, unroll, best * 1e3,
               rows * S / (best * 1e-3) / 1e9, rows / (best * 1e-3) / 1e9);
        fflush(stdout);
      }
}

int main() {
  int n_gpus = 0; CK(cudaGetDeviceCount(&n_gpus));
  const uint32_t n_rows = 2449029;
  uint4 *local = nullptr, *remote = nullptr, *sink = nullptr;
  if (n_gpus >= 2) {
    CK(cudaSetDevice(1)); CK(cudaMalloc(&remote, (size_t)n_rows * 128)); CK(cudaMemset(remote, 1, (size_t)n_rows * 128)); CK(cudaDeviceSynchronize());
    CK(cudaSetDevice(0)); CK(cudaDeviceEnablePeerAccess(1, 0));
  }
  CK(cudaSetDevice(0));
  CK(cudaMalloc(&local, (size_t)n_rows * 128)); CK(cudaMemset(local, 1, (size_t)n_rows * 128)); CK(cudaMalloc(&sink, 64));
  unsigned long long* clk; CK(cudaMalloc(&clk, 148 * 8));
  int* err; CK(cudaMalloc(&err, 4)); CK(cudaMemset(err, 0, 4));
  float* flush; CK(cudaMalloc(&flush, 256 << 20));
  cudaEvent_t a, b; CK(cudaEventCreate(&a)); CK(cudaEventCreate(&b));
  run_ldg("LOCAL", local, n_rows, flush, sink, a, b);
  if (remote != nullptr) run_ldg("PEER ", remote, n_rows, flush, sink, a, b);
  const int rows_per_cta = 8192;
  CK(cudaFuncSetAttribute(gather_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  CK(cudaFuncSetAttribute(gather_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  const uint8_t* table = reinterpret_cast<const uint8_t*>(local);
  for (int mode = 0; mode < 2; ++mode)
    for (int S : {16, 64, 128})
      for (int P : {1, 2, 4, 8, 16})
        for (int NB : {4, 8, 16}) {
          size_t smem = (size_t)P * NB * 32 * S + (size_t)P * NB * 8 + 64;
          if (smem > 200 * 1024) continue;
          float best = 1e9;
          for (int rep = 0; rep < 3; ++rep) {
            CK(cudaMemsetAsync(flush, rep, 256 << 20));
            CK(cudaEventRecord(a));
            if (mode == 0) gather_kernel<0><<<148, 32 * P, smem>>>(table, n_rows, S, rows_per_cta, NB, clk, err);
            else gather_kernel<1><<<148, 32 * P, smem>>>(table, n_rows, S, rows_per_cta, NB, clk, err);
            CK(cudaEventRecord(b));
            CK(cudaDeviceSynchronize());
            float ms; CK(cudaEventElapsedTime(&ms, a, b));
            if (ms < best) best = ms;
          }
          int herr; CK(cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost));
          double bytes = 148.0 * rows_per_cta * S;
          printf("%s S=%3d P=%2d NB=%2d  %8.1f us  %7.1f GB/s  rows/us/SM=%.2f err=%d\n", mode ? "bulk  " : "ldgsts", S, P, NB, best * 1e3,
                 bytes / (best * 1e-3) / 1e9, rows_per_cta / (best * 1e3), herr);
          fflush(stdout);
        }
  return 0;
}
