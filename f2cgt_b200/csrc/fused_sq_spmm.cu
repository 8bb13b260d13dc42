// Fused SQ decode + mean/sum aggregation over a CSC block
// (reference operator sq_decompress_spmm_csr, src/fusion_spmm.cu:143-272).
//
//   out[d, :] = (sum_{k in N(d), CSC order} decode(codes[indices[k], :])) / max(deg(d), 1)
//
// The decoded fp32 rows never exist in memory: a neighbour's compressed row (16..256 B) is fetched
// with one 32/64-bit read-only load per lane, decoded and added to fp32 accumulators in registers,
// in CSC order, which makes the result equal to decode-then-aggregate bit for bit and independent of
// launch geometry.
//
// What bounds it.  Per edge the kernel moves only row_bytes + 8 bytes but must produce feat_dim fp32
// values, so on B200 it is bound by instruction issue and by latency (a sampled block offers ~10^5
// independent rows, each a chain indptr -> indices -> code rows), not by HBM.  The design therefore
// minimises instructions per decoded element and keeps three destination rows per lane group in
// flight:
//
//  * Work layout.  A destination row is owned by a group of G = row_bytes / VEC consecutive lanes
//    (G a power of two; a warp serves 32/G rows at once); lane g owns bytes [g*VEC, (g+1)*VEC) of
//    every neighbour row and the EPL = VEC*8/bits output columns they encode.
//  * Decode.  Every width <= 8 bits is decoded a whole code byte at a time through a shared-memory
//    table built at kernel start WITH THE SAME EXPRESSION as the element-wise decode (hence the same
//    bits): slab `byte` (256 bytes) holds the 8/bits floats the byte encodes, replicated once per
//    bank group so lookups never collide.  With a 256-byte slab stride the lookup offset
//    (byte << 8) | lane_offset is ONE byte-permute of the data word; the lookup is one LDS.64/.128,
//    and the adds are packed two-per-instruction (add.f32x2).  16-bit codes use the arithmetic decode.
//  * Pipeline.  While row i is decoded, the code rows of row i+1, the neighbour ids of row i+2 and
//    the indptr pair of row i+3 are in flight; two register sets alternate through a 2x unrolled loop
//    so that no load result is ever moved (a move would wait for the load and serialise the chain).
//  * Output.  A lane holds EPL consecutive columns, so direct stores would scatter 16-byte pieces
//    over 32 lines per instruction; the warp's sums are staged in shared memory (XOR-swizzled, no
//    bank conflicts either way), read back row by row, divided by the degree with two FMA
//    corrections that reproduce the IEEE quotient, and written as whole 512-byte runs.
//
// Grid: persistent, exactly the resident CTA count; each CTA builds its table once.
#include <mutex>

#include "sq_fused.cuh"

namespace f2c {

int validate_sq(const char* op, int code_dtype, int64_t n_codebooks, int64_t src_dim, int64_t feat_dim, int bits,
                int64_t column_slice);
// streamed kernel (fused_sq_stream.cu); *served = false when it does not take the shape
int launch_sq_stream(int bits, int index_dtype, const void* codes, int code_dtype, const float* codebooks, int64_t n_cb,
                     const void* indptr, const void* indices, float* out, int64_t n_dst, int64_t n_src, int64_t src_dim, int64_t D,
                     int64_t cs, int reduce, const DropoutArgs& drop, cudaStream_t st, const void* const* shards, int world,
                     int64_t rows_per_shard, bool* served);

// Table kernels for 4- and 8-bit codes run as ONE 512-thread CTA per SM whose table starts on a 64 KB boundary of the
// shared window: the base address then lives in the upper half of the byte permute's second source and a lookup
// address costs one instruction.  Measured on B200 (config-2 block): 4 bit 47.1 -> 45.1 us, 8 bit 55.3 -> 51.9 us; the
// 1- and 2-bit kernels (fewer lookups per byte of code, larger staging area) are faster as two 256-thread CTAs.
template <int BITS, int DEC> struct SqCta {
  static constexpr bool kAligned = DEC == DEC_LUT && BITS >= 4;
  static constexpr int kThreads = kAligned ? 512 : 256;
  static constexpr int kCtasPerSm = kAligned ? 1 : 2;
};

struct PeerInfo {
  const void* shard[8];
  int world;
  int64_t rows_per_shard;
  const void* replicated;   // local copy of the leading (most often sampled) rows, or null
  int64_t n_replicated;
};

struct SqParams {
  const uint8_t* codes;
  const float* codebooks;
  const void* indptr;
  const void* indices;
  float* out;
  int64_t n_dst;
  uint32_t row_bytes;
  int feat_dim;
  int column_slice;
  int n_cb;
  int logG;
  int code_kind;
  int reduce;
  // row-sharded table (PEER kernels): id r lives in slot r / rows_per_shard of this pointer table, all of it mapped into
  // this process.  Without replicated rows the slots are the shards.  With n_replicated leading rows kept on every GPU
  // the first ceil(n_replicated / rows_per_shard) slots point into that local copy and the shards follow: the ids of
  // the sharded rows start at the next multiple of rows_per_shard, so one division serves both kinds of row.
  const uint8_t* shard[16];
  uint32_t rows_per_shard;
  unsigned long long shard_magic;  // floor(2^64 / rows_per_shard) + 1: exact 32-bit division by one multiply-high
  int staged;        // 1: rows leave through the shared-memory staging area (feat_dim % 4 == 0)
  int stage_offset;  // byte offset of that area in dynamic shared memory
  DropoutArgs drop;
};

// U = neighbours held in registers per destination row (rows with more take extra, unpipelined rounds).
// PEER: the table is row-sharded over the GPUs of one NVSwitch box and every shard is mapped into this process;
// a neighbour's row is read from its owner's HBM with an ordinary load over NVLink (no collective, no staging copy).
template <int BITS, int VEC, int U, typename IdxT, int DEC, bool PEER = false>
__global__ void __launch_bounds__(SqCta<BITS, DEC>::kThreads, SqCta<BITS, DEC>::kCtasPerSm)
sq_spmm_kernel(const SqParams p) {
  constexpr bool ALIGNED = SqCta<BITS, DEC>::kAligned;
  constexpr int EPL = BITS == 16 ? VEC / 2 : VEC * 8 / BITS;  // output columns per lane
  constexpr bool PACKED = DEC == DEC_LUT && BITS <= 4;
  extern __shared__ __align__(16) unsigned char smem_dyn[];
  // Aligned-table kernels: everything starts at the next 64 KB boundary of the shared window (the launch reserves the
  // slack), so the table's base address is a pure "upper half" value and rides in the permute that forms a lookup address.
  unsigned char* const smem_raw =
      ALIGNED ? smem_dyn + ((0x10000u - ((uint32_t)__cvta_generic_to_shared(smem_dyn) & 0xFFFFu)) & 0xFFFFu) : smem_dyn;

  const int lane = threadIdx.x & 31;
  const int G = 1 << p.logG;
  const int lane_g = lane & (G - 1);
  const int sub = lane >> p.logG;
  const int rows_per_warp = 32 >> p.logG;
  const uint32_t byte0 = (uint32_t)lane_g * VEC;
  const bool lane_active = byte0 < p.row_bytes;
  const int c0 = lane_g * EPL;

  // Codebook row of this lane's columns (the host guarantees they share one row on this path).
  int cb_row = c0 / p.column_slice;
  if (cb_row >= p.n_cb) cb_row = p.n_cb - 1;
  const float emin = __ldg(p.codebooks + cb_row * kCodebookDim + 2);
  const float emax = __ldg(p.codebooks + cb_row * kCodebookDim + 3);
  const float mean = __ldg(p.codebooks + cb_row * kCodebookDim + 4);
  const float scale = sq_scale<BITS>(emin, emax);

  // ---- Pipeline state and priming.  The chain indptr -> neighbour ids -> code rows of the first rows is three dependent
  //      global-load latencies; for 2- and 8-bit codes it is issued BEFORE the decode table is built, so that it overlaps
  //      the construction (measured on B200, same box: 8 bit 51.9 -> 49.5 us, 2 bit 43.0 -> 42.0 us; 1 bit 38.9 -> 43.0
  //      and 4 bit 42.6 -> 43.4 the other way, so those prime after the build).
  constexpr bool PRIME_EARLY = BITS == 2 || BITS == 8;
  const IdxT* __restrict__ indptr = reinterpret_cast<const IdxT*>(p.indptr);
  const IdxT* __restrict__ indices = reinterpret_cast<const IdxT*>(p.indices);
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t stride = (((int64_t)gridDim.x * blockDim.x) >> 5) * rows_per_warp;
  const uint8_t* __restrict__ my_codes = p.codes + byte0;
  // address of this lane's slice of source row `id`
  auto row_ptr = [&](uint32_t id) -> const uint8_t* {
    if (!PEER) return my_codes + (uint64_t)id * p.row_bytes;
    const uint32_t owner = (uint32_t)__umul64hi((unsigned long long)id, p.shard_magic);
    const uint32_t local = id - owner * p.rows_per_shard;
    return p.shard[owner] + byte0 + (uint64_t)local * p.row_bytes;
  };

  // ---- three-deep software pipeline over the rows d, d+stride, d+2*stride, ... of this lane group.
  // Rows are counted in 32 bits (the host checks n_dst < 2^31).
  const int n_dst = (int)p.n_dst;
  const int istride = (int)stride;
  int d = (int)(warp * rows_per_warp) + sub;
  const IdxT* idsA = indices;  // first neighbour id of rows i, i+1, i+2
  const IdxT* idsB = indices;
  const IdxT* idsC = indices;
  int degA = 0, degB = 0, degC = 0;
  // One set of id registers is enough: a stage first issues the row loads that consume them, then
  // overwrites them with the ids of the row after (the hardware scoreboard orders the two).
  uint32_t nidx[U];
  VecLoad<VEC> data[2][U];
  auto prime = [&]() {
    if (d < n_dst && lane_active) { int64_t b = (int64_t)indptr[d]; degA = (int)((int64_t)indptr[d + 1] - b); idsA = indices + b; }
    if (d + istride < n_dst && lane_active) {
      int64_t b = (int64_t)indptr[d + istride]; degB = (int)((int64_t)indptr[d + istride + 1] - b); idsB = indices + b;
    }
    if (d + 2 * istride < n_dst && lane_active) {
      int64_t b = (int64_t)indptr[d + 2 * istride]; degC = (int)((int64_t)indptr[d + 2 * istride + 1] - b); idsC = indices + b;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) nidx[u] = u < degA ? (uint32_t)idsA[u] : 0u;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      data[0][u].zero();
      if (u < degA) data[0][u].load(row_ptr(nidx[u]));
    }
#pragma unroll
    for (int u = 0; u < U; ++u) nidx[u] = u < degB ? (uint32_t)idsB[u] : 0u;
  };
  if (PRIME_EARLY) prime();
  uint32_t lane_off = 0;
  if (DEC == DEC_LUT) {
    using L = Lut<BITS>;
    build_sq_table<BITS, EPL>(smem_raw, reinterpret_cast<float*>(smem_raw + L::TABLE_BYTES + 256), p.codebooks, p.n_cb, p.column_slice,
                              G, p.code_kind, (int)threadIdx.x, (int)blockDim.x, [] { __syncthreads(); });
    lane_off = L::lane_offset(lane);
    if (ALIGNED) lane_off |= (uint32_t)__cvta_generic_to_shared(smem_raw);  // low 16 bits of the base are zero
  }
  const uint32_t table = ALIGNED ? 0u : (uint32_t)__cvta_generic_to_shared(smem_raw);  // aligned: the base is part of lane_off

  // Sums of decoded values are 0 or, in magnitude, between 2^(emin-24) and deg * 2^emax (1 bit: multiples of
  // ~mean); when that interval is well inside the normal range for every lane of the warp, the mean can use
  // the division without the per-element range check.
  const bool div_safe = __all_sync(0xffffffffu, BITS == 1 ? (mean > 1e-20f && mean < 1e20f) : (emin > -80.0f && emax < 80.0f));

  if (!PRIME_EARLY) prime();
  // Neighbour slots beyond a row's degree read slab 0 of a zero-filled copy of the table geometry
  // (their data word is kept 0), so the decode loop needs no divergent branch: adding +0 changes nothing.
  const uint32_t lane_off_zero = lane_off + Lut<BITS>::TABLE_BYTES;

  for (int row_base = (int)(warp * rows_per_warp); row_base < n_dst;) {
#pragma unroll
    for (int P = 0; P < 2; ++P) {
      if (row_base < n_dst) {  // warp uniform
        // (1) code rows of the next destination row -> data[P^1]
#pragma unroll
        for (int u = 0; u < U; ++u) {
          data[P ^ 1][u].zero();
          if (u < degB) data[P ^ 1][u].load(row_ptr(nidx[u]));
        }
        // (2) neighbour ids of the row after it
#pragma unroll
        for (int u = 0; u < U; ++u) nidx[u] = u < degC ? (uint32_t)idsC[u] : 0u;
        // (3) indptr pair three rows ahead
        const IdxT* idsD = indices;
        int degD = 0;
        if (d + 3 * istride < n_dst && lane_active) {
          int64_t b = (int64_t)indptr[d + 3 * istride];
          degD = (int)((int64_t)indptr[d + 3 * istride + 1] - b);
          idsD = indices + b;
        }

        // (4) decode + accumulate the current row from data[P]
        Acc<EPL, PACKED> acc;
        acc.clear();
        const int umax = __reduce_max_sync(0xffffffffu, degA < U ? degA : U);  // slots any row of the warp uses
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (u < umax) {  // warp uniform
            const VecLoad<VEC>& row = data[P][u];
            if (DEC == DEC_LUT) {
              sq_accumulate<BITS, VEC, DEC, ALIGNED>(acc, row, table, u < degA ? lane_off : lane_off_zero, p.code_kind, scale, emin, mean);
            } else if (u < degA) {
              sq_accumulate<BITS, VEC, DEC, ALIGNED>(acc, row, table, lane_off, p.code_kind, scale, emin, mean);
            }
          }
        }
        // destination rows with more than U neighbours: further rounds of four, not pipelined
        for (int k = U; k < degA; k += 4) {
          VecLoad<VEC> extra[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (k + u < degA) extra[u].load(row_ptr((uint32_t)idsA[k + u]));
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (k + u < degA) sq_accumulate<BITS, VEC, DEC, ALIGNED>(acc, extra[u], table, lane_off, p.code_kind, scale, emin, mean);
        }

        // (5) mean / dropout / store
        const bool have_row = d < n_dst && lane_active;
        if (p.staged) {
          float4* stage = reinterpret_cast<float4*>(smem_raw + p.stage_offset) + (threadIdx.x >> 5) * (32 * (EPL / 4));
          sq_store_rows<EPL>(acc, stage, lane, p.logG, degA, have_row, (int64_t)row_base, (int64_t)(n_dst - row_base), p.feat_dim,
                             p.reduce, div_safe, p.drop, p.out);
        } else if (have_row) {
          float* orow = p.out + (int64_t)d * p.feat_dim;
          const float deg = degA == 0 ? 1.0f : (float)degA;
#pragma unroll
          for (int e = 0; e < EPL; ++e) {
            int col = c0 + e;
            if (col < p.feat_dim) {
              float v = p.reduce == F2C_MEAN ? acc.get(e) / deg : acc.get(e);
              if (p.drop.enabled) v = dropout_apply1(v, (uint64_t)((int64_t)d * p.feat_dim + col), p.drop);
              orow[col] = v;
            }
          }
        }
        // rotate the (already resident) scalars; the register sets swap through P
        idsA = idsB; degA = degB; idsB = idsC; degB = degC; idsC = idsD; degC = degD;
        d += istride;
        row_base += istride;
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

// Resident CTAs per SM of one kernel instance at one shared-memory footprint, queried once per device.
struct ResidentCache {
  std::mutex m;
  int value[64] = {};
  size_t smem[64] = {};
};

template <int BITS, int VEC, int U, typename IdxT, int DEC, bool PEER = false>
static int launch_fast(SqParams p, bool vec_store, cudaStream_t st) {
  auto kern = sq_spmm_kernel<BITS, VEC, U, IdxT, DEC, PEER>;
  constexpr int EPL = BITS == 16 ? VEC / 2 : VEC * 8 / BITS;
  // decode table (64 KB) + the decoded code values of each distinct codebook row
  size_t smem = 0;
  if (DEC == DEC_LUT) {
    using L = Lut<BITS>;
    int n_rows = (1 << p.logG) < L::COPIES ? (1 << p.logG) : L::COPIES;
    smem = L::TABLE_BYTES + 256 + (size_t)n_rows * L::NCODE * sizeof(float);
  }
  constexpr int kThreads = SqCta<BITS, DEC>::kThreads;
  constexpr int kWarpsPerCta = kThreads / 32;
  // staging area for coalesced output: warps x 32 lanes x EPL floats
  p.staged = 0;
  p.stage_offset = (int)smem;
  if (vec_store && EPL >= 4) {
    p.staged = 1;
    smem += (size_t)kWarpsPerCta * 32 * EPL * sizeof(float);
  }
  if (SqCta<BITS, DEC>::kAligned) smem += 65536;  // slack for the 64 KB alignment of the table inside the shared window
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "sq_decompress_spmm_csr: %s", cudaGetErrorString(e));
  }
  // persistent grid: exactly as many CTAs as the device keeps resident
  static ResidentCache cache;
  int dev = 0, resident = 1;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
  const int sms = sm_count(dev);
  {
    std::lock_guard<std::mutex> lock(cache.m);
    const int slot = dev & 63;
    if (cache.value[slot] == 0 || cache.smem[slot] != smem) {
      int n = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kThreads, smem) != cudaSuccess || n < 1) n = 1;
      cache.value[slot] = n;
      cache.smem[slot] = smem;
    }
    resident = cache.value[slot];
  }
  int rows_per_cta = kWarpsPerCta * (32 >> p.logG);
  int64_t grid = ceil_div(p.n_dst, rows_per_cta);
  if (grid > (int64_t)sms * resident) grid = (int64_t)sms * resident;
  kern<<<(unsigned)grid, kThreads, smem, st>>>(p);
  return check_launch("sq_decompress_spmm_csr");
}

template <int BITS, typename IdxT>
static int dispatch_fast(const SqParams& p, int vec, bool lut, bool vec_store, cudaStream_t st) {
  constexpr bool CAN_LUT = BITS <= 8;
  constexpr bool CAN_8 = BITS > 2;  // 1/2-bit: 4 bytes per lane already are 32 / 16 columns
  // neighbours held in registers per destination row; measured on B200 (config-2 block, fan-out 12): 8 is fastest
  // for 2- and 4-bit codes (4 bit: 42-43 us against 46 with 12 - the four remaining neighbours take the unpipelined
  // round, but 16 fewer live registers help more; 2 bit: a tie; 4 per row is slower again), 12 for 1- and 8-bit codes
  constexpr int U = (BITS == 2 || BITS == 4) ? 8 : 12;
  if constexpr (CAN_LUT) if (lut) {
    if constexpr (CAN_8) if (vec == 8) return launch_fast<BITS, 8, U, IdxT, DEC_LUT>(p, vec_store, st);
    return launch_fast<BITS, 4, U, IdxT, DEC_LUT>(p, vec_store, st);
  }
  if constexpr (CAN_8) if (vec == 8) return launch_fast<BITS, 8, U, IdxT, DEC_ARITH>(p, vec_store, st);
  return launch_fast<BITS, 4, U, IdxT, DEC_ARITH>(p, vec_store, st);
}

template <int BITS, typename IdxT>
static int launch_sq_spmm(const void* codes, int code_dtype, const float* codebooks, int64_t n_cb, const void* indptr,
                          const void* indices, float* out, int64_t n_dst, int64_t n_src, int64_t src_dim, int64_t D, int64_t cs,
                          int reduce, const DropoutArgs& drop, int variant, cudaStream_t st, const PeerInfo* peer = nullptr) {
  if (n_dst == 0 || D == 0) return F2C_OK;
  const char* op = peer ? "sq_decompress_spmm_csr_peer" : "sq_decompress_spmm_csr";
  // ---- streamed kernel (producer warps + shared-memory ring).  Measured on B200 (2,449,029-row table, outermost block
  //      of 1024 seeds x fan-out 12,12,12, cold L2): 2-bit codes 36.9 us against 41.9 us for the register-prefetch kernel;
  //      1 bit 41-43 against 41, 4 bit 49.5 against 43.7, 8 bit 61.4 against 49.2 - staging the rows costs shared-memory
  //      wavefronts (7.0 M against 4.5 M at 4 bits) that the table decode needs itself, so only the 2-bit shape, whose
  //      rows are cheap to stage and whose prefetch kernel is the most latency-bound, gains.
  const bool stream_by_default = BITS == 2 && peer == nullptr;
  if (variant == F2C_KERNEL_STREAM && peer != nullptr && peer->n_replicated > 0)
    return set_error(F2C_ERR_UNSUPPORTED, "%s: the streamed kernel does not serve a table with replicated leading rows", op);
  if ((variant == F2C_KERNEL_AUTO && stream_by_default) || variant == F2C_KERNEL_STREAM) {
    bool served = false;
    int rc = launch_sq_stream(BITS, sizeof(IdxT) == 4 ? F2C_I32 : F2C_I64, codes, code_dtype, codebooks, n_cb, indptr, indices, out, n_dst,
                              n_src, src_dim, D, cs, reduce, drop, st, peer ? peer->shard : nullptr, peer ? peer->world : 0,
                              peer ? peer->rows_per_shard : 0, &served);
    if (served || rc) return rc;
    if (variant == F2C_KERNEL_STREAM) return set_error(F2C_ERR_UNSUPPORTED, "%s: shape not served by the streamed kernel", op);
  }
  const int code_bytes = dtype_size(code_dtype);
  const int64_t row_bytes = src_dim * code_bytes;
  // ---- can the register-prefetch kernel serve this shape? ----
  // bytes per lane per row: at most two words (two register sets of U rows are live) and at most 32 columns;
  // measured on B200: 8 bytes for 4/8/16-bit codes, 4 bytes for 1/2-bit codes
  constexpr int VMAX = BITS <= 2 ? 4 : 8;
  int vec = 0;
  for (int v = VMAX; v >= 4; v >>= 1)
    if (row_bytes % v == 0 && aligned(codes, v) && row_bytes <= 32 * v) { vec = v; break; }
  const bool natural_dtype = BITS < 8 || (BITS == 8 && code_bytes == 1) || (BITS == 16 && code_bytes == 2);
  // the vector kernel keeps neighbour ids in 32-bit registers
  bool fast = vec != 0 && natural_dtype && n_src < (1ll << 32) && n_dst < (1ll << 30) && variant != F2C_KERNEL_GENERAL;
  int epl = 0, G = 0;
  if (fast) {
    epl = BITS == 16 ? vec / 2 : vec * 8 / BITS;
    G = 1 << ilog2((int)ceil_div(row_bytes, vec));
    fast = n_cb == 1 || cs % epl == 0;  // every lane's columns must share one codebook row
  }
  if (fast) {
    SqParams p;
    p.codes = (const uint8_t*)codes; p.codebooks = codebooks; p.indptr = indptr; p.indices = indices; p.out = out;
    p.n_dst = n_dst; p.row_bytes = (uint32_t)row_bytes; p.feat_dim = (int)D; p.column_slice = (int)cs; p.n_cb = (int)n_cb;
    p.logG = ilog2(G); p.code_kind = code_dtype == F2C_I8 ? CODE_I8 : code_dtype == F2C_U8 ? CODE_U8 : CODE_I16;
    p.reduce = reduce; p.staged = 0; p.stage_offset = 0; p.drop = drop;
    // table copies are shared by lanes l and l + COPIES: they must own the same columns
    int copies = BITS >= 4 ? 32 : BITS == 2 ? 16 : 8;
    bool lut = (n_cb == 1 || copies % G == 0) && variant != F2C_KERNEL_PREFETCH_ARITH;
    if (peer != nullptr) {
      const int head_slots = (int)ceil_div(peer->n_replicated, peer->rows_per_shard);
      for (int k = 0; k < 16; ++k) {
        if (k < head_slots) p.shard[k] = (const uint8_t*)peer->replicated + (uint64_t)k * peer->rows_per_shard * row_bytes;
        else p.shard[k] = (const uint8_t*)peer->shard[k - head_slots < peer->world ? k - head_slots : 0];
      }
      p.rows_per_shard = (uint32_t)peer->rows_per_shard;
      p.shard_magic = ~0ull / (unsigned long long)peer->rows_per_shard + 1ull;
      constexpr int DEC = BITS <= 8 ? DEC_LUT : DEC_ARITH;
      if (vec != VMAX || (BITS <= 8 && !lut))
        return set_error(F2C_ERR_UNSUPPORTED, "%s: shape or codebook layout not served by the peer kernel", op);
      return launch_fast<BITS, VMAX, 12, IdxT, DEC, true>(p, D % 4 == 0 && aligned(out, 16), st);
    }
    return dispatch_fast<BITS, IdxT>(p, vec, lut, D % 4 == 0 && aligned(out, 16), st);
  }
  if (peer != nullptr) return set_error(F2C_ERR_UNSUPPORTED, "%s: shape not served by the peer kernel", op);
  if (variant == F2C_KERNEL_PREFETCH || variant == F2C_KERNEL_PREFETCH_ARITH)
    return set_error(F2C_ERR_UNSUPPORTED, "%s: shape not served by the register-prefetch kernel", op);
  int64_t blocks = ceil_div(n_dst, 8);
  if (blocks > current_sm_count() * 32) blocks = current_sm_count() * 32;
#define F2C_GEN(T) sq_spmm_generic_kernel<BITS, T, IdxT><<<(unsigned)blocks, 256, 0, st>>>( \
      codes, codebooks, (const IdxT*)indptr, (const IdxT*)indices, out, n_dst, src_dim, (int)D, (int)cs, reduce, drop)
  if (code_dtype == F2C_I8) F2C_GEN(int8_t);
  else if (code_dtype == F2C_U8) F2C_GEN(uint8_t);
  else F2C_GEN(int16_t);
#undef F2C_GEN
  return check_launch(op);
}

}  // namespace f2c

using namespace f2c;

extern "C" int f2c_sq_spmm_csr(const void* codes, int code_dtype, const float* codebooks, int64_t n_codebooks,
                               const void* indptr, const void* indices, int index_dtype, float* out, int64_t n_dst,
                               int64_t n_src, int64_t src_dim, int64_t feat_dim, int bits, int64_t column_slice, int reduce,
                               const f2c_epilogue* epilogue, void* stream) {
  const char* op = "sq_decompress_spmm_csr";
  F2C_REQUIRE(n_dst >= 0 && n_src >= 0, F2C_ERR_INVALID, "%s: negative size", op);
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
  const int variant = kernel_variant(epilogue);
  cudaStream_t st = (cudaStream_t)stream;
#define F2C_SQ(B)                                                                                                   \
  return index_dtype == F2C_I32                                                                                     \
             ? launch_sq_spmm<B, int32_t>(codes, code_dtype, codebooks, n_codebooks, indptr, indices, out, n_dst,   \
                                          n_src, src_dim, feat_dim, column_slice, reduce, drop, variant, st)                \
             : launch_sq_spmm<B, int64_t>(codes, code_dtype, codebooks, n_codebooks, indptr, indices, out, n_dst,   \
                                          n_src, src_dim, feat_dim, column_slice, reduce, drop, variant, st)
  switch (bits) {
    case 1: F2C_SQ(1);
    case 2: F2C_SQ(2);
    case 4: F2C_SQ(4);
    case 8: F2C_SQ(8);
    default: F2C_SQ(16);
  }
#undef F2C_SQ
}

extern "C" int f2c_sq_spmm_csr_peer(const void* const* shard_ptrs_host, int world, int64_t rows_per_shard, int code_dtype,
                                    const float* codebooks, int64_t n_codebooks, const void* indptr, const void* indices,
                                    int index_dtype, float* out, int64_t n_dst, int64_t n_src, int64_t src_dim,
                                    int64_t feat_dim, int bits, int64_t column_slice, int reduce,
                                    const f2c_epilogue* epilogue, void* stream) {
  return f2c_sq_spmm_csr_peer_hot(nullptr, 0, shard_ptrs_host, world, rows_per_shard, code_dtype, codebooks, n_codebooks, indptr, indices,
                                  index_dtype, out, n_dst, n_src, src_dim, feat_dim, bits, column_slice, reduce, epilogue, stream);
}

extern "C" int64_t f2c_peer_hot_first_cold_id(int64_t n_replicated, int64_t rows_per_shard) {
  if (n_replicated <= 0 || rows_per_shard <= 0) return 0;
  return ceil_div(n_replicated, rows_per_shard) * rows_per_shard;
}

extern "C" int f2c_sq_spmm_csr_peer_hot(const void* replicated_rows, int64_t n_replicated, const void* const* shard_ptrs_host, int world,
                                        int64_t rows_per_shard, int code_dtype, const float* codebooks, int64_t n_codebooks,
                                        const void* indptr, const void* indices, int index_dtype, float* out, int64_t n_dst,
                                        int64_t n_src, int64_t src_dim, int64_t feat_dim, int bits, int64_t column_slice, int reduce,
                                        const f2c_epilogue* epilogue, void* stream) {
  const char* op = "sq_decompress_spmm_csr_peer";
  F2C_REQUIRE(n_dst >= 0 && n_src >= 0, F2C_ERR_INVALID, "%s: negative size", op);
  F2C_REQUIRE(world >= 1 && world <= 8, F2C_ERR_LIMIT, "%s: 1 to 8 shards (got %d)", op, world);
  F2C_REQUIRE(rows_per_shard >= 2 && rows_per_shard < (1ll << 32), F2C_ERR_INVALID, "%s: rows_per_shard must be in [2, 2^32)", op);
  const int64_t first_cold = f2c_peer_hot_first_cold_id(n_replicated, rows_per_shard);
  F2C_REQUIRE(n_replicated == 0 || aligned(replicated_rows, 16), F2C_ERR_INVALID, "%s: the replicated rows must be 16-byte aligned", op);
  F2C_REQUIRE(n_replicated >= 0 && (n_replicated == 0 || replicated_rows != nullptr) && first_cold / rows_per_shard + world <= 16,
              F2C_ERR_INVALID, "%s: bad replicated row range (the replicated rows and the shards share 16 slots of rows_per_shard ids)", op);
  F2C_REQUIRE(first_cold + rows_per_shard * world >= n_src, F2C_ERR_INVALID,
              "%s: ids up to %lld are not covered by %lld replicated rows and %d shards of %lld rows", op, (long long)n_src,
              (long long)n_replicated, world, (long long)rows_per_shard);
  F2C_REQUIRE(shard_ptrs_host != nullptr, F2C_ERR_INVALID, "%s: null pointer", op);
  int rc = validate_sq(op, code_dtype, n_codebooks, src_dim, feat_dim, bits, column_slice);
  if (rc) return rc;
  F2C_REQUIRE(is_index_dtype(index_dtype), F2C_ERR_UNSUPPORTED, "%s: indptr/indices must be int32 or int64", op);
  F2C_REQUIRE(reduce == F2C_MEAN || reduce == F2C_SUM, F2C_ERR_INVALID, "%s: reduce must be mean or sum", op);
  F2C_REQUIRE(bits >= 8 || n_codebooks == 1 || column_slice % (8 / bits) == 0, F2C_ERR_INVALID,
              "%s: column_slice (%lld) must be a multiple of %d for %d-bit codes", op, (long long)column_slice, 8 / bits, bits);
  F2C_REQUIRE(n_dst * feat_dim == 0 || (indptr && out && codebooks), F2C_ERR_INVALID, "%s: null pointer", op);
  PeerInfo peer{};
  int here = 0;
#define F2C_PEER_CUDA(call)                                                                       \
  do {                                                                                           \
    cudaError_t e_ = (call);                                                                     \
    if (e_ != cudaSuccess) {                                                                     \
      (void)cudaGetLastError();                                                                  \
      return set_error(F2C_ERR_CUDA, "%s: %s failed: %s", op, #call, cudaGetErrorString(e_));  \
    }                                                                                            \
  } while (0)
  F2C_PEER_CUDA(cudaGetDevice(&here));
  for (int r = 0; r < world; ++r) {
    F2C_REQUIRE(shard_ptrs_host[r] != nullptr, F2C_ERR_INVALID, "%s: shard %d is null", op, r);
    peer.shard[r] = shard_ptrs_host[r];
    // A shard that lives on another GPU must be readable from the launching device: peer access is one-directional,
    // so it is requested here (idempotent; f2c_shard_open has normally enabled it already).
    cudaPointerAttributes attr{};
    F2C_PEER_CUDA(cudaPointerGetAttributes(&attr, shard_ptrs_host[r]));
    F2C_REQUIRE(attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged, F2C_ERR_INVALID,
                "%s: shard %d is not device memory", op, r);
    if (attr.type == cudaMemoryTypeDevice && attr.device != here) {
      int can = 0;
      F2C_PEER_CUDA(cudaDeviceCanAccessPeer(&can, here, attr.device));
      F2C_REQUIRE(can, F2C_ERR_UNSUPPORTED, "%s: GPU %d cannot read shard %d on GPU %d (no peer access)", op, here, r,
                  attr.device);
      cudaError_t e = cudaDeviceEnablePeerAccess(attr.device, 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) {
        (void)cudaGetLastError();
      } else {
        F2C_PEER_CUDA(e);
      }
    }
  }
#undef F2C_PEER_CUDA
  peer.world = world;
  peer.rows_per_shard = rows_per_shard;
  peer.replicated = replicated_rows;
  peer.n_replicated = n_replicated;
  DropoutArgs drop = make_dropout(epilogue);
  const int variant = kernel_variant(epilogue);
  cudaStream_t st = (cudaStream_t)stream;
#define F2C_SQP(B)                                                                                                       \
  return index_dtype == F2C_I32                                                                                          \
             ? launch_sq_spmm<B, int32_t>(peer.shard[0], code_dtype, codebooks, n_codebooks, indptr, indices, out, n_dst, \
                                          n_src, src_dim, feat_dim, column_slice, reduce, drop, variant, st, &peer)              \
             : launch_sq_spmm<B, int64_t>(peer.shard[0], code_dtype, codebooks, n_codebooks, indptr, indices, out, n_dst, \
                                          n_src, src_dim, feat_dim, column_slice, reduce, drop, variant, st, &peer)
  switch (bits) {
    case 1: F2C_SQP(1);
    case 2: F2C_SQP(2);
    case 4: F2C_SQP(4);
    case 8: F2C_SQP(8);
    default: F2C_SQP(16);
  }
#undef F2C_SQP
}
