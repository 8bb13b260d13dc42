// Pipelined fused VQ decode + aggregation and the single-launch two-level (hot rows SQ, all other rows VQ)
// aggregation for the common shapes: uint8 codes, 4/8/16 code bytes per row, column_slice in {4,...,128} dividing
// 128, hot rows 8- or 4-bit SQ.  Same arithmetic and CSC summation order as the general kernels of
// fused_vq_spmm.cu (reference: src/fusion_spmm.cu:72-141 for VQ, src/sq_quantization.cu:123-153 for the hot rows).
//
// Why it is shaped like this.  A VQ row is 4..16 bytes, so HBM moves little; every edge pulls feat_dim floats out
// of shared memory (four 128-byte wavefronts per 128 columns) and sits at the end of a chain of dependent global
// loads: indptr -> indices -> (slot ->) code row / hot row.  One warp owns one destination row at a time (a lane
// owns four consecutive columns: one LDS.128 per VQ edge, a coalesced 512-byte row store), and the chain is
// software-pipelined ACROSS the warp's rows: in one loop iteration a warp aggregates row i from registers and
// shared memory while the hot-row bytes of row i+1, the codes and slots of row i+2, the neighbour ids of row i+3
// and the indptr pair of row i+4 are in flight.  Every stage starts by consuming what the previous iteration
// loaded and then re-uses the same registers for its own loads, so no load result is copied while in flight.
//
//  * Codebooks are staged once per CTA.  For column_slice < 32 the subspaces that one quarter-warp reads are
//    interleaved inside 128-byte lines, so that the eight lanes of a quarter-warp always hit eight different
//    16-byte bank groups whatever the codes are (natural layout: conflicts whenever two codes differ by a
//    multiple of 128 / (4*column_slice)).
//  * Lane t of the warp holds neighbour t of the row (id, slot, code row); code rows are handed to the other lanes
//    through a per-warp shared-memory tile (one STS per row, one broadcast LDS.U8 per edge and lane).
//  * Hot rows are decoded through a byte-indexed table built with the same expression as the element-wise decode
//    (same bits), one private copy per lane and bank: a lookup never conflicts.
#include "vq_params.cuh"

namespace f2c {
namespace vqf {

// Threads per CTA (one CTA per SM).  Measured on B200 (config-3 / config-4 blocks): the two-level kernel is fastest with
// 768 threads (85 registers each: no spills, fewer constant reloads; 1024 threads: +9 %, 512: +30 %), the VQ-only
// kernel with 896.
template <int HB> struct VqCta {
  static constexpr int kThreads = HB != 0 ? 768 : 896;
  static constexpr int kWarps = kThreads / 32;
};
constexpr int U = 16;  // hot rows prefetched per destination row (neighbours beyond are fetched on the spot)
constexpr int kLutBytes = 256 * 256;
constexpr size_t kSmemLimit = 227 * 1024;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t lds_u8(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ float4 lds_f4(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ float2 lds_f2(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ float lds_f1(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t ldg_nc_u16(const void* p) {
  uint16_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}

template <int ROWW> struct CodeRow { uint32_t w[ROWW]; };
template <int ROWW> __device__ __forceinline__ void load_code_row(CodeRow<ROWW>& c, const void* p) {
  if (ROWW == 1) c.w[0] = ldg_nc_u32(p);
  else if (ROWW == 2) { uint2 v = ldg_nc_u64(p); c.w[0] = v.x; c.w[1] = v.y; }
  else { uint4 v = ldg_nc_u128(p); c.w[0] = v.x; c.w[1] = v.y; c.w[ROWW > 2 ? 2 : 0] = v.z; c.w[ROWW > 3 ? 3 : 0] = v.w; }
}

// HB = 0: VQ only.  HB = 8 / 4: two-level with 8- / 4-bit hot rows.  ROWW = 32-bit words of one VQ code row.
// PEER: the three tables are row-sharded over the GPUs of the box and every shard is mapped into this process; rows of
// other ranks are read with ordinary loads over NVLink (no collective, no staging copy, nothing waits on another rank).
template <int HB, typename IdxT, int ROWW, bool PEER = false>
__global__ void __launch_bounds__(VqCta<HB>::kThreads, 1) vq_fast_kernel(const VqParams p) {
  constexpr int kThreads = VqCta<HB>::kThreads, kWarps = VqCta<HB>::kWarps;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* cb_s = smem;
  unsigned char* lut_s = smem + p.fast_cb_bytes;
  unsigned char* wbuf_all = lut_s + (HB != 0 ? kLutBytes : 0);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  constexpr int ROWB = ROWW * 4;

  const int part = blockIdx.y;
  const int s_begin = part * p.cb_per_part;
  const int s_end = min(s_begin + p.cb_per_part, p.n_cb);
  const int col_begin = s_begin * p.cs;
  const int col_end = min(s_end * p.cs, p.feat_dim);
  const int K = (int)p.K, cs = p.cs, spq = p.fast_spq, stride = p.fast_stride;

  // ---- stage this part's codebooks (layout in the header comment); column_slice is a power of two here.
  //      Consecutive threads write consecutive 16-byte pieces of shared memory (no bank conflicts while staging).
  {
    const int lg4 = 31 - __clz(cs >> 2);  // log2(float4 pieces per centroid)
    const int n_sub = s_end - s_begin;
    const float4* src = reinterpret_cast<const float4*>(p.codebooks + (int64_t)s_begin * K * cs);
    float4* dst = reinterpret_cast<float4*>(cb_s);
    if (spq > 1) {  // 128-byte line = the centroids `code` of spq consecutive subspaces
      const int n16 = ((n_sub + spq - 1) / spq) * K * 8;
      for (int i = threadIdx.x; i < n16; i += kThreads) {
        const int piece = i & 7, line = i >> 3;
        const int code = line % K, grp = line / K;
        const int sl = grp * spq + (piece >> lg4), q = piece & ((1 << lg4) - 1);
        dst[i] = sl < n_sub ? __ldg(src + ((sl * K + code) << lg4) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    } else {        // natural layout: the staged image equals the global one
      const int n16 = (n_sub * K) << lg4;
      for (int i = threadIdx.x; i < n16; i += kThreads) dst[i] = __ldg(src + i);
    }
  }
  // ---- hot-row decode table: entry (byte, lane) = the floats that `byte` decodes to with the codebook row of
  //      that lane's columns; slab `byte` starts at byte * 256, a lane's entry is 4 (8-bit) or 8 (4-bit) bytes
  if (HB != 0) {
    const int l = threadIdx.x & 31;
    int lcol = col_begin + 4 * l;
    if (lcol >= col_end) lcol = col_begin;
    int row = lcol / p.sq_cs;
    if (row >= p.sq_n_cb) row = p.sq_n_cb - 1;
    const float emin = __ldg(p.sq_codebooks + row * kCodebookDim + 2), emax = __ldg(p.sq_codebooks + row * kCodebookDim + 3);
    const float mean = __ldg(p.sq_codebooks + row * kCodebookDim + 4);
    for (int byte = threadIdx.x >> 5; byte < 256; byte += kWarps) {
      if (HB == 8) {
        const float c = p.sq_signed ? (float)(int8_t)byte : (float)byte;
        reinterpret_cast<float*>(lut_s + byte * 256)[l] = sq_decode<8>(c, sq_scale<8>(emin, emax), emin, mean);
      } else {
        const float sc = sq_scale<4>(emin, emax);
        reinterpret_cast<float2*>(lut_s + byte * 256)[l] =
            make_float2(sq_decode<4>((float)(byte & 15), sc, emin, mean), sq_decode<4>((float)(byte >> 4), sc, emin, mean));
      }
    }
  }
  __syncthreads();

  // ---- lane constants
  const int col = col_begin + 4 * lane;
  const bool active = col < col_end;
  const int colc = active ? col : col_begin;
  const int s = colc / cs, sl = s - s_begin, off = colc - s * cs;
  const uint32_t lane_base = spq > 1 ? (uint32_t)((sl / spq) * K * 128 + (sl % spq) * cs * 4 + off * 4)
                                     : (uint32_t)(sl * K * stride + off * 4);
  const uint32_t cb_addr = smem_u32(cb_s) + lane_base;
  uint32_t* wbuf = reinterpret_cast<uint32_t*>(wbuf_all) + wid * 32 * ROWW;
  const uint32_t wb_addr = smem_u32(wbuf) + (uint32_t)s;  // byte s of every staged code row
  const uint32_t hot_col_off = (uint32_t)((colc * (HB == 0 ? 8 : HB)) / 8);
  const uint8_t* hot_base = (HB != 0 && !PEER) ? p.sq_codes + hot_col_off : nullptr;
  const uint32_t hot_row_bytes = (uint32_t)p.sq_row_bytes;
  const bool clamp = K < 256;

  const IdxT* __restrict__ indptr = reinterpret_cast<const IdxT*>(p.indptr);
  const IdxT* __restrict__ indices = reinterpret_cast<const IdxT*>(p.indices);
  const uint8_t* __restrict__ codes = reinterpret_cast<const uint8_t*>(p.codes);

  float4 acc;
  auto add_vq = [&](uint32_t edge_byte_addr) {
    const uint32_t code = lds_u8(edge_byte_addr);
    const float4 v = lds_f4(cb_addr + code * (uint32_t)stride);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  };
  const uint32_t lane_off = (uint32_t)lane * (HB == 4 ? 8u : 4u);  // < 256: fits the low byte of the permute result
  const uint32_t lut_base = smem_u32(lut_s);
  auto add_hot = [&](uint32_t w) {
    if (HB == 8) {
      const float v0 = lds_f1(lut_base + __byte_perm(w, lane_off, 0x7704)), v1 = lds_f1(lut_base + __byte_perm(w, lane_off, 0x7714));
      const float v2 = lds_f1(lut_base + __byte_perm(w, lane_off, 0x7724)), v3 = lds_f1(lut_base + __byte_perm(w, lane_off, 0x7734));
      acc.x += v0; acc.y += v1; acc.z += v2; acc.w += v3;
    } else {
      const float2 a = lds_f2(lut_base + __byte_perm(w, lane_off, 0x7704)), b = lds_f2(lut_base + __byte_perm(w, lane_off, 0x7714));
      acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
    }
  };
  auto load_hot = [&](int sl_) -> uint32_t {
    const uint8_t* q;
    if (PEER) {
      const uint32_t owner = (uint32_t)__umul64hi((unsigned long long)(uint32_t)sl_, p.peer.magic_hot);
      q = p.peer.hot[owner] + hot_col_off + (uint64_t)((uint32_t)sl_ - owner * p.peer.rps_hot) * hot_row_bytes;
    } else {
      q = hot_base + (uint64_t)(uint32_t)sl_ * hot_row_bytes;
    }
    return HB == 8 ? ldg_nc_u32(q) : ldg_nc_u16(q);
  };
  // code row and slot of source node `id`
  auto fetch_node = [&](int64_t id, CodeRow<ROWW>& c, int& sl_) {
    if (PEER) {
      const uint32_t owner = (uint32_t)__umul64hi((unsigned long long)id, p.peer.magic_nodes);
      const uint32_t local = (uint32_t)id - owner * p.peer.rps_nodes;
      load_code_row<ROWW>(c, p.peer.code[owner] + (uint64_t)local * ROWB);
      if (HB != 0) sl_ = p.peer.slot[0] != nullptr ? __ldg(p.peer.slot[owner] + local) : (id < p.n_hot ? (int)id : -1);
    } else {
      load_code_row<ROWW>(c, codes + id * ROWB);
      if (HB != 0) sl_ = hot_slot_of(p, id);
    }
  };
  auto stage_codes = [&](const CodeRow<ROWW>& c, int cnt) {
    if (lane < cnt) {
#pragma unroll
      for (int w = 0; w < ROWW; ++w) {
        uint32_t x = c.w[w];
        if (clamp) {  // codes >= K read the last centroid, as the general kernel does
          uint32_t y = 0;
#pragma unroll
          for (int b = 0; b < 4; ++b) y |= min((x >> (8 * b)) & 0xFFu, (uint32_t)(K - 1)) << (8 * b);
          x = y;
        }
        wbuf[lane * ROWW + w] = x;
      }
    }
  };

  // ---- pipeline state.  Rows of this warp: r0, r0 + W, r0 + 2W, ...; stage k of iteration `it` works on row
  //      r0 + (it - k) * W for k = 0 (indptr) .. 4 (aggregate).
  const int n_dst = (int)p.n_dst;
  const int W = (int)gridDim.x * kWarps;
  const int r0 = (int)blockIdx.x * kWarps + wid;
  IdxT ptr_lo = 0, ptr_hi = 0;       // indptr pair            (loaded by stage 0, read by stage 1)
  int64_t beg1 = 0; int deg1 = 0;    // row of stage 1 -> 2
  IdxT idx2 = 0;                     // neighbour id of lane   (loaded by stage 1, read by stage 2)
  int64_t beg2 = 0; int deg2 = 0;    // row of stage 2 -> 3
  CodeRow<ROWW> code3;               // code row of lane's edge (loaded by stage 2, read by stage 3)
  int slot3 = -1;                    // slot of lane's edge     (loaded by stage 2, read by stage 3)
  int64_t beg3 = 0; int deg3 = 0;
  CodeRow<ROWW> code4;               // handed from stage 3 to stage 4
  int slot4 = -1; uint32_t mask4 = 0u;
  int64_t beg4 = 0; int deg4 = 0;
  uint32_t hot[HB != 0 ? U : 1];     // hot-row bytes of this lane's columns (loaded by stage 3, read by stage 4)
#pragma unroll
  for (int w = 0; w < ROWW; ++w) { code3.w[w] = 0u; code4.w[w] = 0u; }
#pragma unroll
  for (int u = 0; u < (HB != 0 ? U : 1); ++u) hot[u] = 0u;

  for (int rP = r0;; rP += W) {
    const int rE = rP - 4 * W;  // row aggregated in this iteration
    if (rE >= n_dst) break;
    // ================= stage 4: aggregate row rE
    if (rE >= r0) {
      acc = make_float4(0.f, 0.f, 0.f, 0.f);
      const int cnt0 = min(deg4, 32);
      __syncwarp();
      stage_codes(code4, cnt0);
      __syncwarp();
      if (HB != 0) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (u >= cnt0) break;
          if ((mask4 >> u) & 1u) add_hot(hot[u]);
          else add_vq(wb_addr + u * ROWB);
        }
        for (int u = U; u < cnt0; ++u) {
          const int sl_ = __shfl_sync(0xffffffffu, slot4, u);
          if (sl_ >= 0) add_hot(load_hot(sl_));
          else add_vq(wb_addr + u * ROWB);
        }
      } else {
        int u = 0;
        for (; u + 4 <= cnt0; u += 4) {
          const uint32_t c0 = lds_u8(wb_addr + u * ROWB), c1 = lds_u8(wb_addr + (u + 1) * ROWB);
          const uint32_t c2 = lds_u8(wb_addr + (u + 2) * ROWB), c3 = lds_u8(wb_addr + (u + 3) * ROWB);
          const float4 v0 = lds_f4(cb_addr + c0 * (uint32_t)stride), v1 = lds_f4(cb_addr + c1 * (uint32_t)stride);
          const float4 v2 = lds_f4(cb_addr + c2 * (uint32_t)stride), v3 = lds_f4(cb_addr + c3 * (uint32_t)stride);
          acc.x += v0.x; acc.y += v0.y; acc.z += v0.z; acc.w += v0.w;
          acc.x += v1.x; acc.y += v1.y; acc.z += v1.z; acc.w += v1.w;
          acc.x += v2.x; acc.y += v2.y; acc.z += v2.z; acc.w += v2.w;
          acc.x += v3.x; acc.y += v3.y; acc.z += v3.z; acc.w += v3.w;
        }
        for (; u < cnt0; ++u) add_vq(wb_addr + u * ROWB);
      }
      // rows with more than 32 neighbours: further batches, fetched on the spot
      for (int64_t k0 = beg4 + 32; k0 < beg4 + deg4; k0 += 32) {
        const int cnt = (int)min((int64_t)32, beg4 + deg4 - k0);
        CodeRow<ROWW> c;
#pragma unroll
        for (int w = 0; w < ROWW; ++w) c.w[w] = 0u;
        int sl_mine = -1;
        if (lane < cnt) {
          const int64_t id = (int64_t)indices[k0 + lane];
          fetch_node(id, c, sl_mine);
        }
        __syncwarp();
        stage_codes(c, cnt);
        __syncwarp();
        for (int u = 0; u < cnt; ++u) {
          const int sl_ = HB != 0 ? __shfl_sync(0xffffffffu, sl_mine, u) : -1;
          if (HB != 0 && sl_ >= 0) add_hot(load_hot(sl_));
          else add_vq(wb_addr + u * ROWB);
        }
      }
      if (active) {
        if (p.reduce == F2C_MEAN) {
          const float degf = deg4 == 0 ? 1.0f : (float)deg4;
          acc.x = acc.x / degf; acc.y = acc.y / degf; acc.z = acc.z / degf; acc.w = acc.w / degf;
        }
        const int64_t flat = (int64_t)rE * p.feat_dim + col;
        if (p.drop.enabled) acc = dropout_apply4(acc, (uint64_t)flat, p.drop);
        stg_cs_f4(p.out + flat, acc);
      }
    }
    // ================= stage 3: row rP - 3W: its slots and codes have arrived; fetch the hot rows
    {
      const int rH = rP - 3 * W;
      const bool on = rH >= r0 && rH < n_dst;
      beg4 = beg3; deg4 = on ? deg3 : 0;
#pragma unroll
      for (int w = 0; w < ROWW; ++w) code4.w[w] = code3.w[w];
      if (HB != 0) {
        slot4 = on ? slot3 : -1;
        mask4 = __ballot_sync(0xffffffffu, slot4 >= 0);
        if (mask4 != 0u) {
#pragma unroll
          for (int u = 0; u < U; ++u) {
            if ((mask4 >> u) == 0u) break;
            if ((mask4 >> u) & 1u) hot[u] = load_hot(__shfl_sync(0xffffffffu, slot4, u));
          }
        }
      }
    }
    // ================= stage 2: row rP - 2W: its neighbour ids have arrived; fetch slots and code rows
    {
      const int rC = rP - 2 * W;
      const bool on = rC >= r0 && rC < n_dst;
      beg3 = beg2; deg3 = on ? deg2 : 0;
      slot3 = -1;
      if (on && lane < min(deg2, 32)) {
        const int64_t id = (int64_t)idx2;
        fetch_node(id, code3, slot3);
      }
    }
    // ================= stage 1: row rP - W: its indptr pair has arrived; fetch the neighbour ids
    {
      const int rI = rP - W;
      const bool on = rI >= r0 && rI < n_dst;
      beg2 = (int64_t)ptr_lo; deg2 = on ? (int)((int64_t)ptr_hi - (int64_t)ptr_lo) : 0;
      if (on && lane < min(deg2, 32)) idx2 = indices[beg2 + lane];
    }
    // ================= stage 0: row rP: fetch its indptr pair
    if (rP < n_dst) { ptr_lo = indptr[rP]; ptr_hi = indptr[rP + 1]; }
  }
}

template <int HB, typename IdxT, bool PEER>
static int launch_rows(const VqParams& p, int roww, dim3 grid, size_t smem, cudaStream_t st, const char* op) {
#define F2C_VQF(RW)                                                                                      \
  {                                                                                                      \
    auto kern = vq_fast_kernel<HB, IdxT, RW, PEER>;                                                      \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    if (e != cudaSuccess) return set_error(F2C_ERR_CUDA, "%s: %s", op, cudaGetErrorString(e));           \
    kern<<<grid, VqCta<HB>::kThreads, smem, st>>>(p);                                                               \
    return check_launch(op);                                                                             \
  }
  if (roww == 1) F2C_VQF(1)
  if (roww == 2) F2C_VQF(2)
  F2C_VQF(4)
#undef F2C_VQF
}

}  // namespace vqf

int launch_vq_stream(VqParams& p, int hot_bits, int index_dtype, cudaStream_t st, const char* op, bool* served);

int launch_vq_fast(VqParams& p, int hot_bits, int index_dtype, int variant, cudaStream_t st, const char* op, bool* served,
                   bool peer) {
  using namespace vqf;
  *served = false;
  if (peer && variant == F2C_KERNEL_STREAM) return F2C_OK;  // sharded tables: this file's kernel only
  // The streamed kernels are selectable but not the default here: on B200 (same block as above) VQ 16 x 8 ties (41-43 us),
  // VQ 4 x 32 is 45-49 us against 35 us and the two-level op 130-140 us against 64 us for this file's kernel.
  if (variant == F2C_KERNEL_STREAM) return launch_vq_stream(p, hot_bits, index_dtype, st, op, served);
  const void* codes_base = peer ? (const void*)p.peer.code[0] : p.codes;
  const void* hot_table = peer ? (const void*)p.peer.hot[0] : (const void*)p.sq_codes;
  const int cs = p.cs;
  const int64_t row_bytes = p.n_cb;  // uint8 codes
  if (p.code_kind != 0 || p.K > 256 || p.n_dst >= (1ll << 30)) return F2C_OK;
  if (!(row_bytes == 4 || row_bytes == 8 || row_bytes == 16) || !aligned(codes_base, (size_t)row_bytes)) return F2C_OK;
  if (cs < 4 || cs > 128 || (128 % cs) != 0 || p.feat_dim % 4 != 0 || !aligned(p.out, 16) || !aligned(p.codebooks, 16)) return F2C_OK;
  if (!(hot_bits == 0 || hot_bits == 8 || hot_bits == 4)) return F2C_OK;
  if (hot_bits != 0) {
    if (p.sq_n_cb > 1 && p.sq_cs % 4 != 0) return F2C_OK;
    const int align = hot_bits == 8 ? 4 : 2;
    if (p.sq_row_bytes % align != 0 || p.sq_row_bytes >= (1ll << 31) || !aligned(hot_table, align)) return F2C_OK;
  }
  // a column part = at most 128 columns whose codebooks fit beside the table and the code tiles
  const int sub_per_128 = 128 / cs;
  const int roww = (int)row_bytes / 4;
  const int kWarps = hot_bits != 0 ? VqCta<8>::kWarps : VqCta<0>::kWarps;
  const size_t fixed = (hot_bits != 0 ? kLutBytes : 0) + (size_t)kWarps * 32 * roww * 4;
  const int spq = cs < 32 ? 32 / cs : 1;
  const int stride = cs < 32 ? 128 : cs * 4;
  int per_part = sub_per_128 < p.n_cb ? sub_per_128 : p.n_cb;
  auto cb_bytes = [&](int n_sub) -> size_t {
    return spq > 1 ? (size_t)ceil_div(n_sub, spq) * p.K * 128 : (size_t)n_sub * p.K * cs * 4;
  };
  if (cb_bytes(per_part) + fixed > kSmemLimit) return F2C_OK;
  p.cb_per_part = per_part;
  p.fast_spq = spq;
  p.fast_stride = stride;
  p.fast_cb_bytes = (int)cb_bytes(per_part);
  const int parts = (int)ceil_div(p.n_cb, per_part);
  int64_t grid_x = current_sm_count() / parts;
  if (grid_x < 1) grid_x = 1;
  const int64_t need = ceil_div(p.n_dst, kWarps);
  if (grid_x > need) grid_x = need;
  dim3 grid((unsigned)grid_x, (unsigned)parts);
  const size_t smem = (size_t)p.fast_cb_bytes + fixed;
  *served = true;
#define F2C_VQF_IDX(HB)                                                                                                            \
  if (peer)                                                                                                                        \
    return index_dtype == F2C_I32 ? launch_rows<HB, int32_t, true>(p, roww, grid, smem, st, op)                                    \
                                  : launch_rows<HB, int64_t, true>(p, roww, grid, smem, st, op);                                   \
  return index_dtype == F2C_I32 ? launch_rows<HB, int32_t, false>(p, roww, grid, smem, st, op)                                     \
                                : launch_rows<HB, int64_t, false>(p, roww, grid, smem, st, op)
  if (hot_bits == 0) { F2C_VQF_IDX(0); }
  if (hot_bits == 8) { F2C_VQF_IDX(8); }
  F2C_VQF_IDX(4);
#undef F2C_VQF_IDX
}

}  // namespace f2c
