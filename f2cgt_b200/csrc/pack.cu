// Bit packing of 1/2/4-bit codes (reference operators packbits / unpackbits, src/packbits.cu).
// Bit order: element i of a byte sits at bit offset bits*i; rows are padded to whole bytes and never
// share a byte (src/packbits.cu:30-39,46-47).
//
// Both directions are pure byte streams (HBM bound: 1 + bits/8 bytes per element).  When the row
// length is a whole number of bytes the tensor is one flat stream and each thread converts four
// packed bytes with 128-bit accesses on the unpacked side; ragged rows take a per-byte path.
#include "common.cuh"

namespace f2c {

template <int BITS>
__device__ __forceinline__ uint32_t pack_word(const uint8_t* __restrict__ src) {
  // 4 packed bytes <- 4 * (8/BITS) unpacked bytes starting at src (16-byte aligned for BITS<=2... see caller)
  constexpr int PER = 8 / BITS;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  uint32_t out = 0;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    uint32_t byte = 0;
#pragma unroll
    for (int i = 0; i < PER; ++i) byte |= (uint32_t)(src[b * PER + i] & MASK) << (BITS * i);
    out |= byte << (8 * b);
  }
  return out;
}

// Flat fast path: n_words 32-bit packed words, input 4*PER bytes per word (vector loads via uint2/uint4).
template <int BITS>
__global__ void __launch_bounds__(256) pack_flat_kernel(const uint8_t* __restrict__ unpack,
                                                        uint32_t* __restrict__ pack, int64_t n_words) {
  constexpr int PER = 8 / BITS;
  constexpr int IN_BYTES = 4 * PER;  // 8, 16 or 32
  int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (w >= n_words) return;
  alignas(16) uint8_t buf[IN_BYTES];
  const uint8_t* p = unpack + w * IN_BYTES;
  if (IN_BYTES == 8) {
    *reinterpret_cast<uint2*>(buf) = *reinterpret_cast<const uint2*>(p);
  } else {
#pragma unroll
    for (int i = 0; i < IN_BYTES / 16; ++i)
      reinterpret_cast<uint4*>(buf)[i] = reinterpret_cast<const uint4*>(p)[i];
  }
  pack[w] = pack_word<BITS>(buf);
}

template <int BITS>
__global__ void __launch_bounds__(256) pack_generic_kernel(const uint8_t* __restrict__ unpack,
                                                           uint8_t* __restrict__ pack, int64_t n_out,
                                                           int64_t unpack_dim, int64_t pack_dim) {
  constexpr int PER = 8 / BITS;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= n_out) return;
  int64_t row = o / pack_dim, col = o % pack_dim;
  int64_t begin = col * PER;
  int64_t end = begin + PER < unpack_dim ? begin + PER : unpack_dim;
  const uint8_t* src = unpack + row * unpack_dim;
  uint32_t v = 0;
  for (int64_t i = begin; i < end; ++i) v |= (uint32_t)(src[i] & MASK) << (BITS * (int)(i - begin));
  pack[o] = (uint8_t)v;
}

template <int BITS>
__global__ void __launch_bounds__(256) unpack_flat_kernel(const uint32_t* __restrict__ pack,
                                                          uint8_t* __restrict__ unpack, int64_t n_words) {
  constexpr int PER = 8 / BITS;
  constexpr int OUT_BYTES = 4 * PER;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (w >= n_words) return;
  uint32_t word = pack[w];
  alignas(16) uint8_t buf[OUT_BYTES];
#pragma unroll
  for (int i = 0; i < OUT_BYTES; ++i) buf[i] = (uint8_t)((word >> (BITS * i)) & MASK);
  uint8_t* p = unpack + w * OUT_BYTES;
  if (OUT_BYTES == 8) {
    *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(buf);
  } else {
#pragma unroll
    for (int i = 0; i < OUT_BYTES / 16; ++i) reinterpret_cast<uint4*>(p)[i] = reinterpret_cast<const uint4*>(buf)[i];
  }
}

template <int BITS>
__global__ void __launch_bounds__(256) unpack_generic_kernel(const uint8_t* __restrict__ pack,
                                                             uint8_t* __restrict__ unpack, int64_t n_out,
                                                             int64_t unpack_dim, int64_t pack_dim) {
  constexpr int PER = 8 / BITS;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= n_out) return;
  int64_t row = o / unpack_dim, col = o % unpack_dim;
  unpack[o] = (uint8_t)((pack[row * pack_dim + col / PER] >> (BITS * (int)(col % PER))) & MASK);
}

template <int BITS>
static int launch_pack(const uint8_t* unpack, uint8_t* pack, int64_t rows, int64_t unpack_dim, cudaStream_t st) {
  constexpr int PER = 8 / BITS;
  int64_t pack_dim = ceil_div(unpack_dim, PER);
  int64_t n_out = rows * pack_dim;
  if (n_out == 0) return F2C_OK;
  bool flat = unpack_dim % PER == 0 && n_out % 4 == 0 && aligned(unpack, 16) && aligned(pack, 4);
  if (flat) {
    int64_t n_words = n_out / 4;
    pack_flat_kernel<BITS><<<(unsigned)ceil_div(n_words, 256), 256, 0, st>>>(unpack, (uint32_t*)pack, n_words);
  } else {
    pack_generic_kernel<BITS><<<(unsigned)ceil_div(n_out, 256), 256, 0, st>>>(unpack, pack, n_out, unpack_dim, pack_dim);
  }
  return check_launch("packbits");
}

template <int BITS>
static int launch_unpack(const uint8_t* pack, uint8_t* unpack, int64_t rows, int64_t pack_dim, int64_t unpack_dim,
                         cudaStream_t st) {
  constexpr int PER = 8 / BITS;
  int64_t n_out = rows * unpack_dim;
  if (n_out == 0) return F2C_OK;
  bool flat = unpack_dim == pack_dim * PER && (rows * pack_dim) % 4 == 0 && aligned(unpack, 16) && aligned(pack, 4);
  if (flat) {
    int64_t n_words = rows * pack_dim / 4;
    unpack_flat_kernel<BITS><<<(unsigned)ceil_div(n_words, 256), 256, 0, st>>>((const uint32_t*)pack, unpack, n_words);
  } else {
    unpack_generic_kernel<BITS><<<(unsigned)ceil_div(n_out, 256), 256, 0, st>>>(pack, unpack, n_out, unpack_dim, pack_dim);
  }
  return check_launch("unpackbits");
}

}  // namespace f2c

using namespace f2c;

extern "C" int f2c_packbits(const uint8_t* unpack, uint8_t* pack, int64_t rows, int64_t unpack_dim, int bits,
                            void* stream) {
  F2C_REQUIRE(rows >= 0 && unpack_dim >= 0, F2C_ERR_INVALID, "packbits: negative size");
  F2C_REQUIRE(bits == 1 || bits == 2 || bits == 4, F2C_ERR_UNSUPPORTED,
              "packbits: target_bits must be 1, 2 or 4 (got %d)", bits);
  F2C_REQUIRE(rows * unpack_dim == 0 || (unpack && pack), F2C_ERR_INVALID, "packbits: null pointer");
  F2C_REQUIRE(rows * unpack_dim < (int64_t)1 << 40, F2C_ERR_LIMIT, "packbits: more than 2^40 elements");
  cudaStream_t st = (cudaStream_t)stream;
  switch (bits) {
    case 1: return launch_pack<1>(unpack, pack, rows, unpack_dim, st);
    case 2: return launch_pack<2>(unpack, pack, rows, unpack_dim, st);
    default: return launch_pack<4>(unpack, pack, rows, unpack_dim, st);
  }
}

extern "C" int f2c_unpackbits(const uint8_t* pack, uint8_t* unpack, int64_t rows, int64_t pack_dim,
                              int64_t unpack_dim, int bits, void* stream) {
  F2C_REQUIRE(rows >= 0 && unpack_dim >= 0 && pack_dim >= 0, F2C_ERR_INVALID, "unpackbits: negative size");
  F2C_REQUIRE(bits == 1 || bits == 2 || bits == 4, F2C_ERR_UNSUPPORTED,
              "unpackbits: target_bits must be 1, 2 or 4 (got %d)", bits);
  F2C_REQUIRE(unpack_dim <= pack_dim * (8 / bits), F2C_ERR_INVALID,
              "unpackbits: unpack_dim %lld exceeds the %lld elements a packed row holds", (long long)unpack_dim,
              (long long)(pack_dim * (8 / bits)));
  F2C_REQUIRE(rows * unpack_dim == 0 || (unpack && pack), F2C_ERR_INVALID, "unpackbits: null pointer");
  F2C_REQUIRE(rows * unpack_dim < (int64_t)1 << 40, F2C_ERR_LIMIT, "unpackbits: more than 2^40 elements");
  cudaStream_t st = (cudaStream_t)stream;
  switch (bits) {
    case 1: return launch_unpack<1>(pack, unpack, rows, pack_dim, unpack_dim, st);
    case 2: return launch_unpack<2>(pack, unpack, rows, pack_dim, unpack_dim, st);
    default: return launch_unpack<4>(pack, unpack, rows, pack_dim, unpack_dim, st);
  }
}
