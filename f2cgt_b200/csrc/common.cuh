// Shared helpers of the f2cgt_b200 kernels: status/error plumbing, dtype tags, vector loads,
// the SQ decode expression and the Philox generator used by dropout.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/f2cgt_b200.h"

namespace f2c {

constexpr int kSmCount = 148;          // B200: 2 dies x 74 SMs (sizing default; launches ask sm_count() for the device's own figure)
constexpr int kCodebookDim = 5;        // [fmin, fmax, emin, emax, mean] (reference src/sq_quantization.cu:17)

// ---- error plumbing (defined in api.cu) ----
int set_error(int status, const char* fmt, ...);
int check_launch(const char* what);
int sm_count(int device);  // multiprocessors of `device` (queried once per device)
int current_sm_count();     // the same for the current device

#define F2C_REQUIRE(cond, status, ...)                 \
  do {                                                 \
    if (!(cond)) return f2c::set_error((status), __VA_ARGS__); \
  } while (0)

static inline bool is_index_dtype(int dt) { return dt == F2C_I32 || dt == F2C_I64; }
static inline bool is_code_dtype(int dt) { return dt == F2C_U8 || dt == F2C_I8 || dt == F2C_I16; }
static inline bool is_sq_bits(int b) { return b == 1 || b == 2 || b == 4 || b == 8 || b == 16; }
static inline int dtype_size(int dt) {
  switch (dt) {
    case F2C_U8: case F2C_I8: return 1;
    case F2C_I16: case F2C_F16: return 2;
    case F2C_I32: case F2C_F32: return 4;
    default: return 8;
  }
}
static inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- device helpers ----

// Read-only, L1-bypassing vector loads for streamed gathers.
__device__ __forceinline__ uint32_t ldg_nc_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_nc_u64(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_nc_u128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// Streaming (evict-first) 128-bit store for outputs that are written once and not re-read here.
__device__ __forceinline__ void stg_cs_f4(float* p, float4 v) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" :: "l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// SQ decode of one element.  The expression is the reference's, term by term
// (src/sq_quantization.cu:137-152 == src/fusion_spmm.cu:199-223), compiled with the same default
// nvcc math flags (FMA contraction of |c|*s + emin, libdevice exp2f), so the result has the same
// bits as the reference kernel's on the same GPU.  `c` is the raw code as float (unsigned for
// packed widths).  scale = (emax - emin) / drange.
template <int BITS>
__device__ __forceinline__ float sq_decode(float c, float scale, float emin, float mean) {
  if (BITS == 1) {
    return (c - 0.5f) * (2.0f * mean);
  } else {
    constexpr float drange = (float)(1 << (BITS - 1));
    if (BITS < 8) c -= drange;
    c = c + 0.5f;
    float sign = c >= 0.0f ? 1.0f : -1.0f;
    float e = fabsf(c) * scale + emin;
    return exp2f(e) * sign;
  }
}

template <int BITS>
__device__ __forceinline__ float sq_scale(float emin, float emax) {
  constexpr float drange = (float)(1 << (BITS - 1));
  return (emax - emin) / drange;
}

// a / b with the IEEE round-to-nearest result of the division operator, given rcp = 1.0f / b computed
// once per destination row: two Newton corrections through exact FMA residuals (Markstein) replace the
// ~15-instruction division sequence per element.  Values outside the exponent range where the
// residuals are exact (and inf/nan) take the ordinary division.
__device__ __forceinline__ float div_exact(float a, float b, float rcp) {
  float q = a * rcp;
  float r = fmaf(-q, b, a);
  q = fmaf(r, rcp, q);
  r = fmaf(-q, b, a);
  q = fmaf(r, rcp, q);
  const float aa = fabsf(a);
  if (!(aa < 1e30f) || (aa < 1e-30f && aa != 0.0f) || b > 1048576.0f) q = a / b;
  return q;
}

// The same quotient without the range check, for callers that know |a| is 0 or well inside the normal range
// and b is a small integer.
__device__ __forceinline__ float div_exact_fast(float a, float b, float rcp) {
  float q = a * rcp;
  float r = fmaf(-q, b, a);
  q = fmaf(r, rcp, q);
  r = fmaf(-q, b, a);
  return fmaf(r, rcp, q);
}

// Philox4x32-10 (Salmon et al., SC'11).  One call yields four 32-bit words for counter ctr.
struct Philox {
  uint32_t k0, k1, o0, o1;
  __host__ __device__ Philox(uint64_t seed, uint64_t offset)
      : k0((uint32_t)seed), k1((uint32_t)(seed >> 32)), o0((uint32_t)offset), o1((uint32_t)(offset >> 32)) {}
  __device__ __forceinline__ uint4 operator()(uint64_t ctr) const {
    uint32_t c0 = (uint32_t)ctr, c1 = (uint32_t)(ctr >> 32), c2 = o0, c3 = o1;
    uint32_t a = k0, b = k1;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
      uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
      uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
      uint32_t n0 = hi1 ^ c1 ^ a, n2 = hi0 ^ c3 ^ b;
      c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
      a += 0x9E3779B9u; b += 0xBB67AE85u;
    }
    return make_uint4(c0, c1, c2, c3);
  }
};

// Dropout parameters resolved on the host once per launch.
struct DropoutArgs {
  int enabled;       // 0 = identity
  int drop_all;      // p >= 1
  uint32_t threshold;  // drop iff draw < threshold, threshold = floor(p * 2^32)
  float keep_scale;  // 1 or 1/(1-p)
  uint64_t seed, offset;
};

static inline DropoutArgs make_dropout(const f2c_epilogue* ep) {
  DropoutArgs a{0, 0, 0u, 1.0f, 0, 0};
  if (ep == nullptr || !ep->training) return a;
  a.enabled = 1;
  a.drop_all = ep->p >= 1.0f;
  double t = (double)ep->p * 4294967296.0;
  a.threshold = t <= 0 ? 0u : (t >= 4294967295.0 ? 4294967295u : (uint32_t)t);
  a.keep_scale = (ep->scale && ep->p < 1.0f) ? 1.0f / (1.0f - ep->p) : 1.0f;
  a.seed = ep->seed;
  a.offset = ep->offset;
  return a;
}

// Kernel family a caller asked for (f2c_epilogue::kernel); F2C_KERNEL_AUTO without an options struct.
static inline int kernel_variant(const f2c_epilogue* ep) { return ep == nullptr ? F2C_KERNEL_AUTO : ep->kernel; }

__device__ __forceinline__ float dropout_apply(float v, uint32_t draw, const DropoutArgs& a) {
  bool drop = a.drop_all || draw < a.threshold;
  return drop ? 0.0f : v * a.keep_scale;
}

// Dropout of four consecutive elements whose flat index starts at a multiple of four.
__device__ __forceinline__ float4 dropout_apply4(float4 v, uint64_t flat_index, const DropoutArgs& a) {
  Philox ph(a.seed, a.offset);
  uint4 r = ph(flat_index >> 2);
  v.x = dropout_apply(v.x, r.x, a);
  v.y = dropout_apply(v.y, r.y, a);
  v.z = dropout_apply(v.z, r.z, a);
  v.w = dropout_apply(v.w, r.w, a);
  return v;
}

__device__ __forceinline__ float dropout_apply1(float v, uint64_t flat_index, const DropoutArgs& a) {
  Philox ph(a.seed, a.offset);
  uint4 r = ph(flat_index >> 2);
  uint32_t w = (flat_index & 3) == 0 ? r.x : (flat_index & 3) == 1 ? r.y : (flat_index & 3) == 2 ? r.z : r.w;
  return dropout_apply(v, w, a);
}

}  // namespace f2c
