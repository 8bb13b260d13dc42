// In-place Bernoulli dropout (reference operator dropout_inplace, src/fusion_dropout.cu:6-29):
// x[i] = drop ? 0 : x[i], no rescaling of survivors unless asked for, identity when not training.
//
// The reference initialises one XORWOW state per thread from the wall clock, which costs far more
// than the 8 bytes per element it moves and cannot be reproduced.  Here the mask is a pure function
// of (seed, offset, element index): Philox4x32-10 keyed by the seed, counter = index / 4, one 32-bit
// word per element, dropped iff the word is below floor(p * 2^32).  The same function is applied in
// the epilogue of the fused aggregation kernels, so fusing never changes a result.
#include "common.cuh"

namespace f2c {

__global__ void __launch_bounds__(256) dropout_kernel(float* __restrict__ x, int64_t numel, int64_t n_vec, int vec_ok,
                                                      const DropoutArgs a) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  int64_t base = i * 4;
  if (vec_ok && base + 4 <= numel) {
    float4 v = *reinterpret_cast<float4*>(x + base);
    v = dropout_apply4(v, (uint64_t)base, a);
    *reinterpret_cast<float4*>(x + base) = v;
  } else {
    Philox ph(a.seed, a.offset);
    uint4 r = ph((uint64_t)i);
    uint32_t w[4] = {r.x, r.y, r.z, r.w};
    for (int e = 0; e < 4 && base + e < numel; ++e) x[base + e] = dropout_apply(x[base + e], w[e], a);
  }
}

}  // namespace f2c

using namespace f2c;

extern "C" int f2c_dropout(float* x, int64_t numel, float p, int training, uint64_t seed, uint64_t offset, int scale,
                           void* stream) {
  F2C_REQUIRE(numel >= 0, F2C_ERR_INVALID, "dropout_inplace: negative size");
  F2C_REQUIRE(p >= 0.0f && p <= 1.0f, F2C_ERR_INVALID, "dropout_inplace: p must be in [0, 1] (got %f)", (double)p);
  if (!training || numel == 0) return F2C_OK;  // src/fusion_dropout.cu:11: nothing happens outside training
  F2C_REQUIRE(x != nullptr, F2C_ERR_INVALID, "dropout_inplace: null pointer");
  f2c_epilogue ep{p, training, scale, seed, offset};
  DropoutArgs a = make_dropout(&ep);
  int64_t n_vec = ceil_div(numel, 4);
  dropout_kernel<<<(unsigned)ceil_div(n_vec, 256), 256, 0, (cudaStream_t)stream>>>(x, numel, n_vec, aligned(x, 16) ? 1 : 0, a);
  return check_launch("dropout_inplace");
}
