// Scalar helpers shared by the SIMT kernels and the tensor-core epilogues: output formats, 16-bit packing and the
// approximate exp2 / tanh the softmax math is built on.
//
// With FLCE_HOST_EMULATION defined the two PTX instructions are replaced by libm calls, so that the SIMT kernels
// (row_kernels.cuh, ce_kernels.cuh) can be compiled by a host compiler and run on the host by the CPU tests.
// The library itself is never built that way.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

#ifdef FLCE_HOST_EMULATION
#include <cmath>
#endif

namespace flce {

constexpr float kLog2e = 1.4426950408889634f;

enum OutFormat : int { kOutBf16 = 0, kOutFp16 = 1, kOutFp32 = 2 };

__device__ __forceinline__ uint32_t pack2(float a, float b, int fmt) {
  if (fmt == kOutBf16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float ex2_approx(float x) {
#ifdef FLCE_HOST_EMULATION
  return std::exp2(x);
#else
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
#endif
}

// natural logarithm through lg2.approx (absolute error of the base-2 logarithm about 2^-22 for normal inputs)
__device__ __forceinline__ float ln_approx(float x) {
#ifdef FLCE_HOST_EMULATION
  return std::log(x);
#else
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y * 0.6931471805599453f;
#endif
}

__device__ __forceinline__ float rcp_approx(float x) {
#ifdef FLCE_HOST_EMULATION
  return 1.f / x;
#else
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
#endif
}

// *dst += v for four consecutive floats (16-byte aligned) as one reduction at L2: nothing comes back, nothing to wait for
__device__ __forceinline__ void vector_add_f32x4(float4* dst, const float4& v) {
#ifdef FLCE_HOST_EMULATION
  dst->x += v.x;
  dst->y += v.y;
  dst->z += v.z;
  dst->w += v.w;
#else
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
#endif
}

// tanh without branches: exp-based form away from zero, odd polynomial near zero (where the
// exp form cancels).  Absolute error stays near 3e-7 (2e-7 from fp32 rounding of the exp form, the rest from the
// approximate ex2 / rcp), so a soft-cap of 30 moves a logit by about 1e-5.
__device__ __forceinline__ float tanh_accurate(float x) {
  const float t = ex2_approx(x * (2.f * kLog2e));
  const float r = rcp_approx(1.f + t);
  const float big = fmaf(-2.f, r, 1.f);
  const float x2 = x * x;
  float poly = fmaf(x2, 62.f / 2835.f, -17.f / 315.f);
  poly = fmaf(x2, poly, 2.f / 15.f);
  poly = fmaf(x2, poly, -1.f / 3.f);
  poly = fmaf(x2 * x, poly, x);
  return (fabsf(x) < 0.3f) ? poly : big;
}

}  // namespace flce
