// Scalar device helpers shared by every kernel: storage conversion, the fused nonlinearities
// and the TF32 split.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>
#include "problem.h"

namespace gb {

// One element through the read-only path.  The fp16 overload of __ldg in cuda_fp16.hpp is a
// non-volatile asm statement, which the compiler may hoist above the bounds test that guards it
// (it did: a predicated loop over rows read past the end of a matrix); a volatile one stays put.
__device__ __forceinline__ float ldg1(const float* p) { return __ldg(p); }
__device__ __forceinline__ __half ldg1(const __half* p) {
  unsigned short v;
  asm volatile("ld.global.nc.b16 %0, [%1];" : "=h"(v) : "l"(p));
  return __ushort_as_half(v);
}

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
template <typename T>
__device__ __forceinline__ T from_f(float x);
template <>
__device__ __forceinline__ float from_f<float>(float x) { return x; }
template <>
__device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

// tanh for fp32 results in a handful of instructions (libm's tanhf is about sixty and was half of
// a 128 x 128 epilogue).  |x| < 0.25: odd polynomial, relative error below 4e-7; otherwise
// (1 - e) / (1 + e) with e = exp(-2|x|) from the hardware exponential: the relative error of
// 1 - e stays below 8e-7 because e <= 0.61 there.  Results are within a few ulp of the
// correctly rounded value -- the same class as the rational approximation Eigen's fp32 tanh uses.
__device__ __forceinline__ float tanh_f32(float x) {
  const float ax = fabsf(x);
  const float x2 = x * x;
  const float poly = x * (1.f + x2 * (-0.33333334f + x2 * (0.13333334f + x2 * -0.053968254f)));
  const float e = __expf(-2.f * ax);
  const float big = copysignf(__fdividef(1.f - e, 1.f + e), x);
  return ax < 0.25f ? poly : big;
}

// Forward nonlinearities, following ginn/nonlin.h:93-95 (tanh), :116-118 (relu), :136-145 (sigmoid;
// fp32 uses 0.5*tanh(0.5x)+0.5, Half the sign-split exponential form).  T is the storage type.
template <typename T>
__device__ __forceinline__ float act_forward(int act, float x) {
  switch (act) {
    case ACT_TANH: return sizeof(T) == 4 ? tanh_f32(x) : tanhf(x);
    case ACT_RELU: return fmaxf(x, 0.f);
    case ACT_SIGMOID:
      if (sizeof(T) == 2) {
        if (x > 0.f) return 1.f / (1.f + expf(-x));
        const float e = expf(x);
        return e / (1.f + e);
      }
      return 0.5f * tanh_f32(0.5f * x) + 0.5f;
    default: return x;
  }
}
// Derivative times upstream gradient, expressed through the output y
// (ginn/nonlin.h:96-106, :119-126, :146-152).
template <typename T>
__device__ __forceinline__ float act_backward(int act, float y, float dy) {
  switch (act) {
    case ACT_TANH: return sizeof(T) == 2 ? dy - y * y * dy : (1.f - y * y) * dy;
    case ACT_RELU: return y > 0.f ? dy : 0.f;
    case ACT_SIGMOID: return y * (1.f - y) * dy;
    default: return dy;
  }
}

// Forward nonlinearity for fp16 outputs: hardware approximations (relative error about 2^-11,
// below the rounding of the fp16 result) keep the epilogue a few instructions per element.
__device__ __forceinline__ float act_forward_half(int act, float x) {
  if (act == ACT_TANH) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
  }
  if (act == ACT_SIGMOID) {
    const float e = __expf(-fabsf(x));
    const float r = __fdividef(1.f, 1.f + e);
    return x > 0.f ? r : e * r;
  }
  if (act == ACT_RELU) return fmaxf(x, 0.f);
  return x;
}

// hi = x rounded to TF32 (nearest, ties away from zero, what cvt.rna.tf32 gives); lo = x - hi
// (exact in fp32; the tensor core keeps the top 11 significant bits of it).  The rounding is
// done on the bit pattern with two integer instructions (add half an ulp of the 10-bit mantissa
// to the magnitude, clear the 13 low bits) because the conversion instruction issues at a
// sixteenth of the integer rate and would bound the split.  A carry out of the mantissa bumps
// the exponent, as rounding should.  Values that are not finite, or so large that rounding
// would reach inf (|x| >= 0x7f7ff000 as a bit pattern), go to the hi plane unchanged and leave
// the lo plane zero: the integer add would wrap an all-ones NaN to zero, and inf - inf would
// poison the lo plane.  One comparison covers all of it (NaN compares false).
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
  const float r = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
  const bool ok = fabsf(x) < __uint_as_float(0x7f7ff000u);
  hi = ok ? r : x;
  lo = ok ? x - r : 0.f;
}

// The guard hoisted out of the per-value work: `guard_ok(m)` for m = the largest magnitude of a
// group of values (see absmax4) says whether all of them may take split_fast, which is
// split_tf32 without its compare and selects.  The max instruction drops NaNs, so a NaN among
// finite values takes the fast route: there it lands in the lo plane at the latest (NaN - r) and
// still poisons every result it should; a group of NaNs only fails the test and is guarded.
// Callers test once per thread and k-block and keep two straight-line copies of their loop, so
// that the loads of all pieces stay ahead of the arithmetic (a test per 16-byte piece put a
// branch between the pieces and was slower than the per-value guard).
__device__ __forceinline__ float absmax4(const float4& x) {
  return fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));
}
__device__ __forceinline__ bool guard_ok(float m) { return m < __uint_as_float(0x7f7ff000u); }
template <bool GUARDED>
__device__ __forceinline__ void split4(const float4& x, float4& hi, float4& lo) {
  if (GUARDED) {
    split_tf32(x.x, hi.x, lo.x);
    split_tf32(x.y, hi.y, lo.y);
    split_tf32(x.z, hi.z, lo.z);
    split_tf32(x.w, hi.w, lo.w);
  } else {
    hi.x = __uint_as_float((__float_as_uint(x.x) + 0x1000u) & 0xffffe000u);
    hi.y = __uint_as_float((__float_as_uint(x.y) + 0x1000u) & 0xffffe000u);
    hi.z = __uint_as_float((__float_as_uint(x.z) + 0x1000u) & 0xffffe000u);
    hi.w = __uint_as_float((__float_as_uint(x.w) + 0x1000u) & 0xffffe000u);
    lo.x = x.x - hi.x;
    lo.y = x.y - hi.y;
    lo.z = x.z - hi.z;
    lo.w = x.w - hi.w;
  }
}

}  // namespace gb
