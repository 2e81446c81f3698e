// Numeric primitives shared by every kernel.  All fp32 arithmetic here is IEEE round-to-nearest:
// the translation units are compiled without fast-math, and divisions use __fdiv_rn explicitly.
#pragma once
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace b200q {

// ---- E4M3 ------------------------------------------------------------------------------------
// Two fp32 -> two E4M3 bytes (lo in bits 0-7), round-to-nearest-even, saturating to +-448, NaN -> 0x7F.
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2_sat(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t f32_to_e4m3_sat(float x) { return f32x2_to_e4m3x2_sat(x, 0.f) & 0xffu; }

// torch's float32 -> float8_e4m3fn cast: RNE, |x| up to 464 rounds to 448, larger magnitudes and
// NaN become the NaN code 0x7F with the sign bit kept.
__device__ __forceinline__ uint32_t f32_to_e4m3_torch(float x) {
  uint32_t c = f32_to_e4m3_sat(x);
  if (fabsf(x) > 464.f) c = 0x7fu | ((__float_as_uint(x) >> 24) & 0x80u);
  return c;
}

// E4M3 byte -> fp32 (exact).  The 7 magnitude bits dropped at bit 20 of an fp32 pattern give
// 2^(E-127)(1+m/8) (or the matching subnormal), which 2^120 rebiases to 2^(E-7); 0x7F/0xFF -> NaN.
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
  uint32_t mag = b & 0x7fu;
  float f = __uint_as_float(mag << 20) * 1.329227995784916e36f;  // 2^120
  if (mag == 0x7fu) f = __uint_as_float(0x7fc00000u);
  return __uint_as_float(__float_as_uint(f) | ((b & 0x80u) << 24));
}

// Two E4M3 bytes -> two fp32 through the hardware conversion (exact).
__device__ __forceinline__ float2 e4m3x2_to_f32x2(uint32_t v) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(v)));
  return __half22float2(*reinterpret_cast<__half2*>(&h2));
}

// ---- E2M1 ------------------------------------------------------------------------------------
// Two fp32 -> one byte of two E2M1 codes (`even` in the low nibble), RNE, saturating to +-6,
// NaN -> +6 (0x7).  The sign bit follows the sign bit of the input, so callers that need
// "negative zero only for inputs below zero" canonicalise the input first.
__device__ __forceinline__ uint32_t f32x2_to_e2m1x2(float even, float odd) {
  return __nv_cvt_float2_to_fp4x2(make_float2(even, odd), __NV_E2M1, cudaRoundNearest);
}

// Eight fp32 (four even/odd pairs) -> four bytes of E2M1 codes, first pair in the low byte.
__device__ __forceinline__ uint32_t f32x8_to_e2m1x8(float2 p0, float2 p1, float2 p2, float2 p3) {
  uint32_t r;
  asm("{\n\t.reg .b8 t0, t1, t2, t3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n\t"
      "mov.b32 %0, {t0, t1, t2, t3};\n\t}"
      : "=r"(r)
      : "f"(p0.x), "f"(p0.y), "f"(p1.x), "f"(p1.y), "f"(p2.x), "f"(p2.y), "f"(p3.x), "f"(p3.y));
  return r;
}

// magnitude of an E2M1 code (bits 0-2): 0,.5,1,1.5,2,3,4,6 ; bit 3 is the sign
__device__ __forceinline__ float e2m1_to_f32(uint32_t code) {
  const uint32_t m = code & 7u;
  // m < 2: m*0.5 ; else (2 + (m&1)) * 2^((m>>1)-2)
  float v = (m < 2u) ? 0.5f * static_cast<float>(m)
                     : __uint_as_float(((126u + (m >> 1)) << 23) | ((m & 1u) << 22));
  return (code & 8u) ? -v : v;
}

// ---- correctly rounded division through a reciprocal ---------------------------------------------
// RN(a/d) given y = RN(1/d).  The first product is within 1.5 ulp of the quotient; one residual
// correction makes it faithful and, by Markstein's theorem (y correctly rounded, quotient
// faithful, residual exact in an FMA), the second correction rounds to RN(a/d).  Callers guarantee
// that d and a/d are in the normal range and nothing overflows (see div_safe).  A zero numerator
// of either sign comes out as +0 ((+0) + (-0) = +0 in the corrections).
__device__ __forceinline__ float div_rn_rcp(float a, float d, float y) {
  float q = a * y;
  float e = fmaf(-q, d, a);
  q = fmaf(e, y, q);
  e = fmaf(-q, d, a);
  return fmaf(e, y, q);
}
// the same for two lanes with packed fp32x2 instructions; nd = -d
__device__ __forceinline__ float2 div2_rn_rcp(float2 a, float2 nd, float2 y) {
  float2 q = __fmul2_rn(a, y);
  float2 e = __ffma2_rn(q, nd, a);
  q = __ffma2_rn(e, y, q);
  e = __ffma2_rn(q, nd, a);
  return __ffma2_rn(e, y, q);
}
// divisor (or numerator bound) inside [2^-40, 2^40]: with both there, quotients stay normal
__device__ __forceinline__ bool div_safe(float v) { return v >= 9.094947017729282e-13f && v <= 1099511627776.f; }

// ---- integer fake quant ------------------------------------------------------------------------
struct IntQ {
  float bound, lo;
};
__host__ __device__ inline IntQ make_intq(int num_bits, int is_unsigned, int narrow) {
  IntQ q;
  q.bound = static_cast<float>((1 << (num_bits - 1 + (is_unsigned ? 1 : 0))) - 1);
  q.lo = -(q.bound + (narrow ? 0.f : 1.f));
  return q;
}
// scale = bound/amax is formed once per amax; amax < 2^-24 maps everything to 0.
__device__ __forceinline__ float intq_apply(float x, float scale, bool live, const IntQ& q) {
  float r = rintf(x * scale);
  r = r > q.bound ? q.bound : r;
  r = r < q.lo ? q.lo : r;
  return live ? __fdiv_rn(r, scale) : 0.f;
}

// The same with the division by `scale` done through its reciprocal once per amax.
struct IntScale {
  float scale, y;
  bool live, fast;
};
__device__ __forceinline__ IntScale make_int_scale(const IntQ& q, float amax) {
  IntScale s;
  s.live = !(amax < 5.9604644775390625e-8f);  // 2^-24
  s.scale = __fdiv_rn(q.bound, amax);
  s.fast = div_safe(s.scale);
  s.y = __frcp_rn(s.scale);
  return s;
}
__device__ __forceinline__ float intq_apply(float x, const IntScale& s, const IntQ& q) {
  float r = rintf(x * s.scale);
  r = r > q.bound ? q.bound : r;
  r = r < q.lo ? q.lo : r;
  // |r| is 0 or an integer in [1, 2^24]: the quotient is normal whenever scale is div_safe
  float o = s.fast ? div_rn_rcp(r, s.scale, s.y) : __fdiv_rn(r, s.scale);
  o = (r == 0.f) ? r : o;  // a zero quotient keeps the sign of the rounded value
  return s.live ? o : 0.f;
}

// NaN-propagating min / max (one instruction each), so that the clamp keeps a NaN input as the
// reference's compare-and-select does
__device__ __forceinline__ float fmin_nan(float a, float b) {
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float fmax_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
// Two elements at once on the fast path (scale div_safe, amax live): packed multiply and packed
// reciprocal-and-correct division.  Same results as intq_apply, element by element.
__device__ __forceinline__ float2 intq_apply2_fast(float2 x, const IntScale& s, const IntQ& q) {
  const float2 t = __fmul2_rn(x, make_float2(s.scale, s.scale));
  float2 r;
  r.x = fmax_nan(fmin_nan(rintf(t.x), q.bound), q.lo);
  r.y = fmax_nan(fmin_nan(rintf(t.y), q.bound), q.lo);
  float2 o = div2_rn_rcp(r, make_float2(-s.scale, -s.scale), make_float2(s.y, s.y));
  // the quotient has the sign of the rounded value (scale > 0); only a zero quotient can have lost it
  o.x = __uint_as_float(__float_as_uint(o.x) | (__float_as_uint(r.x) & 0x80000000u));
  o.y = __uint_as_float(__float_as_uint(o.y) | (__float_as_uint(r.y) & 0x80000000u));
  return o;
}
// N (even) elements in place
template <int N>
__device__ __forceinline__ void intq_apply_n(float* f, const IntScale& s, const IntQ& q) {
  if (s.live && s.fast) {
#pragma unroll
    for (int i = 0; i < N; i += 2) {
      const float2 o = intq_apply2_fast(make_float2(f[i], f[i + 1]), s, q);
      f[i] = o.x;
      f[i + 1] = o.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] = intq_apply(f[i], s, q);
  }
}

}  // namespace b200q
