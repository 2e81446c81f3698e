// Real quantisation to 8-bit storage: FP8 E4M3 and INT8, with one scale per tensor, per channel
// or per contiguous block (all expressed as a [outer, axis, inner] view with scale[axis index]).
// The quotient x/scale is rounded to the tensor's own type T before the final cast, because the
// reference divides in T.
#include "numerics.cuh"

namespace b200q {

template <typename T> __device__ __forceinline__ float round_to_t(float v) {
  return Elem<T>::to_float(Elem<T>::from_float(v));
}

struct ToE4m3 {
  template <typename T> static __device__ __forceinline__ uint32_t cvt(float x, float scale) {
    return f32_to_e4m3_torch(round_to_t<T>(__fdiv_rn(x, scale)));
  }
};
// GEMM operand cast: fp32 scale, the quotient clamped to the E4M3 range before the cast (NaN stays
// NaN).  ROUND: the quotient is rounded to T first, as an eager tensor expression does; without it
// the quotient stays in fp32, as in a fused (compiled) graph.
// The division goes through the reciprocal of the scale (y, formed once per thread) with two
// residual corrections, which returns the correctly rounded quotient wherever scale and numerator
// are in the safe range (`fast`: the scale; checked per element: the numerator); zeros keep their
// sign, everything else takes the IEEE division.  The saturating hardware conversion then does the
// clamp to +-448 and the NaN code in one step.
template <typename T, bool ROUND> __device__ __forceinline__ float operand_quotient(float x, float scale, float y, bool fast) {
  float v = !fast ? __fdiv_rn(x, scale)
                  : (x == 0.f ? x : (div_safe(fabsf(x)) ? div_rn_rcp(x, scale, y) : __fdiv_rn(x, scale)));
  if (ROUND) v = round_to_t<T>(v);
  return v;
}
template <typename T, bool ROUND>
__device__ __forceinline__ uint32_t e4m3_operand(float x, float scale, float y, bool fast) {
  return f32_to_e4m3_sat(operand_quotient<T, ROUND>(x, scale, y, fast));
}
// two elements: packed corrections when both numerators are safe (or zero)
template <typename T, bool ROUND>
__device__ __forceinline__ uint32_t e4m3_operand2(float a, float b, float scale, float y, bool fast) {
  const bool za = a == 0.f, zb = b == 0.f;
  float va, vb;
  if (fast && (za || div_safe(fabsf(a))) && (zb || div_safe(fabsf(b)))) {
    const float2 q = div2_rn_rcp(make_float2(a, b), make_float2(-scale, -scale), make_float2(y, y));
    va = za ? a : q.x;
    vb = zb ? b : q.y;
    if (ROUND) { va = round_to_t<T>(va); vb = round_to_t<T>(vb); }
  } else {
    va = operand_quotient<T, ROUND>(a, scale, y, fast);
    vb = operand_quotient<T, ROUND>(b, scale, y, fast);
  }
  return f32x2_to_e4m3x2_sat(va, vb);
}

template <typename T, bool ROUND>
__global__ void __launch_bounds__(256)
fp8_operand_kernel(const T* __restrict__ x, const float* __restrict__ scale, uint8_t* __restrict__ q, int64_t n) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  const float s = __ldg(scale);
  const float y = __frcp_rn(s);
  const bool fast = div_safe(s);
  const int64_t npack = n / P, stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  const bool vec_out = (reinterpret_cast<uintptr_t>(q) & 7u) == 0;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < npack; i += stride) {
    float f[P];
    E::unpack(ld_stream(xv + i), f);
    uint32_t w[P / 4];
#pragma unroll
    for (int k = 0; k < P / 4; ++k)
      w[k] = e4m3_operand2<T, ROUND>(f[4 * k], f[4 * k + 1], s, y, fast) |
             (e4m3_operand2<T, ROUND>(f[4 * k + 2], f[4 * k + 3], s, y, fast) << 16);
    if (vec_out) {
      if (P == 8) *reinterpret_cast<uint2*>(q + i * P) = make_uint2(w[0], w[P / 4 - 1]);
      else *reinterpret_cast<uint32_t*>(q + i * P) = w[0];
    } else {
#pragma unroll
      for (int k = 0; k < P; ++k) q[i * P + k] = static_cast<uint8_t>(w[k / 4] >> (8 * (k % 4)));
    }
  }
  // ragged tail
  for (int64_t i = npack * P + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    q[i] = static_cast<uint8_t>(e4m3_operand<T, ROUND>(E::to_float(x[i]), s, y, fast));
}
struct ToInt8 {
  template <typename T> static __device__ __forceinline__ uint32_t cvt(float x, float scale) {
    float r = rintf(round_to_t<T>(__fdiv_rn(x, scale)));
    r = fminf(127.f, fmaxf(-128.f, r));
    return static_cast<uint32_t>(static_cast<int>(r)) & 0xffu;
  }
};

template <typename T, typename C>
__global__ void __launch_bounds__(256)
qcast_inner_kernel(const T* __restrict__ x, const T* __restrict__ scales, uint8_t* __restrict__ q,
                   int64_t npack, FastDiv axis, FastDiv inner_packs) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < npack; i += 2 * stride) {
    const int64_t j1 = i + stride;
    const uint4 v0 = ld_stream(xv + i);
    const uint4 v1 = j1 < npack ? ld_stream(xv + j1) : v0;
    uint32_t oq, c0, c1;
    axis.divmod(inner_packs.div(static_cast<uint32_t>(i)), oq, c0);        // npack < 2^31 here
    axis.divmod(inner_packs.div(static_cast<uint32_t>(j1 < npack ? j1 : i)), oq, c1);
    const float s0 = E::to_float(scales[c0]);
    const float s1 = E::to_float(scales[c1]);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int64_t j = u ? j1 : i;
      if (j >= npack) break;
      float f[P];
      E::unpack(u ? v1 : v0, f);
      const float s = u ? s1 : s0;
      uint32_t w[P / 4];
#pragma unroll
      for (int k = 0; k < P / 4; ++k) {
        w[k] = C::template cvt<T>(f[4 * k], s) | (C::template cvt<T>(f[4 * k + 1], s) << 8) |
               (C::template cvt<T>(f[4 * k + 2], s) << 16) | (C::template cvt<T>(f[4 * k + 3], s) << 24);
      }
      if (P == 8) *reinterpret_cast<uint2*>(q + j * P) = make_uint2(w[0], w[P / 4 - 1]);
      else *reinterpret_cast<uint32_t*>(q + j * P) = w[0];
    }
  }
}

template <typename T, typename C>
__global__ void qcast_generic_kernel(const T* __restrict__ x, const T* __restrict__ scales,
                                     uint8_t* __restrict__ q, int64_t n, int64_t axis, int64_t inner) {
  pdl_prologue();
  using E = Elem<T>;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float s = E::to_float(scales[(i / inner) % axis]);
    q[i] = static_cast<uint8_t>(C::template cvt<T>(E::to_float(x[i]), s));
  }
}

template <typename C>
static int launch_qcast(const void* x, const void* scales, uint8_t* q, int64_t outer, int64_t axis,
                        int64_t inner, int dtype, cudaStream_t s) {
  return B200Q_DISPATCH(dtype, [&] {
    constexpr int P = Elem<T>::kPerPack;
    const int64_t n = outer * axis * inner;
    const T* xp = static_cast<const T*>(x);
    const T* sp = static_cast<const T*>(scales);
    // a single scale can be treated as one channel spanning the whole tensor
    int64_t ax = axis, in = inner;
    if (axis == 1) { in = outer * inner; }
    if (in % P == 0 && (reinterpret_cast<uintptr_t>(q) & 7u) == 0 && n / P <= kFastDivLimit) {
      const int64_t npack = n / P;
      int grid = grid_for(npack, 512, 8);
      launch_pdl(qcast_inner_kernel<T, C>, grid, 256, 0, s, xp, sp, q, npack, FastDiv(static_cast<uint32_t>(ax)),
                                                    FastDiv(static_cast<uint32_t>(in / P)));
    } else {
      int grid = grid_for(n, 256, 8);
      launch_pdl(qcast_generic_kernel<T, C>, grid, 256, 0, s, xp, sp, q, n, ax, in);
    }
    return launch_status();
  });
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_fp8_quantize(const void* x, const void* scales, uint8_t* q, int64_t outer,
                                  int64_t axis, int64_t inner, int dtype, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(scales); B200Q_REQUIRE_PTR(q);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x);
  if (outer <= 0 || axis <= 0 || inner <= 0) return B200Q_ERR_SHAPE;
  return launch_qcast<ToE4m3>(x, scales, q, outer, axis, inner, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int b200q_fp8_gemm_operand(const void* x, const float* scale, uint8_t* q, int64_t n, int dtype,
                                      int round_quotient, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(scale); B200Q_REQUIRE_PTR(q);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x);
  if (n <= 0) return B200Q_ERR_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return B200Q_DISPATCH(dtype, [&] {
    const int grid = grid_for(n / Elem<T>::kPerPack + 1, 256, 8);
    const T* xp = static_cast<const T*>(x);
    if (round_quotient) launch_pdl(fp8_operand_kernel<T, true>, grid, 256, 0, s, xp, scale, q, n);
    else launch_pdl(fp8_operand_kernel<T, false>, grid, 256, 0, s, xp, scale, q, n);
    return launch_status();
  });
}

extern "C" int b200q_int8_quantize(const void* x, const void* scales, int8_t* q, int64_t outer,
                                   int64_t axis, int64_t inner, int dtype, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(scales); B200Q_REQUIRE_PTR(q);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x);
  if (outer <= 0 || axis <= 0 || inner <= 0) return B200Q_ERR_SHAPE;
  return launch_qcast<ToInt8>(x, scales, reinterpret_cast<uint8_t*>(q), outer, axis, inner, dtype,
                              static_cast<cudaStream_t>(stream));
}
