// Microscaling (MX) formats: one power-of-two (E8M0) scale per block of 8/16/32 elements.
//   fake quantisation for MXFP8 (E4M3, E5M2), MXFP6 (E3M2, E2M3), MXFP4 (E2M1) and MXINT8, and
//   MXFP4 real quantisation (packed E2M1 + E8M0 scale bytes).
// A block is shared by `lanes` adjacent lanes that reduce its abs-max with shuffles; element
// rounding uses the hardware conversions (round-to-nearest-even, saturating).
#include <cuda_fp6.h>

#include "numerics.cuh"

namespace b200q {

enum MxFormat { MX_E4M3 = 0, MX_E5M2 = 1, MX_INT8 = 2, MX_E2M1 = 6, MX_E3M2 = 7, MX_E2M3 = 8 };

__device__ __forceinline__ float mx_format_max(int fmt) {
  switch (fmt) {
    case MX_E4M3: return 448.f;
    case MX_E5M2: return 57344.f;
    case MX_INT8: return 127.f;
    case MX_E2M1: return 6.f;
    case MX_E3M2: return 28.f;
    default: return 7.5f;  // E2M3
  }
}

// unscale = 2^clamp(ceil(log2(amax / fmt_max)), -127, 127) read from the bits of the quotient
// (the reference's "NV" rule); amax of 0 / inf / NaN leaves the block unscaled.
__device__ __forceinline__ void mx_scale(float amax, int fmt, float& scale, float& unscale) {
  if (amax == 0.f || isinf(amax) || isnan(amax)) { scale = unscale = 1.f; return; }
  const uint32_t u = __float_as_uint(__fdiv_rn(amax, mx_format_max(fmt)));
  const uint32_t ef = (u >> 23) & 0xffu, sf = u & 0x7fffffu;
  const int e = (sf > 0 && ef != 0xfeu && !(ef == 0 && sf <= 0x400000u)) ? static_cast<int>(ef) - 126
                                                                          : static_cast<int>(ef) - 127;
  scale = ldexpf(1.f, -e);
  unscale = ldexpf(1.f, e);
}

// round two non-negative values to the element format and back to fp32
template <int FMT> __device__ __forceinline__ float2 mx_round2(float a, float b) {
  if (FMT == MX_INT8) {
    return make_float2(fminf(127.f, fmaxf(-127.f, rintf(a))), fminf(127.f, fmaxf(-127.f, rintf(b))));
  } else if (FMT == MX_E4M3 || FMT == MX_E5M2) {
    const __nv_fp8_interpretation_t k = FMT == MX_E4M3 ? __NV_E4M3 : __NV_E5M2;
    const __nv_fp8x2_storage_t q = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, k);
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(q, k);
    return __half22float2(*reinterpret_cast<const __half2*>(&h));
  } else if (FMT == MX_E2M1) {
    const __nv_fp4x2_storage_t q = __nv_cvt_float2_to_fp4x2(make_float2(a, b), __NV_E2M1, cudaRoundNearest);
    const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2(q, __NV_E2M1);
    return __half22float2(*reinterpret_cast<const __half2*>(&h));
  } else {
    const __nv_fp6_interpretation_t k = FMT == MX_E3M2 ? __NV_E3M2 : __NV_E2M3;
    const __nv_fp6x2_storage_t q = __nv_cvt_float2_to_fp6x2(make_float2(a, b), k, cudaRoundNearest);
    const __half2_raw h = __nv_cvt_fp6x2_to_halfraw2(q, k);
    return __half22float2(*reinterpret_cast<const __half2*>(&h));
  }
}

template <typename T, int FMT, int PPL>
__global__ void __launch_bounds__(256)
mx_fake_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t nblocks, int lanes) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  const int64_t gthread = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t total = nblocks * lanes;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  uint4* yv = reinterpret_cast<uint4*>(y);
  for (int64_t t = gthread; t < ((total + 31) / 32) * 32; t += nthreads) {
    const bool valid = t < total;
    uint4 v[PPL];
    uint32_t acc = 0;
#pragma unroll
    for (int p = 0; p < PPL; ++p) {
      v[p] = valid ? ld_stream(xv + t * PPL + p) : make_uint4(0, 0, 0, 0);
      acc = E::acc_max(acc, v[p]);
    }
    uint32_t bits = E::acc_to_f32bits(acc);
    for (int o = lanes >> 1; o > 0; o >>= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
    float scale, unscale;
    mx_scale(__uint_as_float(bits), FMT, scale, unscale);
    if (!valid) continue;
#pragma unroll
    for (int p = 0; p < PPL; ++p) {
      float f[P];
      E::unpack(v[p], f);
#pragma unroll
      for (int k = 0; k < P; k += 2) {
        const float2 r = mx_round2<FMT>(fabsf(f[k]) * scale, fabsf(f[k + 1]) * scale);
        f[k] = copysignf(r.x * unscale, f[k]);
        f[k + 1] = copysignf(r.y * unscale, f[k + 1]);
      }
      st_stream(yv + t * PPL + p, E::pack(f));
    }
  }
}

// MXFP4 real quantisation as MXFP4QTensor.quantize does it: scale exponent = ceil(max(log2(amax/6),
// -127)), value = x / 2^e, code = (x > 0 ? 0 : 8) + #{bounds strictly below |value|} (ties go to
// the smaller magnitude), even element in the low nibble; scale byte = e + 127.
template <typename T, int PPL>
__global__ void __launch_bounds__(256)
mxfp4_quantize_kernel(const T* __restrict__ x, int64_t nblocks, int lanes, uint8_t* __restrict__ packed,
                      uint8_t* __restrict__ scales) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  const int64_t gthread = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t total = nblocks * lanes;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  for (int64_t t = gthread; t < ((total + 31) / 32) * 32; t += nthreads) {
    const bool valid = t < total;
    uint4 v[PPL];
    uint32_t acc = 0;
#pragma unroll
    for (int p = 0; p < PPL; ++p) {
      v[p] = valid ? ld_stream(xv + t * PPL + p) : make_uint4(0, 0, 0, 0);
      acc = E::acc_max(acc, v[p]);
    }
    uint32_t bits = E::acc_to_f32bits(acc);
    for (int o = lanes >> 1; o > 0; o >>= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
    const float descale = __fdiv_rn(__uint_as_float(bits), 6.f);
    const float e = ceilf(fmaxf(log2f(descale), -127.f));
    // x / 2^e as x * 2^-e: both are exact scalings by a power of two (2^-e is finite for e >= -127)
    const float mul = exp2f(-e);
    if (!valid) continue;
    if ((t & (lanes - 1)) == 0) scales[t / lanes] = static_cast<uint8_t>(static_cast<int>(e + 127.f));
#pragma unroll
    for (int p = 0; p < PPL; ++p) {
      float f[P];
      E::unpack(v[p], f);
      // magnitudes through the hardware conversion (round to nearest even), then the three ties
      // whose even neighbour is the larger one (0.75, 1.75, 3.5) are moved down: the reference
      // counts the bounds strictly below |q|, which sends every tie toward zero.  The sign bit is
      // set for everything that is not > 0, zero included; NaN encodes as magnitude 0.
      uint32_t out = 0;
#pragma unroll
      for (int k = 0; k < P; k += 2) {
        const float q0 = f[k] * mul, q1 = f[k + 1] * mul;
        const float a0 = fabsf(q0), a1 = fabsf(q1);
        const uint32_t byte = f32x2_to_e2m1x2(a0, a1);
        uint32_t m0 = byte & 7u, m1 = (byte >> 4) & 7u;
        m0 -= static_cast<uint32_t>((a0 == 0.75f) | (a0 == 1.75f) | (a0 == 3.5f));
        m1 -= static_cast<uint32_t>((a1 == 0.75f) | (a1 == 1.75f) | (a1 == 3.5f));
        m0 = (a0 == a0) ? m0 : 0u;
        m1 = (a1 == a1) ? m1 : 0u;
        const uint32_t c0 = m0 | ((q0 > 0.f) ? 0u : 8u), c1 = m1 | ((q1 > 0.f) ? 0u : 8u);
        out |= (c0 | (c1 << 4)) << (4 * k);
      }
      uint8_t* dst = packed + (t * PPL + p) * (P / 2);
      if (P == 8) *reinterpret_cast<uint32_t*>(dst) = out;
      else *reinterpret_cast<uint16_t*>(dst) = static_cast<uint16_t>(out);
    }
  }
}

template <typename T, int FMT>
static int launch_mx_fake(const T* x, T* y, int64_t nblocks, int block, cudaStream_t s) {
  constexpr int P = Elem<T>::kPerPack;
  const int packs = block / P;
  if (block % P || packs <= 0 || (packs & (packs - 1)) || packs > 64) return B200Q_ERR_UNSUPPORTED;
  const int ppl = packs >= 2 ? 2 : 1;
  const int lanes = packs / ppl;
  int grid = grid_for(nblocks * lanes, 256, 8);
  if (ppl == 2) launch_pdl(mx_fake_kernel<T, FMT, 2>, grid, 256, 0, s, x, y, nblocks, lanes);
  else launch_pdl(mx_fake_kernel<T, FMT, 1>, grid, 256, 0, s, x, y, nblocks, lanes);
  return launch_status();
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_mx_fake(const void* x, void* y, int64_t nblocks, int block, int dtype, int elem_format,
                             void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(y);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x); B200Q_REQUIRE_ALIGNED(y);
  if (nblocks <= 0 || block <= 0) return B200Q_ERR_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return B200Q_DISPATCH(dtype, [&]() -> int {
    const T* xp = static_cast<const T*>(x);
    T* yp = static_cast<T*>(y);
    switch (elem_format) {
      case MX_E4M3: return launch_mx_fake<T, MX_E4M3>(xp, yp, nblocks, block, s);
      case MX_E5M2: return launch_mx_fake<T, MX_E5M2>(xp, yp, nblocks, block, s);
      case MX_INT8: return launch_mx_fake<T, MX_INT8>(xp, yp, nblocks, block, s);
      case MX_E2M1: return launch_mx_fake<T, MX_E2M1>(xp, yp, nblocks, block, s);
      case MX_E3M2: return launch_mx_fake<T, MX_E3M2>(xp, yp, nblocks, block, s);
      case MX_E2M3: return launch_mx_fake<T, MX_E2M3>(xp, yp, nblocks, block, s);
      default: return B200Q_ERR_ARG;
    }
  });
}

extern "C" int b200q_mxfp4_quantize(const void* x, int64_t nblocks, int block, int dtype, uint8_t* packed,
                                    uint8_t* scales, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(packed); B200Q_REQUIRE_PTR(scales);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x);
  if ((reinterpret_cast<uintptr_t>(packed) & 3u) != 0) return B200Q_ERR_ALIGN;
  if (nblocks <= 0 || block <= 0) return B200Q_ERR_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return B200Q_DISPATCH(dtype, [&]() -> int {
    constexpr int P = Elem<T>::kPerPack;
    const int packs = block / P;
    if (block % P || packs <= 0 || (packs & (packs - 1)) || packs > 64) return B200Q_ERR_UNSUPPORTED;
    const int ppl = packs >= 2 ? 2 : 1;
    const int lanes = packs / ppl;
    int grid = grid_for(nblocks * lanes, 256, 8);
    const T* xp = static_cast<const T*>(x);
    if (ppl == 2) launch_pdl(mxfp4_quantize_kernel<T, 2>, grid, 256, 0, s, xp, nblocks, lanes, packed, scales);
    else launch_pdl(mxfp4_quantize_kernel<T, 1>, grid, 256, 0, s, xp, nblocks, lanes, packed, scales);
    return launch_status();
  });
}
