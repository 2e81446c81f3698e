// INT4 (AWQ) block quantisation: per-block scale 7/amax, values packed two per byte with the first
// element in the high nibble.  The arithmetic runs in the tensor's own type T as the reference
// kernel does (multiply, clamp and the +8 offset are each rounded to T; then roundf, half away
// from zero), so results depend on T and are reproduced step by step here.
#include "numerics.cuh"

namespace b200q {

template <typename T> __device__ __forceinline__ float round_to(float v) {
  return Elem<T>::to_float(Elem<T>::from_float(v));
}

// 7/amax as the reference's Python evaluates it: reciprocal in T, then times 7 in T.
template <typename T> __device__ __forceinline__ float int4_scale_from_amax(float amax) {
  return round_to<T>(round_to<T>(__fdiv_rn(1.f, amax)) * 7.f);
}

template <typename T> __device__ __forceinline__ uint32_t int4_code(float x, float scale) {
  float y = round_to<T>(x * scale);
  y = fmaxf(-8.f, fminf(7.f, y));
  const float z = round_to<T>(y + 8.f);
  return static_cast<uint32_t>(static_cast<int>(roundf(z))) & 0xfu;
}

// nibbles of one pack (P elements) -> P/2 bytes in the low bits of the result
template <typename T> __device__ __forceinline__ uint32_t int4_pack(const uint4& v, float scale) {
  constexpr int P = Elem<T>::kPerPack;
  float f[P];
  Elem<T>::unpack(v, f);
  uint32_t out = 0;
#pragma unroll
  for (int j = 0; j < P / 2; ++j)
    out |= ((int4_code<T>(f[2 * j], scale) << 4) | int4_code<T>(f[2 * j + 1], scale)) << (8 * j);
  return out;
}
// bf16: the multiply, clamp and +8 are the packed bf16 instructions themselves (each rounds to
// bf16 exactly as the step-by-step form does).  z is in [0, 15], so roundf(z) = floor(z + 0.5): after
// z + 0.5 (exact in fp32) a round-toward-zero add of 2^23 leaves that integer n in the low bits of
// the pattern K + n, K = bits(2^23).  The eight nibbles are merged by multiply-adds on the patterns,
// sum (K + n_k) 16^e_k, with K * sum 16^e_k taken off the start value (all modulo 2^32).
template <> __device__ __forceinline__ uint32_t int4_pack<__nv_bfloat16>(const uint4& v, float scale) {
  const __nv_bfloat162 s2 = __float2bfloat162_rn(scale);
  const __nv_bfloat162 hi7 = __float2bfloat162_rn(7.f), lo8 = __float2bfloat162_rn(-8.f),
                       off8 = __float2bfloat162_rn(8.f);
  const float2 half2f = make_float2(0.5f, 0.5f), big2 = make_float2(8388608.f, 8388608.f);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t out = 0u - 0x4b000000u * 0x11111111u;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 y = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]), s2);
    y = __hmax2(lo8, __hmin2(hi7, y));
    const __nv_bfloat162 z = __hadd2(y, off8);
    const uint32_t zw = *reinterpret_cast<const uint32_t*>(&z);
    const float2 z2 = make_float2(__uint_as_float(zw << 16), __uint_as_float(zw & 0xffff0000u));
    const float2 u = __fadd2_rz(__fadd2_rn(z2, half2f), big2);
    out += __float_as_uint(u.x) * (16u << (8 * j));   // first element of the pair: high nibble
    out += __float_as_uint(u.y) * (1u << (8 * j));
  }
  return out;
}

template <typename T> __device__ __forceinline__ void store_codes(uint8_t* dst, uint32_t codes);
template <> __device__ __forceinline__ void store_codes<float>(uint8_t* dst, uint32_t c) {
  *reinterpret_cast<uint16_t*>(dst) = static_cast<uint16_t>(c);
}
template <> __device__ __forceinline__ void store_codes<__half>(uint8_t* dst, uint32_t c) {
  *reinterpret_cast<uint32_t*>(dst) = c;
}
template <> __device__ __forceinline__ void store_codes<__nv_bfloat16>(uint8_t* dst, uint32_t c) {
  *reinterpret_cast<uint32_t*>(dst) = c;
}

// `lanes` adjacent lanes (power of two <= 32) share a block, PPL consecutive packs per lane
// (measured faster here than interleaving the lanes' packs).
template <typename T, int PPL>
__global__ void __launch_bounds__(256)
int4_quantize_kernel(const T* __restrict__ x, int64_t nblocks, int lanes,
                     const T* __restrict__ scales_in, T* __restrict__ scales_out,
                     uint8_t* __restrict__ packed) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  const int64_t gthread = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t total = nblocks * lanes;
  const int lane_shift = __ffs(lanes) - 1;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  for (int64_t t = gthread; t < ((total + 31) / 32) * 32; t += nthreads) {
    const bool valid = t < total;
    uint4 v[PPL];
    uint32_t acc = 0;
#pragma unroll
    const int64_t b = t >> lane_shift;   // lanes is a power of two
#pragma unroll
    for (int p = 0; p < PPL; ++p) v[p] = valid ? ld_stream(xv + t * PPL + p) : make_uint4(0, 0, 0, 0);
    float scale;
    if (scales_in) {
      scale = valid ? E::to_float(scales_in[b]) : 0.f;
    } else {
#pragma unroll
      for (int p = 0; p < PPL; ++p) acc = E::acc_max(acc, v[p]);
      uint32_t bits = E::acc_to_f32bits(acc);
      for (int o = lanes >> 1; o > 0; o >>= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
      scale = int4_scale_from_amax<T>(__uint_as_float(bits));
    }
    if (valid) {
      if (scales_out && (t & (lanes - 1)) == 0) scales_out[b] = E::from_float(scale);
#pragma unroll
      for (int p = 0; p < PPL; ++p)
        store_codes<T>(packed + (t * PPL + p) * (P / 2), int4_pack<T>(v[p], scale));
    }
  }
}

template <typename T>
__global__ void int4_quantize_generic_kernel(const T* __restrict__ x, int64_t nblocks, int block,
                                             const T* __restrict__ scales_in,
                                             T* __restrict__ scales_out, uint8_t* __restrict__ packed) {
  pdl_prologue();
  using E = Elem<T>;
  for (int64_t b = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; b < nblocks;
       b += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float scale;
    if (scales_in) {
      scale = E::to_float(scales_in[b]);
    } else {
      uint32_t bits = 0;
      for (int i = 0; i < block; ++i)
        bits = max(bits, __float_as_uint(fabsf(E::to_float(x[b * block + i]))));
      scale = int4_scale_from_amax<T>(__uint_as_float(bits));
    }
    if (scales_out) scales_out[b] = E::from_float(scale);
    for (int j = 0; j < block / 2; ++j) {
      const uint32_t hi = int4_code<T>(E::to_float(x[b * block + 2 * j]), scale);
      const uint32_t lo = int4_code<T>(E::to_float(x[b * block + 2 * j + 1]), scale);
      packed[(b * block) / 2 + j] = static_cast<uint8_t>((hi << 4) | lo);
    }
  }
}

// one thread: 8 packed bytes -> 16 values
template <typename T>
__global__ void __launch_bounds__(256)
int4_dequantize_kernel(const uint8_t* __restrict__ packed, const T* __restrict__ scales,
                       T* __restrict__ y, int64_t nbytes, int bytes_per_block) {
  pdl_prologue();
  using E = Elem<T>;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < nbytes; j += stride) {
    const uint32_t byte = packed[j];
    const float scale = E::to_float(scales[j / bytes_per_block]);
    const float hi = static_cast<float>(static_cast<int>(byte >> 4) - 8);
    const float lo = static_cast<float>(static_cast<int>(byte & 0xfu) - 8);
    y[2 * j] = E::from_float(__fdiv_rn(hi, scale));
    y[2 * j + 1] = E::from_float(__fdiv_rn(lo, scale));
  }
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_int4_quantize(const void* x, int64_t nblocks, int block, int dtype,
                                   const void* scales_in, void* scales_out, uint8_t* packed,
                                   void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(packed);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x);
  if ((reinterpret_cast<uintptr_t>(packed) & 3u) != 0) return B200Q_ERR_ALIGN;
  if (nblocks <= 0 || block <= 0 || (block & 1)) return B200Q_ERR_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return B200Q_DISPATCH(dtype, [&] {
    constexpr int P = Elem<T>::kPerPack;
    const T* xp = static_cast<const T*>(x);
    const T* sin = static_cast<const T*>(scales_in);
    T* sout = static_cast<T*>(scales_out);
    const int packs = block / P;
    const bool pow2 = block % P == 0 && packs > 0 && (packs & (packs - 1)) == 0;
    if (pow2 && packs <= 64) {
      // two packs per lane (four measured slower)
      const int ppl = packs >= 2 ? 2 : 1;
      const int lanes = packs / ppl;
      int grid = grid_for(nblocks * lanes, 256, 8);
      if (ppl == 2) launch_pdl(int4_quantize_kernel<T, 2>, grid, 256, 0, s, xp, nblocks, lanes, sin, sout, packed);
      else launch_pdl(int4_quantize_kernel<T, 1>, grid, 256, 0, s, xp, nblocks, lanes, sin, sout, packed);
    } else {
      int grid = grid_for(nblocks, 128, 16);
      launch_pdl(int4_quantize_generic_kernel<T>, grid, 128, 0, s, xp, nblocks, block, sin, sout, packed);
    }
    return launch_status();
  });
}

extern "C" int b200q_int4_dequantize(const uint8_t* packed, const void* scales, void* y, int64_t nblocks,
                                     int block, int dtype, void* stream) {
  B200Q_REQUIRE_PTR(packed); B200Q_REQUIRE_PTR(scales); B200Q_REQUIRE_PTR(y);
  B200Q_REQUIRE_DTYPE(dtype);
  if (nblocks <= 0 || block <= 0 || (block & 1)) return B200Q_ERR_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return B200Q_DISPATCH(dtype, [&] {
    const int64_t nbytes = nblocks * (block / 2);
    int grid = grid_for(nbytes, 256, 8);
    launch_pdl(int4_dequantize_kernel<T>, grid, 256, 0, s, packed, static_cast<const T*>(scales),
                                                   static_cast<T*>(y), nbytes, block / 2);
    return launch_status();
  });
}
