// NVFP4 two-level quantisation for block sizes other than 16 (the reference's NVFP4QTensor takes
// any block size; the format's own block is 16 and has the fast kernels).  One thread per block,
// the arithmetic written as the reference's tensor expressions evaluate it:
//   s2 = amax / (6 * 448);  scale = e4m3(block_amax / (6 * s2)) (0 -> 1);  code = e2m1(x / (scale * s2))
#include "numerics.cuh"

namespace b200q {

// the 16-element-unit kernels; pair = two adjacent units share one scale (block 32)
int nvfp4_launch_quantize(const void* x, int64_t nunits, int dtype, const float* global,
                          const uint8_t* scales_in, uint8_t* packed, uint8_t* scales, float* s2_out,
                          int flags, bool pair, cudaStream_t s);
int nvfp4_launch_fake(const void* x, void* y, int64_t nunits, int dtype, const float* amax, bool pair,
                      cudaStream_t s);
int nvfp4_launch_dequantize(const uint8_t* packed, const uint8_t* scales, const float* s2, void* y,
                            int64_t nunits, int dtype, bool pair, cudaStream_t s);

static bool aligned_to(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// kTorchCast: the block-scale cast of torch (NaN code above 464); otherwise saturating (fake quant)
template <bool kTorchCast>
__device__ __forceinline__ uint32_t nv_block_scale_code(float bamax, float s2) {
  float t = __fdiv_rn(bamax, 6.f * s2);
  if (t == 0.f) t = 1.f;
  return kTorchCast ? f32_to_e4m3_torch(t) : f32_to_e4m3_sat(t);
}

// mode 0: quantise (packed, scales);  mode 1: fake quantise into y
template <typename T, int MODE>
__global__ void __launch_bounds__(128)
nvfp4_blocks_kernel(const T* __restrict__ x, int64_t nblocks, int block, const float* __restrict__ global,
                    bool global_is_s2, const uint8_t* __restrict__ scales_in, uint8_t* __restrict__ packed,
                    uint8_t* __restrict__ scales, float* __restrict__ s2_out, T* __restrict__ y) {
  pdl_prologue();
  using E = Elem<T>;
  const float g = __ldg(global);
  const float s2 = global_is_s2 ? g : __fdiv_rn(g, 2688.f);
  if (s2_out && blockIdx.x == 0 && threadIdx.x == 0) *s2_out = s2;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t b = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; b < nblocks; b += stride) {
    const T* xb = x + b * block;
    uint32_t bits = 0;
    for (int i = 0; i < block; ++i) bits = max(bits, __float_as_uint(fabsf(E::to_float(xb[i]))));
    uint32_t code;
    if (scales_in) code = scales_in[b];
    else code = MODE == 0 ? nv_block_scale_code<true>(__uint_as_float(bits), s2)
                          : nv_block_scale_code<false>(__uint_as_float(bits), s2);
    const float d = e4m3_to_f32(code) * s2;
    if (MODE == 0 && scales) scales[b] = static_cast<uint8_t>(code);
    for (int i = 0; i < block; i += 2) {
      // +0: a negative-zero quotient must not set the sign bit (the reference tests v < 0)
      const float e = __fdiv_rn(E::to_float(xb[i]), d) + 0.f;
      const float o = __fdiv_rn(E::to_float(xb[i + 1]), d) + 0.f;
      const uint32_t byte = f32x2_to_e2m1x2(e, o);
      if (MODE == 0) {
        packed[(b * block + i) / 2] = static_cast<uint8_t>(byte);
      } else {
        y[b * block + i] = E::from_float(e2m1_to_f32(byte & 0xfu) * d + 0.f);
        y[b * block + i + 1] = E::from_float(e2m1_to_f32(byte >> 4) * d + 0.f);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
nvfp4_blocks_dequantize_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                               const float* __restrict__ s2p, T* __restrict__ y, int64_t nbytes,
                               int bytes_per_block) {
  pdl_prologue();
  using E = Elem<T>;
  const float s2 = __ldg(s2p);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < nbytes; j += stride) {
    const uint32_t byte = packed[j];
    const float d = e4m3_to_f32(scales[j / bytes_per_block]) * s2;
    y[2 * j] = E::from_float(e2m1_to_f32(byte & 0xfu) * d + 0.f);
    y[2 * j + 1] = E::from_float(e2m1_to_f32(byte >> 4) * d + 0.f);
  }
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_nvfp4_quantize_blocks(const void* x, int64_t nblocks, int block, int dtype,
                                           const float* global, const uint8_t* scales_in, uint8_t* packed,
                                           uint8_t* scales, float* s2_out, int flags, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(global); B200Q_REQUIRE_PTR(packed);
  B200Q_REQUIRE_DTYPE(dtype);
  if (nblocks <= 0 || block <= 0 || (block & 1)) return B200Q_ERR_SHAPE;
  if (flags & ~B200Q_NVFP4_GLOBAL_IS_SCALE2) return B200Q_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (block == 32 && aligned_to(x, 32) && aligned_to(packed, 8))   // block 32 on the fast kernels
    return nvfp4_launch_quantize(x, nblocks * 2, dtype, global, scales_in, packed, scales, s2_out, flags, true, s);
  return B200Q_DISPATCH(dtype, [&] {
    int grid = grid_for(nblocks, 128, 16);
    launch_pdl(nvfp4_blocks_kernel<T, 0>, grid, 128, 0, s, static_cast<const T*>(x), nblocks, block, global,
                                                   (flags & B200Q_NVFP4_GLOBAL_IS_SCALE2) != 0, scales_in, packed,
                                                   scales, s2_out, nullptr);
    return launch_status();
  });
}

extern "C" int b200q_nvfp4_fake_blocks(const void* x, void* y, int64_t nblocks, int block, int dtype,
                                       const float* amax, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(y); B200Q_REQUIRE_PTR(amax);
  B200Q_REQUIRE_DTYPE(dtype);
  if (nblocks <= 0 || block <= 0 || (block & 1)) return B200Q_ERR_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (block == 32 && aligned_to(x, 32) && aligned_to(y, 32))
    return nvfp4_launch_fake(x, y, nblocks * 2, dtype, amax, true, s);
  return B200Q_DISPATCH(dtype, [&] {
    int grid = grid_for(nblocks, 128, 16);
    launch_pdl(nvfp4_blocks_kernel<T, 1>, grid, 128, 0, s, static_cast<const T*>(x), nblocks, block, amax, false, nullptr,
                                                   nullptr, nullptr, nullptr, static_cast<T*>(y));
    return launch_status();
  });
}

extern "C" int b200q_nvfp4_dequantize_blocks(const uint8_t* packed, const uint8_t* scales, const float* s2,
                                             void* y, int64_t nblocks, int block, int dtype, void* stream) {
  B200Q_REQUIRE_PTR(packed); B200Q_REQUIRE_PTR(scales); B200Q_REQUIRE_PTR(s2); B200Q_REQUIRE_PTR(y);
  B200Q_REQUIRE_DTYPE(dtype);
  if (nblocks <= 0 || block <= 0 || (block & 1)) return B200Q_ERR_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (block == 32 && aligned_to(y, 32) && aligned_to(packed, 8))
    return nvfp4_launch_dequantize(packed, scales, s2, y, nblocks * 2, dtype, true, s);
  return B200Q_DISPATCH(dtype, [&] {
    const int64_t nbytes = nblocks * (block / 2);
    int grid = grid_for(nbytes, 256, 8);
    launch_pdl(nvfp4_blocks_dequantize_kernel<T>, grid, 256, 0, s, packed, scales, s2, static_cast<T*>(y), nbytes, block / 2);
    return launch_status();
  });
}
