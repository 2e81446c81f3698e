// NVFP4: two-level scaling (fp32 per-tensor scale, E4M3 scale per 16 elements) and E2M1 values
// packed two per byte.  Real quantisation (codes + scales), dequantisation, fake quantisation,
// and grouped launches that cover a whole list of weight tensors with one grid.
//
// One thread owns one 16-element block: the block arrives with 256-bit loads (one for half/bf16,
// two for fp32), the block abs-max never leaves registers, and the eight packed bytes leave as
// one 8-byte store, so a warp reads 1 KB and writes 256 B + 32 B, all contiguous.
#include "numerics.cuh"

namespace b200q {

#ifndef B200Q_NV_THREADS
#define B200Q_NV_THREADS 256
#endif
#ifndef B200Q_NV_UNROLL
#define B200Q_NV_UNROLL 2
#endif
#ifndef B200Q_NV_CTAS
#define B200Q_NV_CTAS 8
#endif
constexpr int kNvCtasPerSm = B200Q_NV_CTAS;
constexpr int kNvThreads = B200Q_NV_THREADS;
constexpr int kNvUnroll = B200Q_NV_UNROLL;                // blocks in flight per thread
constexpr int kNvTileBlocks = kNvThreads * kNvUnroll;     // 16-element blocks per CTA tile
constexpr int kNvTileElems = kNvTileBlocks * 16;

struct u32x8 { uint32_t w[8]; };

__device__ __forceinline__ u32x8 ld256_stream(const void* p) {
  u32x8 v;
  asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]),
                 "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7])
               : "l"(p));
  return v;
}
// same, asking L2 to keep the line: the quantise pass reads the tensor again right after
__device__ __forceinline__ u32x8 ld256_keep(const void* p) {
  u32x8 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::evict_last.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]),
                 "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7])
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st256_stream(void* p, const u32x8& v) {
  asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.w[0]),
               "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]), "r"(v.w[4]), "r"(v.w[5]), "r"(v.w[6]),
               "r"(v.w[7])
               : "memory");
}

// Raw storage of one 16-element block and its decoding.
template <typename T> struct Block16;
template <> struct Block16<float> {
  u32x8 a, b;
  __device__ __forceinline__ void load(const float* p) { a = ld256_stream(p); b = ld256_stream(p + 8); }
  __device__ __forceinline__ void load_keep(const float* p) { a = ld256_keep(p); b = ld256_keep(p + 8); }
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < 8; ++i) a.w[i] = b.w[i] = 0;
  }
  __device__ __forceinline__ uint32_t amax_f32bits() const {
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = max(m, max(a.w[i] & 0x7fffffffu, b.w[i] & 0x7fffffffu));
    return m;
  }
  __device__ __forceinline__ void decode(float* f) const {
#pragma unroll
    for (int i = 0; i < 8; ++i) { f[i] = __uint_as_float(a.w[i]); f[8 + i] = __uint_as_float(b.w[i]); }
  }
};
template <> struct Block16<__nv_bfloat16> {
  u32x8 a;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { a = ld256_stream(p); }
  __device__ __forceinline__ void load_keep(const __nv_bfloat16* p) { a = ld256_keep(p); }
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < 8; ++i) a.w[i] = 0;
  }
  __device__ __forceinline__ uint32_t amax_f32bits() const {
#ifdef B200Q_NV_HMAX
    // |x| max as packed bf16 arithmetic (NaN-propagating), tree of 7 ops
    __nv_bfloat162 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&a.w[i]));
#pragma unroll
    for (int s = 4; s > 0; s >>= 1)
#pragma unroll
      for (int i = 0; i < s; ++i) v[i] = __hmax2_nan(v[i], v[i + s]);
    const uint32_t m = *reinterpret_cast<uint32_t*>(&v[0]);
#else
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = __vmaxu2(m, a.w[i] & 0x7fff7fffu);
#endif
    return max(m & 0xffffu, m >> 16) << 16;
  }
  __device__ __forceinline__ void decode(float* f) const {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      f[2 * i] = __uint_as_float(a.w[i] << 16);
      f[2 * i + 1] = __uint_as_float(a.w[i] & 0xffff0000u);
    }
  }
};
template <> struct Block16<__half> {
  u32x8 a;
  __device__ __forceinline__ void load(const __half* p) { a = ld256_stream(p); }
  __device__ __forceinline__ void load_keep(const __half* p) { a = ld256_keep(p); }
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < 8; ++i) a.w[i] = 0;
  }
  __device__ __forceinline__ uint32_t amax_f32bits() const {
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = __vmaxu2(m, a.w[i] & 0x7fff7fffu);
    uint16_t h = static_cast<uint16_t>(max(m & 0xffffu, m >> 16));
    return __float_as_uint(__half2float(__ushort_as_half(h)));
  }
  __device__ __forceinline__ void decode(float* f) const {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float2 t = __half22float2(*reinterpret_cast<const __half2*>(&a.w[i]));
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
  }
};

// ---- per-block arithmetic ----------------------------------------------------------------------
// Correctly rounded a/d for two lanes at once, given y = RN(1/d) and nd = -d.  The first product
// is within 1.5 ulp of the quotient; one residual correction makes it faithful and, by Markstein's
// theorem (y correctly rounded, quotient faithful, residual exact in an FMA), the second correction
// rounds to RN(a/d).  Callers guarantee d, a/d in the normal range with no overflow.  A zero
// numerator of either sign comes out as +0 ((+0) + (-0) = +0 in the corrections).
__device__ __forceinline__ float2 div2_rn(float2 a, float2 nd, float2 y) {
  float2 q = __fmul2_rn(a, y);
  float2 e = __ffma2_rn(q, nd, a);
  q = __ffma2_rn(e, y, q);
  e = __ffma2_rn(q, nd, a);
  return __ffma2_rn(e, y, q);
}
__device__ __forceinline__ float div1_rn(float a, float d, float y) {
  float q = a * y;
  float e = fmaf(-q, d, a);
  q = fmaf(e, y, q);
  e = fmaf(-q, d, a);
  return fmaf(e, y, q);
}

constexpr float kTwoP60 = 1152921504606846976.f;        // 2^60
constexpr float kTwoM60 = 8.673617379884035e-19f;       // 2^-60

// Per-tensor constants of the two-level scaling.
struct Nvfp4Tensor {
  float s2;    // weights_scaling_factor_2
  float c;     // 6 * s2
  float rc;    // RN(1/c) when c is in the safe range
  bool c_ok;
  __device__ __forceinline__ explicit Nvfp4Tensor(float s2_) : s2(s2_) {
    c = 6.f * s2;
    c_ok = c >= kTwoM60 && c <= kTwoP60;
    rc = __frcp_rn(c);
  }
};

// block scale code from the block abs-max: t = bamax/c (IEEE quotient), 0 -> 1, cast to E4M3
template <bool kTorchCast>
__device__ __forceinline__ uint32_t nvfp4_scale_code(float bamax, const Nvfp4Tensor& tn) {
  float t;
  if (tn.c_ok && (bamax == 0.f || (bamax >= kTwoM60 && bamax <= kTwoP60)))
    t = div1_rn(bamax, tn.c, tn.rc);
  else
    t = __fdiv_rn(bamax, tn.c);
  if (t == 0.f) t = 1.f;
  return kTorchCast ? f32_to_e4m3_torch(t) : f32_to_e4m3_sat(t);
}

// 16 values -> 8 bytes of E2M1 codes under divisor d = float(block scale) * s2.
// Fast path (16-bit inputs, divisor and block abs-max in a safe range — every ordinary block):
// quotients through div2_rn with one reciprocal per block.  Otherwise the IEEE division per
// element, with +0 added so that a negative-zero quotient does not set the sign bit.
template <bool kAllowFast>
__device__ __forceinline__ uint2 nvfp4_encode16(const float* f, float d, float bamax) {
  uint32_t w[2];
  if (kAllowFast && d >= kTwoM60 && d <= 65536.f && bamax <= kTwoP60) {
    const float r = __frcp_rn(d);
    const float2 y = make_float2(r, r), nd = make_float2(-d, -d);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float2 q[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        q[j] = div2_rn(make_float2(f[8 * h + 2 * j], f[8 * h + 2 * j + 1]), nd, y);
      w[h] = f32x8_to_e2m1x8(q[0], q[1], q[2], q[3]);
    }
  } else {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t acc = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float e = __fdiv_rn(f[8 * h + 2 * j], d) + 0.f;
        const float o = __fdiv_rn(f[8 * h + 2 * j + 1], d) + 0.f;
        acc |= f32x2_to_e2m1x2(e, o) << (8 * j);
      }
      w[h] = acc;
    }
  }
  return make_uint2(w[0], w[1]);
}

// 8 bytes of codes -> 16 values times d.  The hardware conversion gives -0 for the negative-zero
// code; the fused multiply-add with +0 turns the product into +0 as the reference's table has it.
__device__ __forceinline__ void nvfp4_decode16(uint2 codes, float d, float* f) {
  const uint32_t w[2] = {codes.x, codes.y};
  const float2 dd = make_float2(d, d), zz = make_float2(0.f, 0.f);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half2_raw hr = __nv_cvt_fp4x2_to_halfraw2(
          static_cast<__nv_fp4x2_storage_t>((w[h] >> (8 * j)) & 0xffu), __NV_E2M1);
      const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&hr));
      const float2 r = __ffma2_rn(v, dd, zz);
      f[8 * h + 2 * j] = r.x;
      f[8 * h + 2 * j + 1] = r.y;
    }
  }
}

template <typename T>
__device__ __forceinline__ void store16(T* y, const float* f);
template <> __device__ __forceinline__ void store16<float>(float* y, const float* f) {
  u32x8 a, b;
#pragma unroll
  for (int i = 0; i < 8; ++i) { a.w[i] = __float_as_uint(f[i]); b.w[i] = __float_as_uint(f[8 + i]); }
  st256_stream(y, a); st256_stream(y + 8, b);
}
template <> __device__ __forceinline__ void store16<__nv_bfloat16>(__nv_bfloat16* y, const float* f) {
  u32x8 a;
#pragma unroll
  for (int i = 0; i < 8; ++i) a.w[i] = Elem<__nv_bfloat16>::pack2(f[2 * i], f[2 * i + 1]);
  st256_stream(y, a);
}
template <> __device__ __forceinline__ void store16<__half>(__half* y, const float* f) {
  u32x8 a;
#pragma unroll
  for (int i = 0; i < 8; ++i) a.w[i] = Elem<__half>::pack2(f[2 * i], f[2 * i + 1]);
  st256_stream(y, a);
}

// Quantise one loaded block and store codes + scale.
// `pair`: scale blocks of 32 elements = two adjacent 16-element units held by adjacent lanes, which
// share one abs-max and one scale (unit count even, so both lanes of a pair are always active).
template <typename T>
__device__ __forceinline__ void nvfp4_quant_block(const Block16<T>& blk, int64_t b, const Nvfp4Tensor& tn,
                                                  const uint8_t* __restrict__ scales_in,
                                                  uint8_t* __restrict__ packed,
                                                  uint8_t* __restrict__ scales, bool pair = false,
                                                  bool sat_scales = false) {
  uint32_t abits = blk.amax_f32bits();
  if (pair) abits = max(abits, __shfl_xor_sync(__activemask(), abits, 1));
  const float bamax = __uint_as_float(abits);
  const int64_t sb = pair ? (b >> 1) : b;
  uint32_t code;
  if (scales_in) code = scales_in[sb];
  else code = sat_scales ? nvfp4_scale_code<false>(bamax, tn) : nvfp4_scale_code<true>(bamax, tn);
  const float d = e4m3_to_f32(code) * tn.s2;
  float f[16];
  blk.decode(f);
  st_stream(packed + 8 * b, nvfp4_encode16<sizeof(T) == 2>(f, d, bamax));
  if (scales && !(pair && (b & 1))) scales[sb] = static_cast<uint8_t>(code);
}

// ---- single-tensor kernels ---------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kNvThreads)
nvfp4_quantize_kernel(const T* __restrict__ x, int64_t nblocks, const float* __restrict__ global,
                      bool global_is_s2, const uint8_t* __restrict__ scales_in,
                      uint8_t* __restrict__ packed, uint8_t* __restrict__ scales,
                      float* __restrict__ s2_out, bool pair, bool sat_scales) {
  pdl_prologue();
  const float g = __ldg(global);
  const Nvfp4Tensor tn(global_is_s2 ? g : __fdiv_rn(g, 2688.f));
  if (s2_out && blockIdx.x == 0 && threadIdx.x == 0) *s2_out = tn.s2;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t b0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; b0 < nblocks;
       b0 += kNvUnroll * stride) {
    Block16<T> blk[kNvUnroll];
#pragma unroll
    for (int u = 0; u < kNvUnroll; ++u) {
      const int64_t b = b0 + u * stride;
      if (b < nblocks) blk[u].load(x + 16 * b);
    }
#pragma unroll
    for (int u = 0; u < kNvUnroll; ++u) {
      const int64_t b = b0 + u * stride;
      if (b < nblocks) nvfp4_quant_block<T>(blk[u], b, tn, scales_in, packed, scales, pair, sat_scales);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kNvThreads)
nvfp4_fake_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t nblocks,
                  const float* __restrict__ amax, bool pair) {
  pdl_prologue();
  const Nvfp4Tensor tn(__fdiv_rn(__ldg(amax), 2688.f));
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t b0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; b0 < nblocks;
       b0 += kNvUnroll * stride) {
    Block16<T> blk[kNvUnroll];
#pragma unroll
    for (int u = 0; u < kNvUnroll; ++u) {
      const int64_t b = b0 + u * stride;
      if (b < nblocks) blk[u].load(x + 16 * b);
    }
#pragma unroll
    for (int u = 0; u < kNvUnroll; ++u) {
      const int64_t b = b0 + u * stride;
      if (b < nblocks) {
        uint32_t abits = blk[u].amax_f32bits();
        if (pair) abits = max(abits, __shfl_xor_sync(__activemask(), abits, 1));
        const float bamax = __uint_as_float(abits);
        const uint32_t code = nvfp4_scale_code<false>(bamax, tn);
        const float d = e4m3_to_f32(code) * tn.s2;
        float f[16];
        blk[u].decode(f);
        const uint2 q = nvfp4_encode16<sizeof(T) == 2>(f, d, bamax);
        nvfp4_decode16(q, d, f);
        store16<T>(y + 16 * b, f);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kNvThreads)
nvfp4_dequantize_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                        const float* __restrict__ s2p, T* __restrict__ y, int64_t nblocks, bool pair) {
  pdl_prologue();
  const float s2 = __ldg(s2p);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t b = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; b < nblocks; b += stride) {
    const uint2 q = *reinterpret_cast<const uint2*>(packed + 8 * b);
    const float d = e4m3_to_f32(scales[pair ? (b >> 1) : b]) * s2;
    float f[16];
    nvfp4_decode16(q, d, f);
    store16<T>(y + 16 * b, f);
  }
}

// ---- grouped kernels -----------------------------------------------------------------------------
// Tiles of kNvTileBlocks blocks are numbered across all tensors; a CTA takes a contiguous run of
// tiles so that it crosses few tensor boundaries (one amax atomic per tensor it touches).
__device__ __forceinline__ int find_tensor(const b200q_nvfp4_desc* __restrict__ d, int n, int64_t tile) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (d[mid].tile_begin <= tile) lo = mid; else hi = mid - 1;
  }
  return lo;
}

template <typename T>
__global__ void __launch_bounds__(kNvThreads)
nvfp4_group_amax_kernel(const b200q_nvfp4_desc* __restrict__ descs, int n, int64_t total_tiles) {
  pdl_prologue();
  __shared__ uint32_t red[32];
  const int64_t per = (total_tiles + gridDim.x - 1) / gridDim.x;
  const int64_t t0 = blockIdx.x * per, t1 = min(total_tiles, t0 + per);
  if (t0 >= t1) return;
  int ti = find_tensor(descs, n, t0);
  int64_t t = t0;
  while (t < t1) {
    const b200q_nvfp4_desc d = descs[ti];
    const int64_t tensor_tiles = (d.nblocks + kNvTileBlocks - 1) / kNvTileBlocks;
    const int64_t tend = min(t1, d.tile_begin + tensor_tiles);
    const T* x = static_cast<const T*>(d.x);
    uint32_t m = 0;
    for (; t < tend; ++t) {
      const int64_t tb = (t - d.tile_begin) * kNvTileBlocks;
      Block16<T> blk[kNvUnroll];
#pragma unroll
      for (int u = 0; u < kNvUnroll; ++u) {
        const int64_t b = tb + u * kNvThreads + threadIdx.x;
        if (b < d.nblocks) blk[u].load_keep(x + 16 * b); else blk[u].zero();
      }
#pragma unroll
      for (int u = 0; u < kNvUnroll; ++u) m = max(m, blk[u].amax_f32bits());
    }
    m = cta_max_u32(m, red);
    if (threadIdx.x == 0 && m != 0) {
      uint32_t* slot = reinterpret_cast<uint32_t*>(d.amax);
      if (*reinterpret_cast<volatile uint32_t*>(slot) < m) atomicMax(slot, m);
    }
    ++ti;
  }
}

template <typename T>
__global__ void __launch_bounds__(kNvThreads)
nvfp4_group_quantize_kernel(const b200q_nvfp4_desc* __restrict__ descs, int n, int64_t total_tiles) {
  pdl_prologue();
  const int64_t per = (total_tiles + gridDim.x - 1) / gridDim.x;
  const int64_t t0 = blockIdx.x * per, t1 = min(total_tiles, t0 + per);
  if (t0 >= t1) return;
  int ti = find_tensor(descs, n, t0);
  int64_t t = t0;
  while (t < t1) {
    const b200q_nvfp4_desc d = descs[ti];
    const int64_t tensor_tiles = (d.nblocks + kNvTileBlocks - 1) / kNvTileBlocks;
    const int64_t tend = min(t1, d.tile_begin + tensor_tiles);
    const T* x = static_cast<const T*>(d.x);
    const Nvfp4Tensor tn(__fdiv_rn(*d.amax, 2688.f));
    if (t == d.tile_begin && threadIdx.x == 0 && d.s2) *d.s2 = tn.s2;
    for (; t < tend; ++t) {
      const int64_t tb = (t - d.tile_begin) * kNvTileBlocks;
      Block16<T> blk[kNvUnroll];
#pragma unroll
      for (int u = 0; u < kNvUnroll; ++u) {
        const int64_t b = tb + u * kNvThreads + threadIdx.x;
        if (b < d.nblocks) blk[u].load(x + 16 * b);
      }
#pragma unroll
      for (int u = 0; u < kNvUnroll; ++u) {
        const int64_t b = tb + u * kNvThreads + threadIdx.x;
        if (b < d.nblocks) nvfp4_quant_block<T>(blk[u], b, tn, nullptr, d.packed, d.scales);
      }
    }
    ++ti;
  }
}

}  // namespace b200q

using namespace b200q;

#define B200Q_REQUIRE_ALIGNED32(p) \
  do {                             \
    if ((reinterpret_cast<uintptr_t>(p) & 31u) != 0) return B200Q_ERR_ALIGN; \
  } while (0)

extern "C" int b200q_nvfp4_group_tile_elems(void) { return kNvTileElems; }

// Launchers shared with the other-block-size entry points: `pair` = scale blocks of 32 elements.
namespace b200q {

int nvfp4_launch_quantize(const void* x, int64_t nunits, int dtype, const float* global,
                          const uint8_t* scales_in, uint8_t* packed, uint8_t* scales, float* s2_out,
                          int flags, bool pair, cudaStream_t s) {
  return B200Q_DISPATCH(dtype, [&] {
    int grid = grid_for(nunits, kNvTileBlocks, 8);
    launch_pdl(nvfp4_quantize_kernel<T>, grid, kNvThreads, 0, s, static_cast<const T*>(x), nunits, global,
               (flags & B200Q_NVFP4_GLOBAL_IS_SCALE2) != 0, scales_in, packed, scales, s2_out, pair,
               (flags & B200Q_NVFP4_SATURATE_SCALES) != 0);
    return launch_status();
  });
}

int nvfp4_launch_fake(const void* x, void* y, int64_t nunits, int dtype, const float* amax, bool pair,
                      cudaStream_t s) {
  return B200Q_DISPATCH(dtype, [&] {
    int grid = grid_for(nunits, kNvTileBlocks, 8);
    launch_pdl(nvfp4_fake_kernel<T>, grid, kNvThreads, 0, s, static_cast<const T*>(x), static_cast<T*>(y), nunits,
               amax, pair);
    return launch_status();
  });
}

int nvfp4_launch_dequantize(const uint8_t* packed, const uint8_t* scales, const float* s2, void* y,
                            int64_t nunits, int dtype, bool pair, cudaStream_t s) {
  return B200Q_DISPATCH(dtype, [&] {
    int grid = grid_for(nunits, kNvThreads, 8);
    launch_pdl(nvfp4_dequantize_kernel<T>, grid, kNvThreads, 0, s, packed, scales, s2, static_cast<T*>(y), nunits, pair);
    return launch_status();
  });
}

}  // namespace b200q

extern "C" int b200q_nvfp4_quantize(const void* x, int64_t nblocks, int dtype, const float* global,
                                    const uint8_t* scales_in, uint8_t* packed, uint8_t* scales,
                                    float* s2_out, int flags, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(global); B200Q_REQUIRE_PTR(packed);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED32(x);
  if ((reinterpret_cast<uintptr_t>(packed) & 7u) != 0) return B200Q_ERR_ALIGN;
  if (nblocks <= 0) return B200Q_ERR_SHAPE;
  if (flags & ~(B200Q_NVFP4_GLOBAL_IS_SCALE2 | B200Q_NVFP4_SATURATE_SCALES)) return B200Q_ERR_ARG;
  return nvfp4_launch_quantize(x, nblocks, dtype, global, scales_in, packed, scales, s2_out, flags, false,
                               static_cast<cudaStream_t>(stream));
}

extern "C" int b200q_nvfp4_fake(const void* x, void* y, int64_t nblocks, int dtype, const float* amax,
                                void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(y); B200Q_REQUIRE_PTR(amax);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED32(x); B200Q_REQUIRE_ALIGNED32(y);
  if (nblocks <= 0) return B200Q_ERR_SHAPE;
  return nvfp4_launch_fake(x, y, nblocks, dtype, amax, false, static_cast<cudaStream_t>(stream));
}

extern "C" int b200q_nvfp4_dequantize(const uint8_t* packed, const uint8_t* scales, const float* s2,
                                      void* y, int64_t nblocks, int dtype, void* stream) {
  B200Q_REQUIRE_PTR(packed); B200Q_REQUIRE_PTR(scales); B200Q_REQUIRE_PTR(s2); B200Q_REQUIRE_PTR(y);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED32(y);
  if ((reinterpret_cast<uintptr_t>(packed) & 7u) != 0) return B200Q_ERR_ALIGN;
  if (nblocks <= 0) return B200Q_ERR_SHAPE;
  return nvfp4_launch_dequantize(packed, scales, s2, y, nblocks, dtype, false, static_cast<cudaStream_t>(stream));
}

static int check_group(const b200q_nvfp4_desc* descs, int n, int64_t total_tiles, int dtype) {
  B200Q_REQUIRE_PTR(descs);
  B200Q_REQUIRE_DTYPE(dtype);
  if ((reinterpret_cast<uintptr_t>(descs) & 7u) != 0) return B200Q_ERR_ALIGN;
  if (n <= 0 || total_tiles <= 0) return B200Q_ERR_SHAPE;
  return B200Q_OK;
}

extern "C" int b200q_nvfp4_group_amax(const b200q_nvfp4_desc* descs, int n, int64_t total_tiles,
                                      int dtype, void* stream) {
  if (int e = check_group(descs, n, total_tiles, dtype)) return e;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return B200Q_DISPATCH(dtype, [&] {
    int grid = grid_for(total_tiles, 1, kNvCtasPerSm);
    launch_pdl(nvfp4_group_amax_kernel<T>, grid, kNvThreads, 0, s, descs, n, total_tiles);
    return launch_status();
  });
}

extern "C" int b200q_nvfp4_group_quantize(const b200q_nvfp4_desc* descs, int n, int64_t total_tiles,
                                          int dtype, void* stream) {
  if (int e = check_group(descs, n, total_tiles, dtype)) return e;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return B200Q_DISPATCH(dtype, [&] {
    int grid = grid_for(total_tiles, 1, kNvCtasPerSm);
    launch_pdl(nvfp4_group_quantize_kernel<T>, grid, kNvThreads, 0, s, descs, n, total_tiles);
    return launch_status();
  });
}

// ---- grouped quantisation without any allocation -------------------------------------------------
// Some hosts may not allocate device memory at the point where they quantise: an inference-engine
// plugin inside its enqueue call, a service whose memory is handed out once at start-up by a
// budgeting allocator, a process sharing the GPU under a hard memory cap.  The grouped kernels need
// scratch the caller would otherwise have to provide (the descriptor table in device memory and one
// abs-max slot per tensor), so this variant keeps that scratch in the library image itself.
//
// The array below is part of every CUDA context that loads the library (about 62 KB per GPU, held
// until the process exits).  Its name is only a host-side handle: the device address is fetched per
// device with cudaGetSymbolAddress and that pointer is what the kernels receive.
namespace b200q {

constexpr int kNoAllocMaxTensors = 1024;
constexpr size_t kNoAllocDescBytes = sizeof(b200q_nvfp4_desc) * kNoAllocMaxTensors;
constexpr size_t kNoAllocAmaxOffset = (kNoAllocDescBytes + 255) / 256 * 256;
constexpr size_t kNoAllocBytes = kNoAllocAmaxOffset + sizeof(float) * kNoAllocMaxTensors;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

constexpr int kMaxDevices = 64;
constexpr int kNoAllocChunk = 64;                          // descriptors staged per host-to-device copy
static unsigned char* g_noalloc_ptr[kMaxDevices] = {};   // device address of the array, per device

// Device address of the scratch array on the current device (looked up on the first call made
// with that device current; a benign race between threads stores the same value twice).  The
// address is cached for the life of the process; `refresh` asks the runtime again (used once when a
// copy into the cached address fails, which is what a host application's cudaDeviceReset between
// two calls leads to).
static int noalloc_scratch(unsigned char** out, bool refresh) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200Q_ERR_CUDA;
  if (refresh || g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) return B200Q_ERR_CUDA;
    g_noalloc_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return B200Q_OK;
}

}  // namespace b200q

extern "C" int b200q_nvfp4_group_max_tensors_noalloc(void) { return kNoAllocMaxTensors; }

extern "C" int b200q_nvfp4_group_quantize_noalloc(const b200q_nvfp4_desc* host_descs, int n, int dtype,
                                                  void* stream) {
  B200Q_REQUIRE_PTR(host_descs);
  B200Q_REQUIRE_DTYPE(dtype);
  if (n <= 0) return B200Q_ERR_SHAPE;
  if (n > kNoAllocMaxTensors) return B200Q_ERR_CAPACITY;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The table travels from a buffer in this function's frame: a captured copy would keep a pointer
  // into a frame that is gone when the graph replays, so a capturing stream is refused outright.
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &capturing) != cudaSuccess) { cudaGetLastError(); return B200Q_ERR_CUDA; }
  if (capturing != cudaStreamCaptureStatusNone) return B200Q_ERR_UNSUPPORTED;
  // everything is validated before anything is enqueued
  int64_t tiles = 0;
  for (int i = 0; i < n; ++i) {
    const b200q_nvfp4_desc& d = host_descs[i];
    if (d.x == nullptr || d.packed == nullptr) return B200Q_ERR_NULL;
    if (d.nblocks <= 0) return B200Q_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(d.x) & 31u) || (reinterpret_cast<uintptr_t>(d.packed) & 7u)) return B200Q_ERR_ALIGN;
    tiles += (d.nblocks + kNvTileBlocks - 1) / kNvTileBlocks;
  }
  unsigned char* scratch = nullptr;
  if (int e = noalloc_scratch(&scratch, false)) return e;

  // The table is staged through a small buffer in this frame (3.5 KB, so a worker thread with a
  // small stack can call this), kNoAllocChunk descriptors per copy: abs-max slots redirected into
  // the scratch, tiles numbered.  The buffer is pageable host memory, so cudaMemcpyAsync returns
  // only after the runtime has taken its own copy of it (which is what makes reusing the buffer for
  // the next chunk safe) and may wait for earlier work of the stream to do so.
  b200q_nvfp4_desc chunk[kNoAllocChunk];
  int64_t tile_begin = 0;
  for (int c0 = 0; c0 < n; c0 += kNoAllocChunk) {
    const int cn = n - c0 < kNoAllocChunk ? n - c0 : kNoAllocChunk;
    const int64_t chunk_tile_begin = tile_begin;
    for (int attempt = 0;; ++attempt) {
      float* d_amax = reinterpret_cast<float*>(scratch + kNoAllocAmaxOffset);
      tile_begin = chunk_tile_begin;
      for (int i = 0; i < cn; ++i) {
        chunk[i] = host_descs[c0 + i];
        chunk[i].amax = d_amax + c0 + i;
        chunk[i].tile_begin = tile_begin;
        tile_begin += (chunk[i].nblocks + kNvTileBlocks - 1) / kNvTileBlocks;
      }
      b200q_nvfp4_desc* dst = reinterpret_cast<b200q_nvfp4_desc*>(scratch) + c0;
      if (cudaMemcpyAsync(dst, chunk, sizeof(b200q_nvfp4_desc) * cn, cudaMemcpyHostToDevice, s) == cudaSuccess) break;
      cudaGetLastError();
      // first chunk only: the cached address may belong to a context that was reset since
      if (attempt > 0 || c0 > 0) return B200Q_ERR_CUDA;
      if (int e = noalloc_scratch(&scratch, true)) return e;
    }
  }
  b200q_nvfp4_desc* d_descs = reinterpret_cast<b200q_nvfp4_desc*>(scratch);
  float* d_amax = reinterpret_cast<float*>(scratch + kNoAllocAmaxOffset);
  // The array keeps whatever the previous call left: the table is overwritten above and the
  // abs-max slots, which the first kernel only ever raises, are cleared here.
  if (cudaMemsetAsync(d_amax, 0, sizeof(float) * n, s) != cudaSuccess) return B200Q_ERR_CUDA;
  return B200Q_DISPATCH(dtype, [&] {
    int grid = grid_for(tiles, 1, 8);
    launch_pdl(nvfp4_group_amax_kernel<T>, grid, kNvThreads, 0, s, d_descs, n, tiles);
    launch_pdl(nvfp4_group_quantize_kernel<T>, grid, kNvThreads, 0, s, d_descs, n, tiles);
    return launch_status();
  });
}
