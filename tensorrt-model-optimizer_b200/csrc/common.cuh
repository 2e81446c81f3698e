// Shared device/host helpers: 128-bit vector access, element-type traits, launch plumbing.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "../../include/b200q.h"

namespace b200q {

// ---- host-side argument checks -------------------------------------------------------------
#define B200Q_REQUIRE_PTR(p) \
  do {                       \
    if ((p) == nullptr) return B200Q_ERR_NULL; \
  } while (0)
#define B200Q_REQUIRE_ALIGNED(p) \
  do {                           \
    if ((reinterpret_cast<uintptr_t>(p) & 15u) != 0) return B200Q_ERR_ALIGN; \
  } while (0)
#define B200Q_REQUIRE_DTYPE(d) \
  do {                         \
    if ((d) != B200Q_F32 && (d) != B200Q_F16 && (d) != B200Q_BF16) return B200Q_ERR_DTYPE; \
  } while (0)

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? B200Q_OK : B200Q_ERR_CUDA; }

// ---- programmatic dependent launch ----------------------------------------------------------
// Streaming kernels are launched with programmatic stream serialisation and open with
// pdl_prologue(): they let the NEXT kernel of the stream become resident while their own tail
// drains, and then wait until the PREVIOUS kernel has completed and its writes are visible before
// touching global memory.  Results and ordering are those of plain stream order; what overlaps is
// launch latency, block scheduling and per-CTA set-up.  A predecessor that never signals (any
// kernel of another library) simply completes first, as without the attribute.
template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// nothing in global memory may be read or written before this returns
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_prologue() {
  pdl_launch_dependents();
  pdl_wait();
}
#endif

int sm_count_cached();

// Dispatch a generic lambda on the element type.
#define B200Q_DISPATCH(dtype, ...)                         \
  [&] {                                                    \
    switch (dtype) {                                       \
      case B200Q_F32: { using T = float; return __VA_ARGS__(); }          \
      case B200Q_F16: { using T = __half; return __VA_ARGS__(); }         \
      default: { using T = __nv_bfloat16; return __VA_ARGS__(); }        \
    }                                                      \
  }()

// ---- element-type traits --------------------------------------------------------------------
// A "pack" is one 16-byte vector: 4 fp32 or 8 half/bf16 elements.
template <typename T> struct Elem;

template <> struct Elem<float> {
  static constexpr int kPerPack = 4;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                      __float_as_uint(f[3]));
  }
  // max over the pack of the |x| bit patterns, widened to fp32 bit order (NaN stays largest)
  static __device__ __forceinline__ uint32_t absmax_bits(const uint4& v) {
    uint32_t a = max(v.x & 0x7fffffffu, v.y & 0x7fffffffu);
    uint32_t b = max(v.z & 0x7fffffffu, v.w & 0x7fffffffu);
    return max(a, b);
  }
  static __device__ __forceinline__ uint32_t acc_max(uint32_t acc, const uint4& v) {
    return max(acc, absmax_bits(v));
  }
  static __device__ __forceinline__ uint32_t acc_to_f32bits(uint32_t acc) { return acc; }
  static __device__ __forceinline__ float to_float(float x) { return x; }
  static __device__ __forceinline__ float from_float(float x) { return x; }
};

template <> struct Elem<__nv_bfloat16> {
  static constexpr int kPerPack = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
  }
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
  }
  // accumulator is a pair of 15-bit |x| patterns (u16x2); unsigned halfword max keeps NaN largest
  static __device__ __forceinline__ uint32_t acc_max(uint32_t acc, const uint4& v) {
    uint32_t a = __vmaxu2(v.x & 0x7fff7fffu, v.y & 0x7fff7fffu);
    uint32_t b = __vmaxu2(v.z & 0x7fff7fffu, v.w & 0x7fff7fffu);
    return __vmaxu2(acc, __vmaxu2(a, b));
  }
  static __device__ __forceinline__ uint32_t acc_to_f32bits(uint32_t acc) {
    return max(acc & 0xffffu, acc >> 16) << 16;
  }
  static __device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};

template <> struct Elem<__half> {
  static constexpr int kPerPack = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(h[i]);
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
  }
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __half2 p = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
  }
  static __device__ __forceinline__ uint32_t acc_max(uint32_t acc, const uint4& v) {
    uint32_t a = __vmaxu2(v.x & 0x7fff7fffu, v.y & 0x7fff7fffu);
    uint32_t b = __vmaxu2(v.z & 0x7fff7fffu, v.w & 0x7fff7fffu);
    return __vmaxu2(acc, __vmaxu2(a, b));
  }
  static __device__ __forceinline__ uint32_t acc_to_f32bits(uint32_t acc) {
    uint16_t h = static_cast<uint16_t>(max(acc & 0xffffu, acc >> 16));
    return __float_as_uint(__half2float(__ushort_as_half(h)));
  }
  static __device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_float(float x) { return __float2half_rn(x); }
};

// ---- 128-bit global access --------------------------------------------------------------------
// Streaming read that bypasses L1 allocation: every input byte is used exactly once per pass.
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// Read that keeps the line in L2 with priority (used when a second pass re-reads the tensor).
__device__ __forceinline__ uint4 ld_keep(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::evict_last.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream(void* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_stream(void* p, const uint2& v) {
  asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

__device__ __forceinline__ uint32_t warp_max_u32(uint32_t v) { return __reduce_max_sync(0xffffffffu, v); }

// max over the CTA (blockDim.x a multiple of 32, <= 1024); result valid in every thread
__device__ __forceinline__ uint32_t cta_max_u32(uint32_t v, uint32_t* smem32) {
  v = warp_max_u32(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) smem32[warp] = v;
  __syncthreads();
  uint32_t r = (lane < nw) ? smem32[lane] : 0u;
  r = warp_max_u32(r);
  __syncthreads();
  return r;
}

// Persistent-style grid: a multiple of the SM count, capped by the work available.
inline int grid_for(int64_t work_items, int per_cta, int ctas_per_sm) {
  int64_t need = (work_items + per_cta - 1) / per_cta;
  int64_t cap = static_cast<int64_t>(sm_count_cached()) * ctas_per_sm;
  if (need < 1) need = 1;
  return static_cast<int>(need < cap ? need : cap);
}

// Division of a 31-bit index by a launch-invariant divisor as multiply-high + shift (the divisor's
// magic number is computed once on the host): 2 integer instructions instead of the ~50 of a
// 64-bit division in the index arithmetic of every 16-byte pack.
struct FastDiv {
  uint32_t d, mul, shr;
  FastDiv() : d(1), mul(0), shr(0) {}
  explicit FastDiv(uint32_t divisor) : d(divisor), mul(0), shr(0) {
    if (d > 1) {
      uint32_t lg = 0;
      while ((1ull << lg) < d) ++lg;                      // ceil(log2 d)
      const uint32_t p = 31 + lg;
      mul = static_cast<uint32_t>(((1ull << p) + d - 1) / d);
      shr = p - 32;
    }
  }
  // n < 2^31
  __device__ __forceinline__ uint32_t div(uint32_t n) const { return d == 1 ? n : __umulhi(n, mul) >> shr; }
  __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const {
    q = div(n);
    r = n - q * d;
  }
};
constexpr int64_t kFastDivLimit = (1ll << 31) - 1;

}  // namespace b200q
