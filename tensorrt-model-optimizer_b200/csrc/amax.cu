// Abs-max reductions: per tensor, per axis of a [outer, axis, inner] view, per contiguous block.
//
// All three read the input exactly once with 128-bit loads.  |x| is compared as an unsigned bit
// pattern (sign bit cleared), which orders like the magnitude and keeps NaN the largest value,
// and results are folded into the fp32 output slot with atomicMax on that bit pattern, so the
// slot doubles as the running max of a calibrator and as a lane of a flat all-reduce buffer.
#include "common.cuh"

namespace b200q {

static int g_sm_count = 0;
int sm_count_cached() {
  if (g_sm_count == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      g_sm_count = n;
    else
      g_sm_count = 148;
  }
  return g_sm_count;
}

#ifndef B200Q_AMAX_THREADS
// 256 threads x 8 loads of 16 bytes x 4 CTAs per SM = 128 KB in flight per SM, 64 registers per thread.
// Measured on 16 bf16 [8192, 4096] tensors in turn (fraction of the measured copy bandwidth): 0.88;
// 512 x 4 x 4: 0.69, 512 x 8 x 4 (register-limited to 3 CTAs): 0.65, 256 x 8 x 8: 0.86, 128 x 8 x 8: 0.82.
#define B200Q_AMAX_THREADS 256
#define B200Q_AMAX_UNROLL 8
#define B200Q_AMAX_CTAS 4
#endif
constexpr int kAmaxThreads = B200Q_AMAX_THREADS;
constexpr int kAmaxUnroll = B200Q_AMAX_UNROLL;  // 16-byte loads in flight per thread
constexpr int kAmaxCtasPerSm = B200Q_AMAX_CTAS;

template <typename T>
__global__ void __launch_bounds__(kAmaxThreads)
amax_tensor_kernel(const T* __restrict__ x, int64_t n, uint32_t* __restrict__ amax_bits) {
  using E = Elem<T>;
  pdl_prologue();
  __shared__ uint32_t red[32];
  const int64_t npack = n / E::kPerPack;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  uint32_t acc = 0;
  // every round keeps kAmaxUnroll loads per thread in flight, the last (partial) one included: slots
  // beyond the end are zeros, so a tensor of a few packs per thread never falls back to one load at a time
  for (; i < npack; i += kAmaxUnroll * stride) {
    uint4 v[kAmaxUnroll];
#pragma unroll
    for (int u = 0; u < kAmaxUnroll; ++u)
      v[u] = i + u * stride < npack ? ld_stream(xv + i + u * stride) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int u = 0; u < kAmaxUnroll; ++u) acc = E::acc_max(acc, v[u]);
  }
  uint32_t bits = E::acc_to_f32bits(acc);
  // ragged tail (fewer than one pack)
  if (blockIdx.x == 0 && threadIdx.x < n - npack * E::kPerPack) {
    float f = fabsf(E::to_float(x[npack * E::kPerPack + threadIdx.x]));
    bits = max(bits, __float_as_uint(f));
  }
  bits = cta_max_u32(bits, red);
  if (threadIdx.x == 0 && bits != 0) atomicMax(amax_bits, bits);
}

// One CTA walks a slice of one row of length `inner`; row r belongs to channel r % axis.
template <typename T>
__global__ void __launch_bounds__(256)
amax_rows_kernel(const T* __restrict__ x, int64_t rows, int64_t axis, int64_t inner,
                 int slices_per_row, uint32_t* __restrict__ amax_bits) {
  pdl_prologue();
  using E = Elem<T>;
  __shared__ uint32_t red[32];
  const int64_t total = rows * slices_per_row;
  for (int64_t w = blockIdx.x; w < total; w += gridDim.x) {
    const int64_t r = w / slices_per_row;
    const int s = static_cast<int>(w - r * slices_per_row);
    const T* row = x + r * inner;
    const bool vec_ok = (inner % E::kPerPack) == 0;  // rows stay 16-byte aligned
    uint32_t bits = 0;
    if (vec_ok) {
      const int64_t npack = inner / E::kPerPack;
      const int64_t per = (npack + slices_per_row - 1) / slices_per_row;
      const int64_t lo = s * per, hi = min(npack, lo + per);
      const uint4* rv = reinterpret_cast<const uint4*>(row);
      uint32_t acc = 0;
      int64_t i = lo + threadIdx.x;
      for (; i + 3 * blockDim.x < hi; i += 4 * blockDim.x) {
        uint4 v0 = ld_stream(rv + i), v1 = ld_stream(rv + i + blockDim.x),
              v2 = ld_stream(rv + i + 2 * blockDim.x), v3 = ld_stream(rv + i + 3 * blockDim.x);
        acc = E::acc_max(E::acc_max(E::acc_max(E::acc_max(acc, v0), v1), v2), v3);
      }
      for (; i < hi; i += blockDim.x) acc = E::acc_max(acc, ld_stream(rv + i));
      bits = E::acc_to_f32bits(acc);
    } else {
      const int64_t per = (inner + slices_per_row - 1) / slices_per_row;
      const int64_t lo = s * per, hi = min(inner, lo + per);
      for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x)
        bits = max(bits, __float_as_uint(fabsf(E::to_float(row[i]))));
    }
    bits = cta_max_u32(bits, red);
    if (threadIdx.x == 0 && bits != 0) atomicMax(amax_bits + (r % axis), bits);
  }
}

// inner == 1: x is [outer, axis] and the reduction runs down the columns.  Each thread owns one
// pack of adjacent columns and walks a band of rows.
template <typename T>
__global__ void __launch_bounds__(256)
amax_cols_kernel(const T* __restrict__ x, int64_t outer, int64_t axis, int rows_per_band,
                 uint32_t* __restrict__ amax_bits) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  const int64_t cpack = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (cpack * P >= axis) return;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * rows_per_band;
  const int64_t r1 = min(outer, r0 + rows_per_band);
  const uint4* base = reinterpret_cast<const uint4*>(x) + cpack;
  const int64_t rstride = axis / P;
  uint4 m = make_uint4(0, 0, 0, 0);
  auto fold = [&](const uint4& v) {
    if (P == 8) {
      m.x = __vmaxu2(m.x, v.x & 0x7fff7fffu); m.y = __vmaxu2(m.y, v.y & 0x7fff7fffu);
      m.z = __vmaxu2(m.z, v.z & 0x7fff7fffu); m.w = __vmaxu2(m.w, v.w & 0x7fff7fffu);
    } else {
      m.x = max(m.x, v.x & 0x7fffffffu); m.y = max(m.y, v.y & 0x7fffffffu);
      m.z = max(m.z, v.z & 0x7fffffffu); m.w = max(m.w, v.w & 0x7fffffffu);
    }
  };
  int64_t r = r0;
  for (; r + 3 < r1; r += 4) {
    uint4 v0 = ld_stream(base + r * rstride), v1 = ld_stream(base + (r + 1) * rstride),
          v2 = ld_stream(base + (r + 2) * rstride), v3 = ld_stream(base + (r + 3) * rstride);
    fold(v0); fold(v1); fold(v2); fold(v3);
  }
  for (; r < r1; ++r) fold(ld_stream(base + r * rstride));
  const uint32_t w[4] = {m.x, m.y, m.z, m.w};
  uint32_t* out = amax_bits + cpack * P;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (P == 8) {
      // 16-bit patterns -> fp32 bit order (bf16: shift; fp16: convert)
      uint32_t lo = w[k] & 0xffffu, hi = w[k] >> 16;
      uint32_t blo, bhi;
      if (sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value) {
        blo = lo << 16; bhi = hi << 16;
      } else {
        blo = __float_as_uint(__half2float(__ushort_as_half(static_cast<uint16_t>(lo))));
        bhi = __float_as_uint(__half2float(__ushort_as_half(static_cast<uint16_t>(hi))));
      }
      if (blo) atomicMax(out + 2 * k, blo);
      if (bhi) atomicMax(out + 2 * k + 1, bhi);
    } else {
      if (w[k]) atomicMax(out + k, w[k]);
    }
  }
}

// Scalar fallback for views the vector kernels do not cover.
template <typename T>
__global__ void amax_axis_generic_kernel(const T* __restrict__ x, int64_t n, int64_t axis,
                                         int64_t inner, uint32_t* __restrict__ amax_bits) {
  pdl_prologue();
  using E = Elem<T>;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    uint32_t b = __float_as_uint(fabsf(E::to_float(x[i])));
    if (b) atomicMax(amax_bits + (i / inner) % axis, b);
  }
}

// `lanes` adjacent lanes (power of two <= 32) share one block; each lane holds `PPL` packs.
template <typename T, int PPL>
__global__ void __launch_bounds__(256)
amax_blocks_kernel(const T* __restrict__ x, int64_t nblocks, int lanes, float* __restrict__ out) {
  pdl_prologue();
  using E = Elem<T>;
  const int64_t gthread = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t total = nblocks * lanes;  // a multiple of `lanes`, so sub-groups stay whole
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  for (int64_t t = gthread; t < ((total + 31) / 32) * 32; t += nthreads) {
    uint32_t acc = 0;
    if (t < total) {
      uint4 v[PPL];
#pragma unroll
      for (int p = 0; p < PPL; ++p) v[p] = ld_stream(xv + t * PPL + p);
#pragma unroll
      for (int p = 0; p < PPL; ++p) acc = E::acc_max(acc, v[p]);
    }
    uint32_t bits = E::acc_to_f32bits(acc);
    for (int o = lanes >> 1; o > 0; o >>= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
    if (t < total && (t & (lanes - 1)) == 0) out[t >> (__ffs(lanes) - 1)] = __uint_as_float(bits);
  }
}

template <typename T>
__global__ void amax_blocks_generic_kernel(const T* __restrict__ x, int64_t nblocks, int block,
                                           float* __restrict__ out) {
  pdl_prologue();
  using E = Elem<T>;
  for (int64_t b = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; b < nblocks;
       b += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    uint32_t bits = 0;
    for (int i = 0; i < block; ++i)
      bits = max(bits, __float_as_uint(fabsf(E::to_float(x[b * block + i]))));
    out[b] = __uint_as_float(bits);
  }
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_amax_tensor(const void* x, int64_t n, int dtype, float* amax_io, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(amax_io);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x);
  if (n <= 0) return B200Q_ERR_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return B200Q_DISPATCH(dtype, [&] {
    const int64_t npack = n / Elem<T>::kPerPack;
    int grid = grid_for(npack, kAmaxThreads * kAmaxUnroll, kAmaxCtasPerSm);
    launch_pdl(amax_tensor_kernel<T>, grid, kAmaxThreads, 0, s, static_cast<const T*>(x), n,
               reinterpret_cast<uint32_t*>(amax_io));
    return launch_status();
  });
}

extern "C" int b200q_amax_axis(const void* x, int64_t outer, int64_t axis, int64_t inner, int dtype,
                               float* amax_io, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(amax_io);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x);
  if (outer <= 0 || axis <= 0 || inner <= 0) return B200Q_ERR_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t* out = reinterpret_cast<uint32_t*>(amax_io);
  return B200Q_DISPATCH(dtype, [&] {
    constexpr int P = Elem<T>::kPerPack;
    const T* xp = static_cast<const T*>(x);
    if (inner == 1 && axis % P == 0) {
      const int64_t cpacks = axis / P;
      const int bx = static_cast<int>((cpacks + 255) / 256);
      // enough row bands to fill the machine ~8 CTAs per SM deep, at least 16 rows per band
      int64_t want = (static_cast<int64_t>(sm_count_cached()) * 8 + bx - 1) / bx;
      int64_t bands = outer / 16 > 0 ? (outer / 16 < want ? outer / 16 : want) : 1;
      if (bands > 65535) bands = 65535;
      const int rpb = static_cast<int>((outer + bands - 1) / bands);
      dim3 grid(bx, static_cast<unsigned>((outer + rpb - 1) / rpb));
      launch_pdl(amax_cols_kernel<T>, grid, 256, 0, s, xp, outer, axis, rpb, out);
    } else if (inner >= 64 && (inner % P == 0 || inner >= 4096)) {
      const int64_t rows = outer * axis;
      // split long rows so that at least ~4 CTAs per SM have work
      int slices = 1;
      const int64_t want = static_cast<int64_t>(sm_count_cached()) * 4;
      if (rows < want) {
        int64_t sp = (want + rows - 1) / rows;
        int64_t max_sp = inner / (256 * P * 4);
        if (max_sp < 1) max_sp = 1;
        slices = static_cast<int>(sp < max_sp ? sp : max_sp);
      }
      int grid = grid_for(rows * slices, 1, 8);
      launch_pdl(amax_rows_kernel<T>, grid, 256, 0, s, xp, rows, axis, inner, slices, out);
    } else {
      const int64_t n = outer * axis * inner;
      int grid = grid_for(n, 256, 8);
      launch_pdl(amax_axis_generic_kernel<T>, grid, 256, 0, s, xp, n, axis, inner, out);
    }
    return launch_status();
  });
}

extern "C" int b200q_amax_blocks(const void* x, int64_t nblocks, int block, int dtype,
                                 float* amax_out, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(amax_out);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x);
  if (nblocks <= 0 || block <= 0) return B200Q_ERR_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return B200Q_DISPATCH(dtype, [&] {
    constexpr int P = Elem<T>::kPerPack;
    const T* xp = static_cast<const T*>(x);
    const int packs = block / P;
    const bool pow2 = packs > 0 && (packs & (packs - 1)) == 0 && block % P == 0;
    if (pow2 && packs <= 64) {
      // up to 2 packs per lane, then spread over lanes
      const int ppl = packs >= 2 ? 2 : 1;
      const int lanes = packs / ppl;
      int grid = grid_for(nblocks * lanes, 256, 8);
      if (ppl == 2)
        launch_pdl(amax_blocks_kernel<T, 2>, grid, 256, 0, s, xp, nblocks, lanes, amax_out);
      else
        launch_pdl(amax_blocks_kernel<T, 1>, grid, 256, 0, s, xp, nblocks, lanes, amax_out);
    } else {
      int grid = grid_for(nblocks, 256, 8);
      launch_pdl(amax_blocks_generic_kernel<T>, grid, 256, 0, s, xp, nblocks, block, amax_out);
    }
    return launch_status();
  });
}
