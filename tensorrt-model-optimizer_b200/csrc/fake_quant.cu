// Fake quantisation (quantise + dequantise in one pass, output in the input type):
// integer grids (INT8/INT4/...) and FP8 E4M3, per tensor, per channel of a [outer, axis, inner]
// view, and per row with the row abs-max found on chip in the same pass.
//
// Every kernel streams 16-byte packs: several independent loads are issued before the first use
// so that each thread keeps 64 bytes in flight, and results leave with streaming 16-byte stores.
#include "numerics.cuh"

namespace b200q {

constexpr int kEwThreads = 256;
constexpr int kEwUnroll = 4;

// ---- per-element functors -----------------------------------------------------------------------
// A functor is built once per thread from the per-tensor amax, or once per pack from the channel amax.
struct IntFq {
  IntQ q;
  IntScale s;
  __device__ __forceinline__ IntFq() {}
  __device__ __forceinline__ IntFq(const IntQ& q_, float amax) : q(q_), s(make_int_scale(q_, amax)) {}
  __device__ __forceinline__ float operator()(float x) const { return intq_apply(x, s, q); }
  template <int N> __device__ __forceinline__ void apply(float* f) const { intq_apply_n<N>(f, s, q); }
};

struct E4m3Fq {
  float scale, inv;
  bool scaled;
  __device__ __forceinline__ E4m3Fq(const IntQ&, float amax) {
    scaled = true;
    scale = __fdiv_rn(448.f, amax);
    inv = __fdiv_rn(1.f, scale);
  }
  __device__ __forceinline__ E4m3Fq() : scale(1.f), inv(1.f), scaled(false) {}
  template <int N> __device__ __forceinline__ void apply(float* f) const {
#pragma unroll
    for (int i = 0; i < N; i += 2) {
      float a = f[i], b = f[i + 1];
      if (scaled) { a *= scale; b *= scale; }
      float2 r = e4m3x2_to_f32x2(f32x2_to_e4m3x2_sat(a, b));
      if (scaled) { r.x *= inv; r.y *= inv; }
      f[i] = r.x; f[i + 1] = r.y;
    }
  }
  __device__ __forceinline__ float operator()(float x) const {
    float t[2] = {x, 0.f};
    apply<2>(t);
    return t[0];
  }
};

// ---- one amax for the whole tensor -----------------------------------------------------------
template <typename T, typename F>
__global__ void __launch_bounds__(kEwThreads)
fq_tensor_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t n,
                 const float* __restrict__ amax, IntQ q) {
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  pdl_prologue();
  const F f = amax ? F(q, __ldg(amax)) : F(q, 1.f);
  const int64_t npack = n / P;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  uint4* yv = reinterpret_cast<uint4*>(y);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + (kEwUnroll - 1) * stride < npack; i += kEwUnroll * stride) {
    uint4 v[kEwUnroll];
#pragma unroll
    for (int u = 0; u < kEwUnroll; ++u) v[u] = ld_stream(xv + i + u * stride);
#pragma unroll
    for (int u = 0; u < kEwUnroll; ++u) {
      float t[P];
      E::unpack(v[u], t);
      f.template apply<P>(t);
      st_stream(yv + i + u * stride, E::pack(t));
    }
  }
  for (; i < npack; i += stride) {
    float t[P];
    E::unpack(ld_stream(xv + i), t);
    f.template apply<P>(t);
    st_stream(yv + i, E::pack(t));
  }
  if (blockIdx.x == 0 && threadIdx.x < n - npack * P) {
    const int64_t j = npack * P + threadIdx.x;
    y[j] = E::from_float(f(E::to_float(x[j])));
  }
}

// plain E4M3 cast without amax
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
e4m3_cast_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t n) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  const E4m3Fq f;
  const int64_t npack = n / P;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  uint4* yv = reinterpret_cast<uint4*>(y);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < npack; i += stride) {
    float t[P];
    E::unpack(ld_stream(xv + i), t);
    f.template apply<P>(t);
    st_stream(yv + i, E::pack(t));
  }
  if (blockIdx.x == 0 && threadIdx.x < n - npack * P) {
    const int64_t j = npack * P + threadIdx.x;
    y[j] = E::from_float(f(E::to_float(x[j])));
  }
}

// ---- amax per channel, inner a multiple of the pack: a pack lies inside one channel ------------
template <typename T, typename F>
__global__ void __launch_bounds__(kEwThreads)
fq_axis_inner_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t npack, FastDiv axis,
                     FastDiv inner_packs, const float* __restrict__ amax, IntQ q) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  uint4* yv = reinterpret_cast<uint4*>(y);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i < npack; i += kEwUnroll * stride) {
    uint4 v[kEwUnroll];
    float am[kEwUnroll];
#pragma unroll
    for (int u = 0; u < kEwUnroll; ++u) {
      const int64_t j = i + u * stride;
      if (j < npack) {
        v[u] = ld_stream(xv + j);
        uint32_t row = inner_packs.div(static_cast<uint32_t>(j)), oq, ch;   // npack < 2^31 here
        axis.divmod(row, oq, ch);
        am[u] = __ldg(amax + ch);
      }
    }
#pragma unroll
    for (int u = 0; u < kEwUnroll; ++u) {
      const int64_t j = i + u * stride;
      if (j < npack) {
        const F f(q, am[u]);
        float t[P];
        E::unpack(v[u], t);
        f.template apply<P>(t);
        st_stream(yv + j, E::pack(t));
      }
    }
  }
}

// ---- amax per column (inner == 1, axis a multiple of the pack) ---------------------------------
// A thread owns one pack of adjacent channels, forms their scales once and walks a band of rows.
template <typename T, typename F>
__global__ void __launch_bounds__(kEwThreads)
fq_axis_cols_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t outer, int64_t axis,
                    int rows_per_band, const float* __restrict__ amax, IntQ q) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  const int64_t cpack = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (cpack * P >= axis) return;
  F f[P];
#pragma unroll
  for (int k = 0; k < P; ++k) f[k] = F(q, __ldg(amax + cpack * P + k));
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * rows_per_band;
  const int64_t r1 = min(outer, r0 + rows_per_band);
  const int64_t rstride = axis / P;
  const uint4* xv = reinterpret_cast<const uint4*>(x) + cpack;
  uint4* yv = reinterpret_cast<uint4*>(y) + cpack;
  for (int64_t r = r0; r < r1; r += 2) {
    const bool two = r + 1 < r1;
    uint4 v0 = ld_stream(xv + r * rstride);
    uint4 v1 = two ? ld_stream(xv + (r + 1) * rstride) : v0;
    float t[P];
    E::unpack(v0, t);
#pragma unroll
    for (int k = 0; k < P; ++k) t[k] = f[k](t[k]);
    st_stream(yv + r * rstride, E::pack(t));
    if (two) {
      E::unpack(v1, t);
#pragma unroll
      for (int k = 0; k < P; ++k) t[k] = f[k](t[k]);
      st_stream(yv + (r + 1) * rstride, E::pack(t));
    }
  }
}

// ---- scalar fallback for any [outer, axis, inner] ----------------------------------------------
template <typename T, typename F>
__global__ void fq_axis_generic_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t n,
                                       int64_t axis, int64_t inner,
                                       const float* __restrict__ amax, IntQ q) {
  pdl_prologue();
  using E = Elem<T>;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const F f(q, __ldg(amax + (i / inner) % axis));
    y[i] = E::from_float(f(E::to_float(x[i])));
  }
}

// ---- dynamic per-row quantisation: amax and quantise in one pass ------------------------------
// `G` adjacent lanes (power of two <= 32) hold one row in registers, PPL packs per lane.
template <typename T, int PPL>
__global__ void __launch_bounds__(kEwThreads)
fq_rows_warp_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int np, int G,
                    float* __restrict__ amax_out, IntQ q) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  const int lane_in_group = threadIdx.x & (G - 1);
  const int groups_per_cta = blockDim.x / G;
  const int group_in_cta = threadIdx.x / G;
  const int64_t row_stride = static_cast<int64_t>(gridDim.x) * groups_per_cta;
  // all lanes of a warp run the same number of trips: the bound is tested on the warp's first row
  const int groups_per_warp = 32 / G;
  const int64_t warp_first = static_cast<int64_t>(blockIdx.x) * groups_per_cta +
                             (threadIdx.x >> 5) * groups_per_warp;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  uint4* yv = reinterpret_cast<uint4*>(y);
  for (int64_t base = warp_first; base < rows; base += row_stride) {
    const int64_t row = base + (group_in_cta % groups_per_warp);
    const bool valid = row < rows;
    uint4 v[PPL];
    uint32_t acc = 0;
#pragma unroll
    for (int k = 0; k < PPL; ++k) {
      const int p = lane_in_group + G * k;
      v[k] = (valid && p < np) ? ld_stream(xv + row * np + p) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < PPL; ++k) acc = E::acc_max(acc, v[k]);
    uint32_t bits = E::acc_to_f32bits(acc);
    for (int o = G >> 1; o > 0; o >>= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
    const float amax = __uint_as_float(bits);
    const IntFq f(q, amax);
    if (valid && lane_in_group == 0 && amax_out) amax_out[row] = amax;
#pragma unroll
    for (int k = 0; k < PPL; ++k) {
      const int p = lane_in_group + G * k;
      if (valid && p < np) {
        float t[P];
        E::unpack(v[k], t);
        f.apply<P>(t);
        st_stream(yv + row * np + p, E::pack(t));
      }
    }
  }
}

// One CTA holds one row in registers (rows of up to blockDim.x * PPL packs).
template <typename T, int PPL>
__global__ void __launch_bounds__(1024)
fq_rows_cta_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int np,
                   float* __restrict__ amax_out, IntQ q) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  __shared__ uint32_t red[32];
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  uint4* yv = reinterpret_cast<uint4*>(y);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    uint4 v[PPL];
    uint32_t acc = 0;
#pragma unroll
    for (int k = 0; k < PPL; ++k) {
      const int p = threadIdx.x + blockDim.x * k;
      v[k] = (p < np) ? ld_stream(xv + row * np + p) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < PPL; ++k) acc = E::acc_max(acc, v[k]);
    const uint32_t bits = cta_max_u32(E::acc_to_f32bits(acc), red);
    const float amax = __uint_as_float(bits);
    const IntFq f(q, amax);
    if (threadIdx.x == 0 && amax_out) amax_out[row] = amax;
#pragma unroll
    for (int k = 0; k < PPL; ++k) {
      const int p = threadIdx.x + blockDim.x * k;
      if (p < np) {
        float t[P];
        E::unpack(v[k], t);
        f.apply<P>(t);
        st_stream(yv + row * np + p, E::pack(t));
      }
    }
  }
}

// ---- launch helpers ------------------------------------------------------------------------------
template <typename F>
static int launch_fq_tensor(const void* x, void* y, int64_t n, int dtype, const float* amax, IntQ q,
                            cudaStream_t s) {
  return B200Q_DISPATCH(dtype, [&] {
    int grid = grid_for(n / Elem<T>::kPerPack, kEwThreads * kEwUnroll, 8);
    launch_pdl(fq_tensor_kernel<T, F>, grid, kEwThreads, 0, s, static_cast<const T*>(x), static_cast<T*>(y), n,
               amax, q);
    return launch_status();
  });
}

template <typename F>
static int launch_fq_axis(const void* x, void* y, int64_t outer, int64_t axis, int64_t inner,
                          int dtype, const float* amax, IntQ q, cudaStream_t s) {
  return B200Q_DISPATCH(dtype, [&] {
    constexpr int P = Elem<T>::kPerPack;
    const T* xp = static_cast<const T*>(x);
    T* yp = static_cast<T*>(y);
    const int64_t n = outer * axis * inner;
    if (inner % P == 0 && n / P <= kFastDivLimit) {
      const int64_t npack = n / P;
      int grid = grid_for(npack, kEwThreads * kEwUnroll, 8);
      launch_pdl(fq_axis_inner_kernel<T, F>, grid, kEwThreads, 0, s, xp, yp, npack, FastDiv(static_cast<uint32_t>(axis)), FastDiv(static_cast<uint32_t>(inner / P)), amax, q);
    } else if (inner == 1 && axis % P == 0) {
      const int64_t cpacks = axis / P;
      const int bx = static_cast<int>((cpacks + kEwThreads - 1) / kEwThreads);
      int64_t want = (static_cast<int64_t>(sm_count_cached()) * 8 + bx - 1) / bx;
      int64_t bands = outer / 8 > 0 ? (outer / 8 < want ? outer / 8 : want) : 1;
      if (bands > 65535) bands = 65535;
      const int rpb = static_cast<int>((outer + bands - 1) / bands);
      dim3 grid(bx, static_cast<unsigned>((outer + rpb - 1) / rpb));
      launch_pdl(fq_axis_cols_kernel<T, F>, grid, kEwThreads, 0, s, xp, yp, outer, axis, rpb, amax, q);
    } else {
      int grid = grid_for(n, 256, 8);
      launch_pdl(fq_axis_generic_kernel<T, F>, grid, 256, 0, s, xp, yp, n, axis, inner, amax, q);
    }
    return launch_status();
  });
}

}  // namespace b200q

using namespace b200q;

static int check_bits(int num_bits, int is_unsigned) {
  if (num_bits < 1 || num_bits + (is_unsigned ? 1 : 0) > 24) return B200Q_ERR_ARG;
  return B200Q_OK;
}

extern "C" int b200q_fake_int_tensor(const void* x, void* y, int64_t n, int dtype, const float* amax,
                                     int num_bits, int is_unsigned, int narrow_range, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(y); B200Q_REQUIRE_PTR(amax);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x); B200Q_REQUIRE_ALIGNED(y);
  if (n <= 0) return B200Q_ERR_SHAPE;
  if (int e = check_bits(num_bits, is_unsigned)) return e;
  return launch_fq_tensor<IntFq>(x, y, n, dtype, amax, make_intq(num_bits, is_unsigned, narrow_range),
                                 static_cast<cudaStream_t>(stream));
}

extern "C" int b200q_fake_int_axis(const void* x, void* y, int64_t outer, int64_t axis, int64_t inner,
                                   int dtype, const float* amax, int num_bits, int is_unsigned,
                                   int narrow_range, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(y); B200Q_REQUIRE_PTR(amax);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x); B200Q_REQUIRE_ALIGNED(y);
  if (outer <= 0 || axis <= 0 || inner <= 0) return B200Q_ERR_SHAPE;
  if (int e = check_bits(num_bits, is_unsigned)) return e;
  return launch_fq_axis<IntFq>(x, y, outer, axis, inner, dtype, amax,
                               make_intq(num_bits, is_unsigned, narrow_range),
                               static_cast<cudaStream_t>(stream));
}

extern "C" int b200q_fake_int_rows_dynamic(const void* x, void* y, int64_t rows, int64_t cols,
                                           int dtype, float* amax_out, int num_bits,
                                           int is_unsigned, int narrow_range, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(y);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x); B200Q_REQUIRE_ALIGNED(y);
  if (rows <= 0 || cols <= 0) return B200Q_ERR_SHAPE;
  if (int e = check_bits(num_bits, is_unsigned)) return e;
  const IntQ q = make_intq(num_bits, is_unsigned, narrow_range);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return B200Q_DISPATCH(dtype, [&]() -> int {
    constexpr int P = Elem<T>::kPerPack;
    if (cols % P != 0) return B200Q_ERR_UNSUPPORTED;
    const int64_t np64 = cols / P;
    if (np64 > 8192) return B200Q_ERR_UNSUPPORTED;
    const int np = static_cast<int>(np64);
    const T* xp = static_cast<const T*>(x);
    T* yp = static_cast<T*>(y);
    if (np <= 128) {
      // up to 4 packs per lane; lanes per row: next power of two of ceil(np/4)
      int G = 1;
      while (G < 32 && G * 4 < np) G <<= 1;
      const int ppl = (np + G - 1) / G;
      const int64_t groups = rows;
      int grid = grid_for(groups * G, kEwThreads, 8);
      if (ppl <= 1) launch_pdl(fq_rows_warp_kernel<T, 1>, grid, kEwThreads, 0, s, xp, yp, rows, np, G, amax_out, q);
      else if (ppl <= 2) launch_pdl(fq_rows_warp_kernel<T, 2>, grid, kEwThreads, 0, s, xp, yp, rows, np, G, amax_out, q);
      else launch_pdl(fq_rows_warp_kernel<T, 4>, grid, kEwThreads, 0, s, xp, yp, rows, np, G, amax_out, q);
    } else {
      int threads = 256;
      while (threads < 1024 && threads * 4 < np) threads <<= 1;
      const int ppl = (np + threads - 1) / threads;
      int grid = grid_for(rows, 1, 2048 / threads);
      if (ppl <= 1) launch_pdl(fq_rows_cta_kernel<T, 1>, grid, threads, 0, s, xp, yp, rows, np, amax_out, q);
      else if (ppl <= 2) launch_pdl(fq_rows_cta_kernel<T, 2>, grid, threads, 0, s, xp, yp, rows, np, amax_out, q);
      else if (ppl <= 4) launch_pdl(fq_rows_cta_kernel<T, 4>, grid, threads, 0, s, xp, yp, rows, np, amax_out, q);
      else launch_pdl(fq_rows_cta_kernel<T, 8>, grid, threads, 0, s, xp, yp, rows, np, amax_out, q);
    }
    return launch_status();
  });
}

extern "C" int b200q_fake_e4m3_tensor(const void* x, void* y, int64_t n, int dtype, const float* amax,
                                      void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(y);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x); B200Q_REQUIRE_ALIGNED(y);
  if (n <= 0) return B200Q_ERR_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (amax) return launch_fq_tensor<E4m3Fq>(x, y, n, dtype, amax, IntQ{0.f, 0.f}, s);
  return B200Q_DISPATCH(dtype, [&] {
    int grid = grid_for(n / Elem<T>::kPerPack, kEwThreads, 8);
    launch_pdl(e4m3_cast_kernel<T>, grid, kEwThreads, 0, s, static_cast<const T*>(x), static_cast<T*>(y), n);
    return launch_status();
  });
}

extern "C" int b200q_fake_e4m3_axis(const void* x, void* y, int64_t outer, int64_t axis, int64_t inner,
                                    int dtype, const float* amax, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(y); B200Q_REQUIRE_PTR(amax);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x); B200Q_REQUIRE_ALIGNED(y);
  if (outer <= 0 || axis <= 0 || inner <= 0) return B200Q_ERR_SHAPE;
  return launch_fq_axis<E4m3Fq>(x, y, outer, axis, inner, dtype, amax, IntQ{0.f, 0.f},
                                static_cast<cudaStream_t>(stream));
}
