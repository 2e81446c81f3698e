// MSE calibration: the squared fake-quantisation error of a tensor under EVERY candidate amax in one
// pass.  The reference's MseCalibrator.collect runs, per candidate, a fake-quant pass, an elementwise
// squared error and a reduction over the whole tensor (10 candidates = 10 reads and 10 writes of x plus
// temporaries); here x is read once, every element is fake-quantised under each candidate in registers
// and the errors are accumulated per candidate (and per channel).
//
//   loss[s, c] += sum over the elements of channel c of (x - fq(x, cand[s, c]))^2,   x taken as fp32
//
// (the reference converts x to fp32 before it calls the quantiser, so the fake-quantised value is the
// fp32 one, not rounded to the input's 16-bit type).  Partial sums are fp32 per thread, fp64 across
// threads.  With S candidates the kernel issues about 6 S instructions per element against 2-4 bytes
// read: it is bound by instruction issue, not by HBM, for any S >= 2.
#include "numerics.cuh"

namespace b200q {

constexpr int kMseMaxCand = 16;
constexpr int kMseThreads = 256;

enum { kMseInt = 0, kMseE4m3 = 1 };

struct MseCand {      // one candidate of one channel, prepared once
  float scale, y, inv;   // integer: inv holds 1 / scale - y;  E4M3: inv = 1 / scale
  int live_fast;      // bit 0: amax >= 2^-24, bit 1: scale in the range of the reciprocal division, bit 2: see mse_prepare
};

template <int FORMAT>
__device__ __forceinline__ MseCand mse_prepare(float amax, const IntQ& q) {
  MseCand c;
  if (FORMAT == kMseInt) {
    const IntScale s = make_int_scale(q, amax);
    c.scale = s.scale; c.y = s.y;
    c.inv = fmaf(-s.scale, s.y, 1.f) * s.y;      // 1 / scale - y
    // bit 2: the bounds fit the magic-number rounding
    c.live_fast = (s.live ? 1 : 0) | (s.fast ? 2 : 0) | (q.bound <= 4194303.f && q.lo >= -4194304.f ? 4 : 0);
  } else {
    c.scale = __fdiv_rn(448.f, amax);
    c.inv = __fdiv_rn(1.f, c.scale);
    c.y = 0.f; c.live_fast = 7;
  }
  return c;
}

// Squared errors of two elements under one candidate, added to the two lanes of acc.
// Integer fast path, 6 fp32-pipe operations per element:
//  * the clamp is applied before the rounding — the bounds are integers, so clamp(rint(t)) ==
//    rint(clamp(t)) — which bounds |t| by 2^22 and lets (t + 1.5 * 2^23) - 1.5 * 2^23 do the
//    round-half-even in two packed adds instead of two conversion-pipe instructions;
//  * the error x - r / scale is formed without the division: with y = RN(1 / scale) and
//    ey = (1 - scale * y) * y, r / scale = r * y + r * ey to 2^-45, so two FMAs give the error of the
//    exact quotient rounded once.  The stand-alone kernel rounds the quotient to fp32 first: the two
//    errors differ by at most half an ulp of the quotient, with no systematic sign — far inside the
//    noise of the fp32 summation the reference accumulates its losses with (the candidates' amax
//    parity tolerance is 1e-3; losses agree to about 1e-7).
// Everything else (dead amax, scales outside the safe range, E4M3) reproduces the stand-alone kernels'
// per-element results bit for bit.
template <int FORMAT>
__device__ __forceinline__ float2 mse_pair(float x0, float x1, const MseCand& c, const IntQ& q, float2 acc) {
  float q0, q1;
  if (FORMAT == kMseInt) {
    if (c.live_fast == 7) {
      const float2 x = make_float2(x0, x1);
      float2 r = __fmul2_rn(x, make_float2(c.scale, c.scale));
      r.x = fmax_nan(fmin_nan(r.x, q.bound), q.lo);
      r.y = fmax_nan(fmin_nan(r.y, q.bound), q.lo);
      r = __fadd2_rn(__fadd2_rn(r, make_float2(12582912.f, 12582912.f)), make_float2(-12582912.f, -12582912.f));
      float2 d = __ffma2_rn(r, make_float2(-c.y, -c.y), x);
      d = __ffma2_rn(r, make_float2(-c.inv, -c.inv), d);
      return __ffma2_rn(d, d, acc);
    }
    IntScale s;
    s.scale = c.scale; s.y = c.y; s.live = (c.live_fast & 1) != 0; s.fast = (c.live_fast & 2) != 0;
    q0 = intq_apply(x0, s, q); q1 = intq_apply(x1, s, q);
  } else {
    const float2 back = e4m3x2_to_f32x2(f32x2_to_e4m3x2_sat(__fmul_rn(x0, c.scale), __fmul_rn(x1, c.scale)));
    q0 = __fmul_rn(back.x, c.inv); q1 = __fmul_rn(back.y, c.inv);
  }
  const float d0 = __fsub_rn(x0, q0), d1 = __fsub_rn(x1, q1);
  acc.x = fmaf(d0, d0, acc.x);
  acc.y = fmaf(d1, d1, acc.y);
  return acc;
}

// Per tensor: all CTAs stride over the packs; S accumulators per thread; one fp64 atomic per CTA and candidate.
template <typename T, int FORMAT>
__global__ void __launch_bounds__(kMseThreads, 4)
mse_tensor_kernel(const T* __restrict__ x, int64_t n, const float* __restrict__ cand, int n_cand, IntQ q,
                  double* __restrict__ loss) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  __shared__ MseCand cs[kMseMaxCand];
  __shared__ float red[kMseMaxCand][kMseThreads / 32];
  if (threadIdx.x < n_cand) cs[threadIdx.x] = mse_prepare<FORMAT>(__ldg(cand + threadIdx.x), q);
  __syncthreads();
  float2 acc[kMseMaxCand];
#pragma unroll
  for (int s = 0; s < kMseMaxCand; ++s) acc[s] = make_float2(0.f, 0.f);
  const int64_t npack = n / P;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < npack; i += stride) {
    float f[P];
    E::unpack(ld_stream(xv + i), f);
#pragma unroll
    for (int s = 0; s < kMseMaxCand; ++s) {
      if (s < n_cand) {
        const MseCand c = cs[s];
#pragma unroll
        for (int k = 0; k < P; k += 2) acc[s] = mse_pair<FORMAT>(f[k], f[k + 1], c, q, acc[s]);
      }
    }
  }
  if (blockIdx.x == 0 && threadIdx.x < n - npack * P) {      // ragged tail, one element per thread
    const float v = E::to_float(x[npack * P + threadIdx.x]);
#pragma unroll
    for (int s = 0; s < kMseMaxCand; ++s)
      if (s < n_cand) acc[s].x += mse_pair<FORMAT>(v, v, cs[s], q, make_float2(0.f, 0.f)).x;
  }
#pragma unroll
  for (int s = 0; s < kMseMaxCand; ++s) {
    float v = acc[s].x + acc[s].y;
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) red[s][threadIdx.x >> 5] = v;
  }
  __syncthreads();
  if (threadIdx.x < n_cand) {
    double t = 0.0;
    for (int w = 0; w < kMseThreads / 32; ++w) t += static_cast<double>(red[threadIdx.x][w]);
    atomicAdd(loss + threadIdx.x, t);
  }
}

// Per channel, x viewed as [outer, channels, inner] with `inner` contiguous elements per (outer, channel)
// row: one warp per row; the row's S candidates are prepared by lanes 0..S-1 and passed by shuffle.
template <typename T, int FORMAT>
__global__ void __launch_bounds__(kMseThreads, 4)
mse_rows_kernel(const T* __restrict__ x, int64_t rows, int64_t channels, int64_t inner,
                const float* __restrict__ cand, int n_cand, IntQ q, double* __restrict__ loss) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t packs = inner / P;
  for (int64_t r = warp; r < rows; r += nwarps) {
    const int64_t ch = r % channels;
    MseCand mine = {};
    if (lane < n_cand) mine = mse_prepare<FORMAT>(__ldg(cand + lane * channels + ch), q);
    float2 acc[kMseMaxCand];
#pragma unroll
    for (int s = 0; s < kMseMaxCand; ++s) acc[s] = make_float2(0.f, 0.f);
    const uint4* xv = reinterpret_cast<const uint4*>(x + r * inner);
    for (int64_t i = lane; i < packs; i += 32) {
      float f[P];
      E::unpack(ld_stream(xv + i), f);
#pragma unroll
      for (int s = 0; s < kMseMaxCand; ++s) {
        if (s < n_cand) {
          MseCand c;      // loop-invariant: the compiler keeps the row's candidates in registers
          c.scale = __shfl_sync(0xffffffffu, mine.scale, s);
          c.y = __shfl_sync(0xffffffffu, mine.y, s);
          c.inv = __shfl_sync(0xffffffffu, mine.inv, s);
          c.live_fast = __shfl_sync(0xffffffffu, mine.live_fast, s);
#pragma unroll
          for (int k = 0; k < P; k += 2) acc[s] = mse_pair<FORMAT>(f[k], f[k + 1], c, q, acc[s]);
        }
      }
    }
#pragma unroll
    for (int s = 0; s < kMseMaxCand; ++s) {
      if (s < n_cand) {
        float v = acc[s].x + acc[s].y;
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) atomicAdd(loss + s * channels + ch, static_cast<double>(v));
      }
    }
  }
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_mse_candidates(const void* x, int64_t outer, int64_t channels, int64_t inner, int dtype,
                                    const float* cand_amax, int n_cand, int format, int num_bits, int is_unsigned,
                                    int narrow_range, double* loss_io, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(cand_amax); B200Q_REQUIRE_PTR(loss_io);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x);
  if (outer <= 0 || channels <= 0 || inner <= 0) return B200Q_ERR_SHAPE;
  if (n_cand < 1 || n_cand > kMseMaxCand) return B200Q_ERR_ARG;
  if (format != kMseInt && format != kMseE4m3) return B200Q_ERR_ARG;
  if (format == kMseInt && (num_bits < 1 || num_bits + (is_unsigned ? 1 : 0) > 24)) return B200Q_ERR_ARG;
  const IntQ q = format == kMseInt ? make_intq(num_bits, is_unsigned, narrow_range) : IntQ{448.f, -448.f};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return B200Q_DISPATCH(dtype, [&]() -> int {
    constexpr int P = Elem<T>::kPerPack;
    const T* xp = static_cast<const T*>(x);
    if (channels == 1) {
      const int64_t n = outer * inner;
      const int grid = grid_for(n / P, kMseThreads, 4);      // 64 registers: four CTAs per SM are resident
      if (format == kMseInt) launch_pdl(mse_tensor_kernel<T, kMseInt>, grid, kMseThreads, 0, st, xp, n, cand_amax, n_cand, q, loss_io);
      else launch_pdl(mse_tensor_kernel<T, kMseE4m3>, grid, kMseThreads, 0, st, xp, n, cand_amax, n_cand, q, loss_io);
      return launch_status();
    }
    // rows of `inner` contiguous elements: whole 16-byte packs, each row aligned
    if (inner % P || inner < 32 * P) return B200Q_ERR_UNSUPPORTED;
    const int64_t rows = outer * channels;
    const int grid = grid_for(rows * 32, kMseThreads, 4);
    if (format == kMseInt) launch_pdl(mse_rows_kernel<T, kMseInt>, grid, kMseThreads, 0, st, xp, rows, channels, inner, cand_amax, n_cand, q, loss_io);
    else launch_pdl(mse_rows_kernel<T, kMseE4m3>, grid, kMseThreads, 0, st, xp, rows, channels, inner, cand_amax, n_cand, q, loss_io);
    return launch_status();
  });
}
