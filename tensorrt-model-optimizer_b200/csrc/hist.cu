// Histogram calibration: fixed-range, equal-width binning of |x| with 64-bit global counters,
// and the percentile read-out.
//
// Each CTA bins into shared-memory 32-bit counters (several replicas chosen by lane, so that the
// lanes of a warp that hit the same hot bin do not serialise on one address), then adds its
// non-zero bins to the global 64-bit counters once.  Bins beyond the shared range go to global
// atomics directly.  Integer sums make the result independent of the order of batches and ranks.
#include "numerics.cuh"

namespace b200q {

constexpr int kHistThreads = 1024;
constexpr int kHistSmemBytes = 200 * 1024;   // shared-memory budget for the replicated counters

// Shared counters are replicated `replicas` times (a power of two <= 32) and a lane always uses
// replica (lane % replicas).  Replica r starts at word r * (smem_bins + 1): the odd stride puts the
// same bin of different replicas into different banks, so lanes of a warp that hit one hot bin —
// the normal case for activations, whose range is set by a few outliers — neither collide on an
// address nor on a bank.
// kAllShared: every bin has a shared counter (the usual case), so no global-atomic path is compiled.
template <typename T, bool kAllShared>
__global__ void __launch_bounds__(kHistThreads)
hist_collect_kernel(const T* __restrict__ x, int64_t n, int nbins, float range_max, int smem_bins,
                    int replicas, unsigned long long* __restrict__ counts) {
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  extern __shared__ uint32_t sh[];
  const int stride_r = smem_bins + 1;
  for (int i = threadIdx.x; i < stride_r * replicas; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  uint32_t* mine = sh + (threadIdx.x & (replicas - 1)) * stride_r;
  const float fbins = static_cast<float>(nbins);
  // bin = int(RN(|x| * nbins / range_max)): the quotient through one reciprocal per thread; tiny
  // quotients may lose bits there but stay below 1 (bin 0)
  const bool fast = div_safe(range_max);
  const float rcp_range = __frcp_rn(range_max);
  const float2 y2 = make_float2(rcp_range, rcp_range), nd2 = make_float2(-range_max, -range_max);
  const uint32_t last = static_cast<uint32_t>(nbins - 1);

  // a = |x| (non-negative); quot = RN(a * nbins / range_max) < 2^22: its integer part is read from
  // the low mantissa bits after a round-toward-zero add of 2^23 (no float->int conversion)
  auto count = [&](float a, float quot) {
    uint32_t b = __float_as_uint(__fadd_rz(quot, 8388608.f)) & 0x7fffffu;
    b = min(b, last);
    if (a <= range_max) {  // false for out-of-range values and NaN: not counted
      if (kAllShared || b < static_cast<uint32_t>(smem_bins)) atomicAdd(mine + b, 1u);
      else atomicAdd(counts + b, 1ull);
    }
  };
  auto bin_pair = [&](float a0, float a1) {
    const float2 num = __fmul2_rn(make_float2(a0, a1), make_float2(fbins, fbins));
    float2 q;
    if (fast) q = div2_rn_rcp(num, nd2, y2);
    else q = make_float2(__fdiv_rn(num.x, range_max), __fdiv_rn(num.y, range_max));
    count(a0, q.x);
    count(a1, q.y);
  };
  auto bin_pack = [&](uint4 v) {
    if (sizeof(T) == 2) {  // clear both sign bits of a 16-bit pair with one instruction
      v.x &= 0x7fff7fffu; v.y &= 0x7fff7fffu; v.z &= 0x7fff7fffu; v.w &= 0x7fff7fffu;
    } else {
      v.x &= 0x7fffffffu; v.y &= 0x7fffffffu; v.z &= 0x7fffffffu; v.w &= 0x7fffffffu;
    }
    float f[P];
    E::unpack(v, f);
#pragma unroll
    for (int k = 0; k < P; k += 2) bin_pair(f[k], f[k + 1]);
  };

  const int64_t npack = n / P;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < npack; i += 4 * stride) {
    const uint4 v0 = ld_stream(xv + i), v1 = ld_stream(xv + i + stride), v2 = ld_stream(xv + i + 2 * stride),
                v3 = ld_stream(xv + i + 3 * stride);
    bin_pack(v0); bin_pack(v1); bin_pack(v2); bin_pack(v3);
  }
  for (; i < npack; i += stride) bin_pack(ld_stream(xv + i));
  if (blockIdx.x == 0 && threadIdx.x < n - npack * P) {
    const float a = fabsf(E::to_float(x[npack * P + threadIdx.x]));
    count(a, __fdiv_rn(a * fbins, range_max));
  }
  __syncthreads();
  for (int b = threadIdx.x; b < smem_bins; b += blockDim.x) {
    unsigned long long c = 0;
    for (int r = 0; r < replicas; ++r) c += sh[r * stride_r + b];
    if (c) atomicAdd(counts + b, c);
  }
}

// One thread walks the bins in order so that the running sum rounds exactly as a sequential
// float64 cumulative sum does.
__global__ void hist_percentile_kernel(const unsigned long long* __restrict__ counts, int nbins,
                                       const float* __restrict__ edges, float bin_width,
                                       double frac, float* __restrict__ amax_out) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  unsigned long long total = 0;
  for (int i = 0; i < nbins; ++i) total += counts[i];
  const double dt = static_cast<double>(total);
  double cdf = 0.0;
  int idx = nbins;
  for (int i = 0; i < nbins; ++i) {
    cdf += static_cast<double>(counts[i]) / dt;
    if (cdf >= frac) { idx = i; break; }
  }
  *amax_out = edges ? edges[idx] : bin_width * static_cast<float>(idx);
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_hist_collect(const void* x, int64_t n, int dtype, int nbins, float range_max,
                                  unsigned long long* counts, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(counts);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x);
  if (n <= 0 || nbins <= 0) return B200Q_ERR_SHAPE;
  if (!(range_max > 0.f)) return B200Q_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // shared bins: all of them when they fit, replicated as often as the budget allows (<= 32)
  const int max_words = kHistSmemBytes / 4;
  int smem_bins = nbins + 1 <= max_words ? nbins : max_words - 1;
  int replicas = 1;
  while (replicas < 32 && static_cast<int64_t>(smem_bins + 1) * replicas * 2 <= max_words) replicas <<= 1;
  const size_t smem = static_cast<size_t>(smem_bins + 1) * replicas * sizeof(uint32_t);
  return B200Q_DISPATCH(dtype, [&] {
    auto kern = smem_bins == nbins ? hist_collect_kernel<T, true> : hist_collect_kernel<T, false>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kHistSmemBytes) != cudaSuccess)
      return static_cast<int>(B200Q_ERR_CUDA);
    int grid = grid_for(n / Elem<T>::kPerPack, kHistThreads * 4, 1);
    kern<<<grid, kHistThreads, smem, s>>>(static_cast<const T*>(x), n, nbins, range_max, smem_bins,
                                          replicas, counts);
    return launch_status();
  });
}

extern "C" int b200q_hist_percentile(const unsigned long long* counts, int nbins, const float* edges,
                                     float bin_width, double percentile, float* amax_out,
                                     void* stream) {
  B200Q_REQUIRE_PTR(counts); B200Q_REQUIRE_PTR(amax_out);
  if (nbins <= 0) return B200Q_ERR_SHAPE;
  if (!(percentile >= 0.0 && percentile <= 100.0)) return B200Q_ERR_ARG;
  hist_percentile_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      counts, nbins, edges, bin_width, percentile / 100.0, amax_out);
  return launch_status();
}
