// Histogram calibration: fixed-range, equal-width binning of |x| with 64-bit global counters,
// and the percentile read-out.
//
// 16-bit inputs (the activations that calibration sees) have at most 32768 distinct magnitudes, so
// a CTA first counts VALUES: the 15 magnitude bits of an element are the index of a shared 32-bit
// counter (two bit operations and one shared reduction per element, no float arithmetic).  When
// its share of the input is done it maps the values that occurred to bins with the exact reference
// arithmetic (a few thousand divisions per CTA), adds them into shared bin counters and adds the
// non-zero bins to the global 64-bit counters once.
//
// fp32 inputs bin directly: each CTA bins into shared-memory 32-bit counters (several replicas
// chosen by lane, so that the lanes of a warp that hit the same hot bin do not serialise on one
// address), then adds its non-zero bins to the global counters.  Bins beyond the shared range go
// to global atomics directly.  Integer sums make the result independent of the order of batches
// and ranks.
#include <cstring>

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
//
// Open-ended collection: bins continue past nbins - 1 at the same width up to `capacity` bins
// (range `cap_range`); what lies beyond that, NaN and inf are not binned but counted in
// `*overflow` when that is given.  capacity == nbins is the closed histogram of torch.histc.
struct HistOpen {
  int capacity;
  float cap_range;
  unsigned long long* overflow;
};

// Where a launch adds its counts: up to kHistMaxDests histograms (calibrators that were handed the
// very same tensor share one binning pass), each with its own out-of-range counter.
constexpr int kHistMaxDests = 4;
struct HistDests {
  unsigned long long* counts[kHistMaxDests];
  unsigned long long* overflow[kHistMaxDests];
  int n;
};
__device__ __forceinline__ void hist_add(const HistDests& d, uint32_t bin, unsigned long long c) {
#pragma unroll
  for (int i = 0; i < kHistMaxDests; ++i)
    if (i < d.n) atomicAdd(d.counts[i] + bin, c);
}
__device__ __forceinline__ void hist_overflow(const HistDests& d, unsigned long long c) {
#pragma unroll
  for (int i = 0; i < kHistMaxDests; ++i)
    if (i < d.n && d.overflow[i] != nullptr) atomicAdd(d.overflow[i], c);
}

template <typename T, bool kAllShared>
__global__ void __launch_bounds__(kHistThreads)
hist_collect_kernel(const T* __restrict__ x, int64_t n, int nbins, float range_max, HistOpen open,
                    int smem_bins, int replicas, HistDests dests, const float* __restrict__ range_dev) {
  pdl_prologue();
  if (range_dev != nullptr) {   // the range lives on the device (no host round trip before the first batch)
    range_max = *range_dev;
    open.cap_range = open.capacity == nbins ? range_max
                                            : static_cast<float>(static_cast<double>(range_max) * open.capacity / nbins);
    if (!(range_max > 0.f) || !(open.cap_range < 3.0e38f)) open.cap_range = -1.f;   // nothing can be binned
  }
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
  const uint32_t cap_last = static_cast<uint32_t>(open.capacity - 1);
  uint32_t beyond = 0;
  auto count = [&](float a, float quot) {
    uint32_t b = __float_as_uint(__fadd_rz(quot, 8388608.f)) & 0x7fffffu;
    if (a <= open.cap_range) {  // false for values beyond the last bin and for NaN
      b = min(b, a <= range_max ? last : cap_last);
      if (kAllShared || b < static_cast<uint32_t>(smem_bins)) atomicAdd(mine + b, 1u);
      else hist_add(dests, b, 1ull);
    } else {
      ++beyond;
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
    if (c) hist_add(dests, b, c);
  }
  beyond = __reduce_add_sync(0xffffffffu, beyond);
  if (beyond != 0 && (threadIdx.x & 31) == 0) hist_overflow(dests, static_cast<unsigned long long>(beyond));
}

// ---- 16-bit inputs: value counting -------------------------------------------------------------
// Non-negative 16-bit floats order like their bit patterns.  With `hi` the largest pattern whose
// value is <= range_max and `lo` a pattern whose value is <= range_max / (2 nbins) (everything at
// or below it lands in bin 0), an element's counter index is clamp(pattern, lo, hi + 1) - lo:
// index 0 collects all the tiny values, the last index everything beyond the range (NaN and inf
// included), which is dropped.  That leaves about 128 * (log2(nbins) + 1) counters for bf16,
// few enough for `1 << rshift` replicas chosen by lane: with 16 replicas the word of a counter is
// index * 16 + lane % 16, so two lanes of a warp meet in a bank only when they are 16 apart and
// their values have the same parity.
constexpr int kHist16SmemWords = 227 * 1024 / 4;   // the whole shared memory of an SM
constexpr int kHist16MaxSmemBins = 8192;

struct Hist16Layout {
  uint32_t lo, hi1;   // patterns: lower clamp, upper clamp (= hi + 1)
  int values;         // counters per replica: hi1 - lo + 1, padded to a multiple of 4
  int rshift;         // log2(replicas)
  int smem_bins;      // bins with a shared counter
};

// largest 16-bit pattern of type T whose value is <= v (v >= 0), capped at the largest finite
template <typename T> __host__ __device__ inline uint32_t floor_bits16(float v);
template <> __host__ __device__ inline uint32_t floor_bits16<__nv_bfloat16>(float v) {
  uint32_t u;
#ifdef __CUDA_ARCH__
  u = __float_as_uint(v);
#else
  memcpy(&u, &v, 4);
#endif
  u >>= 16;   // truncation rounds a non-negative value down
  return u > 0x7f7fu ? 0x7f7fu : u;
}
template <> __host__ __device__ inline uint32_t floor_bits16<__half>(float v) {
  if (!(v < 65504.f)) return 0x7bffu;
  const __half h = __float2half_rd(v);
  unsigned short r;
#ifdef __CUDA_ARCH__
  r = __half_as_ushort(h);
#else
  memcpy(&r, &h, 2);
#endif
  return r;
}
// counter layout of the value-counting kernel for one range (host: at launch; device: when the range is
// only known there)
template <typename T>
__host__ __device__ inline Hist16Layout hist16_layout(float range_max, float cap_range, int nbins, int smem_bins) {
  Hist16Layout lay;
  lay.hi1 = floor_bits16<T>(cap_range) + 1;
  lay.lo = floor_bits16<T>(range_max / (2.f * static_cast<float>(nbins)));
  if (lay.lo >= lay.hi1) lay.lo = lay.hi1 - 1;
  lay.values = static_cast<int>(lay.hi1 - lay.lo + 1);
  lay.values = (lay.values + 3) & ~3;   // padding counters are never addressed
  lay.smem_bins = smem_bins;
  lay.rshift = 4;   // 16 replicas; measured on 33.5 M-element batches: 8 replicas 17.5 us per launch, 16: 14.0, 32: 17.4
  while (lay.rshift > 0 && (static_cast<int64_t>(lay.values) << lay.rshift) + lay.smem_bins + 3 > kHist16SmemWords)
    --lay.rshift;
  return lay;
}

__device__ __forceinline__ void red_shared_inc(uint32_t addr) {
  asm volatile("red.shared.add.u32 [%0], %1;" ::"r"(addr), "r"(1u) : "memory");
}
template <typename T> __device__ __forceinline__ float value_of_bits16(uint32_t idx);
template <> __device__ __forceinline__ float value_of_bits16<__nv_bfloat16>(uint32_t idx) {
  return __uint_as_float(idx << 16);
}
template <> __device__ __forceinline__ float value_of_bits16<__half>(uint32_t idx) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(idx)));
}

// sh = [values << rshift value counters][smem_bins bin counters]
template <typename T>
__global__ void __launch_bounds__(kHistThreads)
hist16_collect_kernel(const T* __restrict__ x, int64_t n, int nbins, float range_max, HistOpen open,
                      Hist16Layout lay, HistDests dests, const float* __restrict__ range_dev) {
  static_assert(sizeof(T) == 2, "16-bit element types only");
  pdl_launch_dependents();
  extern __shared__ uint32_t sh[];
  uint4* sh4 = reinterpret_cast<uint4*>(sh);
  if (range_dev != nullptr) {
    // The range lives on the device (written by the abs-max kernel of the first batch, or received from
    // another rank): the counter layout the host would have derived from it is derived here.  The
    // predecessor wrote it, so its read waits like every other global access.
    pdl_wait();
    range_max = *range_dev;
    open.cap_range = open.capacity == nbins ? range_max
                                            : static_cast<float>(static_cast<double>(range_max) * open.capacity / nbins);
    const bool valid = range_max > 0.f && open.cap_range < 3.0e38f;
    if (!valid) { range_max = 1.f; open.cap_range = 0.f; }   // every element lands in the out-of-range counter
    lay = hist16_layout<T>(range_max, open.cap_range, nbins, lay.smem_bins);
  }
  const int vwords = lay.values << lay.rshift;             // a multiple of 4 (host pads `values`)
  // clearing the (CTA-private) counters overlaps the previous kernel's tail; global memory is
  // touched only after pdl_wait()
  for (int j = threadIdx.x; j < (vwords + lay.smem_bins + 3) / 4; j += blockDim.x) sh4[j] = make_uint4(0, 0, 0, 0);
  pdl_wait();

  // Four packs per step, loaded one step ahead.
  const int64_t npack = n / 8;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  auto load4 = [&](int64_t at, uint4* v) {
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (at + k * stride < npack) v[k] = ld_stream(xv + at + k * stride);
  };
  uint4 cur[4], nxt[4];
  load4(i, cur);
  // value -> bin with the reference arithmetic: bin = int(RN(RN(a * nbins) / range)), the right edge in
  // the last bin; kSkip for a value beyond the capacity (cannot happen by construction of hi1: a guard).
  // The bins of the first two values that this thread folds after the stream are computed here, while the
  // first loads are in flight, so that the divisions are off the tail that nothing overlaps.
  constexpr uint32_t kSkip = 0xffffffffu;
  const float fbins = static_cast<float>(nbins);
  const uint32_t last = static_cast<uint32_t>(nbins - 1), cap_last = static_cast<uint32_t>(open.capacity - 1);
  const int in_range = static_cast<int>(lay.hi1 - lay.lo);   // index hi1 - lo holds what is out of range
  auto bin_of = [&](int v) -> uint32_t {
    const float a = value_of_bits16<T>(lay.lo + v);
    if (!(a <= open.cap_range)) return kSkip;
    const float quot = __fdiv_rn(a * fbins, range_max);
    const uint32_t b = quot < 8388608.f ? (__float_as_uint(__fadd_rz(quot, 8388608.f)) & 0x7fffffu) : cap_last;
    return min(b, a <= range_max ? last : cap_last);
  };
  const uint32_t bin0 = bin_of(min(static_cast<int>(threadIdx.x), in_range - 1));
  const uint32_t bin1 = bin_of(min(static_cast<int>(threadIdx.x + blockDim.x), in_range - 1));
  __syncthreads();
  const uint32_t rmask = (1u << lay.rshift) - 1u;
  const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(sh));
  // byte address of counter (index, my replica) = index * (4 << rshift) + cbase
  const uint32_t bytes_per_value = 4u << lay.rshift;
  const uint32_t cbase = base + ((threadIdx.x & rmask) << 2) - lay.lo * bytes_per_value;
  const uint32_t lo2 = lay.lo | (lay.lo << 16), hi2 = lay.hi1 | (lay.hi1 << 16);

  auto count_word = [&](uint32_t w) {  // two elements
    const uint32_t t = __vmaxu2(__vminu2(w & 0x7fff7fffu, hi2), lo2);
    red_shared_inc((t & 0xffffu) * bytes_per_value + cbase);
    red_shared_inc((t >> 16) * bytes_per_value + cbase);
  };
  auto count_pack = [&](const uint4& v) { count_word(v.x); count_word(v.y); count_word(v.z); count_word(v.w); };

  for (; i < npack; i += 4 * stride) {
    load4(i + 4 * stride, nxt);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (i + k * stride < npack) count_pack(cur[k]);
#pragma unroll
    for (int k = 0; k < 4; ++k) cur[k] = nxt[k];
  }
  if (blockIdx.x == 0 && threadIdx.x < n - npack * 8) {
    const uint32_t w = reinterpret_cast<const unsigned short*>(x)[npack * 8 + threadIdx.x] & 0x7fffu;
    red_shared_inc(max(min(w, lay.hi1), lay.lo) * bytes_per_value + cbase);
  }
  __syncthreads();

  // values -> bins.  Thread v sums the replicas of value v.
  uint32_t* bins = sh + vwords;
  auto replica_sum = [&](int v) -> uint32_t {
    const uint32_t* row = sh + (v << lay.rshift);
    // This phase reads every replica of every value once (about 100 KB): it runs at the speed of shared
    // memory, so the reads are laid out free of bank conflicts.  A row of 2^rshift words starts at bank
    // (lane << rshift) % 32; lanes whose rows start in the same bank begin at different replicas.
    if (lay.rshift == 4) {        // sixteen replicas: four 16-byte reads, rotated by lane / 2
      const uint4* row4 = reinterpret_cast<const uint4*>(row);
      const uint32_t rot = (threadIdx.x >> 1) & 3u;
      const uint4 p0 = row4[rot], p1 = row4[(rot + 1) & 3u], p2 = row4[(rot + 2) & 3u], p3 = row4[(rot + 3) & 3u];
      return (p0.x + p0.y + p0.z + p0.w) + (p1.x + p1.y + p1.z + p1.w) + (p2.x + p2.y + p2.z + p2.w) +
             (p3.x + p3.y + p3.z + p3.w);
    }
    uint32_t c = 0;
    const uint32_t rot = (threadIdx.x & 31u) >> (5 - lay.rshift);
    for (uint32_t k = 0; k <= rmask; ++k) c += row[(k + rot) & rmask];
    return c;
  };
  auto add_to_bin = [&](uint32_t b, uint32_t c) {
    if (c == 0 || b == kSkip) return;
    if (b < static_cast<uint32_t>(lay.smem_bins)) atomicAdd(bins + b, c);
    else hist_add(dests, b, static_cast<unsigned long long>(c));
  };
  int v = threadIdx.x;
  if (v < in_range) add_to_bin(bin0, replica_sum(v));
  v += blockDim.x;
  if (v < in_range) add_to_bin(bin1, replica_sum(v));
  v += blockDim.x;
  for (; v < in_range; v += blockDim.x) {
    const uint32_t c = replica_sum(v);
    if (c) add_to_bin(bin_of(v), c);
  }
  if (threadIdx.x <= rmask) {   // the index that holds what is out of range
    const uint32_t c = sh[(in_range << lay.rshift) + threadIdx.x];
    if (c) hist_overflow(dests, static_cast<unsigned long long>(c));
  }
  __syncthreads();
  for (int b = threadIdx.x; b < lay.smem_bins; b += blockDim.x) {
    const uint32_t c = bins[b];
    if (c) hist_add(dests, b, static_cast<unsigned long long>(c));
  }
}

// Percentile read-out.  The quotients count / total are formed by all threads; one thread then adds
// them in bin order, so that the running sum rounds exactly as a sequential float64 cumulative sum.
constexpr int kPctThreads = 1024;
constexpr int kPctChunk = 4096;   // quotients staged per round (32 KB of shared memory)

__device__ __forceinline__ void hist_percentile_body(const unsigned long long* __restrict__ counts, int nbins,
                                                     const float* __restrict__ edges, float bin_width, double frac,
                                                     float* __restrict__ amax_out) {
  __shared__ double q[kPctChunk];
  __shared__ unsigned long long warp_sums[kPctThreads / 32];
  __shared__ unsigned long long total_s;
  __shared__ double cdf_s;
  __shared__ int idx_s;
  unsigned long long part = 0;
  for (int i = threadIdx.x; i < nbins; i += blockDim.x) part += counts[i];
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = part;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long t = 0;
    for (int w = 0; w < kPctThreads / 32; ++w) t += warp_sums[w];
    total_s = t; cdf_s = 0.0; idx_s = -1;
  }
  __syncthreads();
  const double dt = static_cast<double>(total_s);
  for (int base = 0; base < nbins; base += kPctChunk) {
    const int len = min(kPctChunk, nbins - base);
    for (int i = threadIdx.x; i < len; i += blockDim.x) q[i] = static_cast<double>(counts[base + i]) / dt;
    __syncthreads();
    if (threadIdx.x == 0 && idx_s < 0) {
      double cdf = cdf_s;
      for (int i = 0; i < len; ++i) {
        cdf += q[i];
        if (cdf >= frac) { idx_s = base + i; break; }
      }
      cdf_s = cdf;
    }
    __syncthreads();
    if (idx_s >= 0) break;
  }
  if (threadIdx.x == 0) {
    const int idx = idx_s < 0 ? nbins : idx_s;
    *amax_out = edges ? edges[idx] : bin_width * static_cast<float>(idx);
  }
}

__global__ void __launch_bounds__(kPctThreads)
hist_percentile_kernel(const unsigned long long* __restrict__ counts, int nbins,
                       const float* __restrict__ edges, float bin_width, double frac,
                       float* __restrict__ amax_out) {
  pdl_prologue();
  hist_percentile_body(counts, nbins, edges, bin_width, frac, amax_out);
}

// One CTA per histogram: the percentile read-out of all calibrators of a model in one launch.
__global__ void __launch_bounds__(kPctThreads)
hist_percentile_batch_kernel(const b200q_hist_desc* __restrict__ descs, double frac, float* __restrict__ amax_out) {
  pdl_prologue();
  const b200q_hist_desc d = descs[blockIdx.x];
  hist_percentile_body(d.counts, d.nbins, d.edges, d.bin_width, frac, amax_out + blockIdx.x);
}

// ---- entropy (KL-divergence) read-out -------------------------------------------------------------
// One CTA per candidate clip point i (the first i bins kept): the kept bins are merged into
// `nlev` equal-width levels, each level's mass spread evenly over its non-empty bins, and
// KL(reference || candidate) taken with the clipped tail added to the reference's last bin
// (reference calib/histogram.py:210-282; bin 0 takes the count of bin 1 first).  Counts are
// integers, so level masses and totals are exact; the divergence is summed in fp64.
constexpr int kEntThreads = 256;
constexpr int kEntMaxLevels = 1 << 12;

__device__ __forceinline__ unsigned long long ent_count(const unsigned long long* c, int j) {
  return c[j == 0 ? 1 : j];   // the reference overwrites bin 0 by bin 1
}

__global__ void __launch_bounds__(kEntThreads)
hist_entropy_kernel(const unsigned long long* __restrict__ counts, int nbins, int nlev, int start_bin,
                    int stride, double* __restrict__ divs) {
  pdl_prologue();
  extern __shared__ unsigned long long ent_sh[];   // [nlev] mass | [nlev] non-empty bins (as u64)
  unsigned long long* mass = ent_sh;
  unsigned long long* cnt = ent_sh + nlev;
  __shared__ double red[kEntThreads / 32];
  __shared__ unsigned long long redu[kEntThreads / 32];
  const int i = start_bin + static_cast<int>(blockIdx.x) * stride;   // bins kept
  for (int l = threadIdx.x; l < 2 * nlev; l += blockDim.x) ent_sh[l] = 0;
  __syncthreads();
  // level of bin j: floor(j * nlev / i)  (nlev is a power of two: the reference's linspace edges are exact)
  unsigned long long tail = 0;
  for (int j = threadIdx.x; j < nbins; j += blockDim.x) {
    const unsigned long long c = ent_count(counts, j);
    if (j < i) {
      if (c) {
        const int l = static_cast<int>((static_cast<long long>(j) * nlev) / i);
        atomicAdd(mass + l, c);
        atomicAdd(cnt + l, 1ull);
      }
    } else {
      tail += c;
    }
  }
  for (int o = 16; o > 0; o >>= 1) tail += __shfl_xor_sync(0xffffffffu, tail, o);
  if ((threadIdx.x & 31) == 0) redu[threadIdx.x >> 5] = tail;
  __syncthreads();
  tail = 0;
  for (int w = 0; w < kEntThreads / 32; ++w) tail += redu[w];
  unsigned long long head = 0;   // sum of the kept bins = sum of the level masses
  for (int l = 0; l < nlev; ++l) head += mass[l];   // nlev <= 4096: cheap, same order in every thread
  const double total = static_cast<double>(head + tail), dhead = static_cast<double>(head);
  double kl = 0.0;
  bool infinite = false;
  for (int j = threadIdx.x; j < i; j += blockDim.x) {
    const unsigned long long c = ent_count(counts, j);
    unsigned long long r = c + (j == i - 1 ? tail : 0ull);
    if (r == 0) continue;
    if (c == 0) { infinite = true; continue; }   // reference mass where the candidate has none
    const int l = static_cast<int>((static_cast<long long>(j) * nlev) / i);
    const double p = static_cast<double>(r) / total;
    const double q = (static_cast<double>(mass[l]) / static_cast<double>(cnt[l])) / dhead;
    kl += p * log(p / q);
  }
  for (int o = 16; o > 0; o >>= 1) kl += __shfl_xor_sync(0xffffffffu, kl, o);
  const bool any_inf = __syncthreads_or(infinite);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = kl;
  __syncthreads();
  if (threadIdx.x == 0) {
    double sum = 0.0;
    for (int w = 0; w < kEntThreads / 32; ++w) sum += red[w];
    divs[blockIdx.x] = any_inf ? __longlong_as_double(0x7ff0000000000000ll) : sum;
  }
}

// last minimum of divs -> amax = edges[index * stride + start_bin]
__global__ void hist_entropy_pick_kernel(const double* __restrict__ divs, int ncand, int start_bin, int stride,
                                         const float* __restrict__ edges, float bin_width,
                                         float* __restrict__ amax_out) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  int best = 0;
  double bv = divs[0];
  for (int k = 1; k < ncand; ++k)
    if (divs[k] <= bv) { bv = divs[k]; best = k; }
  const int idx = best * stride + start_bin;
  *amax_out = edges ? edges[idx] : bin_width * static_cast<float>(idx);
}

// ---- mean-squared-error read-out ---------------------------------------------------------------------
// One CTA per candidate clip point i: amax = centre of bin i, every bin centre is fake quantised to
// `bound` integer levels with that amax and the count-weighted squared error is averaged (fp64).
// The FIRST minimum wins.
__global__ void __launch_bounds__(kEntThreads)
hist_mse_kernel(const unsigned long long* __restrict__ counts, int nbins, const float* __restrict__ edges,
                double bound, int start_bin, int stride, double* __restrict__ errs) {
  pdl_prologue();
  __shared__ double red[kEntThreads / 32];
  const int i = start_bin + static_cast<int>(blockIdx.x) * stride;
  const double amax = (static_cast<double>(edges[i + 1]) + static_cast<double>(edges[i])) / 2.0;
  const double scale = bound / amax;
  double acc = 0.0;
  for (int j = threadIdx.x; j < nbins; j += blockDim.x) {
    const double c = (static_cast<double>(edges[j + 1]) + static_cast<double>(edges[j])) / 2.0;
    double q = rint(c * scale);
    q = fmin(fmax(q, -bound), bound) / scale;
    acc += (q - c) * (q - c) * static_cast<double>(counts[j]);
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double sum = 0.0;
    for (int w = 0; w < kEntThreads / 32; ++w) sum += red[w];
    errs[blockIdx.x] = sum / static_cast<double>(nbins);
  }
}

__global__ void hist_mse_pick_kernel(const double* __restrict__ errs, int ncand, int start_bin, int stride,
                                     const float* __restrict__ edges, float* __restrict__ amax_out) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  int best = 0;
  double bv = errs[0];
  for (int k = 1; k < ncand; ++k)
    if (errs[k] < bv) { bv = errs[k]; best = k; }
  const int i = best * stride + start_bin;
  *amax_out = static_cast<float>((static_cast<double>(edges[i + 1]) + static_cast<double>(edges[i])) / 2.0);
}

}  // namespace b200q

using namespace b200q;

// range_dev == nullptr: the range is `range_max`; otherwise it is read from the device when the kernel runs
// (and the 16-bit kernel sizes its shared memory for the largest counter layout any range can need).
static int hist_collect_impl(const void* x, int64_t n, int dtype, int nbins, float range_max, const float* range_dev,
                             int capacity, const HistDests& dests, void* stream) {
  B200Q_REQUIRE_PTR(x);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x);
  if (dests.n < 1 || dests.n > kHistMaxDests) return B200Q_ERR_ARG;
  for (int i = 0; i < dests.n; ++i) B200Q_REQUIRE_PTR(dests.counts[i]);
  if (n <= 0 || nbins <= 0 || capacity < nbins || capacity > (1 << 22)) return B200Q_ERR_SHAPE;
  HistOpen open;
  open.capacity = capacity;
  open.overflow = nullptr;
  open.cap_range = 0.f;
  if (range_dev == nullptr) {
    if (!(range_max > 0.f)) return B200Q_ERR_ARG;
    // right end of the last bin; for the closed histogram exactly range_max
    open.cap_range = capacity == nbins ? range_max
                                       : static_cast<float>(static_cast<double>(range_max) * capacity / nbins);
    if (!(open.cap_range < 3.0e38f)) return B200Q_ERR_ARG;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // 32-bit shared counters: one launch bins at most 2^36 elements (< 2^32 per CTA)
  const int64_t chunk = int64_t{1} << 36;
  if (dtype != B200Q_F32) {
    const int smem_bins = capacity < kHist16MaxSmemBins ? capacity : kHist16MaxSmemBins;
    return B200Q_DISPATCH(dtype, [&]() -> int {
      if constexpr (sizeof(T) == 2) {
        Hist16Layout lay;
        size_t smem;
        if (range_dev == nullptr) {
          lay = hist16_layout<T>(range_max, open.cap_range, nbins, smem_bins);
          smem = ((static_cast<size_t>(lay.values) << lay.rshift) + ((lay.smem_bins + 3) & ~3)) * sizeof(uint32_t);
        } else {
          lay.lo = lay.hi1 = 0; lay.values = 0; lay.rshift = 0; lay.smem_bins = smem_bins;
          smem = static_cast<size_t>(kHist16SmemWords) * sizeof(uint32_t);
        }
        auto kern = hist16_collect_kernel<T>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kHist16SmemWords * 4) != cudaSuccess)
          return B200Q_ERR_CUDA;
        for (int64_t off = 0; off < n; off += chunk) {
          const int64_t len = n - off < chunk ? n - off : chunk;
          const int grid = grid_for(len / 8, kHistThreads * 4, 1);
          launch_pdl(kern, grid, kHistThreads, smem, s, static_cast<const T*>(x) + off, len, nbins, range_max, open,
                     lay, dests, range_dev);
        }
        return launch_status();
      } else {
        return B200Q_ERR_DTYPE;
      }
    });
  }
  // fp32: shared bins, all of them when they fit, replicated as often as the budget allows (<= 32)
  const int max_words = kHistSmemBytes / 4;
  int smem_bins = nbins + 1 <= max_words ? nbins : max_words - 1;
  int replicas = 1;
  while (replicas < 32 && static_cast<int64_t>(smem_bins + 1) * replicas * 2 <= max_words) replicas <<= 1;
  const size_t smem = static_cast<size_t>(smem_bins + 1) * replicas * sizeof(uint32_t);
  auto kern = smem_bins == capacity ? hist_collect_kernel<float, true> : hist_collect_kernel<float, false>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kHistSmemBytes) != cudaSuccess)
    return B200Q_ERR_CUDA;
  for (int64_t off = 0; off < n; off += chunk) {
    const int64_t len = n - off < chunk ? n - off : chunk;
    const int grid = grid_for(len / 4, kHistThreads * 4, 1);
    launch_pdl(kern, grid, kHistThreads, smem, s, static_cast<const float*>(x) + off, len, nbins, range_max, open, smem_bins,
               replicas, dests, range_dev);
  }
  return launch_status();
}

static HistDests one_dest(unsigned long long* counts, unsigned long long* overflow) {
  HistDests d = {};
  d.counts[0] = counts;
  d.overflow[0] = overflow;
  d.n = 1;
  return d;
}

extern "C" int b200q_hist_collect(const void* x, int64_t n, int dtype, int nbins, float range_max,
                                  unsigned long long* counts, void* stream) {
  B200Q_REQUIRE_PTR(counts);
  return hist_collect_impl(x, n, dtype, nbins, range_max, nullptr, nbins, one_dest(counts, nullptr), stream);
}

extern "C" int b200q_hist_collect_open(const void* x, int64_t n, int dtype, int nbins, float range_max,
                                       int capacity, unsigned long long* counts, unsigned long long* overflow,
                                       void* stream) {
  B200Q_REQUIRE_PTR(counts); B200Q_REQUIRE_PTR(overflow);
  return hist_collect_impl(x, n, dtype, nbins, range_max, nullptr, capacity, one_dest(counts, overflow), stream);
}

extern "C" int b200q_hist_collect_shared(const void* x, int64_t n, int dtype, int nbins, const float* range_dev,
                                         int capacity, unsigned long long* const* counts,
                                         unsigned long long* const* overflow, int n_dest, void* stream) {
  B200Q_REQUIRE_PTR(range_dev); B200Q_REQUIRE_PTR(counts); B200Q_REQUIRE_PTR(overflow);
  if (n_dest < 1 || n_dest > kHistMaxDests) return B200Q_ERR_ARG;
  HistDests d = {};
  d.n = n_dest;
  for (int i = 0; i < n_dest; ++i) {
    B200Q_REQUIRE_PTR(counts[i]); B200Q_REQUIRE_PTR(overflow[i]);
    d.counts[i] = counts[i];
    d.overflow[i] = overflow[i];
  }
  return hist_collect_impl(x, n, dtype, nbins, 0.f, range_dev, capacity, d, stream);
}

extern "C" int b200q_hist_percentile(const unsigned long long* counts, int nbins, const float* edges,
                                     float bin_width, double percentile, float* amax_out,
                                     void* stream) {
  B200Q_REQUIRE_PTR(counts); B200Q_REQUIRE_PTR(amax_out);
  if (nbins <= 0) return B200Q_ERR_SHAPE;
  if (!(percentile >= 0.0 && percentile <= 100.0)) return B200Q_ERR_ARG;
  hist_percentile_kernel<<<1, kPctThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      counts, nbins, edges, bin_width, percentile / 100.0, amax_out);
  return launch_status();
}

extern "C" int b200q_hist_percentile_batch(const b200q_hist_desc* descs, int n, double percentile, float* amax_out,
                                           void* stream) {
  B200Q_REQUIRE_PTR(descs); B200Q_REQUIRE_PTR(amax_out);
  if ((reinterpret_cast<uintptr_t>(descs) & 7u) != 0) return B200Q_ERR_ALIGN;
  if (n <= 0) return B200Q_ERR_SHAPE;
  if (!(percentile >= 0.0 && percentile <= 100.0)) return B200Q_ERR_ARG;
  hist_percentile_batch_kernel<<<n, kPctThreads, 0, static_cast<cudaStream_t>(stream)>>>(descs, percentile / 100.0,
                                                                                        amax_out);
  return launch_status();
}

extern "C" int b200q_hist_entropy(const unsigned long long* counts, int nbins, int num_levels, int start_bin,
                                  int stride, const float* edges, float bin_width, double* divergences,
                                  float* amax_out, void* stream) {
  B200Q_REQUIRE_PTR(counts); B200Q_REQUIRE_PTR(divergences); B200Q_REQUIRE_PTR(amax_out);
  if (nbins < 2 || start_bin < 1 || start_bin > nbins || stride < 1) return B200Q_ERR_SHAPE;
  if (num_levels < 1 || num_levels > kEntMaxLevels || (num_levels & (num_levels - 1))) return B200Q_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int ncand = (nbins - start_bin) / stride + 1;
  hist_entropy_kernel<<<ncand, kEntThreads, 2 * num_levels * sizeof(unsigned long long), s>>>(
      counts, nbins, num_levels, start_bin, stride, divergences);
  hist_entropy_pick_kernel<<<1, 32, 0, s>>>(divergences, ncand, start_bin, stride, edges, bin_width, amax_out);
  return launch_status();
}

extern "C" int b200q_hist_mse(const unsigned long long* counts, int nbins, const float* edges, double bound,
                              int start_bin, int stride, double* errors, float* amax_out, void* stream) {
  B200Q_REQUIRE_PTR(counts); B200Q_REQUIRE_PTR(edges); B200Q_REQUIRE_PTR(errors); B200Q_REQUIRE_PTR(amax_out);
  if (nbins < 2 || start_bin < 0 || start_bin >= nbins || stride < 1) return B200Q_ERR_SHAPE;
  if (!(bound >= 1.0)) return B200Q_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int ncand = (nbins - 1 - start_bin) / stride + 1;
  hist_mse_kernel<<<ncand, kEntThreads, 0, s>>>(counts, nbins, edges, bound, start_bin, stride, errors);
  hist_mse_pick_kernel<<<1, 32, 0, s>>>(errors, ncand, start_bin, stride, edges, amax_out);
  return launch_status();
}
