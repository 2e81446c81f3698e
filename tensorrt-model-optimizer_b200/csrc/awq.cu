// Kernels of the awq_lite search loop: per-input-channel scaling fused with per-block dynamic
// integer fake quantisation of the weight, and the squared-error reduction between two GEMM
// outputs.  The GEMM itself runs between them.
#include "numerics.cuh"

namespace b200q {

template <typename T> __device__ __forceinline__ float round_t(float v) {
  return Elem<T>::to_float(Elem<T>::from_float(v));
}

// w [rows, cols] row-major, s [cols] in T.  For every run of `block` elements along a row:
//   v = T(w * s[col]);  amax = max|v|;  y = T(fake_int(v, amax))
// `lanes` adjacent lanes (power of two <= 32) own one block, PPL packs each.
template <typename T, int PPL>
__global__ void __launch_bounds__(256)
awq_scale_fq_kernel(const T* __restrict__ w, const T* __restrict__ s, T* __restrict__ y,
                    int64_t nblocks, int lanes, FastDiv blocks_per_row, IntQ q) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  const int64_t gthread = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t total = nblocks * lanes;
  const int lane_shift = __ffs(lanes) - 1;
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  const uint4* sv = reinterpret_cast<const uint4*>(s);
  uint4* yv = reinterpret_cast<uint4*>(y);
  for (int64_t t = gthread; t < ((total + 31) / 32) * 32; t += nthreads) {
    const bool valid = t < total;
    // column of this lane's first pack: (block index within its row) * packs per block + lane offset
    uint32_t rowq, colblk;
    blocks_per_row.divmod(static_cast<uint32_t>(valid ? (t >> lane_shift) : 0), rowq, colblk);   // nblocks < 2^31
    // lane l of a block takes packs l, l + lanes, ...: whole sectors per load instruction
    const uint32_t spack = colblk * lanes * PPL + static_cast<uint32_t>(t & (lanes - 1));
    const int64_t wpack = (t >> lane_shift) * (lanes * PPL) + (t & (lanes - 1));
    const int pstride = lanes;
    float v[PPL][P];
    uint32_t bits = 0;
#pragma unroll
    for (int p = 0; p < PPL; ++p) {
      uint4 a = valid ? ld_stream(wv + wpack + p * pstride) : make_uint4(0, 0, 0, 0);
      uint4 b = valid ? __ldg(sv + spack + p * pstride) : make_uint4(0, 0, 0, 0);
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        // packed bf16 multiply = the product rounded to bf16, two elements per instruction
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
        uint32_t acc16 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat162 pr = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&aw[i]),
                                            *reinterpret_cast<const __nv_bfloat162*>(&bw[i]));
          const uint32_t pw = *reinterpret_cast<const uint32_t*>(&pr);
          v[p][2 * i] = __uint_as_float(pw << 16);
          v[p][2 * i + 1] = __uint_as_float(pw & 0xffff0000u);
          acc16 = __vmaxu2(acc16, pw & 0x7fff7fffu);
        }
        bits = max(bits, max(acc16 & 0xffffu, acc16 >> 16) << 16);
      } else {
        float fa[P], fb[P];
        E::unpack(a, fa);
        E::unpack(b, fb);
#pragma unroll
        for (int k = 0; k < P; ++k) {
          v[p][k] = round_t<T>(fa[k] * fb[k]);
          bits = max(bits, __float_as_uint(v[p][k]) & 0x7fffffffu);
        }
      }
    }
    for (int o = lanes >> 1; o > 0; o >>= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
    const IntScale sc = make_int_scale(q, __uint_as_float(bits));
    if (valid) {
#pragma unroll
      for (int p = 0; p < PPL; ++p) {
        intq_apply_n<P>(v[p], sc, q);
        st_stream(yv + wpack + p * pstride, E::pack(v[p]));
      }
    }
  }
}

// sum over i of float(T(a_i - b_i))^2, added to a double accumulator
template <typename T>
__global__ void __launch_bounds__(256)
sq_diff_sum_kernel(const T* __restrict__ a, const T* __restrict__ b, int64_t n, double* __restrict__ out) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  __shared__ float red[8];
  const int64_t npack = n / P;
  const uint4* av = reinterpret_cast<const uint4*>(a);
  const uint4* bv = reinterpret_cast<const uint4*>(b);
  float acc = 0.f;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < npack; i += stride) {
    float fa[P], fb[P];
    E::unpack(ld_stream(av + i), fa);
    E::unpack(ld_stream(bv + i), fb);
#pragma unroll
    for (int k = 0; k < P; ++k) {
      const float d = round_t<T>(fa[k] - fb[k]);
      acc = fmaf(d, d, acc);
    }
  }
  if (blockIdx.x == 0 && threadIdx.x < n - npack * P) {
    const int64_t j = npack * P + threadIdx.x;
    const float d = round_t<T>(E::to_float(a[j]) - E::to_float(b[j]));
    acc = fmaf(d, d, acc);
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double s = 0.0;
    for (int i = 0; i < 8; ++i) s += static_cast<double>(red[i]);
    atomicAdd(out, s);
  }
}

// out[a, m, :] = T(x[m, :] * s[a, :]) for every candidate a: the activations of an awq_lite search step
// under each candidate's inverse scale, written once (the read of x stays in L2 across candidates).
// One thread per 16-byte pack of x; it keeps the pack in registers and loops over the candidates.
template <typename T>
__global__ void __launch_bounds__(256)
awq_scale_acts_kernel(const T* __restrict__ x, const T* __restrict__ s, T* __restrict__ out, int64_t rows,
                      int64_t packs_per_row, int n_alpha) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  const int64_t npack = rows * packs_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  const uint4* sv = reinterpret_cast<const uint4*>(s);
  uint4* ov = reinterpret_cast<uint4*>(out);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < npack; i += stride) {
    const uint4 a = ld_stream(xv + i);
    const int64_t col = i % packs_per_row;
    // candidates in rounds of eight: the eight scale loads of a round are in flight together (one
    // dependent L2 round trip per round instead of one per candidate).  Plain stores: the search kernel
    // reads these tiles next, and most of them are still in L2 then.
    for (int c0 = 0; c0 < n_alpha; c0 += 8) {
      uint4 b[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (c0 + u < n_alpha) b[u] = __ldg(sv + (c0 + u) * packs_per_row + col);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (c0 + u >= n_alpha) break;
        uint4 r;
        if constexpr (std::is_same<T, __nv_bfloat16>::value) {
          const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
          uint32_t rw[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const __nv_bfloat162 pr = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&aw[k]),
                                              *reinterpret_cast<const __nv_bfloat162*>(&bw[k]));
            rw[k] = *reinterpret_cast<const uint32_t*>(&pr);
          }
          r = make_uint4(rw[0], rw[1], rw[2], rw[3]);
        } else {
          float fa[P], fb[P];
          E::unpack(a, fa);
          E::unpack(b[u], fb);
#pragma unroll
          for (int k = 0; k < P; ++k) fa[k] = round_t<T>(fa[k] * fb[k]);
          r = E::pack(fa);
        }
        ov[(c0 + u) * npack + i] = r;
      }
    }
  }
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_awq_scale_acts(const void* x, const void* s, void* out, int64_t rows, int64_t cols, int n_alpha,
                                    int dtype, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(s); B200Q_REQUIRE_PTR(out);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(x); B200Q_REQUIRE_ALIGNED(s); B200Q_REQUIRE_ALIGNED(out);
  if (rows <= 0 || cols <= 0 || n_alpha <= 0) return B200Q_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return B200Q_DISPATCH(dtype, [&]() -> int {
    constexpr int P = Elem<T>::kPerPack;
    if (cols % P) return B200Q_ERR_SHAPE;
    const int64_t ppr = cols / P;
    int grid = grid_for(rows * ppr, 256, 8);
    launch_pdl(awq_scale_acts_kernel<T>, grid, 256, 0, st, static_cast<const T*>(x), static_cast<const T*>(s),
               static_cast<T*>(out), rows, ppr, n_alpha);
    return launch_status();
  });
}

extern "C" int b200q_awq_scale_fake_int(const void* w, const void* s, void* y, int64_t rows, int64_t cols,
                                        int block, int dtype, int num_bits, int is_unsigned,
                                        int narrow_range, void* stream) {
  B200Q_REQUIRE_PTR(w); B200Q_REQUIRE_PTR(s); B200Q_REQUIRE_PTR(y);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(w); B200Q_REQUIRE_ALIGNED(s); B200Q_REQUIRE_ALIGNED(y);
  if (rows <= 0 || cols <= 0 || block <= 0 || cols % block) return B200Q_ERR_SHAPE;
  if (num_bits < 1 || num_bits + (is_unsigned ? 1 : 0) > 24) return B200Q_ERR_ARG;
  const IntQ q = make_intq(num_bits, is_unsigned, narrow_range);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return B200Q_DISPATCH(dtype, [&]() -> int {
    constexpr int P = Elem<T>::kPerPack;
    const int packs = block / P;
    if (block % P || packs <= 0 || (packs & (packs - 1)) || packs > 64) return B200Q_ERR_UNSUPPORTED;
    const int ppl = packs >= 4 ? 4 : packs >= 2 ? 2 : 1;
    const int lanes = packs / ppl;
    const int64_t nblocks = rows * (cols / block);
    if (nblocks > kFastDivLimit) return B200Q_ERR_UNSUPPORTED;
    const FastDiv bpr(static_cast<uint32_t>(cols / block));
    int grid = grid_for(nblocks * lanes, 256, 8);
    const T* wp = static_cast<const T*>(w);
    const T* sp = static_cast<const T*>(s);
    T* yp = static_cast<T*>(y);
    if (ppl == 4) launch_pdl(awq_scale_fq_kernel<T, 4>, grid, 256, 0, st, wp, sp, yp, nblocks, lanes, bpr, q);
    else if (ppl == 2) launch_pdl(awq_scale_fq_kernel<T, 2>, grid, 256, 0, st, wp, sp, yp, nblocks, lanes, bpr, q);
    else launch_pdl(awq_scale_fq_kernel<T, 1>, grid, 256, 0, st, wp, sp, yp, nblocks, lanes, bpr, q);
    return launch_status();
  });
}

extern "C" int b200q_sq_diff_sum(const void* a, const void* b, int64_t n, int dtype, double* sum_io,
                                 void* stream) {
  B200Q_REQUIRE_PTR(a); B200Q_REQUIRE_PTR(b); B200Q_REQUIRE_PTR(sum_io);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(a); B200Q_REQUIRE_ALIGNED(b);
  if (n <= 0) return B200Q_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return B200Q_DISPATCH(dtype, [&] {
    int grid = grid_for(n / Elem<T>::kPerPack, 256 * 4, 8);
    launch_pdl(sq_diff_sum_kernel<T>, grid, 256, 0, st, static_cast<const T*>(a), static_cast<const T*>(b), n, sum_io);
    return launch_status();
  });
}
