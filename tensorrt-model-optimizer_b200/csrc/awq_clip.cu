// awq_clip block search: for every weight block (one output row x `block` input channels) and every
// clip ratio r, the squared error between the block's partial dot products with the calibration
// tokens before and after fake quantisation with the block amax shrunk to amax * r:
//
//   org[t]  = T(sum_j T(x[t, j] * w[j]))
//   cur[t]  = T(sum_j T(x[t, j] * fq_r(w)[j]))          fq_r: integer fake quant with amax = T(amax * r)
//   loss_r += mean_t float(T(cur[t] - org[t]))^2
//
// with every intermediate rounded to the tensor dtype T where the reference's tensor expressions
// round it.  The reference materialises [rows, tokens, blocks, block] products per ratio; here a CTA
// keeps one block column of the tokens in shared memory, each warp quantises one weight block for
// all ratios into shared memory and then every lane accumulates two tokens against all variants.
#include "numerics.cuh"

namespace b200q {

constexpr int kClipThreads = 256;
constexpr int kClipWarps = kClipThreads / 32;
constexpr int kClipTokTile = 64;      // tokens per pass: lanes hold tokens (lane, lane + 32)
constexpr int kClipMaxVariants = 16;  // the unquantised block + up to 15 ratios
constexpr int kClipMaxBlock = 128;
constexpr int kClipRowsPerCta = 64;

template <typename T> __device__ __forceinline__ float clip_round_t(float v) {
  return Elem<T>::to_float(Elem<T>::from_float(v));
}

// A pair of T values in shared memory and their product with a broadcast weight, rounded to T.
template <typename T> struct ClipPair;
template <> struct ClipPair<float> {
  using Store = float2;
  static __device__ __forceinline__ Store make(float a, float b) { return make_float2(a, b); }
  static __device__ __forceinline__ float2 mul(Store x, Store w) { return make_float2(x.x * w.x, x.y * w.y); }
};
template <> struct ClipPair<__nv_bfloat16> {
  using Store = uint32_t;
  static __device__ __forceinline__ Store make(float a, float b) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&p);
  }
  static __device__ __forceinline__ float2 mul(Store x, Store w) {
    const __nv_bfloat162 p = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&x),
                                     *reinterpret_cast<const __nv_bfloat162*>(&w));
    const uint32_t u = *reinterpret_cast<const uint32_t*>(&p);
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
  }
};
template <> struct ClipPair<__half> {
  using Store = uint32_t;
  static __device__ __forceinline__ Store make(float a, float b) {
    const __half2 p = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&p);
  }
  static __device__ __forceinline__ float2 mul(Store x, Store w) {
    const __half2 p = __hmul2(*reinterpret_cast<const __half2*>(&x), *reinterpret_cast<const __half2*>(&w));
    return __half22float2(p);
  }
};

// four consecutive pairs from shared memory (16-byte aligned) with vector loads
__device__ __forceinline__ void clip_load4(const uint32_t* p, uint32_t* out) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
__device__ __forceinline__ void clip_load4(const float2* p, float2* out) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 2);
  out[0] = make_float2(a.x, a.y); out[1] = make_float2(a.z, a.w);
  out[2] = make_float2(b.x, b.y); out[3] = make_float2(b.z, b.w);
}

constexpr int kClipXStride = 33;   // pairs per channel row of the token tile (32 + 1: no bank conflicts)

// grid.x = block column, grid.y = tile of kClipRowsPerCta rows.
// shared: xs[block][33] pairs | wq[kClipWarps][NV][block] pairs | acc[kClipRowsPerCta][NV - 1] floats
template <typename T, int NV>
__global__ void __launch_bounds__(kClipThreads, 2)
awq_clip_loss_kernel(const T* __restrict__ w, const T* __restrict__ x, const T* __restrict__ w_amax,
                     const float* __restrict__ ratios, int nv, float* __restrict__ loss, int rows, int cols,
                     int block, int ntok, IntQ q) {
  using P = ClipPair<T>;
  using Store = typename P::Store;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Store* xs = reinterpret_cast<Store*>(smem_raw);
  Store* wq_all = xs + ((block * kClipXStride + 3) & ~3);
  float* acc_s = reinterpret_cast<float*>(wq_all + kClipWarps * NV * block);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nb = blockIdx.x, nblk = gridDim.x;
  const int row0 = blockIdx.y * kClipRowsPerCta;
  const int nrows = min(kClipRowsPerCta, rows - row0);
  Store* wq = wq_all + warp * NV * block;

  for (int i = threadIdx.x; i < kClipRowsPerCta * (NV - 1); i += blockDim.x) acc_s[i] = 0.f;
  float ratio[NV];
#pragma unroll
  for (int v = 1; v < NV; ++v) ratio[v] = v < nv ? ratios[v - 1] : 1.f;

  for (int t0 = 0; t0 < ntok; t0 += kClipTokTile) {
    __syncthreads();   // previous tile's readers are done; acc_s cleared
    // tokens (t0 + l, t0 + l + 32) of this block column, transposed: xs[j][l]
    for (int i = threadIdx.x; i < block * 32; i += blockDim.x) {
      const int l = i / block, j = i - l * block;   // consecutive threads read consecutive channels
      const int ta = t0 + l, tb = t0 + l + 32;
      const float a = ta < ntok ? Elem<T>::to_float(x[static_cast<int64_t>(ta) * cols + nb * block + j]) : 0.f;
      const float b = tb < ntok ? Elem<T>::to_float(x[static_cast<int64_t>(tb) * cols + nb * block + j]) : 0.f;
      xs[j * kClipXStride + l] = P::make(a, b);
    }
    __syncthreads();
    for (int r = warp; r < nrows; r += kClipWarps) {
      const int row = row0 + r;
      const float amax = Elem<T>::to_float(w_amax[static_cast<int64_t>(row) * nblk + nb]);
      // variant 0: the weights themselves; variant v: fake quantised with amax * ratio[v]
      IntScale sc[NV];
#pragma unroll
      for (int v = 1; v < NV; ++v) sc[v] = make_int_scale(q, clip_round_t<T>(amax * ratio[v]));
      for (int j = lane; j < block; j += 32) {
        const float wf = Elem<T>::to_float(w[static_cast<int64_t>(row) * cols + nb * block + j]);
        wq[j] = P::make(wf, wf);
#pragma unroll
        for (int v = 1; v < NV; ++v) {
          if (v < nv) {
            const float y = clip_round_t<T>(intq_apply(wf, sc[v], q));
            wq[v * block + j] = P::make(y, y);
          }
        }
      }
      __syncwarp();
      float2 acc[NV];
#pragma unroll
      for (int v = 0; v < NV; ++v) acc[v] = make_float2(0.f, 0.f);
      for (int j = 0; j < block; j += 4) {
        Store xv[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) xv[k] = xs[(j + k) * kClipXStride + lane];
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          if (v < nv) {
            Store wv[4];
            clip_load4(wq + v * block + j, wv);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 p = P::mul(xv[k], wv[k]);
              acc[v].x += p.x;
              acc[v].y += p.y;
            }
          }
        }
      }
      __syncwarp();
      const float o0 = clip_round_t<T>(acc[0].x), o1 = clip_round_t<T>(acc[0].y);
#pragma unroll
      for (int v = 1; v < NV; ++v) {
        if (v < nv) {
          const float d0 = clip_round_t<T>(clip_round_t<T>(acc[v].x) - o0);
          const float d1 = clip_round_t<T>(clip_round_t<T>(acc[v].y) - o1);
          float s = d0 * d0 + d1 * d1;
          for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
          if (lane == 0) acc_s[r * (NV - 1) + v - 1] += s;
        }
      }
    }
  }
  __syncthreads();
  const float inv = 1.f / static_cast<float>(ntok);
  for (int i = threadIdx.x; i < nrows * (nv - 1); i += blockDim.x) {
    const int r = i / (nv - 1), v = i - r * (nv - 1);
    float* dst = loss + (static_cast<int64_t>(v) * rows + row0 + r) * nblk + nb;
    *dst += acc_s[r * (NV - 1) + v] * inv;
  }
}

template <typename T, int NV>
static int launch_clip(const T* w, const T* x, const T* w_amax, const float* ratios, int nv, float* loss,
                       int rows, int cols, int block, int ntok, IntQ q, cudaStream_t s) {
  using Store = typename ClipPair<T>::Store;
  const size_t smem = sizeof(Store) * (static_cast<size_t>((block * kClipXStride + 3) & ~3) +
                                       static_cast<size_t>(kClipWarps) * NV * block) +
                      sizeof(float) * kClipRowsPerCta * (NV - 1);
  auto kern = awq_clip_loss_kernel<T, NV>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return B200Q_ERR_CUDA;
  const dim3 grid(static_cast<unsigned>(cols / block), static_cast<unsigned>((rows + kClipRowsPerCta - 1) / kClipRowsPerCta));
  kern<<<grid, kClipThreads, smem, s>>>(w, x, w_amax, ratios, nv, loss, rows, cols, block, ntok, q);
  return launch_status();
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_awq_clip_loss(const void* w, const void* x, const void* w_amax, const float* ratios,
                                   int nratios, float* loss, int64_t rows, int64_t cols, int block, int ntok,
                                   int dtype, int num_bits, int is_unsigned, int narrow_range, void* stream) {
  B200Q_REQUIRE_PTR(w); B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(w_amax); B200Q_REQUIRE_PTR(ratios);
  B200Q_REQUIRE_PTR(loss); B200Q_REQUIRE_DTYPE(dtype);
  if (rows <= 0 || cols <= 0 || ntok <= 0 || block <= 0 || cols % block || block % 4) return B200Q_ERR_SHAPE;
  if (rows > (1 << 22) || cols > (1 << 30)) return B200Q_ERR_SHAPE;
  if (block > kClipMaxBlock || nratios < 1 || nratios > kClipMaxVariants - 1) return B200Q_ERR_UNSUPPORTED;
  if ((rows + kClipRowsPerCta - 1) / kClipRowsPerCta > 65535) return B200Q_ERR_UNSUPPORTED;
  if (num_bits < 1 || num_bits + (is_unsigned ? 1 : 0) > 24) return B200Q_ERR_ARG;
  const IntQ q = make_intq(num_bits, is_unsigned, narrow_range);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int nv = nratios + 1;
  return B200Q_DISPATCH(dtype, [&]() -> int {
    const T* wp = static_cast<const T*>(w);
    const T* xp = static_cast<const T*>(x);
    const T* ap = static_cast<const T*>(w_amax);
    const int r = static_cast<int>(rows), c = static_cast<int>(cols);
    if (nv <= 12) return launch_clip<T, 12>(wp, xp, ap, ratios, nv, loss, r, c, block, ntok, q, s);
    return launch_clip<T, 16>(wp, xp, ap, ratios, nv, loss, r, c, block, ntok, q, s);
  });
}
