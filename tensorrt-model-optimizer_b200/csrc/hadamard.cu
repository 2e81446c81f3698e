// Fast Walsh-Hadamard transform along the last dimension (Sylvester order, power-of-two length),
// used to rotate activations before quantisation.  y = T(T(H x) * 1) then divided by sqrt(n) by the
// caller's choice of `scale` (applied to the T-rounded sums, result rounded to T), which is how
// the reference composes hadamard_transform(x) / sqrt(n).
//
// One warp per row for n <= 1024: lane l holds the n/32 consecutive elements l*n/32 ..; butterflies
// with a stride inside a lane's chunk are register operations, larger strides are one
// __shfl_xor per element.  Longer rows (up to 32768) go through shared memory, one CTA per row.
#include "common.cuh"

namespace b200q {

template <typename T, int EPL>   // elements per lane
__global__ void __launch_bounds__(256)
hadamard_warp_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, float scale) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int N = EPL * 32;
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t r = warp; r < rows; r += nwarps) {
    float v[EPL];
    const T* xr = x + r * N + lane * EPL;
#pragma unroll
    for (int i = 0; i < EPL; ++i) v[i] = E::to_float(xr[i]);
    // strides inside the lane's chunk
#pragma unroll
    for (int s = 1; s < EPL; s <<= 1) {
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        if ((i & s) == 0) {
          const float a = v[i], b = v[i | s];
          v[i] = a + b;
          v[i | s] = a - b;
        }
      }
    }
    // strides across lanes: partner lane = lane ^ d; the lower lane of a pair keeps a + b
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const bool upper = (lane & d) != 0;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const float o = __shfl_xor_sync(0xffffffffu, v[i], d);
        v[i] = upper ? o - v[i] : v[i] + o;
      }
    }
    T* yr = y + r * N + lane * EPL;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const float h = E::to_float(E::from_float(v[i]));       // the transform's output in T
      yr[i] = E::from_float(h * scale);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(512)
hadamard_cta_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int n, float scale) {
  pdl_prologue();
  using E = Elem<T>;
  extern __shared__ float hs[];
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) hs[i] = E::to_float(x[r * n + i]);
    __syncthreads();
    for (int s = 1; s < n; s <<= 1) {
      for (int p = threadIdx.x; p < n / 2; p += blockDim.x) {
        const int i = ((p / s) * 2 * s) + (p % s);     // lower index of pair p at stride s
        const float a = hs[i], b = hs[i + s];
        hs[i] = a + b;
        hs[i + s] = a - b;
      }
      __syncthreads();
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float h = E::to_float(E::from_float(hs[i]));
      y[r * n + i] = E::from_float(h * scale);
    }
    __syncthreads();
  }
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_hadamard(const void* x, void* y, int64_t rows, int n, int dtype, float scale, void* stream) {
  B200Q_REQUIRE_PTR(x); B200Q_REQUIRE_PTR(y); B200Q_REQUIRE_DTYPE(dtype);
  if (rows <= 0 || n < 2 || (n & (n - 1)) || n > 32768) return B200Q_ERR_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return B200Q_DISPATCH(dtype, [&]() -> int {
    const T* xp = static_cast<const T*>(x);
    T* yp = static_cast<T*>(y);
    if (n >= 32 && n <= 1024) {
      const int grid = grid_for(rows, 8, 8);   // 8 warps (rows) per CTA
      switch (n / 32) {
        case 1: launch_pdl(hadamard_warp_kernel<T, 1>, grid, 256, 0, s, xp, yp, rows, scale); break;
        case 2: launch_pdl(hadamard_warp_kernel<T, 2>, grid, 256, 0, s, xp, yp, rows, scale); break;
        case 4: launch_pdl(hadamard_warp_kernel<T, 4>, grid, 256, 0, s, xp, yp, rows, scale); break;
        case 8: launch_pdl(hadamard_warp_kernel<T, 8>, grid, 256, 0, s, xp, yp, rows, scale); break;
        case 16: launch_pdl(hadamard_warp_kernel<T, 16>, grid, 256, 0, s, xp, yp, rows, scale); break;
        default: launch_pdl(hadamard_warp_kernel<T, 32>, grid, 256, 0, s, xp, yp, rows, scale); break;
      }
    } else {
      auto kern = hadamard_cta_kernel<T>;
      const size_t smem = static_cast<size_t>(n) * sizeof(float);
      if (smem > 48 * 1024 &&
          cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
        return B200Q_ERR_CUDA;
      launch_pdl(kern, grid_for(rows, 1, 4), 512, smem, s, xp, yp, rows, n, scale);
    }
    return launch_status();
  });
}
