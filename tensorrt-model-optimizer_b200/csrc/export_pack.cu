// Export-side INT4 packing (the layout deployment checkpoints use): signed two's-complement nibbles
// paired along the OUTPUT dimension — byte [r, c] holds row 2r in the low nibble and row 2r+1 in the
// high nibble — with scale = amax/7 per (row, block of input columns).
#include "numerics.cuh"

namespace b200q {

template <typename T> __device__ __forceinline__ float round_tt(float v) {
  return Elem<T>::to_float(Elem<T>::from_float(v));
}

// q = clamp(round_half_even(w / scale), -8, 7); the quotient is an fp32 division when the scales
// are fp32 (torch promotes), and is rounded to T when the scales have the weight's type.
template <typename T, bool kScaleIsT>
__device__ __forceinline__ uint32_t int4_signed_code(float w, float scale) {
  float q = __fdiv_rn(w, scale);
  if (kScaleIsT) q = round_tt<T>(q);
  q = fminf(7.f, fmaxf(-8.f, rintf(q)));
  return static_cast<uint32_t>(static_cast<int>(q)) & 0xfu;
}

// one thread: one pack of columns of two adjacent rows -> P bytes
template <typename T, bool kScaleIsT>
__global__ void __launch_bounds__(256)
int4_export_pack_kernel(const T* __restrict__ w, const void* __restrict__ scales, uint8_t* __restrict__ out,
                        int64_t row_pairs, FastDiv packs_per_row, int packs_per_block, int blocks_per_row) {
  pdl_prologue();
  using E = Elem<T>;
  constexpr int P = E::kPerPack;
  const int64_t total = row_pairs * packs_per_row.d;
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    uint32_t rp, cp;
    packs_per_row.divmod(static_cast<uint32_t>(i), rp, cp);       // total < 2^31 here
    const int64_t r0 = 2 * static_cast<int64_t>(rp);
    const uint4 a = ld_stream(wv + r0 * packs_per_row.d + cp);
    const uint4 b = ld_stream(wv + (r0 + 1) * packs_per_row.d + cp);
    const int blk = cp / packs_per_block;
    float s0, s1;
    if (kScaleIsT) {
      s0 = E::to_float(static_cast<const T*>(scales)[r0 * blocks_per_row + blk]);
      s1 = E::to_float(static_cast<const T*>(scales)[(r0 + 1) * blocks_per_row + blk]);
    } else {
      s0 = static_cast<const float*>(scales)[r0 * blocks_per_row + blk];
      s1 = static_cast<const float*>(scales)[(r0 + 1) * blocks_per_row + blk];
    }
    float fa[P], fb[P];
    E::unpack(a, fa);
    E::unpack(b, fb);
    uint32_t o[P / 4];
#pragma unroll
    for (int k = 0; k < P / 4; ++k) {
      uint32_t word = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t lo = int4_signed_code<T, kScaleIsT>(fa[4 * k + j], s0);
        const uint32_t hi = int4_signed_code<T, kScaleIsT>(fb[4 * k + j], s1);
        word |= (lo | (hi << 4)) << (8 * j);
      }
      o[k] = word;
    }
    uint8_t* dst = out + static_cast<int64_t>(rp) * packs_per_row.d * P + static_cast<int64_t>(cp) * P;
    if (P == 8) *reinterpret_cast<uint2*>(dst) = make_uint2(o[0], o[P / 4 - 1]);
    else *reinterpret_cast<uint32_t*>(dst) = o[0];
  }
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_int4_export_pack(const void* w, const void* scales, int scales_are_f32, uint8_t* out,
                                      int64_t rows, int64_t cols, int block, int dtype, void* stream) {
  B200Q_REQUIRE_PTR(w); B200Q_REQUIRE_PTR(scales); B200Q_REQUIRE_PTR(out);
  B200Q_REQUIRE_DTYPE(dtype); B200Q_REQUIRE_ALIGNED(w);
  if ((reinterpret_cast<uintptr_t>(out) & 7u) != 0) return B200Q_ERR_ALIGN;
  if (rows <= 0 || cols <= 0 || block <= 0 || (rows & 1) || cols % block) return B200Q_ERR_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return B200Q_DISPATCH(dtype, [&]() -> int {
    constexpr int P = Elem<T>::kPerPack;
    if (cols % P || block % P) return B200Q_ERR_UNSUPPORTED;
    const int64_t total = (rows / 2) * (cols / P);
    if (total > kFastDivLimit) return B200Q_ERR_UNSUPPORTED;
    const FastDiv ppr(static_cast<uint32_t>(cols / P));
    int grid = grid_for(total, 256, 8);
    const T* wp = static_cast<const T*>(w);
    if (scales_are_f32)
      launch_pdl(int4_export_pack_kernel<T, false>, grid, 256, 0, s, wp, scales, out, rows / 2, ppr, block / P,
                                                             static_cast<int>(cols / block));
    else
      launch_pdl(int4_export_pack_kernel<T, true>, grid, 256, 0, s, wp, scales, out, rows / 2, ppr, block / P,
                                                            static_cast<int>(cols / block));
    return launch_status();
  });
}
