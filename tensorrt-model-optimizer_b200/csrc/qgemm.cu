// Real-quantised GEMMs on the 5th-generation tensor cores: the consumers of the packed tensors.
//
//   FP8 per tensor:  out[m, n] = T( (sum_k A8[m, k] * B8[n, k]) * scale_a * scale_b + bias[n] )
//   NVFP4:           out[m, n] = T( T( alpha * sum_b sfa[m, b] * sfb[n, b] * sum_{j<16} A4[m, 16b + j] * B4[n, 16b + j] ) + bias[n] )
//
// A = quantised activations [M, K], B = quantised weights [N, K], K contiguous (E4M3 bytes, or two
// E2M1 codes per byte with the even element in the low nibble).  NVFP4 block scales are E4M3 bytes
// in 128-row x 4-scale tiles of 512 bytes (byte (r % 32) * 16 + (r / 32) * 4 + s of tile
// [r / 128][k / 64]), with the K extent padded to a multiple of 256 elements: the order in which
// tcgen05.cp lays a 32 x 16-byte shared-memory matrix into tensor memory, so a tile goes from
// global memory to tensor memory with one bulk copy and one tcgen05.cp and no shuffling.
//
// One CTA computes one 128 x BN output tile (BN = 128 on two CTAs per SM, or 256).  Warp 0 streams
// 128-byte-wide operand tiles (128 FP8 or 256 FP4 values of K) and the scale tiles into a
// shared-memory ring with TMA, one thread of warp 1 copies the scales into tensor memory and issues
// tcgen05.mma (kind::f8f6f4, or kind::mxf4nvf4 with block scaling) into a TMEM accumulator, warps
// 2-5 read the accumulator with tcgen05.ld, apply scale and bias and store the output rows.
//
// Every mbarrier wait is bounded: when a wait runs out, an error bit is set in the caller's status
// word, the CTA stops waiting anywhere else, lets its outstanding work drain, frees its TMEM and
// returns.
#include <cstdlib>

#include "umma.cuh"

namespace b200q {

constexpr int kQM = 128;            // output rows per CTA
constexpr int kQKBytes = 128;       // bytes of K per ring stage = one 128-byte swizzle row
constexpr int kQThreads = 192;
constexpr int kQMaxStages = 4;
constexpr uint32_t kQSfTile = 512;  // one 128-row x 4-scale tile

enum : int { kQFp8 = 0, kQNvfp4 = 1 };
enum : uint32_t { kQErrProducerWait = 16, kQErrMmaWait = 32, kQErrEpilogueWait = 64 };

template <int KIND, int BN> struct QCfg {
  static constexpr uint32_t kTileA = kQM * kQKBytes;
  static constexpr uint32_t kTileB = BN * kQKBytes;
  // four MMAs per stage, each with its own scale tile per 128 rows
  static constexpr uint32_t kSfA = KIND == kQNvfp4 ? 4 * kQSfTile : 0;
  static constexpr uint32_t kSfB = KIND == kQNvfp4 ? 4 * kQSfTile * (BN / 128) : 0;
  static constexpr uint32_t kStageBytes = kTileA + kTileB + kSfA + kSfB;   // a multiple of 1024
  static constexpr int kStages = BN == 128 ? 3 : 4;
  static constexpr int kCtasPerSm = BN == 128 ? 2 : 1;
  // TMEM columns: the fp32 accumulator, then per MMA of a stage 4 columns of A scales and BN / 32 of B scales
  static constexpr uint32_t kSfAColsPerMma = 4, kSfBColsPerMma = BN / 32;
  static constexpr uint32_t kSfACol = BN, kSfBCol = BN + 4 * kSfAColsPerMma;
  static constexpr uint32_t kUsedCols = KIND == kQNvfp4 ? kSfBCol + 4 * kSfBColsPerMma : BN;
  static constexpr uint32_t kTmemCols = kUsedCols <= 128 ? 128 : (kUsedCols <= 256 ? 256 : 512);
  // instruction descriptor, K-major A and B, N = BN, M = 128:
  //   f8f6f4:   D fp32 (bit 4), A and B E4M3 (format 0)
  //   mxf4nvf4: A and B E2M1 (format 1 at bits 7 and 10), scales UE4M3 (bit 23 clear), scale ids 0
  static constexpr uint32_t kIdesc =
      (KIND == kQNvfp4 ? ((1u << 7) | (1u << 10)) : (1u << 4)) | ((BN >> 3) << 17) | ((kQM >> 4) << 24);
};

struct QGemmSmem {
  uint64_t full[kQMaxStages];
  uint64_t empty[kQMaxStages];
  uint64_t accum;
  uint32_t tmem_base;
  uint32_t abort;
};

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_nvf4(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                          uint32_t accumulate, uint32_t tmem_sfa, uint32_t tmem_sfb) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}
// shared-memory descriptor of one scale tile: 32 rows of 16 bytes, no swizzle, 8-row groups 128 B apart
__device__ __forceinline__ uint64_t sf_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(128 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}
// 32 lanes x 128 bits from shared memory into 4 TMEM columns, repeated in all four lane quarters
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

struct QEpilogue {
  const float* alpha0;   // output scale = *alpha0 * (alpha1 ? *alpha1 : 1)
  const float* alpha1;
  const void* bias;      // [N] of the output type, or null
  void* out;             // [M, N]
  int dtype;             // dtype code of out and bias
  int bias_after_round;  // 1: T(T(acc * alpha) + bias), 0: T(acc * alpha + bias)
};

template <typename T>
__device__ __forceinline__ void q_store_chunk(const QEpilogue& ep, const uint32_t* acc, float alpha, int64_t row,
                                              int64_t N, int col0, int ncols) {
  T* dst = static_cast<T*>(ep.out) + row * N + col0;
  const T* bias = static_cast<const T*>(ep.bias);
  float y[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float v = __uint_as_float(acc[j]) * alpha;
    if (bias && j < ncols) {
      const float b = Elem<T>::to_float(bias[col0 + j]);
      v = ep.bias_after_round ? Elem<T>::to_float(Elem<T>::from_float(v)) + b : v + b;
    }
    y[j] = v;
  }
  if (ncols == 32) {
    constexpr int kPer = 16 / sizeof(T);
#pragma unroll
    for (int v = 0; v < 32 / kPer; ++v) {
      T tmp[kPer];
#pragma unroll
      for (int j = 0; j < kPer; ++j) tmp[j] = Elem<T>::from_float(y[v * kPer + j]);
      reinterpret_cast<uint4*>(dst)[v] = *reinterpret_cast<const uint4*>(tmp);
    }
  } else {
    for (int j = 0; j < ncols; ++j) dst[j] = Elem<T>::from_float(y[j]);
  }
}

template <int KIND, int BN>
__global__ void __launch_bounds__(kQThreads, QCfg<KIND, BN>::kCtasPerSm)
qgemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
             const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb, int64_t M, int64_t N,
             int num_k_blocks, QEpilogue ep, uint32_t* __restrict__ status) {
  using Cfg = QCfg<KIND, BN>;
  constexpr int kStages = Cfg::kStages;
  constexpr uint32_t kStageBytes = Cfg::kStageBytes, kTmemCols = Cfg::kTmemCols;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  QGemmSmem* sm = reinterpret_cast<QGemmSmem*>(ring + kStages * kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // row tiles are the fast grid dimension: CTAs that share a weight tile run together
  const int m0 = blockIdx.x * kQM, n0 = blockIdx.y * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&sm->full[s], 1); mbar_init(&sm->empty[s], 1); }
    mbar_init(&sm->accum, 1);
    sm->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&sm->tmem_base);

  if (warp == 0) {
    if (lane == 0) {
      const int64_t sf_tiles_k = static_cast<int64_t>(num_k_blocks) * 4;   // scale tiles per 128 rows
      for (int kb = 0; kb < num_k_blocks; ++kb) {
        const int s = kb % kStages;
        const uint32_t ph = (kb / kStages) & 1;
        if (!mbar_wait_bounded(&sm->empty[s], ph ^ 1, &sm->abort, status, kQErrProducerWait)) break;
        uint8_t* a = ring + s * kStageBytes;
        mbar_expect_tx(&sm->full[s], kStageBytes);
        tma_load_2d(a, &map_a, &sm->full[s], kb * kQKBytes, m0);
        tma_load_2d(a + Cfg::kTileA, &map_b, &sm->full[s], kb * kQKBytes, n0);
        if constexpr (KIND == kQNvfp4) {
          uint8_t* sa = a + Cfg::kTileA + Cfg::kTileB;
          bulk_load(sa, sfa + ((m0 / 128) * sf_tiles_k + kb * 4) * kQSfTile, 4 * kQSfTile, &sm->full[s]);
#pragma unroll
          for (int t = 0; t < BN / 128; ++t)
            bulk_load(sa + Cfg::kSfA + t * 4 * kQSfTile, sfb + ((n0 / 128 + t) * sf_tiles_k + kb * 4) * kQSfTile,
                      4 * kQSfTile, &sm->full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < num_k_blocks && ok; ++kb) {
        const int s = kb % kStages;
        const uint32_t ph = (kb / kStages) & 1;
        ok = mbar_wait_bounded(&sm->full[s], ph, &sm->abort, status, kQErrMmaWait);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a = smem_u32(ring + s * kStageBytes);
        const uint64_t da = umma_desc(a), db = umma_desc(a + Cfg::kTileA);
        if constexpr (KIND == kQNvfp4) {
          const uint32_t sa = a + Cfg::kTileA + Cfg::kTileB, sb = sa + Cfg::kSfA;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            tmem_cp_sf(tmem + Cfg::kSfACol + k * Cfg::kSfAColsPerMma, sf_desc(sa + k * kQSfTile));
#pragma unroll
            for (int t = 0; t < BN / 128; ++t)
              tmem_cp_sf(tmem + Cfg::kSfBCol + k * Cfg::kSfBColsPerMma + 4 * t, sf_desc(sb + (t * 4 + k) * kQSfTile));
          }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // 32 bytes of K per MMA (32 FP8 or 64 FP4 values): +2 in the descriptor's 16-byte units
          const uint32_t accumulate = (kb | k) != 0 ? 1u : 0u;
          if constexpr (KIND == kQNvfp4) {
            umma_nvf4(tmem, da + 2 * k, db + 2 * k, Cfg::kIdesc, accumulate,
                      tmem + Cfg::kSfACol + k * Cfg::kSfAColsPerMma, tmem + Cfg::kSfBCol + k * Cfg::kSfBColsPerMma);
          } else {
            umma_f8(tmem, da + 2 * k, db + 2 * k, Cfg::kIdesc, accumulate);
          }
        }
        umma_commit(&sm->empty[s]);   // the slot is free once these copies and MMAs have read it
      }
      umma_commit(&sm->accum);        // fires when every MMA issued above has completed
    }
  } else {
    // epilogue warps 2..5: TMEM lanes (warp % 4) * 32 .. + 31 are the rows this warp may read
    const int quarter = warp & 3;
    const bool ok = mbar_wait_bounded(&sm->accum, 0, &sm->abort, status, kQErrEpilogueWait);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      const float alpha = __ldg(ep.alpha0) * (ep.alpha1 ? __ldg(ep.alpha1) : 1.f);
      const int64_t row = m0 + quarter * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t acc[32];
        tmem_ld32(tmem + (static_cast<uint32_t>(quarter * 32) << 16) + c * 32, acc);   // all lanes: .sync.aligned
        const int col0 = n0 + c * 32;
        const int ncols = static_cast<int>(N - col0 < 32 ? N - col0 : 32);
        if (row < M && ncols > 0) {
          if (ep.dtype == B200Q_BF16) q_store_chunk<__nv_bfloat16>(ep, acc, alpha, row, N, col0, ncols);
          else if (ep.dtype == B200Q_F16) q_store_chunk<__half>(ep, acc, alpha, row, N, col0, ncols);
          else q_store_chunk<float>(ep, acc, alpha, row, N, col0, ncols);
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
  }
}

// Linear [rows, cols] E4M3 block scales -> the 128 x 4 tiles the GEMM reads; one thread per 4 scales.
__global__ void __launch_bounds__(256)
nvfp4_swizzle_scales_kernel(const uint8_t* __restrict__ lin, uint32_t* __restrict__ out, int64_t rows, int64_t cols,
                            int64_t tiles_k, int64_t total_words) {
  pdl_prologue();
  const int64_t o = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (o >= total_words) return;
  const int64_t tile = o >> 7;
  const int within = static_cast<int>(o & 127);
  const int64_t row = (tile / tiles_k) * 128 + (within & 3) * 32 + (within >> 2);
  const int64_t c0 = (tile % tiles_k) * 4;
  uint32_t w = 0;
  if (row < rows) {
    const uint8_t* p = lin + row * cols + c0;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (c0 + j < cols) w |= static_cast<uint32_t>(p[j]) << (8 * j);
  }
  out[o] = w;
}

// 2-D byte tensor [rows, kbytes] with K contiguous; boxes of 128 bytes x box_rows, 128-byte swizzle,
// zeros outside the tensor
static bool make_byte_map(CUtensorMap* map, const void* base, int64_t rows, int64_t kbytes, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(kbytes), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(kbytes)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kQKBytes), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int KIND>
static int qgemm_launch(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, int64_t m,
                        int64_t n, int64_t kbytes, const QEpilogue& ep, uint32_t* status, cudaStream_t st) {
  const int64_t sms = sm_count_cached();
  const int64_t mtiles = (m + kQM - 1) / kQM;
  int bn = 128;
  // 128 x 256 tiles (a third less operand traffic per FLOP) when the weight splits evenly and
  // every SM still gets 0.4 tiles or more; else 128 x 128 on two CTAs per SM
  if (n % 256 == 0 && mtiles * (n / 256) * 10 >= sms * 4) bn = 256;
  if (const char* e = getenv("B200Q_QGEMM_TILE")) {
    const int v = atoi(e);
    if (v == 128) bn = 128;
    if (v == 256 && n % 256 == 0) bn = 256;
  }
  const int64_t ntiles = (n + bn - 1) / bn;
  if (ntiles > 65535) return B200Q_ERR_UNSUPPORTED;
  CUtensorMap map_a, map_b;
  if (!make_byte_map(&map_a, a, m, kbytes, kQM) || !make_byte_map(&map_b, b, n, kbytes, bn)) return B200Q_ERR_CUDA;
  const int num_k_blocks = static_cast<int>((kbytes + kQKBytes - 1) / kQKBytes);
  auto launch = [&](auto bn_tag) -> int {
    constexpr int BN = decltype(bn_tag)::value;
    using Cfg = QCfg<KIND, BN>;
    const size_t smem = Cfg::kStages * Cfg::kStageBytes + sizeof(QGemmSmem) + 1024;
    if (cudaFuncSetAttribute(qgemm_kernel<KIND, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return B200Q_ERR_CUDA;
    dim3 grid(static_cast<unsigned>(mtiles), static_cast<unsigned>(ntiles));
    qgemm_kernel<KIND, BN><<<grid, kQThreads, smem, st>>>(map_a, map_b, sfa, sfb, m, n, num_k_blocks, ep, status);
    return launch_status();
  };
  if (bn == 256) return launch(std::integral_constant<int, 256>{});
  return launch(std::integral_constant<int, 128>{});
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_fp8_gemm(const uint8_t* a, const uint8_t* b, const float* scale_a, const float* scale_b,
                              const void* bias, void* out, int64_t m, int64_t n, int64_t k, int dtype,
                              uint32_t* status_io, void* stream) {
  B200Q_REQUIRE_PTR(a); B200Q_REQUIRE_PTR(b); B200Q_REQUIRE_PTR(scale_a); B200Q_REQUIRE_PTR(out);
  B200Q_REQUIRE_PTR(status_io); B200Q_REQUIRE_DTYPE(dtype);
  B200Q_REQUIRE_ALIGNED(a); B200Q_REQUIRE_ALIGNED(b); B200Q_REQUIRE_ALIGNED(out);
  if (m <= 0 || n <= 0 || k <= 0) return B200Q_ERR_SHAPE;
  if (k % 16 || n % 8) return B200Q_ERR_UNSUPPORTED;       // 16-byte rows for TMA, 16-byte output vectors
  if (m > (int64_t(1) << 31) - 256 || n > (int64_t(1) << 31) - 256 || k > (int64_t(1) << 31) - 256) return B200Q_ERR_SHAPE;
  const QEpilogue ep{scale_a, scale_b, bias, out, dtype, 0};
  return qgemm_launch<kQFp8>(a, b, nullptr, nullptr, m, n, k, ep, status_io, static_cast<cudaStream_t>(stream));
}

extern "C" int b200q_nvfp4_gemm(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                                const float* alpha, const void* bias, void* out, int64_t m, int64_t n, int64_t k,
                                int dtype, uint32_t* status_io, void* stream) {
  B200Q_REQUIRE_PTR(a); B200Q_REQUIRE_PTR(b); B200Q_REQUIRE_PTR(sfa); B200Q_REQUIRE_PTR(sfb);
  B200Q_REQUIRE_PTR(alpha); B200Q_REQUIRE_PTR(out); B200Q_REQUIRE_PTR(status_io); B200Q_REQUIRE_DTYPE(dtype);
  B200Q_REQUIRE_ALIGNED(a); B200Q_REQUIRE_ALIGNED(b); B200Q_REQUIRE_ALIGNED(sfa); B200Q_REQUIRE_ALIGNED(sfb);
  B200Q_REQUIRE_ALIGNED(out);
  if (m <= 0 || n <= 0 || k <= 0) return B200Q_ERR_SHAPE;
  if (k % 32 || n % 8) return B200Q_ERR_UNSUPPORTED;       // 16-byte rows of packed codes
  if (m > (int64_t(1) << 31) - 256 || n > (int64_t(1) << 31) - 256 || k > (int64_t(1) << 31) - 256) return B200Q_ERR_SHAPE;
  const QEpilogue ep{alpha, nullptr, bias, out, dtype, 1};
  return qgemm_launch<kQNvfp4>(a, b, sfa, sfb, m, n, k / 2, ep, status_io, static_cast<cudaStream_t>(stream));
}

extern "C" int b200q_nvfp4_swizzle_scales(const uint8_t* scales, uint8_t* swizzled, int64_t rows, int64_t cols,
                                          void* stream) {
  B200Q_REQUIRE_PTR(scales); B200Q_REQUIRE_PTR(swizzled);
  if (reinterpret_cast<uintptr_t>(swizzled) % 16) return B200Q_ERR_ALIGN;
  if (rows <= 0 || cols <= 0) return B200Q_ERR_SHAPE;
  const int64_t tiles_k = (cols + 15) / 16 * 4;            // K padded to 256 elements = 16 scales
  const int64_t total_words = (rows + 127) / 128 * tiles_k * 128;
  const int64_t blocks = (total_words + 255) / 256;
  if (blocks > 0x7fffffff) return B200Q_ERR_SHAPE;
  launch_pdl(nvfp4_swizzle_scales_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0,
             static_cast<cudaStream_t>(stream), scales, reinterpret_cast<uint32_t*>(swizzled), rows, cols, tiles_k,
             total_words);
  return launch_status();
}
