// awq_lite evaluation GEMM on the 5th-generation tensor cores, fused with the loss:
//
//     loss_sum += sum_{m,n} float( bf16( bf16(sum_k A[m,k] * B[n,k]) - R[m,n] ) )^2
//
// A = scaled activations [M, K], B = fake-quantised scaled weights [N, K], R = the unquantised
// layer output [M, N], all bf16 with K (resp. N for R) contiguous.  The product never goes to
// memory: accumulators live in tensor memory and the epilogue reduces the squared error.
//
// One CTA computes one 128 x BN output tile (BN = 128 or 256).  Warp 0 streams 128 x 64 and
// BN x 64 operand tiles into a shared-memory ring with TMA (128-byte swizzle), one thread of warp 1
// issues tcgen05.mma (UMMA 128 x BN x 16, bf16 -> fp32 in TMEM) and frees ring slots with
// tcgen05.commit, warps 2-5 read the accumulator with tcgen05.ld and do the epilogue.
//
// Every mbarrier wait is bounded: when a wait runs out, an error bit is set in the caller's status
// word, the CTA stops waiting anywhere else, lets its outstanding work drain, frees its TMEM and
// returns.
#include <cstdlib>

#include "umma.cuh"

namespace b200q {

constexpr int kGM = 128, kGK = 64;                   // CTA tile rows; kGK bf16 = one 128-byte swizzle row
constexpr int kMaxStages = 4;
constexpr int kUmmaK = 16;
constexpr uint32_t kTileBytesA = kGM * kGK * 2;
constexpr int kGemmThreads = 192;       // producer warp, MMA warp, four epilogue warps
// Two tile widths: 128 x 128 with a 3-deep ring (96 KB, two CTAs per SM, so one CTA's epilogue
// overlaps the other's main loop) and 128 x 256 with a 4-deep ring (192 KB, one CTA per SM, a
// third less operand traffic per FLOP).
// MT = 2 stacks two 128-row tiles on one B tile (256 x 256 per CTA, all 512 TMEM columns): the
// least operand traffic per FLOP, used when the problem still yields enough CTAs.
template <int BN, int MT> struct GemmCfg {
  static constexpr int kStages = (BN == 128 || MT == 2) ? 3 : 4;
  static constexpr uint32_t kTileBytesB = BN * kGK * 2;
  static constexpr uint32_t kStageBytes = MT * kTileBytesA + kTileBytesB;
  static constexpr uint32_t kTmemCols = BN * MT;       // fp32 accumulator columns
  static constexpr int kCtasPerSm = (BN == 128 && MT == 1) ? 2 : 1;
  // Four epilogue warps.  Eight (two per TMEM lane quarter, as the real-quant GEMMs use) make the
  // kernel alone 6-8 % faster, but the search runs it under the next candidate's quantise kernel on
  // a second stream, and with the wider CTA that overlap was lost (2.16-2.23 ms per 21 candidates
  // against 2.04-2.10 ms).
  static constexpr int kThreads = kGemmThreads;
  static constexpr int kColParts = (kThreads / 32 - 2) / 4;
  // instruction descriptor: D fp32, A/B bf16, both K-major, N = BN, M = 128
  static constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((BN >> 3) << 17) | ((kGM >> 4) << 24);
  // The tile of the reference output follows the operands through the ring: 64-column
  // pieces of MT boxes of 128 rows, as many per stage as fit, in the uses right after the last K block.
  static constexpr uint32_t kRefPieceBytes = MT * kTileBytesA;
  static constexpr int kRefPieces = BN / kGK;
  static constexpr int kRefPiecesPerStage = kStageBytes / kRefPieceBytes;
  static constexpr int kRefStages = (kRefPieces + kRefPiecesPerStage - 1) / kRefPiecesPerStage;
  static_assert(kRefStages <= kStages, "the reference tile must fit in the ring");
};

enum : uint32_t { kErrProducerWait = 1, kErrMmaWait = 2, kErrEpilogueWait = 4 };

struct GemmSmem {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t accum;
  uint32_t tmem_base;
  uint32_t abort;
  uint32_t last_split;   // split-K: 1 in the CTA that found the other splits' partial tiles complete
};

// Split-K staging: a warp's 32 x 32 fp32 piece passes through shared memory so that global memory
// sees whole 128-byte row segments (8 lanes per row, 4 rows per instruction) instead of one row per lane.
constexpr uint32_t kSplitPitch = 32 * 4 + 16;
__device__ __forceinline__ void split_store_piece(const uint32_t* acc, uint8_t* stage, int lane, float* dst, int64_t ld) {
  uint4* mine = reinterpret_cast<uint4*>(stage + lane * kSplitPitch);
#pragma unroll
  for (int v = 0; v < 8; ++v) mine[v] = make_uint4(acc[4 * v], acc[4 * v + 1], acc[4 * v + 2], acc[4 * v + 3]);
  __syncwarp();
  const int part = lane & 7, rsub = lane >> 3;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = rsub + 4 * i;
    *reinterpret_cast<uint4*>(dst + r * ld + part * 4) = *reinterpret_cast<const uint4*>(stage + r * kSplitPitch + part * 16);
  }
  __syncwarp();
}
// sum of the `splits` partial pieces (in split order) back into one row per lane
__device__ __forceinline__ void split_load_piece(uint32_t* acc, uint8_t* stage, int lane, const float* src, int64_t ld,
                                                 int64_t split_stride, int splits) {
  const int part = lane & 7, rsub = lane >> 3;
  float4 sum[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) sum[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int z = 0; z < splits; ++z) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 p = __ldcg(reinterpret_cast<const float4*>(src + z * split_stride + (rsub + 4 * i) * ld + part * 4));
      sum[i].x += p.x; sum[i].y += p.y; sum[i].z += p.z; sum[i].w += p.w;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) *reinterpret_cast<float4*>(stage + (rsub + 4 * i) * kSplitPitch + part * 16) = sum[i];
  __syncwarp();
  const uint4* mine = reinterpret_cast<const uint4*>(stage + lane * kSplitPitch);
#pragma unroll
  for (int v = 0; v < 8; ++v) {
    const uint4 q = mine[v];
    acc[4 * v] = q.x; acc[4 * v + 1] = q.y; acc[4 * v + 2] = q.z; acc[4 * v + 3] = q.w;
  }
  __syncwarp();
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, GemmSmem* sm, uint32_t* status,
                                          uint32_t code) {
  return mbar_wait_bounded(bar, parity, &sm->abort, status, code);
}

template <int BN, int MT>
__global__ void __launch_bounds__(GemmCfg<BN, MT>::kThreads, GemmCfg<BN, MT>::kCtasPerSm)
awq_gemm_sqerr_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_r,
                      int64_t N, int total_k_blocks, int kb_per_split,
                      float* __restrict__ partial, uint32_t* __restrict__ counters, double* __restrict__ sum_io,
                      float* __restrict__ c_out, uint32_t* __restrict__ status) {
  using Cfg = GemmCfg<BN, MT>;
  // split-K (gridDim.z > 1): this CTA sums K blocks kb0 .. kb0 + num_k_blocks - 1 and leaves an fp32
  // partial tile in `partial`; the CTA of a tile that finishes last adds the partial tiles in split
  // order (so the sum does not depend on timing) and runs the loss epilogue
  const int splits = gridDim.z;
  const int kb0 = blockIdx.z * kb_per_split;
  const int num_k_blocks = min(kb_per_split, total_k_blocks - kb0);
  constexpr int kStages = Cfg::kStages;
  constexpr uint32_t kStageBytes = Cfg::kStageBytes, kTmemCols = Cfg::kTmemCols;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // operand ring first (1024-byte aligned for the swizzle), control block after it
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  GemmSmem* sm = reinterpret_cast<GemmSmem*>(ring + kStages * kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the (few) row tiles are the fast grid dimension: CTAs that share a B tile run together, so
  // the tile comes from DRAM once and from L2 for the others
  const int m0 = blockIdx.x * kGM * MT, n0 = blockIdx.y * BN;

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
      for (int kb = 0; kb < num_k_blocks; ++kb) {
        const int s = kb % kStages;
        const uint32_t ph = (kb / kStages) & 1;
        if (!mbar_wait(&sm->empty[s], ph ^ 1, sm, status, kErrProducerWait)) break;
        uint8_t* a = ring + s * kStageBytes;
        mbar_expect_tx(&sm->full[s], kStageBytes);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) tma_load_2d(a + mt * kTileBytesA, &map_a, &sm->full[s], (kb0 + kb) * kGK, m0 + mt * kGM);
        tma_load_2d(a + MT * kTileBytesA, &map_b, &sm->full[s], (kb0 + kb) * kGK, n0);
      }
      if (!*reinterpret_cast<volatile uint32_t*>(&sm->abort)) {
        // the reference tile, into the stages the last MMAs free: the epilogue then reads it from shared
        // memory instead of waiting for one L2 round trip per 32-column chunk with the tensor cores idle
        for (int j = 0; j < Cfg::kRefStages; ++j) {
          const int use = num_k_blocks + j, s = use % kStages;
          if (!mbar_wait(&sm->empty[s], ((use / kStages) & 1) ^ 1, sm, status, kErrProducerWait)) break;
          const int first = j * Cfg::kRefPiecesPerStage;
          const int count = min(Cfg::kRefPiecesPerStage, Cfg::kRefPieces - first);
          mbar_expect_tx(&sm->full[s], count * Cfg::kRefPieceBytes);
          uint8_t* dst = ring + s * kStageBytes;
          for (int p = 0; p < count; ++p)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
              tma_load_2d(dst + (p * MT + mt) * kTileBytesA, &map_r, &sm->full[s], n0 + (first + p) * kGK, m0 + mt * kGM);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < num_k_blocks && ok; ++kb) {
        const int s = kb % kStages;
        const uint32_t ph = (kb / kStages) & 1;
        ok = mbar_wait(&sm->full[s], ph, sm, status, kErrMmaWait);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a = smem_u32(ring + s * kStageBytes);
        const uint64_t db = umma_desc(a + MT * kTileBytesA);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint64_t da = umma_desc(a + mt * kTileBytesA);
#pragma unroll
          for (int k = 0; k < kGK / kUmmaK; ++k) {
            // advancing 16 bf16 = 32 bytes along K inside the swizzled row: +2 in 16-byte units
            umma_bf16(tmem + mt * BN, da + 2 * k, db + 2 * k, Cfg::kIdesc, (kb | k) != 0 ? 1u : 0u);
          }
        }
        umma_commit(&sm->empty[s]);   // the slot is free once these MMAs have read it
      }
      umma_commit(&sm->accum);        // fires when every MMA issued above has completed
    }
  } else {
    // epilogue warps 2..: TMEM lanes (warp % 4) * 32 .. + 31 are the rows this warp may read
    const int quarter = warp & 3;
    const int col_part = (warp - 2) >> 2;       // 0 with four epilogue warps; a wider CTA would split the columns
    constexpr int kChunksPerPart = BN / 32 / Cfg::kColParts;
    const bool ok = mbar_wait(&sm->accum, 0, sm, status, kErrEpilogueWait);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    float sq = 0.f;
    bool finish = ok;                       // this CTA runs the loss epilogue
    const int64_t m_total = static_cast<int64_t>(gridDim.x) * kGM * MT;
    // split-K scratch: the ring is idle once the accumulator is complete, except for the stage(s) that hold
    // the reference tile; the scratch sits in the stage after them
    // (split launches run 128 x 128 tiles: one of three stages holds the reference tile)
    uint8_t* stage = ring + ((num_k_blocks + Cfg::kRefStages) % kStages) * kStageBytes + (warp - 2) * 32 * kSplitPitch;
    if (splits > 1) {
      constexpr int kEpiThreads = Cfg::kThreads - 64;
      if (ok) {
#pragma unroll 1
        for (int mt = 0; mt < MT; ++mt) {
          const int64_t row0 = m0 + mt * kGM + quarter * 32;
#pragma unroll 1
          for (int c = col_part * kChunksPerPart; c < (col_part + 1) * kChunksPerPart; ++c) {
            uint32_t acc[32];
            tmem_ld32(tmem + (static_cast<uint32_t>(quarter * 32) << 16) + mt * BN + c * 32, acc);
            split_store_piece(acc, stage, lane, partial + (blockIdx.z * m_total + row0) * N + n0 + c * 32, N);
          }
        }
      }
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");      // the epilogue warps only
      if (threadIdx.x == 64) {
        uint32_t* counter = counters + blockIdx.y * gridDim.x + blockIdx.x;
        const uint32_t seen = atomicAdd(counter, 1u);
        sm->last_split = seen == static_cast<uint32_t>(splits - 1);
        if (sm->last_split) *counter = 0;                                    // ready for the next launch
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
      finish = ok && *reinterpret_cast<volatile uint32_t*>(&sm->last_split) != 0;
      __threadfence();
    }
    if (finish) {
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        const int64_t row0 = m0 + mt * kGM + quarter * 32;
        const int64_t row = row0 + lane;
#pragma unroll 1
        for (int c = col_part * kChunksPerPart; c < (col_part + 1) * kChunksPerPart; ++c) {
          uint32_t acc[32];
          if (splits == 1)
            tmem_ld32(tmem + (static_cast<uint32_t>(quarter * 32) << 16) + mt * BN + c * 32, acc);
          else
            split_load_piece(acc, stage, lane, partial + row0 * N + n0 + c * 32, N, m_total * N, splits);
          // the chunk's 64 bytes of this lane's row sit in the ring (rows of 128 bytes, 16-byte unit u
          // of row r at position u ^ (r & 7)); chunk c is the half (c & 1) of 64-column piece c / 2
          const uint8_t* srow;
          {
            const int piece = c >> 1, j = piece / Cfg::kRefPiecesPerStage, p = piece - j * Cfg::kRefPiecesPerStage;
            const int use = num_k_blocks + j, s = use % kStages;
            if (!__all_sync(0xffffffffu, mbar_wait(&sm->full[s], (use / kStages) & 1, sm, status, kErrEpilogueWait))) break;
            srow = ring + s * kStageBytes + (p * MT + mt) * kTileBytesA + (quarter * 32 + lane) * 128;
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const uint4 r4 = *reinterpret_cast<const uint4*>(srow + ((((c & 1) * 4 + v) ^ (lane & 7)) << 4));
            float rf[8];
            Elem<__nv_bfloat16>::unpack(r4, rf);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float a = __uint_as_float(acc[8 * v + j]);
              const float o = __bfloat162float(__float2bfloat16_rn(a));
              const float d = __bfloat162float(__float2bfloat16_rn(o - rf[j]));
              sq = fmaf(d, d, sq);
            }
          }
          if (c_out) {
            float* cp = c_out + row * N + n0 + c * 32;
#pragma unroll
            for (int j = 0; j < 32; ++j) cp[j] = __uint_as_float(acc[j]);
          }
        }
      }
    }
    if (!finish && warp == 2 && lane == 0) {
      // a CTA that does not run the loss epilogue (another split finishes the tile) still asked for the
      // reference tile: the copy must have landed before this CTA's shared memory is given up
      for (int j = 0; j < Cfg::kRefStages; ++j) {
        const int use = num_k_blocks + j;
        if (!mbar_wait(&sm->full[use % kStages], (use / kStages) & 1, sm, status, kErrEpilogueWait)) break;
      }
    }
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if (lane == 0 && finish) atomicAdd(sum_io, static_cast<double>(sq));
  }

  grace_after_abort(&sm->abort);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
  }
}

// ---- host side -------------------------------------------------------------------------------------
// 2-D bf16 tensor [rows, k] with k contiguous; boxes of kGK x box_rows, 128-byte swizzle
static bool make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kGK), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace b200q

using namespace b200q;

static int awq_gemm_launch(const void* a, const void* b, const void* ref, int64_t m, int64_t n, int64_t k, int splits,
                           float* partial, uint32_t* counters, double* sum_io, float* c_out, uint32_t* status_io,
                           void* stream) {
  B200Q_REQUIRE_PTR(a); B200Q_REQUIRE_PTR(b); B200Q_REQUIRE_PTR(ref); B200Q_REQUIRE_PTR(sum_io);
  B200Q_REQUIRE_PTR(status_io);
  B200Q_REQUIRE_ALIGNED(a); B200Q_REQUIRE_ALIGNED(b); B200Q_REQUIRE_ALIGNED(ref);
  if (m <= 0 || n <= 0 || k <= 0) return B200Q_ERR_SHAPE;
  if (m % kGM || n % 128 || k % kGK || n / 128 > 65535) return B200Q_ERR_UNSUPPORTED;
  // Tile choice: 256 x 256 per CTA when that still gives ~3/4 of the SMs a tile (least operand
  // traffic per FLOP — the kernel is bound by L2 -> SM bandwidth); else 128 x 256 when every SM gets
  // 0.4 tiles or more (fewer, faster CTAs beat more CTAs here); else 128 x 128 on two CTAs per SM.
  const int64_t sms = sm_count_cached();
  int bn = 128, mt = 1;
  if (n % 256 == 0 && (m / kGM) * (n / 256) * 10 >= sms * 4) bn = 256;
  if (n % 256 == 0 && m % 256 == 0 && (m / 256) * (n / 256) * 4 >= sms * 3) { bn = 256; mt = 2; }
  const int total_kb = static_cast<int>(k / kGK);
  if (splits < 1 || splits > 16 || splits > total_kb) return B200Q_ERR_ARG;
  if (splits > 1) { bn = 128; mt = 1; }                   // more, smaller CTAs is the point of splitting
  const int kb_per_split = (total_kb + splits - 1) / splits;
  const int zdim = (total_kb + kb_per_split - 1) / kb_per_split;   // every split has at least one block
  CUtensorMap map_a, map_b, map_r;
  if (!make_map(&map_a, a, m, k, kGM) || !make_map(&map_b, b, n, k, bn) || !make_map(&map_r, ref, m, n, kGM))
    return B200Q_ERR_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto launch = [&](auto bn_tag, auto mt_tag) -> int {
    constexpr int BN = decltype(bn_tag)::value, MT = decltype(mt_tag)::value;
    using Cfg = GemmCfg<BN, MT>;
    const size_t smem = Cfg::kStages * Cfg::kStageBytes + sizeof(GemmSmem) + 1024;
    if (cudaFuncSetAttribute(awq_gemm_sqerr_kernel<BN, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return B200Q_ERR_CUDA;
    dim3 grid(static_cast<unsigned>(m / (kGM * MT)), static_cast<unsigned>(n / BN), static_cast<unsigned>(zdim));
    awq_gemm_sqerr_kernel<BN, MT><<<grid, Cfg::kThreads, smem, st>>>(
        map_a, map_b, map_r, n, total_kb, kb_per_split, partial, counters, sum_io,
        c_out, status_io);
    return launch_status();
  };
  using I1 = std::integral_constant<int, 1>;
  using I2 = std::integral_constant<int, 2>;
  using I128 = std::integral_constant<int, 128>;
  using I256 = std::integral_constant<int, 256>;
  if (bn == 256 && mt == 2) return launch(I256{}, I2{});
  if (bn == 256) return launch(I256{}, I1{});
  return launch(I128{}, I1{});
}

extern "C" int b200q_awq_gemm_sqerr(const void* a, const void* b, const void* ref, int64_t m, int64_t n,
                                    int64_t k, double* sum_io, float* c_out, uint32_t* status_io,
                                    void* stream) {
  return awq_gemm_launch(a, b, ref, m, n, k, 1, nullptr, nullptr, sum_io, c_out, status_io, stream);
}

extern "C" int b200q_awq_gemm_sqerr_splitk(const void* a, const void* b, const void* ref, int64_t m, int64_t n,
                                           int64_t k, int splits, float* workspace, uint32_t* counters,
                                           double* sum_io, float* c_out, uint32_t* status_io, void* stream) {
  if (splits > 1) { B200Q_REQUIRE_PTR(workspace); B200Q_REQUIRE_PTR(counters); B200Q_REQUIRE_ALIGNED(workspace); }
  return awq_gemm_launch(a, b, ref, m, n, k, splits, workspace, counters, sum_io, c_out, status_io, stream);
}
