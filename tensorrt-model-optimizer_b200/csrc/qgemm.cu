// Real-quantised GEMMs on the 5th-generation tensor cores: the consumers of the packed tensors.
//
//   FP8 per tensor:  out[m, n] = T( (sum_k A8[m, k] * B8[n, k]) * scale_a * scale_b + bias[n] )
//   NVFP4:           out[m, n] = T( T( alpha * sum_b sfa[m, b] * sfb[n, b] * sum_{j<16} A4[m, 16b + j] * B4[n, 16b + j] ) + bias[n] )
//
// A = quantised activations [M, K], B = quantised weights [N, K], K contiguous (E4M3 bytes, or two
// E2M1 codes per byte with the even element in the low nibble).  NVFP4 block scales are E4M3 bytes
// in 128-row x 4-scale tiles of 512 bytes (byte (r % 32) * 16 + (r / 32) * 4 + s of tile
// [r / 128][k / 64]), with the K extent padded to a multiple of 256 elements: the order the
// block-scaled MMA reads them in from tensor memory (row r in lane r % 32, column r / 32 of the tile's
// four), so a tile goes from global memory to tensor memory with one bulk copy and four-column
// stores (or one tcgen05.cp) and no shuffling.
//
// One CTA computes MT stacked 128 x BN output tiles on one weight tile (128 x 128 on two CTAs per SM,
// 128 x 256, or 256 x 256 for FP8 / 256 x 192 for NVFP4).  Warp 0 streams
// 128-byte-wide operand tiles (128 FP8 or 256 FP4 values of K) and the scale tiles into a
// shared-memory ring with TMA, one thread of warp 1 issues tcgen05.mma (kind::f8f6f4, or
// kind::mxf4nvf4 with block scaling) into a TMEM accumulator, warps 2-5 move the block scales of
// each stage from shared memory into tensor memory during the main loop (tcgen05.st) and afterwards
// read the accumulator with tcgen05.ld, apply scale and bias and store the output rows.
//
// Every mbarrier wait is bounded: when a wait runs out, an error bit is set in the caller's status
// word, the CTA stops waiting anywhere else, lets its outstanding work drain, frees its TMEM and
// returns.

#include "umma.cuh"

namespace b200q {

constexpr int kQM = 128;            // output rows per CTA
constexpr int kQKBytes = 128;       // bytes of K per ring stage = one 128-byte swizzle row
constexpr int kQThreads = 192;       // producer warp, MMA warp, four epilogue warps
constexpr int kQThreadsWide = 320;   // ... and four more epilogue warps where one CTA has the SM to itself
constexpr int kQMaxStages = 4;
constexpr uint32_t kQSfTile = 512;  // one 128-row x 4-scale tile

enum : int { kQFp8 = 0, kQNvfp4 = 1 };
enum : uint32_t { kQErrProducerWait = 16, kQErrMmaWait = 32, kQErrEpilogueWait = 64 };

template <int KIND, int BN, int MT> struct QCfg {
  static constexpr int kBTiles = (BN + 127) / 128;           // 128-row scale tiles a weight tile touches
  static constexpr uint32_t kTileA = kQM * kQKBytes;
  static constexpr uint32_t kTileB = BN * kQKBytes;
  // four MMAs per stage and row tile, each with its own scale tile per 128 rows
  static constexpr uint32_t kSfA = KIND == kQNvfp4 ? 4 * kQSfTile * MT : 0;
  static constexpr uint32_t kSfB = KIND == kQNvfp4 ? 4 * kQSfTile * kBTiles : 0;
  static constexpr uint32_t kStageBytes = MT * kTileA + kTileB + kSfA + kSfB;   // a multiple of 1024
  static constexpr int kStages = (BN == 128 && MT == 1) ? 3 : (kStageBytes > 56 * 1024 ? 3 : 4);
  static constexpr int kCtasPerSm = (BN == 128 && MT == 1) ? 2 : 1;
  // the un-overlapped epilogue of a lone CTA is drained by eight warps, two per TMEM lane quarter
  static constexpr int kThreads = kCtasPerSm == 1 ? kQThreadsWide : kQThreads;
  static constexpr int kEpiWarps = kThreads / 32 - 2;
  // TMEM columns: MT fp32 accumulators of BN columns, then sets of scale columns: per MMA of a stage
  // 4 columns of A scales per row tile and 4 of B scales per 128 weight rows.  Stages take the sets
  // in turn, so the scale copy of a stage does not wait for the MMAs of the one before.
  static constexpr uint32_t kSfAColsPerMma = 4 * MT, kSfBColsPerMma = 4 * kBTiles;
  static constexpr uint32_t kSfColsPerStage = 4 * (kSfAColsPerMma + kSfBColsPerMma);
  static constexpr uint32_t kAccCols = BN * MT;
  static constexpr uint32_t kTmemBudget = kCtasPerSm == 2 ? 256 : 512;
  static constexpr int kSfSets = KIND == kQNvfp4
      ? ((kTmemBudget - kAccCols) / kSfColsPerStage < kStages ? (kTmemBudget - kAccCols) / kSfColsPerStage : kStages) : 0;
  static_assert(KIND != kQNvfp4 || kSfSets >= 1, "no TMEM left for the block scales");
  // With a set per ring stage, the four otherwise idle epilogue warps move the scales (shared memory
  // -> registers -> tcgen05.st, each warp into its own lane quarter); tcgen05.cp, which takes the
  // tensor pipe for about 130 cycles per 512-byte tile, is left to the tile shape that has no room.
  static constexpr bool kSfByWarps = KIND == kQNvfp4 && kSfSets >= kStages;
  static constexpr uint32_t kSfACol = kAccCols, kSfBCol = kAccCols + 4 * kSfAColsPerMma;
  static constexpr uint32_t kUsedCols = kAccCols + kSfSets * kSfColsPerStage;
  static constexpr uint32_t kTmemCols = kUsedCols <= 128 ? 128 : (kUsedCols <= 256 ? 256 : 512);
  static_assert(kUsedCols <= kTmemBudget, "TMEM overcommitted");
  // instruction descriptor, K-major A and B, N = BN, M = 128:
  //   f8f6f4:   D fp32 (bit 4), A and B E4M3 (format 0)
  //   mxf4nvf4: A and B E2M1 (format 1 at bits 7 and 10), scales UE4M3 (bit 23 clear), scale ids 0
  static constexpr uint32_t kIdesc =
      (KIND == kQNvfp4 ? ((1u << 7) | (1u << 10)) : (1u << 4)) | ((BN >> 3) << 17) | ((kQM >> 4) << 24);
};

struct QGemmSmem {
  uint64_t full[kQMaxStages];
  uint64_t empty[kQMaxStages];
  uint64_t sf_full[kQMaxStages];
  uint64_t sf_ready[kQMaxStages];
  uint64_t accum;
  uint32_t tmem_base;
  uint32_t abort;
};

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
// one warp: lane i writes four 32-bit columns of TMEM lane (lane field of taddr) + i
__device__ __forceinline__ void tmem_st4(uint32_t taddr, uint4 v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};"
               ::"r"(taddr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 128 bits from shared memory into 4 TMEM columns, repeated in all four lane quarters
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

__device__ __forceinline__ void cluster_sync_all() { cluster_barrier(); }

struct QEpilogue {
  const float* alpha0;   // output scale = *alpha0 * (alpha1 ? *alpha1 : 1)
  const float* alpha1;
  const void* bias;      // [N] of the output type, or null
  void* out;             // [M, N]
  int dtype;             // dtype code of out and bias
  int bias_after_round;  // 1: T(T(acc * alpha) + bias), 0: T(acc * alpha + bias)
};

constexpr uint32_t kQEpiPitch = 32 * 4 + 16;   // staging row: 32 fp32 + 16 bytes against bank conflicts

// One 32-row x 32-column piece of the output: lane = row in, scaled and biased, converted to T and
// staged in shared memory so that the global stores go out as whole 64- or 128-byte row segments
// (the accumulator arrives one row per lane; storing it that way writes 32 scattered half sectors).
template <typename T>
__device__ __forceinline__ void q_store_chunk(const QEpilogue& ep, const uint32_t* acc, float alpha, uint8_t* stage,
                                              int lane, int64_t row0, int64_t M, int64_t N, int col0) {
  const T* bias = static_cast<const T*>(ep.bias);
  constexpr int kPer = 16 / sizeof(T);          // elements per 16-byte part
  constexpr int kParts = 32 / kPer;             // parts per row segment
  uint8_t* mine = stage + lane * kQEpiPitch;
#pragma unroll
  for (int v = 0; v < kParts; ++v) {
    T tmp[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int c = v * kPer + j;
      float y = __uint_as_float(acc[c]) * alpha;
      if (bias && col0 + c < N) {
        const float b = Elem<T>::to_float(__ldg(bias + col0 + c));
        y = ep.bias_after_round ? Elem<T>::to_float(Elem<T>::from_float(y)) + b : y + b;
      }
      tmp[j] = Elem<T>::from_float(y);
    }
    *reinterpret_cast<uint4*>(mine + v * 16) = *reinterpret_cast<const uint4*>(tmp);
  }
  __syncwarp();
  const int part = lane % kParts, rsub = lane / kParts;
  T* out = static_cast<T*>(ep.out);
#pragma unroll
  for (int i = 0; i < kParts; ++i) {
    const int r = rsub + i * (32 / kParts);
    const int64_t row = row0 + r;
    const int col = col0 + part * kPer;
    if (row < M && col < N)                    // N is a multiple of 8: a part is inside or outside as a whole
      *reinterpret_cast<uint4*>(out + row * N + col) = *reinterpret_cast<const uint4*>(stage + r * kQEpiPitch + part * 16);
  }
  __syncwarp();
}

// KSPLIT: the two CTAs of a cluster (1, 1, 2) each sum half of the K blocks of one tile; CTA 1 hands
// its fp32 accumulator to CTA 0 through distributed shared memory and CTA 0 adds (own + partner, a
// fixed order) and runs the epilogue.  For shapes with fewer tiles than SMs and a long K.
template <int KIND, int BN, int MT, bool KSPLIT>
__global__ void __launch_bounds__(QCfg<KIND, BN, MT>::kThreads, QCfg<KIND, BN, MT>::kCtasPerSm)
qgemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
             const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb, int64_t M, int64_t N,
             int total_k_blocks, QEpilogue ep, uint32_t* __restrict__ status) {
  using Cfg = QCfg<KIND, BN, MT>;
  static_assert(!KSPLIT || (BN == 128 && MT == 1), "the partner's 128 x 128 fp32 tile must fit in the idle ring");
  const int krank = KSPLIT ? static_cast<int>(blockIdx.z) : 0;
  const int kb_first_half = KSPLIT ? (total_k_blocks + 1) / 2 : total_k_blocks;
  const int kb0 = krank * kb_first_half;
  const int num_k_blocks = krank ? total_k_blocks - kb_first_half : kb_first_half;
  constexpr int kStages = Cfg::kStages;
  constexpr uint32_t kStageBytes = Cfg::kStageBytes, kTmemCols = Cfg::kTmemCols;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  QGemmSmem* sm = reinterpret_cast<QGemmSmem*>(ring + kStages * kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // row tiles are the fast grid dimension: CTAs that share a weight tile run together
  const int m0 = blockIdx.x * kQM * MT, n0 = blockIdx.y * BN;
  // scale tiles of the weight rows n0 .. n0 + BN - 1: they start inside 128-row tile n0 / 128, at
  // 32-row group (n0 % 128) / 32, which is the TMEM column the MMA starts reading B scales from
  const int64_t sfb_tile0 = n0 / 128;
  const uint32_t sfb_col_shift = (n0 % 128) / 32;
  const int64_t sfb_tiles_total = (N + 127) / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sm->full[s], 1); mbar_init(&sm->empty[s], 1);
      mbar_init(&sm->sf_full[s], 1); mbar_init(&sm->sf_ready[s], 4);
    }
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
      const int64_t sf_tiles_k = static_cast<int64_t>(total_k_blocks) * 4;   // scale tiles per 128 rows
      // scale tiles past the last one are not read (their rows lie beyond M or N and are never stored)
      int b_tiles = Cfg::kBTiles;
      if (sfb_tile0 + b_tiles > sfb_tiles_total) b_tiles = static_cast<int>(sfb_tiles_total - sfb_tile0);
      int a_tiles = MT;
      if (m0 / 128 + a_tiles > (M + 127) / 128) a_tiles = static_cast<int>((M + 127) / 128 - m0 / 128);
      for (int kb = 0; kb < num_k_blocks; ++kb) {
        const int s = kb % kStages;
        const uint32_t ph = (kb / kStages) & 1;
        if (!mbar_wait_bounded(&sm->empty[s], ph ^ 1, &sm->abort, status, kQErrProducerWait)) break;
        uint8_t* a = ring + s * kStageBytes;
        if constexpr (KIND == kQNvfp4) {
          // the (small) scale tiles first: with kSfByWarps on a barrier of their own, so the warps
          // that move them to TMEM are done by the time the operand tiles have landed
          uint64_t* sf_bar = Cfg::kSfByWarps ? &sm->sf_full[s] : &sm->full[s];
          const uint32_t sf_tx = (a_tiles + b_tiles) * 4 * kQSfTile;
          if (Cfg::kSfByWarps) {
            mbar_expect_tx(&sm->sf_full[s], sf_tx);
            mbar_expect_tx(&sm->full[s], MT * Cfg::kTileA + Cfg::kTileB);
          } else {
            mbar_expect_tx(&sm->full[s], MT * Cfg::kTileA + Cfg::kTileB + sf_tx);
          }
          uint8_t* sa = a + MT * Cfg::kTileA + Cfg::kTileB;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            if (mt < a_tiles)
              bulk_load(sa + mt * 4 * kQSfTile, sfa + ((m0 / 128 + mt) * sf_tiles_k + (kb0 + kb) * 4) * kQSfTile,
                        4 * kQSfTile, sf_bar);
#pragma unroll
          for (int t = 0; t < Cfg::kBTiles; ++t)
            if (t < b_tiles)
              bulk_load(sa + Cfg::kSfA + t * 4 * kQSfTile, sfb + ((sfb_tile0 + t) * sf_tiles_k + (kb0 + kb) * 4) * kQSfTile,
                        4 * kQSfTile, sf_bar);
        } else {
          mbar_expect_tx(&sm->full[s], kStageBytes);
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          tma_load_2d(a + mt * Cfg::kTileA, &map_a, &sm->full[s], (kb0 + kb) * kQKBytes, m0 + mt * kQM);
        tma_load_2d(a + MT * Cfg::kTileA, &map_b, &sm->full[s], (kb0 + kb) * kQKBytes, n0);
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
        const uint64_t db = umma_desc(a + MT * Cfg::kTileA);
        uint32_t tsf = tmem;                                      // this stage's set of scale columns
        if constexpr (KIND == kQNvfp4) tsf = tmem + ((Cfg::kSfByWarps ? s : kb) % Cfg::kSfSets) * Cfg::kSfColsPerStage;
        if constexpr (Cfg::kSfByWarps) {
          ok = mbar_wait_bounded(&sm->sf_ready[s], ph, &sm->abort, status, kQErrMmaWait);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t sa = a + MT * Cfg::kTileA + Cfg::kTileB, sb = sa + Cfg::kSfA;
        // per 32 bytes of K (32 FP8 or 64 FP4 values): the scale tiles of that slice into TMEM, then
        // its MMAs, so an MMA waits for its own scales only and the later copies run under it
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if constexpr (KIND == kQNvfp4 && !Cfg::kSfByWarps) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
              tmem_cp_sf(tsf + Cfg::kSfACol + k * Cfg::kSfAColsPerMma + 4 * mt, sf_desc(sa + (mt * 4 + k) * kQSfTile));
#pragma unroll
            for (int t = 0; t < Cfg::kBTiles; ++t)
              tmem_cp_sf(tsf + Cfg::kSfBCol + k * Cfg::kSfBColsPerMma + 4 * t, sf_desc(sb + (t * 4 + k) * kQSfTile));
          }
          const uint32_t accumulate = (kb | k) != 0 ? 1u : 0u;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            // +2 per slice in the descriptor's 16-byte units
            const uint64_t da = umma_desc(a + mt * Cfg::kTileA);
            if constexpr (KIND == kQNvfp4) {
              umma_nvf4(tmem + mt * BN, da + 2 * k, db + 2 * k, Cfg::kIdesc, accumulate,
                        tsf + Cfg::kSfACol + k * Cfg::kSfAColsPerMma + 4 * mt,
                        tsf + Cfg::kSfBCol + k * Cfg::kSfBColsPerMma + sfb_col_shift);
            } else {
              umma_f8(tmem + mt * BN, da + 2 * k, db + 2 * k, Cfg::kIdesc, accumulate);
            }
          }
        }
        umma_commit(&sm->empty[s]);   // the slot is free once these copies and MMAs have read it
      }
      umma_commit(&sm->accum);        // fires when every MMA issued above has completed
    }
  } else {
    // epilogue warps 2..: TMEM lanes (warp % 4) * 32 .. + 31 are the rows this warp may read; with
    // eight of them, warps 6..9 take the upper half of the columns
    const int quarter = warp & 3;
    const int col_part = (warp - 2) >> 2;
    constexpr int kColParts = Cfg::kEpiWarps / 4, kChunksPerPart = BN / 32 / kColParts;
    if (Cfg::kSfByWarps && col_part == 0) {
      // during the main loop: the scales of each stage from shared memory into this warp's lane
      // quarter of the stage's TMEM columns (lane i: bytes 16 i .. 16 i + 15 of a tile = its four
      // columns), then one arrival per warp on the stage's sf_ready barrier
      const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
      for (int kb = 0; kb < num_k_blocks; ++kb) {
        const int s = kb % kStages;
        if (!mbar_wait_bounded(&sm->sf_full[s], (kb / kStages) & 1, &sm->abort, status, kQErrEpilogueWait)) break;
        const uint8_t* sf = ring + s * kStageBytes + MT * Cfg::kTileA + Cfg::kTileB + lane * 16;
        const uint32_t tsf = tmem + lane_base + s * Cfg::kSfColsPerStage;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            tmem_st4(tsf + Cfg::kSfACol + k * Cfg::kSfAColsPerMma + 4 * mt,
                     *reinterpret_cast<const uint4*>(sf + (mt * 4 + k) * kQSfTile));
#pragma unroll
          for (int t = 0; t < Cfg::kBTiles; ++t)
            tmem_st4(tsf + Cfg::kSfBCol + k * Cfg::kSfBColsPerMma + 4 * t,
                     *reinterpret_cast<const uint4*>(sf + Cfg::kSfA + (t * 4 + k) * kQSfTile));
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->sf_ready[s]);
      }
    }
    const bool ok = mbar_wait_bounded(&sm->accum, 0, &sm->abort, status, kQErrEpilogueWait);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    constexpr uint32_t kXPitch = BN * 4 + 16;                      // KSPLIT: a row of the partner's fp32 tile
    constexpr uint32_t kXBytes = KSPLIT ? kQM * kXPitch : 0;
    if constexpr (KSPLIT) {
      cluster_sync_all();     // both accumulators are complete and both rings idle
      if (krank == 1 && ok) {
        // this CTA's accumulator rows into CTA 0's ring: lane = row, 128 contiguous bytes per piece
        const uint32_t remote = map_to_cta(ring + (quarter * 32 + lane) * kXPitch, 0);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t acc[32];
          tmem_ld32(tmem + (static_cast<uint32_t>(quarter * 32) << 16) + c * 32, acc);
#pragma unroll
          for (int v = 0; v < 8; ++v)
            asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(remote + c * 128 + v * 16),
                         "r"(acc[4 * v]), "r"(acc[4 * v + 1]), "r"(acc[4 * v + 2]), "r"(acc[4 * v + 3]) : "memory");
        }
      }
      cluster_sync_all();     // the partner's tile has arrived (release / acquire at cluster scope)
    }
    if (ok && krank == 0) {
      // every load of the ring has been consumed by now: its first bytes serve as staging space
      uint8_t* stage = ring + kXBytes + (warp - 2) * 32 * kQEpiPitch;
      const float alpha = __ldg(ep.alpha0) * (ep.alpha1 ? __ldg(ep.alpha1) : 1.f);
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        const int64_t row0 = m0 + mt * kQM + quarter * 32;
        if (row0 >= M) break;                                              // warp-uniform
#pragma unroll 1
        for (int c = col_part * kChunksPerPart; c < (col_part + 1) * kChunksPerPart; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= N) break;                                            // warp-uniform
          uint32_t acc[32];
          tmem_ld32(tmem + (static_cast<uint32_t>(quarter * 32) << 16) + mt * BN + c * 32, acc);   // whole warp
          if constexpr (KSPLIT) {
            const uint4* part = reinterpret_cast<const uint4*>(ring + (quarter * 32 + lane) * kXPitch + c * 128);
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              const uint4 p = part[v];
              acc[4 * v] = __float_as_uint(__uint_as_float(acc[4 * v]) + __uint_as_float(p.x));
              acc[4 * v + 1] = __float_as_uint(__uint_as_float(acc[4 * v + 1]) + __uint_as_float(p.y));
              acc[4 * v + 2] = __float_as_uint(__uint_as_float(acc[4 * v + 2]) + __uint_as_float(p.z));
              acc[4 * v + 3] = __float_as_uint(__uint_as_float(acc[4 * v + 3]) + __uint_as_float(p.w));
            }
          }
          if (ep.dtype == B200Q_BF16) q_store_chunk<__nv_bfloat16>(ep, acc, alpha, stage, lane, row0, M, N, col0);
          else if (ep.dtype == B200Q_F16) q_store_chunk<__half>(ep, acc, alpha, stage, lane, row0, M, N, col0);
          else q_store_chunk<float>(ep, acc, alpha, stage, lane, row0, M, N, col0);
        }
      }
    }
  }
  if constexpr (KSPLIT) {
    // the producer and MMA warps keep the two cluster barriers whole; their lanes left a one-lane
    // loop above, and an .aligned barrier needs the warp converged
    if (warp < 2) { __syncwarp(); cluster_sync_all(); cluster_sync_all(); }
  }

  grace_after_abort(&sm->abort);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (warp == 1) {
    __syncwarp();
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

template <int KIND, int BN, int MT>
static int qgemm_launch_tile(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, int64_t m,
                             int64_t n, int64_t kbytes, const QEpilogue& ep, uint32_t* status, cudaStream_t st) {
  using Cfg = QCfg<KIND, BN, MT>;
  const int64_t mtiles = (m + kQM * MT - 1) / (kQM * MT), ntiles = (n + BN - 1) / BN;
  if (ntiles > 65535) return B200Q_ERR_UNSUPPORTED;
  CUtensorMap map_a, map_b;
  if (!make_byte_map(&map_a, a, m, kbytes, kQM) || !make_byte_map(&map_b, b, n, kbytes, BN)) return B200Q_ERR_CUDA;
  const int num_k_blocks = static_cast<int>((kbytes + kQKBytes - 1) / kQKBytes);
  const size_t smem = Cfg::kStages * Cfg::kStageBytes + sizeof(QGemmSmem) + 1024;
  if (cudaFuncSetAttribute(qgemm_kernel<KIND, BN, MT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return B200Q_ERR_CUDA;
  dim3 grid(static_cast<unsigned>(mtiles), static_cast<unsigned>(ntiles));
  qgemm_kernel<KIND, BN, MT, false><<<grid, Cfg::kThreads, smem, st>>>(map_a, map_b, sfa, sfb, m, n, num_k_blocks, ep,
                                                                       status);
  return launch_status();
}

// 128 x 128 tiles with the K extent shared by the two CTAs of a cluster
template <int KIND>
static int qgemm_launch_ksplit(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, int64_t m,
                               int64_t n, int64_t kbytes, const QEpilogue& ep, uint32_t* status, cudaStream_t st) {
  using Cfg = QCfg<KIND, 128, 1>;
  const int64_t mtiles = (m + kQM - 1) / kQM, ntiles = (n + 127) / 128;
  if (ntiles > 65535) return B200Q_ERR_UNSUPPORTED;
  CUtensorMap map_a, map_b;
  if (!make_byte_map(&map_a, a, m, kbytes, kQM) || !make_byte_map(&map_b, b, n, kbytes, 128)) return B200Q_ERR_CUDA;
  const int num_k_blocks = static_cast<int>((kbytes + kQKBytes - 1) / kQKBytes);
  const size_t smem = Cfg::kStages * Cfg::kStageBytes + sizeof(QGemmSmem) + 1024;
  auto kern = qgemm_kernel<KIND, 128, 1, true>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return B200Q_ERR_CUDA;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(mtiles), static_cast<unsigned>(ntiles), 2);
  cfg.blockDim = dim3(Cfg::kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 2;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kern, map_a, map_b, sfa, sfb, m, n, num_k_blocks, ep, status) != cudaSuccess) {
    cudaGetLastError();
    return B200Q_ERR_CUDA;
  }
  return launch_status();
}

// Tile choice, from measurements on 70B-shape problems.  FP8: 256 x 256 per CTA when that still
// gives every SM two tiles or more, else 128 x 256 while 0.4 tiles per SM or more remain, else
// 128 x 128 on two CTAs per SM.  NVFP4: 128 x 256 under the same condition, else 128 x 128;
// 256 x 192 (384 accumulator columns + the block scales, scale copies by tcgen05.cp) is kept for
// the override: b200q_qgemm_tile_override(128 | 256 (128 x 256) | 512 ("big") | 2 (128 x 128 with
// the K extent shared by a cluster of two CTAs)) forces one for every later launch of the process,
// 0 returns to the automatic choice.
static int g_qgemm_tile_override = 0;
template <int KIND>
static int qgemm_launch(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, int64_t m,
                        int64_t n, int64_t kbytes, const QEpilogue& ep, uint32_t* status, cudaStream_t st) {
  constexpr int kBigN = KIND == kQNvfp4 ? 192 : 256;
  const int64_t sms = sm_count_cached();
  const int64_t mt128 = (m + 127) / 128, big_tiles = ((m + 255) / 256) * ((n + kBigN - 1) / kBigN);
  int choice = 128;
  if (KIND == kQFp8) {
    if (mt128 * ((n + 255) / 256) * 10 >= sms * 4) choice = 256;
    if (m > 128 && big_tiles >= 2 * sms) choice = 512;
  } else if (mt128 * ((n + 255) / 256) * 10 >= sms * 4) {
    choice = 256;
  }
  // no more 128 x 128 tiles than SMs and a long K (80 blocks of 128 bytes or more, from measurements on
  // 128..512 x 4096..8192 x 8192..28672): two CTAs per tile, each summing half of K
  const int64_t kblocks = (kbytes + kQKBytes - 1) / kQKBytes;
  bool ksplit = mt128 * ((n + 127) / 128) <= sms && kblocks >= 80;
  if (const int forced = g_qgemm_tile_override) {
    ksplit = forced == 2 && kblocks >= 2;
    if (forced == 128 || forced == 256 || forced == 512) choice = forced;
  }
  if (ksplit) return qgemm_launch_ksplit<KIND>(a, b, sfa, sfb, m, n, kbytes, ep, status, st);
  if (choice == 512) return qgemm_launch_tile<KIND, kBigN, 2>(a, b, sfa, sfb, m, n, kbytes, ep, status, st);
  if (choice == 256) return qgemm_launch_tile<KIND, 256, 1>(a, b, sfa, sfb, m, n, kbytes, ep, status, st);
  return qgemm_launch_tile<KIND, 128, 1>(a, b, sfa, sfb, m, n, kbytes, ep, status, st);
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_qgemm_tile_override(int tile) {
  const int before = g_qgemm_tile_override;
  if (tile == 0 || tile == 2 || tile == 128 || tile == 256 || tile == 512) g_qgemm_tile_override = tile;
  return before;
}

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
