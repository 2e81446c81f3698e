// awq_lite search, all candidates of one layer and one batch in ONE persistent launch:
//
//   loss[a] += sum_{m,n} float( bf16( bf16( sum_k A[a][m,k] * fq_a(W)[n,k] ) - R[m,n] ) )^2
//   fq_a(W)[n, :] = per-128 block dynamic integer fake quant of bf16(W[n, :] * s[a][:])
//
// A[a] = the activations already divided by candidate a's scale ([n_alpha * M, K] bf16), W the raw
// weight [N, K], s[a] the candidate's per-input-channel scale in bf16, R the unquantised layer output.
// Neither the scaled, fake-quantised weight nor the product ever reaches global memory.
//
// Work item = (candidate, 512-row slab of A, 256-column slab of W), handed round-robin to CTA pairs
// (clusters of two CTAs, one per SM).  A pair keeps the whole 512 x 256 fp32 accumulator in tensor
// memory (each CTA: its 2 x 128 rows x 256 columns = all 512 TMEM columns) and runs M = 256
// tcgen05.mma.cta_group::2 instructions: each CTA loads only ITS 128 rows of every A tile and ITS
// half (128 rows) of the W slab, so per FLOP a CTA asks L2 for a quarter less than a 256 x 256
// single-CTA tile and the W slab is fetched exactly once per candidate.
//
// Warps of a CTA (32; a warp's scheduler is its index modulo 4):
//   0      MMA issuer (even CTA only) and TMEM allocation           } scheduler 0 carries no transform warp, so
//   8      A producer: TMA 128 x 64 tiles into a 3-deep ring,       } these latency-critical threads do not
//          completion counted on the EVEN CTA's barrier             } queue for issue slots behind arithmetic
//   12     W producer: TMA raw 128 x 128 weight units (two swizzled }
//          128 x 64 boxes) and the unit's 128 scale factors into a 4-deep ring
//   4-7, 16-19   epilogue (two warps per TMEM lane quarter): tcgen05.ld the accumulator, squared error
//          against R, one atomic per warp and item.  R's tile for the item (this CTA's rows, 256 columns)
//          is sent by the A producer through the A ring after the item's last A tile, as four 64-column
//          pieces; the MMA issuer skips those stages and the epilogue hands them back
//   1-3, 9-11, 13-15, 21-23, 25-27, 29-31   transform (eighteen warps), in shared memory, in place.  A W unit is sixteen
//          warp-sized tasks of eight rows, taken round-robin across unit boundaries; a lane owns 32
//          consecutive elements of one weight row (four lanes = one 128-block): bf16(W * s), the block
//          abs-max (two shuffles), the integer fake quant, stored back where they came from in the
//          swizzled layout the tensor core reads; then a proxy fence (generic -> async) and an arrival
//          on the even CTA's "unit ready" barrier.
// The MMA thread waits for "A tile landed in both CTAs" and "W unit transformed in both CTAs", issues
// 2 x 4 MMAs per 64-wide K slice, and releases ring slots to both CTAs with tcgen05.commit.  The A
// producer and the transformers run ahead into the next item while the epilogue drains the
// accumulator.  Where few activations are being read at a time, every pair starts its K loop at a different
// offset, so that the pairs, which all read the same activations, do not ask L2 for the same lines at the
// same moment.
//
// Every wait is bounded: when one runs out, an error bit is set in the caller's status word, the CTA
// stops waiting anywhere else, and the kernel ends through its normal exit (TMEM released).
#include "umma.cuh"

// Measurement switches (0 in the library; set when building a throw-away copy to find which stage
// bounds the pipeline): 1 = the transform only waits, fences and arrives; 2 = the epilogue only reads
// the accumulator; 4 = A tiles are loaded for the first ring fill only; 8 = the same for W units.
// B200Q_FUSED_ROTATE 0 starts every pair's K loop at slice 0.
#ifndef B200Q_FUSED_ABLATE
#define B200Q_FUSED_ABLATE 0
#endif
#ifndef B200Q_FUSED_ROTATE
#define B200Q_FUSED_ROTATE 1
#endif

namespace b200q {

constexpr int kFK = 64;                                  // K elements of one A stage: one 128-byte swizzle row
constexpr uint32_t kFTileBytes = 128 * kFK * 2;          // 128 rows x 64 bf16 = 16 KB: one TMA box
constexpr uint32_t kFUnitBytes = 2 * kFTileBytes;        // a W unit: 128 rows x 128 K = two boxes
constexpr int kFPairN = 256;                             // columns of a pair's tile (128 weight rows per CTA)
#ifndef B200Q_FUSED_WUNITS
#define B200Q_FUSED_WUNITS 4
#endif
// W unit slots (landing, being transformed, waiting, being read by the MMAs).  Measured on the 21-candidate
// search of 512 x 14336 x 4096, with the rest of the 227 KB as activation stages: 2 units + 5 stages 1.64 ms,
// 3 + 4 1.09, 4 + 3 1.06, 5 + 2 1.15.
constexpr int kFWUnits = B200Q_FUSED_WUNITS;
constexpr uint32_t kFScaleBytes = 128 * 2;     // one unit's share of a candidate's scale vector
#ifndef B200Q_FUSED_THREADS
#define B200Q_FUSED_THREADS 1024
#endif
constexpr int kFThreads = B200Q_FUSED_THREADS;           // whole groups of four warps; 1024 (64 registers) measured 2-3 % faster than 768
// Warp roles.  A warp's scheduler is its index modulo 4.  Scheduler 0 hosts the latency-critical MMA
// issuer and the A producer and no transform warp, so that neither has to compete for issue slots
// with the arithmetic; the transform warps are the other three of every group of four except the two
// epilogue groups (warps 4-7 and 16-19).
constexpr int kFWarpMma = 0, kFWarpAProducer = 8, kFWarpWProducer = 12;
// three transform warps in every group of four warps except the two epilogue groups
constexpr int kFTransformCount = (kFThreads / 128 - 2) * 3;
constexpr int kFOctets = 16;                             // row octets (warp-sized tasks) per W unit
constexpr int kFEpilogueWarps = 8;       // two per TMEM lane quarter (warps 4-7 and 16-19), alternate column chunks
constexpr int kFMaxStages = 10;
constexpr int kFRefPieces = kFPairN / kFK;   // the reference tile of an item travels as four 64-column pieces

template <int MT> struct FusedCfg {
  // what the transformed-weight ring leaves of the 227 KB goes to the activation ring
  static constexpr int kAStages = (7 - kFWUnits) * 2 / MT;
  static constexpr uint32_t kAStageBytes = MT * kFTileBytes;
  static constexpr uint32_t kRingBytes = kAStages * kAStageBytes + kFWUnits * (kFUnitBytes + kFScaleBytes);
  static constexpr uint32_t kTmemCols = MT * kFPairN;    // 512 or 256: a power of two
  // D fp32, A and B bf16, both K-major, N = 256, M = 256 across the pair
  static constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kFPairN >> 3) << 17) | ((256u >> 4) << 24);
};

enum : uint32_t {
  kFErrAProducer = 0x100, kFErrWProducer = 0x200, kFErrMma = 0x400, kFErrTransform = 0x800, kFErrEpilogue = 0x1000
};

struct FusedSmem {
  uint64_t a_full[kFMaxStages];    // even CTA's copy is the one in use: both CTAs' tiles count on it
  uint64_t a_empty[kFMaxStages];
  uint64_t w_full[kFWUnits];       // raw unit and its scale factors landed (each CTA its own)
  uint64_t b_ready[kFWUnits];      // unit transformed in both CTAs (even CTA's copy)
  uint64_t b_empty[kFWUnits];
  uint64_t acc_full;               // all MMAs of an item complete
  uint64_t acc_empty;              // accumulator read out in both CTAs (even CTA's copy)
  uint64_t r_full[kFRefPieces];    // a piece of the item's reference tile landed (each CTA its own)
  uint32_t r_readers[kFRefPieces]; // epilogue warps that are done with the piece
  uint32_t tmem_base;
  uint32_t abort;
};

// packed fp32x2 arithmetic, each instruction rounded on its own (never contracted)
__device__ __forceinline__ uint64_t f32x2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t f32x2_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f32x2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t f32x2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct FusedItem {
  int alpha, slab_m, slab_n;
};
// item -> (candidate, row slab, column slab); candidates outermost so that the pairs working at the same
// time share one candidate's A in L2
__device__ __forceinline__ FusedItem fused_item(int item, int slabs_m, int slabs_n) {
  FusedItem it;
  const int per_alpha = slabs_m * slabs_n;
  it.alpha = item / per_alpha;
  const int r = item - it.alpha * per_alpha;
  it.slab_m = r / slabs_n;
  it.slab_n = r - it.slab_m * slabs_n;
  return it;
}

template <int MT>
__global__ void __launch_bounds__(kFThreads, 1)
awq_fused_search_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                        const __grid_constant__ CUtensorMap map_r,
                        const __nv_bfloat16* __restrict__ s_all, const __nv_bfloat16* __restrict__ ref,
                        double* __restrict__ loss, float* __restrict__ c_out, int n_alpha, int M, int N, int K,
                        IntQ q, float one, uint32_t* __restrict__ status) {
  using Cfg = FusedCfg<MT>;
  constexpr int SA = Cfg::kAStages, SW = kFWUnits;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* ring_a = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring_w = ring_a + SA * Cfg::kAStageBytes;
  uint8_t* ring_s = ring_w + SW * kFUnitBytes;       // the 128 scale factors of each W unit (256 bytes per slot)
  FusedSmem* sm = reinterpret_cast<FusedSmem*>(ring_s + SW * kFScaleBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // no scale vectors: the weight operand holds every candidate's weight already scaled and fake-quantised
  // (n_alpha * N rows); the transform warps then only hand the landed units on to the MMA issuer
  const bool prequant = s_all == nullptr;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int slab_rows = 256 * MT;
  const int slabs_m = (M + slab_rows - 1) / slab_rows, slabs_n = (N + kFPairN - 1) / kFPairN;
  const int num_items = n_alpha * slabs_m * slabs_n;
  const int k_slices = K / kFK;                      // K is a multiple of 128: an even count
  const int k_units = k_slices / 2;
  // this pair's K loop starts at unit `rot` and wraps around when the activations that the pairs working at the same time read are few (the pairs of one candidate all
  // read the same rows: starting apart keeps them off the same L2 lines at the same moment).  When they are
  // many (long K, few column slabs per candidate) starting together is what keeps a tile in L2 until every
  // pair of its candidate has read it: 512 x 4096 x 14336, 21 candidates, 1.11 ms rotated, 1.03 ms not.
  const bool rotate = B200Q_FUSED_ROTATE && static_cast<int64_t>(num_pairs) * M * K * 2 <=
                                                static_cast<int64_t>(slabs_m) * slabs_n * (16ll << 20);
  const int rot = rotate ? static_cast<int>((static_cast<int64_t>(pair) * k_units) / num_pairs) % k_units : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SA; ++s) { mbar_init(&sm->a_full[s], 1); mbar_init(&sm->a_empty[s], 1); }
    for (int u = 0; u < SW; ++u) {
      mbar_init(&sm->w_full[u], 1);
      mbar_init(&sm->b_ready[u], 2 * kFOctets);   // one arrival per warp-sized task of the unit, both CTAs
      mbar_init(&sm->b_empty[u], 1);
    }
    mbar_init(&sm->acc_full, 1);
    mbar_init(&sm->acc_empty, 2 * kFEpilogueWarps);
    for (int j = 0; j < kFRefPieces; ++j) { mbar_init(&sm->r_full[j], 1); sm->r_readers[j] = 0; }
    sm->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kFWarpMma) {   // the same warp of both CTAs: one allocation for the pair
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)), "r"(Cfg::kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_barrier();   // the peer's barriers are initialised before anything signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&sm->tmem_base);

  if (warp == kFWarpAProducer) {
    // ---------------------------------------------------------------- A producer --------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int item = pair; item < num_items && ok; item += num_pairs) {
        const FusedItem w = fused_item(item, slabs_m, slabs_n);
        // rows of this CTA in 256-row tile t of the slab: alpha * M + slab_m * slab_rows + t * 256 + rank * 128
        const int row0 = w.alpha * M + w.slab_m * slab_rows + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < k_slices; ++kb, ++it) {
          const int s = it % SA;
          ok = mbar_wait_bounded(&sm->a_empty[s], ((it / SA) & 1) ^ 1, &sm->abort, status, kFErrAProducer);
          if (!ok) break;
          if ((B200Q_FUSED_ABLATE & 4) && it >= static_cast<uint32_t>(SA)) continue;
          const uint32_t full_leader = map_to_cta(&sm->a_full[s], 0);
          if (leader) mbar_expect_tx(&sm->a_full[s], 2 * Cfg::kAStageBytes);      // both CTAs' tiles
          uint8_t* dst = ring_a + s * Cfg::kAStageBytes;
          int kr = kb + 2 * rot;
          kr -= kr >= k_slices ? k_slices : 0;
#pragma unroll
          for (int t = 0; t < MT; ++t) tma_load_2d_pair(dst + t * kFTileBytes, &map_a, full_leader, kr * kFK, row0 + t * 256);
        }
        // The item's reference tile (this CTA's rows, 256 columns) follows its last A tile through the same
        // ring, one 64-column piece per stage: the epilogue then reads it from shared memory instead of
        // waiting for L2 sixteen times while the tensor cores stand still.  These stages are not the MMA
        // issuer's: it skips them, and the epilogue hands them back.  The even CTA's "A landed" barrier
        // still gets its arrival (no bytes), so that its phases keep counting the uses of the stage.
        const int ref_row0 = w.slab_m * slab_rows + static_cast<int>(rank) * 128;
        for (int j = 0; j < kFRefPieces && ok; ++j, ++it) {
          const int s = it % SA;
          ok = mbar_wait_bounded(&sm->a_empty[s], ((it / SA) & 1) ^ 1, &sm->abort, status, kFErrAProducer);
          if (!ok) break;
          if (leader) mbar_expect_tx(&sm->a_full[s], 0);
          mbar_expect_tx(&sm->r_full[j], Cfg::kAStageBytes);
          uint8_t* dst = ring_a + s * Cfg::kAStageBytes;
#pragma unroll
          for (int t = 0; t < MT; ++t)
            tma_load_2d(dst + t * kFTileBytes, &map_r, &sm->r_full[j], w.slab_n * kFPairN + j * kFK, ref_row0 + t * 256);
        }
      }
    }
  } else if (warp == kFWarpWProducer) {
    // ---------------------------------------------------------------- W producer --------------
    if (lane == 0) {
      uint32_t wu = 0;
      bool ok = true;
      for (int item = pair; item < num_items && ok; item += num_pairs) {
        const FusedItem w = fused_item(item, slabs_m, slabs_n);
        // pre-quantised weights: candidate a's weight is rows [a * N, (a + 1) * N) of the operand
        const int n_row = (prequant ? w.alpha * N : 0) + w.slab_n * kFPairN + static_cast<int>(rank) * 128;
        const __nv_bfloat16* s_row = prequant ? nullptr : s_all + static_cast<int64_t>(w.alpha) * K;
        for (int ub = 0; ub < k_units; ++ub, ++wu) {
          const int u = wu % SW;
          ok = mbar_wait_bounded(&sm->b_empty[u], ((wu / SW) & 1) ^ 1, &sm->abort, status, kFErrWProducer);
          if (!ok) break;
          int ur = ub + rot;
          ur -= ur >= k_units ? k_units : 0;
          uint8_t* dst = ring_w + u * kFUnitBytes;
          mbar_expect_tx(&sm->w_full[u], kFUnitBytes + (prequant ? 0u : kFScaleBytes));
          if (!prequant) bulk_load(ring_s + u * kFScaleBytes, s_row + ur * 128, kFScaleBytes, &sm->w_full[u]);
          tma_load_2d(dst, &map_w, &sm->w_full[u], ur * 128, n_row);
          tma_load_2d(dst + kFTileBytes, &map_w, &sm->w_full[u], ur * 128 + kFK, n_row);
        }
      }
    }
  } else if (warp == kFWarpMma) {
    // ---------------------------------------------------------------- MMA issuer --------------
    if (lane == 0 && leader) {
      uint32_t it = 0, wu = 0, done = 0;
      bool ok = true;
      // a barrier of the odd CTA sits at the same offset of its shared memory: one address difference
      const uint32_t peer_delta = map_to_cta(sm, 1) - smem_u32(sm);
      auto commit_both = [&](uint64_t* bar) {   // arrives in both CTAs once the MMAs issued so far have completed
        const uint32_t a = smem_u32(bar);
        umma_commit_pair(a);
        umma_commit_pair(a + peer_delta);
      };
      for (int item = pair; item < num_items && ok; item += num_pairs, ++done) {
        if (done > 0) {   // the previous item's accumulator has been read out in both CTAs
          ok = mbar_wait_bounded_cluster(&sm->acc_empty, (done - 1) & 1, &sm->abort, status, kFErrMma);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        for (int ub = 0; ub < k_units && ok; ++ub, ++wu) {
          const int u = wu % SW;
          ok = mbar_wait_bounded_cluster(&sm->b_ready[u], (wu / SW) & 1, &sm->abort, status, kFErrMma);
          if (!ok) break;
          const uint64_t db0 = umma_desc(smem_u32(ring_w + u * kFUnitBytes));
#pragma unroll
          for (int half = 0; half < 2; ++half, ++it) {   // the unit's two 64-wide K slices
            const int s = it % SA;
            ok = mbar_wait_bounded(&sm->a_full[s], (it / SA) & 1, &sm->abort, status, kFErrMma);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da0 = umma_desc(smem_u32(ring_a + s * Cfg::kAStageBytes));
            const uint64_t db = db0 + half * (kFTileBytes >> 4);
#pragma unroll
            for (int t = 0; t < MT; ++t) {
#pragma unroll
              for (int k = 0; k < kFK / 16; ++k)   // 16 bf16 = 32 bytes along K inside the swizzled row: +2 in 16-byte units
                umma_bf16_pair(tmem + t * kFPairN, da0 + t * (kFTileBytes >> 4) + 2 * k, db + 2 * k, Cfg::kIdesc,
                               (ub | half | k) != 0 ? 1u : 0u);
            }
            commit_both(&sm->a_empty[s]);   // the stage is free in both CTAs once these MMAs have read it
          }
          if (!ok) break;
          commit_both(&sm->b_empty[u]);
        }
        if (!ok) break;
        commit_both(&sm->acc_full);   // fires when every MMA issued above has completed
        it += kFRefPieces;            // the stages that carry the item's reference tile to the epilogue
      }
    }
  } else if ((warp & 3) != 0 && (warp >> 2) != 1 && (warp >> 2) != 4) {
    // ---------------------------------------------------------------- transform ---------------
    // A W unit (128 rows x 128 K) is sixteen warp-sized tasks of eight rows; the transform warps
    // take tasks round-robin across unit boundaries, so at any moment they are spread over two or three
    // units and over all phases of a task (waiting for the unit to land, arithmetic, the fence).
    // Lane -> quarter qd = lane >> 3 of the 128-block of one row; the eight lanes of a quarter-warp store
    // to eight consecutive rows, i.e. eight different 16-byte positions of the 128-byte swizzle pattern
    // (chunk j of row r sits at j ^ (r & 7)): conflict-free.
    //
    // Arithmetic, per block: v = bf16(w * s); amax = max |v|; scale = 7 / amax; out = bf16(k / scale) with
    // k = rint(v * scale).  Because the abs-max is the block's own, |v * scale| <= 7 (1 + 2^-24) and the
    // clamp to [-8, 7] never acts.  k / scale takes only 15 values per block, so instead of one exact
    // division per element the four lanes of a block check once, for k = 1..7, that bf16(k * y) with
    // y = RN(1 / scale) equals bf16(RN(k / scale)) (it does except when k * y falls within a rounding
    // error of a bf16 tie) and then multiply; a block that fails the check, a dead or out-of-range
    // scale, or a bit width other than 4 takes the element-wise exact path.  Zeros come out as +0
    // where the stand-alone kernel keeps the sign: the product does not see the difference.
    const int wq = warp >> 2;                                           // 0, 2, 3 or 5
    const int t_id = (wq - (wq >= 2 ? 1 : 0) - (wq >= 5 ? 1 : 0)) * 3 + (warp & 3) - 1;   // 0 .. 11
    const int qd = lane >> 3, r_in = lane & 7;
    const int j0 = (qd & 1) * 4;                                        // first 16-byte chunk in the 64-wide box
    const bool four_bit = q.bound == 7.f && q.lo == -8.f;
    const uint32_t my_items = static_cast<uint32_t>((num_items - pair + num_pairs - 1) / num_pairs);
    const uint32_t units_total = my_items * static_cast<uint32_t>(k_units);
    const uint32_t tasks_total = units_total * kFOctets;
    bool ok = true;
    for (uint32_t task = t_id; task < tasks_total && ok; task += kFTransformCount) {
      const uint32_t wu = task / kFOctets;
      const int u = wu % SW;
      // the raw unit has landed: every lane observes the completed phase itself, and only when it is
      // not there yet does lane 0 poll
      const uint32_t parity = (wu / SW) & 1;
      bool landed = __all_sync(0xffffffffu, mbar_try(&sm->w_full[u], parity));
      if (!landed) {
        landed = lane != 0 || mbar_wait_bounded(&sm->w_full[u], parity, &sm->abort, status, kFErrTransform);
        landed = __all_sync(0xffffffffu, landed) && __all_sync(0xffffffffu, mbar_try(&sm->w_full[u], parity));
      }
      ok = landed;
      if (!ok) break;
      const int row = static_cast<int>(task % kFOctets) * 8 + r_in, sw = row & 7;
      uint8_t* dst = ring_w + u * kFUnitBytes + (qd >> 1) * kFTileBytes + row * 128;
      if (prequant) {      // the unit was written by the async proxy and is read by it: nothing to fence
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(map_to_cta(&sm->b_ready[u], 0));
        continue;
      }
      uint32_t pr[16];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const uint4 v = *reinterpret_cast<const uint4*>(dst + (((j0 + jj) ^ sw) << 4));
        pr[4 * jj] = v.x; pr[4 * jj + 1] = v.y; pr[4 * jj + 2] = v.z; pr[4 * jj + 3] = v.w;
      }
      if (!(B200Q_FUSED_ABLATE & 1)) {
        // this lane's 32 scale factors (the eight lanes of a quarter read the same 64 bytes: broadcast)
        const uint4* sp = reinterpret_cast<const uint4*>(ring_s + u * kFScaleBytes + qd * 64);
        uint32_t mx[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 sv = sp[j];
          const uint32_t ss[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            // packed bf16 multiply = the product rounded to bf16, two elements per instruction
            const __nv_bfloat162 p2 = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&pr[4 * j + i]),
                                              *reinterpret_cast<const __nv_bfloat162*>(&ss[i]));
            pr[4 * j + i] = *reinterpret_cast<const uint32_t*>(&p2);
            mx[i] = __vmaxu2(mx[i], pr[4 * j + i] & 0x7fff7fffu);   // |x| patterns: integer order = magnitude order
          }
        }
        const uint32_t m2 = __vmaxu2(__vmaxu2(mx[0], mx[1]), __vmaxu2(mx[2], mx[3]));
        uint32_t bits = max(m2 & 0xffffu, m2 >> 16) << 16;
        bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, 8));
        bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, 16));
        const IntScale sc = make_int_scale(q, __uint_as_float(bits));
        // this lane's share of the check: k = 2 qd + 1 and 2 qd + 2 (7 twice in the last quarter); done by
        // every lane (a few instructions) so that the shuffles are warp-wide instructions
        const float2 y2 = make_float2(sc.y, sc.y);
        const float ka = static_cast<float>(2 * qd + 1);
        const float2 k2 = make_float2(ka, qd == 3 ? 7.f : ka + 1.f);
        const float2 e2 = div2_rn_rcp(k2, make_float2(-sc.scale, -sc.scale), y2), f2 = __fmul2_rn(k2, y2);
        uint32_t same = Elem<__nv_bfloat16>::pack2(e2.x, e2.y) == Elem<__nv_bfloat16>::pack2(f2.x, f2.y) ? 1u : 0u;
        same &= __shfl_xor_sync(0xffffffffu, same, 8);
        same &= __shfl_xor_sync(0xffffffffu, same, 16);
        // the four lanes of a block agree: same scale, all four checks
        if (four_bit && sc.live && sc.fast && same) {
          // The product is rounded to fp32 BEFORE it is rounded to an integer, as the reference does (a
          // block's own ties, e.g. v / amax = 13 / 14, sit exactly on .5 only after that first rounding).
          const uint64_t scale_p = f32x2_pack(sc.scale, sc.scale), y_p = f32x2_pack(sc.y, sc.y);
          // rint(t) = (t + 1.5 * 2^23) - 1.5 * 2^23, the first sum written as fma(t, one, magic) with `one`
          // = 1.0f arriving as a kernel parameter: the assembler fuses a multiply with a following add
          // even when both carry an explicit rounding mode (observed: ties moved), which would round
          // the exact product instead of t; it cannot fuse a multiply into an existing multiply-add
          const uint64_t one_p = f32x2_pack(one, one), magic = f32x2_pack(12582912.f, 12582912.f),
                         nmagic = f32x2_pack(-12582912.f, -12582912.f);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const uint64_t t2 = f32x2_mul(f32x2_pack(__uint_as_float(pr[i] << 16), __uint_as_float(pr[i] & 0xffff0000u)), scale_p);
            const uint64_t r2 = f32x2_add(f32x2_fma(t2, one_p, magic), nmagic);
            const uint64_t o2 = f32x2_mul(r2, y_p);
            pr[i] = Elem<__nv_bfloat16>::pack2(__uint_as_float(static_cast<uint32_t>(o2)),
                                               __uint_as_float(static_cast<uint32_t>(o2 >> 32)));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float lo = intq_apply(__uint_as_float(pr[i] << 16), sc, q);
            const float hi = intq_apply(__uint_as_float(pr[i] & 0xffff0000u), sc, q);
            pr[i] = Elem<__nv_bfloat16>::pack2(lo, hi);
          }
        }
      }
#pragma unroll
      for (int jj = 0; jj < 4; ++jj)
        *reinterpret_cast<uint4*>(dst + (((j0 + jj) ^ sw) << 4)) =
            make_uint4(pr[4 * jj], pr[4 * jj + 1], pr[4 * jj + 2], pr[4 * jj + 3]);
      fence_async_shared();     // these stores are read next by the tensor cores of both CTAs
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(map_to_cta(&sm->b_ready[u], 0));
    }
  } else if ((warp >> 2) == 1 || (warp >> 2) == 4) {
    // ---------------------------------------------------------------- epilogue ----------------
    const int quarter = warp & 3;        // TMEM lanes quarter * 32 .. + 31 are the rows this warp may read
    const int second = warp >= 16 ? 1 : 0;   // which of the quarter's two warps: it takes the odd chunks
    const uint32_t acc_empty_leader = map_to_cta(&sm->acc_empty, 0);
    uint32_t done = 0;
    bool ok = true;
    for (int item = pair; item < num_items && ok; item += num_pairs, ++done) {
      const FusedItem w = fused_item(item, slabs_m, slabs_n);
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(&sm->acc_full, done & 1, &sm->abort, status, kFErrEpilogue));
      if (!ok) break;                     // warp-uniform: the TMEM loads below are warp-wide
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float sq = 0.f;
      // 16-column chunks of this lane's rows, piece by piece of the reference tile as the pieces land in
      // the A ring (rows of 128 bytes, 16-byte unit u of row r at position u ^ (r & 7)); the quarter's two
      // warps take alternate chunks
      const int chunks_n = min(kFPairN, N - w.slab_n * kFPairN) / 16;          // warp-uniform (N % 32 == 0)
      const int r_in = quarter * 32 + lane;                                     // this lane's row within a 128-row box
      const uint32_t first_use = done * static_cast<uint32_t>(k_slices + kFRefPieces) + static_cast<uint32_t>(k_slices);
      for (int j = 0; j < kFRefPieces && ok; ++j) {
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&sm->r_full[j], done & 1, &sm->abort, status, kFErrEpilogue));
        if (!ok) break;
        const int s = static_cast<int>((first_use + j) % SA);
        const uint8_t* piece = ring_a + s * Cfg::kAStageBytes + r_in * 128;
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          const int row = w.slab_m * slab_rows + t * 256 + static_cast<int>(rank) * 128 + r_in;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int cp = 2 * c + second;                  // chunk within the piece: 16-byte units 2 cp, 2 cp + 1
            const int cc = j * (kFK / 16) + cp;
            if (cc >= chunks_n) continue;                   // warp-uniform
            uint32_t acc[16];
            tmem_ld16(tmem + (static_cast<uint32_t>(quarter * 32) << 16) + t * kFPairN + cc * 16, acc);
            if (row < M && !(B200Q_FUSED_ABLATE & 2)) {
              const uint8_t* src = piece + t * kFTileBytes;
              const uint4 r0 = *reinterpret_cast<const uint4*>(src + (((2 * cp) ^ (r_in & 7)) << 4));
              const uint4 r1 = *reinterpret_cast<const uint4*>(src + (((2 * cp + 1) ^ (r_in & 7)) << 4));
              // bf16(bf16(acc) - ref) two elements at a time: the packed bf16 subtraction rounds the exact
              // difference once, which is what rounding the fp32 difference of two bf16 values gives
              const uint32_t rr[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const uint32_t o2 = Elem<__nv_bfloat16>::pack2(__uint_as_float(acc[2 * i]), __uint_as_float(acc[2 * i + 1]));
                const __nv_bfloat162 d2 = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&o2),
                                                  *reinterpret_cast<const __nv_bfloat162*>(&rr[i]));
                const uint32_t db = *reinterpret_cast<const uint32_t*>(&d2);
                const float d_lo = __uint_as_float(db << 16), d_hi = __uint_as_float(db & 0xffff0000u);
                sq = fmaf(d_lo, d_lo, sq);
                sq = fmaf(d_hi, d_hi, sq);
              }
              if (c_out) {
                float* cp_out = c_out + (static_cast<int64_t>(w.alpha) * M + row) * N + w.slab_n * kFPairN + cc * 16;
#pragma unroll
                for (int i = 0; i < 16; ++i) cp_out[i] = __uint_as_float(acc[i]);
              }
            }
          }
        }
        // the last of this CTA's eight epilogue warps to finish the piece gives the stage back to the A producer
        __syncwarp();
        if (lane == 0 && atomicAdd(&sm->r_readers[j], 1u) == kFEpilogueWarps - 1) {
          sm->r_readers[j] = 0;
          mbar_arrive_remote(map_to_cta(&sm->a_empty[s], rank));
        }
      }
      if (!ok) break;
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(acc_empty_leader);   // the accumulator may be overwritten
      for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if (lane == 0) atomicAdd(loss + w.alpha, static_cast<double>(sq));
    }
  }

  grace_after_abort(&sm->abort);
  __syncwarp();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_barrier();   // neither CTA leaves (or frees the pair's TMEM) while the other still works
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (warp == kFWarpMma) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(Cfg::kTmemCols));
  }
}

// 2-D bf16 tensor [rows, k] with k contiguous; boxes of 64 x 128, 128-byte swizzle
static bool fused_make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kFK), 128u};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int MT>
static int fused_launch(const CUtensorMap& map_a, const CUtensorMap& map_w, const CUtensorMap& map_r, const __nv_bfloat16* s_all,
                        const __nv_bfloat16* ref, double* loss, float* c_out, int n_alpha, int m, int n, int k,
                        IntQ q, uint32_t* status, int64_t items, cudaStream_t st) {
  using Cfg = FusedCfg<MT>;
  const size_t smem = Cfg::kRingBytes + sizeof(FusedSmem) + 1024;
  auto kern = awq_fused_search_kernel<MT>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) {
    cudaGetLastError();
    return B200Q_ERR_CUDA;
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.blockDim = dim3(kFThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  // one pair per two SMs that can hold a cluster at the same time (asked once per device and MT)
  static int pairs_cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200Q_ERR_CUDA;
  if (pairs_cached[dev] == 0) {
    int clusters = 0;
    cfg.gridDim = dim3(static_cast<unsigned>(sm_count_cached() / 2 * 2));
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      clusters = sm_count_cached() / 2;
    }
    pairs_cached[dev] = clusters;
  }
  const int64_t pairs = items < pairs_cached[dev] ? items : pairs_cached[dev];
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
  if (cudaLaunchKernelEx(&cfg, kern, map_a, map_w, map_r, s_all, ref, loss, c_out, n_alpha, m, n, k, q, 1.0f, status) != cudaSuccess) {
    cudaGetLastError();
    return B200Q_ERR_CUDA;
  }
  return launch_status();
}

}  // namespace b200q

using namespace b200q;

static int fused_entry(const void* a_all, const void* w, int64_t w_rows, const void* s_all, const void* ref,
                       int n_alpha, int64_t m, int64_t n, int64_t k, IntQ q, double* loss_io, float* c_out,
                       uint32_t* status_io, void* stream) {
  if (n_alpha * m > (1ll << 30) || w_rows > (1ll << 30) || k > (1ll << 30)) return B200Q_ERR_UNSUPPORTED;
  const int mt = m > 256 ? 2 : 1;
  const int64_t slabs_m = (m + 256 * mt - 1) / (256 * mt), slabs_n = (n + kFPairN - 1) / kFPairN;
  const int64_t items = n_alpha * slabs_m * slabs_n;
  if (items > (1ll << 30)) return B200Q_ERR_UNSUPPORTED;
  CUtensorMap map_a, map_w, map_r;
  if (!fused_make_map(&map_a, a_all, static_cast<int64_t>(n_alpha) * m, k) || !fused_make_map(&map_w, w, w_rows, k) ||
      !fused_make_map(&map_r, ref, m, n))
    return B200Q_ERR_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* sp = static_cast<const __nv_bfloat16*>(s_all);
  const __nv_bfloat16* rp = static_cast<const __nv_bfloat16*>(ref);
  if (mt == 2)
    return fused_launch<2>(map_a, map_w, map_r, sp, rp, loss_io, c_out, n_alpha, static_cast<int>(m), static_cast<int>(n),
                           static_cast<int>(k), q, status_io, items, st);
  return fused_launch<1>(map_a, map_w, map_r, sp, rp, loss_io, c_out, n_alpha, static_cast<int>(m), static_cast<int>(n),
                         static_cast<int>(k), q, status_io, items, st);
}

extern "C" int b200q_awq_search_fused(const void* a_all, const void* w, const void* s_all, const void* ref,
                                      int n_alpha, int64_t m, int64_t n, int64_t k, int block, int num_bits,
                                      int is_unsigned, int narrow_range, double* loss_io, float* c_out,
                                      uint32_t* status_io, void* stream) {
  B200Q_REQUIRE_PTR(a_all); B200Q_REQUIRE_PTR(w); B200Q_REQUIRE_PTR(s_all); B200Q_REQUIRE_PTR(ref);
  B200Q_REQUIRE_PTR(loss_io); B200Q_REQUIRE_PTR(status_io);
  B200Q_REQUIRE_ALIGNED(a_all); B200Q_REQUIRE_ALIGNED(w); B200Q_REQUIRE_ALIGNED(s_all); B200Q_REQUIRE_ALIGNED(ref);
  if (n_alpha <= 0 || m <= 0 || n <= 0 || k <= 0) return B200Q_ERR_SHAPE;
  if (num_bits < 1 || num_bits + (is_unsigned ? 1 : 0) > 24) return B200Q_ERR_ARG;
  // one W unit = one quantisation block = two swizzle rows; the epilogue masks whole 32-column chunks
  if (block != 128 || k % 128 || n % 32) return B200Q_ERR_UNSUPPORTED;
  return fused_entry(a_all, w, n, s_all, ref, n_alpha, m, n, k, make_intq(num_bits, is_unsigned, narrow_range),
                     loss_io, c_out, status_io, stream);
}

extern "C" int b200q_awq_search_prequant(const void* a_all, const void* wq_all, const void* ref, int n_alpha,
                                         int64_t m, int64_t n, int64_t k, double* loss_io, float* c_out,
                                         uint32_t* status_io, void* stream) {
  B200Q_REQUIRE_PTR(a_all); B200Q_REQUIRE_PTR(wq_all); B200Q_REQUIRE_PTR(ref);
  B200Q_REQUIRE_PTR(loss_io); B200Q_REQUIRE_PTR(status_io);
  B200Q_REQUIRE_ALIGNED(a_all); B200Q_REQUIRE_ALIGNED(wq_all); B200Q_REQUIRE_ALIGNED(ref);
  if (n_alpha <= 0 || m <= 0 || n <= 0 || k <= 0) return B200Q_ERR_SHAPE;
  if (k % 128 || n % 32) return B200Q_ERR_UNSUPPORTED;
  return fused_entry(a_all, wq_all, static_cast<int64_t>(n_alpha) * n, nullptr, ref, n_alpha, m, n, k, IntQ{7.f, -8.f},
                     loss_io, c_out, status_io, stream);
}
