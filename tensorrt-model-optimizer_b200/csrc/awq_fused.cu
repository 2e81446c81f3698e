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
// Warps of a CTA (16):
//   0      A producer: TMA 128 x 64 tiles into a 4-deep ring, completion counted on the EVEN CTA's barrier
//   1      MMA issuer (even CTA only) and TMEM allocation
//   2      W producer: TMA raw 128 x 128 weight units (two swizzled 128 x 64 boxes) and the unit's 128
//          scale factors into a 3-deep ring
//   4-7    epilogue: tcgen05.ld the accumulator, squared error against R, one atomic per warp and item
//   8-15   transform, two groups of four warps taking alternate units: in shared memory, in place:
//          bf16(W * s), block abs-max (2 lanes = one 128-block), integer fake quant, then a proxy fence
//          and an arrival on the even CTA's "unit ready" barrier
// The MMA thread waits for "A tile landed in both CTAs" and "W unit transformed in both CTAs", issues
// 2 x 4 MMAs per 64-wide K slice, and releases ring slots to both CTAs with tcgen05.commit.  Producers
// and transformers run ahead into the next item while the epilogue drains the accumulator.
//
// Every wait is bounded: when one runs out, an error bit is set in the caller's status word, the CTA
// stops waiting anywhere else, and the kernel ends through its normal exit (TMEM released).
#include "umma.cuh"

namespace b200q {

constexpr int kFK = 64;                                  // K elements of one A stage: one 128-byte swizzle row
constexpr uint32_t kFTileBytes = 128 * kFK * 2;          // 128 rows x 64 bf16 = 16 KB: one TMA box
constexpr uint32_t kFUnitBytes = 2 * kFTileBytes;        // a W unit: 128 rows x 128 K = two boxes
constexpr int kFPairN = 256;                             // columns of a pair's tile (128 weight rows per CTA)
constexpr int kFWUnits = 3;
constexpr uint32_t kFScaleBytes = 128 * 2;               // one unit's share of a candidate's scale vector
constexpr int kFThreads = 512;
constexpr int kFTransformWarps = 8, kFEpilogueWarps = 4;
constexpr int kFMaxStages = 6;

template <int MT> struct FusedCfg {
  static constexpr int kAStages = MT == 2 ? 4 : 6;
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
  uint64_t w_full[kFWUnits];       // raw unit landed (each CTA its own)
  uint64_t b_ready[kFWUnits];      // unit transformed in both CTAs (even CTA's copy)
  uint64_t b_empty[kFWUnits];
  uint64_t acc_full;               // all MMAs of an item complete
  uint64_t acc_empty;              // accumulator read out in both CTAs (even CTA's copy)
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
__device__ __forceinline__ uint64_t f32x2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
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
                        const __nv_bfloat16* __restrict__ s_all, const __nv_bfloat16* __restrict__ ref,
                        double* __restrict__ loss, float* __restrict__ c_out, int n_alpha, int M, int N, int K,
                        IntQ q, uint32_t* __restrict__ status) {
  using Cfg = FusedCfg<MT>;
  constexpr int SA = Cfg::kAStages, SW = kFWUnits;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* ring_a = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring_w = ring_a + SA * Cfg::kAStageBytes;
  uint8_t* ring_s = ring_w + SW * kFUnitBytes;       // the 128 scale factors of each W unit (256 bytes per slot)
  FusedSmem* sm = reinterpret_cast<FusedSmem*>(ring_s + SW * kFScaleBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int slab_rows = 256 * MT;
  const int slabs_m = (M + slab_rows - 1) / slab_rows, slabs_n = (N + kFPairN - 1) / kFPairN;
  const int num_items = n_alpha * slabs_m * slabs_n;
  const int k_slices = K / kFK;                      // K is a multiple of 128: an even count

  if (threadIdx.x == 0) {
    for (int s = 0; s < SA; ++s) { mbar_init(&sm->a_full[s], 1); mbar_init(&sm->a_empty[s], 1); }
    for (int u = 0; u < SW; ++u) {
      mbar_init(&sm->w_full[u], 1);
      mbar_init(&sm->b_ready[u], 2 * (kFTransformWarps / 2));   // one group of transform warps per unit, both CTAs
      mbar_init(&sm->b_empty[u], 1);
    }
    mbar_init(&sm->acc_full, 1);
    mbar_init(&sm->acc_empty, 2 * kFEpilogueWarps);
    sm->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // the same warp of both CTAs: one allocation for the pair
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)), "r"(Cfg::kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_barrier();   // the peer's barriers are initialised before anything signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&sm->tmem_base);

  if (warp == 0) {
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
          const uint32_t full_leader = map_to_cta(&sm->a_full[s], 0);
          if (leader) mbar_expect_tx(&sm->a_full[s], 2 * Cfg::kAStageBytes);      // both CTAs' tiles
          uint8_t* dst = ring_a + s * Cfg::kAStageBytes;
#pragma unroll
          for (int t = 0; t < MT; ++t) tma_load_2d_pair(dst + t * kFTileBytes, &map_a, full_leader, kb * kFK, row0 + t * 256);
        }
      }
    }
  } else if (warp == 2) {
    // ---------------------------------------------------------------- W producer --------------
    if (lane == 0) {
      uint32_t wu = 0;
      bool ok = true;
      for (int item = pair; item < num_items && ok; item += num_pairs) {
        const FusedItem w = fused_item(item, slabs_m, slabs_n);
        const int n_row = w.slab_n * kFPairN + static_cast<int>(rank) * 128;
        const __nv_bfloat16* s_row = s_all + static_cast<int64_t>(w.alpha) * K;
        for (int ub = 0; ub < k_slices / 2; ++ub, ++wu) {
          const int u = wu % SW;
          ok = mbar_wait_bounded(&sm->b_empty[u], ((wu / SW) & 1) ^ 1, &sm->abort, status, kFErrWProducer);
          if (!ok) break;
          uint8_t* dst = ring_w + u * kFUnitBytes;
          mbar_expect_tx(&sm->w_full[u], kFUnitBytes + kFScaleBytes);
          bulk_load(ring_s + u * kFScaleBytes, s_row + ub * 128, kFScaleBytes, &sm->w_full[u]);
          tma_load_2d(dst, &map_w, &sm->w_full[u], ub * 128, n_row);
          tma_load_2d(dst + kFTileBytes, &map_w, &sm->w_full[u], ub * 128 + kFK, n_row);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer --------------
    if (lane == 0 && leader) {
      uint32_t it = 0, wu = 0, done = 0;
      bool ok = true;
      for (int item = pair; item < num_items && ok; item += num_pairs, ++done) {
        if (done > 0) {   // the previous item's accumulator has been read out in both CTAs
          ok = mbar_wait_bounded_cluster(&sm->acc_empty, (done - 1) & 1, &sm->abort, status, kFErrMma);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        int u = 0;
        for (int kb = 0; kb < k_slices; ++kb, ++it) {
          if ((kb & 1) == 0) {
            u = wu % SW;
            ok = mbar_wait_bounded_cluster(&sm->b_ready[u], (wu / SW) & 1, &sm->abort, status, kFErrMma);
            if (!ok) break;
          }
          const int s = it % SA;
          ok = mbar_wait_bounded(&sm->a_full[s], (it / SA) & 1, &sm->abort, status, kFErrMma);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(ring_a + s * Cfg::kAStageBytes);
          const uint64_t db = umma_desc(smem_u32(ring_w + u * kFUnitBytes + (kb & 1) * kFTileBytes));
#pragma unroll
          for (int t = 0; t < MT; ++t) {
            const uint64_t da = umma_desc(a_addr + t * kFTileBytes);
#pragma unroll
            for (int k = 0; k < kFK / 16; ++k)   // 16 bf16 = 32 bytes along K inside the swizzled row: +2 in 16-byte units
              umma_bf16_pair(tmem + t * kFPairN, da + 2 * k, db + 2 * k, Cfg::kIdesc, (kb | k) != 0 ? 1u : 0u);
          }
          // the slot is free in both CTAs once these MMAs have read it
          umma_commit_pair(map_to_cta(&sm->a_empty[s], 0));
          umma_commit_pair(map_to_cta(&sm->a_empty[s], 1));
          if (kb & 1) {
            umma_commit_pair(map_to_cta(&sm->b_empty[u], 0));
            umma_commit_pair(map_to_cta(&sm->b_empty[u], 1));
            ++wu;
          }
        }
        if (!ok) break;
        umma_commit_pair(map_to_cta(&sm->acc_full, 0));   // fires when every MMA issued above has completed
        umma_commit_pair(map_to_cta(&sm->acc_full, 1));
      }
    }
  } else if (warp >= 8) {
    // ---------------------------------------------------------------- transform ---------------
    // The eight warps form two groups of four; a group takes every other W unit, so two units are in
    // the transform stage at a time and one group's latencies (barrier, shared-memory round trips, the
    // proxy fence) hide under the other's arithmetic.  Within a unit a lane owns one row of one 64-wide
    // box at a time (64 elements, 8 swizzled 16-byte chunks: chunk j of row r sits at j ^ (r & 7));
    // lanes l and l + 16 hold the two halves of a 128-block; a warp covers 32 rows in two passes.
    //
    // Arithmetic, per block: v = bf16(w * s); amax = max |v|; scale = 7 / amax; out = bf16(k / scale) with
    // k = rint(v * scale).  Because the abs-max is the block's own, |v * scale| <= 7 (1 + 2^-24) and the
    // clamp to [-8, 7] never acts.  k / scale takes only 15 values per block, so instead of one exact
    // division per element the two lanes of a block check once, for k = 1..7, that bf16(k * y) with
    // y = RN(1 / scale) equals bf16(RN(k / scale)) (it does except when k * y falls within a rounding
    // error of a bf16 tie) and then multiply; a block that fails the check, a dead or out-of-range
    // scale, or a bit width other than 4 takes the element-wise exact path.  Zeros come out as +0
    // where the stand-alone kernel keeps the sign: the product does not see the difference.
    const int group = (warp - 8) >> 2, gw = (warp - 8) & 3, box = lane >> 4;
    const bool four_bit = q.bound == 7.f && q.lo == -8.f;
    bool ok = true;
    const uint32_t units_total = static_cast<uint32_t>((num_items - pair + num_pairs - 1) / num_pairs) * (k_slices / 2);
    for (uint32_t wu = group; wu < units_total && ok; wu += 2) {
      const int u = wu % SW;
      // every lane observes the barrier itself; the decision to go on is the warp's (shuffles follow)
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(&sm->w_full[u], (wu / SW) & 1, &sm->abort, status, kFErrTransform));
      if (!ok) break;
      // this lane's 64 scale factors of the unit (the lanes of a box read the same addresses: broadcast)
      const uint4* sp = reinterpret_cast<const uint4*>(ring_s + u * kFScaleBytes + box * 128);
#pragma unroll 1
      for (int pass = 0; pass < 2; ++pass) {
        const int row = gw * 32 + pass * 16 + (lane & 15), sw = row & 7;
        uint8_t* rowp = ring_w + u * kFUnitBytes + box * kFTileBytes + row * 128;
        uint32_t pr[32];
        uint32_t mx = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint4 wv = *reinterpret_cast<const uint4*>(rowp + ((j ^ sw) << 4));
          const uint4 sv = sp[j];
          const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w}, ss[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            // packed bf16 multiply = the product rounded to bf16, two elements per instruction
            const __nv_bfloat162 p2 = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&ww[i]),
                                              *reinterpret_cast<const __nv_bfloat162*>(&ss[i]));
            pr[4 * j + i] = *reinterpret_cast<const uint32_t*>(&p2);
            mx = __vmaxu2(mx, pr[4 * j + i] & 0x7fff7fffu);     // |x| patterns: integer order = magnitude order
          }
        }
        uint32_t bits = max(mx & 0xffffu, mx >> 16) << 16;
        bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, 16));
        const IntScale sc = make_int_scale(q, __uint_as_float(bits));
        bool fast = four_bit && sc.live && sc.fast;
        const float2 y2 = make_float2(sc.y, sc.y);
        {
          // this lane's share of the check: k = 1..4 (first box) or 4..7 (second box); done by every
          // lane (a few instructions) so that the shuffle below is one warp-wide instruction
          const float k0 = box ? 4.f : 1.f;
          const float2 nd = make_float2(-sc.scale, -sc.scale);
          const float2 ka = make_float2(k0, k0 + 1.f), kb = make_float2(k0 + 2.f, k0 + 3.f);
          const float2 ea = div2_rn_rcp(ka, nd, y2), eb = div2_rn_rcp(kb, nd, y2);
          const float2 fa = __fmul2_rn(ka, y2), fb = __fmul2_rn(kb, y2);
          const bool same = Elem<__nv_bfloat16>::pack2(ea.x, ea.y) == Elem<__nv_bfloat16>::pack2(fa.x, fa.y) &&
                            Elem<__nv_bfloat16>::pack2(eb.x, eb.y) == Elem<__nv_bfloat16>::pack2(fb.x, fb.y);
          const bool peer_same = __shfl_xor_sync(0xffffffffu, same ? 1 : 0, 16) != 0;
          fast = fast && same && peer_same;      // the two lanes of a block agree: same scale, both checks
        }
        if (fast) {
          // The product is rounded to fp32 BEFORE it is rounded to an integer, as the reference does (a
          // block's own ties, e.g. v / amax = 13 / 14, sit exactly on .5 only after that first rounding):
          // the rounding instruction between the two multiplies also keeps either from being fused
          // with anything.
          const uint64_t scale_p = f32x2_pack(sc.scale, sc.scale), y_p = f32x2_pack(sc.y, sc.y);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const uint64_t t2 = f32x2_mul(f32x2_pack(__uint_as_float(pr[i] << 16), __uint_as_float(pr[i] & 0xffff0000u)), scale_p);
            const float r_lo = rintf(__uint_as_float(static_cast<uint32_t>(t2)));
            const float r_hi = rintf(__uint_as_float(static_cast<uint32_t>(t2 >> 32)));
            const uint64_t o2 = f32x2_mul(f32x2_pack(r_lo, r_hi), y_p);
            pr[i] = Elem<__nv_bfloat16>::pack2(__uint_as_float(static_cast<uint32_t>(o2)),
                                               __uint_as_float(static_cast<uint32_t>(o2 >> 32)));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float lo = intq_apply(__uint_as_float(pr[i] << 16), sc, q);
            const float hi = intq_apply(__uint_as_float(pr[i] & 0xffff0000u), sc, q);
            pr[i] = Elem<__nv_bfloat16>::pack2(lo, hi);
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(rowp + ((j ^ sw) << 4)) = make_uint4(pr[4 * j], pr[4 * j + 1], pr[4 * j + 2], pr[4 * j + 3]);
      }
      fence_async_shared();     // these stores are read next by the tensor cores of both CTAs
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(&sm->b_ready[u], 0));
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- epilogue ----------------
    const int quarter = warp & 3;        // TMEM lanes quarter * 32 .. + 31 are the rows this warp may read
    const uint32_t acc_empty_leader = map_to_cta(&sm->acc_empty, 0);
    uint32_t done = 0;
    bool ok = true;
    for (int item = pair; item < num_items && ok; item += num_pairs, ++done) {
      const FusedItem w = fused_item(item, slabs_m, slabs_n);
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(&sm->acc_full, done & 1, &sm->abort, status, kFErrEpilogue));
      if (!ok) break;                     // warp-uniform: the TMEM loads below are warp-wide
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float sq = 0.f;
#pragma unroll 1
      for (int t = 0; t < MT; ++t) {
        const int row = w.slab_m * slab_rows + t * 256 + static_cast<int>(rank) * 128 + quarter * 32 + lane;
        const bool row_ok = row < M;
        const __nv_bfloat16* rrow = ref + static_cast<int64_t>(row) * N;
        float* crow = c_out ? c_out + (static_cast<int64_t>(w.alpha) * M + row) * N : nullptr;
#pragma unroll 1
        for (int cc = 0; cc < kFPairN / 32; ++cc) {
          const int col0 = w.slab_n * kFPairN + cc * 32;
          if (col0 >= N) break;                                           // warp-uniform (N % 32 == 0)
          uint32_t acc[32];
          tmem_ld32(tmem + (static_cast<uint32_t>(quarter * 32) << 16) + t * kFPairN + cc * 32, acc);
          if (row_ok) {
            const uint4* rp = reinterpret_cast<const uint4*>(rrow + col0);
#pragma unroll
            for (int vv = 0; vv < 4; ++vv) {
              const uint4 r4 = __ldg(rp + vv);
              float rf[8];
              Elem<__nv_bfloat16>::unpack(r4, rf);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float a = __uint_as_float(acc[8 * vv + j]);
                const float o = __bfloat162float(__float2bfloat16_rn(a));
                const float d = __bfloat162float(__float2bfloat16_rn(o - rf[j]));
                sq = fmaf(d, d, sq);
              }
            }
            if (crow) {
#pragma unroll
              for (int j = 0; j < 32; ++j) crow[col0 + j] = __uint_as_float(acc[j]);
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader);   // the accumulator may be overwritten
      for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if (lane == 0) atomicAdd(loss + w.alpha, static_cast<double>(sq));
    }
  }

  __syncwarp();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_barrier();   // neither CTA leaves (or frees the pair's TMEM) while the other still works
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (warp == 1) {
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
static int fused_launch(const CUtensorMap& map_a, const CUtensorMap& map_w, const __nv_bfloat16* s_all,
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
  if (cudaLaunchKernelEx(&cfg, kern, map_a, map_w, s_all, ref, loss, c_out, n_alpha, m, n, k, q, status) != cudaSuccess) {
    cudaGetLastError();
    return B200Q_ERR_CUDA;
  }
  return launch_status();
}

}  // namespace b200q

using namespace b200q;

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
  if (n_alpha * m > (1ll << 30) || n > (1ll << 30) || k > (1ll << 30)) return B200Q_ERR_UNSUPPORTED;
  const int mt = m > 256 ? 2 : 1;
  const int64_t slabs_m = (m + 256 * mt - 1) / (256 * mt), slabs_n = (n + kFPairN - 1) / kFPairN;
  const int64_t items = n_alpha * slabs_m * slabs_n;
  if (items > (1ll << 30)) return B200Q_ERR_UNSUPPORTED;
  CUtensorMap map_a, map_w;
  if (!fused_make_map(&map_a, a_all, static_cast<int64_t>(n_alpha) * m, k) || !fused_make_map(&map_w, w, n, k))
    return B200Q_ERR_CUDA;
  const IntQ q = make_intq(num_bits, is_unsigned, narrow_range);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* sp = static_cast<const __nv_bfloat16*>(s_all);
  const __nv_bfloat16* rp = static_cast<const __nv_bfloat16*>(ref);
  if (mt == 2)
    return fused_launch<2>(map_a, map_w, sp, rp, loss_io, c_out, n_alpha, static_cast<int>(m), static_cast<int>(n),
                           static_cast<int>(k), q, status_io, items, st);
  return fused_launch<1>(map_a, map_w, sp, rp, loss_io, c_out, n_alpha, static_cast<int>(m), static_cast<int>(n),
                         static_cast<int>(k), q, status_io, items, st);
}
