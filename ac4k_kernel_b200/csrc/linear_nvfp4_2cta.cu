// NVFP4 block-scaled GEMM for sm_100a, CTA-pair variant (tcgen05 cta_group::2).
//
// Two CTAs of a cluster share one 256 x 256 output tile: CTA r of the pair loads A rows
// [128 r, 128 r + 128) and B rows (output columns) [128 r, 128 r + 128) of the tile, the leader
// CTA issues one tcgen05.mma over both (M = 256, N = 256, each CTA accumulating its 128 rows x
// 256 columns in its own tensor memory, the B halves read from both CTAs' shared memory).  Per
// FLOP this moves a third less operand data from L2 into shared memory than 128 x 256 tiles of
// single CTAs.  No multicast loads are used.
//
// A pipeline stage is K = 512 elements (8 MMAs of K = 64): every role's per-stage bookkeeping
// (mbarrier waits ~75-100 cycles each, tcgen05.commit ~110, a tcgen05.mma issue ~75-125, remote
// arrives) was measured to be latency-bound, so fewer, larger stages keep each role's loop shorter
// than the 1024 cycles the tensor pipe needs per stage.
//
// Roles per CTA (512 threads):
//   warp 0      TMA producer: A and B of this CTA, 4 boxes of 128 rows x 128 B per stage, 3 stages
//   warp 1      MMA issuer (leader CTA only): 8 MMAs + 1 commit per stage; learns that a stage is
//               ready from a counter in shared memory instead of waiting on mbarriers itself
//   warps 2-5   scale warps: scale bytes shared memory -> registers -> tensor memory (tcgen05.st),
//               one TMEM lane quarter each; 2-deep rings in shared and in tensor memory
//   warp 10     scale feeder: bulk copies of scale bytes, as soon as the scale warps freed a slot
//   warp 11     barrier watcher (leader CTA only): waits for each stage's operands + scales and
//               publishes the count of ready stages
//   warps 6-9, 12-15  epilogue: tcgen05.ld of 128 accumulator columns per warp into registers
//               (* alpha, + bias, packed to 16 bit), hand the accumulator back, then store
// Barriers that gate the MMA live in the leader CTA and are signalled by both CTAs; barriers that
// release stages / publish the accumulator exist in both CTAs and are signalled by one
// tcgen05.commit whose arrival fans out to both.
#include "gemm_common.cuh"

namespace ac4k {
using namespace ptx;

#ifdef AC4K_TRACE_ENABLED
// region 0: MMA issuer, region 1: epilogue warp 6, region 2: scale warp 2 (all leader CTA, cluster 0)
#define AC4K_TR(region, it, ev)                                                              \
  do {                                                                                      \
    if (p.trace != nullptr && cluster_id == 0 && rank == 0 && (it) < 128)                   \
      p.trace[((size_t)(region) * 128 + (it)) * 8 + (ev)] = clock64();                      \
  } while (0)
// wall-clock (ns) stamps, comparable across the two CTAs of cluster 0
#define AC4K_TRG(region, it, ev)                                                             \
  do {                                                                                      \
    if (p.trace != nullptr && cluster_id == 0 && (it) < 128)                                \
      p.trace[((size_t)(region) * 128 + (it)) * 8 + (ev)] = globaltimer();                  \
  } while (0)
#else
#define AC4K_TR(region, it, ev) do { } while (0)
#define AC4K_TRG(region, it, ev) do { } while (0)
#endif

namespace pair {
static constexpr int BN = 256;                      // output columns of the pair tile
static constexpr int BMP = 256;                     // output rows of the pair tile
static constexpr int KS = 8;                        // K = 64 steps per stage
static constexpr int HALF_BYTES = 128 * BKB;        // one 128-row x 128-byte box
static constexpr int A_BYTES = 2 * HALF_BYTES;      // this CTA's 128 rows of A, K = 512
static constexpr int B_BYTES = 2 * HALF_BYTES;      // this CTA's 128 rows of B, K = 512
static constexpr int SFA_BYTES = KS * 512;
static constexpr int SFB_BYTES = 2 * KS * 512;
static constexpr int STAGES = 3;                    // operand ring
static constexpr int SF_STAGES = 2;                 // scale rings (shared memory and tensor memory)
static constexpr int BIAS_BYTES = 8 * 128 * 4;          // one tile's bias as fp32, 128 columns per epilogue warp
static constexpr int SMEM_BYTES = STAGES * (A_BYTES + B_BYTES) + SF_STAGES * (SFA_BYTES + SFB_BYTES) + 1024 + 512 + BIAS_BYTES;
static constexpr int SFA_COL = 256, SFA_COLS = KS * 4, SFB_COL = SFA_COL + SF_STAGES * SFA_COLS, SFB_COLS = KS * 8;
static_assert(SFB_COL + SF_STAGES * SFB_COLS <= kTmemCols, "tensor memory overflow");
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory overflow");
static constexpr int kThreadsPair = 512;
}  // namespace pair

template <bool SF_TILED, int OUT_DT, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pair::kThreadsPair, 1)
linear_nvfp4_2cta_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                         const __grid_constant__ CUtensorMap tma_sfa, const __grid_constant__ CUtensorMap tma_sfb,
                         const GemmArgs p) {
  using namespace pair;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA = smem_base;
  const uint32_t sB = sA + STAGES * A_BYTES;
  const uint32_t sSFA = sB + STAGES * B_BYTES;
  const uint32_t sSFB = sSFA + SF_STAGES * SFA_BYTES;
  const uint32_t bars = sSFB + SF_STAGES * SFB_BYTES;
  const uint32_t full_bar = bars;                     // [STAGES] leader: operands of both CTAs landed + all scales in TMEM
  const uint32_t empty_bar = full_bar + 8 * STAGES;   // [STAGES] both: MMAs that used the stage are done
  const uint32_t sffull_bar = empty_bar + 8 * STAGES; // [SF_STAGES] local: scale bytes landed
  const uint32_t sffree_bar = sffull_bar + 8 * SF_STAGES;   // [SF_STAGES] local: 4 scale warps have read the slot
  const uint32_t tfull_bar = sffree_bar + 8 * SF_STAGES;    // both: accumulator complete
  const uint32_t tempty_bar = tfull_bar + 8;          // leader: 16 epilogue warps drained the accumulator
  const uint32_t ready_word = tempty_bar + 8;         // leader: stages the watcher has seen complete
  const uint32_t tmem_slot = ready_word + 8;
  const uint32_t sBias = bars + 512;                  // [8 epilogue warps][128] fp32
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_tiles = (p.KT + KS - 1) / KS;
  const int last_nk = p.KT - (k_tiles - 1) * KS;      // K = 64 steps in the last stage of a tile

  if (threadIdx.x == 0) AC4K_TR(3, 0, 0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar + 8 * s, 9);           // producer's expect_tx arrival + 8 scale warps
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int s = 0; s < SF_STAGES; ++s) {
      mbar_init(sffull_bar + 8 * s, 1);
      mbar_init(sffree_bar + 8 * s, 4);
    }
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, 16);                  // 8 epilogue warps in each CTA
    st_shared_release(ready_word, 0);
    fence_barrier_init();
    prefetch_tmap(&tma_a);
    prefetch_tmap(&tma_b);
    if (!SF_TILED) {
      prefetch_tmap(&tma_sfa);
      prefetch_tmap(&tma_sfb);
    }
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();          // peer's barriers are initialised before anything is signalled remotely
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(smem_gen + (tmem_slot - smem_base));
  // Everything above touched only this CTA's own resources, so it may overlap the tail of the kernel
  // before this one in the stream; from here on global memory is read and written.
  grid_launch_dependents();
  grid_dependency_wait();
  if (threadIdx.x == 0) AC4K_TR(3, 0, 1);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (A and B)
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      bool ok = true;
      uint32_t leader_full[STAGES];
#pragma unroll
      for (int i = 0; i < STAGES; ++i) leader_full[i] = map_to_cta(full_bar + 8 * i, 0);
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * BMP + (int)rank * 128;        // this CTA's rows of A
        const int nb0 = tn * BN + (int)rank * 128;        // this CTA's rows of B
        for (int kt = 0; kt < k_tiles; ++kt) {
          if (!mbar_wait(empty_bar + 8 * s, ph ^ 1)) { atomicExch(p.status, kStatusTimeoutProducer); ok = false; break; }
          const uint32_t lf = s == 0 ? leader_full[0] : (s == 1 ? leader_full[1] : leader_full[2]);
          if (rank == 0) mbar_arrive_expect_tx(full_bar + 8 * s, 2 * (A_BYTES + B_BYTES));
          const int kb = kt * (2 * BKB);
          tma_load_2d_pair(sA + s * A_BYTES, &tma_a, kb, m0, lf);
          tma_load_2d_pair(sB + s * B_BYTES, &tma_b, kb, nb0, lf);
          tma_load_2d_pair(sA + s * A_BYTES + HALF_BYTES, &tma_a, kb + BKB, m0, lf);
          tma_load_2d_pair(sB + s * B_BYTES + HALF_BYTES, &tma_b, kb + BKB, nb0, lf);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_mxf4nvf4(BMP, BN);
      uint32_t s = 0, sf = 0, it = 0;
      bool ok = true;
      const uint64_t adesc0 = make_smem_desc(sA, 16, 1024, kSwizzle128B);
      const uint64_t bdesc0 = make_smem_desc(sB, 16, 1024, kSwizzle128B);
      uint32_t acc_ph = 0;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        // the accumulator must have been drained by all 16 epilogue warps of the pair; waited for
        // here and not through the watcher: it is the last link of the chain between two tiles
        AC4K_TRG(0, it, 6);
        if (!mbar_wait(tempty_bar, acc_ph ^ 1)) { ok = false; break; }
        AC4K_TRG(0, it, 7);
        acc_ph ^= 1;
        for (int kt = 0; kt < k_tiles; ++kt) {
          AC4K_TR(0, it, 0);
          uint32_t seen = ld_shared_volatile(ready_word);
          if (seen <= it) {
            const unsigned long long t0 = globaltimer();
            while ((seen = ld_shared_volatile(ready_word)) <= it) {
              // back off: a hot spin here takes issue slots from the epilogue and scale warps that
              // share this scheduler, which is exactly what the issuer is waiting for
              __nanosleep(40);
              if (globaltimer() - t0 > kWaitTimeoutNs) { seen = 0xFFFFFFFFu; break; }
            }
          }
          if (seen == 0xFFFFFFFFu) { ok = false; break; }
          tc_fence_after();
          AC4K_TR(0, it, 1);
          if (it == 0) AC4K_TR(3, 0, 2);
          const uint32_t t_sfa = tmem_base + SFA_COL + sf * SFA_COLS;
          const uint32_t t_sfb = tmem_base + SFB_COL + sf * SFB_COLS;
          const uint64_t adesc = adesc0 + (uint64_t)(s * (A_BYTES >> 4));
          const uint64_t bdesc = bdesc0 + (uint64_t)(s * (B_BYTES >> 4));
          const int nk = (kt + 1 < k_tiles) ? KS : last_nk;
          if (nk == KS) {
#pragma unroll
            for (int j = 0; j < KS; ++j) {
              // K step j: box j / 4 of the stage, 32 bytes further inside the 128-byte swizzle atom per step
              const uint32_t off = (j >> 2) * (HALF_BYTES >> 4) + 2 * (j & 3);
              mma_mxf4nvf4_pair(tmem_base, adesc + off, bdesc + off, idesc, t_sfa + j * 4, t_sfb + j * 8,
                                (kt > 0 || j > 0) ? 1u : 0u);
            }
          } else {
            for (int j = 0; j < nk; ++j) {
              const uint32_t off = (j >> 2) * (HALF_BYTES >> 4) + 2 * (j & 3);
              mma_mxf4nvf4_pair(tmem_base, adesc + off, bdesc + off, idesc, t_sfa + j * 4, t_sfb + j * 8,
                                (kt > 0 || j > 0) ? 1u : 0u);
            }
          }
          AC4K_TR(0, it, 3);
          tc_commit_pair_both(empty_bar + 8 * s, 3);                 // stage free in both CTAs
          if (kt == k_tiles - 1) tc_commit_pair_both(tfull_bar, 3);  // accumulator complete in both CTAs
          AC4K_TR(0, it, 5);
          ++it;
          sf ^= 1;
          if (++s == STAGES) s = 0;
        }
      }
      if (!ok) atomicExch(p.status, kStatusTimeoutMma);
    }
  } else if (warp == 11) {
    // ------------------------------------------------------------------ barrier watcher (leader CTA)
    if (lane == 0 && rank == 0) {
      uint32_t s = 0, ph = 0, count = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        for (int kt = 0; kt < k_tiles && ok; ++kt) {
          ok = mbar_wait(full_bar + 8 * s, ph);
          if (!ok) break;
          st_shared_release(ready_word, ++count);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) {
        atomicExch(p.status, kStatusTimeoutMma);
        st_shared_release(ready_word, 0xFFFFFFFFu);
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------------ scale feeder
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * BMP + (int)rank * 128, n0 = tn * BN;
        const int64_t mt = m0 / 128;
        const bool a_ok = SF_TILED ? (mt * 128 < p.rows_sfa) : (m0 < p.rows_sfa);
        const int nb_valid = min(2, (p.rows_sfb - n0) / 128);                       // tiled layout
        for (int kt = 0; kt < k_tiles; ++kt) {
          if (!mbar_wait(sffree_bar + 8 * s, ph ^ 1)) { atomicExch(p.status, kStatusTimeoutSf); ok = false; break; }
          const int nk = (kt + 1 < k_tiles) ? KS : last_nk;
          const uint32_t bar = sffull_bar + 8 * s;
          const int64_t k64 = (int64_t)kt * KS;
          if (SF_TILED) {
            mbar_arrive_expect_tx(bar, ((a_ok ? 1 : 0) + nb_valid) * nk * 512);
            if (a_ok) bulk_load_1d_local(sSFA + s * SFA_BYTES, p.sfa + (mt * p.KT + k64) * 512, nk * 512, bar);
            for (int nb = 0; nb < nb_valid; ++nb)
              bulk_load_1d_local(sSFB + s * SFB_BYTES + nb * (KS * 512),
                                 p.sfb + ((int64_t)(n0 / 128 + nb) * p.KT + k64) * 512, nk * 512, bar);
          } else {
            // row layout: one box of [8 K steps][128 or 256 rows] words per operand; rows and K steps
            // outside the tensor arrive as zeros and count towards the transaction bytes
            mbar_arrive_expect_tx(bar, SFA_BYTES + SFB_BYTES);
            tma_load_2d_local(sSFA + s * SFA_BYTES, &tma_sfa, m0, (int)k64, bar);
            tma_load_2d_local(sSFB + s * SFB_BYTES, &tma_sfb, n0, (int)k64, bar);
          }
          if (++s == SF_STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ scale warps
    // Lane l of the warp owning TMEM lane quarter q writes, for K step j and row group g, the word
    // of row 32 g + l into column (j * groups + g) of lane 32 q + l.  A tensor-memory slot is
    // rewritten once the MMAs of the stage that used it two stages ago are done.
    const int q = warp & 3;
    uint32_t s = 0, ph = 0;          // scale rings (depth 2)
    uint32_t os = 0, oph = 0;        // operand ring position of the current stage (depth 3)
    uint32_t ps = 0, pph = 0;        // operand ring position of the stage two stages back
    uint32_t it = 0;
    bool ok = true;
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    uint32_t leader_full[STAGES];
#pragma unroll
    for (int i = 0; i < STAGES; ++i) leader_full[i] = map_to_cta(full_bar + 8 * i, 0);
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
      for (int kt = 0; kt < k_tiles; ++kt) {
        if (warp == 2 && lane == 0) AC4K_TR(2, it, 0);
        if (!mbar_wait(sffull_bar + 8 * s, ph)) { if (lane == 0) atomicExch(p.status, kStatusTimeoutSf); ok = false; break; }
        if (warp == 2 && lane == 0) AC4K_TR(2, it, 1);
        const uint8_t *a_src = smem_gen + (sSFA + s * SFA_BYTES - smem_base);
        const uint8_t *b_src = smem_gen + (sSFB + s * SFB_BYTES - smem_base);
        uint32_t ra[32], rb[64];
        if (SF_TILED) {
#pragma unroll
          for (int j = 0; j < KS; ++j) {
            const uint4 v = *reinterpret_cast<const uint4 *>(a_src + j * 512 + lane * 16);
            ra[j * 4 + 0] = v.x; ra[j * 4 + 1] = v.y; ra[j * 4 + 2] = v.z; ra[j * 4 + 3] = v.w;
#pragma unroll
            for (int nb = 0; nb < 2; ++nb) {
              const uint4 w = *reinterpret_cast<const uint4 *>(b_src + (nb * KS + j) * 512 + lane * 16);
              rb[j * 8 + nb * 4 + 0] = w.x; rb[j * 8 + nb * 4 + 1] = w.y;
              rb[j * 8 + nb * 4 + 2] = w.z; rb[j * 8 + nb * 4 + 3] = w.w;
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < KS; ++j) {
#pragma unroll
            for (int g = 0; g < 4; ++g) ra[j * 4 + g] = reinterpret_cast<const uint32_t *>(a_src + j * 512)[g * 32 + lane];
#pragma unroll
            for (int g = 0; g < 8; ++g) rb[j * 8 + g] = reinterpret_cast<const uint32_t *>(b_src + j * 1024)[g * 32 + lane];
          }
        }
        if (warp == 2 && lane == 0) AC4K_TR(2, it, 2);
        if (it >= SF_STAGES) {
          if (!mbar_wait(empty_bar + 8 * ps, pph)) { if (lane == 0) atomicExch(p.status, kStatusTimeoutSf); ok = false; break; }
          if (++ps == STAGES) { ps = 0; pph ^= 1; }
        }
        if (warp == 2 && lane == 0) AC4K_TR(2, it, 3);
        tc_fence_after();
        tmem_st_32x32b_x32(lane_base + SFA_COL + s * SFA_COLS, ra);
        tmem_st_32x32b_x64(lane_base + SFB_COL + s * SFB_COLS, rb);
        tmem_st_wait();
        if (warp == 2 && lane == 0) AC4K_TR(2, it, 5);
        tc_fence_before();
        __syncwarp();
        // The shared-memory slot goes back to the feeder only now, after tcgen05.st has consumed the
        // registers: an arrive issued right behind the loads can overtake them (they queue behind the
        // tensor core's operand reads for hundreds of cycles), and the refill then landed under a
        // warp that was still reading - seen as scales of two stages ahead in one lane quarter.
        if (lane == 0) mbar_arrive(sffree_bar + 8 * s);
        if (lane == 0) mbar_arrive_cluster(os == 0 ? leader_full[0] : (os == 1 ? leader_full[1] : leader_full[2]));
        ++it;
        if (++s == SF_STAGES) { s = 0; ph ^= 1; }
        if (++os == STAGES) { os = 0; oph ^= 1; }
      }
    }
    (void)oph;
  } else {
    // ------------------------------------------------------------------ epilogue (warps 6-9, 12-15)
    // Two warps per tensor-memory lane quarter, 128 accumulator columns each.  Phase 1: tcgen05.ld,
    // * alpha, + bias, pack to 16 bit, all into registers; then the accumulator goes back to the
    // MMA issuer.  Phase 2: each thread stores its 256-byte row segment; it overlaps the next
    // tile's main loop.
    using T = typename OutT<OUT_DT>::type;
    const int q = warp & 3;
    const int half = warp >= 12 ? 1 : 0;
    uint32_t acc_ph = 0;
    int ti = 0;
    const float alpha = __fmul_rn(__ldg(p.a_gs), __ldg(p.b_gs));
    const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + half * 128;
    const uint32_t leader_tempty = map_to_cta(tempty_bar, 0);
    for (int t = cluster_id; t < num_tiles; t += num_clusters) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      const int row = tm * BMP + (int)rank * 128 + q * 32 + lane;
      const int col0 = tn * BN + half * 128;
      const uint32_t bias_s = sBias + (uint32_t)(half * 4 + q) * 512u;
      if (p.bias != nullptr) {
        // this warp's 128 bias values go to shared memory while the tile's MMAs are still running, so
        // that the drain below - which sits between two tiles - only adds broadcast shared-memory loads
        float b4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int n = col0 + lane * 4 + i;
          b4[i] = n < p.N ? load_bias(p.bias, p.bias_dt, n) : 0.0f;
        }
        st_shared_v4f(bias_s + lane * 16, b4[0], b4[1], b4[2], b4[3]);
        __syncwarp();
      }
      if (!mbar_wait(tfull_bar, acc_ph)) { if (lane == 0) atomicExch(p.status, kStatusTimeoutEpilogue); break; }
      tc_fence_after();
      if (warp == 6 && lane == 0) AC4K_TR(1, ti, 0);
      if (lane == 0 && ti < 16) AC4K_TRG(4 + rank, ti * 8 + q + 4 * half, 0);
      uint32_t w[64];
      if (p.bias == nullptr) {
        // two 64-column loads: each load-and-wait costs a full tensor-memory round trip, and this
        // drain is on the critical path between two tiles
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[64];
          tmem_ld_32x32b_x64_sync(t_row + c * 64, r);
#pragma unroll
          for (int i = 0; i < 32; ++i)
            w[c * 32 + i] = (OUT_DT == AC4K_DT_BF16) ? scale_pack_bf16x2(r[2 * i], r[2 * i + 1], alpha)
                                                     : scale_pack_f16x2(r[2 * i], r[2 * i + 1], alpha);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[64];
          tmem_ld_32x32b_x64_sync(t_row + c * 64, r);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float4 bb = ld_shared_v4f(bias_s + (c * 16 + i) * 16);
            if (OUT_DT == AC4K_DT_BF16) {
              w[c * 32 + 2 * i] = scale_bias_pack_bf16x2(r[4 * i], r[4 * i + 1], alpha, bb.x, bb.y);
              w[c * 32 + 2 * i + 1] = scale_bias_pack_bf16x2(r[4 * i + 2], r[4 * i + 3], alpha, bb.z, bb.w);
            } else {
              w[c * 32 + 2 * i] = scale_bias_pack_f16x2(r[4 * i], r[4 * i + 1], alpha, bb.x, bb.y);
              w[c * 32 + 2 * i + 1] = scale_bias_pack_f16x2(r[4 * i + 2], r[4 * i + 3], alpha, bb.z, bb.w);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (warp == 6 && lane == 0) AC4K_TR(1, ti, 1);
      if (lane == 0) mbar_arrive_cluster(leader_tempty);
      if (lane == 0 && ti < 16) AC4K_TRG(4 + rank, ti * 8 + q + 4 * half, 1);
      const int64_t col_base = p.col_off + col0;
      const bool last_tile = t + num_clusters >= num_tiles;
      if (EPI == EPI_REQUANT) {
        // w[] holds this row's 128 outputs as packed bf16 - the quantiser's input format.  Quantise
        // them here (8 blocks of 16 along N, which is the next layer's K) instead of storing them.
        if (row < p.q_rows) {
          const float g = __ldg(p.q_gs);
          const float alpha_o = g == 0.0f ? 0.0f : __frcp_rn(g);
          uint32_t codes[16];
          uint32_t sfw[2] = {0u, 0u};
#pragma unroll
          for (int b = 0; b < 8; ++b) {
            const float amax = amax16_bf16(&w[8 * b]);
            const float s = __fmul_rn(alpha_o, __fmul_rn(amax, kOneSixth));
            uint16_t pk;
            asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pk) : "f"(0.0f), "f"(s));
            const uint32_t sb = pk & 0x7Fu;
            const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)sb, __NV_E4M3);
            const float r = sb ? __fmul_rn(alpha_o, __frcp_rn(__half2float(__half(h)))) : 0.0f;
            codes[2 * b] = quantize8_x2(w[8 * b], w[8 * b + 1], w[8 * b + 2], w[8 * b + 3], r);
            codes[2 * b + 1] = quantize8_x2(w[8 * b + 4], w[8 * b + 5], w[8 * b + 6], w[8 * b + 7], r);
            sfw[b >> 2] |= (row < p.M ? sb : 0u) << (8 * (b & 3));
          }
          const int kt_out = p.N / 64;
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {
            const int c64 = col0 + 64 * h2;
            if (c64 >= p.N) break;
            if (row < p.M) {
              uint4 *dst = reinterpret_cast<uint4 *>(p.q_out + (int64_t)row * (p.N / 2) + c64 / 2);
              __stcs(dst, make_uint4(codes[8 * h2], codes[8 * h2 + 1], codes[8 * h2 + 2], codes[8 * h2 + 3]));
              __stcs(dst + 1, make_uint4(codes[8 * h2 + 4], codes[8 * h2 + 5], codes[8 * h2 + 6], codes[8 * h2 + 7]));
            }
            const int k64 = c64 / 64;
            uint32_t *sfp;
            if (p.q_layout == AC4K_SF_AC4K)
              sfp = reinterpret_cast<uint32_t *>(p.q_sf) + (int64_t)k64 * p.q_rows + row;
            else
              sfp = reinterpret_cast<uint32_t *>(p.q_sf) + ((int64_t)(row / 128) * kt_out + k64) * 128 + (row & 31) * 4 +
                    ((row & 127) >> 5);
            *sfp = sfw[h2];
          }
        }
      } else
      if (row < p.M && !(p.dbg & 8)) {
        // Each lane owns one row, so a store instruction touches 32 different rows however it is
        // shaped; 32-byte stores make every one of those touches a full sector, and a short pause
        // between them keeps the SM's memory pipe free for the barrier and shared-memory traffic of
        // the warps that run the next tile's main loop (the stores have a whole tile time to finish).
        T *dst = static_cast<T *>(p.D) + (int64_t)row * p.ldd + col_base;
        const bool vec32 = col0 + 128 <= p.N && ((p.ldd | p.col_off) * (int64_t)sizeof(T)) % 32 == 0 &&
                           (reinterpret_cast<uintptr_t>(p.D) & 31) == 0;
        if (vec32) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            st_global_v8(reinterpret_cast<uint8_t *>(dst) + 32 * i, w[8 * i], w[8 * i + 1], w[8 * i + 2], w[8 * i + 3],
                         w[8 * i + 4], w[8 * i + 5], w[8 * i + 6], w[8 * i + 7]);
            if (!last_tile) __nanosleep(200);      // nothing left to make room for after the last tile
          }
        } else {
          // ragged right edge or rows that are only 16-byte aligned: 16-byte groups
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (col0 + 8 * i < p.N)
              __stcs(reinterpret_cast<uint4 *>(dst) + i, make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]));
        }
      }
      if (EPI == EPI_GATHER && p.n_dst > 1 && !(p.dbg & 8)) {
        // Fused all-gather: forward this warp's 32 rows x 256 bytes to the other destinations (peer
        // GPUs' buffers, reached over NVLink).  The registers hold one row per lane, which would make
        // every peer store a scatter of 32-byte pieces; NVLink wants long contiguous writes.  So the
        // block is read back from this GPU's L2 in the other orientation - 16 lanes x 16 bytes cover a
        // row's 256 bytes, two rows per instruction - and stored to each peer in that shape.
        __syncwarp();                               // the warp's own stores above are ordered before its loads
        const int row0 = tm * BMP + (int)rank * 128 + q * 32 + (lane >> 4);
        const int cchunk = (lane & 15) * 8;         // first column of this lane's 16-byte piece
        const bool col_ok = col0 + cchunk < p.N;
        const T *src = static_cast<const T *>(p.D) + col_base + cchunk;
        uint4 v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int r = row0 + 2 * i;
          if (col_ok && r < p.M) v[i] = ld_global_cg_v4(src + (int64_t)r * p.ldd);
        }
        // peer after peer (storing each piece to every peer in turn was measured slower at 8 GPUs: 594
        // against 627 GB/s per direction)
#pragma unroll
        for (int d = 1; d < kMaxDst; ++d) {
          if (d >= p.n_dst) break;
          T *peer = static_cast<T *>(p.D_more[d - 1]) + col_base + cchunk;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int r = row0 + 2 * i;
            if (col_ok && r < p.M) st_global_v4(peer + (int64_t)r * p.ldd, v[i]);
          }
        }
      }
      if (warp == 6 && lane == 0) AC4K_TR(1, ti, 2);
      if (warp == 6 && lane == 0) AC4K_TR(3, 0, 3);
      ++ti;
      acc_ph ^= 1;
    }
  }

  if (threadIdx.x == 0) AC4K_TR(3, 0, 4);
  tc_fence_before();
  __syncthreads();
  cluster_sync();          // neither CTA leaves while the other may still read its memory or barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) AC4K_TR(3, 0, 5);
}

template <bool SF_TILED, int OUT_DT, int EPI>
static int launch_pair(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tsa, const CUtensorMap &tsb,
                       const GemmArgs &args, int sms, cudaStream_t stream) {
  auto kern = linear_nvfp4_2cta_kernel<SF_TILED, OUT_DT, EPI>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev]) {
    AC4K_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pair::SMEM_BYTES));
    attr_set[dev] = true;
  }
  // how many CTA pairs can be resident at once (not every SM can be paired on every part); the
  // kernel is persistent, so launching more clusters than that would serialise whole waves
  static int max_clusters[64] = {};
  if (max_clusters[dev] == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms & ~1);
    cfg.blockDim = dim3(pair::kThreadsPair);
    cfg.dynamicSmemBytes = pair::SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    AC4K_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
    if (n < 1) return fail(AC4K_ERR_DEVICE, "no CTA pair of the GEMM kernel fits on this device");
    max_clusters[dev] = n;
  }
  const int num_tiles = args.tiles_m * args.tiles_n;
  int clusters = max_clusters[dev];
  if (num_tiles < clusters) clusters = num_tiles;
  // launched so that its set-up may overlap the previous kernel's tail (see grid_dependency_wait)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters);
  cfg.blockDim = dim3(pair::kThreadsPair);
  cfg.dynamicSmemBytes = pair::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = (args.dbg & 64) ? 0 : 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  AC4K_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, ta, tb, tsa, tsb, args));
  return 0;
}

int launch_linear_2cta(int d_dtype, bool sf_tiled, const CUtensorMap &ta, const CUtensorMap &tb,
                       const CUtensorMap &tsa, const CUtensorMap &tsb, GemmArgs args, cudaStream_t stream) {
  DeviceInfo di;
  if (int e = get_device_info(&di)) return e;
  args.tiles_m = (int)ceil_div(args.M, pair::BMP);
  args.tiles_n = (int)ceil_div(args.N, pair::BN);
  // the instantiations that forward tiles to further destinations or re-quantise the output are
  // separate: their extra registers and code would otherwise slow the plain GEMM down
  if (args.q_out != nullptr) {
    if (d_dtype != AC4K_DT_BF16) return fail(AC4K_ERR_UNSUPPORTED, "the re-quantising epilogue rounds to bf16 first");
    return sf_tiled ? launch_pair<true, AC4K_DT_BF16, EPI_REQUANT>(ta, tb, tsa, tsb, args, di.sms, stream)
                    : launch_pair<false, AC4K_DT_BF16, EPI_REQUANT>(ta, tb, tsa, tsb, args, di.sms, stream);
  }
  const bool gather = args.n_dst > 1;
  if (d_dtype == AC4K_DT_BF16) {
    if (gather)
      return sf_tiled ? launch_pair<true, AC4K_DT_BF16, EPI_GATHER>(ta, tb, tsa, tsb, args, di.sms, stream)
                      : launch_pair<false, AC4K_DT_BF16, EPI_GATHER>(ta, tb, tsa, tsb, args, di.sms, stream);
    return sf_tiled ? launch_pair<true, AC4K_DT_BF16, EPI_PLAIN>(ta, tb, tsa, tsb, args, di.sms, stream)
                    : launch_pair<false, AC4K_DT_BF16, EPI_PLAIN>(ta, tb, tsa, tsb, args, di.sms, stream);
  }
  if (d_dtype == AC4K_DT_FP16) {
    if (gather)
      return sf_tiled ? launch_pair<true, AC4K_DT_FP16, EPI_GATHER>(ta, tb, tsa, tsb, args, di.sms, stream)
                      : launch_pair<false, AC4K_DT_FP16, EPI_GATHER>(ta, tb, tsa, tsb, args, di.sms, stream);
    return sf_tiled ? launch_pair<true, AC4K_DT_FP16, EPI_PLAIN>(ta, tb, tsa, tsb, args, di.sms, stream)
                    : launch_pair<false, AC4K_DT_FP16, EPI_PLAIN>(ta, tb, tsa, tsb, args, di.sms, stream);
  }
  return fail(AC4K_ERR_UNSUPPORTED, "the CTA-pair kernel stores 16-bit outputs only");
}

}  // namespace ac4k
