// NVFP4 block-scaled GEMM for sm_100a, CTA-pair variant (tcgen05 cta_group::2).
//
// Two CTAs of a cluster share one 256 x 256 output tile: CTA r of the pair loads A rows
// [128 r, 128 r + 128) and B rows (output columns) [128 r, 128 r + 128) of the tile, the leader
// CTA issues one tcgen05.mma over both (M = 256, N = 256, each CTA accumulating its 128 rows x
// 256 columns in its own tensor memory, the B halves read from both CTAs' shared memory).  Per
// FLOP this moves a third less operand data from L2 into shared memory than 128 x 256 tiles of
// single CTAs, which is what bounds the single-CTA kernel (measured: its TMA stream alone takes
// longer than its MMAs).  No multicast loads are used.
//
// Roles per CTA (512 threads): warp 0 TMA producer (A, B), warp 1 MMA issuer (leader CTA only),
// warps 2-5 scale warps (shared memory -> tcgen05.st -> tensor memory), warp 10 scale feeder
// (bulk copies of scale bytes, running ahead of the operands), warp 11 barrier watcher (leader
// CTA only), warps 6-9 and 12-15 epilogue (tcgen05.ld, *alpha, +bias, convert, 128-byte-swizzled
// staging in shared memory, TMA store).
// Barriers that gate the MMA (operands landed, scales written, accumulator drained) live in the
// leader CTA and are signalled by both CTAs; barriers that release shared-memory stages and
// publish the accumulator exist in both CTAs and are signalled by two tcgen05.commit each.
#include "gemm_common.cuh"

namespace ac4k {
using namespace ptx;

#ifdef AC4K_TRACE_ENABLED
#define AC4K_TRACEC(it, ev)                                                                 \
  do {                                                                                      \
    if (p.trace != nullptr && cluster_id == 0 && (it) < 128)                                \
      p.trace[((size_t)rank * 128 + (it)) * 8 + (ev)] = clock64();                          \
  } while (0)
#define AC4K_TRACES(it, ev)                                                                 \
  do {                                                                                      \
    if (p.trace != nullptr && cluster_id == 0 && rank == 0 && warp == 2 && lane == 0 && (it) < 128) \
      p.trace[((size_t)2 * 128 + (it)) * 8 + (ev)] = clock64();                             \
  } while (0)
#define AC4K_TRACE(it, ev)                                                                  \
  do {                                                                                      \
    if (p.trace != nullptr && cluster_id == 0 && (it) < 128)                                \
      p.trace[((size_t)rank * 128 + (it)) * 8 + (ev)] = globaltimer();                      \
  } while (0)

#else
#define AC4K_TRACEC(it, ev) do { } while (0)
#define AC4K_TRACES(it, ev) do { } while (0)
#define AC4K_TRACE(it, ev) do { } while (0)
#endif

namespace pair {
static constexpr int BN = 256;                      // output columns of the pair tile
static constexpr int BMP = 256;                     // output rows of the pair tile
static constexpr int A_BYTES = 128 * BKB;           // this CTA's 128 rows of A
static constexpr int B_BYTES = 128 * BKB;           // this CTA's 128 rows of B
static constexpr int SFA_BYTES = K64_PER_STAGE * 512;
static constexpr int SFB_BYTES = 2 * K64_PER_STAGE * 512;
static constexpr int STAGES = 5;                    // operand ring, scale ring and TMEM scale ring
static constexpr int OUT_CHUNK_BYTES = 128 * 128;   // 128 rows x 64 16-bit columns
static constexpr int OUT_CHUNKS = 2;                // double-buffered staging of the epilogue
static constexpr int SMEM_BYTES = STAGES * (A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES) +
                                  OUT_CHUNKS * OUT_CHUNK_BYTES + 1024 + 512;
static constexpr int SFA_COL = 256, SFA_COLS = 16, SFB_COL = SFA_COL + STAGES * SFA_COLS, SFB_COLS = 32;
static_assert(SFB_COL + STAGES * SFB_COLS <= kTmemCols, "tensor memory overflow");
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory overflow");
static constexpr int kThreadsPair = 512;           // 16 warps, see the role list in the kernel
}  // namespace pair

// Walks the (tile, K-step) sequence of one cluster.
struct StageCursor {
  int t, kt, k_tiles, num_tiles, step;
  __device__ StageCursor(int first_tile, int step_, int num_tiles_, int k_tiles_)
      : t(first_tile), kt(0), k_tiles(k_tiles_), num_tiles(num_tiles_), step(step_) {}
  __device__ bool valid() const { return t < num_tiles; }
  __device__ void next() {
    if (++kt == k_tiles) { kt = 0; t += step; }
  }
};

template <bool SF_TILED, int OUT_DT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pair::kThreadsPair, 1)
linear_nvfp4_2cta_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                         const __grid_constant__ CUtensorMap tma_d, const GemmArgs p) {
  using namespace pair;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA = smem_base;
  const uint32_t sB = sA + STAGES * A_BYTES;
  const uint32_t sOut = sB + STAGES * B_BYTES;
  const uint32_t sSFA = sOut + OUT_CHUNKS * OUT_CHUNK_BYTES;
  const uint32_t sSFB = sSFA + STAGES * SFA_BYTES;
  const uint32_t bars = sSFB + STAGES * SFB_BYTES;
  const uint32_t full_bar = bars;                     // [STAGES] leader: A/B of both CTAs landed and all scales in TMEM
  const uint32_t sffull_bar = bars + 8 * STAGES;      // [STAGES] local: scale bytes landed
  const uint32_t empty_bar = bars + 24 * STAGES;      // [STAGES] local: MMAs that used the stage are done
  const uint32_t tfull_bar = bars + 32 * STAGES;      // local: accumulator complete
  const uint32_t tempty_bar = tfull_bar + 8;          // leader: 8 epilogue warps drained the accumulator
  const uint32_t sffree_bar = tempty_bar + 8;         // [STAGES] local: 4 scale warps have read the slot
  const uint32_t ready_word = sffree_bar + 8 * STAGES;   // leader: number of stages the watcher has seen complete
  const uint32_t tmem_slot = ready_word + 8;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_tiles = (p.KT + K64_PER_STAGE - 1) / K64_PER_STAGE;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar + 8 * s, 9);          // producer's expect_tx arrival + 8 scale warps
      mbar_init(sffull_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
      mbar_init(sffree_bar + 8 * s, 4);
    }
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, 16);          // 8 epilogue warps in each CTA
    st_shared_release(ready_word, 0);
    fence_barrier_init();
    prefetch_tmap(&tma_a);
    prefetch_tmap(&tma_b);
    prefetch_tmap(&tma_d);
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

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (A and B)
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * BMP + (int)rank * 128;        // this CTA's rows of A
        const int nb0 = tn * BN + (int)rank * 128;        // this CTA's rows of B
        for (int kt = 0; kt < k_tiles; ++kt) {
          if (!mbar_wait(empty_bar + 8 * s, ph ^ 1)) { atomicExch(p.status, kStatusTimeoutProducer); ok = false; break; }
          AC4K_TRACEC(it, 2);
          ++it;
          const uint32_t leader_full = map_to_cta(full_bar + 8 * s, 0);
          if (rank == 0) mbar_arrive_expect_tx(full_bar + 8 * s, ((p.dbg & 512) ? 1 : 2) * (A_BYTES + B_BYTES));
          if ((p.dbg & 512) && rank == 1) { if (++s == STAGES) { s = 0; ph ^= 1; } continue; }
          if ((p.dbg & 256) && rank == 0) {
            tma_load_2d_local(sA + s * A_BYTES, &tma_a, kt * BKB, m0, full_bar + 8 * s);
            tma_load_2d_local(sB + s * B_BYTES, &tma_b, kt * BKB, nb0, full_bar + 8 * s);
          } else {
            tma_load_2d_pair(sA + s * A_BYTES, &tma_a, kt * BKB, m0, leader_full);
            tma_load_2d_pair(sB + s * B_BYTES, &tma_b, kt * BKB, nb0, leader_full);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA)
    if (lane == 0 && rank == 0) {
      // The MMA pipe accepts a new instruction only as an earlier one retires (about every 128
      // cycles at N = 256), and whatever this thread does between two issues that takes longer
      // than that becomes a bubble in the pipe.  So the per-stage bookkeeping is spread over the
      // gaps between the four MMAs of a stage: the wait for the NEXT stage sits after the first
      // MMA, the commit after the last.
      constexpr uint32_t idesc = make_idesc_mxf4nvf4(BMP, BN);
      // Every mbarrier or tcgen05 instruction holds this thread for roughly 75-110 cycles, and four
      // MMAs (4 x ~92) plus a commit (~109) already fill most of the 512 cycles a stage takes in the
      // pipe.  Waiting on the stage's barriers is therefore delegated to the watcher warp, which
      // publishes a running count of ready stages in shared memory; polling that word costs a
      // shared-memory load (~30 cycles).
      uint32_t s = 0, it = 0;
      bool ok = true;
      const uint64_t adesc0 = make_smem_desc(sA, 16, 1024, kSwizzle128B);
      const uint64_t bdesc0 = make_smem_desc(sB, 16, 1024, kSwizzle128B);
      const int last_nk = p.KT - (k_tiles - 1) * K64_PER_STAGE;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        for (int kt = 0; kt < k_tiles; ++kt) {
          AC4K_TRACEC(it, 0);
          uint32_t seen = ld_shared_volatile(ready_word);
          if (seen <= it) {
            const unsigned long long t0 = globaltimer();
            while ((seen = ld_shared_volatile(ready_word)) <= it) {
              if (globaltimer() - t0 > kWaitTimeoutNs) { seen = 0xFFFFFFFFu; break; }
            }
          }
          if (seen == 0xFFFFFFFFu) { ok = false; break; }
          tc_fence_after();
          const uint32_t t_sfa = tmem_base + SFA_COL + s * SFA_COLS;
          const uint32_t t_sfb = tmem_base + SFB_COL + s * SFB_COLS;
          const uint64_t adesc = adesc0 + (uint64_t)(s * (A_BYTES >> 4));
          const uint64_t bdesc = bdesc0 + (uint64_t)(s * (B_BYTES >> 4));
          AC4K_TRACEC(it, 1);
          if (kt + 1 < k_tiles || last_nk == K64_PER_STAGE) {
            mma_mxf4nvf4_pair(tmem_base, adesc, bdesc, idesc, t_sfa, t_sfb, kt > 0 ? 1u : 0u);
            mma_mxf4nvf4_pair(tmem_base, adesc + 2, bdesc + 2, idesc, t_sfa + 4, t_sfb + 8, 1u);
            mma_mxf4nvf4_pair(tmem_base, adesc + 4, bdesc + 4, idesc, t_sfa + 8, t_sfb + 16, 1u);
            mma_mxf4nvf4_pair(tmem_base, adesc + 6, bdesc + 6, idesc, t_sfa + 12, t_sfb + 24, 1u);
          } else {
            for (int j = 0; j < last_nk; ++j)
              mma_mxf4nvf4_pair(tmem_base, adesc + 2 * j, bdesc + 2 * j, idesc, t_sfa + j * 4, t_sfb + j * 8,
                                (kt > 0 || j > 0) ? 1u : 0u);
          }
          AC4K_TRACEC(it, 3);
          tc_commit_pair_both(empty_bar + 8 * s, 3);                 // stage free in both CTAs
          if (kt == k_tiles - 1) tc_commit_pair_both(tfull_bar, 3);  // accumulator complete in both CTAs
          AC4K_TRACEC(it, 5);
          ++it;
          if (++s == STAGES) s = 0;
        }
      }
      if (!ok) atomicExch(p.status, kStatusTimeoutMma);
    }
  } else if (warp == 11) {
    // ------------------------------------------------------------------ barrier watcher (leader CTA)
    // Waits, in the order the MMA issuer consumes them, for the accumulator hand-back (first stage
    // of a tile) and for each stage's operands and scales, and publishes the count.
    if (lane == 0 && rank == 0) {
      uint32_t s = 0, ph = 0, acc_ph = 0, count = 0;
      bool ok = true;
      for (StageCursor c(cluster_id, num_clusters, num_tiles, k_tiles); c.valid(); c.next()) {
        if (c.kt == 0) {
          ok = mbar_wait(tempty_bar, acc_ph ^ 1);
          acc_ph ^= 1;
        }
        ok = ok && mbar_wait(full_bar + 8 * s, ph);
        if (!ok) break;
        AC4K_TRACEC(count, 4);
        st_shared_release(ready_word, ++count);
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
      if (!ok) {
        atomicExch(p.status, kStatusTimeoutMma);
        st_shared_release(ready_word, 0xFFFFFFFFu);
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------------ scale feeder
    // Issues the bulk copies of the scale bytes into the shared-memory scale ring as soon as the
    // four scale warps have read a slot into registers: the scales run ahead of the operands
    // and never sit on the MMA's critical path.
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      for (StageCursor c(cluster_id, num_clusters, num_tiles, k_tiles); c.valid(); c.next()) {
        if (!mbar_wait(sffree_bar + 8 * s, ph ^ 1)) { atomicExch(p.status, kStatusTimeoutSf); break; }
        int tm, tn;
        tile_coords(c.t, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * BMP + (int)rank * 128, n0 = tn * BN;
        const int nk = min(K64_PER_STAGE, p.KT - c.kt * K64_PER_STAGE);
        const uint32_t bar = sffull_bar + 8 * s;
        const int64_t k64 = (int64_t)c.kt * K64_PER_STAGE;
        if (SF_TILED) {
          const int64_t mt = m0 / 128;
          const bool a_ok = mt * 128 < p.rows_sfa;
          const int nb_valid = min(2, (p.rows_sfb - n0) / 128);
          mbar_arrive_expect_tx(bar, (a_ok ? nk * 512 : 0) + nb_valid * nk * 512);
          if (a_ok) bulk_load_1d_local(sSFA + s * SFA_BYTES, p.sfa + (mt * p.KT + k64) * 512, nk * 512, bar);
          for (int nb = 0; nb < nb_valid; ++nb)
            bulk_load_1d_local(sSFB + s * SFB_BYTES + nb * (K64_PER_STAGE * 512),
                               p.sfb + ((int64_t)(n0 / 128 + nb) * p.KT + k64) * 512, nk * 512, bar);
        } else {
          const int ra = 4 * max(0, min(128, p.rows_sfa - m0)), rb = 4 * min(BN, p.rows_sfb - n0);
          mbar_arrive_expect_tx(bar, nk * (ra + rb));
          for (int j = 0; j < nk; ++j) {
            if (ra > 0)
              bulk_load_1d_local(sSFA + s * SFA_BYTES + j * 512, p.sfa + ((k64 + j) * p.rows_sfa + m0) * 4, ra, bar);
            bulk_load_1d_local(sSFB + s * SFB_BYTES + j * 1024, p.sfb + ((k64 + j) * p.rows_sfb + n0) * 4, rb, bar);
          }
        }
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ scale warps
    // shared memory -> registers -> tensor memory.  A slot of the tensor-memory scale ring is
    // rewritten once the MMAs that used it have completed (the stage's `empty` barrier).
    const int q = warp & 3;
    uint32_t s = 0, ph = 0;
    int it = 0;
    bool ok = true;
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    for (StageCursor cur(cluster_id, num_clusters, num_tiles, k_tiles); cur.valid() && ok; cur.next()) {
      AC4K_TRACES(it, 0);
      if (!mbar_wait(sffull_bar + 8 * s, ph)) { if (lane == 0) atomicExch(p.status, kStatusTimeoutSf); ok = false; break; }
      AC4K_TRACES(it, 1);
      const uint8_t *a_src = smem_gen + (sSFA + s * SFA_BYTES - smem_base);
      const uint8_t *b_src = smem_gen + (sSFB + s * SFB_BYTES - smem_base);
      uint32_t ra[16], rb[32];
      if (SF_TILED) {
#pragma unroll
        for (int j = 0; j < K64_PER_STAGE; ++j) {
          const uint4 v = *reinterpret_cast<const uint4 *>(a_src + j * 512 + lane * 16);
          ra[j * 4 + 0] = v.x; ra[j * 4 + 1] = v.y; ra[j * 4 + 2] = v.z; ra[j * 4 + 3] = v.w;
#pragma unroll
          for (int nb = 0; nb < 2; ++nb) {
            const uint4 w = *reinterpret_cast<const uint4 *>(b_src + (nb * K64_PER_STAGE + j) * 512 + lane * 16);
            rb[j * 8 + nb * 4 + 0] = w.x; rb[j * 8 + nb * 4 + 1] = w.y;
            rb[j * 8 + nb * 4 + 2] = w.z; rb[j * 8 + nb * 4 + 3] = w.w;
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < K64_PER_STAGE; ++j) {
#pragma unroll
          for (int g = 0; g < 4; ++g) ra[j * 4 + g] = reinterpret_cast<const uint32_t *>(a_src + j * 512)[g * 32 + lane];
#pragma unroll
          for (int g = 0; g < 8; ++g) rb[j * 8 + g] = reinterpret_cast<const uint32_t *>(b_src + j * 1024)[g * 32 + lane];
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(sffree_bar + 8 * s);      // this warp holds the slot in registers
      AC4K_TRACES(it, 2);
      // tensor-memory slot s is free once the MMAs of the step that last used it are done
      if (!mbar_wait(empty_bar + 8 * s, ph ^ 1)) { if (lane == 0) atomicExch(p.status, kStatusTimeoutSf); ok = false; break; }
      AC4K_TRACES(it, 3);
      tc_fence_after();
      tmem_st_32x32b_x16(lane_base + SFA_COL + s * SFA_COLS, ra);
      tmem_st_32x32b_x32(lane_base + SFB_COL + s * SFB_COLS, rb);
      AC4K_TRACES(it, 4);
      tmem_st_wait();
      AC4K_TRACES(it, 5);
      tc_fence_before();
      __syncwarp();
      if (warp == 2 && lane == 0) AC4K_TRACEC(it, 6);
      ++it;
      if (lane == 0) mbar_arrive_cluster(map_to_cta(full_bar + 8 * s, 0));
      if (++s == STAGES) { s = 0; ph ^= 1; }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 6-9, 12-15)
    // Two warps per tensor-memory lane quarter, each draining 128 of the 256 accumulator columns.
    // Phase 1: tcgen05.ld, * alpha, + bias, pack to 16 bit, all into registers, then the
    // accumulator is handed back to the MMA issuer at once.  Phase 2 (two rounds of swizzled
    // staging + TMA store per tile) overlaps the next tile's main loop.
    using T = typename OutT<OUT_DT>::type;
    const int q = warp & 3;
    const int half = warp >= 12 ? 1 : 0;
    const int row_l = q * 32 + lane;
    const bool store_thread = (warp == 6 && lane == 0);
    uint32_t acc_ph = 0;
    int ti = 0;
    const float alpha = __fmul_rn(__ldg(p.a_gs), __ldg(p.b_gs));
    const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + half * 128;
    const uint32_t leader_tempty = map_to_cta(tempty_bar, 0);
    for (int t = cluster_id; t < num_tiles; t += num_clusters) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      const int m0 = tm * BMP + (int)rank * 128, n0 = tn * BN;
      if (!mbar_wait(tfull_bar, acc_ph)) { if (lane == 0) atomicExch(p.status, kStatusTimeoutEpilogue); break; }
      tc_fence_after();
      if (warp == 6 && lane == 0) AC4K_TRACEC(120 + ti, 7);
      uint32_t w[64];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + half * 128 + c * 32;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float v0 = __fmul_rn(__uint_as_float(r[2 * i]), alpha), v1 = __fmul_rn(__uint_as_float(r[2 * i + 1]), alpha);
          if (p.bias != nullptr) {
            if (col + 2 * i < p.N) v0 = __fadd_rn(v0, load_bias(p.bias, p.bias_dt, col + 2 * i));
            if (col + 2 * i + 1 < p.N) v1 = __fadd_rn(v1, load_bias(p.bias, p.bias_dt, col + 2 * i + 1));
          }
          if (OUT_DT == AC4K_DT_BF16) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
            w[c * 16 + i] = *reinterpret_cast<uint32_t *>(&h);
          } else {
            __half2 h = __floats2half2_rn(v0, v1);
            w[c * 16 + i] = *reinterpret_cast<uint32_t *>(&h);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (warp == 6 && lane == 0 && p.trace != nullptr && cluster_id == 0) p.trace[((size_t)rank * 128 + 112 + ti) * 8 + 7] = clock64();
      if (lane == 0) mbar_arrive_cluster(leader_tempty);
      if (!(p.dbg & 8)) {
        // staging buffer `half` holds columns [half*128 + round*64, +64) in round `round`
#pragma unroll
        for (int round = 0; round < 2; ++round) {
          if (store_thread) bulk_wait_group_read0();     // earlier stores have finished reading the staging
          named_barrier_sync(1, 256);
          // 128-byte-swizzled staging: 16-byte chunk index XOR (row % 8), as the TMA store expects
          uint8_t *buf = smem_gen + (sOut + half * OUT_CHUNK_BYTES - smem_base) + row_l * 128;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int chunk = i ^ (row_l & 7);
            *reinterpret_cast<uint4 *>(buf + chunk * 16) =
                make_uint4(w[round * 32 + 4 * i], w[round * 32 + 4 * i + 1], w[round * 32 + 4 * i + 2],
                           w[round * 32 + 4 * i + 3]);
          }
          fence_proxy_async_smem();
          named_barrier_sync(1, 256);
          if (store_thread) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int col0 = n0 + h * 128 + round * 64;
              if (m0 < p.M && col0 < p.N) tma_store_2d(&tma_d, col0 * (int)sizeof(T), m0, sOut + h * OUT_CHUNK_BYTES);
            }
            bulk_commit_group();
          }
        }
      }
      if (ti < 7) ++ti;
      acc_ph ^= 1;
    }
    if (store_thread) bulk_wait_group0();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();          // neither CTA leaves while the other may still read its memory or barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <bool SF_TILED, int OUT_DT>
static int launch_pair(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &td, const GemmArgs &args,
                       int sms, cudaStream_t stream) {
  auto kern = linear_nvfp4_2cta_kernel<SF_TILED, OUT_DT>;
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
  kern<<<2 * clusters, pair::kThreadsPair, pair::SMEM_BYTES, stream>>>(ta, tb, td, args);
  AC4K_LAUNCH_CHECK("linear_nvfp4_2cta_kernel");
  return 0;
}

int launch_linear_2cta(int d_dtype, bool sf_tiled, const CUtensorMap &ta, const CUtensorMap &tb,
                       const CUtensorMap &td, GemmArgs args, cudaStream_t stream) {
  DeviceInfo di;
  if (int e = get_device_info(&di)) return e;
  args.tiles_m = (int)ceil_div(args.M, pair::BMP);
  args.tiles_n = (int)ceil_div(args.N, pair::BN);
  if (d_dtype == AC4K_DT_BF16)
    return sf_tiled ? launch_pair<true, AC4K_DT_BF16>(ta, tb, td, args, di.sms, stream)
                    : launch_pair<false, AC4K_DT_BF16>(ta, tb, td, args, di.sms, stream);
  if (d_dtype == AC4K_DT_FP16)
    return sf_tiled ? launch_pair<true, AC4K_DT_FP16>(ta, tb, td, args, di.sms, stream)
                    : launch_pair<false, AC4K_DT_FP16>(ta, tb, td, args, di.sms, stream);
  return fail(AC4K_ERR_UNSUPPORTED, "the CTA-pair kernel stores 16-bit outputs only");
}

}  // namespace ac4k
