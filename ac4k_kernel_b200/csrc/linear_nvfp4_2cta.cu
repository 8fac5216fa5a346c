// NVFP4 block-scaled GEMM for sm_100a, CTA-pair variant (tcgen05 cta_group::2).
//
// Two CTAs of a cluster share one 256 x 256 output tile: CTA r of the pair loads A rows
// [128 r, 128 r + 128) and B rows (output columns) [128 r, 128 r + 128) of the tile, the leader
// CTA issues one tcgen05.mma over both (M = 256, N = 256, each CTA accumulating its 128 rows x
// 256 columns in its own tensor memory, the B halves read from both CTAs' shared memory).  Per
// FLOP this moves a third less operand data from L2 into shared memory than 128 x 256 tiles of
// single CTAs.  No multicast loads are used.
//
// A pipeline stage is K = 256 elements: one 128-row x 128-byte box of A, one of B, and the block
// scales of the stage (2 KB for this CTA's A rows, 4 KB for all 256 B rows), 38 KB per CTA, five
// stages.  The scales go from shared to tensor memory with tcgen05.cp, issued by the MMA warp right
// in front of the MMAs that use them: the copies run in issue order with the MMAs and overlap them
// (measured: 12 copies + 4 MMAs take 523 cycles, the 4 MMAs alone 520), so no other warp and no
// barrier stands between a stage's arrival and its MMAs.
//
// Roles per CTA (448 threads); every role that issues TMA or tcgen05 instructions runs with its whole
// warp converged and predicates those instructions on one elected lane (see elect_one()):
//   warp 0      TMA producer: A, B and - for tiled scales - three scale boxes per stage, all
//               completing on the leader CTA's barrier of the stage
//   warp 1      MMA issuer (leader CTA only): per stage 12 scale copies, 4 MMAs, 1 commit
//   warps 2-5   only for scales in the row layout [K/64][rows][4] when M or N is not a multiple of 4:
//               each warp takes every fourth stage, reads the stage's scale words from global
//               memory and writes them to shared memory in the 32 x 16-byte order tcgen05.cp wants
//   warps 6-13  epilogue: tcgen05.ld of 128 accumulator columns per warp into registers
//               (* alpha, + bias, packed to 16 bit), hand the accumulator back, then store
// Scales in the row layout, M and N multiples of 4 (SF_MODE == kSfPerm): tcgen05.cp puts word w of a 512-byte
// chunk on lane w / 4, column w % 4, and the MMA takes the scales of its row q * 32 + l from lane l, column q.
// So the 512 bytes that hold the scale words of 128 consecutive rows in row order are the chunk of those rows in
// the order (4 l + q -> q * 32 + l): the operand boxes are loaded with their rows in that order (rank-3 tensor
// maps: bytes, row / 4, row % 4), the scales arrive by TMA as they lie in memory, and nothing is re-ordered by
// threads (the generic-proxy stores of the scale warps slow the tensor pipe down by 12 - 30 % per stage).  The
// accumulator's rows and columns come out in the same order; the epilogue maps its lane to row 4 l + q, pairs
// the columns back in registers and stores through a rank-3 map of the output.
// Barriers that gate the MMA live in the leader CTA and are signalled by both CTAs; barriers that
// release stages / publish the accumulator exist in both CTAs and are signalled by one
// tcgen05.commit whose arrival fans out to both.
#include "gemm_common.cuh"

namespace ac4k {
using namespace ptx;

#ifdef AC4K_TRACE_ENABLED
// region 0: MMA issuer, region 1: epilogue warp 6 (both leader CTA, cluster 0), region 3: kernel phases
#define AC4K_TR(region, it, ev)                                                              \
  do {                                                                                      \
    if (p.trace != nullptr && cluster_id == 0 && rank == 0 && (it) < 128)                   \
      p.trace[((size_t)(region) * 128 + (it)) * 8 + (ev)] = clock64();                      \
  } while (0)
// region 5: one line per launch (index from a counter in the last slot of region 4): wall-clock ns and
// clock64 at kernel start and end of cluster 0's leader, for the gaps between launches and the SM clock
#define AC4K_TR_LAUNCH(begin)                                                                \
  do {                                                                                      \
    if (p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {                        \
      unsigned long long *ctr = p.trace + ((size_t)4 * 128 + 127) * 8;                      \
      if (begin) launch_slot = (unsigned)atomicAdd(ctr, 1ull) & 127u;                       \
      unsigned long long *line = p.trace + ((size_t)5 * 128 + launch_slot) * 8;             \
      line[(begin) ? 0 : 2] = globaltimer();                                                \
      line[(begin) ? 1 : 3] = clock64();                                                    \
    }                                                                                       \
  } while (0)
#else
#define AC4K_TR(region, it, ev) do { } while (0)
#define AC4K_TR_LAUNCH(begin) do { } while (0)
#endif

namespace pair {
static constexpr int BN = 256;                      // output columns of the pair tile
static constexpr int BMP = 256;                     // output rows of the pair tile
static constexpr int KS = 4;                        // K = 64 steps per stage
static constexpr int A_BYTES = 128 * BKB;           // this CTA's 128 rows of A, K = 256
static constexpr int B_BYTES = 128 * BKB;           // this CTA's 128 rows of B, K = 256
static constexpr int SFA_BYTES = KS * 512;          // [K step][32 x 16 B]
static constexpr int SFB_BYTES = 2 * KS * 512;      // [128-row block of B][K step][32 x 16 B]
static constexpr int STAGE_TX = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;    // bytes one CTA's TMA loads of a stage bring
static constexpr int STAGES = 5;
// Tensor memory (512 columns): two accumulators of 256 columns that share 48 columns, and the scales
// of one stage.  Tiles alternate between the accumulators; the shared columns are the last 48 of the
// first accumulator's tile and the first 48 of the second one's, so between two tiles only those 48
// columns have to be read out before the next tile's first MMA may write them - the other 208 are
// drained while the next tile's MMAs already run.
static constexpr int ACC1_COL = 208;                // accumulator 0: columns 0 - 255, accumulator 1: 208 - 463
static constexpr int SHARED_COLS = BN - ACC1_COL;   // 48
static constexpr int SF_COL = ACC1_COL + BN;        // 464: per K step 4 columns for A, then 8 per K step for B
static constexpr int SF_COLS = KS * 12;
static constexpr int BIAS_BYTES = 8 * 128 * 4;      // one tile's bias as fp32, 128 columns per epilogue warp
static constexpr int OUT_STAGE_BYTES = 32 * 128;    // per epilogue warp: 32 rows x 64 columns of 16-bit outputs
static constexpr int BAR_BYTES = 256;
// no slack for aligning the base: the kernel declares the array 1024-byte aligned and checks it
static constexpr int SMEM_BYTES = STAGES * STAGE_TX + 8 * OUT_STAGE_BYTES + BIAS_BYTES + BAR_BYTES;
static_assert(SF_COL + SF_COLS <= kTmemCols, "tensor memory overflow");
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory overflow");
static constexpr int kThreadsPair = 448;           // 14 warps: 144 registers per thread for the epilogue
}  // namespace pair

// N accumulator columns starting at COL0 of this thread's 128-column segment: * alpha (+ bias from shared
// memory), rounded to the 16-bit output type, two per word into w[COL0 / 2 ...].
template <int OUT_DT, int COL0, int N>
__device__ __forceinline__ void pack_cols(const uint32_t (&r)[N], uint32_t (&w)[64], float alpha, bool has_bias, uint32_t bias_s) {
  static_assert(COL0 % 4 == 0 && N % 4 == 0, "whole 16-byte bias groups");
  if (!has_bias) {
#pragma unroll
    for (int i = 0; i < N / 2; ++i)
      w[COL0 / 2 + i] = (OUT_DT == AC4K_DT_BF16) ? scale_pack_bf16x2(r[2 * i], r[2 * i + 1], alpha)
                                                 : scale_pack_f16x2(r[2 * i], r[2 * i + 1], alpha);
  } else {
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      const float4 bb = ld_shared_v4f(bias_s + (COL0 + 4 * i) * 4);
      if (OUT_DT == AC4K_DT_BF16) {
        w[COL0 / 2 + 2 * i] = scale_bias_pack_bf16x2(r[4 * i], r[4 * i + 1], alpha, bb.x, bb.y);
        w[COL0 / 2 + 2 * i + 1] = scale_bias_pack_bf16x2(r[4 * i + 2], r[4 * i + 3], alpha, bb.z, bb.w);
      } else {
        w[COL0 / 2 + 2 * i] = scale_bias_pack_f16x2(r[4 * i], r[4 * i + 1], alpha, bb.x, bb.y);
        w[COL0 / 2 + 2 * i + 1] = scale_bias_pack_f16x2(r[4 * i + 2], r[4 * i + 3], alpha, bb.z, bb.w);
      }
    }
  }
}

// One output word of the row-permuted variant: accumulator values of output columns col, col + 1 of this thread's
// 128-column segment.
template <int OUT_DT, bool BIAS>
__device__ __forceinline__ uint32_t pack_pair(uint32_t lo, uint32_t hi, float alpha, uint32_t bias_s, int col) {
  if (!BIAS) return (OUT_DT == AC4K_DT_BF16) ? scale_pack_bf16x2(lo, hi, alpha) : scale_pack_f16x2(lo, hi, alpha);
  const float2 bb = ld_shared_v2f(bias_s + col * 4);
  return (OUT_DT == AC4K_DT_BF16) ? scale_bias_pack_bf16x2(lo, hi, alpha, bb.x, bb.y) : scale_bias_pack_f16x2(lo, hi, alpha, bb.x, bb.y);
}

// Drain of this warp's 128 accumulator columns in the row-permuted variant.  Column c holds output column
// 4 (c % 32) + c / 32 of the segment: output columns 4 l, 4 l + 1 (word 2 l) come from columns l and 32 + l, output
// columns 4 l + 2, 4 l + 3 (word 2 l + 1) from 64 + l and 96 + l.  Step S = 2 u + v reads columns 64 u + 16 v + [0, 16)
// and the 16 columns 32 further on and packs words 2 l + u, l = 16 v + [0, 16); the first two steps are read together,
// later ones are in flight while a step is packed.
template <int S>
__device__ __forceinline__ void drain_issue(uint32_t t_row, uint32_t (&lo)[16], uint32_t (&hi)[16]) {
  tmem_ld_32x32b_x16(t_row + (S >> 1) * 64 + (S & 1) * 16, lo);
  tmem_ld_32x32b_x16(t_row + (S >> 1) * 64 + (S & 1) * 16 + 32, hi);
}
template <int OUT_DT, bool BIAS, int S>
__device__ __forceinline__ void drain_pack(uint32_t (&w)[64], const uint32_t (&lo)[16], const uint32_t (&hi)[16], float alpha,
                                           uint32_t bias_s) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    constexpr int u = S >> 1, v = S & 1;
    w[2 * (16 * v + i) + u] = pack_pair<OUT_DT, BIAS>(lo[i], hi[i], alpha, bias_s, 4 * (16 * v + i) + 2 * u);
  }
}
// Steps in the order S0 .. S3; after the first two (which must cover the columns both accumulators share, if this
// warp has any of them: `arrive`) the shared columns are reported free.
template <int OUT_DT, bool BIAS, int S0, int S1, int S2, int S3>
__device__ __forceinline__ void drain_permuted(uint32_t (&w)[64], uint32_t t_row, bool arrive, float alpha, uint32_t bias_s,
                                               int lane, uint32_t leader_shared_free) {
  uint32_t a_lo[16], a_hi[16], b_lo[16], b_hi[16];
  drain_issue<S0>(t_row, a_lo, a_hi);
  drain_issue<S1>(t_row, b_lo, b_hi);
  tmem_ld_wait();
  tmem_pin(a_lo);
  tmem_pin(a_hi);
  tmem_pin(b_lo);
  tmem_pin(b_hi);
  if (arrive) {
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster(leader_shared_free);
  }
  drain_pack<OUT_DT, BIAS, S0>(w, a_lo, a_hi, alpha, bias_s);
  drain_issue<S2>(t_row, a_lo, a_hi);
  drain_pack<OUT_DT, BIAS, S1>(w, b_lo, b_hi, alpha, bias_s);
  tmem_ld_wait();
  tmem_pin(a_lo);
  tmem_pin(a_hi);
  drain_issue<S3>(t_row, b_lo, b_hi);
  drain_pack<OUT_DT, BIAS, S2>(w, a_lo, a_hi, alpha, bias_s);
  tmem_ld_wait();
  tmem_pin(b_lo);
  tmem_pin(b_hi);
  drain_pack<OUT_DT, BIAS, S3>(w, b_lo, b_hi, alpha, bias_s);
}

// where the block scales come from: kSfWarps - row layout, re-ordered by warps 2-5; kSfTiled - 128x4 tiles by TMA;
// kSfPerm - row layout by TMA, operand rows permuted instead
enum { kSfWarps = 0, kSfTiled = 1, kSfPerm = 2 };

template <int SF_MODE, int OUT_DT, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pair::kThreadsPair, 1)
linear_nvfp4_2cta_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                         const __grid_constant__ CUtensorMap tma_sfa, const __grid_constant__ CUtensorMap tma_sfb,
                         const __grid_constant__ DstMaps dmaps, const GemmArgs p) {
  using namespace pair;
  constexpr bool SF_TILED = SF_MODE != kSfWarps;      // the scales arrive by TMA, laid out for tcgen05.cp
  constexpr bool PERM = SF_MODE == kSfPerm;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = smem_u32(smem_raw);
  if (smem_base & 1023u) {      // the swizzled boxes need 1024-byte alignment; never seen, but not promised either
    if (threadIdx.x == 0) atomicExch(p.status, kStatusSmemAlign);
    return;
  }
  const uint32_t sA = smem_base;
  const uint32_t sB = sA + STAGES * A_BYTES;
  const uint32_t sSFA = sB + STAGES * B_BYTES;
  const uint32_t sSFB = sSFA + STAGES * SFA_BYTES;
  const uint32_t sOut = sSFB + STAGES * SFB_BYTES;     // [8 epilogue warps][32 rows x 128 B], swizzled like the TMA box
  const uint32_t sBias = sOut + 8 * OUT_STAGE_BYTES;   // [8 epilogue warps][128] fp32
  const uint32_t bars = sBias + BIAS_BYTES;
  const uint32_t full_bar = bars;                     // [STAGES] leader: operands and scales of both CTAs are in shared memory
  const uint32_t empty_bar = full_bar + 8 * STAGES;   // [STAGES] both: the MMAs that used the stage are done
  const uint32_t tfull_bar = empty_bar + 8 * STAGES;  // [2] both: accumulator complete
  const uint32_t tempty_bar = tfull_bar + 16;         // [2] leader: 16 epilogue warps drained the accumulator
  const uint32_t shared_free_bar = tempty_bar + 16;   // leader: the 8 warps that own the shared columns have read them
  const uint32_t tmem_slot = shared_free_bar + 8;
  uint8_t *smem_gen = smem_raw;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_tiles = (p.KT + KS - 1) / KS;
  const int last_nk = p.KT - (k_tiles - 1) * KS;      // K = 64 steps in the last stage of a tile

  if (threadIdx.x == 0) AC4K_TR(3, 0, 0);
#ifdef AC4K_TRACE_ENABLED
  unsigned launch_slot = 0;
#endif
  AC4K_TR_LAUNCH(true);
#ifdef AC4K_TRACE_ENABLED
  if (p.trace != nullptr && rank == 0 && threadIdx.x == 0 && cluster_id < 120) p.trace[((size_t)4 * 128 + cluster_id) * 8 + 0] = globaltimer();
#endif
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar + 8 * s, SF_TILED ? 1 : 3);   // producer's expect_tx arrival (+ one scale warp per CTA)
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar + 8 * a, 1);
      mbar_init(tempty_bar + 8 * a, 16);        // 8 epilogue warps in each CTA
    }
    mbar_init(shared_free_bar, 8);              // 4 of them in each CTA
    fence_barrier_init();
    prefetch_tmap(&tma_a);
    prefetch_tmap(&tma_b);
    if (SF_TILED) {
      prefetch_tmap(&tma_sfa);
      prefetch_tmap(&tma_sfb);
    }
    if (EPI != EPI_REQUANT) prefetch_tmap(&dmaps.m[0]);
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
  if (warp == 2 && cluster_id < num_tiles && !AC4K_DBG(p, 128)) {
    // While the kernel before this one may still be running: ask L2 for the operands of this CTA's first
    // stages.  A prefetch returns no data, so the dependency wait below still orders every real read.
    const uint32_t el = elect_one();
    int tm, tn;
    tile_coords(cluster_id, p.tiles_m, p.tiles_n, tm, tn);
    const int m0 = tm * BMP + (int)rank * 128, nb0 = tn * BN + (int)rank * 128;
    const int npre = k_tiles < STAGES ? k_tiles : STAGES;
    for (int kt = 0; kt < npre; ++kt) {
      if (PERM) {
        tma_prefetch_3d_if(el, &tma_a, kt * BKB, m0 >> 2, 0);
        tma_prefetch_3d_if(el, &tma_b, kt * BKB, nb0 >> 2, 0);
      } else {
        tma_prefetch_2d_if(el, &tma_a, kt * BKB, m0);
        tma_prefetch_2d_if(el, &tma_b, kt * BKB, nb0);
      }
    }
  }
  grid_dependency_wait();
  if (threadIdx.x == 0) AC4K_TR(3, 0, 1);
#ifdef AC4K_TRACE_ENABLED
  if (p.trace != nullptr && rank == 0 && threadIdx.x == 0 && cluster_id < 120) p.trace[((size_t)4 * 128 + cluster_id) * 8 + 1] = globaltimer();
#endif

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    const uint32_t el = elect_one();
    uint32_t s = 0, ph = 0;
    const uint32_t leader_full0 = map_to_cta(full_bar, 0);
    for (int t = cluster_id; t < num_tiles; t += num_clusters) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      const int m0 = tm * BMP + (int)rank * 128;        // this CTA's rows of A
      const int nb0 = tn * BN + (int)rank * 128;        // this CTA's rows of B
      const int sfa_row0 = (m0 / 128) * p.KT;           // tiled scales: row of [row block][K step] x 512 B
      const int sfb_row0 = (tn * (BN / 128)) * p.KT;
      bool ok = true;
      for (int kt = 0; kt < k_tiles; ++kt) {
        ok = warp_all(mbar_wait(empty_bar + 8 * s, ph ^ 1, p.wait_ns));
        if (!ok) break;
        const uint32_t lf = leader_full0 + 8 * s;
        if (AC4K_DBG(p, 256) && kt == 0 && t == cluster_id) {
          // wait-expiry test (debug-hook builds): this stage is never loaded, nothing arrives on its barrier, and
          // every role of the pair must find its way out through its bounded waits
          if (++s == STAGES) { s = 0; ph ^= 1; }
          continue;
        }
        // the leader announces the bytes of both CTAs; K steps past the end of K arrive as zeros
        // (or as the next row block's scales, unused) and count all the same
        if (rank == 0) mbar_arrive_expect_tx_if(el, full_bar + 8 * s, 2 * (SF_TILED ? STAGE_TX : A_BYTES + B_BYTES));
        if (PERM) {
          // rows 4 l + q of the 128-row block land on shared-memory row q * 32 + l; the scale words of K step k lie
          // in row order at word k * rows + row: one box of 128 words x 4 K steps per 128-row block
          tma_load_3d_pair_if(el, sA + s * A_BYTES, &tma_a, kt * BKB, m0 >> 2, 0, lf);
          tma_load_3d_pair_if(el, sB + s * B_BYTES, &tma_b, kt * BKB, nb0 >> 2, 0, lf);
          tma_load_2d_pair_if(el, sSFA + s * SFA_BYTES, &tma_sfa, m0, kt * KS, lf);
          tma_load_2d_pair_if(el, sSFB + s * SFB_BYTES, &tma_sfb, tn * BN, kt * KS, lf);
          tma_load_2d_pair_if(el, sSFB + s * SFB_BYTES + KS * 512, &tma_sfb, tn * BN + 128, kt * KS, lf);
          if (++s == STAGES) { s = 0; ph ^= 1; }
          continue;
        }
        tma_load_2d_pair_if(el, sA + s * A_BYTES, &tma_a, kt * BKB, m0, lf);
        tma_load_2d_pair_if(el, sB + s * B_BYTES, &tma_b, kt * BKB, nb0, lf);
        if (SF_TILED) {
          tma_load_2d_pair_if(el, sSFA + s * SFA_BYTES, &tma_sfa, 0, sfa_row0 + kt * KS, lf);
          tma_load_2d_pair_if(el, sSFB + s * SFB_BYTES, &tma_sfb, 0, sfb_row0 + kt * KS, lf);
          tma_load_2d_pair_if(el, sSFB + s * SFB_BYTES + KS * 512, &tma_sfb, 0, sfb_row0 + p.KT + kt * KS, lf);
        }
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
      if (!ok) { if (el) atomicExch(p.status, kStatusTimeoutProducer); break; }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA)
    if (rank == 0) {
      const uint32_t el = elect_one();
      constexpr uint32_t idesc = make_idesc_mxf4nvf4(BMP, BN);
      uint32_t s = 0, ph = 0, it = 0, ti = 0, acc_phs = 0, shared_ph = 0;
      const uint64_t adesc0 = make_smem_desc(sA, 16, 1024, kSwizzle128B);
      const uint64_t bdesc0 = make_smem_desc(sB, 16, 1024, kSwizzle128B);
      // scale chunks: 32 rows x 16 bytes, 8-row groups 128 bytes apart, not swizzled
      const uint64_t sfadesc0 = make_smem_desc(sSFA, 0, 128, kSwizzleNone);
      const uint64_t sfbdesc0 = make_smem_desc(sSFB, 0, 128, kSwizzleNone);
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        // this tile's accumulator must have been drained (by the tile before the previous one), and the
        // previous tile's epilogue must have read the columns both accumulators share
        const uint32_t acc = ti & 1;
        ok = warp_all(mbar_wait(tempty_bar + 8 * acc, ((acc_phs >> acc) & 1) ^ 1, p.wait_ns));
        if (!ok) break;
        acc_phs ^= 1u << acc;
        ok = warp_all(mbar_wait(shared_free_bar, shared_ph ^ 1, p.wait_ns));
        if (!ok) break;
        shared_ph ^= 1;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC1_COL;
        for (int kt = 0; kt < k_tiles; ++kt) {
          if (el) AC4K_TR(0, it, 0);
          ok = warp_all(mbar_wait(full_bar + 8 * s, ph, p.wait_ns));
          if (!ok) break;
          tc_fence_after();
          if (el) AC4K_TR(0, it, 1);
          const uint32_t t_sf = tmem_base + SF_COL;
          const uint64_t adesc = adesc0 + (uint64_t)(s * (A_BYTES >> 4));
          const uint64_t bdesc = bdesc0 + (uint64_t)(s * (B_BYTES >> 4));
          const uint64_t sfadesc = sfadesc0 + (uint64_t)(s * (SFA_BYTES >> 4));
          const uint64_t sfbdesc = sfbdesc0 + (uint64_t)(s * (SFB_BYTES >> 4));
          const int nk = (kt + 1 < k_tiles) ? KS : last_nk;
          if (nk == KS) {
#pragma unroll
            for (int j = 0; j < KS; ++j) {
              tmem_cp_32x128b_warpx4_pair_if(el, t_sf + j * 4, sfadesc + j * 32);
              tmem_cp_32x128b_warpx4_pair_if(el, t_sf + KS * 4 + j * 8, sfbdesc + j * 32);
              tmem_cp_32x128b_warpx4_pair_if(el, t_sf + KS * 4 + j * 8 + 4, sfbdesc + (KS + j) * 32);
            }
#pragma unroll
            for (int j = 0; j < KS; ++j)    // K step j: 32 bytes further inside the 128-byte swizzle atom
              mma_mxf4nvf4_pair_if(el, d_tmem, adesc + 2 * j, bdesc + 2 * j, idesc, t_sf + j * 4, t_sf + KS * 4 + j * 8,
                                   (kt > 0 || j > 0) ? 1u : 0u);
          } else {
            for (int j = 0; j < nk; ++j) {
              tmem_cp_32x128b_warpx4_pair_if(el, t_sf + j * 4, sfadesc + j * 32);
              tmem_cp_32x128b_warpx4_pair_if(el, t_sf + KS * 4 + j * 8, sfbdesc + j * 32);
              tmem_cp_32x128b_warpx4_pair_if(el, t_sf + KS * 4 + j * 8 + 4, sfbdesc + (KS + j) * 32);
            }
            for (int j = 0; j < nk; ++j)
              mma_mxf4nvf4_pair_if(el, d_tmem, adesc + 2 * j, bdesc + 2 * j, idesc, t_sf + j * 4, t_sf + KS * 4 + j * 8,
                                   (kt > 0 || j > 0) ? 1u : 0u);
          }
          tc_commit_pair_both_if(el, empty_bar + 8 * s, 3);                 // stage free in both CTAs
          if (kt == k_tiles - 1) tc_commit_pair_both_if(el, tfull_bar + 8 * acc, 3);  // accumulator complete in both CTAs
          if (el) AC4K_TR(0, it, 2);
          ++it;
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        ++ti;
      }
      if (!ok && el) atomicExch(p.status, kStatusTimeoutMma);
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ scale warps (row layout only)
    // Scales stored as [K/64][rows][4 bytes]: the word of row r at K step k sits at word k * rows + r.
    // tcgen05.cp wants, per K step and 128-row block, 32 rows of 16 bytes where row l holds the words
    // of rows l, 32 + l, 64 + l, 96 + l.  Warp w takes the stages with (stage number % 4) == w - 2:
    // its loads are in flight while the three stages before it are consumed.
    if (!SF_TILED) {
      const int w4 = warp - 2;
      uint32_t s = 0, ph = 0, it = 0;
      const uint32_t leader_full0 = map_to_cta(full_bar, 0);
      const uint32_t *sfa_w = reinterpret_cast<const uint32_t *>(p.sfa);
      const uint32_t *sfb_w = reinterpret_cast<const uint32_t *>(p.sfb);
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * BMP + (int)rank * 128, n0 = tn * BN;
        for (int kt = 0; kt < k_tiles; ++kt) {
          static_assert(STAGES >= 4, "four scale warps: each may run at most one round of the ring ahead");
          if ((int)(it & 3) == w4) {
            uint32_t wa[KS][4], wb[KS][8];
#pragma unroll
            for (int j = 0; j < KS; ++j) {
              const int k64 = kt * KS + j;
              const bool k_ok = k64 < p.KT;
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                const int r = m0 + 32 * g + lane;
                wa[j][g] = (k_ok && r < p.rows_sfa) ? __ldg(sfa_w + (int64_t)k64 * p.rows_sfa + r) : 0u;
              }
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                const int r = n0 + 32 * g + lane;
                wb[j][g] = (k_ok && r < p.rows_sfb) ? __ldg(sfb_w + (int64_t)k64 * p.rows_sfb + r) : 0u;
              }
            }
            ok = warp_all(mbar_wait(empty_bar + 8 * s, ph ^ 1, p.wait_ns));
            if (!ok) break;
#pragma unroll
            for (int j = 0; j < KS; ++j) {
              st_shared_v4u(sSFA + s * SFA_BYTES + j * 512 + lane * 16, wa[j][0], wa[j][1], wa[j][2], wa[j][3]);
              st_shared_v4u(sSFB + s * SFB_BYTES + j * 512 + lane * 16, wb[j][0], wb[j][1], wb[j][2], wb[j][3]);
              st_shared_v4u(sSFB + s * SFB_BYTES + (KS + j) * 512 + lane * 16, wb[j][4], wb[j][5], wb[j][6], wb[j][7]);
            }
            fence_proxy_async_smem();       // the tensor core reads these bytes through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_full0 + 8 * s);
          }
          ++it;
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (!ok && lane == 0) atomicExch(p.status, kStatusTimeoutSf);
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 6-13)
    // Two warps per tensor-memory lane quarter, 128 accumulator columns each.  Phase 1: tcgen05.ld,
    // * alpha, + bias, pack to 16 bit, all into registers; then the accumulator goes back to the
    // MMA issuer.  Phase 2: each thread stores its 256-byte row segment; it overlaps the next
    // tile's main loop.  The warp whose 128 columns contain the 48 columns that both accumulators
    // share reads those first and reports them free at once: that is all the next tile waits for.
    using T = typename OutT<OUT_DT>::type;
    const int q = warp & 3;
    const int half = warp >= 10 ? 1 : 0;
    uint32_t acc_phs = 0;
    int ti = 0;
    const float alpha = __fmul_rn(__ldg(p.a_gs), __ldg(p.b_gs));
    const bool has_bias = p.bias != nullptr;
    const uint32_t leader_tempty = map_to_cta(tempty_bar, 0);
    const uint32_t leader_shared_free = map_to_cta(shared_free_bar, 0);
    for (int t = cluster_id; t < num_tiles; t += num_clusters) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      const int row = tm * BMP + (int)rank * 128 + (PERM ? 4 * lane + q : q * 32 + lane);
      const int col0 = tn * BN + half * 128;
      const uint32_t bias_s = sBias + (uint32_t)(half * 4 + q) * 512u;
      const uint32_t acc = ti & 1;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * ACC1_COL + half * 128;
      if (has_bias) {
        // this warp's 128 bias values go to shared memory while the tile's MMAs are still running, so
        // that the drain below only adds broadcast shared-memory loads
        float b4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int n = col0 + lane * 4 + i;
          b4[i] = n < p.N ? load_bias(p.bias, p.bias_dt, n) : 0.0f;
        }
        st_shared_v4f(bias_s + lane * 16, b4[0], b4[1], b4[2], b4[3]);
        __syncwarp();
      }
      if (!mbar_wait(tfull_bar + 8 * acc, (acc_phs >> acc) & 1, p.wait_ns)) { if (lane == 0) atomicExch(p.status, kStatusTimeoutEpilogue); break; }
      acc_phs ^= 1u << acc;
      tc_fence_after();
      if (warp == 6 && lane == 0) AC4K_TR(1, ti, 0);
      uint32_t w[64];
      if (PERM) {
        // the columns both accumulators share are the first 48 of accumulator 1's columns 0 - 127 and the last 48 of
        // accumulator 0's columns 128 - 255: the first two steps cover them
        const bool shared = half != (int)acc;
        if (shared && half == 1) {
          if (has_bias) drain_permuted<OUT_DT, true, 3, 2, 0, 1>(w, t_row, true, alpha, bias_s, lane, leader_shared_free);
          else drain_permuted<OUT_DT, false, 3, 2, 0, 1>(w, t_row, true, alpha, bias_s, lane, leader_shared_free);
        } else {
          if (has_bias) drain_permuted<OUT_DT, true, 0, 1, 2, 3>(w, t_row, shared, alpha, bias_s, lane, leader_shared_free);
          else drain_permuted<OUT_DT, false, 0, 1, 2, 3>(w, t_row, shared, alpha, bias_s, lane, leader_shared_free);
        }
      } else if (half == (int)acc) {
        // none of the shared columns: columns 0 - 127 of accumulator 0 or 128 - 255 of accumulator 1
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[64];
          tmem_ld_32x32b_x64_sync(t_row + c * 64, r);
          if (c == 0) pack_cols<OUT_DT, 0, 64>(r, w, alpha, has_bias, bias_s);
          else pack_cols<OUT_DT, 64, 64>(r, w, alpha, has_bias, bias_s);
        }
      } else if (half == 0) {
        // accumulator 1, tile columns 0 - 127: the shared ones are this warp's first 48
        {
          uint32_t r0[32], r1[16];
          tmem_ld_32x32b_x32(t_row, r0);
          tmem_ld_32x32b_x16(t_row + 32, r1);
          tmem_ld_wait();
          tmem_pin(r0);
          tmem_pin(r1);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(leader_shared_free);
          pack_cols<OUT_DT, 0, 32>(r0, w, alpha, has_bias, bias_s);
          pack_cols<OUT_DT, 32, 16>(r1, w, alpha, has_bias, bias_s);
        }
        {
          uint32_t r[64];
          tmem_ld_32x32b_x64_sync(t_row + 48, r);
          pack_cols<OUT_DT, 48, 64>(r, w, alpha, has_bias, bias_s);
        }
        {
          uint32_t r[16];
          tmem_ld_32x32b_x16(t_row + 112, r);
          tmem_ld_wait();
          tmem_pin(r);
          pack_cols<OUT_DT, 112, 16>(r, w, alpha, has_bias, bias_s);
        }
      } else {
        // accumulator 0, tile columns 128 - 255: the shared ones are this warp's last 48
        {
          uint32_t r0[16], r1[32];
          tmem_ld_32x32b_x16(t_row + 80, r0);
          tmem_ld_32x32b_x32(t_row + 96, r1);
          tmem_ld_wait();
          tmem_pin(r0);
          tmem_pin(r1);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(leader_shared_free);
          pack_cols<OUT_DT, 80, 16>(r0, w, alpha, has_bias, bias_s);
          pack_cols<OUT_DT, 96, 32>(r1, w, alpha, has_bias, bias_s);
        }
        {
          uint32_t r[64];
          tmem_ld_32x32b_x64_sync(t_row, r);
          pack_cols<OUT_DT, 0, 64>(r, w, alpha, has_bias, bias_s);
        }
        {
          uint32_t r[16];
          tmem_ld_32x32b_x16(t_row + 64, r);
          tmem_ld_wait();
          tmem_pin(r);
          pack_cols<OUT_DT, 64, 16>(r, w, alpha, has_bias, bias_s);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (warp == 6 && lane == 0) AC4K_TR(1, ti, 1);
      if (lane == 0) mbar_arrive_cluster(leader_tempty + 8 * acc);
      const int64_t col_base = p.col_off + col0;
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
      } else if (!AC4K_DBG(p, 8)) {
        // The registers hold one row per lane; stored from there, every instruction would touch 32
        // different rows, and that scatter was measured to slow the next tile's main loop down by
        // 20 % while it lasted.  So each half (64 columns = 128 bytes per row) goes through this warp's
        // 4 KB staging buffer in the 128-byte-swizzled order and leaves as one TMA store of 32 rows,
        // clipped by the tensor map at the edges of the output.  With several destinations (the fused
        // all-gather: this GPU's buffer and the peers', reached over NVLink) the same buffer is stored
        // once per destination.
        const uint32_t stage_buf = sOut + (uint32_t)(half * 4 + q) * OUT_STAGE_BYTES;
        // (row-permuted variant: this warp's lanes hold rows y0 + q, y0 + q + 4, ...: box {64, 32, 1} at {x, y0 / 4, q})
        const int y0 = tm * BMP + (int)rank * 128 + (PERM ? 0 : q * 32);
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          const int x0 = (int)col_base + 64 * h2;
          if (col0 + 64 * h2 >= p.N || y0 >= p.M) break;     // warp-uniform: nothing of this box is inside the output
          if (lane == 0) bulk_wait_group_read0();            // the previous store has read the buffer
          __syncwarp();
#pragma unroll
          for (int c = 0; c < 8; ++c)
            st_shared_v4u(stage_buf + lane * 128 + ((c ^ (lane & 7)) << 4), w[32 * h2 + 4 * c], w[32 * h2 + 4 * c + 1],
                          w[32 * h2 + 4 * c + 2], w[32 * h2 + 4 * c + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (PERM) tma_store_3d(&dmaps.m[0], x0, y0 >> 2, q, stage_buf);
            else tma_store_2d(&dmaps.m[0], x0, y0, stage_buf);
            if (EPI == EPI_GATHER) {
              // peers in turn, starting behind this rank, so that the ranks do not all write to the same GPU at once
              for (int d = 1; d < p.n_dst; ++d) {
                if (PERM) tma_store_3d(&dmaps.m[d], x0, y0 >> 2, q, stage_buf);
                else tma_store_2d(&dmaps.m[d], x0, y0, stage_buf);
              }
            }
            bulk_commit_group();
          }
        }
      }
      if (warp == 6 && lane == 0) AC4K_TR(1, ti, 2);
      if (warp == 6 && lane == 0) AC4K_TR(3, 0, 3);
      ++ti;
    }
    if (lane == 0) bulk_wait_group_read0(); // the staging buffer has been read by this warp's last stores before the CTA exits
  }

  if (threadIdx.x == 0) AC4K_TR(3, 0, 4);
  tc_fence_before();
  __syncthreads();
  cluster_sync_relaxed();  // neither CTA leaves while the other may still read its memory or barriers (nothing is handed over)
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) AC4K_TR(3, 0, 5);
#ifdef AC4K_TRACE_ENABLED
  if (p.trace != nullptr && rank == 0 && threadIdx.x == 0 && cluster_id < 120) p.trace[((size_t)4 * 128 + cluster_id) * 8 + 2] = globaltimer();
#endif
  AC4K_TR_LAUNCH(false);
}

template <int SF_MODE, int OUT_DT, int EPI>
static int launch_pair(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tsa, const CUtensorMap &tsb,
                       const DstMaps &dm, const GemmArgs &args, int sms, cudaStream_t stream) {
  auto kern = linear_nvfp4_2cta_kernel<SF_MODE, OUT_DT, EPI>;
  // Once per device: the shared-memory attribute, and how many CTA pairs can be resident at once (not every
  // SM can be paired on every part); the kernel is persistent, so launching more clusters than that would
  // serialise whole waves.
  static PerDevice<int> max_clusters;
  int clusters = 0;
  if (int e = max_clusters.get(&clusters, [&](int &v) {
        AC4K_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pair::SMEM_BYTES));
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
        v = n;
        return 0;
      }))
    return e;
  const int num_tiles = args.tiles_m * args.tiles_n;

  if (num_tiles < clusters) clusters = num_tiles;
  // launched so that its set-up may overlap the previous kernel's tail (see grid_dependency_wait)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters);
  cfg.blockDim = dim3(pair::kThreadsPair);
  cfg.dynamicSmemBytes = pair::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = AC4K_DBG(args, 64) ? 0 : 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  AC4K_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, ta, tb, tsa, tsb, dm, args));
  return 0;
}

template <int OUT_DT, int EPI>
static int launch_pair_mode(int sf_mode, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tsa, const CUtensorMap &tsb,
                            const DstMaps &dm, const GemmArgs &args, int sms, cudaStream_t stream) {
  if (sf_mode == kSfTiled) return launch_pair<kSfTiled, OUT_DT, EPI>(ta, tb, tsa, tsb, dm, args, sms, stream);
  if (sf_mode == kSfPerm) return launch_pair<kSfPerm, OUT_DT, EPI>(ta, tb, tsa, tsb, dm, args, sms, stream);
  return launch_pair<kSfWarps, OUT_DT, EPI>(ta, tb, tsa, tsb, dm, args, sms, stream);
}

// sf_mode: 0 - scales in the row layout, re-ordered by warps (operand and output maps of rank 2); 1 - scales in 128x4
// tiles; 2 - scales in the row layout with the operands' and the output's maps of rank 3 (rows as row / 4, row % 4)
int launch_linear_2cta(int d_dtype, int sf_mode, const CUtensorMap &ta, const CUtensorMap &tb,
                       const CUtensorMap &tsa, const CUtensorMap &tsb, const DstMaps &dm, GemmArgs args, cudaStream_t stream) {
  DeviceInfo di;
  if (int e = get_device_info(&di)) return e;
  args.tiles_m = (int)ceil_div(args.M, pair::BMP);
  args.tiles_n = (int)ceil_div(args.N, pair::BN);
  // the instantiations that forward tiles to further destinations or re-quantise the output are
  // separate: their extra registers and code would otherwise slow the plain GEMM down
  if (args.q_out != nullptr) {
    if (d_dtype != AC4K_DT_BF16) return fail(AC4K_ERR_UNSUPPORTED, "the re-quantising epilogue rounds to bf16 first");
    return launch_pair_mode<AC4K_DT_BF16, EPI_REQUANT>(sf_mode, ta, tb, tsa, tsb, dm, args, di.sms, stream);
  }
  const bool gather = args.n_dst > 1;
  if (d_dtype == AC4K_DT_BF16) {
    if (gather) return launch_pair_mode<AC4K_DT_BF16, EPI_GATHER>(sf_mode, ta, tb, tsa, tsb, dm, args, di.sms, stream);
    return launch_pair_mode<AC4K_DT_BF16, EPI_PLAIN>(sf_mode, ta, tb, tsa, tsb, dm, args, di.sms, stream);
  }
  if (d_dtype == AC4K_DT_FP16) {
    if (gather) return launch_pair_mode<AC4K_DT_FP16, EPI_GATHER>(sf_mode, ta, tb, tsa, tsb, dm, args, di.sms, stream);
    return launch_pair_mode<AC4K_DT_FP16, EPI_PLAIN>(sf_mode, ta, tb, tsa, tsb, dm, args, di.sms, stream);
  }
  return fail(AC4K_ERR_UNSUPPORTED, "the CTA-pair kernel stores 16-bit outputs only");
}

}  // namespace ac4k
