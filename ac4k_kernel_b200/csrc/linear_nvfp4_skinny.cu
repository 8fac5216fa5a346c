// NVFP4 block-scaled GEMM for sm_100a, decode shapes: a handful of activation rows (M <= 64) against a
// large weight matrix.  Such a call streams the weights once and does almost no arithmetic, so the kernel
// is built around the weight stream (it stands in for the same reference kernel as linear_nvfp4.cu,
// lib/cuda/sm120/linear_nvfp4.cu:337-901, on the shapes of lib/cuda/sm120/linear_nvfp4.cu:586-633):
//
//   * The operands are swapped on the tensor core: 128 weight rows are the M side of the MMA, the
//     activation rows (padded to NT = 16 / 32 / 64) the N side.  The accumulator is 128 lanes x NT columns,
//     an activation box is NT x 128 bytes instead of 128 x 128, and a call with M = 1 costs what M = 16 costs.
//   * One work item per CTA: a tile of 128 weight rows x one slice of K.  The `splits` (1, 2 or 4) slices of a
//     tile are the CTAs of one cluster.  The 128 rows of the tile are four quarters of 32 (one per epilogue
//     warp); quarter q is finished by CTA q % splits: the other slices copy their fp32 partial sums of that
//     quarter into a small region of its shared memory (one bulk copy through distributed shared memory,
//     completing on the owner's mbarrier), it adds them in slice order, applies alpha and bias and stores.
//     No workspace, no second kernel, no waiting for a leader.
//   * A CTA needs 97 - 111 KB of shared memory and 128 tensor-memory columns, so two of them fit on an
//     SM and the CTAs of the next call of the stream (programmatic dependent launch) become resident while this
//     call still runs; before they wait for it they ask L2 for their whole share of the weights (a prefetch
//     returns no data, so the dependency is kept), and the weight stream of call i+1 runs under the tail of call i.
//
// Roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer (scales to tensor memory with tcgen05.cp, then
// four MMAs per stage), warps 2-5 epilogue; for scales in the row layout [K/64][rows][4] the epilogue warps
// also re-order each stage's scale words into the 32 x 16-byte chunks tcgen05.cp wants (every fourth stage
// each).  Issuing roles run warp-wide with an elected lane (see elect_one()).
#include "gemm_common.cuh"

namespace ac4k {
using namespace ptx;

namespace skinny {
static constexpr int KS = 4;                     // K = 64 steps per stage (K = 256)
static constexpr int W_BYTES = 128 * BKB;        // 128 weight rows x 128 bytes
static constexpr int SF_BYTES = KS * 512;        // scale chunks of one 128-row block
static constexpr int kThreads = 192;
static constexpr int TMEM_COLS = 128;            // accumulator (<= 64 columns), weight scales at 64, activation scales at 80
static constexpr int SFW_COL = 64, SFX_COL = 80;
template <int NT>
struct Cfg {
  static constexpr int X_BYTES = NT * BKB;
  static constexpr int STAGES = NT == 64 ? 3 : 4;       // two CTAs of this kernel fit on an SM in every configuration
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES + 2 * SF_BYTES;
  // partial sums received from the other slices: up to 3 units of [NT][32] fp32 (4 slices: this CTA's one
  // quarter from 3 slices; 2 slices: its two quarters from 1 slice each)
  static constexpr int PART_UNIT = NT * 128;
  static constexpr int PART_BYTES = 3 * PART_UNIT;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + PART_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
  static constexpr int MIN_CTAS = 2;                     // CTAs of this kernel that fit on an SM
  static_assert(MIN_CTAS * (SMEM_BYTES + 1024) <= 228 * 1024, "shared memory per SM");
};
}  // namespace skinny

__device__ __forceinline__ void st_shared_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cta.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// bulk copy from this CTA's shared memory into the shared memory of a CTA of the cluster, completing (bytes) on an
// mbarrier of that CTA; 16-byte aligned addresses and size
__device__ __forceinline__ void bulk_copy_to_cluster(uint32_t dst_cluster_addr, uint32_t src, uint32_t bytes, uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_cluster_addr), "r"(src), "r"(bytes), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ float ld_shared_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cta.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

template <int NT>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[NT]) {
  if constexpr (NT == 16) tmem_ld_32x32b_x16(taddr, r);
  else if constexpr (NT == 32) tmem_ld_32x32b_x32(taddr, r);
  else tmem_ld_32x32b_x64(taddr, r);
  tmem_ld_wait();
  tmem_pin(r);
}

// The owner of a quarter of the rows: add the K slices in slice order (whichever of them this CTA computed
// itself: `own`; the others from the partial-sum units, which skip the owner's own slice), apply alpha and
// bias, round and store row by row.  Eight activation rows at a time so that their shared-memory loads are
// independent of one another.
template <int NT, int SPLITS, int OUT_DT>
__device__ __forceinline__ void finish_rows(const uint32_t (&own)[NT], uint32_t part0, int slice, const GemmArgs &p, int n,
                                            typename OutT<OUT_DT>::type *dst) {
  using T = typename OutT<OUT_DT>::type;
  constexpr int UNIT = NT * 128;
  const float alpha = __fmul_rn(__ldg(p.a_gs), __ldg(p.b_gs));
  const float b = p.bias != nullptr ? load_bias(p.bias, p.bias_dt, n) : 0.0f;
#pragma unroll
  for (int m0 = 0; m0 < NT; m0 += 8) {
    if (m0 >= p.M) break;
    float x[SPLITS > 1 ? SPLITS - 1 : 1][8];
    if (SPLITS > 1) {
#pragma unroll
      for (int j = 0; j < SPLITS - 1; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) x[j][i] = ld_shared_f32(part0 + j * UNIT + (m0 + i) * 128);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int m = m0 + i;
      float v = 0.0f;
#pragma unroll
      for (int sl = 0; sl < SPLITS; ++sl) {
        float t = __uint_as_float(own[m]);
        if (SPLITS > 1) {
          // slice sl sits in unit sl if it comes before the owner's own slice, else in unit sl - 1
          const float before = x[sl < SPLITS - 1 ? sl : SPLITS - 2][i], after = x[sl > 0 ? sl - 1 : 0][i];
          t = sl == slice ? t : (sl < slice ? before : after);
        }
        v = sl == 0 ? t : __fadd_rn(v, t);
      }
      v = __fmul_rn(v, alpha);
      if (p.bias != nullptr) v = __fadd_rn(v, b);
      if (m < p.M) {
        if (OUT_DT == AC4K_DT_BF16) dst[(int64_t)m * p.N] = (T)__float2bfloat16_rn(v);
        else if (OUT_DT == AC4K_DT_FP16) dst[(int64_t)m * p.N] = (T)__float2half_rn(v);
        else dst[(int64_t)m * p.N] = (T)v;
      }
    }
  }
}

template <int NT, bool SF_TILED, int OUT_DT>
__global__ void __launch_bounds__(skinny::kThreads, skinny::Cfg<NT>::MIN_CTAS)
linear_nvfp4_skinny_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_w,
                           const GemmArgs p) {
  using namespace skinny;
  using C = skinny::Cfg<NT>;
  constexpr int STAGES = C::STAGES;
  using T = typename OutT<OUT_DT>::type;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sW = smem_base;
  const uint32_t sX = sW + STAGES * W_BYTES;
  const uint32_t sSFW = sX + STAGES * C::X_BYTES;
  const uint32_t sSFX = sSFW + STAGES * SF_BYTES;
  const uint32_t sPart = sSFX + STAGES * SF_BYTES;
  const uint32_t bars = sPart + C::PART_BYTES;
  const uint32_t full_bar = bars, empty_bar = bars + 8 * STAGES;
  const uint32_t tfull_bar = bars + 16 * STAGES;
  const uint32_t part_bar = tfull_bar + 8;      // [2] the other slices' partial sums of this CTA's first / second quarter have landed
  const uint32_t tmem_slot = part_bar + 16;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

#ifdef AC4K_TRACE_ENABLED
  // wall-clock stamps of every 4th CTA: [0] entry, [1] dependency wait passed, [2] exit, [3] first stage ready,
  // [4] last MMA issued, [5] accumulator complete seen, [6] partial sums exchanged
#define AC4K_TRS(ev) do { if (p.trace != nullptr && (blockIdx.x & 3) == 0 && (blockIdx.x >> 2) < 127) p.trace[((size_t)4 * 128 + (blockIdx.x >> 2)) * 8 + (ev)] = globaltimer(); } while (0)
#else
#define AC4K_TRS(ev) do { } while (0)
#endif
  if (threadIdx.x == 0) AC4K_TRS(0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // work item of this CTA: the K slices of one tile are the consecutive CTAs of a cluster
  const int tn = blockIdx.x / p.splits;
  const int slice = p.splits > 1 ? (int)cluster_ctarank() : 0;
  const int k_tiles_all = (p.KT + KS - 1) / KS;
  const int kt0 = slice * p.kt_per_split, kt1 = min(k_tiles_all, kt0 + p.kt_per_split);
  const int n0 = tn * 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar + 8 * s, SF_TILED ? 1 : 2);   // producer's expect_tx arrival (+ the stage's scale warp)
      mbar_init(empty_bar + 8 * s, 1);
    }
    mbar_init(tfull_bar, 1);
    mbar_init(part_bar, 1);
    mbar_init(part_bar + 8, 1);
    if (p.splits > 1) {
      // this CTA finishes 4 / splits quarters; each receives one copy of NT x 128 bytes from every other slice
      for (int lq = 0; lq < 4 / p.splits; ++lq) mbar_arrive_expect_tx(part_bar + 8 * lq, (p.splits - 1) * C::PART_UNIT);
    }
    fence_barrier_init();
    prefetch_tmap(&tma_x);
    prefetch_tmap(&tma_w);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 2) {
    // This CTA's whole share of the weight stream, requested from HBM now, while the kernel before this
    // one in the stream may still be running (see the file comment).
    const uint32_t el = elect_one();
    for (int kt = kt0; kt < kt1; ++kt) tma_prefetch_2d_if(el, &tma_w, kt * BKB, n0);
    if (SF_TILED && kt1 > kt0)
      bulk_prefetch_l2_if(el, p.sfb + ((int64_t)tn * p.KT + (int64_t)kt0 * KS) * 512,
                          (uint32_t)(min(kt1 * KS, p.KT) - kt0 * KS) * 512u);
  }
  tc_fence_before();
  __syncthreads();
  if (p.splits > 1) cluster_sync();     // the other slices' barriers exist before anything is signalled remotely
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(smem_gen + (tmem_slot - smem_base));
  grid_launch_dependents();
  grid_dependency_wait();
  if (threadIdx.x == 0) AC4K_TRS(1);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    const uint32_t el = elect_one();
    uint32_t s = 0, ph = 0;
    bool ok = true;
    for (int kt = kt0; kt < kt1; ++kt) {
      ok = warp_all(mbar_wait(empty_bar + 8 * s, ph ^ 1, p.wait_ns));
      if (!ok) break;
      const int nk = min(KS, p.KT - kt * KS);
      const uint32_t fb = full_bar + 8 * s;
      mbar_arrive_expect_tx_if(el, fb, W_BYTES + C::X_BYTES + (SF_TILED ? 2 * nk * 512 : 0));
      tma_load_2d_if(el, sW + s * W_BYTES, &tma_w, kt * BKB, n0, fb);
      tma_load_2d_if(el, sX + s * C::X_BYTES, &tma_x, kt * BKB, 0, fb);
      if (SF_TILED) {
        // [row block of 128][K/64][512 B]: the nk chunks of one row block are contiguous
        const int64_t k64 = (int64_t)kt * KS;
        bulk_load_1d_if(el, sSFW + s * SF_BYTES, p.sfb + ((int64_t)tn * p.KT + k64) * 512, nk * 512, fb);
        bulk_load_1d_if(el, sSFX + s * SF_BYTES, p.sfa + k64 * 512, nk * 512, fb);
      }
      if (++s == STAGES) { s = 0; ph ^= 1; }
    }
    if (!ok && el) atomicExch(p.status, kStatusTimeoutProducer);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t el = elect_one();
    constexpr uint32_t idesc = make_idesc_mxf4nvf4(128, NT);
    uint32_t s = 0, ph = 0;
    bool ok = true;
    const uint64_t wdesc0 = make_smem_desc(sW, 16, 1024, kSwizzle128B);
    const uint64_t xdesc0 = make_smem_desc(sX, 16, 1024, kSwizzle128B);
    const uint64_t sfwdesc0 = make_smem_desc(sSFW, 0, 128, kSwizzleNone);
    const uint64_t sfxdesc0 = make_smem_desc(sSFX, 0, 128, kSwizzleNone);
    const uint32_t t_sfw = tmem_base + SFW_COL, t_sfx = tmem_base + SFX_COL;
    for (int kt = kt0; kt < kt1; ++kt) {
      ok = warp_all(mbar_wait(full_bar + 8 * s, ph, p.wait_ns));
      if (!ok) break;
      tc_fence_after();
      if (el && kt == kt0) AC4K_TRS(3);
      const int nk = min(KS, p.KT - kt * KS);
      const uint64_t wdesc = wdesc0 + (uint64_t)(s * (W_BYTES >> 4));
      const uint64_t xdesc = xdesc0 + (uint64_t)(s * (C::X_BYTES >> 4));
      const uint64_t sfwdesc = sfwdesc0 + (uint64_t)(s * (SF_BYTES >> 4));
      const uint64_t sfxdesc = sfxdesc0 + (uint64_t)(s * (SF_BYTES >> 4));
      if (nk == KS) {
#pragma unroll
        for (int j = 0; j < KS; ++j) {
          tmem_cp_32x128b_warpx4_if(el, t_sfw + j * 4, sfwdesc + j * 32);
          tmem_cp_32x128b_warpx4_if(el, t_sfx + j * 4, sfxdesc + j * 32);
        }
#pragma unroll
        for (int j = 0; j < KS; ++j)
          mma_mxf4nvf4_if(el, tmem_base, wdesc + 2 * j, xdesc + 2 * j, idesc, t_sfw + j * 4, t_sfx + j * 4,
                          (kt > kt0 || j > 0) ? 1u : 0u);
      } else {
        for (int j = 0; j < nk; ++j) {
          tmem_cp_32x128b_warpx4_if(el, t_sfw + j * 4, sfwdesc + j * 32);
          tmem_cp_32x128b_warpx4_if(el, t_sfx + j * 4, sfxdesc + j * 32);
        }
        for (int j = 0; j < nk; ++j)
          mma_mxf4nvf4_if(el, tmem_base, wdesc + 2 * j, xdesc + 2 * j, idesc, t_sfw + j * 4, t_sfx + j * 4,
                          (kt > kt0 || j > 0) ? 1u : 0u);
      }
      tc_commit_if(el, empty_bar + 8 * s);
      if (++s == STAGES) { s = 0; ph ^= 1; }
    }
    if (ok) tc_commit_if(el, tfull_bar);
    if (el) AC4K_TRS(4);
    if (!ok && el) atomicExch(p.status, kStatusTimeoutMma);
  } else {
    // ------------------------------------------------------------------ scale re-ordering (row layout), then epilogue
    const int q = warp & 3;                   // tensor-memory lane quarter of this warp (warps 2-5 -> 2, 3, 0, 1)
    if (!SF_TILED) {
      // [K/64][rows][4 bytes] -> per K step 32 rows of 16 bytes, row l holding the words of rows l, 32 + l,
      // 64 + l, 96 + l of the block; warp w takes the stages whose number is w - 2 modulo NW.  NW never exceeds
      // the depth of the ring: a warp then moves on by at most one round of the ring per stage it handles, which
      // the parity of the stage's barrier can tell apart (two rounds ahead it could not).
      constexpr int NW = STAGES < 4 ? STAGES : 4;
      const int w4 = warp - 2;
      uint32_t s = 0, ph = 0, it = 0;
      const uint32_t *sfx_w = reinterpret_cast<const uint32_t *>(p.sfa);
      const uint32_t *sfw_w = reinterpret_cast<const uint32_t *>(p.sfb);
      bool ok = true;
      for (int kt = kt0; kt < kt1; ++kt) {
        if ((int)(it % NW) == w4) {
          uint32_t ww[KS][4], wx[KS][4];
#pragma unroll
          for (int j = 0; j < KS; ++j) {
            const int k64 = kt * KS + j;
            const bool k_ok = k64 < p.KT;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int rw = n0 + 32 * g + lane, rx = 32 * g + lane;
              ww[j][g] = (k_ok && rw < p.rows_sfb) ? __ldg(sfw_w + (int64_t)k64 * p.rows_sfb + rw) : 0u;
              wx[j][g] = (k_ok && rx < p.rows_sfa) ? __ldg(sfx_w + (int64_t)k64 * p.rows_sfa + rx) : 0u;
            }
          }
          ok = warp_all(mbar_wait(empty_bar + 8 * s, ph ^ 1, p.wait_ns));
          if (!ok) break;
#pragma unroll
          for (int j = 0; j < KS; ++j) {
            st_shared_v4u(sSFW + s * SF_BYTES + j * 512 + lane * 16, ww[j][0], ww[j][1], ww[j][2], ww[j][3]);
            st_shared_v4u(sSFX + s * SF_BYTES + j * 512 + lane * 16, wx[j][0], wx[j][1], wx[j][2], wx[j][3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(full_bar + 8 * s);
        }
        ++it;
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
      if (!ok && lane == 0) atomicExch(p.status, kStatusTimeoutSf);
    }
    // ---- epilogue: lane l of quarter q owns weight row (output column) n0 + 32 q + l, its NT accumulator
    // columns are the activation rows
    const int row_l = q * 32 + lane;
    const int n = n0 + row_l;
    const bool tfull_ok = mbar_wait(tfull_bar, 0, p.wait_ns);
    if (!tfull_ok && lane == 0) atomicExch(p.status, kStatusTimeoutEpilogue);
    tc_fence_after();
    if (warp == 2 && lane == 0) AC4K_TRS(5);
    uint32_t r[NT];
    tmem_ld_cols<NT>(tmem_base + ((uint32_t)(q * 32) << 16), r);
    const int owner = q % p.splits;           // the slice (CTA of the cluster) that finishes this quarter of the rows
    const int lq = q / p.splits;              // which of the owner's quarters it is
    if (owner != slice) {
      // This warp's partial sums go to the owner: unit [lq][source slice, skipping the owner's own][m][lane].
      // They are laid out in this CTA's first weight buffer (free: all its MMAs are complete) and travel as one
      // bulk copy; plain remote stores were measured at ~0.1 us per activation row.
      const int unit = lq * (p.splits - 1) + (slice < owner ? slice : slice - 1);
      const uint32_t scratch = sW + (uint32_t)(warp - 2) * C::PART_UNIT;
#pragma unroll
      for (int m = 0; m < NT; ++m) st_shared_f32(scratch + m * 128 + lane * 4, __uint_as_float(r[m]));
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0)
        bulk_copy_to_cluster(map_to_cta(sPart + unit * C::PART_UNIT, owner), scratch, C::PART_UNIT,
                             map_to_cta(part_bar + 8 * lq, owner));
      if (warp == 2 && lane == 0) AC4K_TRS(6);
    } else {
      if (p.splits > 1) {
        const bool got = mbar_wait(part_bar + 8 * lq, 0, p.wait_ns);
        if (!got && lane == 0) atomicExch(p.status, kStatusTimeoutEpilogue);
      }
      if (warp == 2 && lane == 0) AC4K_TRS(6);
      if (n < p.N && tfull_ok) {
        const uint32_t part0 = sPart + lq * (p.splits - 1) * C::PART_UNIT + lane * 4;
        T *dst = static_cast<T *>(p.D) + n;
        if (p.splits == 4) finish_rows<NT, 4, OUT_DT>(r, part0, slice, p, n, dst);
        else if (p.splits == 2) finish_rows<NT, 2, OUT_DT>(r, part0, slice, p, n, dst);
        else finish_rows<NT, 1, OUT_DT>(r, part0, slice, p, n, dst);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  // The bulk copies read this CTA's shared memory and complete on the owners' barriers only: every owner has
  // seen its copies arrive before it reaches this barrier, so no CTA leaves while a copy still reads from it.
  // (A relaxed arrive: nothing is handed over here, and the release form would also wait for this CTA's output
  // stores - measured at 0.2 us per activation row.)
  if (p.splits > 1) cluster_sync_relaxed();
  if (threadIdx.x == 0) AC4K_TRS(2);
}

template <int NT, bool SF_TILED, int OUT_DT>
static int launch_skinny(const CUtensorMap &tx, const CUtensorMap &tw, const GemmArgs &args, cudaStream_t stream) {
  using C = skinny::Cfg<NT>;
  auto kern = linear_nvfp4_skinny_kernel<NT, SF_TILED, OUT_DT>;
  static PerDevice<int> attr_set;
  int unused = 0;
  if (int e = attr_set.get(&unused, [&](int &v) {
        AC4K_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
        v = 1;
        return 0;
      }))
    return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(args.tiles_n * args.splits);
  cfg.blockDim = dim3(skinny::kThreads);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.numAttrs = 1;
  if (args.splits > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = args.splits;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  cfg.attrs = attr;
  AC4K_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tx, tw, args));
  return 0;
}

template <int NT, bool SF_TILED>
static int launch_skinny_dt(int d_dtype, const CUtensorMap &tx, const CUtensorMap &tw, const GemmArgs &a, cudaStream_t st) {
  switch (d_dtype) {
    case AC4K_DT_BF16: return launch_skinny<NT, SF_TILED, AC4K_DT_BF16>(tx, tw, a, st);
    case AC4K_DT_FP16: return launch_skinny<NT, SF_TILED, AC4K_DT_FP16>(tx, tw, a, st);
    default: return launch_skinny<NT, SF_TILED, AC4K_DT_FP32>(tx, tw, a, st);
  }
}

// args: M <= nt, tiles_n = ceil(N / 128), splits in {1, 2, 4}, kt_per_split stages of K = 256 per slice
int launch_linear_skinny(int d_dtype, bool sf_tiled, int nt, const CUtensorMap &tx, const CUtensorMap &tw, const GemmArgs &args,
                         cudaStream_t stream) {
  if (nt == 16)
    return sf_tiled ? launch_skinny_dt<16, true>(d_dtype, tx, tw, args, stream) : launch_skinny_dt<16, false>(d_dtype, tx, tw, args, stream);
  if (nt == 32)
    return sf_tiled ? launch_skinny_dt<32, true>(d_dtype, tx, tw, args, stream) : launch_skinny_dt<32, false>(d_dtype, tx, tw, args, stream);
  return sf_tiled ? launch_skinny_dt<64, true>(d_dtype, tx, tw, args, stream) : launch_skinny_dt<64, false>(d_dtype, tx, tw, args, stream);
}

}  // namespace ac4k
