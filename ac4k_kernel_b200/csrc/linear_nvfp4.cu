// NVFP4 block-scaled GEMM for sm_100a:  D[M,N] = cast((gA*gB) * A_fp4[M,K] * B_fp4[N,K]^T + bias).
//
// Stands in for ac4k_kernel's lib/cuda/sm120/linear_nvfp4.cu:337-901 (an mma.sync kernel that
// does not assemble for sm_100a).  This one is a persistent, warp-specialised tcgen05 kernel:
//
//   warp 0   TMA producer: per K-step of 256 elements, one 128-byte-swizzled box of A
//            (128 rows x 128 B), one of B (BN rows x 128 B) and the scale bytes of both,
//            into a multi-stage shared-memory ring guarded by full/empty mbarriers
//   warp 1   MMA issuer: per stage the scales' tcgen05.cp copies (shared -> tensor memory), four
//            K=64 tcgen05.mma kind::mxf4nvf4.block_scale into a TMEM accumulator, and the
//            tcgen05.commit that releases the stage / publishes the accumulator
//   warp 2   before the dependency wait: L2 prefetch of the weight bytes of the CTA's first work item
//   warps 2-5 only for scales in the row layout [K/64][rows][4]: each warp takes every fourth stage,
//            reads its scale words from global memory and writes them to shared memory in the
//            32 x 16-byte order tcgen05.cp wants
//   warps 6-9 epilogue: tcgen05.ld of the accumulator (one TMEM lane quarter per warp),
//            * (gA*gB), + bias, convert, store
// The roles that issue TMA or tcgen05 instructions run with their whole warp converged and predicate
// those instructions on one elected lane (see elect_one()).
//
// Scale factors in tensor memory: the four e4m3 scales of row r for one K=64 step sit in lane
// r % 32 (replicated in all four lane quarters), 32-bit column r / 32, so A (128 rows) takes 4
// columns and B (BN rows) BN/32 columns per step.
#include <mutex>
#include <vector>

#include <cstring>

#include "gemm_common.cuh"

namespace ac4k {
using namespace ptx;

#ifdef AC4K_TRACE_ENABLED
// per-stage clock64 stamps of CTA 0 (region 0: MMA issuer, region 1: epilogue warp 6, region 3: kernel phases)
#define AC4K_TR1(region, it, ev)                                                             \
  do {                                                                                      \
    if (p.trace != nullptr && blockIdx.x == 0 && (it) < 128)                                \
      p.trace[((size_t)(region) * 128 + (it)) * 8 + (ev)] = clock64();                      \
  } while (0)
#else
#define AC4K_TR1(region, it, ev) do { } while (0)
#endif

template <int BN, bool SF_TILED, int OUT_DT>
__global__ void __launch_bounds__(kNumThreads, 1)
linear_nvfp4_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const GemmArgs p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA = smem_base;
  const uint32_t sB = sA + C::STAGES * C::A_BYTES;
  const uint32_t sSFA = sB + C::STAGES * C::B_BYTES;
  const uint32_t sSFB = sSFA + C::STAGES * C::SFA_BYTES;
  const uint32_t bars = sSFB + C::STAGES * C::SFB_BYTES;
  const uint32_t full_bar = bars, empty_bar = bars + 8 * C::STAGES;
  const uint32_t tfull_bar = bars + 16 * C::STAGES, tempty_bar = tfull_bar + 8 * C::ACC_STAGES;
  const uint32_t tmem_slot = tempty_bar + 8 * C::ACC_STAGES;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));   // generic pointer to smem_base

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // work item = (tile, K split); consecutive items walk the tiles first so that concurrent CTAs
  // stream different weight rows
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_work = num_tiles * p.splits;
  const int k_tiles_all = (p.KT + K64_PER_STAGE - 1) / K64_PER_STAGE;
  auto work_item = [&](int wi, int &t, int &split) { t = wi % num_tiles; split = wi / num_tiles; };

  if (threadIdx.x == 0) AC4K_TR1(3, 0, 0);
#ifdef AC4K_TRACE_ENABLED
#define AC4K_TRW(ev) do { if (p.trace != nullptr && blockIdx.x < 127) p.trace[((size_t)4 * 128 + blockIdx.x) * 8 + (ev)] = globaltimer(); } while (0)
#else
#define AC4K_TRW(ev) do { } while (0)
#endif
  if (threadIdx.x == 0) AC4K_TRW(0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full_bar + 8 * s, SF_TILED ? 1 : 2);   // producer's expect_tx arrival (+ the stage's scale warp)
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int a = 0; a < C::ACC_STAGES; ++a) {
      mbar_init(tfull_bar + 8 * a, 1);
      mbar_init(tempty_bar + 8 * a, 4);
    }
    fence_barrier_init();
    prefetch_tmap(&tma_a);
    prefetch_tmap(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  if (warp == 2 && (int)blockIdx.x < num_work) {
    // While the kernel before this one may still be running: ask L2 for the weight bytes of this CTA's
    // first work item (a prefetch returns no data, so the dependency wait below still orders every real
    // read).  On decode shapes that is the CTA's whole share of the weight stream, requested from HBM at
    // once instead of one ring of stages at a time.
    const uint32_t el = elect_one();
    int t, split;
    work_item(blockIdx.x, t, split);
    const int kt0 = split * p.kt_per_split, kt1 = min(k_tiles_all, kt0 + p.kt_per_split);
    int tm, tn;
    tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
    const int npre = min(kt1 - kt0, 48);
    for (int i = 0; i < npre; ++i) tma_prefetch_2d_if(el, &tma_b, (kt0 + i) * BKB, tn * BN);
    if (SF_TILED) {
      for (int nb = 0; nb < BN / 128; ++nb) {
        const int64_t nt = (int64_t)tn * (BN / 128) + nb;
        if (nt * 128 < p.rows_sfb)
          bulk_prefetch_l2_if(el, p.sfb + (nt * p.KT + (int64_t)kt0 * K64_PER_STAGE) * 512,
                              (uint32_t)min((int64_t)npre * K64_PER_STAGE, (int64_t)p.KT - (int64_t)kt0 * K64_PER_STAGE) * 512u);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(smem_gen + (tmem_slot - smem_base));
  // set-up done on this CTA's own resources only; global memory is read and written from here on
  grid_launch_dependents();
  grid_dependency_wait();
  if (threadIdx.x == 0) AC4K_TR1(3, 0, 1);
  if (threadIdx.x == 0) AC4K_TRW(1);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    const uint32_t el = elect_one();
    uint32_t s = 0, ph = 0;
    bool ok = true;
    for (int wi = blockIdx.x; wi < num_work && ok; wi += gridDim.x) {
      int t, split;
      work_item(wi, t, split);
      const int kt0 = split * p.kt_per_split, kt1 = min(k_tiles_all, kt0 + p.kt_per_split);
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      const int m0 = tm * BM, n0 = tn * BN;
      for (int kt = kt0; kt < kt1; ++kt) {
        ok = warp_all(mbar_wait(empty_bar + 8 * s, ph ^ 1, p.wait_ns));
        if (!ok) break;
        const int nk = min(K64_PER_STAGE, p.KT - kt * K64_PER_STAGE);
        uint32_t sf_bytes = 0;
        if (SF_TILED) {
          const int nb_valid = min(BN / 128, (p.rows_sfb - n0) / 128);
          sf_bytes = (1 + nb_valid) * nk * 512;
        }
        const uint32_t fb = full_bar + 8 * s;
        mbar_arrive_expect_tx_if(el, fb, C::A_BYTES + C::B_BYTES + sf_bytes);
        tma_load_2d_if(el, sB + s * C::B_BYTES, &tma_b, kt * BKB, n0, fb);
        tma_load_2d_if(el, sA + s * C::A_BYTES, &tma_a, kt * BKB, m0, fb);
        if (SF_TILED) {
          // [row tile of 128][K/64][512 B]: the nk chunks of one row tile are contiguous
          const int64_t k64 = (int64_t)kt * K64_PER_STAGE;
          bulk_load_1d_if(el, sSFA + s * C::SFA_BYTES, p.sfa + ((int64_t)tm * p.KT + k64) * 512, nk * 512, fb);
          for (int nb = 0; nb < BN / 128; ++nb) {
            const int64_t nt = n0 / 128 + nb;
            if (nt * 128 < p.rows_sfb)
              bulk_load_1d_if(el, sSFB + s * C::SFB_BYTES + nb * (K64_PER_STAGE * 512),
                              p.sfb + (nt * p.KT + k64) * 512, nk * 512, fb);
          }
        }
        if (++s == C::STAGES) { s = 0; ph ^= 1; }
      }
    }
    if (!ok && el) atomicExch(p.status, kStatusTimeoutProducer);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t el = elect_one();
    constexpr uint32_t idesc = make_idesc_mxf4nvf4(BM, BN);
    constexpr int NB = BN / 128;
    uint32_t s = 0, ph = 0, acc = 0, acc_ph = 0;
    bool ok = true;
    int it = 0;
    const uint64_t adesc0 = make_smem_desc(sA, 16, 1024, kSwizzle128B);
    const uint64_t bdesc0 = make_smem_desc(sB, 16, 1024, kSwizzle128B);
    // scale chunks: 32 rows x 16 bytes, 8-row groups 128 bytes apart, not swizzled
    const uint64_t sfadesc0 = make_smem_desc(sSFA, 0, 128, kSwizzleNone);
    const uint64_t sfbdesc0 = make_smem_desc(sSFB, 0, 128, kSwizzleNone);
    const uint32_t t_sfa = tmem_base + C::SF_COL, t_sfb = t_sfa + K64_PER_STAGE * 4;
    for (int wi = blockIdx.x; wi < num_work && ok; wi += gridDim.x) {
      int t_unused, split;
      work_item(wi, t_unused, split);
      const int kt0 = split * p.kt_per_split, kt1 = min(k_tiles_all, kt0 + p.kt_per_split);
      ok = warp_all(mbar_wait(tempty_bar + 8 * acc, acc_ph ^ 1, p.wait_ns));
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kt = kt0; kt < kt1; ++kt) {
        if (el) AC4K_TR1(0, it, 0);
        ok = warp_all(mbar_wait(full_bar + 8 * s, ph, p.wait_ns));
        if (!ok) break;
        tc_fence_after();
        if (el) AC4K_TR1(0, it, 1);
        if (el && it == 0) AC4K_TRW(3);
        const int nk = min(K64_PER_STAGE, p.KT - kt * K64_PER_STAGE);
        const uint64_t adesc = adesc0 + (uint64_t)(s * (C::A_BYTES >> 4));
        const uint64_t bdesc = bdesc0 + (uint64_t)(s * (C::B_BYTES >> 4));
        const uint64_t sfadesc = sfadesc0 + (uint64_t)(s * (C::SFA_BYTES >> 4));
        const uint64_t sfbdesc = sfbdesc0 + (uint64_t)(s * (C::SFB_BYTES >> 4));
        // The scales of the stage go to tensor memory with tcgen05.cp right in front of the MMAs that read
        // them (same thread: executed in issue order, overlapping the MMAs).  K step j: +32 bytes inside the
        // 128-byte swizzle atom = start-address field + 2.
        if (nk == K64_PER_STAGE) {
#pragma unroll
          for (int j = 0; j < K64_PER_STAGE; ++j) {
            tmem_cp_32x128b_warpx4_if(el, t_sfa + j * 4, sfadesc + j * 32);
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
              tmem_cp_32x128b_warpx4_if(el, t_sfb + j * (BN / 32) + nb * 4, sfbdesc + (nb * K64_PER_STAGE + j) * 32);
          }
#pragma unroll
          for (int j = 0; j < K64_PER_STAGE; ++j)
            mma_mxf4nvf4_if(el, d_tmem, adesc + 2 * j, bdesc + 2 * j, idesc, t_sfa + j * 4, t_sfb + j * (BN / 32),
                            (kt > kt0 || j > 0) ? 1u : 0u);
        } else {
          for (int j = 0; j < nk; ++j) {
            tmem_cp_32x128b_warpx4_if(el, t_sfa + j * 4, sfadesc + j * 32);
            for (int nb = 0; nb < NB; ++nb)
              tmem_cp_32x128b_warpx4_if(el, t_sfb + j * (BN / 32) + nb * 4, sfbdesc + (nb * K64_PER_STAGE + j) * 32);
          }
          for (int j = 0; j < nk; ++j)
            mma_mxf4nvf4_if(el, d_tmem, adesc + 2 * j, bdesc + 2 * j, idesc, t_sfa + j * 4, t_sfb + j * (BN / 32),
                            (kt > kt0 || j > 0) ? 1u : 0u);
        }
        tc_commit_if(el, empty_bar + 8 * s);
        if (el) AC4K_TR1(0, it, 3);
        ++it;
        if (++s == C::STAGES) { s = 0; ph ^= 1; }
      }
      if (ok) tc_commit_if(el, tfull_bar + 8 * acc);
      if (el) AC4K_TRW(4);
      if (++acc == C::ACC_STAGES) { acc = 0; acc_ph ^= 1; }
    }
    if (!ok && el) atomicExch(p.status, kStatusTimeoutMma);
  } else if (warp < 6) {
    // ------------------------------------------------------------------ scale warps (row layout only)
    // Scales stored as [K/64][rows][4 bytes]: the word of row r at K step k sits at word k * rows + r.
    // tcgen05.cp wants, per K step and 128-row block, 32 rows of 16 bytes where row l holds the words of
    // rows l, 32 + l, 64 + l, 96 + l.  Warp w takes the stages whose running number is w - 2 modulo 4:
    // its loads are in flight while the stages before it are consumed.
    if (!SF_TILED) {
      const int w4 = warp - 2;
      constexpr int GB = BN / 32;
      uint32_t s = 0, ph = 0, it = 0;
      const uint32_t *sfa_w = reinterpret_cast<const uint32_t *>(p.sfa);
      const uint32_t *sfb_w = reinterpret_cast<const uint32_t *>(p.sfb);
      bool ok = true;
      for (int wi = blockIdx.x; wi < num_work && ok; wi += gridDim.x) {
        int t, split;
        work_item(wi, t, split);
        const int kt0 = split * p.kt_per_split, kt1 = min(k_tiles_all, kt0 + p.kt_per_split);
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kt = kt0; kt < kt1; ++kt) {
          static_assert(C::STAGES >= 4, "four scale warps: each may run at most one round of the ring ahead");
          if ((int)(it & 3) == w4) {
            uint32_t wa[K64_PER_STAGE][4], wb[K64_PER_STAGE][GB];
#pragma unroll
            for (int j = 0; j < K64_PER_STAGE; ++j) {
              const int k64 = kt * K64_PER_STAGE + j;
              const bool k_ok = k64 < p.KT;
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                const int r = m0 + 32 * g + lane;
                wa[j][g] = (k_ok && r < p.rows_sfa) ? __ldg(sfa_w + (int64_t)k64 * p.rows_sfa + r) : 0u;
              }
#pragma unroll
              for (int g = 0; g < GB; ++g) {
                const int r = n0 + 32 * g + lane;
                wb[j][g] = (k_ok && r < p.rows_sfb) ? __ldg(sfb_w + (int64_t)k64 * p.rows_sfb + r) : 0u;
              }
            }
            ok = warp_all(mbar_wait(empty_bar + 8 * s, ph ^ 1, p.wait_ns));
            if (!ok) break;
#pragma unroll
            for (int j = 0; j < K64_PER_STAGE; ++j) {
              st_shared_v4u(sSFA + s * C::SFA_BYTES + j * 512 + lane * 16, wa[j][0], wa[j][1], wa[j][2], wa[j][3]);
#pragma unroll
              for (int nb = 0; nb < BN / 128; ++nb)
                st_shared_v4u(sSFB + s * C::SFB_BYTES + (nb * K64_PER_STAGE + j) * 512 + lane * 16, wb[j][4 * nb],
                              wb[j][4 * nb + 1], wb[j][4 * nb + 2], wb[j][4 * nb + 3]);
            }
            fence_proxy_async_smem();       // the tensor core reads these bytes through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(full_bar + 8 * s);
          }
          ++it;
          if (++s == C::STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (!ok && lane == 0) atomicExch(p.status, kStatusTimeoutSf);
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;                   // TMEM lane quarter this warp may read
    uint32_t acc = 0, acc_ph = 0;
    const float alpha = __fmul_rn(__ldg(p.a_gs), __ldg(p.b_gs));
    const bool vec_ok = (OUT_DT == AC4K_DT_FP32) ? (p.N % 4 == 0) : (p.N % 8 == 0);
    for (int wi = blockIdx.x; wi < num_work; wi += gridDim.x) {
      int t, split;
      work_item(wi, t, split);
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      const bool tfull_ok = mbar_wait(tfull_bar + 8 * acc, acc_ph, p.wait_ns);
      if (!tfull_ok && lane == 0) atomicExch(p.status, kStatusTimeoutEpilogue);
      if (!tfull_ok) break;
      tc_fence_after();
      if (warp == 6 && lane == 0) AC4K_TR1(1, 0, 0);
      if (warp == 6 && lane == 0) AC4K_TRW(5);
      const int row = tm * BM + q * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32_sync(t_row + c, r);
        const int col = tn * BN + c;
        const int ncols = min(32, p.N - col);
        if (p.splits > 1) {
          // split-K: raw fp32 partial sums go to the workspace; alpha, bias and the cast are applied
          // by the reduction kernel
          if (row < p.M && ncols > 0) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
            store_row32<AC4K_DT_FP32>(p.ws, ((int64_t)split * p.M + row) * p.N + col, v, ncols, p.N % 4 == 0);
          }
        } else if (row < p.M && ncols > 0 && !AC4K_DBG(p, 8)) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __fmul_rn(__uint_as_float(r[i]), alpha);
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < ncols) v[i] = __fadd_rn(v[i], load_bias(p.bias, p.bias_dt, col + i));
          }
          store_row32<OUT_DT>(p.D, (int64_t)row * p.N + col, v, ncols, vec_ok);
        }
      }
      if (warp == 6 && lane == 0) AC4K_TR1(1, 0, 1);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar + 8 * acc);
      if (++acc == C::ACC_STAGES) { acc = 0; acc_ph ^= 1; }
    }
  }

  if (threadIdx.x == 0) AC4K_TR1(3, 0, 4);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) AC4K_TR1(3, 0, 5);
  if (threadIdx.x == 0) AC4K_TRW(2);
}

// out[m, n] = cast(alpha * sum_s ws[s, m, n] + bias[n]) for the split-K path; one thread per
// four consecutive columns (N % 4 == 0 on this path).
template <int OUT_DT>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(void *__restrict__ D, const float *__restrict__ ws, const float *__restrict__ a_gs,
                     const float *__restrict__ b_gs, const void *__restrict__ bias, int bias_dt, int splits,
                     int64_t M, int64_t N) {
  using T = typename OutT<OUT_DT>::type;
  const int64_t i4 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total4 = M * N / 4;
  if (i4 >= total4) return;
  const float alpha = __fmul_rn(__ldg(a_gs), __ldg(b_gs));
  float4 acc = __ldcs(reinterpret_cast<const float4 *>(ws) + i4);
  for (int s = 1; s < splits; ++s) {
    const float4 v = __ldcs(reinterpret_cast<const float4 *>(ws + (int64_t)s * M * N) + i4);
    acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y);
    acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
  }
  float o[4] = {__fmul_rn(acc.x, alpha), __fmul_rn(acc.y, alpha), __fmul_rn(acc.z, alpha), __fmul_rn(acc.w, alpha)};
  if (bias != nullptr) {
    const int n = (int)((i4 * 4) % N);
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = __fadd_rn(o[j], load_bias(bias, bias_dt, n + j));
  }
  T *dst = static_cast<T *>(D) + i4 * 4;
  if (OUT_DT == AC4K_DT_FP32) {
    *reinterpret_cast<float4 *>(dst) = make_float4(o[0], o[1], o[2], o[3]);
  } else if (OUT_DT == AC4K_DT_BF16) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
    *reinterpret_cast<uint2 *>(dst) = make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
  } else {
    __half2 lo = __floats2half2_rn(o[0], o[1]), hi = __floats2half2_rn(o[2], o[3]);
    *reinterpret_cast<uint2 *>(dst) = make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Tensor maps depend only on (pointer, shape, box); encoding one costs a driver call, so the last few
// are kept, per device, behind a mutex.  The reference re-encodes five per call (linear_nvfp4.cu:842-886).
struct TmapKey {
  const void *ptr;
  int64_t d0, d1, pitch;   // extents: innermost (elements), outer; row pitch in elements
  int box0, box1, kind, dev;
  bool rows4;              // rank 3: the d1 rows as (row / 4, row % 4), box {box0, box1, box2}
  int box2;
  bool operator==(const TmapKey &o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && pitch == o.pitch && box0 == o.box0 && box1 == o.box1 &&
           kind == o.kind && dev == o.dev && rows4 == o.rows4 && box2 == o.box2;
  }
};
struct TmapEntry { TmapKey key; CUtensorMap map; };
enum { kTmapOperand = 0, kTmapWords = 1, kTmapOut16 = 2, kTmapOperand64 = 3 };

// kind kTmapOperand / kTmapOperand64: bytes, 128- / 64-byte swizzle; kTmapWords: 32-bit words, not swizzled;
// kTmapOut16: 16-bit elements, 128-byte swizzle.
// rows4: a rank-3 map {d0, d1 / 4, 4} with strides {4 * pitch, pitch}: coordinate (x, i, q) is row 4 i + q, and a box
// {box0, box1, box2} lands in shared memory with q outermost.
static int encode_cached(int kind, const void *ptr, int64_t d0, int64_t d1, int64_t pitch, int box0, int box1,
                         CUtensorMap *out, bool rows4 = false, int box2 = 1) {
  static std::mutex mu;
  static std::vector<TmapEntry> cache;
  int dev = 0;
  cudaGetDevice(&dev);
  TmapKey key{ptr, d0, d1, pitch, box0, box1, kind, dev, rows4, box2};
  {
    std::lock_guard<std::mutex> lk(mu);
    for (auto &e : cache)
      if (e.key == key) { *out = e.map; return 0; }
  }
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return fail(AC4K_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  const bool bytes = kind == kTmapOperand || kind == kTmapOperand64;
  const int esize = bytes ? 1 : (kind == kTmapWords ? 4 : 2);
  const CUtensorMapSwizzle swz = (kind == kTmapOperand || kind == kTmapOut16) ? CU_TENSOR_MAP_SWIZZLE_128B
                                 : (kind == kTmapOperand64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE);
  const CUtensorMapDataType dt = bytes ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : (kind == kTmapWords ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16);
  cuuint64_t gdim[3] = {(cuuint64_t)d0, (cuuint64_t)d1, 1};
  cuuint64_t gstride[2] = {(cuuint64_t)pitch * esize, 0};
  cuuint32_t box[3] = {(cuuint32_t)box0, (cuuint32_t)box1, (cuuint32_t)box2};
  cuuint32_t estr[3] = {1, 1, 1};
  if (rows4) {
    gdim[1] = (cuuint64_t)(d1 / 4);
    gdim[2] = 4;
    gstride[0] = (cuuint64_t)pitch * esize * 4;
    gstride[1] = (cuuint64_t)pitch * esize;
  }
  CUtensorMap m;
  CUresult r = enc(&m, dt, rows4 ? 3 : 2,
                   const_cast<void *>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swz,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail((int)r > 0 ? (int)r : 999, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  {
    std::lock_guard<std::mutex> lk(mu);
    if (cache.size() >= 64) cache.erase(cache.begin());
    cache.push_back({key, m});
  }
  *out = m;
  return 0;
}

// packed operand [rows, row_bytes]: boxes of 128 bytes x box_rows rows, 128-byte swizzle
int get_tmap(const void *ptr, int64_t rows, int64_t row_bytes, int box_rows, CUtensorMap *out) {
  return encode_cached(kTmapOperand, ptr, row_bytes, rows, row_bytes, BKB, box_rows, out);
}

// Tiled scale factors [row blocks of 128][K/64][512 bytes] seen as a matrix of 512-byte rows: a box of
// `box_ksteps` rows is the scale image of that many K steps of one row block, contiguous in shared
// memory.  Rows past the end of the tensor read as zero.
int get_tmap_sf_tiled(const void *ptr, int64_t row_blocks, int64_t kt, int box_ksteps, CUtensorMap *out) {
  return encode_cached(kTmapWords, ptr, 128, row_blocks * kt, 128, 128, box_ksteps, out);
}

int get_tmap_out16(const void *ptr, int64_t rows, int64_t cols, int64_t ld, CUtensorMap *out) {
  return encode_cached(kTmapOut16, ptr, cols, rows, ld, 64, 32, out);
}

int get_tmap_rows4(const void *ptr, int64_t rows, int64_t row_bytes, CUtensorMap *out) {
  return encode_cached(kTmapOperand, ptr, row_bytes, rows, row_bytes, BKB, 32, out, true, 4);
}

int get_tmap_out16_rows4(const void *ptr, int64_t rows, int64_t cols, int64_t ld, CUtensorMap *out) {
  return encode_cached(kTmapOut16, ptr, cols, rows, ld, 64, 32, out, true, 1);
}

// Scale factors in the row layout [K/64][rows][4 bytes] seen as a [K/64, rows] matrix of words: the 128 words of a
// 128-row block at 4 K steps.  Words past the rows or the K steps read as zero.
int get_tmap_sf_rows(const void *ptr, int64_t rows, int64_t kt, CUtensorMap *out) {
  return encode_cached(kTmapWords, ptr, rows, kt, rows, 128, 4, out);
}

// packed operand [rows, row_bytes] whose contraction rows are 64 bytes: boxes of 64 bytes x box_rows rows, 64-byte swizzle
int get_tmap64(const void *ptr, int64_t rows, int64_t row_bytes, int box_rows, CUtensorMap *out) {
  return encode_cached(kTmapOperand64, ptr, row_bytes, rows, row_bytes, 64, box_rows, out);
}

// bf16 tensor [B, H, N, D] given by element strides (D contiguous): boxes of D x box_rows x 1 x 1, not swizzled.  Rows
// past N read as zero.  Kept in a small cache of its own (key: pointer, shape, strides, box).
int get_tmap_bf16_4d(const void *ptr, const int64_t shape[4], const int64_t stride[4], int box_rows, CUtensorMap *out) {
  struct Key { const void *ptr; int64_t sh[4], st[3]; int box, dev; };
  struct Entry { Key k; CUtensorMap m; };
  static std::mutex mu;
  static std::vector<Entry> cache;
  int dev = 0;
  cudaGetDevice(&dev);
  Key key{ptr, {shape[0], shape[1], shape[2], shape[3]}, {stride[0], stride[1], stride[2]}, box_rows, dev};
  auto same = [](const Key &a, const Key &b) {
    return a.ptr == b.ptr && a.box == b.box && a.dev == b.dev && a.sh[0] == b.sh[0] && a.sh[1] == b.sh[1] && a.sh[2] == b.sh[2] &&
           a.sh[3] == b.sh[3] && a.st[0] == b.st[0] && a.st[1] == b.st[1] && a.st[2] == b.st[2];
  };
  {
    std::lock_guard<std::mutex> lk(mu);
    for (auto &e : cache)
      if (same(e.k, key)) { *out = e.m; return 0; }
  }
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return fail(AC4K_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[4] = {(cuuint64_t)shape[3], (cuuint64_t)shape[2], (cuuint64_t)shape[1], (cuuint64_t)shape[0]};
  cuuint64_t gstride[3] = {(cuuint64_t)stride[2] * 2, (cuuint64_t)stride[1] * 2, (cuuint64_t)stride[0] * 2};
  cuuint32_t box[4] = {(cuuint32_t)shape[3], (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMap m;
  CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void *>(ptr), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail((int)r > 0 ? (int)r : 999, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  {
    std::lock_guard<std::mutex> lk(mu);
    if (cache.size() >= 32) cache.erase(cache.begin());
    cache.push_back({key, m});
  }
  *out = m;
  return 0;
}

int get_device_info(DeviceInfo *out) {
  static PerDevice<DeviceInfo> info;
  return info.get(out, [](DeviceInfo &v) {
    int dev = 0;
    AC4K_CUDA_TRY(cudaGetDevice(&dev));
    AC4K_CUDA_TRY(cudaDeviceGetAttribute(&v.sms, cudaDevAttrMultiProcessorCount, dev));
    AC4K_CUDA_TRY(cudaDeviceGetAttribute(&v.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    v.ok = true;
    return 0;
  });
}

template <int BN, bool SF_TILED, int OUT_DT>
static int launch(const CUtensorMap &ta, const CUtensorMap &tb, const GemmArgs &args, int sms, cudaStream_t stream) {
  using C = Cfg<BN>;
  auto kern = linear_nvfp4_kernel<BN, SF_TILED, OUT_DT>;
  static PerDevice<int> attr_set;
  int unused = 0;
  if (int e = attr_set.get(&unused, [&](int &v) {
        AC4K_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
        v = 1;
        return 0;
      }))
    return e;
  const int num_work = args.tiles_m * args.tiles_n * args.splits;
  const int grid = num_work < sms ? num_work : sms;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kNumThreads);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  // set-up may overlap the previous kernel's tail (see grid_dependency_wait)
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = AC4K_DBG(args, 64) ? 0 : 1;
  cfg.numAttrs = 1;
  cfg.attrs = attr;
  AC4K_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, ta, tb, args));
  return 0;
}

template <int BN, bool SF_TILED>
static int launch_dt(int d_dtype, const CUtensorMap &ta, const CUtensorMap &tb, const GemmArgs &a, int sms,
                     cudaStream_t st) {
  switch (d_dtype) {
    case AC4K_DT_BF16: return launch<BN, SF_TILED, AC4K_DT_BF16>(ta, tb, a, sms, st);
    case AC4K_DT_FP16: return launch<BN, SF_TILED, AC4K_DT_FP16>(ta, tb, a, sms, st);
    default: return launch<BN, SF_TILED, AC4K_DT_FP32>(ta, tb, a, sms, st);
  }
}

}  // namespace ac4k

using namespace ac4k;

// Measurement switches.  They exist only in builds with -DAC4K_DEBUG_HOOKS (the trace build implies it); the
// library built by default neither exports these symbols nor contains the branches they steer.  They are
// process-wide and unsynchronised: for benchmarks and experiments, never for production use.
//   ac4k_debug_set_tile_n(bn)   0 automatic; 128 / 256 force the single-CTA kernel with that tile
//                               width; 512 forces the CTA-pair kernel
//   ac4k_debug_set_splits(n)    0 automatic; 1 never cut K into slices; n > 1 force n slices
//   ac4k_debug_set_flags(bits)  8 skip the epilogue's stores; 64 launch without the
//                               programmatic-stream-serialization attribute; 128 no L2 prefetch before the
//                               dependency wait (pair kernel)
//                               256 the pair kernel's producer leaves out the loads of its very first stage, so that
//                               the waits for it expire (the wait-expiry test)
//   ac4k_debug_set_wait_ns(ns)  limit of the device-side waits of later launches (0 = the default 2 s)
//   ac4k_debug_set_trace(ptr)   device buffer for the clock stamps of builds with -DAC4K_TRACE_ENABLED
#ifdef AC4K_DEBUG_HOOKS
static int g_force_bn = 0;
static int g_force_splits = 0;
static int g_dbg = 0;
static unsigned long long *g_trace = nullptr;
static unsigned long long g_wait_ns = 0;
extern "C" __attribute__((visibility("default"))) void ac4k_debug_set_wait_ns(unsigned long long ns) { g_wait_ns = ns; }
extern "C" __attribute__((visibility("default"))) void ac4k_debug_set_splits(int n) { g_force_splits = n; }
extern "C" __attribute__((visibility("default"))) void ac4k_debug_set_trace(void *p) { g_trace = static_cast<unsigned long long *>(p); }
extern "C" __attribute__((visibility("default"))) void ac4k_debug_set_flags(int f) { g_dbg = f; }
extern "C" __attribute__((visibility("default"))) void ac4k_debug_set_tile_n(int bn) { g_force_bn = bn; }
#else
static constexpr int g_force_bn = 0, g_force_splits = 0, g_dbg = 0;
static constexpr unsigned long long *g_trace = nullptr;
static constexpr unsigned long long g_wait_ns = 0;
#endif
// the clock-stamp buffer of trace builds for the other kernels of the library (NULL otherwise)
unsigned long long *ac4k::debug_trace_ptr() { return g_trace; }

// Split-K plan of the single-CTA kernel for shapes with too few output tiles to occupy the GPU (65 <= M <= 128,
// or any M with an output the other kernels do not store): how many K slices, and the fp32 workspace
// [splits, M, N] they need.  splits == 1 means no workspace.  (M <= 64 takes the decode-shape kernel, whose
// slices are added inside a cluster.)
struct SplitPlan { int splits; int kt_per_split; size_t ws_bytes; };

static SplitPlan plan_split(int64_t M, int64_t N, int64_t K, int bn, int sms) {
  SplitPlan pl{1, (int)ceil_div(K / 64, K64_PER_STAGE), 0};
  const int64_t tiles = ceil_div(M, BM) * ceil_div(N, bn);
  const int k_tiles = pl.kt_per_split;
  if (g_force_splits == 1 || N % 4 != 0 || tiles * 2 > sms) return pl;
  // Measured on decode-like shapes (graph timing): with K = 4096 (16 stages) no split wins for any tile
  // count (9.0 vs 9.5 - 12.6 us at 64 x 4096 x 4096); with K = 8192 slices pay when few tiles would
  // leave most SMs idle (32 x 2048 x 8192: 13.5 -> 9.1 us with 8 slices) and, at 64 tiles, only for a
  // small M, whose partial sums are cheap to add (16 rows: 15.9 -> 14.4 us; 128 rows: 16.1 -> 17.1 us)
  if (g_force_splits == 0 && (k_tiles < 32 || (M > 64 && tiles >= 32))) return pl;
  if (k_tiles < 8) return pl;
  int splits = g_force_splits > 1 ? g_force_splits : (int)(sms / tiles);
  if (splits > k_tiles / 4) splits = k_tiles / 4;      // at least four pipeline stages per slice
  if (splits < 2) return pl;
  pl.kt_per_split = (int)ceil_div(k_tiles, splits);
  pl.splits = (int)ceil_div(k_tiles, pl.kt_per_split);
  pl.ws_bytes = (size_t)pl.splits * (size_t)M * (size_t)N * sizeof(float);
  return pl;
}

// ws_mode: 0 = workspace from the stream-ordered allocator (cudaMallocAsync / cudaFreeAsync),
//          1 = fixed workspace of ws_capacity bytes, its address obtained from ws_fixed() only when a
//              call really needs scratch (no allocation in this call)
// `more`: further destinations that receive the same tile stores (the fused all-gather), each a
// [M, ldd] buffer written at columns [col_off, col_off + N); NULL / 0 for the plain GEMM, which
// writes D as a dense [M, N] matrix.
struct OutSpec { void *const *more; int n_more; int64_t ldd; int64_t col_off;
                 // re-quantising epilogue: packed output, its scales, its global scale, scale layout
                 uint8_t *q_out = nullptr; uint8_t *q_sf = nullptr; const float *q_gs = nullptr; int q_layout = 0; };

static int linear_impl(void *D, int d_dtype, const void *A, const void *A_sf, const float *A_gs,
                       const void *B, const void *B_sf, const float *B_gs, const void *bias,
                       int bias_dtype, int64_t M, int64_t N, int64_t K, int sf_layout,
                       cudaStream_t stream, int ws_mode, int (*ws_fixed)(float **), size_t ws_capacity,
                       const OutSpec *out = nullptr) {
  if (M < 0 || N < 0 || K < 0) return fail(AC4K_ERR_SHAPE, "negative dimension");
  if (d_dtype < 0 || d_dtype > 2) return fail(AC4K_ERR_ENUM, "unknown d_dtype %d", d_dtype);
  if (bias && (bias_dtype < 0 || bias_dtype > 2)) return fail(AC4K_ERR_ENUM, "unknown bias_dtype %d", bias_dtype);
  if (sf_layout != AC4K_SF_AC4K && sf_layout != AC4K_SF_TILE128X4)
    return fail(AC4K_ERR_ENUM, "unknown sf_layout %d", sf_layout);
  if (M == 0 || N == 0) return 0;
  const bool requant = out && out->q_out;
  if ((!D && !requant) || !A || !B || !A_sf || !B_sf || !A_gs || !B_gs) return fail(AC4K_ERR_NULL, "a required pointer is NULL");
  if (K == 0 || K % 64 != 0)
    return fail(AC4K_ERR_SHAPE, "K = %lld must be a positive multiple of 64 (the quantiser pads K to 64)", (long long)K);
  if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return fail(AC4K_ERR_SHAPE, "dimension too large");
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(A_sf) & 15) || (reinterpret_cast<uintptr_t>(B_sf) & 15) ||
      (reinterpret_cast<uintptr_t>(D) & 15))
    return fail(AC4K_ERR_ALIGN, "A, B, A_sf, B_sf and D must be 16-byte aligned");
  DeviceInfo di;
  if (int e = get_device_info(&di)) return e;
  if (di.cc_major != 10) return fail(AC4K_ERR_DEVICE, "linear_nvfp4 needs an sm_100 device (found sm_%d0)", di.cc_major);
  unsigned int *status = device_status_ptr();
  if (!status) return fail(AC4K_ERR_DEVICE, "cannot resolve the device status word");

  // kernel choice: CTA pairs (256 x 256 tiles; the epilogue packs 16-bit outputs and stores 32-byte
  // row pieces, which needs N % 8 == 0) when there are at least two row tiles to pair; otherwise single
  // CTAs with 128 x 256 or 128 x 128 tiles.  g_force_bn: 128 / 256 force the single-CTA kernel, 512 forces pairs.
  const bool pair_ok = d_dtype != AC4K_DT_FP32 && (N % 8 == 0);
  bool use_pair = pair_ok && M > 128 && N > 128;
  if (out) {
    // strided / multi-destination output exists in the pair kernel only
    if (!pair_ok) return fail(AC4K_ERR_UNSUPPORTED, "the gathered output needs a 16-bit output type and N %% 8 == 0");
    use_pair = true;
  }
  int bn = N > 128 ? 256 : 128;
  if (!out && (g_force_bn == 128 || g_force_bn == 256)) { use_pair = false; bn = g_force_bn; }
  if (g_force_bn == 512 && pair_ok) use_pair = true;
  SplitPlan pl{1, (int)ceil_div(K / 64, K64_PER_STAGE), 0};
  if (!use_pair) {
    // few output tiles (decode shapes): narrower tiles and K slices put more SMs on the weight stream
    if (g_force_bn == 0 && ceil_div(M, BM) * ceil_div(N, 256) * 2 <= di.sms) bn = 128;
    pl = plan_split(M, N, K, bn, di.sms);
  }
  // Decode shapes (a few activation rows): the kernel built around the weight stream.  K slices of a tile run
  // as one cluster and add their partial sums through distributed shared memory: no scratch memory.
  if (!out && M <= 64 && g_force_bn == 0) {
    const int nt = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    const int64_t tiles_n = ceil_div(N, 128);
    const int k_tiles = (int)ceil_div(K / 64, 4);
    int splits = 1;
    for (int cand = 4; cand >= 2; cand /= 2)      // 4, 2 or 1 slices: as many as keep one wave of CTAs (two per SM)
      if (tiles_n * cand <= 2 * di.sms && k_tiles / cand >= 4) { splits = cand; break; }
    if (g_force_splits >= 1) splits = g_force_splits >= 4 ? 4 : (g_force_splits >= 2 ? 2 : 1);
    while (splits > 1 && ceil_div(k_tiles, ceil_div(k_tiles, splits)) != splits) splits /= 2;   // every slice non-empty
    CUtensorMap tx, tw;
    if (int e = get_tmap(A, M, K / 2, nt, &tx)) return e;
    if (int e = get_tmap(B, N, K / 2, 128, &tw)) return e;
    GemmArgs a = {};
    a.sfa = static_cast<const uint8_t *>(A_sf);
    a.sfb = static_cast<const uint8_t *>(B_sf);
    a.D = D;
    a.n_dst = 1;
    a.ldd = N;
    a.a_gs = A_gs; a.b_gs = B_gs;
    a.bias = bias; a.bias_dt = bias_dtype;
    a.status = status;
    a.M = (int)M; a.N = (int)N; a.K = (int)K; a.KT = (int)(K / 64);
    const int pad = sf_layout == AC4K_SF_AC4K ? 16 : 128;
    a.rows_sfa = (int)align_up(M, pad);
    a.rows_sfb = (int)align_up(N, pad);
    a.tiles_m = 1;
    a.tiles_n = (int)tiles_n;
    a.kt_per_split = (int)ceil_div(k_tiles, splits);
    a.splits = splits;
    a.trace = g_trace;
    a.wait_ns = g_wait_ns ? g_wait_ns : kWaitTimeoutNs;
    return launch_linear_skinny(d_dtype, sf_layout == AC4K_SF_TILE128X4, nt, tx, tw, a, stream);
  }
  CUtensorMap ta, tb;
  if (int e = get_tmap(A, M, K / 2, BM, &ta)) return e;
  if (int e = get_tmap(B, N, K / 2, use_pair ? 128 : bn, &tb)) return e;

  GemmArgs a = {};
  a.sfa = static_cast<const uint8_t *>(A_sf);
  a.sfb = static_cast<const uint8_t *>(B_sf);
  a.D = D;
  a.n_dst = 1;
  a.ldd = N;
  a.col_off = 0;
  for (int i = 0; i < kMaxDst - 1; ++i) a.D_more[i] = nullptr;
  a.q_out = nullptr; a.q_sf = nullptr; a.q_gs = nullptr; a.q_layout = 0; a.q_rows = 0;
  if (out) {
    a.n_dst = 1 + out->n_more;
    a.ldd = out->ldd;
    a.col_off = out->col_off;
    for (int i = 0; i < out->n_more; ++i) a.D_more[i] = out->more[i];
    if (out->q_out) {
      a.q_out = out->q_out; a.q_sf = out->q_sf; a.q_gs = out->q_gs; a.q_layout = out->q_layout;
      a.q_rows = (int)align_up(M, out->q_layout == AC4K_SF_AC4K ? 16 : 128);
    }
  }
  a.a_gs = A_gs;
  a.b_gs = B_gs;
  a.bias = bias;
  a.status = status;
  a.bias_dt = bias_dtype;
  a.M = (int)M; a.N = (int)N; a.K = (int)K;
  a.KT = (int)(K / 64);
  const int pad = sf_layout == AC4K_SF_AC4K ? 16 : 128;
  a.rows_sfa = (int)align_up(M, pad);
  a.rows_sfb = (int)align_up(N, pad);
  a.tiles_m = (int)ceil_div(M, BM);
  a.tiles_n = (int)ceil_div(N, bn);
  a.dbg = g_dbg;
  a.trace = g_trace;
  a.wait_ns = g_wait_ns ? g_wait_ns : kWaitTimeoutNs;
  a.splits = pl.splits;
  a.kt_per_split = pl.kt_per_split;
  a.ws = nullptr;
  if (!use_pair && pl.splits > 1 && ws_mode == 1 && pl.ws_bytes > ws_capacity)
    return fail(AC4K_ERR_SHAPE, "split-K workspace of %zu bytes exceeds the fixed scratch of %zu bytes",
                pl.ws_bytes, ws_capacity);
  const bool tiled = sf_layout == AC4K_SF_TILE128X4;
  if (use_pair) {
    // Scales in the reference's row layout: with M and N multiples of 4 the operands are loaded with their rows
    // permuted inside each 128-row block, so that the scales can be used as they lie in memory (rank-3 maps; a
    // row count that is no multiple of 4 would let such a map reach up to 3 rows past the tensor); otherwise
    // warps of the kernel re-order the scales.  g_dbg bit 0x200 keeps the re-ordering warps (measurement).
    const bool perm = !tiled && M % 4 == 0 && N % 4 == 0 && !(g_dbg & 0x200);
    const int sf_mode = tiled ? 1 : (perm ? 2 : 0);
    CUtensorMap tsa = ta, tsb = tb;      // placeholders when the scales are read with plain loads
    if (tiled) {
      if (int e = get_tmap_sf_tiled(A_sf, a.rows_sfa / 128, a.KT, 4, &tsa)) return e;
      if (int e = get_tmap_sf_tiled(B_sf, a.rows_sfb / 128, a.KT, 4, &tsb)) return e;
    } else if (perm) {
      if (int e = get_tmap_rows4(A, M, K / 2, &ta)) return e;
      if (int e = get_tmap_rows4(B, N, K / 2, &tb)) return e;
      if (int e = get_tmap_sf_rows(A_sf, a.rows_sfa, a.KT, &tsa)) return e;
      if (int e = get_tmap_sf_rows(B_sf, a.rows_sfb, a.KT, &tsb)) return e;
    }
    // destinations of the epilogue's TMA stores: columns [0, col_off + N) of each [M, ldd] buffer, so that the
    // stores are clipped at this launch's last column
    DstMaps dm;
    for (int i = 0; i < kMaxDst; ++i) dm.m[i] = ta;
    if (!requant) {
      auto out_map = perm ? get_tmap_out16_rows4 : get_tmap_out16;
      if (int e = out_map(D, M, a.col_off + N, a.ldd, &dm.m[0])) return e;
      for (int i = 1; i < a.n_dst; ++i)
        if (int e = out_map(a.D_more[i - 1], M, a.col_off + N, a.ldd, &dm.m[i])) return e;
    }
    return launch_linear_2cta(d_dtype, sf_mode, ta, tb, tsa, tsb, dm, a, stream);
  }
  if (pl.splits > 1) {
    if (ws_mode == 1) {
      if (int e = ws_fixed(&a.ws)) return e;
    } else {
      void *wsp = nullptr;
      AC4K_CUDA_TRY(cudaMallocAsync(&wsp, pl.ws_bytes, stream));
      a.ws = static_cast<float *>(wsp);
    }
  }
  int rc;
  if (bn == 256)
    rc = tiled ? launch_dt<256, true>(d_dtype, ta, tb, a, di.sms, stream)
               : launch_dt<256, false>(d_dtype, ta, tb, a, di.sms, stream);
  else
    rc = tiled ? launch_dt<128, true>(d_dtype, ta, tb, a, di.sms, stream)
               : launch_dt<128, false>(d_dtype, ta, tb, a, di.sms, stream);
  if (pl.splits > 1) {
    if (rc == 0) {
      const int64_t total4 = M * N / 4;
      const unsigned blocks = (unsigned)ceil_div(total4, 256);
      switch (d_dtype) {
        case AC4K_DT_BF16:
          splitk_reduce_kernel<AC4K_DT_BF16><<<blocks, 256, 0, stream>>>(D, a.ws, A_gs, B_gs, bias, bias_dtype, pl.splits, M, N);
          break;
        case AC4K_DT_FP16:
          splitk_reduce_kernel<AC4K_DT_FP16><<<blocks, 256, 0, stream>>>(D, a.ws, A_gs, B_gs, bias, bias_dtype, pl.splits, M, N);
          break;
        default:
          splitk_reduce_kernel<AC4K_DT_FP32><<<blocks, 256, 0, stream>>>(D, a.ws, A_gs, B_gs, bias, bias_dtype, pl.splits, M, N);
      }
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) rc = cuda_fail(e, "splitk_reduce_kernel");
    }
    if (ws_mode == 0) {
      cudaError_t e = cudaFreeAsync(a.ws, stream);
      if (e != cudaSuccess && rc == 0) rc = cuda_fail(e, "cudaFreeAsync");
    }
  }
  return rc;
}

extern "C" int ac4k_linear_nvfp4(void *D, int d_dtype, const void *A, const void *A_sf, const float *A_gs,
                                 const void *B, const void *B_sf, const float *B_gs, const void *bias,
                                 int bias_dtype, int64_t M, int64_t N, int64_t K, int sf_layout,
                                 ac4k_stream_t stream_) {
  return linear_impl(D, d_dtype, A, A_sf, A_gs, B, B_sf, B_gs, bias, bias_dtype, M, N, K, sf_layout,
                     static_cast<cudaStream_t>(stream_), 0, nullptr, 0);
}

// ------------------------------------------------------------------------------------------
// Allocation-free variant
// ------------------------------------------------------------------------------------------
// Some hosts of this library may not allocate device memory while they run: code that executes
// inside a memory-budgeted serving process whose pools are sized once at start-up, plugins that
// are handed device buffers by a framework and are forbidden to call the CUDA allocator, or
// latency-critical loops where an allocator call (even a stream-ordered one) is not acceptable.
// The regular entry point takes the split-K scratch from cudaMallocAsync; this one takes it from
// a fixed array that lives in the library's device image instead.
static constexpr size_t kFixedScratchBytes = 8u << 20;   // 8 MiB, held by every GPU that loads the library
static __device__ __align__(256) unsigned char g_fixed_scratch[kFixedScratchBytes];

// In host code `g_fixed_scratch` is only a handle for the symbol, not a device address: the address
// is looked up once per device, with that device current, and then handed to the kernels.
static int fixed_scratch_ptr(float **out) {
  static PerDevice<float *> scratch;
  return scratch.get(out, [](float *&v) {
    void *ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_fixed_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_fixed_scratch)");
    v = static_cast<float *>(ptr);
    return 0;
  });
}

extern "C" int ac4k_linear_nvfp4_noalloc(void *D, int d_dtype, const void *A, const void *A_sf,
                                         const float *A_gs, const void *B, const void *B_sf,
                                         const float *B_gs, const void *bias, int bias_dtype, int64_t M,
                                         int64_t N, int64_t K, int sf_layout, ac4k_stream_t stream_) {
  return linear_impl(D, d_dtype, A, A_sf, A_gs, B, B_sf, B_gs, bias, bias_dtype, M, N, K, sf_layout,
                     static_cast<cudaStream_t>(stream_), 1, fixed_scratch_ptr, kFixedScratchBytes);
}

// ------------------------------------------------------------------------------------------
// GEMM with the all-gather of its output fused into the epilogue
// ------------------------------------------------------------------------------------------
extern "C" int ac4k_linear_nvfp4_gather(void *const *D_dsts, int n_dst, int64_t ldd, int64_t col_off, int d_dtype,
                                        const void *A, const void *A_sf, const float *A_gs, const void *B,
                                        const void *B_sf, const float *B_gs, const void *bias, int bias_dtype,
                                        int64_t M, int64_t N, int64_t K, int sf_layout, ac4k_stream_t stream_) {
  if (!D_dsts) return fail(AC4K_ERR_NULL, "D_dsts is NULL");
  if (n_dst < 1 || n_dst > kMaxDst) return fail(AC4K_ERR_SHAPE, "n_dst = %d, must be 1..%d", n_dst, kMaxDst);
  if (N < 0 || col_off < 0 || ldd < col_off + N) return fail(AC4K_ERR_SHAPE, "columns [col_off, col_off + N) do not fit in ldd");
  if (ldd % 8 != 0 || col_off % 8 != 0)
    return fail(AC4K_ERR_ALIGN, "ldd and col_off must be multiples of 8 elements (16-byte row segments)");
  for (int i = 0; i < n_dst; ++i) {
    if (!D_dsts[i]) return fail(AC4K_ERR_NULL, "destination %d is NULL", i);
    if (reinterpret_cast<uintptr_t>(D_dsts[i]) & 15) return fail(AC4K_ERR_ALIGN, "destination %d is not 16-byte aligned", i);
  }
  OutSpec out{D_dsts + 1, n_dst - 1, ldd, col_off};
  return linear_impl(D_dsts[0], d_dtype, A, A_sf, A_gs, B, B_sf, B_gs, bias, bias_dtype, M, N, K, sf_layout,
                     static_cast<cudaStream_t>(stream_), 0, nullptr, 0, &out);
}

// ------------------------------------------------------------------------------------------
// Device buffers that other processes of the node can map (CUDA IPC)
// ------------------------------------------------------------------------------------------
extern "C" int ac4k_peer_alloc(int64_t bytes, void **ptr_out, unsigned char handle_out[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (!ptr_out || !handle_out) return fail(AC4K_ERR_NULL, "a required pointer is NULL");
  if (bytes <= 0) return fail(AC4K_ERR_SHAPE, "bytes must be positive");
  void *p = nullptr;
  AC4K_CUDA_TRY(cudaMalloc(&p, (size_t)bytes));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(e, "cudaIpcGetMemHandle");
  }
  memcpy(handle_out, &h, 64);
  *ptr_out = p;
  return 0;
}

extern "C" int ac4k_peer_free(void *ptr) {
  if (ptr) AC4K_CUDA_TRY(cudaFree(ptr));
  return 0;
}

extern "C" int ac4k_peer_open(const unsigned char handle[64], void **ptr_out) {
  if (!handle || !ptr_out) return fail(AC4K_ERR_NULL, "a required pointer is NULL");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void *p = nullptr;
  AC4K_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr_out = p;
  return 0;
}

extern "C" int ac4k_peer_close(void *ptr) {
  if (ptr) AC4K_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return 0;
}

// ------------------------------------------------------------------------------------------
// GEMM whose epilogue re-quantises the bf16 result to NVFP4 (input of the next linear layer)
// ------------------------------------------------------------------------------------------
extern "C" int ac4k_linear_nvfp4_requant(void *out_fp4, void *out_sf, const float *out_gs, int out_sf_layout,
                                         const void *A, const void *A_sf, const float *A_gs, const void *B,
                                         const void *B_sf, const float *B_gs, const void *bias, int bias_dtype,
                                         int64_t M, int64_t N, int64_t K, int sf_layout, ac4k_stream_t stream_) {
  if (!out_fp4 || !out_sf || !out_gs) return fail(AC4K_ERR_NULL, "a required output pointer is NULL");
  if (out_sf_layout != AC4K_SF_AC4K && out_sf_layout != AC4K_SF_TILE128X4)
    return fail(AC4K_ERR_ENUM, "unknown out_sf_layout %d", out_sf_layout);
  if (N % 64 != 0) return fail(AC4K_ERR_UNSUPPORTED, "the re-quantising epilogue needs N %% 64 == 0 (N = %lld)", (long long)N);
  if ((reinterpret_cast<uintptr_t>(out_fp4) & 15) || (reinterpret_cast<uintptr_t>(out_sf) & 15))
    return fail(AC4K_ERR_ALIGN, "out_fp4 and out_sf must be 16-byte aligned");
  OutSpec out{nullptr, 0, N, 0};
  out.q_out = static_cast<uint8_t *>(out_fp4);
  out.q_sf = static_cast<uint8_t *>(out_sf);
  out.q_gs = out_gs;
  out.q_layout = out_sf_layout;
  // D is not written in this mode; the packed output stands in for the alignment checks
  return linear_impl(out_fp4, AC4K_DT_BF16, A, A_sf, A_gs, B, B_sf, B_gs, bias, bias_dtype, M, N, K, sf_layout,
                     static_cast<cudaStream_t>(stream_), 0, nullptr, 0, &out);
}
