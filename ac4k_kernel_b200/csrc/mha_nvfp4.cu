// NVFP4 multi-head attention forward for sm_100a: O = softmax(sm_scale * Q K^T) V with Q, K, V and the
// probabilities P all in NVFP4 (e2m1 values, one e4m3 scale per 16 elements of the contraction dimension, an
// fp32 global scale per tensor).  Stands in for ac4k_kernel's lib/cuda/sm120/mha_nvfp4.cu:322-1077 (an mma.sync
// kernel for sm_120a) behind the same binding (lib/cuda_bindings.cc:49-56, include/ac4k_kernel/ops.h:13-17);
// the arithmetic follows that kernel: S = (gQ gK sm_scale) * Q K^T, running row maximum and row sum in fp32,
// P = exp(S - max) re-quantised per 16 keys with the fixed global scale 1 / (6 * 448)
// (mha_nvfp4.cu:246-319), O accumulated in fp32 and divided by the row sum at the end.
//
// One CTA per (batch, head, 128 query rows); it walks the keys in tiles of 128:
//   warp 0     TMA producer: Q once; per key tile K [128 keys x D] and V^T [D x 128 keys] with their scale
//              chunks, two stages
//   warp 1     MMA issuer: S = Q K^T (tcgen05.mma kind::mxf4nvf4, M = 128 queries, N = 128 keys, K = D) into
//              tensor memory; after the softmax warps have written P: O (+)= P V (M = 128, N = D, K = 128 keys).
//              Block scales go from shared to tensor memory with tcgen05.cp in front of the MMAs.
//   warps 2-5  softmax: thread = query row.  Read S from tensor memory, update the running maximum, rescale O
//              in tensor memory when it moved, exponentiate, quantise P to e2m1 + e4m3 block scales and write
//              both into shared memory in the layouts the tensor core reads (64-byte-swizzled K-major operand,
//              32 x 16-byte scale chunks); at the end scale O by gV / (6 * 448 * row sum) and store bf16.
// All contraction rows are 64 bytes (128 e2m1), hence the 64-byte swizzle everywhere.
//
// Supported: head dimension 128 for Q/K and V (padded by the quantiser), scales in the tiled layout
// [.., 128-row block, K/64, 32 x 16 B]; V quantised along the keys (cross dimension = head dimension) with the
// reference's K permutation (quantize(v, 3, N_dim, swizzle=True), python/ac4k_kernel/ops/attention.py:113-118):
// P is written in the same key order, so scale blocks of P and V cover the same 16 keys as in the reference.
#include "gemm_common.cuh"

namespace ac4k {
using namespace ptx;

namespace mha {
static constexpr int BQ = 128, BKV = 128, D = 128;
static constexpr int kThreads = 192;
static constexpr int TILE_BYTES = 128 * 64;       // 128 rows x 128 e2m1
static constexpr int SF_BYTES = 2 * 512;          // the two K = 64 steps of a 128-wide contraction
static constexpr int KV_STAGES = 2;
static constexpr int SMEM_BYTES = (2 + 2 * KV_STAGES) * TILE_BYTES + (2 + 2 * KV_STAGES) * SF_BYTES + 1024 + 256;
// tensor memory: S (128 keys) | O (128 = D) | scales of Q, K, P, V (8 columns each: 4 per K = 64 step)
static constexpr int S_COL = 0, O_COL = 128, SFQ_COL = 256, SFK_COL = 264, SFP_COL = 272, SFV_COL = 280;
static constexpr int TMEM_COLS = 512;
static constexpr float kPGlobal = 2688.0f;        // 6 * 448: reciprocal of P's fixed global scale
}  // namespace mha

struct MhaArgs {
  const uint8_t *sfq, *sfk, *sfv;       // tiled scales
  const float *q_gs, *k_gs, *v_gs;
  void *O;
  int64_t o_b, o_h, o_n, o_d;           // strides of O in elements
  int B, H, Nq, Nkv, Dv;
  int q_blocks, kv_blocks;              // ceil(Nq / 128), ceil(Nkv / 128)
  int v_k64;                            // align64(Nkv) / 64: K = 64 steps of V^T that exist
  float sm_scale;
  unsigned int *status;
  unsigned long long wait_ns;
};

__device__ __forceinline__ uint32_t e4m3_byte(float s) {
  uint16_t pk;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pk) : "f"(0.0f), "f"(s));
  return pk & 0xFFu;
}
__device__ __forceinline__ float e4m3_to_float(uint32_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(__half(h));
}
__device__ __forceinline__ void st_shared_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared::cta.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x32_f(uint32_t taddr, const float (&v)[32]) {
  uint32_t u[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) u[i] = __float_as_uint(v[i]);
  tmem_st_32x32b_x32(taddr, u);
}

__global__ void __launch_bounds__(mha::kThreads, 1)
mha_nvfp4_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                     const __grid_constant__ CUtensorMap tma_v, const MhaArgs p) {
  using namespace mha;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = smem_base;
  const uint32_t sK = sQ + TILE_BYTES;
  const uint32_t sV = sK + KV_STAGES * TILE_BYTES;
  const uint32_t sP = sV + KV_STAGES * TILE_BYTES;
  const uint32_t sSFQ = sP + TILE_BYTES;
  const uint32_t sSFK = sSFQ + SF_BYTES;
  const uint32_t sSFV = sSFK + KV_STAGES * SF_BYTES;
  const uint32_t sSFP = sSFV + KV_STAGES * SF_BYTES;
  const uint32_t bars = sSFP + SF_BYTES;
  const uint32_t q_full = bars, k_full = bars + 8, v_full = k_full + 8 * KV_STAGES, kv_empty = v_full + 8 * KV_STAGES;
  const uint32_t s_full = kv_empty + 8 * KV_STAGES, p_full = s_full + 8, o_done = p_full + 8, tmem_slot = o_done + 8;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int64_t bh = (int64_t)b * p.H + h;
  const int q_row0 = (int)(bh * p.Nq) + qt * BQ;          // row of Q in the [B*H*Nq, D/2] byte matrix
  const int k_row0 = (int)(bh * p.Nkv);
  const int v_row0 = (int)(bh * p.Dv);              // V^T rows of this head; rows past Dv belong to the next head and are not stored

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(k_full + 8 * s, 1);
      mbar_init(v_full + 8 * s, 1);
      mbar_init(kv_empty + 8 * s, 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);         // the four softmax warps
    mbar_init(o_done, 1);
    fence_barrier_init();
    prefetch_tmap(&tma_q);
    prefetch_tmap(&tma_k);
    prefetch_tmap(&tma_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(smem_gen + (tmem_slot - smem_base));
  grid_launch_dependents();
  grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    const uint32_t el = elect_one();
    mbar_arrive_expect_tx_if(el, q_full, TILE_BYTES + SF_BYTES);
    tma_load_2d_if(el, sQ, &tma_q, 0, q_row0, q_full);
    bulk_load_1d_if(el, sSFQ, p.sfq + ((bh * p.q_blocks + qt) * 2) * 512, SF_BYTES, q_full);
    bool ok = true;
    for (int j = 0; j < p.kv_blocks; ++j) {
      const int s = j & 1;
      ok = warp_all(mbar_wait(kv_empty + 8 * s, ((j >> 1) & 1) ^ 1, p.wait_ns));
      if (!ok) break;
      mbar_arrive_expect_tx_if(el, k_full + 8 * s, TILE_BYTES + SF_BYTES);
      tma_load_2d_if(el, sK + s * TILE_BYTES, &tma_k, 0, k_row0 + j * BKV, k_full + 8 * s);
      bulk_load_1d_if(el, sSFK + s * SF_BYTES, p.sfk + ((bh * p.kv_blocks + j) * 2) * 512, SF_BYTES, k_full + 8 * s);
      // V^T: D rows x 128 keys; of the tile's two K = 64 steps only those below align64(Nkv) exist
      const int nk = min(2, p.v_k64 - 2 * j);
      mbar_arrive_expect_tx_if(el, v_full + 8 * s, TILE_BYTES + nk * 512);
      tma_load_2d_if(el, sV + s * TILE_BYTES, &tma_v, j * 64, v_row0, v_full + 8 * s);
      bulk_load_1d_if(el, sSFV + s * SF_BYTES, p.sfv + (bh * p.v_k64 + 2 * j) * 512, nk * 512, v_full + 8 * s);
    }
    if (!ok && el) atomicExch(p.status, kStatusTimeoutProducer);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t el = elect_one();
    constexpr uint32_t idesc = make_idesc_mxf4nvf4(128, 128);
    const uint64_t qdesc = make_smem_desc(sQ, 16, 512, kSwizzle64B);
    const uint64_t pdesc = make_smem_desc(sP, 16, 512, kSwizzle64B);
    const uint64_t sfqdesc = make_smem_desc(sSFQ, 0, 128, kSwizzleNone);
    const uint64_t sfpdesc = make_smem_desc(sSFP, 0, 128, kSwizzleNone);
    const uint32_t t_s = tmem_base + S_COL, t_o = tmem_base + O_COL;
    bool ok = warp_all(mbar_wait(q_full, 0, p.wait_ns));
    for (int j = 0; j < p.kv_blocks && ok; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      const uint64_t kdesc = make_smem_desc(sK + s * TILE_BYTES, 16, 512, kSwizzle64B);
      const uint64_t vdesc = make_smem_desc(sV + s * TILE_BYTES, 16, 512, kSwizzle64B);
      const uint64_t sfkdesc = make_smem_desc(sSFK + s * SF_BYTES, 0, 128, kSwizzleNone);
      const uint64_t sfvdesc = make_smem_desc(sSFV + s * SF_BYTES, 0, 128, kSwizzleNone);
      ok = warp_all(mbar_wait(k_full + 8 * s, ph, p.wait_ns));
      if (!ok) break;
      tc_fence_after();
      // S = Q K^T over D = 128: two K = 64 steps, 32 bytes apart inside the 64-byte rows
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        if (j == 0) tmem_cp_32x128b_warpx4_if(el, tmem_base + SFQ_COL + 4 * i, sfqdesc + 32 * i);
        tmem_cp_32x128b_warpx4_if(el, tmem_base + SFK_COL + 4 * i, sfkdesc + 32 * i);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
        mma_mxf4nvf4_if(el, t_s, qdesc + 2 * i, kdesc + 2 * i, idesc, tmem_base + SFQ_COL + 4 * i, tmem_base + SFK_COL + 4 * i,
                        i > 0 ? 1u : 0u);
      tc_commit_if(el, s_full);
      // O (+)= P V once the softmax warps have written P (they have also rescaled O by then)
      ok = warp_all(mbar_wait(p_full, j & 1, p.wait_ns));
      if (!ok) break;
      ok = warp_all(mbar_wait(v_full + 8 * s, ph, p.wait_ns));
      if (!ok) break;
      tc_fence_after();
      const int nk = min(2, p.v_k64 - 2 * j);
      for (int i = 0; i < nk; ++i) {
        tmem_cp_32x128b_warpx4_if(el, tmem_base + SFP_COL + 4 * i, sfpdesc + 32 * i);
        tmem_cp_32x128b_warpx4_if(el, tmem_base + SFV_COL + 4 * i, sfvdesc + 32 * i);
      }
      for (int i = 0; i < nk; ++i)
        mma_mxf4nvf4_if(el, t_o, pdesc + 2 * i, vdesc + 2 * i, idesc, tmem_base + SFP_COL + 4 * i, tmem_base + SFV_COL + 4 * i,
                        (j > 0 || i > 0) ? 1u : 0u);
      tc_commit_if(el, kv_empty + 8 * s);
      tc_commit_if(el, o_done);
    }
    if (!ok && el) atomicExch(p.status, kStatusTimeoutMma);
  } else {
    // ------------------------------------------------------------------ softmax, correction, epilogue
    const int q = warp & 3;                   // tensor-memory lane quarter (warps 2-5 -> 2, 3, 0, 1)
    const int row_l = q * 32 + lane;          // query row inside the tile = tensor-memory lane
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t t_s = tmem_base + lane_addr + S_COL, t_o = tmem_base + lane_addr + O_COL;
    // scores in units of log2: p = exp2(s * c1 - m)
    const float c1 = __ldg(p.q_gs) * __ldg(p.k_gs) * p.sm_scale * 1.4426950408889634f;
    float m = -INFINITY, l = 0.0f;
    bool ok = true;
    for (int j = 0; j < p.kv_blocks; ++j) {
      ok = mbar_wait(s_full, j & 1, p.wait_ns);
      if (!ok) break;
      tc_fence_after();
      const int ncols = min(BKV, p.Nkv - j * BKV);       // keys of this tile that exist
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32_sync(t_s + 32 * c, r);
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (32 * c + i < ncols) mx = fmaxf(mx, __uint_as_float(r[i]));
      }
      const float m_new = fmaxf(m, mx * c1);
      if (j > 0) {
        // the previous tile's P V must be complete before O is touched
        ok = mbar_wait(o_done, (j - 1) & 1, p.wait_ns);
        if (!ok) break;
        tc_fence_after();
        const float a = exp2f(m - m_new);
        if (__any_sync(0xffffffffu, a != 1.0f)) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32_sync(t_o + 32 * c, r);
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * a;
            tmem_st_32x32b_x32_f(t_o + 32 * c, v);
          }
          tmem_st_wait();
        }
        l *= a;
      }
      m = m_new;
      // pass 2: probabilities, row sum, NVFP4 quantisation of P (per 16 keys, global scale 1 / 2688)
      uint32_t sfw[2] = {0u, 0u};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32_sync(t_s + 32 * c, r);
        // keys are stored in the order the reference's V quantiser uses ("swizzle": every 32 keys viewed as
        // [4, 4, 2] and transposed to [4(b), 4(a), 2]), so that position n of P meets position n of V^T
        float pr[32];
#pragma unroll
        for (int n = 0; n < 32; ++n) {
          const int i = (((n >> 1) & 3) * 4 + (n >> 3)) * 2 + (n & 1);     // key of this tile chunk held at position n
          pr[n] = (32 * c + i < ncols) ? exp2f(__uint_as_float(r[i]) * c1 - m) : 0.0f;
          l += pr[n];
        }
        uint32_t codes[4];
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
          float bmax = pr[16 * blk];
#pragma unroll
          for (int i = 1; i < 16; ++i) bmax = fmaxf(bmax, pr[16 * blk + i]);
          const uint32_t sb = e4m3_byte(__fmul_rn(kPGlobal, __fmul_rn(bmax, kOneSixth)));
          const float sd = e4m3_to_float(sb);
          const float scale = sd != 0.0f ? __fdiv_rn(kPGlobal, sd) : 0.0f;
          float x[8];
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = __fmul_rn(pr[16 * blk + 8 * hh + i], scale);
            codes[2 * blk + hh] = f32x8_to_e2m1x8(x);
          }
          sfw[c >> 1] |= sb << (8 * (2 * (c & 1) + blk));
        }
        // 16-byte chunk c of this row's 64 bytes, 64-byte swizzle: chunk index ^ ((row / 2) % 4)
        st_shared_v4u(sP + row_l * 64 + ((c ^ ((row_l >> 1) & 3)) << 4), codes[0], codes[1], codes[2], codes[3]);
      }
      // scale chunk of K = 64 step i: 32 rows of 16 bytes, row l holding the words of rows l, 32 + l, 64 + l, 96 + l
      st_shared_u32(sSFP + lane * 16 + q * 4, sfw[0]);
      st_shared_u32(sSFP + 512 + lane * 16 + q * 4, sfw[1]);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok) ok = mbar_wait(o_done, (p.kv_blocks - 1) & 1, p.wait_ns);
    if (!ok) {
      if (lane == 0) atomicExch(p.status, kStatusTimeoutEpilogue);
    } else {
      tc_fence_after();
      const int n = qt * BQ + row_l;
      const float out_scale = __ldg(p.v_gs) / (kPGlobal * l);
      __nv_bfloat16 *dst = static_cast<__nv_bfloat16 *>(p.O) + (int64_t)b * p.o_b + (int64_t)h * p.o_h + (int64_t)n * p.o_n;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32_sync(t_o + 32 * c, r);
        if (n < p.Nq) {
          if (p.o_d == 1 && p.Dv == D && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t w[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 2 * k]) * out_scale,
                                                                __uint_as_float(r[8 * i + 2 * k + 1]) * out_scale);
                w[k] = *reinterpret_cast<const uint32_t *>(&h2);
              }
              reinterpret_cast<uint4 *>(dst + 32 * c)[i] = make_uint4(w[0], w[1], w[2], w[3]);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (32 * c + i < p.Dv) dst[(int64_t)(32 * c + i) * p.o_d] = __float2bfloat16_rn(__uint_as_float(r[i]) * out_scale);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace ac4k

using namespace ac4k;

extern "C" int ac4k_mha_nvfp4_fwd(void *O, const int64_t o_stride[4], const void *Q, const void *Q_sf, const float *Q_gs,
                                  const void *K, const void *K_sf, const float *K_gs, const void *V, const void *V_sf,
                                  const float *V_gs, int64_t B, int64_t H, int64_t Nq, int64_t Nkv, int64_t Dqk, int64_t Dv,
                                  float sm_scale, int sf_layout, ac4k_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!O || !o_stride || !Q || !Q_sf || !Q_gs || !K || !K_sf || !K_gs || !V || !V_sf || !V_gs)
    return fail(AC4K_ERR_NULL, "a required pointer is NULL");
  if (B < 0 || H < 0 || Nq < 0 || Nkv < 0) return fail(AC4K_ERR_SHAPE, "negative dimension");
  if (B == 0 || H == 0 || Nq == 0) return 0;
  if (Nkv == 0) return fail(AC4K_ERR_SHAPE, "attention over zero keys");
  if (Dqk <= 64 || Dqk > 128 || Dv <= 64 || Dv > 128)
    return fail(AC4K_ERR_UNSUPPORTED, "head dimensions in (64, 128] are built (Dqk = %lld, Dv = %lld)", (long long)Dqk, (long long)Dv);
  if (sf_layout != AC4K_SF_TILE128X4)
    return fail(AC4K_ERR_UNSUPPORTED, "the attention kernel reads block scales in the tiled layout (AC4K_SF_TILE128X4)");
  if (B > 65535 || H > 65535 || B * H * Nq > (1ll << 31) - 256 || B * H * Nkv > (1ll << 31) - 256)
    return fail(AC4K_ERR_SHAPE, "dimension too large");
  for (const void *ptr : {Q, Q_sf, K, K_sf, V, V_sf})
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return fail(AC4K_ERR_ALIGN, "Q, K, V and their scales must be 16-byte aligned");
  DeviceInfo di;
  if (int e = get_device_info(&di)) return e;
  if (di.cc_major != 10) return fail(AC4K_ERR_DEVICE, "mha_nvfp4_fwd needs an sm_100 device (found sm_%d0)", di.cc_major);
  unsigned int *status = device_status_ptr();
  if (!status) return fail(AC4K_ERR_DEVICE, "cannot resolve the device status word");
  const int64_t v_k64 = ceil_div(Nkv, 64);
  CUtensorMap tq, tk, tv;
  // Q, K: [B*H*N, 64 bytes] (head dimension padded to 128 by the quantiser); V^T: [B*H*Dv, align64(Nkv)/2 bytes]
  if (int e = get_tmap64(Q, B * H * Nq, 64, 128, &tq)) return e;
  if (int e = get_tmap64(K, B * H * Nkv, 64, 128, &tk)) return e;
  if (int e = get_tmap64(V, B * H * Dv, v_k64 * 32, 128, &tv)) return e;
  MhaArgs a = {};
  a.sfq = static_cast<const uint8_t *>(Q_sf);
  a.sfk = static_cast<const uint8_t *>(K_sf);
  a.sfv = static_cast<const uint8_t *>(V_sf);
  a.q_gs = Q_gs; a.k_gs = K_gs; a.v_gs = V_gs;
  a.O = O;
  a.o_b = o_stride[0]; a.o_h = o_stride[1]; a.o_n = o_stride[2]; a.o_d = o_stride[3];
  a.B = (int)B; a.H = (int)H; a.Nq = (int)Nq; a.Nkv = (int)Nkv; a.Dv = (int)Dv;
  a.q_blocks = (int)ceil_div(Nq, 128);
  a.kv_blocks = (int)ceil_div(Nkv, 128);
  a.v_k64 = (int)v_k64;
  a.sm_scale = sm_scale;
  a.status = status;
  a.wait_ns = kWaitTimeoutNs;
  static PerDevice<int> attr_set;
  int unused = 0;
  if (int e = attr_set.get(&unused, [&](int &v) {
        AC4K_CUDA_TRY(cudaFuncSetAttribute(mha_nvfp4_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mha::SMEM_BYTES));
        v = 1;
        return 0;
      }))
    return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)a.q_blocks, (unsigned)H, (unsigned)B);
  cfg.blockDim = dim3(mha::kThreads);
  cfg.dynamicSmemBytes = mha::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  AC4K_CUDA_TRY(cudaLaunchKernelEx(&cfg, mha_nvfp4_fwd_kernel, tq, tk, tv, a));
  return 0;
}
