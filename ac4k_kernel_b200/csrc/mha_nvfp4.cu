// NVFP4 multi-head attention forward for sm_100a: O = softmax(sm_scale * Q K^T) V with Q, K, V and the
// probabilities P all in NVFP4 (e2m1 values, one e4m3 scale per 16 elements of the contraction dimension, an
// fp32 global scale per tensor).  Stands in for ac4k_kernel's lib/cuda/sm120/mha_nvfp4.cu:322-1077 (an mma.sync
// kernel for sm_120a) behind the same binding (lib/cuda_bindings.cc:49-56, include/ac4k_kernel/ops.h:13-17);
// the arithmetic follows that kernel: S = (gQ gK sm_scale) * Q K^T, running row maximum and row sum in fp32,
// P = exp(S - max) re-quantised per 16 keys with the fixed global scale 1 / (6 * 448)
// (mha_nvfp4.cu:246-319), O accumulated in fp32 and divided by the row sum at the end.
//
// One CTA per (batch, head, 128 query rows), two CTAs per SM; a CTA walks the keys in tiles of 64:
//   warp 0     TMA producer: Q once; per key tile K [64 keys x D], V^T [D x 64 keys] and their scale chunks, four stages
//   warp 1     MMA issuer: S = Q K^T (tcgen05.mma kind::mxf4nvf4, M = 128 queries, N = 64 keys, K = D) into tensor
//              memory; once the softmax warps have written P: O (+)= P V (M = 128, N = D, K = 64 keys).  Block scales
//              go from shared to tensor memory with tcgen05.cp in front of the MMAs.  S of the next key tile is
//              issued as soon as the softmax warps hold the current S in registers, before the current P V.
//   warps 2-5  softmax: thread = query row.  One pass over the 64 scores in registers: running maximum, O rescaled
//              in tensor memory when a maximum of the warp moved, ex2.approx, row sum, P quantised to e2m1 + e4m3
//              block scales (fixed global scale 1 / 2688) and written into shared memory in the layouts the tensor
//              core reads (32-byte-swizzled K-major operand, 32 x 16-byte scale chunk); at the end
//              O * gV / (2688 * row sum) is stored as bf16.
// The softmax is what bounds this kernel (16 ex2 per clock per SM: 1024 cycles for 128 x 128 scores against 330 for
// the four-bit MMAs), hence two CTAs per SM: eight softmax warps, and one CTA's MMAs, waits and TMEM traffic run under
// the other's arithmetic.  Tensor memory per CTA: S 64 + O 128 + scales 24 columns of the 256 allocated.
//
// Supported: head dimensions in (64, 128] (padded to 128 by the quantiser), scales in the tiled layout
// [.., 128-row block, K/64, 32 x 16 B]; V quantised along the keys (cross dimension = head dimension) with the
// reference's K permutation (quantize(v, 3, N_dim, swizzle=True), python/ac4k_kernel/ops/attention.py:113-118):
// P is written in the same key order, so scale blocks of P and V cover the same 16 keys as in the reference.
#include "gemm_common.cuh"

namespace ac4k {
using namespace ptx;

namespace mha {
static constexpr int BQ = 128, BKV = 64, D = 128;
static constexpr int kThreads = 192;
static constexpr int Q_BYTES = BQ * 64;           // 128 rows x 128 e2m1, 64-byte rows
static constexpr int K_BYTES = BKV * 64;          // 64 keys x 128 e2m1
static constexpr int V_BYTES = D * 32;            // 128 head-dimension rows x 64 keys, 32-byte rows
static constexpr int P_BYTES = BQ * 32;           // 128 query rows x 64 keys
static constexpr int SFQ_BYTES = 2 * 512;         // two K = 64 steps of D = 128, 128 rows
static constexpr int SFK_BYTES = 2 * 512;         // the 128-key block the tile lies in (its half is picked by column)
static constexpr int SFV_BYTES = 512;             // one K = 64 step, 128 head-dimension rows
static constexpr int SFP_BYTES = 512;
static constexpr int KV_STAGES = 4;
static constexpr int STAGE_BYTES = K_BYTES + V_BYTES + SFK_BYTES + SFV_BYTES;       // 9 728
static constexpr int SMEM_BYTES = Q_BYTES + 2 * P_BYTES + KV_STAGES * STAGE_BYTES + SFQ_BYTES + 2 * SFP_BYTES + 1024 + 256;
// tensor memory columns
static constexpr int S_COL = 0, O_COL = 64, SFQ_COL = 192, SFK_COL = 200, SFP_COL = 208, SFV_COL = 212;
static constexpr int TMEM_COLS = 256;
static constexpr float kPGlobal = 2688.0f;        // 6 * 448: reciprocal of P's fixed global scale
static_assert(STAGE_BYTES % 512 == 0 && K_BYTES % 1024 == 0 && V_BYTES % 1024 == 0, "tile alignment");
}  // namespace mha

struct MhaArgs {
  const uint8_t *sfq, *sfk, *sfv;       // tiled scales
  const float *q_gs, *k_gs, *v_gs;
  void *O;
  int64_t o_b, o_h, o_n, o_d;           // strides of O in elements
  int B, H, Nq, Nkv, Dv;
  int q_blocks, k_blocks;               // ceil(Nq / 128), ceil(Nkv / 128): 128-row blocks of the Q and K scales
  int kv_tiles;                         // ceil(Nkv / 64): key tiles = K = 64 steps of V^T
  float sm_scale;
  unsigned int *status;
  unsigned long long wait_ns;
  unsigned long long *trace;            // clock stamps (builds with -DAC4K_TRACE_ENABLED), else NULL
};

// Trace builds: CTA (0, 0, 0) stamps clock64 into trace[(region * 128 + key tile) * 8 + event]; region 0 = softmax warp
// of lane quarter 0, region 1 = MMA issuer.
#ifdef AC4K_TRACE_ENABLED
#define AC4K_TRM(region, it, ev)                                                                     \
  do {                                                                                               \
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (it) < 128)   \
      p.trace[((size_t)(region) * 128 + (it)) * 8 + (ev)] = clock64();                               \
  } while (0)
#else
#define AC4K_TRM(region, it, ev) do { } while (0)
#endif

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// max of three (one FMNMX3), and two fp32 operations in one instruction on an aligned register pair
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n.reg .b64 ra, rb, rc, rd;\nmov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\nmov.b64 rc, {%6, %7};\n"
      "fma.rn.f32x2 rd, ra, rb, rc;\nmov.b64 {%0, %1}, rd;\n}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  float2 d;
  asm("{\n.reg .b64 ra, rb, rd;\nmov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\n"
      "mul.rn.f32x2 rd, ra, rb;\nmov.b64 {%0, %1}, rd;\n}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("{\n.reg .b64 ra, rb, rd;\nmov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\n"
      "add.rn.f32x2 rd, ra, rb;\nmov.b64 {%0, %1}, rd;\n}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
// two non-negative fp32 -> two e4m3 bytes (a in the low byte) and their values back as fp32
__device__ __forceinline__ uint32_t e4m3x2_round_trip(float a, float b, float &fa, float &fb) {
  uint16_t pk;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pk) : "f"(b), "f"(a));
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(pk));
  const __half2 hh = *reinterpret_cast<const __half2 *>(&h2);
  fa = __low2float(hh);
  fb = __high2float(hh);
  return pk;
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

__global__ void __launch_bounds__(mha::kThreads, 2)
mha_nvfp4_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                     const __grid_constant__ CUtensorMap tma_v, const MhaArgs p) {
  using namespace mha;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = smem_base;
  const uint32_t sP = sQ + Q_BYTES;
  const uint32_t sKV = sP + 2 * P_BYTES;             // per stage: K | V^T | SFK | SFV   (P and its scales: two buffers)
  const uint32_t sSFQ = sKV + KV_STAGES * STAGE_BYTES;
  const uint32_t sSFP = sSFQ + SFQ_BYTES;
  const uint32_t bars = sSFP + 2 * SFP_BYTES;
  const uint32_t q_full = bars, kv_full = bars + 8, kv_empty = kv_full + 8 * KV_STAGES;
  const uint32_t s_full = kv_empty + 8 * KV_STAGES, s_free = s_full + 8, p_full = s_free + 8, o_done = p_full + 8;
  const uint32_t tmem_slot = o_done + 16;            // o_done: one barrier per P buffer (key tiles of equal parity)
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int64_t bh = (int64_t)b * p.H + h;
  const int q_row0 = (int)(bh * p.Nq) + qt * BQ;    // row of Q in the [B*H*Nq, 64-byte] matrix
  const int k_row0 = (int)(bh * p.Nkv);
  const int v_row0 = (int)(bh * p.Dv);              // V^T rows of this head; rows past Dv belong to the next head and are not stored
  const int n_tiles = p.kv_tiles;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(kv_full + 8 * s, 1);
      mbar_init(kv_empty + 8 * s, 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_free, 4);         // the four softmax warps hold S in registers
    mbar_init(p_full, 4);         // ... have written P and its scales
    mbar_init(o_done, 1);
    mbar_init(o_done + 8, 1);
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
    mbar_arrive_expect_tx_if(el, q_full, Q_BYTES + SFQ_BYTES);
    tma_load_2d_if(el, sQ, &tma_q, 0, q_row0, q_full);
    bulk_load_1d_if(el, sSFQ, p.sfq + ((bh * p.q_blocks + qt) * 2) * 512, SFQ_BYTES, q_full);
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j % KV_STAGES;
      ok = warp_all(mbar_wait(kv_empty + 8 * s, ((j / KV_STAGES) & 1) ^ 1, p.wait_ns));
      if (!ok) break;
      const uint32_t st = sKV + s * STAGE_BYTES, fb = kv_full + 8 * s;
      mbar_arrive_expect_tx_if(el, fb, STAGE_BYTES);
      tma_load_2d_if(el, st, &tma_k, 0, k_row0 + j * BKV, fb);
      tma_load_2d_if(el, st + K_BYTES, &tma_v, j * 32, v_row0, fb);
      bulk_load_1d_if(el, st + K_BYTES + V_BYTES, p.sfk + ((bh * p.k_blocks + (j >> 1)) * 2) * 512, SFK_BYTES, fb);
      bulk_load_1d_if(el, st + K_BYTES + V_BYTES + SFK_BYTES, p.sfv + (bh * p.kv_tiles + j) * 512, SFV_BYTES, fb);
    }
    if (!ok && el) atomicExch(p.status, kStatusTimeoutProducer);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t el = elect_one();
    constexpr uint32_t idesc_s = make_idesc_mxf4nvf4(128, BKV);
    constexpr uint32_t idesc_o = make_idesc_mxf4nvf4(128, D);
    const uint64_t qdesc = make_smem_desc(sQ, 16, 512, kSwizzle64B);
    const uint64_t sfqdesc = make_smem_desc(sSFQ, 0, 128, kSwizzleNone);
    const uint32_t t_s = tmem_base + S_COL, t_o = tmem_base + O_COL;
    bool ok = warp_all(mbar_wait(q_full, 0, p.wait_ns));
    // S of key tile j: two K = 64 steps over D, 32 bytes apart inside the 64-byte rows of Q and K.  The K scales of
    // the tile's 64 keys are columns 2 * (j & 1) and the next of the 128-key block's four.
    auto issue_s = [&](int j) {
      const int s = j % KV_STAGES;
      const uint32_t st = sKV + s * STAGE_BYTES;
      const uint64_t kdesc = make_smem_desc(st, 16, 512, kSwizzle64B);
      const uint64_t sfkdesc = make_smem_desc(st + K_BYTES + V_BYTES, 0, 128, kSwizzleNone);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        if (j == 0) tmem_cp_32x128b_warpx4_if(el, tmem_base + SFQ_COL + 4 * i, sfqdesc + 32 * i);
        tmem_cp_32x128b_warpx4_if(el, tmem_base + SFK_COL + 4 * i, sfkdesc + 32 * i);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
        mma_mxf4nvf4_if(el, t_s, qdesc + 2 * i, kdesc + 2 * i, idesc_s, tmem_base + SFQ_COL + 4 * i,
                        tmem_base + SFK_COL + 4 * i + 2 * (j & 1), i > 0 ? 1u : 0u);
      tc_commit_if(el, s_full);
    };
    if (ok) {
      ok = warp_all(mbar_wait(kv_full, 0, p.wait_ns));
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
    }
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j % KV_STAGES;
      if (el) AC4K_TRM(1, j, 0);
      if (j + 1 < n_tiles) {
        ok = warp_all(mbar_wait(kv_full + 8 * ((j + 1) % KV_STAGES), ((j + 1) / KV_STAGES) & 1, p.wait_ns));
        if (!ok) break;
        ok = warp_all(mbar_wait(s_free, j & 1, p.wait_ns));       // S of tile j is in the softmax warps' registers
        if (!ok) break;
        tc_fence_after();
        if (el) AC4K_TRM(1, j, 1);
        issue_s(j + 1);
        if (el) AC4K_TRM(1, j, 2);
      }
      // O (+)= P V once the softmax warps have written P (they have also rescaled O by then)
      ok = warp_all(mbar_wait(p_full, j & 1, p.wait_ns));
      if (!ok) break;
      tc_fence_after();
      if (el) AC4K_TRM(1, j, 3);
      const uint32_t st = sKV + s * STAGE_BYTES;
      const uint64_t vdesc = make_smem_desc(st + K_BYTES, 16, 256, kSwizzle32B);
      const uint64_t sfvdesc = make_smem_desc(st + K_BYTES + V_BYTES + SFK_BYTES, 0, 128, kSwizzleNone);
      const uint64_t pdesc = make_smem_desc(sP + (j & 1) * P_BYTES, 16, 256, kSwizzle32B);
      const uint64_t sfpdesc = make_smem_desc(sSFP + (j & 1) * SFP_BYTES, 0, 128, kSwizzleNone);
      tmem_cp_32x128b_warpx4_if(el, tmem_base + SFP_COL, sfpdesc);
      tmem_cp_32x128b_warpx4_if(el, tmem_base + SFV_COL, sfvdesc);
      mma_mxf4nvf4_if(el, t_o, pdesc, vdesc, idesc_o, tmem_base + SFP_COL, tmem_base + SFV_COL, j > 0 ? 1u : 0u);
      tc_commit_if(el, kv_empty + 8 * s);
      tc_commit_if(el, o_done + 8 * (j & 1));
      if (el) AC4K_TRM(1, j, 4);
    }
    if (!ok && el) atomicExch(p.status, kStatusTimeoutMma);
  } else {
    // ------------------------------------------------------------------ softmax, correction, epilogue
    const int q = warp & 3;                   // tensor-memory lane quarter (warps 2-5 -> 2, 3, 0, 1)
    const int row_l = q * 32 + lane;          // query row inside the tile = tensor-memory lane
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t t_s = tmem_base + lane_addr + S_COL, t_o = tmem_base + lane_addr + O_COL;
    // scores in units of log2: p = exp2(s * c1 - m)
    // (c1 >= 0: the host rejects a negative sm_scale; the floor keeps -inf * c1 = -inf for masked keys when a global
    // scale is 0)
    const float c1 = fmaxf(__ldg(p.q_gs) * __ldg(p.k_gs) * p.sm_scale * 1.4426950408889634f, 1.17549435e-38f);
    const uint32_t p_row0 = sP + row_l * 32;
    const uint32_t p_xor = (uint32_t)((row_l >> 2) & 1) << 4;       // 32-byte swizzle: 16-byte chunk ^ ((row / 4) % 2)
    float m = -INFINITY, l = 0.0f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      if (q == 0 && lane == 0) AC4K_TRM(0, j, 0);
      ok = warp_all(mbar_wait(s_full, j & 1, p.wait_ns));
      if (!ok) break;
      tc_fence_after();
      if (q == 0 && lane == 0) AC4K_TRM(0, j, 1);
      uint32_t r[64];
      tmem_ld_32x32b_x64_sync(t_s, r);
      if (q == 0 && lane == 0) AC4K_TRM(0, j, 2);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);
      const int ncols = p.Nkv - j * BKV;                 // keys of this tile that exist (>= 64 except in the last tile)
      if (ncols < BKV) {
#pragma unroll
        for (int i = 0; i < BKV; ++i)
          if (i >= ncols) r[i] = 0xff800000u;            // -inf: out of the maximum, probability 0
      }
      // Maxima of the scores per block of 16 in the stored key order (the reference's V quantiser's "swizzle": every 32
      // keys viewed as [4, 4, 2] and transposed to [4(b), 4(a), 2]; positions n, n + 1 hold keys key0(n), key0(n) + 1),
      // and the row maximum from them.  ex2 is monotonic, so a block's largest probability is ex2 of its largest score.
      float bs[4];
#pragma unroll
      for (int bk = 0; bk < 4; ++bk) {
        float v[16];
#pragma unroll
        for (int n = 0; n < 16; n += 2) {
          const int nn = 16 * (bk & 1) + n;
          const int i = 32 * (bk >> 1) + (((nn >> 1) & 3) * 4 + (nn >> 3)) * 2;
          v[n] = __uint_as_float(r[i]);
          v[n + 1] = __uint_as_float(r[i + 1]);
        }
        float t = max3(v[0], v[1], v[2]);
#pragma unroll
        for (int n = 3; n < 15; n += 2) t = max3(t, v[n], v[n + 1]);
        bs[bk] = fmaxf(t, v[15]);
      }
      const float m_new = fmaxf(m, fmaxf(max3(bs[0], bs[1], bs[2]), bs[3]) * c1);
      if (j > 0 && __any_sync(0xffffffffu, m_new != m)) {
        // a maximum of this warp's rows moved: O is rescaled, once the previous tile's P V is complete
        ok = warp_all(mbar_wait(o_done + 8 * ((j - 1) & 1), ((j - 1) >> 1) & 1, p.wait_ns));
        if (!ok) break;
        tc_fence_after();
        const float a = ex2_approx(m - m_new);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t ro[32];
          tmem_ld_32x32b_x32_sync(t_o + 32 * c, ro);
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(ro[i]) * a;
          tmem_st_32x32b_x32_f(t_o + 32 * c, v);
        }
        tmem_st_wait();
        l *= a;
      }
      if (q == 0 && lane == 0) AC4K_TRM(0, j, 3);
      // This tile's P buffer was last read by the P V of two tiles ago.  That MMA was issued before this tile's S, and
      // the tensor pipe completes MMAs (and the commits behind them) in issue order: s_full of this tile, seen above,
      // implies it is complete, so no wait is needed here.
      m = m_new;
      if (q == 0 && lane == 0) AC4K_TRM(0, j, 4);
      // probabilities, row sum, NVFP4 quantisation of P: four blocks of 16 keys, so that position n of P meets position n
      // of V^T
      const uint32_t p_row = p_row0 + (j & 1) * P_BYTES;
      float2 lsum = make_float2(0.0f, 0.0f);
      const float2 c1_2 = make_float2(c1, c1), negm2 = make_float2(-m, -m);
      uint32_t sfw = 0;
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        float2 pr[16];
#pragma unroll
        for (int n = 0; n < 32; n += 2) {
          const int i = 32 * g + (((n >> 1) & 3) * 4 + (n >> 3)) * 2;     // keys held at positions n, n + 1
          const float2 e = ffma2(make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), c1_2, negm2);
          pr[n >> 1] = make_float2(ex2_approx(e.x), ex2_approx(e.y));
          lsum = fadd2(lsum, pr[n >> 1]);
        }
        const float bm0 = ex2_approx(fmaf(bs[2 * g], c1, -m)), bm1 = ex2_approx(fmaf(bs[2 * g + 1], c1, -m));
        float sd0, sd1;
        const uint32_t sb2 = e4m3x2_round_trip(__fmul_rn(kPGlobal, __fmul_rn(bm0, kOneSixth)),
                                               __fmul_rn(kPGlobal, __fmul_rn(bm1, kOneSixth)), sd0, sd1);
        sfw |= sb2 << (16 * g);
        const float sc0 = sd0 != 0.0f ? kPGlobal * rcp_approx(sd0) : 0.0f, sc1 = sd1 != 0.0f ? kPGlobal * rcp_approx(sd1) : 0.0f;
        uint32_t codes[4];
#pragma unroll
        for (int hh = 0; hh < 4; ++hh) {
          const float sc = hh < 2 ? sc0 : sc1;
          const float2 sc2 = make_float2(sc, sc);
          float x[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 y = fmul2(pr[4 * hh + i], sc2);
            x[2 * i] = y.x;
            x[2 * i + 1] = y.y;
          }
          codes[hh] = f32x8_to_e2m1x8(x);
        }
        st_shared_v4u(p_row + (((uint32_t)g << 4) ^ p_xor), codes[0], codes[1], codes[2], codes[3]);
      }
      l += lsum.x + lsum.y;
      // scale chunk: 32 rows of 16 bytes, row `lane` holding the words of query rows lane, 32 + lane, 64 + lane, 96 + lane
      st_shared_u32(sSFP + (j & 1) * SFP_BYTES + lane * 16 + q * 4, sfw);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (q == 0 && lane == 0) AC4K_TRM(0, j, 5);
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok) ok = warp_all(mbar_wait(o_done + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, p.wait_ns));
    if (!ok) {
      if (lane == 0) atomicExch(p.status, kStatusTimeoutEpilogue);
    } else {
      tc_fence_after();
      const int n = qt * BQ + row_l;
      const float out_scale = __ldg(p.v_gs) / (kPGlobal * l);
      __nv_bfloat16 *dst = static_cast<__nv_bfloat16 *>(p.O) + (int64_t)b * p.o_b + (int64_t)h * p.o_h + (int64_t)n * p.o_n;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t ro[32];
        tmem_ld_32x32b_x32_sync(t_o + 32 * c, ro);
        if (n < p.Nq) {
          if (p.o_d == 1 && p.Dv == D && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t w[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(ro[8 * i + 2 * k]) * out_scale,
                                                                __uint_as_float(ro[8 * i + 2 * k + 1]) * out_scale);
                w[k] = *reinterpret_cast<const uint32_t *>(&h2);
              }
              reinterpret_cast<uint4 *>(dst + 32 * c)[i] = make_uint4(w[0], w[1], w[2], w[3]);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (32 * c + i < p.Dv) dst[(int64_t)(32 * c + i) * p.o_d] = __float2bfloat16_rn(__uint_as_float(ro[i]) * out_scale);
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
  if (!(sm_scale >= 0.0f)) return fail(AC4K_ERR_UNSUPPORTED, "sm_scale must be >= 0 (the row maximum is taken before scaling)");
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
  const int64_t kv_tiles = ceil_div(Nkv, 64);
  CUtensorMap tq, tk, tv;
  // Q, K: [B*H*N, 64 bytes] (head dimension padded to 128 by the quantiser); V^T: [B*H*Dv, align64(Nkv)/2 bytes]
  if (int e = get_tmap64(Q, B * H * Nq, 64, mha::BQ, &tq)) return e;
  if (int e = get_tmap64(K, B * H * Nkv, 64, mha::BKV, &tk)) return e;
  if (int e = get_tmap32(V, B * H * Dv, kv_tiles * 32, 128, &tv)) return e;
  MhaArgs a = {};
  a.sfq = static_cast<const uint8_t *>(Q_sf);
  a.sfk = static_cast<const uint8_t *>(K_sf);
  a.sfv = static_cast<const uint8_t *>(V_sf);
  a.q_gs = Q_gs; a.k_gs = K_gs; a.v_gs = V_gs;
  a.O = O;
  a.o_b = o_stride[0]; a.o_h = o_stride[1]; a.o_n = o_stride[2]; a.o_d = o_stride[3];
  a.B = (int)B; a.H = (int)H; a.Nq = (int)Nq; a.Nkv = (int)Nkv; a.Dv = (int)Dv;
  a.q_blocks = (int)ceil_div(Nq, 128);
  a.k_blocks = (int)ceil_div(Nkv, 128);
  a.kv_tiles = (int)kv_tiles;
  a.sm_scale = sm_scale;
  a.status = status;
  a.wait_ns = kWaitTimeoutNs;
  a.trace = debug_trace_ptr();
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
