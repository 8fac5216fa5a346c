// NVFP4 multi-head attention forward for sm_100a: O = softmax(sm_scale * Q K^T) V with Q, K, V and the
// probabilities P all in NVFP4 (e2m1 values, one e4m3 scale per 16 elements of the contraction dimension, an
// fp32 global scale per tensor).  Stands in for ac4k_kernel's lib/cuda/sm120/mha_nvfp4.cu:322-1077 (an mma.sync
// kernel for sm_120a) behind the same binding (lib/cuda_bindings.cc:49-56, include/ac4k_kernel/ops.h:13-17);
// the arithmetic follows that kernel: S = (gQ gK sm_scale) * Q K^T, running row maximum and row sum in fp32,
// P = exp(S - max) re-quantised per 16 keys with the fixed global scale 1 / (6 * 448)
// (mha_nvfp4.cu:246-319), O accumulated in fp32 and divided by the row sum at the end.
//
// One CTA per (batch, head, 256 query rows), one CTA per SM; the CTA holds two query tiles of 128 rows (groups A, B)
// and walks the keys in tiles of 128:
//   warp 0     TMA producer: both Q tiles once; per key tile K [128 keys x D], V^T [D x 128 keys] and their scale
//              chunks, four stages, shared by the two groups
//   warp 1     MMA issuer: S = Q K^T (tcgen05.mma kind::mxf4nvf4, M = 128 queries, N = 128 keys, K = D) into ONE
//              128-column score buffer in tensor memory that the groups use in turn (a group copies its scores to
//              registers at once, which frees the buffer for the other group's MMA); once a group has written P:
//              O_g (+)= P V (M = 128, N = D, K = 128 keys).  Block scales go from shared to tensor memory with
//              tcgen05.cp in front of the MMAs.
//   warps 2-5  softmax of group A, warps 6-9 of group B: thread = query row.  One pass over the 128 scores in
//              registers: running maximum, O rescaled in tensor memory when a maximum of the warp moved, ex2.approx,
//              row sum, P quantised to e2m1 + e4m3 block scales (fixed global scale 1 / 2688) and written into shared
//              memory in the layouts the tensor core reads (64-byte-swizzled K-major operand, 32 x 16-byte scale
//              chunks); at the end O * gV / (2688 * row sum) is stored as bf16.
// The softmax bounds this kernel: an SM retires 16 ex2 per clock, 1024 cycles for 128 x 128 scores against 330 for the
// four-bit MMAs.  One warp per scheduler keeps the ex2 pipe ~65 % busy, two keep it full, but two groups that run in
// step also sit together in the phases that do not use it (wait for S, copy it out, maxima, rescale, fences, barrier
// traffic: ~800 cycles per key tile).  Sharing one score buffer keeps the groups a few hundred cycles apart (group B's S
// is issued when group A has copied its own out); an explicit token that made a group wait until the other was half way
// through its exponentials helped earlier versions of this kernel and costs 3 % in this one.
// Tensor memory: S 128 + O_A 128 + O_B 128 + scales 40 columns of 512.
//
// Supported: head dimensions up to 128 (padded to 64 or 128 by the quantiser); block scales in the tiled layout
// [.., 128-row block, K/64, 32 x 16 B] or in the reference's [.., K/64, align16(rows), 4]; V quantised along the keys (cross dimension = head dimension) with the
// reference's K permutation (quantize(v, 3, N_dim, swizzle=True), python/ac4k_kernel/ops/attention.py:113-118):
// P is written in the same key order, so scale blocks of P and V cover the same 16 keys as in the reference.
#include "gemm_common.cuh"
#include "mha_common.cuh"

namespace ac4k {
using namespace ptx;

namespace mha {
static constexpr int BQ = 128, BKV = 128, D = 128;
static constexpr int kThreads = 352;              // producer, MMA issuer, 2 x 4 softmax warps, scale re-order warp
static constexpr int Q_BYTES = BQ * 64;           // 128 rows x 128 e2m1, 64-byte rows
static constexpr int K_BYTES = BKV * 64;          // 128 keys x 128 e2m1
static constexpr int V_BYTES = D * 64;            // 128 head-dimension rows x 128 keys
static constexpr int P_BYTES = BQ * 64;           // 128 query rows x 128 keys
static constexpr int SF_BYTES = 2 * 512;          // two K = 64 steps of 128 rows
static constexpr int KV_STAGES = 4;
static constexpr int STAGE_BYTES = K_BYTES + V_BYTES + 2 * SF_BYTES;       // 18 432
static constexpr int LUT_BYTES = 128 * 4;         // 2688 / e4m3 value for the 127 finite non-negative e4m3 bytes
static constexpr int SMEM_BYTES = 2 * Q_BYTES + 4 * P_BYTES + KV_STAGES * STAGE_BYTES + 2 * SF_BYTES + 4 * SF_BYTES + LUT_BYTES + 1024 + 256;
// tensor memory columns
static constexpr int S_COL = 0, O_COL = 128 /* + 128 * group */, SFQ_COL = 384 /* + 8 * group */, SFK_COL = 400, SFP_COL = 408,
                     SFV_COL = 416;
static constexpr int TMEM_COLS = 512;
static constexpr float kPGlobal = 2688.0f;        // 6 * 448: reciprocal of P's fixed global scale
static_assert(STAGE_BYTES % 1024 == 0, "tile alignment");
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory overflow");
}  // namespace mha

struct MhaArgs {
  const uint8_t *sfq, *sfk, *sfv;       // block scales: tiled layout, or the reference's [K/64, align16(rows), 4]
  const float *q_gs, *k_gs, *v_gs;
  void *O;
  int64_t o_b, o_h, o_n, o_d;           // strides of O in elements
  int B, H, Nq, Nkv, Dv;
  int q_blocks, kv_tiles;               // ceil(Nq / 128), ceil(Nkv / 128): 128-row blocks of Q and of the keys
  int v_k64;                            // align64(Nkv) / 64: K = 64 steps of V^T that exist
  int nkq;                              // align64(Dqk) / 64: K = 64 steps of the head dimension (1 or 2)
  int q_pad, k_pad, v_pad;              // align16 of Nq, Nkv, Dv: scale rows per K step in the reference's layout
  float sm_scale;
  unsigned int *status;
  unsigned long long wait_ns;
  unsigned long long *trace;            // clock stamps (builds with -DAC4K_TRACE_ENABLED), else NULL
};

// Trace builds: CTA (0, 0, 0) stamps clock64 into trace[(region * 128 + key tile) * 8 + event]; region 0 / 2 = softmax warp
// of lane quarter 0 of group A / B, region 1 = MMA issuer.
#ifdef AC4K_TRACE_ENABLED
#define AC4K_TRM(region, it, ev)                                                                     \
  do {                                                                                               \
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (it) < 128)   \
      p.trace[((size_t)(region) * 128 + (it)) * 8 + (ev)] = clock64();                               \
  } while (0)
#else
#define AC4K_TRM(region, it, ev) do { } while (0)
#endif

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

// SF_TILED: block scales arrive as 512-byte chunks that tensor memory takes as they are (bulk copies).  Otherwise they
// are in the reference's layout, one 32-bit word per row and K = 64 step, rows contiguous: warp 10 transposes each
// chunk (128 words -> 32 rows of 4 words) into shared memory with plain loads.
template <bool SF_TILED>
__global__ void __launch_bounds__(mha::kThreads, 1)
mha_nvfp4_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                     const __grid_constant__ CUtensorMap tma_v, const MhaArgs p) {
  using namespace mha;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = smem_base;                     // [group]
  const uint32_t sP = sQ + 2 * Q_BYTES;              // [group][buffer]
  const uint32_t sKV = sP + 4 * P_BYTES;             // per stage: K | V^T | SFK | SFV
  const uint32_t sSFQ = sKV + KV_STAGES * STAGE_BYTES;   // [group]
  const uint32_t sSFP = sSFQ + 2 * SF_BYTES;         // [group][buffer]
  const uint32_t sLUT = sSFP + 4 * SF_BYTES;
  const uint32_t bars = sLUT + LUT_BYTES;
  const uint32_t q_full = bars, kv_full = bars + 8, kv_empty = kv_full + 8 * KV_STAGES;
  const uint32_t s_full = kv_empty + 8 * KV_STAGES;  // [group]
  const uint32_t s_free = s_full + 16;
  const uint32_t p_full = s_free + 8;                // [group]
  const uint32_t o_done = p_full + 16;               // [group][P buffer]
  const uint32_t tmem_slot = o_done + 32;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int64_t bh = (int64_t)b * p.H + h;
  const int q_row0 = (int)(bh * p.Nq) + qt * 2 * BQ; // row of Q in the [B*H*Nq, 64-byte] matrix
  const int k_row0 = (int)(bh * p.Nkv);
  const int v_row0 = (int)(bh * p.Dv);               // V^T rows of this head; rows past Dv belong to the next head and are not stored
  const int n_tiles = p.kv_tiles;
  const bool both = 2 * qt + 1 < p.q_blocks;         // group B has query rows

  if (threadIdx.x == 0) {
    mbar_init(q_full, SF_TILED ? 1 : 2);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(kv_full + 8 * s, SF_TILED ? 1 : 2);
      mbar_init(kv_empty + 8 * s, 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(s_full + 8 * g, 1);
      mbar_init(p_full + 8 * g, 4);     // the group's four warps have written P and its scales
      mbar_init(o_done + 16 * g, 1);
      mbar_init(o_done + 16 * g + 8, 1);
    }
    mbar_init(s_free, 4);               // the four warps of the group whose turn it is hold S in registers
    fence_barrier_init();
    prefetch_tmap(&tma_q);
    prefetch_tmap(&tma_k);
    prefetch_tmap(&tma_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  if (threadIdx.x >= 64 && threadIdx.x < 192) {
    // what a block's probabilities are multiplied with, by the block's e4m3 scale byte: 2688 / scale (0 for scale 0)
    const uint32_t bte = threadIdx.x - 64;
    const __half_raw hr = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)bte, __NV_E4M3);
    const float sd = __half2float(__half(hr));
    const float sc = (bte != 0 && bte != 127) ? __fdiv_rn(kPGlobal, sd) : 0.0f;
    asm volatile("st.shared::cta.f32 [%0], %1;" ::"r"(sLUT + bte * 4), "f"(sc) : "memory");
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
    const int ng = both ? 2 : 1;
    mbar_arrive_expect_tx_if(el, q_full, ng * (Q_BYTES + (SF_TILED ? p.nkq * 512 : 0)));
    for (int g = 0; g < ng; ++g) {
      tma_load_2d_if(el, sQ + g * Q_BYTES, &tma_q, 0, q_row0 + g * BQ, q_full);
      if (SF_TILED)
        bulk_load_1d_if(el, sSFQ + g * SF_BYTES, p.sfq + ((bh * p.q_blocks + 2 * qt + g) * p.nkq) * 512, p.nkq * 512, q_full);
    }
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j % KV_STAGES;
      ok = warp_all(mbar_wait(kv_empty + 8 * s, ((j / KV_STAGES) & 1) ^ 1, p.wait_ns));
      if (!ok) break;
      const uint32_t st = sKV + s * STAGE_BYTES, fb = kv_full + 8 * s;
      // V^T: D rows x 128 keys; of the tile's two K = 64 steps only those below align64(Nkv) exist
      const int nk = min(2, p.v_k64 - 2 * j);
      mbar_arrive_expect_tx_if(el, fb, K_BYTES + V_BYTES + (SF_TILED ? (p.nkq + nk) * 512 : 0));
      tma_load_2d_if(el, st, &tma_k, 0, k_row0 + j * BKV, fb);
      tma_load_2d_if(el, st + K_BYTES, &tma_v, j * 64, v_row0, fb);
      if (SF_TILED) {
        bulk_load_1d_if(el, st + K_BYTES + V_BYTES, p.sfk + ((bh * p.kv_tiles + j) * p.nkq) * 512, p.nkq * 512, fb);
        bulk_load_1d_if(el, st + K_BYTES + V_BYTES + SF_BYTES, p.sfv + (bh * p.v_k64 + 2 * j) * 512, nk * 512, fb);
      }
    }
    if (!ok && el) atomicExch(p.status, kStatusTimeoutProducer);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t el = elect_one();
    constexpr uint32_t idesc = make_idesc_mxf4nvf4(128, 128);
    const uint32_t t_s = tmem_base + S_COL;
    bool ok = warp_all(mbar_wait(q_full, 0, p.wait_ns));
    // S of group g and key tile j into the shared score buffer: two K = 64 steps over D, 32 bytes apart inside the
    // 64-byte rows of Q and K
    auto issue_s = [&](int g, int j) {
      const uint32_t st = sKV + (j % KV_STAGES) * STAGE_BYTES;
      const uint64_t qdesc = make_smem_desc(sQ + g * Q_BYTES, 16, 512, kSwizzle64B);
      const uint64_t kdesc = make_smem_desc(st, 16, 512, kSwizzle64B);
      const uint64_t sfqdesc = make_smem_desc(sSFQ + g * SF_BYTES, 0, 128, kSwizzleNone);
      const uint64_t sfkdesc = make_smem_desc(st + K_BYTES + V_BYTES, 0, 128, kSwizzleNone);
      const uint32_t t_sfq = tmem_base + SFQ_COL + 8 * g;
      // (a head dimension of 64 or less is one K step: the rows are 32 bytes, the upper half of the 64-byte tile rows is
      // filled with zeros by TMA and never multiplied)
      for (int i = 0; i < p.nkq; ++i) {
        if (j == 0) tmem_cp_32x128b_warpx4_if(el, t_sfq + 4 * i, sfqdesc + 32 * i);
        tmem_cp_32x128b_warpx4_if(el, tmem_base + SFK_COL + 4 * i, sfkdesc + 32 * i);
      }
      for (int i = 0; i < p.nkq; ++i)
        mma_mxf4nvf4_if(el, t_s, qdesc + 2 * i, kdesc + 2 * i, idesc, t_sfq + 4 * i, tmem_base + SFK_COL + 4 * i, i > 0 ? 1u : 0u);
      tc_commit_if(el, s_full + 8 * g);
    };
    // O_g (+)= P V: two K = 64 steps over the tile's keys (one when only the first exists)
    auto issue_pv = [&](int g, int j) {
      const uint32_t st = sKV + (j % KV_STAGES) * STAGE_BYTES;
      const uint64_t pdesc = make_smem_desc(sP + (2 * g + (j & 1)) * P_BYTES, 16, 512, kSwizzle64B);
      const uint64_t vdesc = make_smem_desc(st + K_BYTES, 16, 512, kSwizzle64B);
      const uint64_t sfpdesc = make_smem_desc(sSFP + (2 * g + (j & 1)) * SF_BYTES, 0, 128, kSwizzleNone);
      const uint64_t sfvdesc = make_smem_desc(st + K_BYTES + V_BYTES + SF_BYTES, 0, 128, kSwizzleNone);
      const int nk = min(2, p.v_k64 - 2 * j);
      for (int i = 0; i < nk; ++i) {
        tmem_cp_32x128b_warpx4_if(el, tmem_base + SFP_COL + 4 * i, sfpdesc + 32 * i);
        tmem_cp_32x128b_warpx4_if(el, tmem_base + SFV_COL + 4 * i, sfvdesc + 32 * i);
      }
      for (int i = 0; i < nk; ++i)
        mma_mxf4nvf4_if(el, tmem_base + O_COL + 128 * g, pdesc + 2 * i, vdesc + 2 * i, idesc, tmem_base + SFP_COL + 4 * i,
                        tmem_base + SFV_COL + 4 * i, (j > 0 || i > 0) ? 1u : 0u);
      tc_commit_if(el, o_done + 16 * g + 8 * (j & 1));
    };
    // The score buffer is used in the order A(0), B(0), A(1), B(1), ... (A(0), A(1), ... without group B); use n of the
    // buffer may be issued when use n - 1 has been copied to registers (s_free phase n - 1).
    int n_use = 0;
    auto issue_s_when_free = [&](int g, int j) {
      bool good = true;
      if (n_use > 0) good = warp_all(mbar_wait(s_free, (n_use - 1) & 1, p.wait_ns));
      if (good) {
        tc_fence_after();
        issue_s(g, j);
        ++n_use;
      }
      return good;
    };
    auto wait_kv = [&](int j) { return warp_all(mbar_wait(kv_full + 8 * (j % KV_STAGES), (j / KV_STAGES) & 1, p.wait_ns)); };
    if (ok) ok = wait_kv(0);
    if (ok) ok = issue_s_when_free(0, 0);
    if (ok && both) ok = issue_s_when_free(1, 0);
    if (ok && n_tiles > 1) {
      ok = wait_kv(1);
      if (ok) ok = issue_s_when_free(0, 1);
    }
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (el) AC4K_TRM(1, j, 0);
      ok = warp_all(mbar_wait(p_full, j & 1, p.wait_ns));
      if (!ok) break;
      tc_fence_after();
      issue_pv(0, j);
      if (el) AC4K_TRM(1, j, 1);
      if (both) {
        if (j + 1 < n_tiles) {
          ok = issue_s_when_free(1, j + 1);
          if (!ok) break;
        }
        if (el) AC4K_TRM(1, j, 2);
        ok = warp_all(mbar_wait(p_full + 8, j & 1, p.wait_ns));
        if (!ok) break;
        tc_fence_after();
        issue_pv(1, j);
        if (el) AC4K_TRM(1, j, 3);
      }
      tc_commit_if(el, kv_empty + 8 * (j % KV_STAGES));
      if (j + 2 < n_tiles) {
        ok = wait_kv(j + 2);
        if (!ok) break;
        ok = issue_s_when_free(0, j + 2);
        if (!ok) break;
      }
      if (el) AC4K_TRM(1, j, 4);
    }
    if (!ok && el) atomicExch(p.status, kStatusTimeoutMma);
  } else if (warp == 10) {
    // ------------------------------------------------------------------ scale re-order (reference layout only)
    if (!SF_TILED) {
      // chunk of K = 64 step k and rows [row0, row0 + 128) of a [K/64, pad, 4-byte] scale array: lane l takes the words
      // of rows row0 + l, + 32, + 64, + 96 (coalesced over the lanes) and stores them as its 16-byte row of the chunk
      auto put_chunk = [&](uint32_t dst, const uint8_t *base, int k, int pad, int row0) {
        const uint32_t *src = reinterpret_cast<const uint32_t *>(base) + (int64_t)k * pad;
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = row0 + 32 * i + lane;
          w[i] = r < pad ? __ldg(src + r) : 0u;
        }
        st_shared_v4u(dst + lane * 16, w[0], w[1], w[2], w[3]);
      };
      const uint8_t *q_base = p.sfq + bh * p.nkq * (int64_t)p.q_pad * 4;
      const uint8_t *k_base = p.sfk + bh * p.nkq * (int64_t)p.k_pad * 4;
      const uint8_t *v_base = p.sfv + bh * (int64_t)p.v_k64 * p.v_pad * 4;
      for (int g = 0; g < (both ? 2 : 1); ++g)
        for (int i = 0; i < p.nkq; ++i) put_chunk(sSFQ + g * SF_BYTES + i * 512, q_base, i, p.q_pad, (2 * qt + g) * BQ);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_full);
      bool ok = true;
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % KV_STAGES;
        ok = warp_all(mbar_wait(kv_empty + 8 * s, ((j / KV_STAGES) & 1) ^ 1, p.wait_ns));
        if (!ok) break;
        const uint32_t st = sKV + s * STAGE_BYTES + K_BYTES + V_BYTES;
        const int nk = min(2, p.v_k64 - 2 * j);
        for (int i = 0; i < p.nkq; ++i) put_chunk(st + i * 512, k_base, i, p.k_pad, j * BKV);
        for (int i = 0; i < nk; ++i) put_chunk(st + SF_BYTES + i * 512, v_base, 2 * j + i, p.v_pad, 0);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(kv_full + 8 * s);
      }
      if (!ok && lane == 0) atomicExch(p.status, kStatusTimeoutSf);
    }
  } else if (warp < 6 || both) {
    // ------------------------------------------------------------------ softmax, correction, epilogue
    const int g = (warp - 2) >> 2;            // group: query tile A or B
    const int q = warp & 3;                   // tensor-memory lane quarter (warps 2-5 and 6-9 -> 2, 3, 0, 1)
    const int row_l = q * 32 + lane;          // query row inside the tile = tensor-memory lane
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t t_s = tmem_base + lane_addr + S_COL, t_o = tmem_base + lane_addr + O_COL + 128 * g;
    // scores in units of log2: p = exp2(s * c1 - m)
    // (c1 >= 0: the host rejects a negative sm_scale; the floor keeps -inf * c1 = -inf for masked keys when a global
    // scale is 0)
    const float c1 = fmaxf(__ldg(p.q_gs) * __ldg(p.k_gs) * p.sm_scale * 1.4426950408889634f, 1.17549435e-38f);
    const uint32_t p_row0 = sP + 2 * g * P_BYTES + row_l * 64;
    const uint32_t p_xor = (uint32_t)((row_l >> 1) & 3) << 4;       // 64-byte swizzle: 16-byte chunk ^ ((row / 2) % 4)
    const uint32_t sfp0 = sSFP + 2 * g * SF_BYTES + lane * 16 + q * 4;
    const uint32_t my_s_full = s_full + 8 * g, my_p_full = p_full + 8 * g, my_o_done = o_done + 16 * g;
    const bool tracer = (q == 0 && lane == 0);
    float m = -INFINITY, l = 0.0f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      if (tracer) AC4K_TRM(2 * g, j, 0);
      ok = warp_all(mbar_wait(my_s_full, j & 1, p.wait_ns));
      if (!ok) break;
      tc_fence_after();
      if (tracer) AC4K_TRM(2 * g, j, 1);
      uint32_t lo[64], hi[64];               // scores of keys 0-63 and 64-127
      tmem_ld_32x32b_x64(t_s, lo);
      tmem_ld_32x32b_x64(t_s + 64, hi);
      tmem_ld_wait();
      tmem_pin(lo);
      tmem_pin(hi);
#define AC4K_S(i) ((i) < 64 ? lo[(i) & 63] : hi[(i) & 63])
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);
      if (tracer) AC4K_TRM(2 * g, j, 2);
      const int ncols = p.Nkv - j * BKV;                 // keys of this tile that exist (>= 128 except in the last tile)
      if (ncols < BKV) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          if (i >= ncols) lo[i] = 0xff800000u;           // -inf: out of the maximum, probability 0
          if (64 + i >= ncols) hi[i] = 0xff800000u;
        }
      }
      // Maxima of the scores per block of 16 in the stored key order (the reference's V quantiser's "swizzle": every 32
      // keys viewed as [4, 4, 2] and transposed to [4(b), 4(a), 2]; positions n, n + 1 hold keys key0(n), key0(n) + 1),
      // and the row maximum from them.  ex2 is monotonic, so a block's largest probability is ex2 of its largest score:
      // it is known before the block's probabilities are, and their conversion does not have to wait for all of them.
      float bs[8];
#pragma unroll
      for (int bk = 0; bk < 8; ++bk) {
        float v[16];
#pragma unroll
        for (int n = 0; n < 16; n += 2) {
          const int nn = 16 * (bk & 1) + n;
          const int i = 32 * (bk >> 1) + (((nn >> 1) & 3) * 4 + (nn >> 3)) * 2;
          v[n] = __uint_as_float(AC4K_S(i));
          v[n + 1] = __uint_as_float(AC4K_S(i + 1));
        }
        const float t0 = max3(v[0], v[1], v[2]), t1 = max3(v[3], v[4], v[5]), t2 = max3(v[6], v[7], v[8]);
        const float t3 = max3(v[9], v[10], v[11]), t4 = max3(v[12], v[13], v[14]);
        bs[bk] = fmaxf(max3(t0, t1, t2), max3(t3, t4, v[15]));
      }
      const float m_new = fmaxf(m, fmaxf(max3(bs[0], bs[1], bs[2]), max3(bs[3], bs[4], max3(bs[5], bs[6], bs[7]))) * c1);
      if (j > 0 && __any_sync(0xffffffffu, m_new != m)) {
        // a maximum of this warp's rows moved: O is rescaled, once the previous tile's P V is complete
        ok = warp_all(mbar_wait(my_o_done + 8 * ((j - 1) & 1), ((j - 1) >> 1) & 1, p.wait_ns));
        if (!ok) break;
        tc_fence_after();
        const float a = ex2_approx(m - m_new);
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t ro[16];
          tmem_ld_32x32b_x16(t_o + 16 * c, ro);
          tmem_ld_wait();
          tmem_pin(ro);
#pragma unroll
          for (int i = 0; i < 16; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * a);
          tmem_st_32x32b_x16(t_o + 16 * c, ro);
        }
        tmem_st_wait();
        l *= a;
      }
      m = m_new;
      if (tracer) AC4K_TRM(2 * g, j, 3);
      if (tracer) AC4K_TRM(2 * g, j, 4);
      // This tile's P buffer was last read by the P V of two tiles ago.  That MMA was issued before this tile's S, and
      // the tensor pipe completes MMAs (and the commits behind them) in issue order: s_full of this tile, seen above,
      // implies it is complete, so no wait is needed here.
      // Probabilities, row sum, NVFP4 quantisation of P in eight blocks of 16 keys.  P is stored in the key order of the
      // reference's V quantiser ("swizzle": every 32 keys viewed as [4, 4, 2] and transposed to [4(b), 4(a), 2]; positions
      // n, n + 1 hold keys key0(n), key0(n) + 1), so that position n of P meets position n of V^T.
      const uint32_t p_row = p_row0 + (j & 1) * P_BYTES;
      float2 lsum[4];
      const float2 c1_2 = make_float2(c1, c1), negm2 = make_float2(-m, -m);
      uint32_t sfw[2] = {0u, 0u};
#pragma unroll
      for (int gg = 0; gg < 4; ++gg) {
        float2 pr[16];
        lsum[gg] = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int n = 0; n < 32; n += 2) {
          const int i = 32 * gg + (((n >> 1) & 3) * 4 + (n >> 3)) * 2;     // keys held at positions n, n + 1
          const float2 e = ffma2(make_float2(__uint_as_float(AC4K_S(i)), __uint_as_float(AC4K_S(i + 1))), c1_2, negm2);
          // every fourth pair on the FMA pipe, the others on the ex2 pipe (every second pair measured 7 % slower)
          pr[n >> 1] = ((n >> 1) & 3) == 1 ? exp2_fma_pipe(e) : make_float2(ex2_approx(e.x), ex2_approx(e.y));
          lsum[gg] = fadd2(lsum[gg], pr[n >> 1]);
        }
        float bm[2];
        bm[0] = ex2_approx(fmaf(bs[2 * gg], c1, -m));
        bm[1] = ex2_approx(fmaf(bs[2 * gg + 1], c1, -m));
        uint16_t sb2;
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(sb2) : "f"(__fmul_rn(kPGlobal, __fmul_rn(bm[1], kOneSixth))),
            "f"(__fmul_rn(kPGlobal, __fmul_rn(bm[0], kOneSixth))));
        sfw[gg >> 1] |= (uint32_t)sb2 << (16 * (gg & 1));
        float sc0, sc1;
        // (the table is written once before the first barrier: these loads may be scheduled freely)
        asm("ld.shared::cta.f32 %0, [%1];" : "=f"(sc0) : "r"(sLUT + ((uint32_t)sb2 & 0xffu) * 4));
        asm("ld.shared::cta.f32 %0, [%1];" : "=f"(sc1) : "r"(sLUT + ((uint32_t)sb2 >> 8) * 4));
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
        st_shared_v4u(p_row + (((uint32_t)gg << 4) ^ p_xor), codes[0], codes[1], codes[2], codes[3]);
      }
#undef AC4K_S
      l += (lsum[0].x + lsum[0].y) + (lsum[1].x + lsum[1].y) + ((lsum[2].x + lsum[2].y) + (lsum[3].x + lsum[3].y));
      if (tracer) AC4K_TRM(2 * g, j, 5);
      // scale chunks of the two K = 64 steps: 32 rows of 16 bytes, row `lane` holding the words of query rows lane,
      // 32 + lane, 64 + lane, 96 + lane
      st_shared_u32(sfp0 + (j & 1) * SF_BYTES, sfw[0]);
      st_shared_u32(sfp0 + (j & 1) * SF_BYTES + 512, sfw[1]);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(my_p_full);
      if (tracer) AC4K_TRM(2 * g, j, 6);
    }
    if (ok) ok = warp_all(mbar_wait(my_o_done + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, p.wait_ns));
    if (!ok) {
      if (lane == 0) atomicExch(p.status, kStatusTimeoutEpilogue);
    } else {
      tc_fence_after();
      const int n = (2 * qt + g) * BQ + row_l;
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
  if (Dqk <= 0 || Dqk > 128 || Dv <= 0 || Dv > 128)
    return fail(AC4K_ERR_UNSUPPORTED, "head dimensions up to 128 are built (Dqk = %lld, Dv = %lld)", (long long)Dqk, (long long)Dv);
  if (sf_layout != AC4K_SF_TILE128X4 && sf_layout != AC4K_SF_AC4K) return fail(AC4K_ERR_ENUM, "unknown scale layout %d", sf_layout);
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
  // Q, K: [B*H*N, 32 or 64 bytes] (head dimension padded to 64 or 128 by the quantiser); V^T: [B*H*Dv, align64(Nkv)/2 bytes]
  const int64_t nkq = ceil_div(Dqk, 64);
  if (int e = get_tmap64(Q, B * H * Nq, nkq * 32, mha::BQ, &tq)) return e;
  if (int e = get_tmap64(K, B * H * Nkv, nkq * 32, mha::BKV, &tk)) return e;
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
  a.kv_tiles = (int)ceil_div(Nkv, 128);
  a.v_k64 = (int)v_k64;
  a.nkq = (int)nkq;
  a.q_pad = (int)align_up(Nq, 16);
  a.k_pad = (int)align_up(Nkv, 16);
  a.v_pad = (int)align_up(Dv, 16);
  a.sm_scale = sm_scale;
  a.status = status;
  a.wait_ns = kWaitTimeoutNs;
  a.trace = debug_trace_ptr();
  const bool tiled = sf_layout == AC4K_SF_TILE128X4;
  static PerDevice<int> attr_set;
  int unused = 0;
  if (int e = attr_set.get(&unused, [&](int &v) {
        AC4K_CUDA_TRY(cudaFuncSetAttribute(mha_nvfp4_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, mha::SMEM_BYTES));
        AC4K_CUDA_TRY(cudaFuncSetAttribute(mha_nvfp4_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, mha::SMEM_BYTES));
        v = 1;
        return 0;
      }))
    return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((a.q_blocks + 1) / 2), (unsigned)H, (unsigned)B);
  cfg.blockDim = dim3(mha::kThreads);
  cfg.dynamicSmemBytes = mha::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (tiled)
    AC4K_CUDA_TRY(cudaLaunchKernelEx(&cfg, mha_nvfp4_fwd_kernel<true>, tq, tk, tv, a));
  else
    AC4K_CUDA_TRY(cudaLaunchKernelEx(&cfg, mha_nvfp4_fwd_kernel<false>, tq, tk, tv, a));
  return 0;
}
