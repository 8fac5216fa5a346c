// INT8 x FP8 multi-head attention forward for sm_100a: O = softmax(sm_scale * Q K^T) V with Q, K in INT8 (one fp32 scale
// per block of tokens), P and V in FP8 e4m3 (V with one fp32 scale per head-dimension channel).  Stands in for
// ac4k_kernel's lib/cuda/sm120/mha_int8_x_fp8.cu:403-975 (an mma.sync kernel for sm_120a) behind the same binding
// (lib/cuda_bindings.cc:57-58, include/ac4k_kernel/ops.h:19-25; checks :979-1060).  The arithmetic follows that kernel:
//   S = int32(Q K^T) * (sm_scale * log2 e * q_scale[block of the row] * k_scale[block of the key tile]),
//   running maximum m = max(m, rowmax(S) - 7.5)  (the offset lets P use e4m3's range: P <= 2^7.5, mha_int8_x_fp8.cu:119-121,711),
//   P = exp2(S - m) rounded to e4m3, row sum of the unrounded P in fp32, O = O * exp2(m_old - m) + P V,
//   out = O * v_scale[channel] / row sum.
// One difference: the reference accumulates the P V of one key tile in fp16 (its MMA's accumulator) before adding it
// to the fp32 O; tcgen05's kind::f8f6f4 accumulates in fp32 throughout.
//
// Structure as in mha_nvfp4.cu: one CTA per (batch, head, 256 query rows) with two groups of four softmax warps (one
// 128-row query tile each), one 128-column score buffer in tensor memory used by the groups in turn, key tiles of 128,
// S by four tcgen05.mma kind::i8 (M 128, N 128, K 32) into int32 columns, P V by four kind::f8f6f4 from the P tile the
// group wrote to shared memory (128-byte-swizzled K-major, in the key order of the reference's V quantiser: every 16
// keys viewed as [2, 4, 2] and transposed to [4, 2, 2]).  The exponentials bound the kernel (16 ex2 per clock per SM);
// a quarter of the exponentials run as a polynomial on the FMA pipe.  Because of the 7.5 offset a row's maximum rarely moves after the first tiles, so O is rarely rescaled.
//
// Supported: head dimensions up to 128 for Q/K (rows padded to a multiple of 16 bytes by the quantiser) and up to 128
// for V; Q and K quantised in blocks of 16, 32, 64 or 128 tokens (the reference's defaults: 64 and 128).
#include "gemm_common.cuh"
#include "mha_common.cuh"

namespace ac4k {
using namespace ptx;

namespace mha8 {
static constexpr int BQ = 128, BKV = 128, D = 128;
static constexpr int kThreads = 320;              // producer, MMA issuer, 2 x 4 softmax warps
static constexpr int TILE_BYTES = 128 * 128;      // 128 rows of 128 bytes (Q, K, V^T and P tiles alike)
static constexpr int KV_STAGES = 3;
static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
static constexpr int SMEM_BYTES = 2 * TILE_BYTES + 4 * TILE_BYTES + KV_STAGES * STAGE_BYTES + 1024 + 256;
static constexpr int S_COL = 0, O_COL = 128 /* + 128 * group */;
static constexpr int TMEM_COLS = 512;
static constexpr float kExpOffset = 7.5f;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory overflow");
}  // namespace mha8

struct Mha8Args {
  const float *q_sf, *k_sf, *v_sf;      // [B, H, ceil(Nq / q_block)], [B, H, ceil(Nkv / k_block)], [B, H, align16(Dv)]
  void *O;
  int64_t o_b, o_h, o_n, o_d;           // strides of O in elements
  int B, H, Nq, Nkv, Dv;
  int q_blocks, kv_tiles;               // ceil(Nq / 128), ceil(Nkv / 128)
  int q_block, q_nblk, v_pad;           // tokens per Q scale, Q scales per head, align16(Dv)
  int k_shift, k_nblk;                  // log2 of the tokens per K scale (4 .. 7), K scales per head
  float sm_scale_log2;                  // sm_scale * log2(e)
  unsigned int *status;
  unsigned long long wait_ns;
};

// Instruction descriptors of the 8-bit kinds: accumulator format in [4,6) (1 = f32, 2 = s32), A and B formats in [7,10)
// and [10,13) (kind::i8: 1 = signed; kind::f8f6f4: 0 = e4m3), both K-major, N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t make_idesc_i8(int m, int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__host__ __device__ constexpr uint32_t make_idesc_e4m3(int m, int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void mma_i8_if(uint32_t pred, uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.b32 p, %4, 0;\nsetp.ne.b32 q, %5, 0;\n"
      "@q tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(pred)
      : "memory");
}
__device__ __forceinline__ void mma_f8_if(uint32_t pred, uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.b32 p, %4, 0;\nsetp.ne.b32 q, %5, 0;\n"
      "@q tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(pred)
      : "memory");
}
// four fp32 -> four e4m3 bytes, a in the lowest
__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  uint32_t r;
  asm("{\n.reg .b16 lo, hi;\ncvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\ncvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\nmov.b32 %0, {lo, hi};\n}"
      : "=r"(r) : "f"(a), "f"(b), "f"(c), "f"(d));
  return r;
}

// K128: K is quantised in blocks of 128 tokens (the reference's default): one scale per key tile instead of one per 16 keys.
template <bool K128>
__global__ void __launch_bounds__(mha8::kThreads, 1)
mha_int8_fp8_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                        const __grid_constant__ CUtensorMap tma_v, const Mha8Args p) {
  using namespace mha8;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = smem_base;                     // [group]
  const uint32_t sP = sQ + 2 * TILE_BYTES;           // [group][buffer]
  const uint32_t sKV = sP + 4 * TILE_BYTES;          // per stage: K | V^T
  const uint32_t bars = sKV + KV_STAGES * STAGE_BYTES;
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
  const int q_row0 = (int)(bh * p.Nq) + qt * 2 * BQ; // row of Q in the [B*H*Nq, row bytes] matrix
  const int k_row0 = (int)(bh * p.Nkv);
  const int v_row0 = (int)(bh * p.Dv);               // V^T rows of this head; rows past Dv belong to the next head and are not stored
  const int n_tiles = p.kv_tiles;
  const bool both = 2 * qt + 1 < p.q_blocks;         // group B has query rows

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(kv_full + 8 * s, 1);
      mbar_init(kv_empty + 8 * s, 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(s_full + 8 * g, 1);
      mbar_init(p_full + 8 * g, 4);     // the group's four warps have written P
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
    mbar_arrive_expect_tx_if(el, q_full, ng * TILE_BYTES);
    for (int g = 0; g < ng; ++g) tma_load_2d_if(el, sQ + g * TILE_BYTES, &tma_q, 0, q_row0 + g * BQ, q_full);
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j % KV_STAGES;
      ok = warp_all(mbar_wait(kv_empty + 8 * s, ((j / KV_STAGES) & 1) ^ 1, p.wait_ns));
      if (!ok) break;
      const uint32_t st = sKV + s * STAGE_BYTES, fb = kv_full + 8 * s;
      mbar_arrive_expect_tx_if(el, fb, STAGE_BYTES);
      tma_load_2d_if(el, st, &tma_k, 0, k_row0 + j * BKV, fb);
      tma_load_2d_if(el, st + TILE_BYTES, &tma_v, j * BKV, v_row0, fb);    // keys past the row's end read as 0
    }
    if (!ok && el) atomicExch(p.status, kStatusTimeoutProducer);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t el = elect_one();
    constexpr uint32_t idesc_s = make_idesc_i8(128, 128);
    constexpr uint32_t idesc_o = make_idesc_e4m3(128, 128);
    const uint32_t t_s = tmem_base + S_COL;
    bool ok = warp_all(mbar_wait(q_full, 0, p.wait_ns));
    // S of group g and key tile j into the shared score buffer: four K = 32 steps over D, 32 bytes apart inside the
    // 128-byte rows of Q and K
    auto issue_s = [&](int g, int j) {
      const uint32_t st = sKV + (j % KV_STAGES) * STAGE_BYTES;
      const uint64_t qdesc = make_smem_desc(sQ + g * TILE_BYTES, 16, 1024, kSwizzle128B);
      const uint64_t kdesc = make_smem_desc(st, 16, 1024, kSwizzle128B);
#pragma unroll
      for (int i = 0; i < 4; ++i) mma_i8_if(el, t_s, qdesc + 2 * i, kdesc + 2 * i, idesc_s, i > 0 ? 1u : 0u);
      tc_commit_if(el, s_full + 8 * g);
    };
    // O_g (+)= P V: four K = 32 steps over the tile's keys
    auto issue_pv = [&](int g, int j) {
      const uint32_t st = sKV + (j % KV_STAGES) * STAGE_BYTES;
      const uint64_t pdesc = make_smem_desc(sP + (2 * g + (j & 1)) * TILE_BYTES, 16, 1024, kSwizzle128B);
      const uint64_t vdesc = make_smem_desc(st + TILE_BYTES, 16, 1024, kSwizzle128B);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        mma_f8_if(el, tmem_base + O_COL + 128 * g, pdesc + 2 * i, vdesc + 2 * i, idesc_o, (j > 0 || i > 0) ? 1u : 0u);
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
      ok = warp_all(mbar_wait(p_full, j & 1, p.wait_ns));
      if (!ok) break;
      tc_fence_after();
      issue_pv(0, j);
      if (both) {
        if (j + 1 < n_tiles) {
          ok = issue_s_when_free(1, j + 1);
          if (!ok) break;
        }
        ok = warp_all(mbar_wait(p_full + 8, j & 1, p.wait_ns));
        if (!ok) break;
        tc_fence_after();
        issue_pv(1, j);
      }
      tc_commit_if(el, kv_empty + 8 * (j % KV_STAGES));
      if (j + 2 < n_tiles) {
        ok = wait_kv(j + 2);
        if (!ok) break;
        ok = issue_s_when_free(0, j + 2);
        if (!ok) break;
      }
    }
    if (!ok && el) atomicExch(p.status, kStatusTimeoutMma);
  } else if (warp < 6 || both) {
    // ------------------------------------------------------------------ softmax, correction, epilogue
    const int g = (warp - 2) >> 2;            // group: query tile A or B
    const int q = warp & 3;                   // tensor-memory lane quarter (warps 2-5 and 6-9 -> 2, 3, 0, 1)
    const int row_l = q * 32 + lane;          // query row inside the tile = tensor-memory lane
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t t_s = tmem_base + lane_addr + S_COL, t_o = tmem_base + lane_addr + O_COL + 128 * g;
    const int n_row = (2 * qt + g) * BQ + row_l;                 // query row in the head
    // scores in units of log2: s = int32 * c_row * k_scale[tile]
    const float c_row = p.sm_scale_log2 * __ldg(p.q_sf + bh * p.q_nblk + min(n_row / p.q_block, p.q_nblk - 1));
    const float *k_sf = p.k_sf + bh * p.k_nblk;
    const uint32_t p_row0 = sP + 2 * g * TILE_BYTES + row_l * 128;
    const uint32_t p_xor = (uint32_t)(row_l & 7) << 4;           // 128-byte swizzle: 16-byte chunk ^ (row % 8)
    const uint32_t my_s_full = s_full + 8 * g, my_p_full = p_full + 8 * g, my_o_done = o_done + 16 * g;
    float m = -INFINITY, l = 0.0f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      ok = warp_all(mbar_wait(my_s_full, j & 1, p.wait_ns));
      if (!ok) break;
      tc_fence_after();
      uint32_t lo[64], hi[64];               // scores of keys 0-63 and 64-127 (int32)
      tmem_ld_32x32b_x64(t_s, lo);
      tmem_ld_32x32b_x64(t_s + 64, hi);
      tmem_ld_wait();
      tmem_pin(lo);
      tmem_pin(hi);
#define AC4K_S(i) ((i) < 64 ? lo[(i) & 63] : hi[(i) & 63])
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);
      // to fp32 in place (|S| <= 127 * 127 * 128 < 2^24: exact)
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        lo[i] = __float_as_uint(__int2float_rn((int)lo[i]));
        hi[i] = __float_as_uint(__int2float_rn((int)hi[i]));
      }
      const int ncols = p.Nkv - j * BKV;                 // keys of this tile that exist (>= 128 except in the last tile)
      if (ncols < BKV) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          if (i >= ncols) lo[i] = 0xff800000u;           // -inf: out of the maximum, probability 0
          if (64 + i >= ncols) hi[i] = 0xff800000u;
        }
      }
      // Scale of every 16 keys of the tile (K is quantised in blocks of 16 to 128 tokens: one to eight scales per tile).
      // c >= 0 (scales and sm_scale are; the host rejects a negative sm_scale); the floor keeps -inf * c = -inf.
      float c16[8];
      if (K128) {
        const float c = fmaxf(c_row * __ldg(k_sf + j), 1.17549435e-38f);
#pragma unroll
        for (int bk = 0; bk < 8; ++bk) c16[bk] = c;
      } else {
#pragma unroll
        for (int bk = 0; bk < 8; ++bk)
          c16[bk] = fmaxf(c_row * __ldg(k_sf + min((j * BKV + 16 * bk) >> p.k_shift, p.k_nblk - 1)), 1.17549435e-38f);
      }
      float bs[8];
#pragma unroll
      for (int bk = 0; bk < 8; ++bk) {
        float v[16];
#pragma unroll
        for (int n = 0; n < 16; ++n) v[n] = __uint_as_float(AC4K_S(16 * bk + n));
        const float t0 = max3(v[0], v[1], v[2]), t1 = max3(v[3], v[4], v[5]), t2 = max3(v[6], v[7], v[8]);
        const float t3 = max3(v[9], v[10], v[11]), t4 = max3(v[12], v[13], v[14]);
        bs[bk] = fmaxf(max3(t0, t1, t2), max3(t3, t4, v[15]));
        if (!K128) bs[bk] *= c16[bk];
      }
      float rowmax = fmaxf(max3(bs[0], bs[1], bs[2]), max3(bs[3], bs[4], max3(bs[5], bs[6], bs[7])));
      if (K128) rowmax *= c16[0];
      const float m_new = fmaxf(m, rowmax - kExpOffset);
      if (j > 0 && __any_sync(0xffffffffu, m_new != m)) {
        // a maximum of this warp's rows moved: O is rescaled, once the previous tile's P V is complete
        ok = warp_all(mbar_wait(my_o_done + 8 * ((j - 1) & 1), ((j - 1) >> 1) & 1, p.wait_ns));
        if (!ok) break;
        tc_fence_after();
        const float a = ex2_approx(m - m_new);
#pragma unroll 1
        for (int cc = 0; cc < 8; ++cc) {
          uint32_t ro[16];
          tmem_ld_32x32b_x16(t_o + 16 * cc, ro);
          tmem_ld_wait();
          tmem_pin(ro);
#pragma unroll
          for (int i = 0; i < 16; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * a);
          tmem_st_32x32b_x16(t_o + 16 * cc, ro);
        }
        tmem_st_wait();
        l *= a;
      }
      m = m_new;
      // This tile's P buffer was last read by the P V of two tiles ago, which was issued before this tile's S: s_full
      // of this tile implies that it is complete (the tensor pipe completes MMAs and commits in issue order).
      // Probabilities, row sum, P to e4m3 in the key order of the reference's V quantiser: position n of every 16 keys
      // holds key ((n / 2) % 2 * 4 + n / 4) * 2 + n % 2.
      const uint32_t p_row = p_row0 + (j & 1) * TILE_BYTES;
      float2 lsum[4];
      const float2 negm2 = make_float2(-m, -m);
#pragma unroll
      for (int gg = 0; gg < 4; ++gg) {          // 32 keys = two 16-byte chunks of P
        float2 pr[16];
        lsum[gg] = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int n = 0; n < 32; n += 2) {
          const int n16 = n & 15;
          const int i = 32 * gg + (n & 16) + (((n16 >> 1) & 1) * 4 + (n16 >> 2)) * 2;     // keys held at positions n, n + 1
          const float cc = c16[2 * gg + (n >> 4)];
          const float2 e = ffma2(make_float2(__uint_as_float(AC4K_S(i)), __uint_as_float(AC4K_S(i + 1))), make_float2(cc, cc), negm2);
          // every fourth pair on the FMA pipe, the others on the ex2 pipe
          pr[n >> 1] = ((n >> 1) & 3) == 1 ? exp2_fma_pipe(e) : make_float2(ex2_approx(e.x), ex2_approx(e.y));
          lsum[gg] = fadd2(lsum[gg], pr[n >> 1]);
        }
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          const float2 *q8 = pr + 8 * ch;
          st_shared_v4u(p_row + (((uint32_t)(2 * gg + ch) << 4) ^ p_xor), e4m3x4(q8[0].x, q8[0].y, q8[1].x, q8[1].y),
                        e4m3x4(q8[2].x, q8[2].y, q8[3].x, q8[3].y), e4m3x4(q8[4].x, q8[4].y, q8[5].x, q8[5].y),
                        e4m3x4(q8[6].x, q8[6].y, q8[7].x, q8[7].y));
        }
      }
#undef AC4K_S
      l += (lsum[0].x + lsum[0].y) + (lsum[1].x + lsum[1].y) + ((lsum[2].x + lsum[2].y) + (lsum[3].x + lsum[3].y));
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(my_p_full);
    }
    if (ok) ok = warp_all(mbar_wait(my_o_done + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, p.wait_ns));
    if (!ok) {
      if (lane == 0) atomicExch(p.status, kStatusTimeoutEpilogue);
    } else {
      tc_fence_after();
      const float inv_l = 1.0f / l;
      const float *v_sf = p.v_sf + bh * p.v_pad;
      __nv_bfloat16 *dst = static_cast<__nv_bfloat16 *>(p.O) + (int64_t)b * p.o_b + (int64_t)h * p.o_h + (int64_t)n_row * p.o_n;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t ro[32];
        tmem_ld_32x32b_x32_sync(t_o + 32 * cc, ro);
        if (n_row < p.Nq) {
          float o[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 32 * cc + i < p.Dv ? __uint_as_float(ro[i]) * (inv_l * __ldg(v_sf + 32 * cc + i)) : 0.0f;
          if (p.o_d == 1 && p.Dv == D && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t w[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const __nv_bfloat162 h2 = __floats2bfloat162_rn(o[8 * i + 2 * k], o[8 * i + 2 * k + 1]);
                w[k] = *reinterpret_cast<const uint32_t *>(&h2);
              }
              reinterpret_cast<uint4 *>(dst + 32 * cc)[i] = make_uint4(w[0], w[1], w[2], w[3]);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (32 * cc + i < p.Dv) dst[(int64_t)(32 * cc + i) * p.o_d] = __float2bfloat16_rn(o[i]);
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

extern "C" int ac4k_mha_int8_x_fp8_fwd(void *O, const int64_t o_stride[4], const void *Q, const float *Q_sf, int64_t q_block,
                                       const void *K, const float *K_sf, int64_t k_block, const void *V, const float *V_sf,
                                       int64_t B, int64_t H, int64_t Nq, int64_t Nkv, int64_t Dqk, int64_t Dv, float sm_scale,
                                       ac4k_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!O || !o_stride || !Q || !Q_sf || !K || !K_sf || !V || !V_sf) return fail(AC4K_ERR_NULL, "a required pointer is NULL");
  if (B < 0 || H < 0 || Nq < 0 || Nkv < 0) return fail(AC4K_ERR_SHAPE, "negative dimension");
  if (B == 0 || H == 0 || Nq == 0) return 0;
  if (Nkv == 0) return fail(AC4K_ERR_SHAPE, "attention over zero keys");
  if (!(sm_scale >= 0.0f)) return fail(AC4K_ERR_UNSUPPORTED, "sm_scale must be >= 0 (the row maximum is taken before scaling)");
  if (Dqk <= 0 || Dqk > 128 || Dv <= 0 || Dv > 128)
    return fail(AC4K_ERR_UNSUPPORTED, "head dimensions up to 128 are built (Dqk = %lld, Dv = %lld)", (long long)Dqk, (long long)Dv);
  if (k_block < 16 || k_block > 128 || (k_block & (k_block - 1)) || q_block < 16 || q_block > 128 || (q_block & (q_block - 1)))
    return fail(AC4K_ERR_UNSUPPORTED, "Q and K must be quantised in blocks of 16, 32, 64 or 128 tokens, got %lld and %lld", (long long)q_block,
                (long long)k_block);
  if (B > 65535 || H > 65535 || B * H * Nq > (1ll << 31) - 256 || B * H * Nkv > (1ll << 31) - 256) return fail(AC4K_ERR_SHAPE, "dimension too large");
  for (const void *ptr : {Q, K, V})
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return fail(AC4K_ERR_ALIGN, "Q, K and V must be 16-byte aligned");
  DeviceInfo di;
  if (int e = get_device_info(&di)) return e;
  if (di.cc_major != 10) return fail(AC4K_ERR_DEVICE, "mha_int8_x_fp8_fwd needs an sm_100 device (found sm_%d0)", di.cc_major);
  unsigned int *status = device_status_ptr();
  if (!status) return fail(AC4K_ERR_DEVICE, "cannot resolve the device status word");
  CUtensorMap tq, tk, tv;
  // Q, K: [B*H*N, align16(Dqk) bytes]; V^T: [B*H*Dv, align16(Nkv) bytes] (the FP8 quantiser pads the keys to 16)
  const int64_t dp = align_up(Dqk, 16), kp = align_up(Nkv, 16);
  if (int e = get_tmap(Q, B * H * Nq, dp, mha8::BQ, &tq)) return e;
  if (int e = get_tmap(K, B * H * Nkv, dp, mha8::BKV, &tk)) return e;
  if (int e = get_tmap(V, B * H * Dv, kp, 128, &tv)) return e;
  Mha8Args a = {};
  a.q_sf = Q_sf; a.k_sf = K_sf; a.v_sf = V_sf;
  a.O = O;
  a.o_b = o_stride[0]; a.o_h = o_stride[1]; a.o_n = o_stride[2]; a.o_d = o_stride[3];
  a.B = (int)B; a.H = (int)H; a.Nq = (int)Nq; a.Nkv = (int)Nkv; a.Dv = (int)Dv;
  a.q_blocks = (int)ceil_div(Nq, 128);
  a.kv_tiles = (int)ceil_div(Nkv, 128);
  a.q_block = (int)q_block;
  a.q_nblk = (int)ceil_div(Nq, q_block);
  a.v_pad = (int)align_up(Dv, 16);
  a.k_shift = k_block == 16 ? 4 : (k_block == 32 ? 5 : (k_block == 64 ? 6 : 7));
  a.k_nblk = (int)ceil_div(Nkv, k_block);
  a.sm_scale_log2 = sm_scale * 1.4426950408889634f;
  a.status = status;
  a.wait_ns = kWaitTimeoutNs;
  static PerDevice<int> attr_set;
  int unused = 0;
  if (int e = attr_set.get(&unused, [&](int &v) {
        AC4K_CUDA_TRY(cudaFuncSetAttribute(mha_int8_fp8_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, mha8::SMEM_BYTES));
        AC4K_CUDA_TRY(cudaFuncSetAttribute(mha_int8_fp8_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, mha8::SMEM_BYTES));
        v = 1;
        return 0;
      }))
    return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((a.q_blocks + 1) / 2), (unsigned)H, (unsigned)B);
  cfg.blockDim = dim3(mha8::kThreads);
  cfg.dynamicSmemBytes = mha8::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (k_block == 128)
    AC4K_CUDA_TRY(cudaLaunchKernelEx(&cfg, mha_int8_fp8_fwd_kernel<true>, tq, tk, tv, a));
  else
    AC4K_CUDA_TRY(cudaLaunchKernelEx(&cfg, mha_int8_fp8_fwd_kernel<false>, tq, tk, tv, a));
  return 0;
}
