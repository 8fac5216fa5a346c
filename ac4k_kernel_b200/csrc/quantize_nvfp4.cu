// BF16 -> NVFP4 quantiser and the global-scale (amax) reduction for sm_100a.
//
// Semantics follow ac4k_kernel's lib/cuda/sm120/quantize_nvfp4.cu:49-157 (block of 16,
// pair of scales packed four to a word, K padded to 64, scale rows padded to 16) with its
// approximate reciprocals replaced by correctly rounded fp32 operations:
//     alpha = 1 / g ;  sf = e4m3(alpha * (amax16 * fp32(1/6))) ;
//     r = sf ? alpha * (1 / float(sf)) : 0 ;  code = e2m1(float(x) * r)
// Three kernels: a tiled one for rows that are contiguous along K (the linear path), a transposing one
// for rows that are contiguous along the cross dimension (attention's V), and a strided one (any
// cross/reduce strides, optional K permutation) for everything else.
#include "common.cuh"

namespace ac4k {

__device__ __forceinline__ uint32_t quantize8(const uint4 &v, float r) {
  float f[8];
  f[0] = __fmul_rn(__uint_as_float(v.x << 16), r);
  f[1] = __fmul_rn(__uint_as_float(v.x & 0xFFFF0000u), r);
  f[2] = __fmul_rn(__uint_as_float(v.y << 16), r);
  f[3] = __fmul_rn(__uint_as_float(v.y & 0xFFFF0000u), r);
  f[4] = __fmul_rn(__uint_as_float(v.z << 16), r);
  f[5] = __fmul_rn(__uint_as_float(v.z & 0xFFFF0000u), r);
  f[6] = __fmul_rn(__uint_as_float(v.w << 16), r);
  f[7] = __fmul_rn(__uint_as_float(v.w & 0xFFFF0000u), r);
  return f32x8_to_e2m1x8(f);
}

// ----------------------------------------------------------------------------------------
// Tiled kernel: one CTA = 128 rows x 256 K-elements, one thread = one 16-element block per
// pass (16 rows x 16 blocks per pass, 8 passes).  A thread loads its block with one 32-byte
// load (half a warp reads 512 contiguous bytes of a row), needs no shuffle for the block amax,
// multiplies with packed fp32x2 instructions, stores 8 bytes of codes (a warp writes two runs
// of 128 bytes) and drops its scale byte into a shared-memory image of the scale tile that is
// written out with full-width stores at the end.  The reciprocal of the e4m3 scale comes from
// a 128-entry table built once per CTA (the scale has only 127 non-negative values).
// The kernel is instruction-issue bound, not bandwidth bound, if written naively: the first
// version (one thread = 8 elements, pair shuffle, IEEE reciprocal per thread) issued ~113
// instructions per 8 elements and reached 4.7 TB/s.
// ----------------------------------------------------------------------------------------
static constexpr int kTileRows = 128;
static constexpr int kThreads = 256;
static constexpr int kBatch = 4;      // passes whose loads are issued together

struct Block16 { uint32_t w[8]; };

template <bool WIDE>
__device__ __forceinline__ Block16 load_block16(const uint16_t *p) {
  Block16 b;
  if (WIDE) {
    uint64_t a0, a1, a2, a3;
    asm volatile("ld.global.nc.L1::no_allocate.v4.b64 {%0, %1, %2, %3}, [%4];"
                 : "=l"(a0), "=l"(a1), "=l"(a2), "=l"(a3) : "l"(p));
    b.w[0] = (uint32_t)a0; b.w[1] = (uint32_t)(a0 >> 32); b.w[2] = (uint32_t)a1; b.w[3] = (uint32_t)(a1 >> 32);
    b.w[4] = (uint32_t)a2; b.w[5] = (uint32_t)(a2 >> 32); b.w[6] = (uint32_t)a3; b.w[7] = (uint32_t)(a3 >> 32);
  } else {
    const uint4 lo = __ldcs(reinterpret_cast<const uint4 *>(p)), hi = __ldcs(reinterpret_cast<const uint4 *>(p) + 1);
    b.w[0] = lo.x; b.w[1] = lo.y; b.w[2] = lo.z; b.w[3] = lo.w;
    b.w[4] = hi.x; b.w[5] = hi.y; b.w[6] = hi.z; b.w[7] = hi.w;
  }
  return b;
}

// TK: K elements of a CTA's tile, 256 or - for rows of at most 128 elements (attention's q and k: one head's
// features), where half of a 256-wide tile's threads would have nothing to load - 128.
template <int SF_LAYOUT, bool WIDE, int TK>
__global__ void __launch_bounds__(kThreads)
nvfp4_quantize_tiled_kernel(uint8_t *__restrict__ out, uint32_t *__restrict__ sf,
                            const uint16_t *__restrict__ in, const float *__restrict__ gscale,
                            int64_t M, int64_t K, int64_t d1, int64_t stride0, int64_t stride1,
                            int64_t row_stride) {
  constexpr int kTileK = TK, kTileKch = TK / 64;
  constexpr int kRowThreads = TK / 16;                  // threads (16-element blocks) per row of the tile
  constexpr int kPassRows = kThreads / kRowThreads;     // rows the CTA covers per pass
  __shared__ uint32_t s_sf[kTileKch * kTileRows];
  __shared__ float s_rcp[128];

  const int64_t Kp = align_up(K, 64);
  const int64_t KT = Kp / 64;
  const int64_t M16 = align_up(M, 16);
  const int64_t MT = ceil_div(M, 128);
  const int64_t batch = blockIdx.z;
  const int64_t r0 = (int64_t)blockIdx.y * kTileRows;
  const int64_t k0 = (int64_t)blockIdx.x * kTileK;
  const int blk = threadIdx.x % kRowThreads, prow = threadIdx.x / kRowThreads;

  if (threadIdx.x < 128) {
    // 1 / float(e4m3 byte), correctly rounded; entry 0 is 0 so that a zero scale zeroes the block
    const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)threadIdx.x, __NV_E4M3);
    const float v = __half2float(__half(h));
    s_rcp[threadIdx.x] = threadIdx.x ? __frcp_rn(v) : 0.0f;
  }
  __syncthreads();

  const float alpha = load_alpha(gscale);
  const int64_t k = k0 + blk * 16;
  const bool k_live = k < Kp;   // block belongs to the (padded) output
  const bool k_data = k < K;    // block has input data (K % 16 == 0 on this path)
  const uint16_t *in_p = in + (batch / d1) * stride0 + (batch % d1) * stride1 + (r0 + prow) * row_stride + k;
  uint8_t *out_p = out + (batch * M + r0 + prow) * (Kp / 2) + k / 2;
  uint8_t *s_bytes = reinterpret_cast<uint8_t *>(s_sf);
  const int kch = blk >> 2, sub = blk & 3;

#pragma unroll 1
  for (int p0 = 0; p0 < kTileRows / kPassRows; p0 += kBatch) {
    Block16 v[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int64_t row = r0 + (p0 + u) * kPassRows + prow;
#pragma unroll
      for (int i = 0; i < 8; ++i) v[u].w[i] = 0;
      if (row < M && k_data) v[u] = load_block16<WIDE>(in_p + (int64_t)(p0 + u) * kPassRows * row_stride);
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int row_l = (p0 + u) * kPassRows + prow;
      const bool row_ok = r0 + row_l < M;
      const Block16 &b = v[u];
      uint32_t m = max_bf16x2(max_bf16x2(max_bf16x2(abs_bf16x2(b.w[0]), abs_bf16x2(b.w[1])),
                                         max_bf16x2(abs_bf16x2(b.w[2]), abs_bf16x2(b.w[3]))),
                              max_bf16x2(max_bf16x2(abs_bf16x2(b.w[4]), abs_bf16x2(b.w[5])),
                                         max_bf16x2(abs_bf16x2(b.w[6]), abs_bf16x2(b.w[7]))));
      const float amax = hmax_bf16x2_to_f32(m);
      const float s = __fmul_rn(alpha, __fmul_rn(amax, kOneSixth));
      uint16_t pk;
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pk) : "f"(0.0f), "f"(s));
      const uint32_t sb = pk & 0x7Fu;
      const float r = __fmul_rn(alpha, s_rcp[sb]);
      if (row_ok && k_live) {
        uint2 codes;
        codes.x = quantize8_x2(b.w[0], b.w[1], b.w[2], b.w[3], r);
        codes.y = quantize8_x2(b.w[4], b.w[5], b.w[6], b.w[7], r);
        __stcs(reinterpret_cast<uint2 *>(out_p + (int64_t)(p0 + u) * kPassRows * (Kp / 2)), codes);
      }
      int off;
      if (SF_LAYOUT == AC4K_SF_AC4K)
        off = (kch * kTileRows + row_l) * 4 + sub;
      else
        off = kch * 512 + (row_l & 31) * 16 + (row_l >> 5) * 4 + sub;
      s_bytes[off] = row_ok ? (uint8_t)sb : (uint8_t)0;
    }
  }
  __syncthreads();

  // write the scale image: kTileKch groups of 128 words
  for (int t = threadIdx.x; t < kTileKch * kTileRows; t += kThreads) {
    const int c = t >> 7, w = t & 127;
    const int64_t k64 = k0 / 64 + c;
    if (k64 >= KT) continue;
    if (SF_LAYOUT == AC4K_SF_AC4K) {
      const int64_t row = r0 + w;
      if (row < M16) sf[(batch * KT + k64) * M16 + row] = s_sf[t];
    } else {
      sf[((batch * MT + blockIdx.y) * KT + k64) * 128 + w] = s_sf[t];
    }
  }
}

// ----------------------------------------------------------------------------------------
// Strided kernel: one thread = one 16-element block, scalar loads with arbitrary element
// strides; `PERMUTE` applies the K permutation of quantize_nvfp4.cu:86-100 (each group of
// 32 viewed as [4][4][2] and transposed in its first two modes).  Threads are laid out so
// that neighbouring lanes walk the dimension with the smaller stride.
// ----------------------------------------------------------------------------------------
template <int SF_LAYOUT, bool PERMUTE, bool ROW_FASTEST>
__global__ void __launch_bounds__(256)
nvfp4_quantize_strided_kernel(uint8_t *__restrict__ out, uint8_t *__restrict__ sf,
                              const uint16_t *__restrict__ in, const float *__restrict__ gscale,
                              int64_t M, int64_t K, int64_t d1, int64_t stride0, int64_t stride1,
                              int64_t stride_m, int64_t stride_k) {
  const int64_t Kp = align_up(K, 64);
  const int64_t KT = Kp / 64;
  const int64_t nblk = Kp / 16;
  const int64_t M16 = align_up(M, 16);
  const int64_t MT = ceil_div(M, 128);
  const int64_t rows_sf = (SF_LAYOUT == AC4K_SF_AC4K) ? M16 : MT * 128;
  const int64_t batch = blockIdx.z;

  int64_t row, blk;
  if (ROW_FASTEST) {   // 32 rows x 8 blocks per CTA
    row = (int64_t)blockIdx.y * 32 + (threadIdx.x & 31);
    blk = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  } else {             // 8 rows x 32 blocks per CTA
    row = (int64_t)blockIdx.y * 8 + (threadIdx.x >> 5);
    blk = (int64_t)blockIdx.x * 32 + (threadIdx.x & 31);
  }
  if (row >= rows_sf || blk >= nblk) return;

  const uint16_t *in_b = in + (batch / d1) * stride0 + (batch % d1) * stride1;
  const float alpha = load_alpha(gscale);

  uint32_t w[8];
  uint32_t amax = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint32_t pair = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int64_t p = blk * 16 + j * 2 + h;   // position in the (permuted) output row
      int64_t src = p;
      if (PERMUTE) {
        const int64_t q = p & 31;
        src = (p - q) + 8 * ((q & 7) >> 1) + 2 * (q >> 3) + (q & 1);
      }
      uint32_t e = 0;
      if (row < M && src < K) e = __ldg(in_b + row * stride_m + src * stride_k);
      pair |= e << (16 * h);
      const uint32_t a = e & 0x7FFFu;
      amax = a > amax ? a : amax;
    }
    w[j] = pair;
  }
  const BlockScale bs = block_scale(bf16_bits_to_f32(amax), alpha);

  if (row < M) {
    uint4 lo = make_uint4(w[0], w[1], w[2], w[3]), hi = make_uint4(w[4], w[5], w[6], w[7]);
    uint2 codes = make_uint2(quantize8(lo, bs.r), quantize8(hi, bs.r));
    *reinterpret_cast<uint2 *>(out + (batch * M + row) * (Kp / 2) + blk * 8) = codes;
  }
  const uint8_t b = (row < M) ? bs.byte : (uint8_t)0;
  const int64_t k64 = blk >> 2;
  if (SF_LAYOUT == AC4K_SF_AC4K) {
    sf[((batch * KT + k64) * M16 + row) * 4 + (blk & 3)] = b;
  } else {
    const int64_t mt = row >> 7, rl = row & 127;
    sf[((batch * MT + mt) * KT + k64) * 512 + (rl & 31) * 16 + (rl >> 5) * 4 + (blk & 3)] = b;
  }
}

// ----------------------------------------------------------------------------------------
// Transposing kernel: rows contiguous in memory along the CROSS dimension (stride_m == 1) and strided
// along K -- attention's V, quantised along the keys with the head dimension as output rows.  The
// strided kernel above reads 64 bytes per warp load there and writes 8-byte pieces 'Kp / 2' apart.
// Here one CTA takes 128 K-elements x 128 rows: a thread loads 32 words (two neighbouring rows x 32
// consecutive K-elements; a warp reads 128 contiguous bytes per load), quantises its four blocks of
// 16 in registers, and codes and scale bytes go through shared memory so that each output row leaves
// as 64 contiguous bytes and the scales as whole words.
// ----------------------------------------------------------------------------------------
template <int SF_LAYOUT, bool PERMUTE>
__global__ void __launch_bounds__(256)
nvfp4_quantize_transposed_kernel(uint8_t *__restrict__ out, uint8_t *__restrict__ sf, const uint16_t *__restrict__ in,
                                 const float *__restrict__ gscale, int64_t M, int64_t K, int64_t d1, int64_t stride0,
                                 int64_t stride1, int64_t stride_k) {
  __shared__ uint4 s_codes[128][4 + 1];          // [row][32-element group of the tile], padded
  __shared__ uint32_t s_sf[2][128];              // [K = 64 step of the tile][row]: four scale bytes
  const int64_t Kp = align_up(K, 64), KT = Kp / 64, M16 = align_up(M, 16), MT = ceil_div(M, 128);
  const int64_t batch = blockIdx.z;
  const int64_t k0 = (int64_t)blockIdx.x * 128, m0 = (int64_t)blockIdx.y * 128;
  const int cx = threadIdx.x & 63, kg = threadIdx.x >> 6;
  const int64_t m = m0 + 2 * cx, kb = k0 + 32 * kg;           // this thread: rows m, m + 1; K-elements kb .. kb + 31
  const uint16_t *base = in + (batch / d1) * stride0 + (batch % d1) * stride1;
  const float alpha = load_alpha(gscale);

  uint32_t w[32];                                // w[j]: element kb + j of row m (low half) and of row m + 1 (high half)
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    w[j] = 0u;
    if (m < M && kb + j < K) w[j] = __ldg(reinterpret_cast<const uint32_t *>(base + (kb + j) * stride_k + m));
  }
  uint32_t bytes[2] = {0u, 0u};                  // the two block scales of this group, for row m and row m + 1
  uint4 codes[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    // pairs of consecutive K-elements of row m + r, in output order: position pair j holds elements src(2 j), src(2 j) + 1
    uint32_t pr[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      int e = 2 * j;
      if (PERMUTE) e = 8 * (((2 * j) & 7) >> 1) + 2 * ((2 * j) >> 3);
      pr[j] = __byte_perm(w[e], w[e + 1], r == 0 ? 0x5410 : 0x7632);
    }
    uint32_t cw[4];
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      uint32_t amax = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t a = pr[8 * blk + j] & 0x7FFF7FFFu;
        amax = max(amax, max(a & 0xFFFFu, a >> 16));
      }
      const BlockScale bs = block_scale(bf16_bits_to_f32(amax), alpha);
      cw[2 * blk] = quantize8(make_uint4(pr[8 * blk], pr[8 * blk + 1], pr[8 * blk + 2], pr[8 * blk + 3]), bs.r);
      cw[2 * blk + 1] = quantize8(make_uint4(pr[8 * blk + 4], pr[8 * blk + 5], pr[8 * blk + 6], pr[8 * blk + 7]), bs.r);
      bytes[r] |= (uint32_t)((m + r < M) ? bs.byte : (uint8_t)0) << (8 * blk);
    }
    codes[r] = make_uint4(cw[0], cw[1], cw[2], cw[3]);
  }
  s_codes[2 * cx][kg] = codes[0];
  s_codes[2 * cx + 1][kg] = codes[1];
  // scale bytes: group kg covers blocks 2 (kg & 1), 2 (kg & 1) + 1 of K = 64 step kg >> 1
  reinterpret_cast<uint16_t *>(&s_sf[kg >> 1][2 * cx])[kg & 1] = (uint16_t)bytes[0];
  reinterpret_cast<uint16_t *>(&s_sf[kg >> 1][2 * cx + 1])[kg & 1] = (uint16_t)bytes[1];
  __syncthreads();
  // codes: 128 rows x 64 bytes, four threads per row
  for (int v = threadIdx.x; v < 512; v += 256) {
    const int row = v >> 2, g = v & 3;
    if (m0 + row < M && k0 + 32 * g < Kp)
      *reinterpret_cast<uint4 *>(out + (batch * M + m0 + row) * (Kp / 2) + (k0 + 32 * g) / 2) = s_codes[row][g];
  }
  // scales: one word per row and K = 64 step
  {
    const int row = threadIdx.x & 127, ks = threadIdx.x >> 7;
    const int64_t k64 = k0 / 64 + ks, rg = m0 + row;
    const int64_t rows_sf = (SF_LAYOUT == AC4K_SF_AC4K) ? M16 : MT * 128;
    if (k64 < KT && rg < rows_sf) {
      uint32_t *sfw = reinterpret_cast<uint32_t *>(sf);
      if (SF_LAYOUT == AC4K_SF_AC4K)
        sfw[(batch * KT + k64) * M16 + rg] = s_sf[ks][row];
      else
        sfw[((batch * MT + blockIdx.y) * KT + k64) * 128 + (row & 31) * 4 + (row >> 5)] = s_sf[ks][row];
    }
  }
}

// ----------------------------------------------------------------------------------------
// Global scale: max|x| / max_scale.  Division is monotonic, so each CTA divides its own
// maximum and combines with an integer atomicMax on the (non-negative) float bits, the
// same scheme as the reference's Triton kernel (python/ac4k_kernel/ops/quant.py:21-46).
// ----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512)
global_scale_kernel(const uint16_t *__restrict__ x, int64_t n, float max_scale, float *g_out) {
  uint32_t m2 = 0;   // packed pair of running maxima (bf16 bits, sign cleared)
  uint32_t m1 = 0;   // scalar head/tail
  // head: elements before the first 16-byte boundary
  const uintptr_t addr = reinterpret_cast<uintptr_t>(x);
  int64_t head = ((16 - (addr & 15)) & 15) / 2;
  if (head > n) head = n;
  const int64_t nvec = (n - head) / 8;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthr = (int64_t)gridDim.x * blockDim.x;
  const uint4 *xv = reinterpret_cast<const uint4 *>(x + head);
  int64_t i = tid;
  for (; i + 3 * nthr < nvec; i += 4 * nthr) {
    uint4 a = __ldcs(xv + i), b = __ldcs(xv + i + nthr), c = __ldcs(xv + i + 2 * nthr),
          d = __ldcs(xv + i + 3 * nthr);
    uint32_t ma = max_bf16x2(max_bf16x2(abs_bf16x2(a.x), abs_bf16x2(a.y)),
                             max_bf16x2(abs_bf16x2(a.z), abs_bf16x2(a.w)));
    uint32_t mb = max_bf16x2(max_bf16x2(abs_bf16x2(b.x), abs_bf16x2(b.y)),
                             max_bf16x2(abs_bf16x2(b.z), abs_bf16x2(b.w)));
    uint32_t mc = max_bf16x2(max_bf16x2(abs_bf16x2(c.x), abs_bf16x2(c.y)),
                             max_bf16x2(abs_bf16x2(c.z), abs_bf16x2(c.w)));
    uint32_t md = max_bf16x2(max_bf16x2(abs_bf16x2(d.x), abs_bf16x2(d.y)),
                             max_bf16x2(abs_bf16x2(d.z), abs_bf16x2(d.w)));
    m2 = max_bf16x2(m2, max_bf16x2(max_bf16x2(ma, mb), max_bf16x2(mc, md)));
  }
  for (; i < nvec; i += nthr) {
    uint4 a = __ldcs(xv + i);
    m2 = max_bf16x2(m2, max_bf16x2(max_bf16x2(abs_bf16x2(a.x), abs_bf16x2(a.y)),
                                   max_bf16x2(abs_bf16x2(a.z), abs_bf16x2(a.w))));
  }
  if (tid < head) m1 = x[tid] & 0x7FFFu;
  const int64_t tail0 = head + nvec * 8;
  if (tail0 + tid < n) {
    uint32_t e = x[tail0 + tid] & 0x7FFFu;
    m1 = e > m1 ? e : m1;
  }
  uint32_t m = max(max(m2 & 0xFFFFu, m2 >> 16), m1);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  __shared__ uint32_t s_m[16];
  if ((threadIdx.x & 31) == 0) s_m[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    m = threadIdx.x < (blockDim.x >> 5) ? s_m[threadIdx.x] : 0;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (threadIdx.x == 0 && m != 0) {
      const float g = __fdiv_rn(bf16_bits_to_f32(m), max_scale);
      atomicMax(reinterpret_cast<int *>(g_out), __float_as_int(g));
    }
  }
}

}  // namespace ac4k

using namespace ac4k;

static int check_view(const int64_t shape[4], const int64_t stride[4]) {
  if (!shape || !stride) return fail(AC4K_ERR_NULL, "shape/stride is NULL");
  for (int i = 0; i < 4; ++i)
    if (shape[i] < 0) return fail(AC4K_ERR_SHAPE, "shape[%d] = %lld is negative", i, (long long)shape[i]);
  return 0;
}

extern "C" int ac4k_global_scale_bf16(const void *x, int64_t numel, float max_scale, float *g_out,
                                      ac4k_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!g_out) return fail(AC4K_ERR_NULL, "g_out is NULL");
  if (numel < 0) return fail(AC4K_ERR_SHAPE, "numel is negative");
  if (numel > 0 && !x) return fail(AC4K_ERR_NULL, "x is NULL");
  if (reinterpret_cast<uintptr_t>(x) & 1) return fail(AC4K_ERR_ALIGN, "x must be 2-byte aligned");
  if (!(max_scale > 0.0f)) return fail(AC4K_ERR_SHAPE, "max_scale must be positive");
  AC4K_CUDA_TRY(cudaMemsetAsync(g_out, 0, sizeof(float), stream));
  if (numel == 0) return 0;
  const int threads = 512;
  DeviceInfo di;
  if (int e = get_device_info(&di)) return e;
  int64_t blocks = ceil_div(ceil_div(numel, 8), (int64_t)threads * 4);
  if (blocks > (int64_t)di.sms * 4) blocks = (int64_t)di.sms * 4;     // four resident CTAs of 512 threads per SM
  if (blocks < 1) blocks = 1;
  global_scale_kernel<<<(unsigned)blocks, threads, 0, stream>>>(static_cast<const uint16_t *>(x), numel,
                                                               max_scale, g_out);
  AC4K_LAUNCH_CHECK("global_scale_kernel");
  return 0;
}

extern "C" int ac4k_quantize_nvfp4(void *out, void *sf, const void *in, const float *global_scale,
                                   const int64_t shape[4], const int64_t stride[4], int swizzle,
                                   int sf_layout, ac4k_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (int e = check_view(shape, stride)) return e;
  if (!out || !sf || !global_scale) return fail(AC4K_ERR_NULL, "out/sf/global_scale is NULL");
  if (sf_layout != AC4K_SF_AC4K && sf_layout != AC4K_SF_TILE128X4)
    return fail(AC4K_ERR_ENUM, "unknown sf_layout %d", sf_layout);
  const int64_t d0 = shape[0], d1 = shape[1], M = shape[2], K = shape[3];
  const int64_t nbatch = d0 * d1;
  if (nbatch == 0 || M == 0 || K == 0) return 0;   // nothing to write (padding needs K > 0 rows)
  if (!in) return fail(AC4K_ERR_NULL, "in is NULL");
  if (nbatch > 65535) return fail(AC4K_ERR_SHAPE, "outer dims product %lld exceeds 65535", (long long)nbatch);
  if ((reinterpret_cast<uintptr_t>(out) & 7) || (reinterpret_cast<uintptr_t>(sf) & 3))
    return fail(AC4K_ERR_ALIGN, "out must be 8-byte and sf 4-byte aligned");
  const int64_t Kp = align_up(K, 64);
  const uint16_t *inp = static_cast<const uint16_t *>(in);

  const bool vec_ok = !swizzle && stride[3] == 1 && (K % 16 == 0) && (stride[2] % 8 == 0) &&
                      (stride[0] % 8 == 0) && (stride[1] % 8 == 0) &&
                      ((reinterpret_cast<uintptr_t>(in) & 15) == 0);
  if (vec_ok) {
    const bool wide = (stride[2] % 16 == 0) && (stride[0] % 16 == 0) && (stride[1] % 16 == 0) &&
                      ((reinterpret_cast<uintptr_t>(in) & 31) == 0);
    const int tile_k = Kp <= 128 ? 128 : 256;
    dim3 grid((unsigned)ceil_div(Kp, (int64_t)tile_k), (unsigned)ceil_div(M, kTileRows), (unsigned)nbatch);
    if (ceil_div(M, kTileRows) > 65535) return fail(AC4K_ERR_SHAPE, "M too large");
#define AC4K_LAUNCH_TILED(L, W, T)                                                                \
  nvfp4_quantize_tiled_kernel<L, W, T><<<grid, kThreads, 0, stream>>>(                            \
      static_cast<uint8_t *>(out), static_cast<uint32_t *>(sf), inp, global_scale, M, K, d1,      \
      stride[0], stride[1], stride[2])
#define AC4K_LAUNCH_TILED_K(L, W)                                                                 \
  do { if (tile_k == 128) AC4K_LAUNCH_TILED(L, W, 128); else AC4K_LAUNCH_TILED(L, W, 256); } while (0)
    if (sf_layout == AC4K_SF_AC4K) {
      if (wide) AC4K_LAUNCH_TILED_K(AC4K_SF_AC4K, true); else AC4K_LAUNCH_TILED_K(AC4K_SF_AC4K, false);
    } else {
      if (wide) AC4K_LAUNCH_TILED_K(AC4K_SF_TILE128X4, true); else AC4K_LAUNCH_TILED_K(AC4K_SF_TILE128X4, false);
    }
#undef AC4K_LAUNCH_TILED_K
#undef AC4K_LAUNCH_TILED
    AC4K_LAUNCH_CHECK("nvfp4_quantize_tiled_kernel");
    return 0;
  }

  const int64_t rows_sf = (sf_layout == AC4K_SF_AC4K) ? align_up(M, 16) : align_up(M, 128);
  const bool row_fastest = stride[2] < stride[3];
  // rows contiguous along the cross dimension, K strided: the transposing kernel
  const bool tr_ok = stride[2] == 1 && M % 2 == 0 && stride[3] % 2 == 0 && stride[0] % 2 == 0 && stride[1] % 2 == 0 &&
                     ((reinterpret_cast<uintptr_t>(in) & 3) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) &&
                     ceil_div(M, 128) <= 65535;
  if (tr_ok) {
    dim3 g((unsigned)ceil_div(Kp, 128), (unsigned)ceil_div(M, 128), (unsigned)nbatch);
#define AC4K_LAUNCH_TR(L, P)                                                                                        \
  nvfp4_quantize_transposed_kernel<L, P><<<g, 256, 0, stream>>>(static_cast<uint8_t *>(out), static_cast<uint8_t *>(sf), inp, \
                                                                global_scale, M, K, d1, stride[0], stride[1], stride[3])
    if (sf_layout == AC4K_SF_AC4K) {
      if (swizzle) AC4K_LAUNCH_TR(AC4K_SF_AC4K, true); else AC4K_LAUNCH_TR(AC4K_SF_AC4K, false);
    } else {
      if (swizzle) AC4K_LAUNCH_TR(AC4K_SF_TILE128X4, true); else AC4K_LAUNCH_TR(AC4K_SF_TILE128X4, false);
    }
#undef AC4K_LAUNCH_TR
    AC4K_LAUNCH_CHECK("nvfp4_quantize_transposed_kernel");
    return 0;
  }
  dim3 grid;
  if (row_fastest)
    grid = dim3((unsigned)ceil_div(Kp / 16, 8), (unsigned)ceil_div(rows_sf, 32), (unsigned)nbatch);
  else
    grid = dim3((unsigned)ceil_div(Kp / 16, 32), (unsigned)ceil_div(rows_sf, 8), (unsigned)nbatch);
  if (grid.y > 65535) return fail(AC4K_ERR_SHAPE, "M too large for the strided path");
#define AC4K_LAUNCH_STRIDED(L, P, R)                                                             \
  nvfp4_quantize_strided_kernel<L, P, R><<<grid, 256, 0, stream>>>(                              \
      static_cast<uint8_t *>(out), static_cast<uint8_t *>(sf), inp, global_scale, M, K, d1,      \
      stride[0], stride[1], stride[2], stride[3])
  const int sel = (sf_layout == AC4K_SF_TILE128X4 ? 4 : 0) | (swizzle ? 2 : 0) | (row_fastest ? 1 : 0);
  switch (sel) {
    case 0: AC4K_LAUNCH_STRIDED(AC4K_SF_AC4K, false, false); break;
    case 1: AC4K_LAUNCH_STRIDED(AC4K_SF_AC4K, false, true); break;
    case 2: AC4K_LAUNCH_STRIDED(AC4K_SF_AC4K, true, false); break;
    case 3: AC4K_LAUNCH_STRIDED(AC4K_SF_AC4K, true, true); break;
    case 4: AC4K_LAUNCH_STRIDED(AC4K_SF_TILE128X4, false, false); break;
    case 5: AC4K_LAUNCH_STRIDED(AC4K_SF_TILE128X4, false, true); break;
    case 6: AC4K_LAUNCH_STRIDED(AC4K_SF_TILE128X4, true, false); break;
    default: AC4K_LAUNCH_STRIDED(AC4K_SF_TILE128X4, true, true); break;
  }
#undef AC4K_LAUNCH_STRIDED
  AC4K_LAUNCH_CHECK("nvfp4_quantize_strided_kernel");
  return 0;
}
