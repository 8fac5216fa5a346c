// Pieces shared by the 1-CTA and 2-CTA NVFP4 GEMM kernels: tile constants, kernel arguments,
// tile rasterisation, epilogue helpers, and the host-side tensor-map cache.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ac4k {
using namespace ptx;

#if defined(AC4K_TRACE_ENABLED) && !defined(AC4K_DEBUG_HOOKS)
#define AC4K_DEBUG_HOOKS 1
#endif
// experiment switch `bit` of the kernel arguments / launch arguments `p`; constant 0 in the default build
#ifdef AC4K_DEBUG_HOOKS
#define AC4K_DBG(p, bit) ((p).dbg & (bit))
#else
#define AC4K_DBG(p, bit) 0
#endif

static constexpr int BM = 128;        // rows of A per tile (= TMEM lanes)
static constexpr int BKB = 128;       // bytes of packed K per stage (= 256 elements = 4 MMA K-steps)
static constexpr int K64_PER_STAGE = 4;
static constexpr int kNumThreads = 320;
static constexpr int kTmemCols = 512;
static constexpr int kGroupM = 8;     // tile rasterisation: walk 8 M-tiles per N-tile

enum : unsigned { kStatusTimeoutProducer = 0xA1, kStatusTimeoutMma = 0xA2, kStatusTimeoutSf = 0xA3,
                  kStatusTimeoutEpilogue = 0xA4, kStatusSmemAlign = 0xB1 };

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * BKB;
  static constexpr int B_BYTES = BN * BKB;
  static constexpr int SFA_BYTES = K64_PER_STAGE * 512;
  static constexpr int SFB_BYTES = (BN / 128) * K64_PER_STAGE * 512;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int STAGES = (BN == 128) ? 6 : 4;
  static constexpr int ACC_STAGES = (BN == 128) ? 2 : 1;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 512 /*barriers*/;
  // tensor-memory columns: accumulators, then the scales of one stage (A: 4 columns per K step, then B)
  static constexpr int SF_COL = ACC_STAGES * BN;
  static constexpr int SF_COLS = K64_PER_STAGE * (4 + BN / 32);
  static_assert(SF_COL + SF_COLS <= kTmemCols, "tensor memory overflow");
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory overflow");
};

enum { EPI_PLAIN = 0, EPI_GATHER = 1, EPI_REQUANT = 2 };   // epilogue variants of the pair kernel
static constexpr int kMaxDst = 8;     // output destinations of one launch (this GPU + up to 7 peers)

// Tensor maps of the output destinations of the pair kernel's TMA-store epilogue: [0] this GPU's buffer,
// [1 .. n_dst) the further destinations of the fused all-gather.
struct DstMaps { CUtensorMap m[kMaxDst]; };

struct GemmArgs {
  const uint8_t *sfa;
  const uint8_t *sfb;
  void *D;              // first (or only) destination
  void *D_more[kMaxDst - 1];   // further destinations of the same tile stores (pair kernel only), n_dst - 1 used
  int n_dst;            // 1 for the plain GEMM
  int64_t ldd;          // leading dimension of every destination, in elements (N for the plain GEMM)
  int64_t col_off;      // first destination column of this launch's N columns (0 for the plain GEMM)
  // re-quantising epilogue (pair kernel, EPI_REQUANT): the bf16 result is not stored but quantised to
  // NVFP4 with the given global scale, exactly as the quantiser would quantise the stored bf16 matrix
  uint8_t *q_out;       // [M, N / 2] packed e2m1
  uint8_t *q_sf;        // block scales of the output in q_layout
  const float *q_gs;    // global scale of the output (device scalar)
  int q_layout;         // AC4K_SF_AC4K or AC4K_SF_TILE128X4
  int q_rows;           // padded row count of q_sf (16- or 128-aligned M)
  const float *a_gs;
  const float *b_gs;
  const void *bias;
  unsigned int *status;
  int bias_dt;
  int M, N, K;          // K in elements, multiple of 64
  int KT;               // K / 64
  int rows_sfa, rows_sfb;   // padded row counts of the scale tensors (16- or 128-aligned)
  int tiles_m, tiles_n;
  int splits;           // split-K factor (1-CTA kernel only); > 1 writes fp32 partials to `ws`
  int kt_per_split;     // K stages (of 256 elements) per split
  float *ws;            // [splits, M, N] fp32 partial sums when splits > 1
  unsigned long long wait_ns;   // limit of every device-side wait of the launch (kWaitTimeoutNs; shorter in the wait-expiry test)
  int dbg;              // experiment switches (builds with -DAC4K_DEBUG_HOOKS), else 0
  unsigned long long *trace;   // clock stamps (builds with -DAC4K_TRACE_ENABLED), else NULL
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int &tm, int &tn) {
  const int group = kGroupM * tiles_n;
  const int g = t / group;
  const int first_m = g * kGroupM;
  const int gm = min(tiles_m - first_m, kGroupM);
  const int r = t - g * group;
  tm = first_m + r % gm;
  tn = r / gm;
}

__device__ __forceinline__ float load_bias(const void *bias, int dt, int n) {
  if (dt == AC4K_DT_BF16) return __bfloat162float(static_cast<const __nv_bfloat16 *>(bias)[n]);
  if (dt == AC4K_DT_FP16) return __half2float(static_cast<const __half *>(bias)[n]);
  return static_cast<const float *>(bias)[n];
}

template <int OUT_DT>
struct OutT;
template <> struct OutT<AC4K_DT_BF16> { using type = __nv_bfloat16; };
template <> struct OutT<AC4K_DT_FP16> { using type = __half; };
template <> struct OutT<AC4K_DT_FP32> { using type = float; };

template <int OUT_DT>
__device__ __forceinline__ void store_row32(void *D, int64_t off, const float (&v)[32], int ncols, bool vec_ok) {
  using T = typename OutT<OUT_DT>::type;
  T *dst = static_cast<T *>(D) + off;
  if (vec_ok && ncols == 32) {
    if (OUT_DT == AC4K_DT_FP32) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        reinterpret_cast<float4 *>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (OUT_DT == AC4K_DT_BF16) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
            w[j] = *reinterpret_cast<uint32_t *>(&h);
          } else {
            __half2 h = __floats2half2_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
            w[j] = *reinterpret_cast<uint32_t *>(&h);
          }
        }
        reinterpret_cast<uint4 *>(dst)[i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  } else {
    for (int i = 0; i < ncols; ++i) {
      if (OUT_DT == AC4K_DT_BF16) dst[i] = (T)__float2bfloat16_rn(v[i]);
      else if (OUT_DT == AC4K_DT_FP16) dst[i] = (T)__float2half_rn(v[i]);
      else dst[i] = (T)v[i];
    }
  }
}


// host helpers (linear_nvfp4.cu)
// 2-D byte tensor map [rows, row_bytes] with a (128 B x box_rows) box and 128-byte swizzle
int get_tmap(const void *ptr, int64_t rows, int64_t row_bytes, int box_rows, CUtensorMap *out);
// same bytes with the rows as (row / 4, row % 4): a box of 128 B x 32 x 4 brings rows 4 l + q of a 128-row block to
// shared-memory row q * 32 + l; rows must be a multiple of 4
int get_tmap_rows4(const void *ptr, int64_t rows, int64_t row_bytes, CUtensorMap *out);
// tiled scales [row blocks][K/64][512 B] as a matrix of 512-byte rows, boxes of box_ksteps rows
int get_tmap_sf_tiled(const void *ptr, int64_t row_blocks, int64_t kt, int box_ksteps, CUtensorMap *out);
// scales in the row layout [K/64][rows] words: boxes of 128 words (the rows of a 128-row block) x 4 K steps
int get_tmap_sf_rows(const void *ptr, int64_t rows, int64_t kt, CUtensorMap *out);
// 2-D byte tensor map with a (64 B x box_rows) box and 64-byte swizzle
int get_tmap64(const void *ptr, int64_t rows, int64_t row_bytes, int box_rows, CUtensorMap *out);
unsigned long long *debug_trace_ptr();
// bf16 [B, H, N, D] by element strides (D contiguous, the others multiples of 8): boxes of D x box_rows x 1 x 1
int get_tmap_bf16_4d(const void *ptr, const int64_t shape[4], const int64_t stride[4], int box_rows, CUtensorMap *out);
// 16-bit output [rows, cols] with a row pitch of ld elements: boxes of 64 columns x 32 rows, 128-byte swizzle
int get_tmap_out16(const void *ptr, int64_t rows, int64_t cols, int64_t ld, CUtensorMap *out);
// the same output with the rows as (row / 4, row % 4): boxes of 64 columns x 32 x 1; rows must be a multiple of 4
int get_tmap_out16_rows4(const void *ptr, int64_t rows, int64_t cols, int64_t ld, CUtensorMap *out);
// 2-CTA kernel launcher (linear_nvfp4_2cta.cu); D must be bf16/fp16 with N % 8 == 0.  sf_mode 0: scales in the row
// layout read with plain loads (ta, tb, dm from get_tmap / get_tmap_out16); 1: tiled scales (tsa, tsb from
// get_tmap_sf_tiled); 2: scales in the row layout by TMA (tsa, tsb from get_tmap_sf_rows; ta, tb from get_tmap_rows4,
// dm from get_tmap_out16_rows4)
int launch_linear_2cta(int d_dtype, int sf_mode, const CUtensorMap &ta, const CUtensorMap &tb,
                       const CUtensorMap &tsa, const CUtensorMap &tsb, const DstMaps &dm, GemmArgs args, cudaStream_t stream);

// decode-shape kernel (linear_nvfp4_skinny.cu): M <= nt activation rows, nt in {16, 32, 64}
int launch_linear_skinny(int d_dtype, bool sf_tiled, int nt, const CUtensorMap &tx, const CUtensorMap &tw, const GemmArgs &args,
                         cudaStream_t stream);

}  // namespace ac4k
