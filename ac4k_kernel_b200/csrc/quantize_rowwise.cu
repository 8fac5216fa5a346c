// Per-row ("per-token") FP8-E4M3 and INT8 quantisers for sm_100a.
//
// Semantics follow ac4k_kernel's lib/cuda/sm120/quantize_fp8.cu:57-185 and
// quantize_int8.cu:61-168: amax over the whole reduce dimension of a row, stored scale
// amax / scale_max (fp32, for all align16(M) rows, 0 for padding rows), elements
// x * (scale_max / amax) converted with round-to-nearest-even and saturation; K is padded
// to 16 with zeros.  A row of zeros gives 0 * inf = NaN exactly like the reference (e4m3
// 0x7F, int8 0).  Unlike the reference the row is read from memory once: a thread group
// keeps its slice of the row in registers between the amax pass and the conversion pass.
#include "common.cuh"

namespace ac4k {

enum { kFmtE4M3 = 0, kFmtS8 = 1 };

template <int FMT>
__device__ __forceinline__ uint2 convert8(const uint4 &v, float r) {
  float f[8];
  f[0] = __fmul_rn(__uint_as_float(v.x << 16), r);
  f[1] = __fmul_rn(__uint_as_float(v.x & 0xFFFF0000u), r);
  f[2] = __fmul_rn(__uint_as_float(v.y << 16), r);
  f[3] = __fmul_rn(__uint_as_float(v.y & 0xFFFF0000u), r);
  f[4] = __fmul_rn(__uint_as_float(v.z << 16), r);
  f[5] = __fmul_rn(__uint_as_float(v.z & 0xFFFF0000u), r);
  f[6] = __fmul_rn(__uint_as_float(v.w << 16), r);
  f[7] = __fmul_rn(__uint_as_float(v.w & 0xFFFF0000u), r);
  uint2 o;
  if (FMT == kFmtE4M3) {
    o.x = f32x4_to_e4m3x4(f[0], f[1], f[2], f[3]);
    o.y = f32x4_to_e4m3x4(f[4], f[5], f[6], f[7]);
  } else {
    o.x = f32x4_to_s8x4(f[0], f[1], f[2], f[3]);
    o.y = f32x4_to_s8x4(f[4], f[5], f[6], f[7]);
  }
  return o;
}

template <int FMT>
__device__ __forceinline__ uint8_t convert1(uint32_t bits16, float r) {
  float f = __fmul_rn(bf16_bits_to_f32(bits16), r);
  if (FMT == kFmtE4M3) return (uint8_t)(f32x4_to_e4m3x4(f, 0.f, 0.f, 0.f) & 0xFF);
  return (uint8_t)f32_to_s8_rni_sat(f);
}

__device__ __forceinline__ float load_scale_max(const void *p, int is_int) {
  return is_int ? (float)__ldg(static_cast<const int32_t *>(p)) : __ldg(static_cast<const float *>(p));
}

// ----------------------------------------------------------------------------------------
// Contiguous rows.  A group of G threads (32 = one warp, or 256 = the CTA) owns one row and
// caches up to CACHE 16-byte chunks per thread; longer rows are re-read for the second pass.
// ----------------------------------------------------------------------------------------
template <int FMT, int G, int CACHE>
__global__ void __launch_bounds__(256)
rowwise_quantize_kernel(uint8_t *__restrict__ out, float *__restrict__ sf,
                        const uint16_t *__restrict__ in, const void *__restrict__ scale_max_p,
                        int scale_max_is_int, int64_t M, int64_t K, int64_t d1, int64_t stride0,
                        int64_t stride1, int64_t row_stride) {
  constexpr int ROWS = 256 / G;
  __shared__ uint32_t s_m[8];
  const int64_t Kp = align_up(K, 16);
  const int64_t M16 = align_up(M, 16);
  const int64_t batch = blockIdx.y;
  const int g = threadIdx.x / G, t = threadIdx.x % G;
  const int64_t row = (int64_t)blockIdx.x * ROWS + g;
  const uint16_t *in_r = in + (batch / d1) * stride0 + (batch % d1) * stride1 + row * row_stride;
  const int64_t nchunk = Kp / 8;          // 8-element chunks in the padded row
  const int64_t nfull = K / 8;            // chunks fully inside the data (K % 8 == 0 here)
  const bool live = row < M;

  uint4 v[CACHE];
  uint32_t m2 = 0;
#pragma unroll
  for (int c = 0; c < CACHE; ++c) {
    const int64_t ch = (int64_t)c * G + t;
    v[c] = make_uint4(0, 0, 0, 0);
    if (live && ch < nfull) v[c] = __ldcs(reinterpret_cast<const uint4 *>(in_r + ch * 8));
  }
#pragma unroll
  for (int c = 0; c < CACHE; ++c)
    m2 = max_bf16x2(m2, max_bf16x2(max_bf16x2(abs_bf16x2(v[c].x), abs_bf16x2(v[c].y)),
                                   max_bf16x2(abs_bf16x2(v[c].z), abs_bf16x2(v[c].w))));
  if (live)
    for (int64_t ch = (int64_t)CACHE * G + t; ch < nfull; ch += G) {
      uint4 a = __ldg(reinterpret_cast<const uint4 *>(in_r + ch * 8));
      m2 = max_bf16x2(m2, max_bf16x2(max_bf16x2(abs_bf16x2(a.x), abs_bf16x2(a.y)),
                                     max_bf16x2(abs_bf16x2(a.z), abs_bf16x2(a.w))));
    }
  uint32_t m = max(m2 & 0xFFFFu, m2 >> 16);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  if (G == 256) {
    if ((threadIdx.x & 31) == 0) s_m[threadIdx.x >> 5] = m;
    __syncthreads();
    m = s_m[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) m = max(m, s_m[i]);
  }
  const float amax = bf16_bits_to_f32(m);
  const float smax = load_scale_max(scale_max_p, scale_max_is_int);
  if (t == 0 && row < M16) sf[batch * M16 + row] = live ? __fdiv_rn(amax, smax) : 0.0f;
  if (!live) return;
  const float r = __fdiv_rn(smax, amax);
  uint8_t *out_r = out + (batch * M + row) * Kp;
#pragma unroll
  for (int c = 0; c < CACHE; ++c) {
    const int64_t ch = (int64_t)c * G + t;
    if (ch < nchunk) __stcs(reinterpret_cast<uint2 *>(out_r + ch * 8), convert8<FMT>(v[c], r));
  }
  for (int64_t ch = (int64_t)CACHE * G + t; ch < nchunk; ch += G) {
    uint4 a = make_uint4(0, 0, 0, 0);
    if (ch < nfull) a = __ldg(reinterpret_cast<const uint4 *>(in_r + ch * 8));
    __stcs(reinterpret_cast<uint2 *>(out_r + ch * 8), convert8<FMT>(a, r));
  }
}

// ----------------------------------------------------------------------------------------
// Strided rows (any element strides, optional FP8 K permutation of quantize_fp8.cu:141-151:
// every 16 elements viewed as [2][4][2] and transposed in the first two modes).  One warp
// per row, scalar loads, two passes.
// ----------------------------------------------------------------------------------------
template <int FMT, bool PERMUTE>
__global__ void __launch_bounds__(256)
rowwise_quantize_strided_kernel(uint8_t *__restrict__ out, float *__restrict__ sf,
                                const uint16_t *__restrict__ in, const void *__restrict__ scale_max_p,
                                int scale_max_is_int, int64_t M, int64_t K, int64_t d1,
                                int64_t stride0, int64_t stride1, int64_t stride_m, int64_t stride_k) {
  const int64_t Kp = align_up(K, 16);
  const int64_t M16 = align_up(M, 16);
  const int64_t batch = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= M16) return;
  const bool live = row < M;
  const uint16_t *in_r = in + (batch / d1) * stride0 + (batch % d1) * stride1 + row * stride_m;
  uint32_t m = 0;
  if (live)
    for (int64_t k = lane; k < K; k += 32) {
      uint32_t e = __ldg(in_r + k * stride_k) & 0x7FFFu;
      m = e > m ? e : m;
    }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  const float amax = bf16_bits_to_f32(m);
  const float smax = load_scale_max(scale_max_p, scale_max_is_int);
  if (lane == 0) sf[batch * M16 + row] = live ? __fdiv_rn(amax, smax) : 0.0f;
  if (!live) return;
  const float r = __fdiv_rn(smax, amax);
  uint8_t *out_r = out + (batch * M + row) * Kp;
  for (int64_t p = lane; p < Kp; p += 32) {
    int64_t src = p;
    if (PERMUTE) {
      const int64_t q = p & 15;
      src = (p - q) + 8 * ((q & 3) >> 1) + 2 * (q >> 2) + (q & 1);
    }
    const uint32_t e = src < K ? __ldg(in_r + src * stride_k) : 0u;
    out_r[p] = convert1<FMT>(e, r);
  }
}

// ----------------------------------------------------------------------------------------
// Rows strided, columns contiguous (stride_m == 1): the V operand of attention, quantised along the keys
// with the head dimension as rows of the output.  The one-warp-per-row kernel above reads 2 bytes per
// 32-byte sector here; these three kernels read the input in its own order instead:
//   1. column maxima: CTAs walk chunks of 256 reduce-rows, a warp reads 128 contiguous bytes of a row,
//      per-column maxima meet in shared memory and leave as one atomicMax per column and CTA (on the
//      bit pattern: non-negative floats order like integers) into the scale array, zeroed before;
//   2. quantise + transpose: tiles of 64 reduce-rows x 128 columns through shared memory, written out as
//      16-byte pieces along the reduce dimension (with the K permutation if asked for);
//   3. scale array: maxima -> maxima / scale_max, padding rows 0.
// ----------------------------------------------------------------------------------------
static constexpr int kTrCols = 128, kTrRows = 64, kTrChunk = 256;

__global__ void __launch_bounds__(256)
colmax_kernel(float *__restrict__ sf, const uint16_t *__restrict__ in, int64_t M, int64_t K, int64_t M16, int64_t d1,
              int64_t stride0, int64_t stride1, int64_t stride_k) {
  __shared__ uint32_t red[4][kTrCols];
  const int64_t batch = blockIdx.z;
  const int cx = threadIdx.x & 63, ry = threadIdx.x >> 6;
  const int64_t col = (int64_t)blockIdx.y * kTrCols + 2 * cx;
  const uint16_t *base = in + (batch / d1) * stride0 + (batch % d1) * stride1;
  const int64_t k0 = (int64_t)blockIdx.x * kTrChunk, k1 = min(k0 + kTrChunk, K);
  uint32_t m0 = 0, m1 = 0;
  if (col < M)
    for (int64_t k = k0 + ry; k < k1; k += 4) {
      const uint32_t w = __ldg(reinterpret_cast<const uint32_t *>(base + k * stride_k + col));
      m0 = max(m0, w & 0x7FFFu);
      m1 = max(m1, (w >> 16) & 0x7FFFu);
    }
  red[ry][2 * cx] = m0;
  red[ry][2 * cx + 1] = m1;
  __syncthreads();
  if (threadIdx.x < kTrCols) {
    const int64_t c = (int64_t)blockIdx.y * kTrCols + threadIdx.x;
    if (c < M) {
      const uint32_t m = max(max(red[0][threadIdx.x], red[1][threadIdx.x]), max(red[2][threadIdx.x], red[3][threadIdx.x]));
      atomicMax(reinterpret_cast<unsigned int *>(sf + batch * M16 + c), m << 16);
    }
  }
}

template <int FMT, bool PERMUTE>
__global__ void __launch_bounds__(256)
transpose_quantize_kernel(uint8_t *__restrict__ out, const float *__restrict__ amax_bits, const uint16_t *__restrict__ in,
                          const void *__restrict__ scale_max_p, int scale_max_is_int, int64_t M, int64_t K, int64_t M16, int64_t d1,
                          int64_t stride0, int64_t stride1, int64_t stride_k) {
  __shared__ uint32_t tile[kTrCols][kTrRows / 4 + 1];       // [column][4 reduce-rows per word], padded
  __shared__ float rs[kTrCols];
  const int64_t batch = blockIdx.z;
  const int64_t Kp = align_up(K, 16);
  const int64_t c0 = (int64_t)blockIdx.y * kTrCols, k0 = (int64_t)blockIdx.x * kTrRows;
  const uint16_t *base = in + (batch / d1) * stride0 + (batch % d1) * stride1;
  const float smax = load_scale_max(scale_max_p, scale_max_is_int);
  if (threadIdx.x < kTrCols) {
    const int64_t c = c0 + threadIdx.x;
    rs[threadIdx.x] = c < M ? __fdiv_rn(smax, __ldg(amax_bits + batch * M16 + c)) : 0.0f;
  }
  __syncthreads();
  const int cx = threadIdx.x & 63, ry = threadIdx.x >> 6;
  const int64_t col = c0 + 2 * cx;
  const float r0 = rs[2 * cx], r1 = rs[2 * cx + 1];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int kq = ry + 4 * i;                                  // word index: reduce-rows 4 kq .. 4 kq + 3 of the tile
    float a[4], b[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t k = k0 + 4 * kq + j;
      uint32_t w = 0;
      if (col < M && k < K) w = __ldg(reinterpret_cast<const uint32_t *>(base + k * stride_k + col));
      a[j] = __fmul_rn(__uint_as_float(w << 16), r0);
      b[j] = __fmul_rn(__uint_as_float(w & 0xFFFF0000u), r1);
      // (padding of the reduce dimension reads as 0 and is multiplied like the rest: 0 * inf = NaN for a zero row,
      // as in the reference and the one-warp-per-row kernel)
    }
    if (FMT == kFmtE4M3) {
      tile[2 * cx][kq] = f32x4_to_e4m3x4(a[0], a[1], a[2], a[3]);
      tile[2 * cx + 1][kq] = f32x4_to_e4m3x4(b[0], b[1], b[2], b[3]);
    } else {
      tile[2 * cx][kq] = f32x4_to_s8x4(a[0], a[1], a[2], a[3]);
      tile[2 * cx + 1][kq] = f32x4_to_s8x4(b[0], b[1], b[2], b[3]);
    }
  }
  __syncthreads();
  // 128 columns x 4 groups of 16 reduce-rows: one 16-byte store each
  for (int v = threadIdx.x; v < kTrCols * (kTrRows / 16); v += 256) {
    const int c = v >> 2, g = v & 3;
    const int64_t k = k0 + 16 * g;
    if (c0 + c >= M || k >= Kp) continue;
    const uint32_t n0 = tile[c][4 * g], n1 = tile[c][4 * g + 1], n2 = tile[c][4 * g + 2], n3 = tile[c][4 * g + 3];
    uint4 o;
    if (PERMUTE) {          // every 16 viewed as [2][4][2], first two modes transposed: positions 0-3 = elements 0, 1, 8, 9, ...
      o.x = __byte_perm(n0, n2, 0x5410);
      o.y = __byte_perm(n0, n2, 0x7632);
      o.z = __byte_perm(n1, n3, 0x5410);
      o.w = __byte_perm(n1, n3, 0x7632);
    } else {
      o = make_uint4(n0, n1, n2, n3);
    }
    *reinterpret_cast<uint4 *>(out + (batch * M + c0 + c) * Kp + k) = o;
  }
}

__global__ void colmax_to_scale_kernel(float *__restrict__ sf, const void *__restrict__ scale_max_p, int scale_max_is_int, int64_t M,
                                       int64_t M16, int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float smax = load_scale_max(scale_max_p, scale_max_is_int);
  sf[i] = (i % M16) < M ? __fdiv_rn(sf[i], smax) : 0.0f;
}

template <int FMT>
static int launch_rowwise(void *out, float *sf, const void *in, const void *scale_max, int is_int,
                          const int64_t shape[4], const int64_t stride[4], int swizzle,
                          cudaStream_t stream) {
  if (!shape || !stride) return fail(AC4K_ERR_NULL, "shape/stride is NULL");
  for (int i = 0; i < 4; ++i)
    if (shape[i] < 0) return fail(AC4K_ERR_SHAPE, "shape[%d] is negative", i);
  if (!out || !sf || !scale_max) return fail(AC4K_ERR_NULL, "out/sf/scale_max is NULL");
  const int64_t d1 = shape[1], M = shape[2], K = shape[3];
  const int64_t nbatch = shape[0] * shape[1];
  if (nbatch == 0 || M == 0) return 0;
  if (!in && K > 0) return fail(AC4K_ERR_NULL, "in is NULL");
  if (nbatch > 65535) return fail(AC4K_ERR_SHAPE, "outer dims product %lld exceeds 65535", (long long)nbatch);
  const int64_t M16 = align_up(M, 16);
  const uint16_t *inp = static_cast<const uint16_t *>(in);
  uint8_t *outp = static_cast<uint8_t *>(out);

  const bool vec_ok = !swizzle && stride[3] == 1 && K > 0 && (K % 8 == 0) && (stride[2] % 8 == 0) &&
                      (stride[0] % 8 == 0) && (stride[1] % 8 == 0) &&
                      ((reinterpret_cast<uintptr_t>(in) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(out) & 7) == 0);
  if (vec_ok) {
    if (K <= 32 * 8 * 4) {   // short rows: one warp per row, 8 rows per CTA
      dim3 grid((unsigned)ceil_div(M16, 8), (unsigned)nbatch);
      rowwise_quantize_kernel<FMT, 32, 4><<<grid, 256, 0, stream>>>(outp, sf, inp, scale_max, is_int, M, K,
                                                                   d1, stride[0], stride[1], stride[2]);
    } else {                 // long rows: one CTA per row, 8192 elements cached in registers
      dim3 grid((unsigned)M16, (unsigned)nbatch);
      rowwise_quantize_kernel<FMT, 256, 4><<<grid, 256, 0, stream>>>(outp, sf, inp, scale_max, is_int, M, K,
                                                                    d1, stride[0], stride[1], stride[2]);
    }
    AC4K_LAUNCH_CHECK("rowwise_quantize_kernel");
    return 0;
  }
  // columns contiguous, rows strided: the transposing kernels
  const bool tr_ok = stride[2] == 1 && K > 0 && M % 2 == 0 && stride[3] % 2 == 0 && stride[0] % 2 == 0 && stride[1] % 2 == 0 &&
                     ((reinterpret_cast<uintptr_t>(in) & 3) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) &&
                     ceil_div(K, kTrRows) <= 0x7fffffff && ceil_div(M, kTrCols) <= 65535;
  if (tr_ok) {
    AC4K_CUDA_TRY(cudaMemsetAsync(sf, 0, (size_t)(nbatch * M16) * sizeof(float), stream));
    dim3 g1((unsigned)ceil_div(K, kTrChunk), (unsigned)ceil_div(M, kTrCols), (unsigned)nbatch);
    colmax_kernel<<<g1, 256, 0, stream>>>(sf, inp, M, K, M16, d1, stride[0], stride[1], stride[3]);
    AC4K_LAUNCH_CHECK("colmax_kernel");
    dim3 g2((unsigned)ceil_div(align_up(K, 16), kTrRows), (unsigned)ceil_div(M, kTrCols), (unsigned)nbatch);
    if (swizzle)
      transpose_quantize_kernel<FMT, true><<<g2, 256, 0, stream>>>(outp, sf, inp, scale_max, is_int, M, K, M16, d1, stride[0],
                                                                   stride[1], stride[3]);
    else
      transpose_quantize_kernel<FMT, false><<<g2, 256, 0, stream>>>(outp, sf, inp, scale_max, is_int, M, K, M16, d1, stride[0],
                                                                    stride[1], stride[3]);
    AC4K_LAUNCH_CHECK("transpose_quantize_kernel");
    const int64_t total = nbatch * M16;
    colmax_to_scale_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, stream>>>(sf, scale_max, is_int, M, M16, total);
    AC4K_LAUNCH_CHECK("colmax_to_scale_kernel");
    return 0;
  }
  dim3 grid((unsigned)ceil_div(M16, 8), (unsigned)nbatch);
  if (swizzle)
    rowwise_quantize_strided_kernel<FMT, true><<<grid, 256, 0, stream>>>(
        outp, sf, inp, scale_max, is_int, M, K, d1, stride[0], stride[1], stride[2], stride[3]);
  else
    rowwise_quantize_strided_kernel<FMT, false><<<grid, 256, 0, stream>>>(
        outp, sf, inp, scale_max, is_int, M, K, d1, stride[0], stride[1], stride[2], stride[3]);
  AC4K_LAUNCH_CHECK("rowwise_quantize_strided_kernel");
  return 0;
}

}  // namespace ac4k

using namespace ac4k;

extern "C" int ac4k_quantize_fp8(void *out, float *sf, const void *in, const float *scale_max,
                                 const int64_t shape[4], const int64_t stride[4], int swizzle,
                                 ac4k_stream_t stream) {
  return launch_rowwise<kFmtE4M3>(out, sf, in, scale_max, 0, shape, stride, swizzle,
                                  static_cast<cudaStream_t>(stream));
}

extern "C" int ac4k_quantize_int8(void *out, float *sf, const void *in, const int32_t *scale_max,
                                  const int64_t shape[4], const int64_t stride[4],
                                  ac4k_stream_t stream) {
  return launch_rowwise<kFmtS8>(out, sf, in, scale_max, 1, shape, stride, 0,
                                static_cast<cudaStream_t>(stream));
}
