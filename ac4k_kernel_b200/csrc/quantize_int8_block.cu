// Block-of-tokens INT8 quantiser of the INT8 x FP8 attention path: x[b, h, n, :] bf16 (any strides) ->
// y[b, h, n, align16(D)] int8 and one fp32 scale per block of `block` consecutive tokens (all D features):
//   scale = max|x| / 127 over the block,  y = trunc(x / scale)  (0 when the block is all zero), padding columns 0.
// Optionally x is first reduced by a bf16 vector per head, x - sub rounded to bf16 (the reference takes the mean over
// the tokens off K with a tensor subtraction of its own, attention.py:157: one pass over K less).
// Stands in for the Triton kernel and its wrapper in ac4k_kernel's python/ac4k_kernel/ops/attention.py:18-48 and
// :51-99 (`tl.cast(fp32 -> int8)` truncates toward zero; the division is a true fp32 division).
//
// One CTA per (token block, head, batch entry): the block (at most 128 x 256 bf16) is read once,
// reduced to its maximum through shared memory, and written back as bytes.  HBM traffic 2 + 1 bytes per element.
// Three kernels: the block staged in shared memory by a TMA load (features a multiple of 8 and at most 256, aligned
// strides: the usual case), 16-byte vectors held in registers, single elements for anything else.
#include <algorithm>

#include "gemm_common.cuh"

namespace ac4k {

static constexpr int kQ8Threads = 256;
static constexpr int kQ8MaxElemsPerThread = 128;     // 128 tokens x 256 features / 256 threads

// EPT: elements per thread, >= block * align16(D) / 256
template <int EPT>
__global__ void __launch_bounds__(kQ8Threads) quantize_int8_block_kernel(
    int8_t *__restrict__ y, float *__restrict__ scale, const uint16_t *__restrict__ x, int N, int D, int Dp, int block, int nblk,
    int64_t sb, int64_t sh, int64_t sn, int64_t sd, int H, const uint16_t *__restrict__ sub, int64_t ub, int64_t uh) {
  __shared__ float red[kQ8Threads / 32];
  const int blk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n0 = blk * block;
  const int rows = min(block, N - n0);
  const uint16_t *src = x + b * sb + h * sh;
  const int total = block * Dp;                       // elements of the output tile, padding columns included
  float v[EPT];
  float amax = 0.0f;
  grid_dependency_wait();
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int e = i * kQ8Threads + threadIdx.x;       // consecutive threads take consecutive features
    v[i] = 0.0f;
    if (e < total) {
      const int r = e / Dp, c = e - r * Dp;
      if (r < rows && c < D) {
        v[i] = __uint_as_float((uint32_t)__ldg(src + (int64_t)(n0 + r) * sn + (int64_t)c * sd) << 16);
        if (sub != nullptr)      // x - sub rounded to bf16, as a bf16 tensor subtraction gives it
          v[i] = __bfloat162float(__float2bfloat16_rn(v[i] - __uint_as_float((uint32_t)__ldg(sub + b * ub + h * uh + c) << 16)));
        amax = fmaxf(amax, fabsf(v[i]));
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < kQ8Threads / 32; ++w) amax = fmaxf(amax, red[w]);
  const float s = __fdiv_rn(amax, 127.0f);
  if (threadIdx.x == 0) scale[((int64_t)b * H + h) * nblk + blk] = s;
  int8_t *dst = y + (((int64_t)b * H + h) * N + n0) * Dp;
#pragma unroll
  for (int i = 0; i < EPT; ++i) {
    const int e = i * kQ8Threads + threadIdx.x;
    if (e < rows * Dp) dst[e] = s == 0.0f ? (int8_t)0 : (int8_t)__float2int_rz(__fdiv_rn(v[i], s));
  }
  grid_launch_dependents();
}

// The usual case: features contiguous, D a multiple of 8, rows 16-byte aligned.  A thread takes 16-byte vectors of eight
// features (consecutive threads = consecutive vectors of a row, then the next row), keeps them packed in registers,
// and writes eight bytes per vector.  VPT: vectors per thread, >= block * D / 8 / 256.
template <int VPT>
__global__ void __launch_bounds__(kQ8Threads) quantize_int8_block_vec_kernel(
    int8_t *__restrict__ y, float *__restrict__ scale, const uint16_t *__restrict__ x, int N, int D, int Dp, int block, int nblk,
    int64_t sb, int64_t sh, int64_t sn, int H, const uint16_t *__restrict__ sub, int64_t ub, int64_t uh) {
  __shared__ float red[kQ8Threads / 32];
  const int blk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n0 = blk * block;
  const int rows = min(block, N - n0);
  const uint16_t *src = x + b * sb + h * sh + (int64_t)n0 * sn;
  const int vpr = D / 8, vpr_out = Dp / 8;            // vectors per input row / per output row (padding included)
  const int nvec = rows * vpr_out;
  uint4 v[VPT];
  __nv_bfloat162 am2 = __floats2bfloat162_rn(0.0f, 0.0f);
  grid_dependency_wait();
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int e = i * kQ8Threads + threadIdx.x;
    v[i] = make_uint4(0u, 0u, 0u, 0u);
    if (e < nvec) {
      const int r = e / vpr_out, c = e - r * vpr_out;
      if (c < vpr) {
        v[i] = __ldcs(reinterpret_cast<const uint4 *>(src + (int64_t)r * sn) + c);
        __nv_bfloat162 *h2 = reinterpret_cast<__nv_bfloat162 *>(&v[i]);
        if (sub != nullptr) {      // x - sub rounded to bf16, as a bf16 tensor subtraction gives it
          const uint4 u = __ldg(reinterpret_cast<const uint4 *>(sub + b * ub + h * uh) + c);
          const __nv_bfloat162 *u2 = reinterpret_cast<const __nv_bfloat162 *>(&u);
#pragma unroll
          for (int k = 0; k < 4; ++k) h2[k] = __hsub2(h2[k], u2[k]);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) am2 = __hmax2(am2, __habs2(h2[k]));
      }
    }
  }
  float amax = fmaxf(__low2float(am2), __high2float(am2));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < kQ8Threads / 32; ++w) amax = fmaxf(amax, red[w]);
  const float s = __fdiv_rn(amax, 127.0f);
  if (threadIdx.x == 0) scale[((int64_t)b * H + h) * nblk + blk] = s;
  uint2 *dst = reinterpret_cast<uint2 *>(y + (((int64_t)b * H + h) * N + n0) * Dp);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int e = i * kQ8Threads + threadIdx.x;
    if (e < nvec) {
      const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
      uint32_t o[2] = {0u, 0u};
      if (s != 0.0f) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float f = __uint_as_float((k & 1) ? (w[k >> 1] & 0xffff0000u) : (w[k >> 1] << 16));
          o[k >> 2] |= ((uint32_t)__float2int_rz(__fdiv_rn(f, s)) & 0xffu) << (8 * (k & 3));
        }
      }
      __stcs(dst + e, make_uint2(o[0], o[1]));
    }
  }
  grid_launch_dependents();
}

// Eight elements of a 16-byte vector -> eight int8 codes trunc(RN(f / s)), |f / s| <= 127, without a division or a
// float -> int conversion per element (both run on the 16-per-clock pipe, which bounds the kernel otherwise).  With
// rs = RN(1 / s), t = f * rs is within 1.5 * 2^-23 * |f / s| < 2.3e-5 of the correctly rounded quotient, so the two
// truncate alike unless t lies that close to an integer.  floor(|t|) comes from adding 2^23 with round-down, its
// fraction is exact, and the code is the low byte of sign(t) * floor(|t|) + 1.5 * 2^23 (two's complement for free).
// Returns false - and the caller takes the true division for the whole vector - if any fraction is within 1e-4 of an
// integer (zero, infinities and NaNs included).
__device__ __forceinline__ bool quantize8_by_reciprocal(const uint4 &v, float rs, uint32_t (&o)[2]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t m[8];
  bool ok = true;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float f = __uint_as_float((k & 1) ? (w[k >> 1] & 0xffff0000u) : (w[k >> 1] << 16));
    const float t = __fmul_rn(f, rs);
    const float fl = __fsub_rn(__fadd_rd(fabsf(t), 8388608.0f), 8388608.0f);
    const float frac = __fsub_rn(fabsf(t), fl);
    ok = ok && (fabsf(__fsub_rn(frac, 0.5f)) < 0.4999f);
    m[k] = __float_as_uint(__fadd_rn(copysignf(fl, t), 12582912.0f));
  }
  o[0] = __byte_perm(__byte_perm(m[0], m[1], 0x0040), __byte_perm(m[2], m[3], 0x0040), 0x5410);
  o[1] = __byte_perm(__byte_perm(m[4], m[5], 0x0040), __byte_perm(m[6], m[7], 0x0040), 0x5410);
  return ok;
}

// The same quantiser with the block staged in shared memory by one TMA load (a box of D features x `block` tokens of the
// [B, H, N, D] tensor, whatever its strides; tokens past N arrive as zeros): no thread holds the block in registers
// while it is in flight, so seven CTAs fit on an SM instead of four and the loads of all of them are outstanding at
// once.  D a multiple of 8 and at most 256, strides multiples of 8 elements, base 16-byte aligned.
__global__ void __launch_bounds__(kQ8Threads) quantize_int8_block_tma_kernel(
    const __grid_constant__ CUtensorMap tmap, int8_t *__restrict__ y, float *__restrict__ scale, int N, int D, int Dp, int block,
    int nblk, int H, const uint16_t *__restrict__ sub, int64_t ub, int64_t uh, unsigned int *status, unsigned long long wait_ns) {
  extern __shared__ __align__(128) uint8_t q8_tile[];
  __shared__ __align__(8) uint64_t bar_mem;
  __shared__ float red[kQ8Threads / 32];
  using namespace ptx;
  const int blk = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n0 = blk * block;
  const int rows = min(block, N - n0);
  const uint32_t bar = smem_u32(&bar_mem), tile = smem_u32(q8_tile);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    fence_barrier_init();
  }
  __syncthreads();
  grid_dependency_wait();
  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(bar, (uint32_t)(block * D * 2));     // the whole box, rows past N included (zeros)
    tma_load_4d(tile, &tmap, 0, n0, h, b, bar);
  }
  if (!mbar_wait(bar, 0, wait_ns)) {
    if (threadIdx.x == 0) atomicExch(status, kStatusTimeoutProducer);
    return;
  }
  const int vpr = D / 8, vpr_out = Dp / 8;            // vectors per input row / per output row (padding included)
  const int nvec = rows * vpr_out;
  const int shift = (vpr_out & (vpr_out - 1)) == 0 ? __ffs(vpr_out) - 1 : -1;     // rows of a power of two of vectors
  auto row_col = [&](int e, int &r, int &c) {
    if (shift >= 0) { r = e >> shift; c = e & (vpr_out - 1); }
    else { r = e / vpr_out; c = e - r * vpr_out; }
  };
  const uint16_t *subp = sub != nullptr ? sub + b * ub + h * uh : nullptr;
  auto load_vec = [&](int r, int c) {
    uint4 v;
    asm volatile("ld.shared::cta.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(tile + (uint32_t)(r * D + c * 8) * 2u));
    if (subp != nullptr) {      // x - sub rounded to bf16, as a bf16 tensor subtraction gives it
      __nv_bfloat162 *h2 = reinterpret_cast<__nv_bfloat162 *>(&v);
      const uint4 u = __ldg(reinterpret_cast<const uint4 *>(subp) + c);
      const __nv_bfloat162 *u2 = reinterpret_cast<const __nv_bfloat162 *>(&u);
#pragma unroll
      for (int k = 0; k < 4; ++k) h2[k] = __hsub2(h2[k], u2[k]);
    }
    return v;
  };
  __nv_bfloat162 am2 = __floats2bfloat162_rn(0.0f, 0.0f);
  for (int e = threadIdx.x; e < nvec; e += kQ8Threads) {
    int r, c;
    row_col(e, r, c);
    if (c < vpr) {
      const uint4 v = load_vec(r, c);
      const __nv_bfloat162 *h2 = reinterpret_cast<const __nv_bfloat162 *>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) am2 = __hmax2(am2, __habs2(h2[k]));
    }
  }
  float amax = fmaxf(__low2float(am2), __high2float(am2));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < kQ8Threads / 32; ++w) amax = fmaxf(amax, red[w]);
  const float s = __fdiv_rn(amax, 127.0f);
  const float rs = __frcp_rn(s);
  if (threadIdx.x == 0) scale[((int64_t)b * H + h) * nblk + blk] = s;
  uint2 *dst = reinterpret_cast<uint2 *>(y + (((int64_t)b * H + h) * N + n0) * Dp);
  for (int e = threadIdx.x; e < nvec; e += kQ8Threads) {
    int r, c;
    row_col(e, r, c);
    uint32_t o[2] = {0u, 0u};
    if (c < vpr && s != 0.0f) {
      const uint4 v = load_vec(r, c);
      if (!quantize8_by_reciprocal(v, rs, o)) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        o[0] = o[1] = 0u;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float f = __uint_as_float((k & 1) ? (w[k >> 1] & 0xffff0000u) : (w[k >> 1] << 16));
          o[k >> 2] |= ((uint32_t)__float2int_rz(__fdiv_rn(f, s)) & 0xffu) << (8 * (k & 3));
        }
      }
    }
    __stcs(dst + e, make_uint2(o[0], o[1]));
  }
  grid_launch_dependents();
}

}  // namespace ac4k

using namespace ac4k;

extern "C" int ac4k_quantize_int8_block(void *out, float *scale, const void *in, const int64_t shape[4], const int64_t stride[4],
                                        int64_t block, const void *sub, const int64_t sub_stride[2], ac4k_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!shape || !stride) return fail(AC4K_ERR_NULL, "shape/stride is NULL");
  const int64_t B = shape[0], H = shape[1], N = shape[2], D = shape[3];
  if (B < 0 || H < 0 || N < 0 || D < 0) return fail(AC4K_ERR_SHAPE, "negative dimension");
  if (block < 16 || block > 128 || (block & (block - 1))) return fail(AC4K_ERR_SHAPE, "the token block must be a power of two in [16, 128], got %lld", (long long)block);
  if (B == 0 || H == 0 || N == 0 || D == 0) return 0;
  if (!out || !scale || !in) return fail(AC4K_ERR_NULL, "out/scale/in is NULL");
  const int64_t Dp = align_up(D, 16);
  if (block * Dp > (int64_t)kQ8MaxElemsPerThread * kQ8Threads)
    return fail(AC4K_ERR_UNSUPPORTED, "block x align16(D) up to %d elements is built, got %lld x %lld", kQ8MaxElemsPerThread * kQ8Threads,
                (long long)block, (long long)Dp);
  if (H > 65535 || B > 65535 || N > INT32_MAX) return fail(AC4K_ERR_SHAPE, "dimension too large");
  if ((reinterpret_cast<uintptr_t>(in) & 1) || (reinterpret_cast<uintptr_t>(scale) & 3)) return fail(AC4K_ERR_ALIGN, "in must be 2-byte and scale 4-byte aligned");
  if (sub && !sub_stride) return fail(AC4K_ERR_NULL, "sub_stride is NULL");
  const uint16_t *subp = static_cast<const uint16_t *>(sub);
  const int64_t ub = sub ? sub_stride[0] : 0, uh = sub ? sub_stride[1] : 0;
  const int64_t nblk = ceil_div(N, block);
  dim3 grid((unsigned)nblk, (unsigned)H, (unsigned)B);
  const bool vec = stride[3] == 1 && D % 8 == 0 && stride[0] % 8 == 0 && stride[1] % 8 == 0 && stride[2] % 8 == 0 &&
                   (reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 7) == 0 &&
                   (!sub || ((reinterpret_cast<uintptr_t>(sub) & 15) == 0 && ub % 8 == 0 && uh % 8 == 0));
  // the TMA-staged kernel: additionally D <= 256 (one box row), and a device of compute capability 10
  if (vec && D <= 256 && stride[2] > 0) {
    DeviceInfo di;
    if (int e = get_device_info(&di)) return e;
    CUtensorMap tm;
    if (di.cc_major == 10 && get_tmap_bf16_4d(in, shape, stride, (int)block, &tm) == 0) {
      unsigned int *status = device_status_ptr();
      if (!status) return fail(AC4K_ERR_DEVICE, "cannot resolve the device status word");
      const size_t smem = (size_t)block * D * 2;
      static PerDevice<int> attr_set;
      int dummy = 0;
      if (int e = attr_set.get(&dummy, [&](int &v) {
            AC4K_CUDA_TRY(cudaFuncSetAttribute(quantize_int8_block_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 256 * 2));
            v = 1;
            return 0;
          }))
        return e;
      quantize_int8_block_tma_kernel<<<grid, kQ8Threads, smem, stream>>>(tm, static_cast<int8_t *>(out), scale, (int)N, (int)D, (int)Dp,
                                                                         (int)block, (int)nblk, (int)H, subp, ub, uh, status,
                                                                         ptx::kWaitTimeoutNs);
      AC4K_LAUNCH_CHECK("quantize_int8_block_tma_kernel");
      return 0;
    }
  }
  if (vec) {
    const int64_t vpt = ceil_div(block * (Dp / 8), kQ8Threads);
#define AC4K_Q8V_LAUNCH(V)                                                                                                            \
  quantize_int8_block_vec_kernel<V><<<grid, kQ8Threads, 0, stream>>>(static_cast<int8_t *>(out), scale, static_cast<const uint16_t *>(in), \
                                                                      (int)N, (int)D, (int)Dp, (int)block, (int)nblk, stride[0], stride[1],  \
                                                                      stride[2], (int)H, subp, ub, uh)
    if (vpt <= 2) AC4K_Q8V_LAUNCH(2);
    else if (vpt <= 4) AC4K_Q8V_LAUNCH(4);
    else if (vpt <= 8) AC4K_Q8V_LAUNCH(8);
    else AC4K_Q8V_LAUNCH(16);
#undef AC4K_Q8V_LAUNCH
    AC4K_LAUNCH_CHECK("quantize_int8_block_vec_kernel");
    return 0;
  }
  const int64_t ept = ceil_div(block * Dp, kQ8Threads);
#define AC4K_Q8_LAUNCH(E)                                                                                                          \
  quantize_int8_block_kernel<E><<<grid, kQ8Threads, 0, stream>>>(static_cast<int8_t *>(out), scale, static_cast<const uint16_t *>(in), \
                                                                  (int)N, (int)D, (int)Dp, (int)block, (int)nblk, stride[0], stride[1],  \
                                                                  stride[2], stride[3], (int)H, subp, ub, uh)
  if (ept <= 16) AC4K_Q8_LAUNCH(16);
  else if (ept <= 32) AC4K_Q8_LAUNCH(32);
  else if (ept <= 64) AC4K_Q8_LAUNCH(64);
  else AC4K_Q8_LAUNCH(128);
#undef AC4K_Q8_LAUNCH
  AC4K_LAUNCH_CHECK("quantize_int8_block_kernel");
  return 0;
}
