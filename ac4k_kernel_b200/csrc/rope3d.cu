// 3-D rotary position embedding for sm_100a: out[b, s, n, 2c : 2c + 2] = x[b, s, n, 2c : 2c + 2] * freq (complex), where
// position s of a [F, H, W] grid takes its C = D / 2 complex factors from three rows of one table: pairs [0, c1) from
// row f, [c1, c1 + c2) from row h, the rest from row w (c2 = C / 3, c1 = C - 2 c2).  Stands in for ac4k_kernel's
// lib/cuda/sm120/rope3d.cu:23-129 (kernel) and :133-187 (checks) behind the same binding (lib/cuda_bindings.cc:91-97).
//
// Arithmetic as in the reference: bf16 -> fp64, the four products and two sums in fp64 (no fused multiply-add), -> fp32
// -> bf16, so results equal the reference's Python oracle (test/test_rope_3d_apply.py:14-42) bit for bit.  One
// difference, deliberate: positions behind the grid (s >= F * H * W) are copied through, which is what that oracle
// returns; the reference's kernel leaves them unwritten.
//
// HBM-bound: 4 bytes of traffic per element.  The reference runs one thread per (position, head) row over 256-byte
// rows with scalar loads and re-reads 64 table entries per row; here one CTA walks whole positions (all heads, N * D
// contiguous elements) with 16-byte loads and stores.  When C divides 4 * 256 (the usual head dimensions) a thread
// meets the same four pairs in every vector it handles and keeps the position's four factors in registers; otherwise
// the position's C factors are staged in shared memory once.
#include <algorithm>
#include <climits>

#include "common.cuh"

namespace ac4k {

static constexpr int kRopeThreads = 256;
static constexpr int kRopeCtasPerSm = 5;     // 48 registers per thread; the grid is this many CTAs per SM
static constexpr int kRopeMaxC = 1024;      // complex pairs per head staged in shared memory (D <= 2048)

__device__ __forceinline__ uint32_t rope_pair(uint32_t xy, double2 f) {
  const double xr = (double)__uint_as_float(xy << 16), xi = (double)__uint_as_float(xy & 0xffff0000u);
  const double re = __dsub_rn(__dmul_rn(xr, f.x), __dmul_rn(xi, f.y));
  const double im = __dadd_rn(__dmul_rn(xr, f.y), __dmul_rn(xi, f.x));
  const __nv_bfloat162 o = __floats2bfloat162_rn((float)re, (float)im);
  return *reinterpret_cast<const uint32_t *>(&o);
}

// row of the table that pair c of a position takes
__device__ __forceinline__ int rope_row(int c, int c1, int c2, int fi, int hi, int wi) { return c < c1 ? fi : (c < c1 + c2 ? hi : wi); }

// MODE 0: 16-byte accesses, and a thread meets the same four pairs in every vector it handles (4 * threads % C == 0):
//         the position's factors live in registers, nothing is shared, warps run free of one another.
// MODE 1: 16-byte accesses, the position's C factors staged in shared memory (two CTA barriers per position).
// MODE 2: one pair per access (D % 8 != 0 or tensors not 16-byte aligned), factors in shared memory.
template <int MODE>
__global__ void __launch_bounds__(kRopeThreads, kRopeCtasPerSm) rope3d_kernel(const uint16_t *__restrict__ x, const int32_t *__restrict__ grid_sizes,
                                                               const double2 *__restrict__ freqs, uint16_t *__restrict__ out,
                                                               int64_t BS, int S, int N, int D, int C, int max_pos) {
  __shared__ double2 sf[MODE == 0 ? 1 : kRopeMaxC];
  const int c2 = C / 3, c1 = C - 2 * c2;
  const int64_t row_elems = (int64_t)N * D;
  const int c0 = (int)((threadIdx.x * 4) % C);                  // MODE 0: this thread's four pairs
  grid_dependency_wait();
  for (int64_t ps = blockIdx.x; ps < BS; ps += gridDim.x) {
    const int b = (int)(ps / S), pos = (int)(ps % S);
    const int F = __ldg(grid_sizes + 3 * b), H = __ldg(grid_sizes + 3 * b + 1), W = __ldg(grid_sizes + 3 * b + 2);
    const uint16_t *src = x + ps * row_elems;
    uint16_t *dst = out + ps * row_elems;
    const bool inside = (int64_t)pos < (int64_t)F * H * W;       // warp- and CTA-uniform
    // rows of the table for this position (an index past the table reads its last row instead of faulting)
    const int hw = max(H * W, 1), wd = max(W, 1);
    const int fi = min(pos / hw, max_pos - 1), hi = min((pos % hw) / wd, max_pos - 1), wi = min(pos % wd, max_pos - 1);
    if (MODE == 0) {
      double2 f[4];
      if (inside) {
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = __ldg(freqs + (int64_t)rope_row(c0 + i, c1, c2, fi, hi, wi) * C + c0 + i);
      }
      const int64_t nvec = row_elems / 8;
      const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
      uint4 *d4 = reinterpret_cast<uint4 *>(dst);
      for (int64_t v = threadIdx.x; v < nvec; v += kRopeThreads) {
        uint4 q = __ldcs(s4 + v);
        if (inside) {
          q.x = rope_pair(q.x, f[0]);
          q.y = rope_pair(q.y, f[1]);
          q.z = rope_pair(q.z, f[2]);
          q.w = rope_pair(q.w, f[3]);
        }
        __stcs(d4 + v, q);
      }
      continue;
    }
    if (inside) {
      __syncthreads();                                            // the previous position's factors are no longer read
      for (int c = threadIdx.x; c < C; c += kRopeThreads) sf[c] = __ldg(freqs + (int64_t)rope_row(c, c1, c2, fi, hi, wi) * C + c);
      __syncthreads();
    }
    if (MODE == 1) {
      const int64_t nvec = row_elems / 8;
      const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
      uint4 *d4 = reinterpret_cast<uint4 *>(dst);
      for (int64_t v = threadIdx.x; v < nvec; v += kRopeThreads) {
        uint4 q = __ldcs(s4 + v);
        if (inside) {
          const int cv = (int)((v * 4) % C);                      // first of this vector's four pairs
          q.x = rope_pair(q.x, sf[cv]);
          q.y = rope_pair(q.y, sf[cv + 1]);
          q.z = rope_pair(q.z, sf[cv + 2]);
          q.w = rope_pair(q.w, sf[cv + 3]);
        }
        __stcs(d4 + v, q);
      }
    } else {
      const int64_t npair = row_elems / 2;
      for (int64_t v = threadIdx.x; v < npair; v += kRopeThreads) {
        uint32_t q = (uint32_t)src[2 * v] | ((uint32_t)src[2 * v + 1] << 16);
        if (inside) q = rope_pair(q, sf[(int)(v % C)]);
        dst[2 * v] = (uint16_t)q;
        dst[2 * v + 1] = (uint16_t)(q >> 16);
      }
    }
  }
  grid_launch_dependents();
}

}  // namespace ac4k

using namespace ac4k;

extern "C" int ac4k_rope3d(void *out, const void *x, const int32_t *grid_sizes, const void *freqs, int64_t B, int64_t S,
                           int64_t N, int64_t D, int64_t max_pos, ac4k_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (B < 0 || S < 0 || N < 0 || D < 0 || max_pos < 0) return fail(AC4K_ERR_SHAPE, "negative dimension");
  if (D % 2) return fail(AC4K_ERR_SHAPE, "the feature dimension must be even (complex pairs), got %lld", (long long)D);
  if (B == 0 || S == 0 || N == 0 || D == 0) return 0;
  if (!out || !x || !grid_sizes || !freqs) return fail(AC4K_ERR_NULL, "a required pointer is NULL");
  if (max_pos == 0) return fail(AC4K_ERR_SHAPE, "the frequency table is empty");
  if (D / 2 > kRopeMaxC) return fail(AC4K_ERR_UNSUPPORTED, "feature dimensions up to %d are built, got %lld", 2 * kRopeMaxC, (long long)D);
  if (S > INT32_MAX || N > INT32_MAX || max_pos > INT32_MAX || B > INT32_MAX) return fail(AC4K_ERR_SHAPE, "dimension too large");
  if ((reinterpret_cast<uintptr_t>(out) & 1) || (reinterpret_cast<uintptr_t>(x) & 1) || (reinterpret_cast<uintptr_t>(grid_sizes) & 3) ||
      (reinterpret_cast<uintptr_t>(freqs) & 15))
    return fail(AC4K_ERR_ALIGN, "x/out must be 2-byte, grid_sizes 4-byte and freqs 16-byte aligned");
  DeviceInfo di;
  if (int e = get_device_info(&di)) return e;
  const int64_t BS = B * S;
  const unsigned blocks = (unsigned)std::min<int64_t>(BS, (int64_t)di.sms * kRopeCtasPerSm);
  const bool vec = (D % 8 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  const int mode = !vec ? 2 : ((kRopeThreads * 4) % (D / 2) == 0 ? 0 : 1);
  const uint16_t *xp = static_cast<const uint16_t *>(x);
  uint16_t *op = static_cast<uint16_t *>(out);
  const double2 *fp = static_cast<const double2 *>(freqs);
  if (mode == 0)
    rope3d_kernel<0><<<blocks, kRopeThreads, 0, stream>>>(xp, grid_sizes, fp, op, BS, (int)S, (int)N, (int)D, (int)(D / 2), (int)max_pos);
  else if (mode == 1)
    rope3d_kernel<1><<<blocks, kRopeThreads, 0, stream>>>(xp, grid_sizes, fp, op, BS, (int)S, (int)N, (int)D, (int)(D / 2), (int)max_pos);
  else
    rope3d_kernel<2><<<blocks, kRopeThreads, 0, stream>>>(xp, grid_sizes, fp, op, BS, (int)S, (int)N, (int)D, (int)(D / 2), (int)max_pos);
  AC4K_LAUNCH_CHECK("rope3d_kernel");
  return 0;
}
