/*
 * ac4k_b200.h - C ABI of ac4k_kernel's operators on B200 (sm_100a): the NVFP4 linear path
 * (quantisers and block-scaled GEMM), the two attention kernels and 3-D RoPE.
 *
 * A shared library exporting these symbols replaces the compiled half of ac4k_kernel's
 * `_cuda_ops` extension (all seven functions of lib/cuda_bindings.cc:37-97).  Every entry point takes raw
 * device pointers, sizes and a CUDA stream; no torch types cross the boundary.  The file
 * and line given with each declaration is the reference interface it stands in for
 * (paths inside the ac4k_kernel project).
 *
 * Conventions
 *   - return value: 0 = success; < 0 = rejected argument (see AC4K_ERR_*); > 0 = the
 *     cudaError_t / CUresult reported by the runtime.  Nothing throws, nothing exits.
 *     `ac4k_last_error()` returns a thread-local message for the last non-zero return.
 *   - all work is enqueued on `stream` and is asynchronous; the caller owns every buffer and
 *     must keep it alive until the stream reaches that point.  Outputs are fully written,
 *     padding included (callers allocate them uninitialised, like the reference's Python).
 *   - `shape`/`stride` describe the bf16 input as a 4-D view ordered
 *     [outer0, outer1, cross (M), reduce (K)], strides in elements; lower ranks are padded
 *     with leading 1s, exactly like quantize_nvfp4.cu:226-241 does after its checks.
 *   - scale-factor layouts for NVFP4:
 *       AC4K_SF_AC4K      [.., ceil(K/64), align16(M), 4]   the reference's wire format
 *                         (quantize_nvfp4.cu:56-60,150-155)
 *       AC4K_SF_TILE128X4 [.., ceil(M/128), ceil(K/64), 32, 4, 4]  the 512-byte tiles that
 *                         `tcgen05.cp.32x128b.warpx4` copies to tensor memory unchanged
 *                         (the un-layout is test/utils.py:15-23)
 */
#ifndef AC4K_B200_H_
#define AC4K_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *ac4k_stream_t; /* cudaStream_t */

enum {
  AC4K_OK = 0,
  AC4K_ERR_NULL = -1,        /* required pointer is NULL                       */
  AC4K_ERR_SHAPE = -2,       /* negative / inconsistent sizes                  */
  AC4K_ERR_ALIGN = -3,       /* pointer or stride alignment not supported      */
  AC4K_ERR_ENUM = -4,        /* unknown dtype / layout code                    */
  AC4K_ERR_UNSUPPORTED = -5, /* valid in the reference, not built here         */
  AC4K_ERR_DEVICE = -6,      /* current device is not an sm_100 part           */
  AC4K_ERR_TIMEOUT = -7      /* returned by ac4k_device_status only: a bounded device-side
                                wait of an earlier launch gave up                          */
};

enum { AC4K_SF_AC4K = 0, AC4K_SF_TILE128X4 = 1 };
enum { AC4K_DT_BF16 = 0, AC4K_DT_FP16 = 1, AC4K_DT_FP32 = 2 };

/* Library identity: mirrors the module attributes of lib/cuda_bindings.cc:41-44. */
const char *ac4k_arch(void);             /* "sm100" */
const char *ac4k_arch_description(void);
const char *ac4k_backend(void);          /* "cuda"  */
const char *ac4k_version(void);          /* "0.1.0" */
const char *ac4k_last_error(void);

/* Device-side status word of the current device: 0, or the code left by a kernel whose
 * bounded wait expired (0xA1 TMA producer, 0xA2 MMA issuer, 0xA3 scale warps, 0xA4 epilogue).
 * Synchronises the device.  `clear` != 0 resets the word.  Returns AC4K_ERR_TIMEOUT when such a code is
 * found, 0 when the word is 0.  Launches are asynchronous, so an entry point that enqueued the kernel has
 * long returned 0 by then: this call is the only place where an expired wait is reported, and the outputs of
 * the launch that left the code are undefined.  Every device-side wait (mbarrier, flag) is bounded (2 s) and
 * the kernel leaves through its normal exit, releasing tensor memory, so the context stays usable. */
int ac4k_device_status(uint32_t *status_out, int clear);

/* g_out[0] = max|x| / max_scale over `numel` contiguous bf16 values (0 for numel == 0).
 * Replaces `_global_scale` + `_triton_global_scale_kernel`,
 * python/ac4k_kernel/ops/quant.py:21-59. */
int ac4k_global_scale_bf16(const void *x, int64_t numel, float max_scale, float *g_out,
                           ac4k_stream_t stream);

/* bf16 -> packed e2m1 + e4m3 block scales, given the fp32 global scale on the device.
 * Replaces ac4k::quantize_nvfp4, include/ac4k_kernel/ops.h:27-29 and
 * lib/cuda/sm120/quantize_nvfp4.cu:164-271.
 *   out: [outer0, outer1, M, align64(K)/2] bytes;  sf: see layouts above. */
int ac4k_quantize_nvfp4(void *out, void *sf, const void *in, const float *global_scale,
                        const int64_t shape[4], const int64_t stride[4], int swizzle,
                        int sf_layout, ac4k_stream_t stream);

/* Per-row (whole reduce dim) e4m3 quantiser.  Replaces ac4k::quantize_fp8,
 * include/ac4k_kernel/ops.h:31-33, lib/cuda/sm120/quantize_fp8.cu:192-290.
 *   out: [outer0, outer1, M, align16(K)] e4m3;  sf: [outer0, outer1, align16(M)] fp32. */
int ac4k_quantize_fp8(void *out, float *sf, const void *in, const float *scale_max,
                      const int64_t shape[4], const int64_t stride[4], int swizzle,
                      ac4k_stream_t stream);

/* Per-row int8 quantiser (scale_max is an int32 on the device).  Replaces
 * ac4k::quantize_int8, include/ac4k_kernel/ops.h:35-37,
 * lib/cuda/sm120/quantize_int8.cu:175-262. */
int ac4k_quantize_int8(void *out, float *sf, const void *in, const int32_t *scale_max,
                       const int64_t shape[4], const int64_t stride[4],
                       ac4k_stream_t stream);

/* D[M,N] = cast((A_gs*B_gs) * A_fp4[M,K] * B_fp4[N,K]^T + bias[N]).
 * Replaces ac4k::linear_nvfp4, include/ac4k_kernel/ops.h:43-48,
 * lib/cuda/sm120/linear_nvfp4.cu:753-901.
 *   A: [M, K/2] bytes, B: [N, K/2] bytes, K a multiple of 64 (what the quantiser emits);
 *   A_sf/B_sf in `sf_layout`; A_gs/B_gs: device fp32 scalars; bias: NULL or N values of
 *   `bias_dtype`; D row-major contiguous of `d_dtype`. */
int ac4k_linear_nvfp4(void *D, int d_dtype, const void *A, const void *A_sf,
                      const float *A_gs, const void *B, const void *B_sf, const float *B_gs,
                      const void *bias, int bias_dtype, int64_t M, int64_t N, int64_t K,
                      int sf_layout, ac4k_stream_t stream);

/* Same computation and arguments as ac4k_linear_nvfp4, for callers that must not allocate device
 * memory while running (a plugin living inside someone else's fixed memory budget, a serving loop
 * that forbids allocator calls).  No counterpart in the reference, which never needs scratch.
 *
 * Where ac4k_linear_nvfp4 would take split-K scratch from the stream-ordered allocator, this entry
 * point uses a fixed 8 MiB array inside the library's device image (every GPU that loads the
 * library holds those 8 MiB until the process exits).  It calls no cudaMalloc / cudaFree of any
 * kind.  Shapes whose split-K partial sums ([K slices, M, N] fp32) need more than 8 MiB are
 * rejected with AC4K_ERR_SHAPE and a message; shapes that need no scratch run as usual.
 *
 *  - The first call on each device that needs scratch looks up the array's device address (device
 *    must be current); make such a call before starting any stream capture.
 *  - All calls share the one array and it keeps whatever the last call left in it.  Nothing in
 *    it needs clearing: each call overwrites every partial sum it later reads.  Two calls that
 *    can overlap on the GPU (different streams) would race on it: serialise them. */
int ac4k_linear_nvfp4_noalloc(void *D, int d_dtype, const void *A, const void *A_sf,
                              const float *A_gs, const void *B, const void *B_sf, const float *B_gs,
                              const void *bias, int bias_dtype, int64_t M, int64_t N, int64_t K,
                              int sf_layout, ac4k_stream_t stream);

/* The GEMM of ac4k_linear_nvfp4 with the all-gather of its output fused into the epilogue: every
 * finished tile is stored to `n_dst` destinations (1..8) instead of one.  No counterpart in the
 * reference, which is single-GPU; this is the exchange step of the column-parallel layer, where
 * rank r owns N of the `ldd` output columns and every rank wants the whole [M, ldd] matrix.
 *   D_dsts[i]: base of a row-major [M, ldd] buffer of `d_dtype` (bf16 or fp16), 16-byte aligned;
 *              entry 0 is normally this GPU's own buffer, the others are peers' buffers mapped into
 *              this process (see ac4k_peer_open).  The launch writes columns
 *              [col_off, col_off + N) of every destination; ldd and col_off are multiples of 8.
 * Every piece of a tile is staged once in shared memory and stored to each destination with one TMA
 * store (bulk tensor store, no multicast; the peers' buffers are reached over NVLink).  The stores are
 * complete when the kernel has finished; a peer may read its buffer after it has synchronised with this
 * GPU's stream past the launch (e.g. a stream-ordered barrier among the ranks).  That barrier orders the
 * reads of step i after the stores of step i - not the stores of step i+1 after a slower rank's reads of
 * step i: callers that launch step after step use two destination sets in turn, or synchronise the ranks
 * once more between the readers of a buffer and the next launch that writes it. */
int ac4k_linear_nvfp4_gather(void *const *D_dsts, int n_dst, int64_t ldd, int64_t col_off, int d_dtype,
                             const void *A, const void *A_sf, const float *A_gs, const void *B,
                             const void *B_sf, const float *B_gs, const void *bias, int bias_dtype,
                             int64_t M, int64_t N, int64_t K, int sf_layout, ac4k_stream_t stream);

/* The GEMM of ac4k_linear_nvfp4 whose epilogue re-quantises the result to NVFP4 instead of storing
 * it: out = quantize_nvfp4(bf16(alpha * A * B^T + bias), out_gs) with blocks of 16 along N, i.e. the
 * activation operand of the next linear layer, bit-identical to running ac4k_linear_nvfp4 (bf16
 * output) followed by ac4k_quantize_nvfp4 with the same global scale.  The reference has no such
 * entry point for the linear path (it re-quantises in registers only inside its attention kernel,
 * lib/cuda/sm120/mha_nvfp4.cu:246-319); this saves the bf16 round trip through HBM and two launches.
 *   out_fp4: [M, N / 2] bytes; out_sf: block scales in `out_sf_layout` ([N/64, align16(M), 4] or
 *   [ceil(M/128), N/64, 32, 4, 4]), padding rows written as 0; out_gs: device fp32 scalar, chosen by
 *   the caller (calibrated), since the amax of the output is not known before the GEMM has run.
 *   N must be a multiple of 64. */
int ac4k_linear_nvfp4_requant(void *out_fp4, void *out_sf, const float *out_gs, int out_sf_layout,
                              const void *A, const void *A_sf, const float *A_gs, const void *B,
                              const void *B_sf, const float *B_gs, const void *bias, int bias_dtype,
                              int64_t M, int64_t N, int64_t K, int sf_layout, ac4k_stream_t stream);

/* O = softmax(sm_scale * Q K^T) V with Q, K, V and the probabilities in NVFP4, bf16 output.
 * Replaces ac4k::mha_nvfp4_fwd, include/ac4k_kernel/ops.h:13-17, lib/cuda_bindings.cc:49-56,
 * lib/cuda/sm120/mha_nvfp4.cu:897-1077 (checks) and :322-893 (kernel).
 *   Q: [B, H, Nq, align64(Dqk)/2] bytes, K: [B, H, Nkv, align64(Dqk)/2] bytes (quantised along the head dimension);
 *   V: [B, H, Dv, align64(Nkv)/2] bytes, quantised along the keys with the K permutation (swizzle = 1);
 *   Q_sf, K_sf, V_sf: block scales of those quantiser calls, all three in `sf_layout` (the tiled layout is
 *   copied as it is; the reference's is re-ordered by one more warp of the kernel);
 *   *_gs: device fp32 scalars; O: bf16, element (b, h, n, d) at O + b*o_stride[0] + h*o_stride[1] + n*o_stride[2] +
 *   d*o_stride[3] (elements), so both the [B, H, N, D] and the permuted [B, N, H, D] outputs of the reference work.
 * Built for Dqk, Dv <= 128 (as the reference) and sm_scale >= 0. */
int ac4k_mha_nvfp4_fwd(void *O, const int64_t o_stride[4], const void *Q, const void *Q_sf, const float *Q_gs,
                       const void *K, const void *K_sf, const float *K_gs, const void *V, const void *V_sf,
                       const float *V_gs, int64_t B, int64_t H, int64_t Nq, int64_t Nkv, int64_t Dqk, int64_t Dv,
                       float sm_scale, int sf_layout, ac4k_stream_t stream);

/* Block-of-tokens INT8 quantiser of the INT8 x FP8 attention path: one fp32 scale = max|x| / 127 per `block`
 * consecutive tokens of a head (all features), y = trunc(x / scale), feature padding to a multiple of 16 written as 0.
 * Replaces the Triton kernel `_triton_block_token_quantize` and `_int8_quantize`,
 * python/ac4k_kernel/ops/attention.py:18-48, :51-99.
 *   in: bf16, logical [B, H, N, D] given by shape[4] = {B, H, N, D} and element strides stride[4] (so both tensor
 *   layouts of the reference work); out: int8 [B, H, N, align16(D)] contiguous; scale: fp32 [B, H, ceil(N / block)].
 *   block: power of two in [16, 128], block * align16(D) <= 32768.
 *   sub: NULL, or bf16 vectors of D contiguous features, one per head at sub + b * sub_stride[0] + h * sub_stride[1]
 *   (elements): x - sub, rounded to bf16 as a bf16 tensor subtraction rounds it, is quantised instead of x (the
 *   reference subtracts the mean over the tokens from K with a torch operation first, attention.py:157). */
int ac4k_quantize_int8_block(void *out, float *scale, const void *in, const int64_t shape[4], const int64_t stride[4],
                             int64_t block, const void *sub, const int64_t sub_stride[2], ac4k_stream_t stream);

/* O = softmax(sm_scale * Q K^T) V with Q, K in INT8 (scales per block of tokens), P and V in FP8 e4m3 (V with one scale
 * per channel), bf16 output.  Replaces ac4k::mha_int8_x_fp8_fwd, include/ac4k_kernel/ops.h:19-25,
 * lib/cuda_bindings.cc:57-58, lib/cuda/sm120/mha_int8_x_fp8.cu:979-1137 (checks) and :403-975 (kernel).
 *   Q: int8 [B, H, Nq, align16(Dqk)], Q_sf: fp32 [B, H, ceil(Nq / q_block)]; K: int8 [B, H, Nkv, align16(Dqk)],
 *   K_sf: fp32 [B, H, ceil(Nkv / k_block)]; V: e4m3 [B, H, Dv, align16(Nkv)], quantised along the keys with the FP8 K
 *   permutation (swizzle = 1) and max_scale 2.25, V_sf: fp32 [B, H, align16(Dv)]; O: bf16 by element strides as in
 *   ac4k_mha_nvfp4_fwd.
 * Built for Dqk, Dv <= 128, q_block and k_block in {16, 32, 64, 128} (the reference's defaults: 64 and 128), sm_scale >= 0; the
 * P V products accumulate in fp32 (the reference: fp16 within a key tile). */
int ac4k_mha_int8_x_fp8_fwd(void *O, const int64_t o_stride[4], const void *Q, const float *Q_sf, int64_t q_block,
                            const void *K, const float *K_sf, int64_t k_block, const void *V, const float *V_sf,
                            int64_t B, int64_t H, int64_t Nq, int64_t Nkv, int64_t Dqk, int64_t Dv, float sm_scale,
                            ac4k_stream_t stream);

/* 3-D rotary position embedding: out[b, s, n, 2c..2c+1] = x[b, s, n, 2c..2c+1] * freqs[row(s, c), c] as complex numbers,
 * row = the position's frame, height or width index in the [F, H, W] grid of its batch entry, by thirds of the C = D / 2
 * pairs (c1 = C - 2 (C / 3) frame pairs, then C / 3 height pairs, then C / 3 width pairs).
 * Replaces ac4k::rope3d, include/ac4k_kernel/ops.h:50-54, lib/cuda_bindings.cc:91-97, lib/cuda/sm120/rope3d.cu:23-187.
 *   x, out: bf16 [B, S, N, D] contiguous; grid_sizes: int32 [B, 3] on the device; freqs: complex128 [max_pos, D / 2].
 * fp64 arithmetic as in the reference.  Positions s >= F * H * W are copied from x (the reference's kernel leaves them
 * unwritten; its Python oracle, test/test_rope_3d_apply.py:14-42, copies them).  A grid index >= max_pos reads the last
 * row of the table.  D even, D <= 2048. */
int ac4k_rope3d(void *out, const void *x, const int32_t *grid_sizes, const void *freqs, int64_t B, int64_t S,
                int64_t N, int64_t D, int64_t max_pos, ac4k_stream_t stream);

/* Device buffers that the other processes of the node can map (CUDA IPC), for the destinations of
 * ac4k_linear_nvfp4_gather.  No counterpart in the reference.
 *   ac4k_peer_alloc: cudaMalloc on the current device + its 64-byte IPC handle.
 *   ac4k_peer_open:  maps a buffer another process allocated (handle received by any host-side
 *                    channel) into this process, enabling peer access; returns its address here.
 *   ac4k_peer_close / ac4k_peer_free: undo the above (close every mapping before the owner frees). */
int ac4k_peer_alloc(int64_t bytes, void **ptr_out, unsigned char handle_out[64]);
int ac4k_peer_open(const unsigned char handle[64], void **ptr_out);
int ac4k_peer_close(void *ptr);
int ac4k_peer_free(void *ptr);

#ifdef __cplusplus
}
#endif
#endif /* AC4K_B200_H_ */
