// Shared host/device helpers for the sm_100a NVFP4 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "ac4k_b200.h"

namespace ac4k {

// ---- host-side error plumbing -----------------------------------------------------------
void set_last_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);     // records the message, returns code
int cuda_fail(cudaError_t e, const char *what);

#define AC4K_CUDA_TRY(expr)                                                     \
  do {                                                                          \
    cudaError_t _e = (expr);                                                    \
    if (_e != cudaSuccess) return ::ac4k::cuda_fail(_e, #expr);                 \
  } while (0)

#define AC4K_LAUNCH_CHECK(what)                                                 \
  do {                                                                          \
    cudaError_t _e = cudaGetLastError();                                        \
    if (_e != cudaSuccess) return ::ac4k::cuda_fail(_e, what);                  \
  } while (0)

// A value that is computed once per CUDA device (devices 0 - 63), by whichever thread needs it first:
// get() runs `init(value)` under std::call_once for the current device and hands the value out afterwards.
// An init that fails is not retried; its return code is given to every later caller.
template <typename T>
struct PerDevice {
  std::once_flag once[64];
  T value[64] = {};
  int status[64] = {};
  template <typename F>
  int get(T *out, F &&init) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(AC4K_ERR_DEVICE, "device index %d out of range", dev);
    std::call_once(once[dev], [&] { status[dev] = init(value[dev]); });
    if (status[dev] != 0) return fail(status[dev], "per-device set-up failed earlier with code %d", status[dev]);
    *out = value[dev];
    return 0;
  }
};

// SM count and compute capability of the current device (queried once per device)
struct DeviceInfo { int sms = 0; int cc_major = 0; bool ok = false; };
int get_device_info(DeviceInfo *out);

// Address of the device status word of the current device (one per device, lives in this
// library's module); kernels with bounded waits receive it as an argument.  NULL on error.
unsigned int *device_status_ptr();

// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization
// attribute may start while the kernel before it in the stream is still running; it must execute
// grid_dependency_wait() before it touches memory that the earlier kernel reads or writes (the wait
// returns at once if the kernel was launched normally).  grid_launch_dependents() lets the NEXT
// kernel of the stream be scheduled onto SMs as this grid's CTAs leave them.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- small integer helpers --------------------------------------------------------------
__host__ __device__ constexpr int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ constexpr int64_t align_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

// ---- conversions (device) ---------------------------------------------------------------
// 8 fp32 -> 8 e2m1 packed in a 32-bit word, element 2j in the low nibble of byte j.
// `cvt.rn.satfinite.e2m1x2.f32 d, a, b` puts a in the HIGH nibble, b in the low one.
__device__ __forceinline__ uint32_t f32x8_to_e2m1x8(const float (&v)[8]) {
  uint32_t r;
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3};\n"
      "}"
      : "=r"(r)
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
  return r;
}

// 4 fp32 -> 4 e4m3 (RNE, satfinite), element 0 in the low byte.
__device__ __forceinline__ uint32_t f32x4_to_e4m3x4(float a, float b, float c, float d) {
  uint32_t r;
  asm("{\n"
      ".reg .b16 lo, hi;\n"
      "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n"
      "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n"
      "mov.b32 %0, {lo, hi};\n"
      "}"
      : "=r"(r)
      : "f"(a), "f"(b), "f"(c), "f"(d));
  return r;
}

// one fp32 (>= 0) -> e4m3 byte and its exact fp32 value
__device__ __forceinline__ uint8_t f32_to_e4m3(float s, float &back) {
  uint16_t p;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(p) : "f"(0.0f), "f"(s));
  uint8_t b = (uint8_t)(p & 0xFF);
  __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  back = __half2float(__half(h));
  return b;
}

__device__ __forceinline__ int8_t f32_to_s8_rni_sat(float x) {
  int r;
  asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(x));
  return (int8_t)r;
}

// 4 fp32 -> 4 int8 (round to nearest even, saturating), element 0 in the low byte.  The float ->
// s32 conversions clamp and map NaN to 0 exactly like cvt.rni.sat.s8.f32 does; cvt.pack saturates
// two s32 to s8, puts them in the low half-word (first operand in the upper byte) and moves the low
// half-word of its third operand to the top: 6 instructions for 4 values instead of 4 conversions
// plus shifts, masks and ors.
__device__ __forceinline__ uint32_t f32x4_to_s8x4(float a, float b, float c, float d) {
  uint32_t r;
  asm("{\n"
      ".reg .s32 ia, ib, ic, id;\n"
      ".reg .b32 hi;\n"
      "cvt.rni.s32.f32 ia, %1;\n cvt.rni.s32.f32 ib, %2;\n cvt.rni.s32.f32 ic, %3;\n cvt.rni.s32.f32 id, %4;\n"
      "cvt.pack.sat.s8.s32.b32 hi, id, ic, 0;\n"
      "cvt.pack.sat.s8.s32.b32 %0, ib, ia, hi;\n"
      "}"
      : "=r"(r)
      : "f"(a), "f"(b), "f"(c), "f"(d));
  return r;
}

// |x| of two packed bf16 (clears the sign bits), max of packed bf16 pairs
__device__ __forceinline__ uint32_t abs_bf16x2(uint32_t v) { return v & 0x7FFF7FFFu; }
__device__ __forceinline__ uint32_t max_bf16x2(uint32_t a, uint32_t b) {
  __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162 *>(&a);
  __nv_bfloat162 y = *reinterpret_cast<__nv_bfloat162 *>(&b);
  __nv_bfloat162 m = __hmax2(x, y);
  return *reinterpret_cast<uint32_t *>(&m);
}
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t lo16) { return __uint_as_float(lo16 << 16); }
// max of the two halves of an abs'd bf16x2 word, as fp32
__device__ __forceinline__ float hmax_bf16x2_to_f32(uint32_t v) {
  uint32_t a = v & 0xFFFFu, b = v >> 16;   // non-negative bf16: integer order == value order
  return bf16_bits_to_f32(a > b ? a : b);
}

// ---- NVFP4 block quantisation (shared by the quantiser and the GEMM's re-quantising epilogue) ----
static constexpr float kOneSixth = 0.16666667163372040f;

struct BlockScale {
  float r;       // multiplier applied to the elements
  uint8_t byte;  // e4m3 scale
};

__device__ __forceinline__ BlockScale block_scale(float amax, float alpha) {
  BlockScale o;
  float s = __fmul_rn(alpha, __fmul_rn(amax, kOneSixth));
  float sf_f;
  o.byte = f32_to_e4m3(s, sf_f);
  o.r = (sf_f != 0.0f) ? __fmul_rn(alpha, __frcp_rn(sf_f)) : 0.0f;
  return o;
}

__device__ __forceinline__ float load_alpha(const float *gscale) {
  float g = __ldg(gscale);
  return g == 0.0f ? 0.0f : __frcp_rn(g);
}

// four packed bf16 pairs -> 8 e2m1 codes (one word); products in fp32, round to nearest
__device__ __forceinline__ uint32_t quantize8_x2(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, float r) {
  uint32_t out;
  asm("{\n"
      ".reg .b64 rr, p0, p1, p2, p3;\n"
      ".reg .b32 l0, l1, l2, l3, h0, h1, h2, h3;\n"
      ".reg .f32 x0, x1, x2, x3, y0, y1, y2, y3;\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "mov.b64 rr, {%5, %5};\n"
      "shl.b32 l0, %1, 16;\n and.b32 h0, %1, 0xFFFF0000;\n mov.b64 p0, {l0, h0};\n"
      "shl.b32 l1, %2, 16;\n and.b32 h1, %2, 0xFFFF0000;\n mov.b64 p1, {l1, h1};\n"
      "shl.b32 l2, %3, 16;\n and.b32 h2, %3, 0xFFFF0000;\n mov.b64 p2, {l2, h2};\n"
      "shl.b32 l3, %4, 16;\n and.b32 h3, %4, 0xFFFF0000;\n mov.b64 p3, {l3, h3};\n"
      "mul.rn.f32x2 p0, p0, rr;\n mul.rn.f32x2 p1, p1, rr;\n"
      "mul.rn.f32x2 p2, p2, rr;\n mul.rn.f32x2 p3, p3, rr;\n"
      "mov.b64 {x0, y0}, p0;\n mov.b64 {x1, y1}, p1;\n mov.b64 {x2, y2}, p2;\n mov.b64 {x3, y3}, p3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, y0, x0;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b1, y1, x1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, y2, x2;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b3, y3, x3;\n"
      "mov.b32 %0, {b0, b1, b2, b3};\n"
      "}"
      : "=r"(out)
      : "r"(w0), "r"(w1), "r"(w2), "r"(w3), "f"(r));
  return out;
}

// amax of 16 packed bf16 values (8 words) as fp32
__device__ __forceinline__ float amax16_bf16(const uint32_t *w) {
  const uint32_t m = max_bf16x2(max_bf16x2(max_bf16x2(abs_bf16x2(w[0]), abs_bf16x2(w[1])),
                                           max_bf16x2(abs_bf16x2(w[2]), abs_bf16x2(w[3]))),
                                max_bf16x2(max_bf16x2(abs_bf16x2(w[4]), abs_bf16x2(w[5])),
                                           max_bf16x2(abs_bf16x2(w[6]), abs_bf16x2(w[7]))));
  return hmax_bf16x2_to_f32(m);
}

}  // namespace ac4k
