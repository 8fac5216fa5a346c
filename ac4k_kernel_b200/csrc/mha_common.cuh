// Arithmetic helpers shared by the attention kernels (mha_nvfp4.cu, mha_int8_fp8.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ac4k {

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
// 2^x for two x (<= 8) on the FMA and integer pipes, for the share of the exponentials that the ex2 pipe (16 per clock per
// SM, the bottleneck of the attention kernels) is relieved of: x = n + f with n = round(x), |f| <= 1/2; 2^f from a quartic with
// relative error < 2.8e-6 (near-minimax on [-1/2, 1/2]; a cubic's 7.5e-5 moved enough roundings of the 4-bit P to show
// against the CPU restatement on short sequences); n is added to the exponent field.  x is clamped at -125, where
// the result (2.4e-38) is far below anything that survives the 4-bit quantisation of P or moves the row sum.
__device__ __forceinline__ float2 exp2_fma_pipe(float2 x) {
  constexpr float kMagic = 12582912.0f;        // 1.5 * 2^23: x + kMagic holds round(x) in its low mantissa bits
  x.x = fmaxf(x.x, -125.0f);
  x.y = fmaxf(x.y, -125.0f);
  const float2 fi = fadd2(x, make_float2(kMagic, kMagic));
  const float2 n = fadd2(fi, make_float2(-kMagic, -kMagic));
  const float2 f = ffma2(n, make_float2(-1.0f, -1.0f), x);
  float2 q = ffma2(f, make_float2(0.00957010128f, 0.00957010128f), make_float2(0.0559178591f, 0.0559178591f));
  q = ffma2(q, f, make_float2(0.240247443f, 0.240247443f));
  q = ffma2(q, f, make_float2(0.693121791f, 0.693121791f));
  q = ffma2(q, f, make_float2(0.999999285f, 0.999999285f));
  return make_float2(__int_as_float(__float_as_int(q.x) + (__float_as_int(fi.x) << 23)),
                     __int_as_float(__float_as_int(q.y) + (__float_as_int(fi.y) << 23)));
}
}  // namespace ac4k
