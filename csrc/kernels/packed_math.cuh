// Small arithmetic helpers for the softmax loops of the attention kernels: the
// sm_100 two-wide fp32 instructions (fma / mul / add on register pairs), the
// three-input max, the bare ex2 approximation, a polynomial 2^x that keeps off the
// special-function unit, and two-at-a-time conversions to 16-bit.  They exist to cut the instruction count per score element; the
// results equal the scalar forms up to the documented ex2.approx error.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace ft {
namespace pm {

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}

__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// 2^x for a pair of values on the fma pipe instead of the special-function unit: n = round(x) by
// the 1.5 * 2^23 addition, a cubic for 2^(x - n) on [-0.5, 0.5] (relative error 7.5e-5, far below
// the rounding of the 16-bit value the result becomes), n added into the exponent field.  x is
// clamped to -126 from below; there is no upper guard (callers overwrite what they mask).
__device__ __forceinline__ void ex2_poly2(float x0, float x1, float& y0, float& y1) {
  const float kMagic = 12582912.f;
  const uint64_t x = pack2(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
  const uint64_t t = add2(x, pack2(kMagic, kMagic));
  const uint64_t n = add2(t, pack2(-kMagic, -kMagic));
  const uint64_t f = fma2(n, pack2(-1.f, -1.f), x);
  uint64_t p = fma2(pack2(0.0551716685f, 0.0551716685f), f, pack2(0.2426111251f, 0.2426111251f));
  p = fma2(p, f, pack2(0.6932609677f, 0.6932609677f));
  p = fma2(p, f, pack2(0.9999280572f, 0.9999280572f));
  float p0, p1, t0, t1;
  unpack2(p, p0, p1);
  unpack2(t, t0, t1);
  y0 = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
  y1 = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
}

// Two floats -> one 32-bit word of two 16-bit values, `lo` in the low half.
template <typename T>
__device__ __forceinline__ uint32_t cvt2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t cvt2<__nv_bfloat16>(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
template <>
__device__ __forceinline__ uint32_t cvt2<__half>(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

}  // namespace pm
}  // namespace ft
