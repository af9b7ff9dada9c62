// Arithmetic helpers of the softmax warps of the prefill kernels: exponentials on two pipes, two float32 lanes per
// instruction, three-input maxima.
#pragma once

#include <cuda_bf16.h>

#include "common.cuh"

namespace relux {

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// ---- two float32 lanes per instruction (add / fma on a 64-bit register pair) ----
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// 2^x for two arguments on the FMA pipe instead of the special-function unit (which delivers 16 exponentials per clock
// and SM: 1024 clocks for the 128 x 128 scores of a tile, as long as the tile's MMAs).  x = n + f with n the nearest
// integer (magic-number rounding) and f in [-1/2, 1/2]; 2^f by a cubic (relative error 7.5e-5, well inside the bf16
// rounding of P); n goes into the exponent field.  x is clamped to [-126, ..): results stay normal numbers.
__device__ __forceinline__ uint64_t ex2_poly2(uint64_t x2) {
  float x0, x1;
  unpack2(x2, x0, x1);
  x2 = pack2(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
  const uint64_t magic = pack2(12582912.f, 12582912.f), neg_magic = pack2(-12582912.f, -12582912.f), neg_one = pack2(-1.f, -1.f);
  const uint64_t t2 = add2(x2, magic);            // low mantissa bits = n (two's complement)
  const uint64_t n2 = add2(t2, neg_magic);
  const uint64_t f2 = fma2(n2, neg_one, x2);
  uint64_t p2 = fma2(pack2(0.0551716648f, 0.0551716648f), f2, pack2(0.2426111251f, 0.2426111251f));
  p2 = fma2(p2, f2, pack2(0.6932609677f, 0.6932609677f));
  p2 = fma2(p2, f2, pack2(0.9999280572f, 0.9999280572f));
  float t0, t1, p0, p1;
  unpack2(t2, t0, t1);
  unpack2(p2, p0, p1);
  p0 = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
  p1 = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
  return pack2(p0, p1);
}

// exp2(score * scale - max) for 32 consecutive scores of one row: bf16 P values, two per 32-bit word in key order, into
// pw; the two partial row sums are added to ps2.  kPoly: kPolyPairs pairs of every eight take the polynomial (a row with
// masked keys among the 32 must not: ex2(-inf) = 0 exactly, the polynomial clamps).
template <bool kPoly, int kPolyPairs>
__device__ __forceinline__ void exp_chunk32(const uint32_t (&sv)[32], uint64_t scale2, uint64_t neg_m2, uint32_t (&pw)[16], uint64_t& ps2) {
#pragma unroll
  for (int c = 0; c < 32; c += 2) {
    const uint64_t x2 = fma2(pack2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), scale2, neg_m2);
    uint64_t p2;
    if (kPoly && ((c >> 1) & 7) < kPolyPairs) {
      p2 = ex2_poly2(x2);
    } else {
      float x0, x1;
      unpack2(x2, x0, x1);
      p2 = pack2(ex2_approx(x0), ex2_approx(x1));
    }
    ps2 = add2(ps2, p2);
    float p0, p1;
    unpack2(p2, p0, p1);
    __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
    pw[c >> 1] = *reinterpret_cast<uint32_t*>(&b2);
  }
}

}  // namespace relux
