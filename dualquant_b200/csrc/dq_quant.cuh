// Per-token int4 quantiser arithmetic shared by every kernel that produces activation codes
// (the stand-alone quantisers and the decode kernel that quantises in its own prologue), so that
// all of them emit bit-identical scales and codes.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace dq {

__device__ __forceinline__ float round_to_bf16(float v) {
  unsigned short bits;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(bits) : "f"(v));
  return __uint_as_float(static_cast<uint32_t>(bits) << 16);
}

// Flag in the scale_fp16 argument of the quantisers: codes are written as E4M3 bytes of the same
// integers (the operand format of the FP8-path prefill GEMM) instead of int8.
constexpr int kCodesE4M3 = 0x100;

// scale_fp16 (low byte): 0 = fp32 scale, 1 = scale rounded to fp16, 2 = "bf16 arithmetic": the quantiser as
// torch evaluates it on a bf16 tensor (every intermediate rounded to bf16), which is what the
// reference's PermLinear does when there is neither an activation scale nor an online Hadamard
// (activations/perm_linear.py:131-133 with formats/rtn_int.py:62-67).
__device__ __forceinline__ float token_scale(float amax, int scale_fp16) {
  scale_fp16 &= 0xFF;
  float s = __fdiv_rn(amax, 7.0f);
  if (scale_fp16 == 2) s = round_to_bf16(s);
  if (amax == 0.f) s = 1.0f;
  if (scale_fp16 == 1) {
    s = __half2float(__float2half_rn(fminf(s, 65504.0f)));
    if (s == 0.f) s = 1.0f;
  }
  return s;
}

// clamp(rint(v / s), -8, 7) with v / s correctly rounded, i.e. bit-identical to the IEEE
// division, at a fraction of its instruction count: t = v * (1/s) is within 2 ulp of the true
// quotient, so rint(t) can only differ from rint(v / s) when t lies within a few ulp of a
// half-integer (|t| <= ~7 here, 4 ulp < 4e-6); only those rare elements take the exact division.
// Rounding and the float -> int step avoid the conversion instructions (quarter-rate pipe; at
// prefill sizes this kernel is bound by instruction issue, not by memory): adding and subtracting
// 1.5 * 2^23 rounds to the nearest integer, ties to even, for |t| < 2^22, and the low byte of the
// bit pattern of (q + 1.5 * 2^23) is q as a two's-complement int8.
constexpr float kRoundMagic = 12582912.0f;
// Eight codes at once.  The fast estimate runs for all of them; only if one of them lies within
// reach of a rounding boundary (or the estimate is not finite) does the thread redo all eight with
// the IEEE division - in a branch of its own, so that the division sequence stays out of the
// common path instead of being predicated into it.
__device__ __forceinline__ void quant_codes8(const float* v, float s, float inv_s, float* q) {
  bool exact = false;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float t = __fmul_rn(v[e], inv_s);
    const float qe = __fsub_rn(__fadd_rn(t, kRoundMagic), kRoundMagic);
    const float dist = fabsf(fabsf(__fsub_rn(t, qe)) - 0.5f);
    // the negated comparison also catches a NaN or infinite estimate (1/s overflowed for a denormal
    // scale): t - qe is then NaN.  A finite estimate of any size rounds correctly above (beyond 2^22
    // it is an integer already) and is clamped below.
    exact |= !(dist >= 1e-5f);
    q[e] = fminf(fmaxf(qe, -8.0f), 7.0f);
  }
  if (exact) {
#pragma unroll
    for (int e = 0; e < 8; ++e) q[e] = fminf(fmaxf(rintf(__fdiv_rn(v[e], s)), -8.0f), 7.0f);
  }
}
// The same in bf16 arithmetic: the quotient is rounded to bf16 before it is rounded to an integer.
__device__ __forceinline__ void quant_codes8_bf16(const float* v, float s, float* q) {
#pragma unroll
  for (int e = 0; e < 8; ++e)
    q[e] = fminf(fmaxf(rintf(round_to_bf16(__fdiv_rn(v[e], s))), -8.0f), 7.0f);
}
// four codes in [-8, 7] (as floats) -> four int8 in one word, first code in the low byte
__device__ __forceinline__ uint32_t pack_codes4(float q0, float q1, float q2, float q3) {
  const uint32_t u0 = __float_as_uint(__fadd_rn(q0, kRoundMagic));
  const uint32_t u1 = __float_as_uint(__fadd_rn(q1, kRoundMagic));
  const uint32_t u2 = __float_as_uint(__fadd_rn(q2, kRoundMagic));
  const uint32_t u3 = __float_as_uint(__fadd_rn(q3, kRoundMagic));
  return __byte_perm(__byte_perm(u0, u1, 0x0040), __byte_perm(u2, u3, 0x0040), 0x5410);
}
// the same four codes as E4M3 bytes (integers up to 8 are exact in E4M3; -0 is stored as +0)
__device__ __forceinline__ uint32_t pack_codes4_e4m3(float q0, float q1, float q2, float q3) {
  unsigned short lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(__fadd_rn(q1, 0.f)), "f"(__fadd_rn(q0, 0.f)));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(__fadd_rn(q3, 0.f)), "f"(__fadd_rn(q2, 0.f)));
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

}  // namespace dq
