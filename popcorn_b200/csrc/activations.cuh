// fp32 gate functions shared by the SwiGLU / GEGLU kernels and the gated RMSNorm.
#pragma once

#include "common.cuh"

namespace b200 {

// Two ways to evaluate silu(a) = a / (1 + exp(-a)) in fp32:
//  MATH 0  expf and an IEEE division: the reference's own operation sequence.
//          About 32 instructions per element in total, which makes the bf16
//          kernel issue-bound (0.78 of the HBM roofline on a B200).
//  MATH 1  exp(-a) = 2^t with t = fp32(-a*log2(e)): the hardware ex2
//          approximation, corrected to first order for the rounding of t and
//          for the low bits of log2(e); the quotient from the reciprocal
//          approximation plus one Newton step (exact remainder, one fused
//          multiply-add).  About 20 instructions per element, HBM-bound, and on
//          the full 32768 x 14336 bf16 configuration bit-identical to MATH 0
//          and to the PyTorch CPU reference (the rounding of silu to bf16
//          hides the last-bit fp32 differences).
// 16-bit dtypes use MATH 1; fp32, whose results are not rounded again, uses MATH 0.
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
template <int MATH>
__device__ __forceinline__ float exp_neg(float a) {
  if constexpr (MATH == 0) {
    return expf(-a);
  } else {
    constexpr float kNegLog2e = -1.4426950216293335f;       // fp32(-log2(e))
    constexpr float kNegLog2eLo = -1.9259629911266175e-8f;  // -log2(e) - fp32(-log2(e))
    // |a| <= 88 keeps every intermediate finite (exp(88) < 2^127); beyond that the quotient
    // below is 0 or a itself whatever the exponential is.  A NaN a becomes -88 here and is
    // restored by the multiplication with a in silu_f32.
    const float ac = fminf(fmaxf(a, -88.0f), 88.0f);
    const float t = __fmul_rn(ac, kNegLog2e);
    float lo = __fmaf_rn(ac, kNegLog2e, -t);  // what the rounding of t dropped
    lo = __fmaf_rn(ac, kNegLog2eLo, lo);
    const float e = ex2_approx(t);
    return __fmaf_rn(e, __fmul_rn(lo, 0.6931471805599453f), e);  // 2^(t + lo) ~ 2^t * (1 + lo*ln 2)
  }
}
// Argument t of the gate x / (1 + exp(-t)): t = x gives silu(x); t = 2*sqrt(2/pi)*(x + 0.044715*x^3)
// gives the tanh-approximate gelu, since 0.5*(1 + tanh(u)) = 1 / (1 + exp(-2u)).
enum Act { kSilu = 0, kGeluTanh = 1, kSigmoidGate = 2 };  // kSigmoidGate: the gate is sigmoid(x) itself, not x * sigmoid(t)
template <int ACT>
__device__ __forceinline__ float gate_argument(float x) {
  if constexpr (ACT == kSilu) {
    return x;
  } else {
    const float cube = __fmul_rn(__fmul_rn(x, x), x);
    const float inner = __fmul_rn(0.7978845608028654f, __fadd_rn(x, __fmul_rn(0.044715f, cube)));
    return __fmul_rn(2.0f, inner);
  }
}

template <int MATH, int ACT = kSilu>
__device__ __forceinline__ float silu_f32(float a) {
  const float d = __fadd_rn(1.0f, exp_neg<MATH>(gate_argument<ACT>(a)));
  if constexpr (MATH == 0) {
    return __fdiv_rn(a, d);
  } else {
    const float r = rcp_approx(d);  // 0 once d exceeds 2^126
    const float q = __fmul_rn(a, r);
    const float rem = __fmaf_rn(-q, d, a);
    const float q1 = __fmaf_rn(rem, r, q);
    // a = +inf: q = inf is the answer and the remainder is NaN.  a = -inf: d >= 2^126, the
    // reciprocal flushes to 0 and q = -inf * 0 = NaN, as in the reference (-inf / inf).
    return (rem != rem) ? q : q1;
  }
}


// sigmoid(x) = 1 / (1 + exp(-x)) with the same two evaluation modes.
template <int MATH>
__device__ __forceinline__ float sigmoid_f32(float x) {
  const float d = __fadd_rn(1.0f, exp_neg<MATH>(x));
  if constexpr (MATH == 0) {
    return __fdiv_rn(1.0f, d);
  } else {
    const float r = rcp_approx(d);                       // 0 once d exceeds 2^126
    return __fmaf_rn(__fmaf_rn(-r, d, 1.0f), r, r);      // one Newton step; exact 0 stays 0
  }
}

}  // namespace b200
