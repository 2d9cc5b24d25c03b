// One element of an element-wise kind on raw 32-bit words: the arithmetic every
// element-wise kernel (and a reduction's finishing kind) shares.  Include only
// from files compiled with -fmad=false: kinds the reference defines as
// separate roundings must keep them.
#pragma once
#include "device_math.cuh"
#include "kinds.h"

namespace b200 {
using namespace kind;

__device__ __forceinline__ void set_err(int* err, int code) {
  if (err) atomicCAS(err, 0, code);
}

// One element of kind K on raw words.  `s1`, `s2` are the op's immediates.
template <uint32_t K>
__device__ __forceinline__ uint32_t ev(uint32_t ua, uint32_t ub, uint32_t uc, float s1, float s2,
                                       int* err) {
  const float a = __uint_as_float(ua), b = __uint_as_float(ub), c = __uint_as_float(uc);
  const int32_t ia = (int32_t)ua, ib = (int32_t)ub;
  const int32_t is = (int32_t)__float_as_uint(s1);
  (void)a; (void)b; (void)c; (void)ia; (void)ib; (void)is; (void)s2; (void)err;
#define F(x) __float_as_uint(x)
#define BOOLW(x) ((x) ? 1u : 0u)
  if constexpr (K == ADD || K == ADD_ROW) return F(a + b);
  else if constexpr (K == SUB) return F(a - b);
  else if constexpr (K == MUL) return F(a * b);
  else if constexpr (K == MUL_SCALAR) return F(a * s1);
  else if constexpr (K == ADD_SCALAR) return F(a + s1);
  else if constexpr (K == RELU) return relu_bits(ua);
  else if constexpr (K == RELU_BACKWARD) return positive_not_nan(ua) ? ub : 0u;
  else if constexpr (K == RECIP) return F(1.0f / a);
  else if constexpr (K == DIV) return F(a / b);
  else if constexpr (K == DIV_SCALAR) return F(a / s1);
  else if constexpr (K == EXP) return F(expf(a));
  else if constexpr (K == LOG) return F(logf(a));
  else if constexpr (K == BOOL_NOT) return BOOLW(ua == 0);
  else if constexpr (K == BOOL_AND) return BOOLW(ua != 0 && ub != 0);
  else if constexpr (K == BOOL_OR) return BOOLW(ua != 0 || ub != 0);
  else if constexpr (K == BOOL_XOR) return BOOLW((ua != 0) != (ub != 0));
  else if constexpr (K == NEG) return ua ^ 0x80000000u;
  else if constexpr (K == ABS) return ua & 0x7fffffffu;
  else if constexpr (K == SIGN) {
    if (a != a) return ua;
    return a > 0.f ? F(1.0f) : (a < 0.f ? F(-1.0f) : 0u);
  } else if constexpr (K == CLAMP) return F(a < s1 ? s1 : (a > s2 ? s2 : a));
  else if constexpr (K == CLAMP_MIN) return F(a != a ? s1 : (s1 != s1 ? a : (a > s1 ? a : s1)));
  else if constexpr (K == CLAMP_MAX) return F(a != a ? s1 : (s1 != s1 ? a : (a < s1 ? a : s1)));
  else if constexpr (K == LEAKY_RELU) return F(a >= 0.f ? a : s1 * a);
  else if constexpr (K == HARD_SIGMOID) {
    float t = s1 * a + s2;
    return F(t < 0.f ? 0.f : (t > 1.f ? 1.f : t));
  } else if constexpr (K == EQ) return BOOLW(a == b);
  else if constexpr (K == NE) return BOOLW(a != b);
  else if constexpr (K == GT) return BOOLW(a > b);
  else if constexpr (K == GE) return BOOLW(a >= b);
  else if constexpr (K == LT) return BOOLW(a < b);
  else if constexpr (K == LE) return BOOLW(a <= b);
  else if constexpr (K == EQ_S) return BOOLW(a == s1);
  else if constexpr (K == NE_S) return BOOLW(a != s1);
  else if constexpr (K == GT_S) return BOOLW(a > s1);
  else if constexpr (K == GE_S) return BOOLW(a >= s1);
  else if constexpr (K == LT_S) return BOOLW(a < s1);
  else if constexpr (K == LE_S) return BOOLW(a <= s1);
  else if constexpr (K == IS_NAN) return BOOLW(a != a);
  else if constexpr (K == IS_INF) return BOOLW((ua & 0x7fffffffu) == 0x7f800000u);
  else if constexpr (K == MASK_FILL || K == INT_MASK_FILL || K == BOOL_MASK_FILL)
    return ub != 0 ? F(s1) : ua;
  else if constexpr (K == MASK_WHERE || K == INT_MASK_WHERE || K == BOOL_MASK_WHERE)
    return ub != 0 ? uc : ua;
  else if constexpr (K == PRELU) return F(a >= 0.f ? a : b * a);
  else if constexpr (K == FILL) return F(s1);
  else if constexpr (K == SQRT) return F(sqrtf(a));
  else if constexpr (K == RSQRT) return F(1.0f / sqrtf(a));
  else if constexpr (K == LOG1P) return F(log1pf(a));
  else if constexpr (K == POW) return F(powf(a, b));
  else if constexpr (K == POW_S) return F(powf(a, s1));
  else if constexpr (K == POW_I) return F(powf(a, (float)ib));
  else if constexpr (K == I32_TO_F32 || K == BOOL_TO_F32) return F((float)ia);
  else if constexpr (K == BOOL_TO_I32) return ua;
  else if constexpr (K == INDEX_TO_I32) return (uint32_t)__float2int_rz(a);
  else if constexpr (K == INT_ABS) return ia < 0 ? (uint32_t)0 - ua : ua;
  else if constexpr (K == EXPM1) return F(expm1f(a));
  else if constexpr (K == SIGMOID) return F(sigmoid_flex(a));
  else if constexpr (K == SIGMOID_BACKWARD) return F((b * a) * (1.0f - a));
  else if constexpr (K == TANH) return F(tanhf(a));
  else if constexpr (K == ERF) return F(erff(a));
  else if constexpr (K == GELU) return F(gelu_erf(a));
  else if constexpr (K == GELU_TANH) return F(gelu_tanh(a));
  else if constexpr (K == GELU_BACKWARD) {
    // g (Phi(a) + a phi(a))
    float cdf = 0.5f * (1.0f + erff(a * 0.70710678118654752440f));
    float pdf = 0.39894228040143267794f * expf(-0.5f * a * a);
    return F(b * (cdf + a * pdf));
  } else if constexpr (K == SINH) return F(sinhf(a));
  else if constexpr (K == COSH) return F(coshf(a));
  else if constexpr (K == ASINH) return F(asinhf(a));
  else if constexpr (K == ACOSH) return F(acoshf(a));
  else if constexpr (K == ATANH) return F(atanhf(a));
  else if constexpr (K == LOG_SIGMOID) {
    // ln(sigmoid a) = -(max(-a,0) + log1p(exp(-|a|)))
    float m = a < 0.f ? -a : 0.f;
    return F(-(m + log1pf(expf(-fabsf(a)))));
  } else if constexpr (K == LOG_SIGMOID_BACKWARD) return F(b * sigmoid_flex(-a));
  else if constexpr (K == SIN) return F(sinf(a));
  else if constexpr (K == COS) return F(cosf(a));
  else if constexpr (K == TAN) return F(tanf(a));
  else if constexpr (K == ATAN) return F(atanf(a));
  else if constexpr (K == ATAN2) return F(atan2f(a, b));
  else if constexpr (K == ASIN) return F(asinf(a));
  else if constexpr (K == ACOS) return F(acosf(a));
  else if constexpr (K == REM) return F(fmodf(fmodf(a, b) + b, b));
  else if constexpr (K == REM_S) return F(fmodf(fmodf(a, s1) + s1, s1));
  else if constexpr (K == ROUND) return F(rintf(a));
  else if constexpr (K == FLOOR) return F(floorf(a));
  else if constexpr (K == CEIL) return F(ceilf(a));
  else if constexpr (K == TRUNC) return F(truncf(a));
  else if constexpr (K == F32_TO_I32) return (uint32_t)__float2int_rz(a);  // saturates, NaN -> 0
  else if constexpr (K == POW2_FLOOR) return ua & 0x7f800000u;
  else if constexpr (K == POW2_FLOOR_INV) {
    uint32_t e = ua & 0x7f800000u;
    return e >= 0x7f000000u ? 0x00800000u : 0x7f000000u - e;
  } else if constexpr (K == INT_ADD) return ua + ub;
  else if constexpr (K == INT_SUB) return ua - ub;
  else if constexpr (K == INT_MUL) return ua * ub;
  else if constexpr (K == INT_AND) return ua & ub;
  else if constexpr (K == INT_OR) return ua | ub;
  else if constexpr (K == INT_XOR) return ua ^ ub;
  else if constexpr (K == INT_SHL) return ua << (ub & 31);
  else if constexpr (K == INT_SHR) return (uint32_t)(ia >> (ub & 31));
  else if constexpr (K == INT_EQ) return BOOLW(ia == ib);
  else if constexpr (K == INT_NE) return BOOLW(ia != ib);
  else if constexpr (K == INT_GT) return BOOLW(ia > ib);
  else if constexpr (K == INT_GE) return BOOLW(ia >= ib);
  else if constexpr (K == INT_LT) return BOOLW(ia < ib);
  else if constexpr (K == INT_LE) return BOOLW(ia <= ib);
  else if constexpr (K == INT_NOT) return ~ua;
  else if constexpr (K == INT_ADD_S) return ua + (uint32_t)is;
  else if constexpr (K == INT_SUB_S) return ua - (uint32_t)is;
  else if constexpr (K == INT_MUL_S) return ua * (uint32_t)is;
  else if constexpr (K == INT_AND_S) return ua & (uint32_t)is;
  else if constexpr (K == INT_OR_S) return ua | (uint32_t)is;
  else if constexpr (K == INT_XOR_S) return ua ^ (uint32_t)is;
  else if constexpr (K == INT_SHL_S) return ua << (is & 31);
  else if constexpr (K == INT_SHR_S) return (uint32_t)(ia >> (is & 31));
  else if constexpr (K == INT_EQ_S) return BOOLW(ia == is);
  else if constexpr (K == INT_NE_S) return BOOLW(ia != is);
  else if constexpr (K == INT_GT_S) return BOOLW(ia > is);
  else if constexpr (K == INT_GE_S) return BOOLW(ia >= is);
  else if constexpr (K == INT_LT_S) return BOOLW(ia < is);
  else if constexpr (K == INT_LE_S) return BOOLW(ia <= is);
  else if constexpr (K == INT_DIV || K == INT_DIV_S || K == INT_REM || K == INT_REM_S) {
    const int32_t d = (K == INT_DIV || K == INT_REM) ? ib : is;
    if (d == 0) { set_err(err, 6 /* DOMAIN */); return 0u; }
    if (d == -1) return (K == INT_DIV || K == INT_DIV_S) ? (uint32_t)0 - ua : 0u;  // wrapping
    return (K == INT_DIV || K == INT_DIV_S) ? (uint32_t)(ia / d) : (uint32_t)(ia % d);
  } else if constexpr (K == ADD_RELU) return relu_bits(F(a + b));
  else if constexpr (K == SILU) return F(a * sigmoid_flex(a));
  else if constexpr (K == SILU_MUL) return F((a * sigmoid_flex(a)) * b);
  else if constexpr (K == SUB_EXP) return F(expf(a - b));
  else if constexpr (K == MUL_ADD) return F(c + a * b);
  else if constexpr (K == SCALE_MASK_FILL) return ub != 0 ? F(s2) : F(a * s1);
  else return 0u;
#undef F
#undef BOOLW
}

}  // namespace b200
