// Scalar device helpers shared by the kernel files.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// Sixteen bytes stored once at a multicast address (an NVLS multicast object that maps the same buffer of every
// GPU of a group): the NVSwitch delivers the store to every GPU bound to the object, so a rank that owes its
// tile to g ranks sends it over its links once, not g - 1 times.  A store only: nothing is loaded through the address.
__device__ __forceinline__ void st_multicast_16(void* addr, uint4 v) {
  asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(addr), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// "positive and not NaN" on raw bits: the test the reference's relu family uses
// (crates/tt-kernels/src/sfpu/ops.rs:3877-3906): relu(NaN) = 0, relu(-0) = +0.
__device__ __forceinline__ bool positive_not_nan(uint32_t u) {
  return u != 0u && u <= 0x7f800000u;
}
__device__ __forceinline__ uint32_t relu_bits(uint32_t u) { return positive_not_nan(u) ? u : 0u; }

// BF16 narrowing as the reference defines it (crates/tt-kernels/src/bf16.rs:1-4;
// model at crates/tt-tests/tests/step270_native_bf16.rs:244-255): ties to even,
// NaNs quieted keeping sign and high payload, results below 2^-126 to signed zero.
__device__ __forceinline__ uint16_t f32_to_bf16_bits(uint32_t x) {
  uint32_t r;
  if ((x & 0x7fffffffu) > 0x7f800000u) r = x | 0x00400000u;
  else r = x + 0x7fffu + ((x >> 16) & 1u);
  r &= 0xffff0000u;
  if ((r & 0x7fffffffu) < 0x00800000u) r &= 0x80000000u;
  return (uint16_t)(r >> 16);
}
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t h) {
  return __uint_as_float((uint32_t)h << 16);
}

// burn-flex's sigmoid: two branches on the sign, one exp(-|x|)
// (crates/tt-kernels/src/sfpu/ops.rs:772-775).
__device__ __forceinline__ float sigmoid_flex(float x) {
  const float e = expf(-fabsf(x));
  const float d = 1.0f + e;
  return (x >= 0.f) ? (1.0f / d) : (e / d);
}

// 0.5 x (1 + erf(x / sqrt 2))  (crates/tt-kernels/src/sfpu/ops.rs:135)
// 1 + erf(z) is taken as erfc(-z): for x well below zero the sum would cancel and lose
// the relative accuracy the contract asks for.
__device__ __forceinline__ float gelu_erf(float x) {
  return (0.5f * x) * erfcf(-x * 0.70710678118654752440f);
}
// 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
// 0.5 (1 + tanh y) = sigmoid(2y), which keeps its relative accuracy for y << 0.
// The argument t = 2 sqrt(2/pi) (x + 0.044715 x^3) reaches 11 at |x| = 4 and exp(-t) multiplies every relative error of t
// by t, so an F32 t (three roundings and a rounded constant) would cost some 30 units in the last place of the result.
// t is therefore formed in F64 and handed to the exponential as an F32 head and tail: exp(-(h + l)) = exp(-h) (1 - l).
__device__ __forceinline__ float gelu_tanh(float x) {
  const double xd = (double)x;
  const double t = 1.5957691216057308 * xd * (1.0 + 0.044715 * xd * xd);
  const double a = fmin(fabs(t), 128.0);   // exp(-128) is already 0 in F32; the bound keeps the head finite (a NaN t gives 128, x itself carries the NaN)
  const float ah = (float)a;
  const float al = (float)(a - (double)ah);
  float e = expf(-ah);
  e = e - e * al;
  const float d = 1.0f + e;
  return x * ((t >= 0.0) ? (1.0f / d) : (e / d));
}

// One BFP8 datum under its group's exponent, as BF16 bits: crates/tt-isa/src/tile.rs:619-634 (`bfp8_to_bf16`), line for line.
__device__ __forceinline__ uint16_t bfp8_to_bf16_bits(uint32_t datum, uint32_t exp_bits) {
  const uint32_t sign = datum >> 7;
  uint32_t mag = (datum << 1) & 0xffu;
  if (mag == 0) return sign ? 0xff80u : 0u;
  const uint32_t lz = __clz(mag) - 24;
  mag = (mag << lz) & 0xffu;
  const uint32_t e = (exp_bits - lz) & 0xffu;   // `ExpBits -= LZ` on a uint8_t: it wraps
  return (uint16_t)((sign << 15) | (e << 7) | (mag & 0x7eu));
}
__device__ __forceinline__ float bfp8_value(uint32_t datum, uint32_t exp_bits) {
  return __uint_as_float((uint32_t)bfp8_to_bf16_bits(datum, exp_bits) << 16);
}

}  // namespace b200
