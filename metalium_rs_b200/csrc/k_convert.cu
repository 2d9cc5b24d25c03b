// Storage conversions beyond the whole-buffer F32 <-> BF16 cast.
//
//  * `cast_block`: `Engine::cast_block` (crates/burn-tt/src/server.rs:137, `Session::cast_block`
//    crates/tt-kernels/src/session.rs:3732): the F32 <-> BF16 conversion of a block of a buffer into a
//    new buffer of the block's dims, bit for bit the whole-buffer cast of those elements.
//  * `cast_f16`: `Engine::cast_f16` (server.rs:779): F32 <-> IEEE binary16 held in two-byte storage.
//    The rule is the reference's integer programs' (crates/tt-kernels/src/fp16.rs:172-176, 271-275):
//    narrowing rounds ties to even on the binary16 grid, subnormal results included, |x| >= 65520 and
//    infinity give infinity, a NaN keeps its sign and its top ten payload bits and is made quiet;
//    widening is exact, a NaN keeping sign and payload with the quiet bit set.
//
// Both are one read and one write an element: HBM-bound, a thread per group of elements, coalesced.
#include <cstdint>
#include <cuda_runtime.h>

#include "device_math.cuh"
#include "kernels.h"
#include "pdl.cuh"

namespace b200 {
namespace {

__device__ __forceinline__ uint16_t f32_to_f16_bits(uint32_t x) {
  const uint32_t sign = (x >> 16) & 0x8000u, a = x & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u | ((a >> 13) & 0x3ffu));   // NaN: quiet, payload kept
  if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);                          // rounds to 2^16 or beyond
  if (a >= 0x38800000u) {                                                          // a normal binary16
    const uint32_t r = a + 0xfffu + ((a >> 13) & 1u);
    return (uint16_t)(sign | ((r >> 13) - 0x1c000u));
  }
  if (a <= 0x33000000u) return (uint16_t)sign;                                     // at most 2^-25: zero (the tie is even)
  const uint32_t shift = 126u - (a >> 23);                                         // 14 .. 24
  const uint32_t m = (a & 0x7fffffu) | 0x800000u;
  const uint32_t lsb = (m >> shift) & 1u;
  return (uint16_t)(sign | ((m + ((1u << (shift - 1)) - 1u) + lsb) >> shift));     // the 2^-24 grid
}

// Two at once: the hardware's conversion is the same rule for every number (nearest even on the binary16 grid, subnormal
// results, overflow to infinity); only a NaN differs (the hardware gives the canonical one), so those take the integer rule.
// The integer program alone, some thirty instructions an element, made the narrowing ALU-bound (0.76 of the copy rate).
__device__ __forceinline__ uint32_t f32x2_to_f16x2_bits(uint32_t lo, uint32_t hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(__uint_as_float(hi)), "f"(__uint_as_float(lo)));
  if ((lo & 0x7fffffffu) > 0x7f800000u) r = (r & 0xffff0000u) | f32_to_f16_bits(lo);
  if ((hi & 0x7fffffffu) > 0x7f800000u) r = (r & 0x0000ffffu) | ((uint32_t)f32_to_f16_bits(hi) << 16);
  return r;
}

__device__ __forceinline__ uint32_t f16_to_f32_bits(uint32_t h) {
  const uint32_t sign = (h & 0x8000u) << 16, a = h & 0x7fffu;
  if (a >= 0x7c00u) return sign | 0x7f800000u | ((a & 0x3ffu) << 13) | (a > 0x7c00u ? 0x400000u : 0u);
  if (a >= 0x400u) return sign | ((a << 13) + 0x38000000u);
  return sign | __float_as_uint((float)a * 5.9604644775390625e-8f);                 // m * 2^-24, exact
}

// Widening by the hardware's (exact) conversion, a NaN by the integer rule.
__device__ __forceinline__ uint32_t f16_to_f32_fast(uint32_t h) {
  if ((h & 0x7fffu) > 0x7c00u) return f16_to_f32_bits(h);
  float f;
  asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"((uint16_t)h));
  return __float_as_uint(f);
}

__global__ void __launch_bounds__(256)
cast_f16_kernel(const void* __restrict__ in, void* __restrict__ out, uint64_t n, int to_f16) {
  pdl_enter();
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x * 4;
  for (uint64_t i = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (to_f16) {
      const uint32_t* s = reinterpret_cast<const uint32_t*>(in);
      uint16_t* d = reinterpret_cast<uint16_t*>(out);
      if (i + 3 < n) {                          // both bases come from the pool: 256-byte aligned
        const uint4 v = *reinterpret_cast<const uint4*>(s + i);
        uint2 o;
        o.x = f32x2_to_f16x2_bits(v.x, v.y);
        o.y = f32x2_to_f16x2_bits(v.z, v.w);
        *reinterpret_cast<uint2*>(d + i) = o;
      } else {
        for (uint64_t j = i; j < n; ++j) d[j] = f32_to_f16_bits(s[j]);
      }
    } else {
      const uint16_t* s = reinterpret_cast<const uint16_t*>(in);
      uint32_t* d = reinterpret_cast<uint32_t*>(out);
      if (i + 3 < n) {
        const uint2 v = *reinterpret_cast<const uint2*>(s + i);
        uint4 o;
        o.x = f16_to_f32_fast(v.x & 0xffffu); o.y = f16_to_f32_fast(v.x >> 16);
        o.z = f16_to_f32_fast(v.y & 0xffffu); o.w = f16_to_f32_fast(v.y >> 16);
        *reinterpret_cast<uint4*>(d + i) = o;
      } else {
        for (uint64_t j = i; j < n; ++j) d[j] = f16_to_f32_bits(s[j]);
      }
    }
  }
}

// A block of a wider buffer: rows of `cols` elements, `in_ld` apart; the result is dense.  A warp a row at a
// time, four elements a lane where the block's rows are whole 16-byte pieces at 16-byte addresses.
__global__ void __launch_bounds__(256)
cast_block_kernel(const void* __restrict__ in, uint64_t in_ld, void* __restrict__ out, uint64_t rows, uint32_t cols,
                  int to_bf16, int vec4) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  for (uint64_t r = warp; r < rows; r += nwarps) {
    if (to_bf16) {
      const uint32_t* s = reinterpret_cast<const uint32_t*>(in) + r * in_ld;
      uint16_t* d = reinterpret_cast<uint16_t*>(out) + r * cols;
      if (vec4) {
        for (uint32_t c = lane * 4; c < cols; c += 128) {
          const uint4 v = *reinterpret_cast<const uint4*>(s + c);
          uint2 o;
          o.x = (uint32_t)f32_to_bf16_bits(v.x) | ((uint32_t)f32_to_bf16_bits(v.y) << 16);
          o.y = (uint32_t)f32_to_bf16_bits(v.z) | ((uint32_t)f32_to_bf16_bits(v.w) << 16);
          *reinterpret_cast<uint2*>(d + c) = o;
        }
      } else {
        for (uint32_t c = lane; c < cols; c += 32) d[c] = f32_to_bf16_bits(s[c]);
      }
    } else {
      const uint16_t* s = reinterpret_cast<const uint16_t*>(in) + r * in_ld;
      uint32_t* d = reinterpret_cast<uint32_t*>(out) + r * cols;
      if (vec4) {
        for (uint32_t c = lane * 4; c < cols; c += 128) {
          const uint2 v = *reinterpret_cast<const uint2*>(s + c);
          *reinterpret_cast<uint4*>(d + c) = make_uint4(v.x << 16, v.x & 0xffff0000u, v.y << 16, v.y & 0xffff0000u);
        }
      } else {
        for (uint32_t c = lane; c < cols; c += 32) d[c] = (uint32_t)s[c] << 16;
      }
    }
  }
}

}  // namespace

cudaError_t launch_cast_f16(const void* in, void* out, uint64_t n, int to_f16, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  uint64_t blocks = (n / 4 + 255) / 256 + 1;
  if (blocks > 148ull * 64) blocks = 148ull * 64;
  launch_pdl(cast_f16_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, in, out, n, to_f16);
  return cudaGetLastError();
}

cudaError_t launch_cast_block(const void* in, uint64_t in_ld, void* out, uint64_t rows, uint64_t cols, int to_bf16,
                              cudaStream_t stream) {
  if (rows == 0 || cols == 0) return cudaSuccess;
  if (in_ld == cols) return launch_cast(in, out, rows * cols, to_bf16, stream);   // whole rows: the dense cast
  const uint64_t in_eb = to_bf16 ? 4 : 2;
  const int vec4 = cols % 4 == 0 && in_ld % 4 == 0 && (reinterpret_cast<uintptr_t>(in) % (4 * in_eb)) == 0 &&
                   (reinterpret_cast<uintptr_t>(out) % 16) == 0;
  uint64_t blocks = (rows + 7) / 8;
  if (blocks > 148ull * 16) blocks = 148ull * 16;
  launch_pdl(cast_block_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, in, in_ld, out, rows, (uint32_t)cols, to_bf16, vec4);
  return cudaGetLastError();
}

}  // namespace b200
