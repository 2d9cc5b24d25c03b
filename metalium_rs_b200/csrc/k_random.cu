// A tensor drawn on the device from a seed: `Engine::random_dram` (crates/burn-tt/src/server.rs:768), the
// six draws of crates/burn-tt/src/random.rs:73-90 built as crates/tt-kernels/src/prng.rs:449-595 builds
// them from unit uniforms.
//
// The reference's words come from the Tensix lane generators and differ between its simulator and its
// silicon (prng.rs:49-50), so no stream of it is a value to reproduce.  What is kept is the contract: a
// datum depends on (base, role, position) only, never on how the work is cut; a word is turned into a
// uniform as `(0x3f800000 | word >> 9) - 1.0`, exactly k 2^-23; and every distribution is the reference's
// arithmetic on such uniforms, step for step:
//   Unit        u
//   Uniform     min(fl(fl(u fl(hi - lo)) + lo), the float below hi)
//   Bernoulli   u < p ? 1 : 0 (F32 or I32)
//   Normal      mean + std sqrt(-2 ln(1 - u1)) cos(2 pi u2), u1 and u2 from two roles; `int`: truncated
//   IntRange    lo + trunc(u (hi - lo))
//   IntWords    the word itself
// The word of position i in role r is the high half of splitmix64(splitmix64(base ^ r) + i golden): the
// reference's tile seed function (prng.rs:34-36) taken per element instead of per tile.
#include <cstdint>
#include <cuda_runtime.h>

#include "kernels.h"
#include "pdl.cuh"

namespace b200 {
namespace {

enum { D_UNIT, D_UNIFORM, D_BERNOULLI, D_NORMAL, D_INT_RANGE, D_INT_WORDS };
enum { R_UNIT, R_UNIFORM, R_BERNOULLI, R_NORMAL_RADIUS, R_NORMAL_ANGLE, R_INT_RANGE, R_INT_WORD };

__host__ __device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}
__device__ __forceinline__ uint32_t word_at(uint64_t role_seed, uint64_t i) {
  return (uint32_t)(splitmix64(role_seed + i * 0x9e3779b97f4a7c15ull) >> 32);
}
__device__ __forceinline__ float unit_of(uint32_t w) { return __fsub_rn(__uint_as_float(0x3f800000u | (w >> 9)), 1.0f); }

__global__ void __launch_bounds__(256)
random_kernel(uint32_t* __restrict__ out, uint64_t n, int draw, float p0, float p1, int32_t i0, int32_t i1, int as_int,
              uint64_t seed_a, uint64_t seed_b) {
  pdl_enter();
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const uint32_t w = word_at(seed_a, i);
    const float u = unit_of(w);
    uint32_t r;
    switch (draw) {
      case D_UNIT: r = __float_as_uint(u); break;
      case D_UNIFORM: {
        const float v = __fadd_rn(__fmul_rn(u, __fsub_rn(p1, p0)), p0);
        const float top = __uint_as_float((uint32_t)i1);       // the float below hi, from the host
        r = __float_as_uint(v < top ? v : top);
        break;
      }
      case D_BERNOULLI: r = u < p0 ? (as_int ? 1u : 0x3f800000u) : 0u; break;
      case D_NORMAL: {
        const float u2 = unit_of(word_at(seed_b, i));
        const float radius = sqrtf(__fmul_rn(-2.0f, logf(__fsub_rn(1.0f, u))));
        const float z = __fmul_rn(radius, cosf(__fmul_rn(6.2831853071795864769f, u2)));
        const float v = __fadd_rn(__fmul_rn(z, p1), p0);
        r = as_int ? (uint32_t)__float2int_rz(v) : __float_as_uint(v);
        break;
      }
      case D_INT_RANGE: r = (uint32_t)(i0 + __float2int_rz(__fmul_rn(u, p0))); break;
      default: r = w; break;
    }
    out[i] = r;
  }
}

}  // namespace

cudaError_t launch_random(uint32_t* out, uint64_t n, int draw, float p0, float p1, int32_t i0, int32_t i1, int as_int,
                          uint64_t base, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  static const int role_of[6][2] = {{R_UNIT, R_UNIT}, {R_UNIFORM, R_UNIFORM}, {R_BERNOULLI, R_BERNOULLI},
                                    {R_NORMAL_RADIUS, R_NORMAL_ANGLE}, {R_INT_RANGE, R_INT_RANGE}, {R_INT_WORD, R_INT_WORD}};
  if (draw < 0 || draw > 5) return cudaErrorNotSupported;
  const uint64_t seed_a = splitmix64(base ^ (uint64_t)role_of[draw][0]), seed_b = splitmix64(base ^ (uint64_t)role_of[draw][1]);
  uint64_t blocks = (n + 255) / 256;
  if (blocks > 148ull * 16) blocks = 148ull * 16;
  launch_pdl(random_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, out, n, draw, p0, p1, i0, i1, as_int, seed_a, seed_b);
  return cudaGetLastError();
}

}  // namespace b200
