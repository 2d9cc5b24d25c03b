// Window means of a BF16 matrix: `Engine::pool_bf16` (crates/burn-tt/src/server.rs:118;
// crates/tt-kernels/src/fpu.rs:39-132).  A window is a list of [row, col] coordinates of the input the
// host built (an average pool's taps); result element w is the F32 sum of the window's BF16 values
// divided by the window's divisor.  The reference sums a window sixteen values at a time (one pooling
// block a step), adds the blocks' F32 partial sums in order and divides once (`DIV` by the count as
// F32); the same three steps here, the values of a block added in window order.  The result stays F32
// (fpu.rs:3977 "results remain F32 until the caller casts").
//
// A thread a window: windows are a few values (a 3x3 pool reads nine), the reads are gathers of two
// bytes out of a matrix that mostly sits in L2, the writes are coalesced.
#include <cstdint>
#include <cuda_runtime.h>

#include "kernels.h"
#include "pdl.cuh"

namespace b200 {
namespace {

__global__ void __launch_bounds__(256)
pool_windows_kernel(const uint16_t* __restrict__ in, const uint32_t* __restrict__ offsets, const uint32_t* __restrict__ flat,
                    const float* __restrict__ divisors, uint64_t n, float* __restrict__ out) {
  pdl_enter();
  for (uint64_t w = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; w < n; w += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t b = offsets[w], e = offsets[w + 1];
    float total = 0.f;
    for (uint32_t i0 = b; i0 < e; i0 += 16) {
      float part = 0.f;
      const uint32_t i1 = i0 + 16 < e ? i0 + 16 : e;
      for (uint32_t i = i0; i < i1; ++i) part = __fadd_rn(part, __uint_as_float((uint32_t)in[flat[i]] << 16));
      total = i0 == b ? part : __fadd_rn(total, part);
    }
    out[w] = __fdiv_rn(total, divisors[w]);
  }
}

}  // namespace

cudaError_t launch_pool_windows(const uint16_t* in, const uint32_t* offsets_dev, const uint32_t* flat_dev, const float* divisors_dev,
                                uint64_t n, float* out, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  uint64_t blocks = (n + 255) / 256;
  if (blocks > 148ull * 16) blocks = 148ull * 16;
  launch_pdl(pool_windows_kernel, dim3((unsigned)blocks), dim3(256), 0, s, in, offsets_dev, flat_dev, divisors_dev, n, out);
  return cudaGetLastError();
}

}  // namespace b200
