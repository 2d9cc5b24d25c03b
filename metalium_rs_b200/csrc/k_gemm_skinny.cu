// C[m, n] = A[m, k] B[k, n] for a handful of rows (m <= 4): a decode step's projections
// (`Engine::matmul_dram_bf16` with one token a sequence, crates/burn-tt/src/server.rs:191).  BF16
// operands as they are stored ([m, k] and [k, n] row-major), F32 accumulation, F32 or BF16 result.
//
// The work is reading B once, so the bound is HBM (or, for the small B of a 135M-parameter layer,
// launch latency); a 128-row tensor-core tile with one live row spends ~10 us on it.  Here a block
// owns 64 columns of C and all of k: a thread holds a 16-byte column group (8 columns) of one k-row
// slice, 8 groups x 64 slices a block, so a warp's load is four 128-byte row segments; A sits in
// shared memory as F32 and is broadcast; the slices are joined by two shuffles and one pass through
// shared memory.  Measured in the SmolLM2-135M-shape decode step: one row 2.07 -> 1.63 ms a step against the
// tensor-core tile; at eight rows the tile is the faster one again (2.21 against 2.41 ms), so the
// kernel takes up to four.
#include <cstdint>
#include <cuda_runtime.h>

#include "device_math.cuh"
#include "kernels.h"
#include "pdl.cuh"

namespace b200 {
namespace {

constexpr int SK_THREADS = 512;
constexpr int SK_SLICES = SK_THREADS / 8;   // k-row slices a block
constexpr int SK_COLS = 64;                 // columns of C a block

template <int MT>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const uint16_t* __restrict__ a, uint64_t lda, const uint16_t* __restrict__ b, uint64_t ldb,
                   void* __restrict__ c, uint64_t ldc, int out_bf16, int m, uint64_t n, int k) {
  extern __shared__ float sm[];
  pdl_enter();
  float* as = sm;                                   // [MT][k]
  float* red = sm + (size_t)MT * k;                 // [16 warps][MT][64]
  const int tid = threadIdx.x, cg = tid & 7, ks = tid >> 3, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < MT * k; i += SK_THREADS) {
    const int r = i / k, e = i - r * k;
    as[i] = r < m ? __uint_as_float((uint32_t)a[(uint64_t)r * lda + e] << 16) : 0.f;
  }
  __syncthreads();
  const uint64_t col = (uint64_t)blockIdx.x * SK_COLS + cg * 8;
  float acc[MT][8];
#pragma unroll
  for (int r = 0; r < MT; ++r)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[r][e] = 0.f;
  if (col < n) {                                    // n is a multiple of 8: a group is whole or absent
    const uint16_t* bp = b + col;
    for (int k0 = ks; k0 < k; k0 += SK_SLICES * 4) {
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int kk = k0 + u * SK_SLICES;
        if (kk < k) raw[u] = __ldg(reinterpret_cast<const uint4*>(bp + (uint64_t)kk * ldb));
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int kk = k0 + u * SK_SLICES;
        if (kk < k) {
          float x[8];
          x[0] = __uint_as_float(raw[u].x << 16); x[1] = __uint_as_float(raw[u].x & 0xffff0000u);
          x[2] = __uint_as_float(raw[u].y << 16); x[3] = __uint_as_float(raw[u].y & 0xffff0000u);
          x[4] = __uint_as_float(raw[u].z << 16); x[5] = __uint_as_float(raw[u].z & 0xffff0000u);
          x[6] = __uint_as_float(raw[u].w << 16); x[7] = __uint_as_float(raw[u].w & 0xffff0000u);
#pragma unroll
          for (int r = 0; r < MT; ++r) {
            const float av = as[(size_t)r * k + kk];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[r][e] = fmaf(av, x[e], acc[r][e]);
          }
        }
      }
    }
  }
  // a warp holds four slices of the same eight groups: lanes 8 and 16 apart
#pragma unroll
  for (int r = 0; r < MT; ++r)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float v = acc[r][e];
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      acc[r][e] = v;
    }
  if (lane < 8) {
#pragma unroll
    for (int r = 0; r < MT; ++r)
#pragma unroll
      for (int e = 0; e < 8; ++e) red[((size_t)warp * MT + r) * SK_COLS + lane * 8 + e] = acc[r][e];
  }
  __syncthreads();
  for (int i = tid; i < MT * SK_COLS; i += SK_THREADS) {
    const int r = i / SK_COLS, cc = i - r * SK_COLS;
    const uint64_t oc = (uint64_t)blockIdx.x * SK_COLS + cc;
    if (r < m && oc < n) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < SK_THREADS / 32; ++w) t += red[((size_t)w * MT + r) * SK_COLS + cc];
      if (out_bf16) reinterpret_cast<uint16_t*>(c)[(uint64_t)r * ldc + oc] = f32_to_bf16_bits(__float_as_uint(t));
      else reinterpret_cast<float*>(c)[(uint64_t)r * ldc + oc] = t;
    }
  }
}

}  // namespace

bool gemm_skinny_supported(const GemmArgs& g) {
  if (!(g.in_bf16 && g.batch <= 1 && !g.batches_dev && !g.a_trans && !g.b_trans && g.m >= 1 && g.m <= 4 && g.n >= 8 &&
        g.n % 8 == 0 && g.ldb % 8 == 0 && g.k >= 1 && (((uintptr_t)g.b) & 15) == 0))
    return false;
  const uint64_t mt = g.m <= 1 ? 1 : (g.m <= 2 ? 2 : (g.m <= 4 ? 4 : 8));
  return (mt * g.k + (uint64_t)(SK_THREADS / 32) * mt * SK_COLS) * sizeof(float) <= 200 * 1024;   // A and the join fit shared memory
}

cudaError_t launch_gemm_skinny(const GemmArgs& g, cudaStream_t stream) {
  const int mt = g.m <= 1 ? 1 : (g.m <= 2 ? 2 : (g.m <= 4 ? 4 : 8));
  const size_t smem = ((size_t)mt * g.k + (size_t)(SK_THREADS / 32) * mt * SK_COLS) * sizeof(float);
  const unsigned grid = (unsigned)((g.n + SK_COLS - 1) / SK_COLS);
#define GO(MT)                                                                                                   \
  do {                                                                                                           \
    {                                                                                                            \
      const cudaError_t e = ensure_dynamic_smem((const void*)gemm_skinny_kernel<MT>, smem);                      \
      if (e != cudaSuccess) return e;                                                                            \
    }                                                                                                            \
    launch_pdl(gemm_skinny_kernel<MT>, dim3(grid), dim3(SK_THREADS), smem, stream, (const uint16_t*)g.a, g.lda, (const uint16_t*)g.b, g.ldb, \
               g.c, g.ldc, g.out_bf16, (int)g.m, g.n, (int)g.k);                                                   \
  } while (0)
  if (mt == 1) GO(1); else if (mt == 2) GO(2); else GO(4);
#undef GO
  return cudaGetLastError();
}

}  // namespace b200
