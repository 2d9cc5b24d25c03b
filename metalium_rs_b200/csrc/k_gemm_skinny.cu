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

// The same against a B stored [n, k] (`matmul_dram(a, false, b, true)`: a tied language-model head, logits = x table^T,
// crates/tt-models/src/llama.rs:1090): every output is the dot product of a row of A with a contiguous row of B, so a
// warp takes rows of B four at a time, a lane the 16-byte units lane, lane + 32, ... of each (whole 128-byte lines a
// load), A in shared memory as F32, and a butterfly of shuffles joins the lanes' sums.  The 128-row tensor-core tile read
// SmolLM2-135M's 57 MB table at 3.6 TB/s (15.8 us); one row here 5.7 TB/s (10.0 us).  With four and eight rows of A this
// kernel is bound by its reads of A from shared memory (22.7 and 37.6 us), so it takes one or two rows and the tile the rest.
constexpr int SKT_THREADS = 256;
constexpr int SKT_ROWS = 4;                  // rows of B a warp has in flight

template <int MT>
__global__ void __launch_bounds__(SKT_THREADS)
gemm_skinny_t_kernel(const uint16_t* __restrict__ a, uint64_t lda, const uint16_t* __restrict__ b, uint64_t ldb,
                     void* __restrict__ c, uint64_t ldc, int out_bf16, int m, uint64_t n, int k, uint32_t rows_a_warp) {
  extern __shared__ float sm[];
  pdl_enter();
  float* as = sm;                                   // [MT][k]
  const int tid = threadIdx.x, lane = tid & 31;
  for (int i = tid; i < MT * k; i += SKT_THREADS) {
    const int r = i / k, e = i - r * k;
    as[i] = r < m ? __uint_as_float((uint32_t)a[(uint64_t)r * lda + e] << 16) : 0.f;
  }
  __syncthreads();
  const uint64_t warp = ((uint64_t)blockIdx.x * SKT_THREADS + tid) >> 5;
  const uint64_t v0 = warp * rows_a_warp, v1 = v0 + rows_a_warp < n ? v0 + rows_a_warp : n;
  const int units = k / 8;                          // k is a multiple of 8
  for (uint64_t v = v0; v < v1; v += SKT_ROWS) {
    float acc[SKT_ROWS][MT];
#pragma unroll
    for (int q = 0; q < SKT_ROWS; ++q)
#pragma unroll
      for (int r = 0; r < MT; ++r) acc[q][r] = 0.f;
    for (int u = lane; u < units; u += 32) {
      uint4 raw[SKT_ROWS];
#pragma unroll
      for (int q = 0; q < SKT_ROWS; ++q) {
        const uint64_t row = v + q < v1 ? v + q : v1 - 1;          // (a row past the warp's share reads its last again)
        raw[q] = __ldg(reinterpret_cast<const uint4*>(b + row * ldb) + u);
      }
      float4 xa[MT], xb[MT];
#pragma unroll
      for (int r = 0; r < MT; ++r) {
        xa[r] = *reinterpret_cast<const float4*>(as + (size_t)r * k + u * 8);
        xb[r] = *reinterpret_cast<const float4*>(as + (size_t)r * k + u * 8 + 4);
      }
#pragma unroll
      for (int q = 0; q < SKT_ROWS; ++q) {
        const float w0 = __uint_as_float(raw[q].x << 16), w1 = __uint_as_float(raw[q].x & 0xffff0000u);
        const float w2 = __uint_as_float(raw[q].y << 16), w3 = __uint_as_float(raw[q].y & 0xffff0000u);
        const float w4 = __uint_as_float(raw[q].z << 16), w5 = __uint_as_float(raw[q].z & 0xffff0000u);
        const float w6 = __uint_as_float(raw[q].w << 16), w7 = __uint_as_float(raw[q].w & 0xffff0000u);
#pragma unroll
        for (int r = 0; r < MT; ++r) {
          float t = acc[q][r];
          t = fmaf(xa[r].x, w0, t); t = fmaf(xa[r].y, w1, t); t = fmaf(xa[r].z, w2, t); t = fmaf(xa[r].w, w3, t);
          t = fmaf(xb[r].x, w4, t); t = fmaf(xb[r].y, w5, t); t = fmaf(xb[r].z, w6, t); t = fmaf(xb[r].w, w7, t);
          acc[q][r] = t;
        }
      }
    }
#pragma unroll
    for (int q = 0; q < SKT_ROWS; ++q)
#pragma unroll
      for (int r = 0; r < MT; ++r) {
        float t = acc[q][r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        acc[q][r] = t;
      }
    // lane q * MT + r stores output (row r of A, row v + q of B)
#pragma unroll
    for (int q = 0; q < SKT_ROWS; ++q)
#pragma unroll
      for (int r = 0; r < MT; ++r)
        if (lane == q * MT + r && r < m && v + q < v1) {
          if (out_bf16) reinterpret_cast<uint16_t*>(c)[(uint64_t)r * ldc + v + q] = f32_to_bf16_bits(__float_as_uint(acc[q][r]));
          else reinterpret_cast<float*>(c)[(uint64_t)r * ldc + v + q] = acc[q][r];
        }
  }
}

}  // namespace

bool gemm_skinny_supported(const GemmArgs& g) {
  if (g.in_bf16 && g.batch <= 1 && !g.batches_dev && !g.a_trans && g.b_trans && g.m >= 1 && g.m <= 2 && g.n >= 1024 &&
      g.k >= 8 && g.k % 8 == 0 && g.ldb % 8 == 0 && (((uintptr_t)g.b) & 15) == 0 && !g.n_more && !g.multicast && g.epi_mode == 0)
    return (uint64_t)8 * g.k * sizeof(float) <= 96 * 1024;   // B stored [n, k]: the transposed kernel, A in shared memory
  if (!(g.in_bf16 && g.batch <= 1 && !g.batches_dev && !g.a_trans && !g.b_trans && g.m >= 1 && g.m <= 4 && g.n >= 8 &&
        g.n % 8 == 0 && g.ldb % 8 == 0 && g.k >= 1 && (((uintptr_t)g.b) & 15) == 0))
    return false;
  const uint64_t mt = g.m <= 1 ? 1 : (g.m <= 2 ? 2 : (g.m <= 4 ? 4 : 8));
  return (mt * g.k + (uint64_t)(SK_THREADS / 32) * mt * SK_COLS) * sizeof(float) <= 200 * 1024;   // A and the join fit shared memory
}

cudaError_t launch_gemm_skinny(const GemmArgs& g, cudaStream_t stream) {
  if (g.b_trans) {
    const int mt = g.m <= 1 ? 1 : (g.m <= 2 ? 2 : (g.m <= 4 ? 4 : 8));
    const size_t smem = (size_t)mt * g.k * sizeof(float);
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // about four blocks an SM, every warp whole groups of SKT_ROWS rows of B
    const uint64_t warps_wanted = (uint64_t)sms * 4 * (SKT_THREADS / 32);
    uint64_t per = (g.n + warps_wanted - 1) / warps_wanted;
    per = (per + SKT_ROWS - 1) / SKT_ROWS * SKT_ROWS;
    const uint64_t warps = (g.n + per - 1) / per;
    const unsigned grid = (unsigned)((warps + SKT_THREADS / 32 - 1) / (SKT_THREADS / 32));
#define GOT(MT)                                                                                                  \
  do {                                                                                                           \
    {                                                                                                            \
      const cudaError_t e = ensure_dynamic_smem((const void*)gemm_skinny_t_kernel<MT>, smem);                    \
      if (e != cudaSuccess) return e;                                                                            \
    }                                                                                                            \
    launch_pdl(gemm_skinny_t_kernel<MT>, dim3(grid), dim3(SKT_THREADS), smem, stream, (const uint16_t*)g.a, g.lda, (const uint16_t*)g.b, g.ldb, \
               g.c, g.ldc, g.out_bf16, (int)g.m, g.n, (int)g.k, (uint32_t)per);                                   \
  } while (0)
    if (mt == 1) GOT(1); else if (mt == 2) GOT(2); else if (mt == 4) GOT(4); else GOT(8);
#undef GOT
    return cudaGetLastError();
  }
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
