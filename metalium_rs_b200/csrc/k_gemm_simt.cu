// SIMT product: C = op(A) op(B) for any shape, any transposes, F32 or BF16 operands,
// F32 accumulation by FMA in ascending k for every output element (so a result never
// depends on the tile an element fell in), result F32 or rounded once to BF16.
// The engine takes this path for shapes the tensor-core kernels refuse (ragged or tiny:
// the MLP's [64,784]x[784,128], a head's [512,64] blocks) and for F32 products.
// Boundary: `Engine::matmul_dram`, `matmul_dram_bf16`, `matmul_dram_batched`
// (crates/burn-tt/src/server.rs:178,191,229).
#include "device_math.cuh"
#include "kernels.h"

namespace b200 {
namespace {

constexpr int BM = 128, BN = 128, BK = 16, THREADS = 256;

template <bool BF16>
__device__ __forceinline__ float ld_elem(const void* p, uint64_t i) {
  if constexpr (BF16) return bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(p)[i]);
  else return reinterpret_cast<const float*>(p)[i];
}

// Logical A is [m,k]; stored [m,k] (lda) or, transposed, [k,m].  Same for B [k,n].
template <bool IN_BF16, bool OUT_BF16>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(GemmArgs g) {
  __shared__ float As[2][BK][BM + 4];
  __shared__ float Bs[2][BK][BN + 4];
  uint64_t a_off = 0, b_off = 0, c_off = 0;
  int a_trans = g.a_trans, b_trans = g.b_trans;
  if (g.batches_dev) {
    const GemmBatch bt = g.batches_dev[blockIdx.z];
    a_off = bt.a_off; b_off = bt.b_off; c_off = bt.c_off; a_trans = bt.a_trans; b_trans = bt.b_trans;
  }
  const uint64_t m0 = (uint64_t)blockIdx.y * BM, n0 = (uint64_t)blockIdx.x * BN;
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;  // 16 x 16 threads, 8 x 8 each

  // loader mapping: 8 elements of A and 8 of B a thread a k-tile
  // not transposed A ([m,k], k contiguous): thread -> (m = e / 16, k = e % 16)
  // transposed A ([k,m], m contiguous):     thread -> (k = e / 128, m = e % 128)
  float ra[8], rb[8];
  auto load_tiles = [&](uint64_t k0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = tid + i * THREADS;
      int mm, kk;
      if (!a_trans) { mm = e / BK; kk = e % BK; } else { kk = e / BM; mm = e % BM; }
      const uint64_t gm = m0 + mm, gk = k0 + kk;
      float v = 0.f;
      if (gm < g.m && gk < g.k)
        v = ld_elem<IN_BF16>(g.a, a_off + (a_trans ? gk * g.lda + gm : gm * g.lda + gk));
      ra[i] = v;
      int nn;
      if (!b_trans) { kk = e / BN; nn = e % BN; } else { nn = e / BK; kk = e % BK; }
      const uint64_t gn = n0 + nn, gk2 = k0 + kk;
      v = 0.f;
      if (gn < g.n && gk2 < g.k)
        v = ld_elem<IN_BF16>(g.b, b_off + (b_trans ? gn * g.ldb + gk2 : gk2 * g.ldb + gn));
      rb[i] = v;
    }
  };
  auto store_tiles = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = tid + i * THREADS;
      int mm, kk, nn;
      if (!a_trans) { mm = e / BK; kk = e % BK; } else { kk = e / BM; mm = e % BM; }
      As[buf][kk][mm] = ra[i];
      if (!b_trans) { kk = e / BN; nn = e % BN; } else { nn = e / BK; kk = e % BK; }
      Bs[buf][kk][nn] = rb[i];
    }
  };

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  const uint64_t ktiles = (g.k + BK - 1) / BK;
  if (ktiles > 0) {
    load_tiles(0);
    store_tiles(0);
  }
  __syncthreads();
  for (uint64_t kt = 0; kt < ktiles; ++kt) {
    const int buf = (int)(kt & 1);
    if (kt + 1 < ktiles) load_tiles((kt + 1) * BK);
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[8], bv[8];
      // rows ty*4..+3 and 64+ty*4..+3; cols tx*4..+3 and 64+tx*4..+3
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
      av[0] = a0.x; av[1] = a0.y; av[2] = a0.z; av[3] = a0.w; av[4] = a1.x; av[5] = a1.y; av[6] = a1.z; av[7] = a1.w;
      bv[0] = b0.x; bv[1] = b0.y; bv[2] = b0.z; bv[3] = b0.w; bv[4] = b1.x; bv[5] = b1.y; bv[6] = b1.z; bv[7] = b1.w;
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (kt + 1 < ktiles) store_tiles(buf ^ 1);
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint64_t gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (gm >= g.m) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint64_t gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
      if (gn >= g.n) continue;
      const uint64_t o = c_off + gm * g.ldc + gn;
      if constexpr (OUT_BF16) reinterpret_cast<uint16_t*>(g.c)[o] = f32_to_bf16_bits(__float_as_uint(acc[i][j]));
      else reinterpret_cast<float*>(g.c)[o] = acc[i][j];
    }
  }
}

}  // namespace

cudaError_t launch_gemm_simt(const GemmArgs& g, cudaStream_t stream) {
  if (g.m == 0 || g.n == 0 || g.batch == 0) return cudaSuccess;
  const uint64_t gy = (g.m + BM - 1) / BM, gx = (g.n + BN - 1) / BN;
  if (gy > 65535 || g.batch > 65535) return cudaErrorInvalidValue;
  dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)g.batch);
  if (g.in_bf16) {
    if (g.out_bf16) gemm_simt_kernel<true, true><<<grid, THREADS, 0, stream>>>(g);
    else gemm_simt_kernel<true, false><<<grid, THREADS, 0, stream>>>(g);
  } else {
    if (g.out_bf16) gemm_simt_kernel<false, true><<<grid, THREADS, 0, stream>>>(g);
    else gemm_simt_kernel<false, false><<<grid, THREADS, 0, stream>>>(g);
  }
  return cudaGetLastError();
}

}  // namespace b200
