// Block-float (BFP8) weight storage: `Engine::cast_bfp` (crates/burn-tt/src/server.rs:141), the format of
// crates/tt-kernels/src/bfp.rs:60-63 -- sixteen consecutive datums of a row share one 8-bit exponent, a datum is a sign
// bit over a 7-bit magnitude -- and a few-row product that reads such a matrix as its B, decoding in its load path
// (crates/burn-tt/src/storage.rs:117-123: "a BF16 stream's weights, which a product reads as its B against a BF16
// activation").
//
// A stored matrix [rows, cols] (cols a multiple of 16) is rows * cols datum bytes, row-major, followed by
// rows * cols / 16 exponent bytes, row-major: 17 bytes for 16 values where BF16 takes 32.  The reference keeps the same
// groups (a 16-datum face row is sixteen consecutive columns of one matrix row) inside 32 x 32 tiles; tiling is its
// device's layout, not part of the values.
//
// Decoding is the reference's own routine, crates/tt-isa/src/tile.rs:619-634 (`bfp8_to_bf16`, proven over its whole
// domain by the test at :1118): magnitude 0 is +0 (or, under a set sign bit, -infinity: the format has no -0), otherwise
// the magnitude is normalised and the shared exponent reduced by the shift.  Every decoded value is a BF16 value.
//
// Encoding is this engine's (the reference's encoder is its packer hardware): the group's exponent is the largest F32
// exponent in the group, a magnitude is |x| 2^(133 - E) rounded to nearest, ties to even; if a magnitude rounds up to
// 128 the exponent is raised by one and the group rounded again.  So a decoded value lies within half a step
// 2^(E - 133) of what was stored.  A value that rounds to magnitude 0 is stored +0.  A group whose largest exponent is 7
// or less (below 2^-119) is stored as zeros, since the decoder's exponent arithmetic would wrap there.  A group that
// holds an infinity or a NaN keeps those (exponent 255) and stores its finite members as zeros.
#include <cstdint>
#include <cuda_runtime.h>

#include "device_math.cuh"
#include "kernels.h"
#include "pdl.cuh"

namespace b200 {
namespace {

// One thread a group of sixteen values.
template <bool IN_BF16>
__global__ void __launch_bounds__(256)
bfp8_encode_kernel(const void* __restrict__ in, uint64_t groups, uint8_t* __restrict__ datums, uint8_t* __restrict__ exps) {
  for (uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += (uint64_t)gridDim.x * blockDim.x) {
    uint32_t w[16];
    if (IN_BF16) {
      const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(in) + g * 16);
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const uint4 v = p[q];
        w[q * 8 + 0] = v.x << 16; w[q * 8 + 1] = v.x & 0xffff0000u; w[q * 8 + 2] = v.y << 16; w[q * 8 + 3] = v.y & 0xffff0000u;
        w[q * 8 + 4] = v.z << 16; w[q * 8 + 5] = v.z & 0xffff0000u; w[q * 8 + 6] = v.w << 16; w[q * 8 + 7] = v.w & 0xffff0000u;
      }
    } else {
      const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const uint32_t*>(in) + g * 16);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 v = p[q];
        w[q * 4 + 0] = v.x; w[q * 4 + 1] = v.y; w[q * 4 + 2] = v.z; w[q * 4 + 3] = v.w;
      }
    }
    uint32_t E = 0;
    bool nonfinite = false;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t e = (w[i] >> 23) & 0xffu;
      E = e > E ? e : E;
    }
    nonfinite = E == 255u;
    uint32_t mag[16];
    if (nonfinite) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t a = w[i] & 0x7fffffffu;
        mag[i] = a > 0x7f800000u ? 96u : (a == 0x7f800000u ? 64u : 0u);
      }
    } else if (E <= 7u) {
      E = 0;
#pragma unroll
      for (int i = 0; i < 16; ++i) mag[i] = 0;
    } else {
      for (int pass = 0; pass < 2; ++pass) {
        const float scale = __uint_as_float((260u - E) << 23);   // 2^(133 - E), exact
        bool over = false;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int m = __float2int_rn(__uint_as_float(w[i] & 0x7fffffffu) * scale);
          over |= m >= 128;
          mag[i] = (uint32_t)(m > 127 ? 127 : m);
        }
        if (!over || E >= 254u) break;
        ++E;                                                      // the largest magnitude rounded up to 128: one exponent up
      }
    }
    uint32_t out[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t d = mag[i] ? (((w[i] >> 31) << 7) | mag[i]) : 0u;
      out[i >> 2] |= d << ((i & 3) * 8);
    }
    reinterpret_cast<uint4*>(datums)[g] = make_uint4(out[0], out[1], out[2], out[3]);
    exps[g] = (uint8_t)E;
  }
}

template <bool OUT_BF16>
__global__ void __launch_bounds__(256)
bfp8_decode_kernel(const uint8_t* __restrict__ datums, const uint8_t* __restrict__ exps, uint64_t groups, void* __restrict__ out) {
  for (uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += (uint64_t)gridDim.x * blockDim.x) {
    const uint4 d = reinterpret_cast<const uint4*>(datums)[g];
    const uint32_t e = exps[g];
    const uint32_t dw[4] = {d.x, d.y, d.z, d.w};
    uint16_t h[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) h[i] = bfp8_to_bf16_bits((dw[i >> 2] >> ((i & 3) * 8)) & 0xffu, e);
    if (OUT_BF16) {
      uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out) + g * 16);
#pragma unroll
      for (int q = 0; q < 2; ++q)
        o[q] = make_uint4((uint32_t)h[q * 8 + 0] | ((uint32_t)h[q * 8 + 1] << 16), (uint32_t)h[q * 8 + 2] | ((uint32_t)h[q * 8 + 3] << 16),
                          (uint32_t)h[q * 8 + 4] | ((uint32_t)h[q * 8 + 5] << 16), (uint32_t)h[q * 8 + 6] | ((uint32_t)h[q * 8 + 7] << 16));
    } else {
      uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<uint32_t*>(out) + g * 16);
#pragma unroll
      for (int q = 0; q < 4; ++q)
        o[q] = make_uint4((uint32_t)h[q * 4 + 0] << 16, (uint32_t)h[q * 4 + 1] << 16, (uint32_t)h[q * 4 + 2] << 16, (uint32_t)h[q * 4 + 3] << 16);
    }
  }
}

// The few-row product of k_gemm_skinny.cu with B read as BFP8: the same block shape (64 columns and all of k a block,
// a thread a group of 8 columns of one k-row slice, the same joins), so a product with a BFP8 B has the bits of the
// product with that B widened to BF16 -- a thread's load is 8 datum bytes and the group's exponent byte instead of 16.
constexpr int SKB_THREADS = 512;
constexpr int SKB_SLICES = SKB_THREADS / 8;
constexpr int SKB_COLS = 64;

template <int MT>
__global__ void __launch_bounds__(SKB_THREADS)
gemm_skinny_bfp_kernel(const uint16_t* __restrict__ a, uint64_t lda, const uint8_t* __restrict__ datums, const uint8_t* __restrict__ exps,
                       void* __restrict__ c, uint64_t ldc, int out_bf16, int m, uint64_t n, int k) {
  extern __shared__ float sm[];
  pdl_enter();
  float* as = sm;                                   // [MT][k]
  float* red = sm + (size_t)MT * k;                 // [16 warps][MT][64]
  const int tid = threadIdx.x, cg = tid & 7, ks = tid >> 3, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < MT * k; i += SKB_THREADS) {
    const int r = i / k, e = i - r * k;
    as[i] = r < m ? __uint_as_float((uint32_t)a[(uint64_t)r * lda + e] << 16) : 0.f;
  }
  __syncthreads();
  const uint64_t col = (uint64_t)blockIdx.x * SKB_COLS + cg * 8;
  const uint64_t egroups = n / 16;
  float acc[MT][8];
#pragma unroll
  for (int r = 0; r < MT; ++r)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[r][e] = 0.f;
  if (col < n) {
    const uint8_t* bp = datums + col;
    const uint8_t* ep = exps + col / 16;
    for (int k0 = ks; k0 < k; k0 += SKB_SLICES * 4) {
      uint2 raw[4];
      uint32_t ex[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int kk = k0 + u * SKB_SLICES;
        if (kk < k) {
          raw[u] = __ldg(reinterpret_cast<const uint2*>(bp + (uint64_t)kk * n));
          ex[u] = __ldg(ep + (uint64_t)kk * egroups);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int kk = k0 + u * SKB_SLICES;
        if (kk < k) {
          float x[8];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            x[e] = bfp8_value((raw[u].x >> (e * 8)) & 0xffu, ex[u]);
            x[4 + e] = bfp8_value((raw[u].y >> (e * 8)) & 0xffu, ex[u]);
          }
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
      for (int e = 0; e < 8; ++e) red[((size_t)warp * MT + r) * SKB_COLS + lane * 8 + e] = acc[r][e];
  }
  __syncthreads();
  for (int i = tid; i < MT * SKB_COLS; i += SKB_THREADS) {
    const int r = i / SKB_COLS, cc = i - r * SKB_COLS;
    const uint64_t oc = (uint64_t)blockIdx.x * SKB_COLS + cc;
    if (r < m && oc < n) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < SKB_THREADS / 32; ++w) t += red[((size_t)w * MT + r) * SKB_COLS + cc];
      if (out_bf16) reinterpret_cast<uint16_t*>(c)[(uint64_t)r * ldc + oc] = f32_to_bf16_bits(__float_as_uint(t));
      else reinterpret_cast<float*>(c)[(uint64_t)r * ldc + oc] = t;
    }
  }
}

inline unsigned grid_for(uint64_t groups) {
  const uint64_t b = (groups + 255) / 256;
  return (unsigned)(b < 148ull * 16 ? (b ? b : 1) : 148ull * 16);
}

}  // namespace

cudaError_t launch_bfp8_encode(const void* in, int in_bf16, uint64_t rows, uint64_t cols, uint8_t* datums, uint8_t* exps,
                               cudaStream_t s) {
  const uint64_t groups = rows * cols / 16;
  if (groups == 0) return cudaSuccess;
  if (in_bf16) bfp8_encode_kernel<true><<<grid_for(groups), 256, 0, s>>>(in, groups, datums, exps);
  else bfp8_encode_kernel<false><<<grid_for(groups), 256, 0, s>>>(in, groups, datums, exps);
  return cudaGetLastError();
}

cudaError_t launch_bfp8_decode(const uint8_t* datums, const uint8_t* exps, uint64_t rows, uint64_t cols, void* out, int out_bf16,
                               cudaStream_t s) {
  const uint64_t groups = rows * cols / 16;
  if (groups == 0) return cudaSuccess;
  if (out_bf16) bfp8_decode_kernel<true><<<grid_for(groups), 256, 0, s>>>(datums, exps, groups, out);
  else bfp8_decode_kernel<false><<<grid_for(groups), 256, 0, s>>>(datums, exps, groups, out);
  return cudaGetLastError();
}

bool gemm_skinny_bfp_supported(uint64_t m, uint64_t n, uint64_t k) {
  if (!(m >= 1 && m <= 4 && n >= 16 && n % 16 == 0 && k >= 1)) return false;
  const uint64_t mt = m <= 1 ? 1 : (m <= 2 ? 2 : 4);
  return (mt * k + (uint64_t)(SKB_THREADS / 32) * mt * SKB_COLS) * sizeof(float) <= 200 * 1024;
}

cudaError_t launch_gemm_skinny_bfp(const uint16_t* a, uint64_t lda, const uint8_t* datums, const uint8_t* exps, void* c, uint64_t ldc,
                                   int out_bf16, uint64_t m, uint64_t n, uint64_t k, cudaStream_t stream) {
  const int mt = m <= 1 ? 1 : (m <= 2 ? 2 : 4);
  const size_t smem = ((size_t)mt * k + (size_t)(SKB_THREADS / 32) * mt * SKB_COLS) * sizeof(float);
  const unsigned grid = (unsigned)((n + SKB_COLS - 1) / SKB_COLS);
#define GO(MT)                                                                                                      \
  do {                                                                                                              \
    const cudaError_t e = ensure_dynamic_smem((const void*)gemm_skinny_bfp_kernel<MT>, smem);                       \
    if (e != cudaSuccess) return e;                                                                                 \
    launch_pdl(gemm_skinny_bfp_kernel<MT>, dim3(grid), dim3(SKB_THREADS), smem, stream, a, lda, datums, exps, c, ldc, out_bf16, \
               (int)m, n, (int)k);                                                                                  \
  } while (0)
  if (mt == 1) GO(1); else if (mt == 2) GO(2); else GO(4);
#undef GO
  return cudaGetLastError();
}

}  // namespace b200
