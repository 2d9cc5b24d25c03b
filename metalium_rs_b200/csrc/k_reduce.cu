// Reductions, row softmax, RMS statistics / RMSNorm and row argmax.
//
//  - reduce: crates/tt-kernels/src/sfpu/reduce.rs:56 (`ReduceOp`), :117 (`Axis`).
//    Sum over rows is a left fold from +0.0, top to bottom, one thread a column
//    (reduce.rs:31-38, :296): bit for bit a sequential sum.  Sums over columns use a
//    fixed tree, so a result never depends on the launch.
//  - full sum / mean: crates/burn-tt/src/ops.rs:3246-3398.  Two stages in a fixed order.
//  - softmax rows: crates/tt-kernels/src/sfpu/softmax.rs:1-45; one read and one write of
//    the scores, the row held in registers between the three phases.
//  - rms / rms_norm: crates/tt-kernels/src/sfpu/norm.rs:1-25.
//  - argmax: first maximum, first NaN wins (crates/tt-tests/tests/step211_argmax_row.rs:8-10).
//
// Compiled with -fmad=false so every rounding the reference names is kept.
#include <cooperative_groups.h>
#include <float.h>
#include <stdio.h>
#include <stdlib.h>

#include <mutex>
#include <string>

#include "eltwise_ev.cuh"
#include "kernels.h"
#include "pdl.cuh"

namespace b200 {
namespace {

enum { SUM = 0, MAX = 1, PROD = 2, ALL = 3, ANY = 4, BITOR = 5, SUM_I32 = 6, PROD_I32 = 7, MIN_I32 = 8, MAX_I32 = 9 };

template <int OP> __device__ __forceinline__ uint32_t identity() {
  if constexpr (OP == MAX) return 0xff800000u;
  else if constexpr (OP == PROD) return 0x3f800000u;
  else if constexpr (OP == ALL || OP == PROD_I32) return 1u;
  else if constexpr (OP == MIN_I32) return 0x7fffffffu;
  else if constexpr (OP == MAX_I32) return 0x80000000u;
  else return 0u;
}
// Total order on float bits in which a positive NaN is above everything (reduce.rs:24-26).
__device__ __forceinline__ uint32_t order_key(uint32_t u) {
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
template <int OP> __device__ __forceinline__ uint32_t combine(uint32_t acc, uint32_t x) {
  if constexpr (OP == SUM) return __float_as_uint(__uint_as_float(acc) + __uint_as_float(x));
  else if constexpr (OP == MAX) return order_key(acc) < order_key(x) ? x : acc;
  else if constexpr (OP == PROD) return __float_as_uint(__uint_as_float(acc) * __uint_as_float(x));
  else if constexpr (OP == ALL) return (acc != 0 && x != 0) ? 1u : 0u;
  else if constexpr (OP == ANY) return (acc != 0 || x != 0) ? 1u : 0u;
  else if constexpr (OP == BITOR) return acc | x;
  else if constexpr (OP == SUM_I32) return acc + x;
  else if constexpr (OP == PROD_I32) return acc * x;
  else if constexpr (OP == MIN_I32) return (int32_t)x < (int32_t)acc ? x : acc;
  else return (int32_t)x > (int32_t)acc ? x : acc;
}

// The finishing kind of a reduction (tensor.rs:6038 `ReduceThen`): exact unary kinds only.
__device__ __forceinline__ uint32_t apply_then(uint32_t v, uint32_t then_kind, uint32_t then_bits) {
  const float s = __uint_as_float(then_bits);
  switch (then_kind) {
    case 0: return v;
    case kind::NEG: return ev<kind::NEG>(v, 0, 0, s, 0.f, nullptr);
    case kind::ABS: return ev<kind::ABS>(v, 0, 0, s, 0.f, nullptr);
    case kind::SIGN: return ev<kind::SIGN>(v, 0, 0, s, 0.f, nullptr);
    case kind::RELU: return ev<kind::RELU>(v, 0, 0, s, 0.f, nullptr);
    case kind::CLAMP_MIN: return ev<kind::CLAMP_MIN>(v, 0, 0, s, 0.f, nullptr);
    case kind::CLAMP_MAX: return ev<kind::CLAMP_MAX>(v, 0, 0, s, 0.f, nullptr);
    case kind::INT_ABS: return ev<kind::INT_ABS>(v, 0, 0, s, 0.f, nullptr);
    default: return v;
  }
}

__device__ __forceinline__ uint32_t ld_word(const void* p, int bf16, uint64_t i) {
  if (bf16) return (uint32_t)reinterpret_cast<const uint16_t*>(p)[i] << 16;
  return reinterpret_cast<const uint32_t*>(p)[i];
}

// ---- over rows: [rows, cols] -> [1, cols]; in order, one thread a column ----------
template <int OP>
__global__ void __launch_bounds__(128)
reduce_rows_kernel(const void* a, int bf16, uint64_t rows, uint64_t cols, uint32_t then_kind,
                   uint32_t then_bits, uint32_t* out) {
  const uint64_t c = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  uint32_t acc = identity<OP>();
  uint64_t r = 0;
  constexpr int U = 16;
  for (; r + U <= rows; r += U) {
    uint32_t v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = ld_word(a, bf16, (r + u) * cols + c);
#pragma unroll
    for (int u = 0; u < U; ++u) acc = combine<OP>(acc, v[u]);
  }
  for (; r < rows; ++r) acc = combine<OP>(acc, ld_word(a, bf16, r * cols + c));
  out[c] = apply_then(acc, then_kind, then_bits);
}

// ---- over columns: [rows, cols] -> [rows, 1] ----------------------------------
template <int OP> __device__ __forceinline__ uint32_t warp_reduce(uint32_t v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = combine<OP>(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// THREADS threads a row (32: a warp a row, several rows a block).
template <int OP, int THREADS>
__global__ void __launch_bounds__(256)
reduce_cols_kernel(const void* a, int bf16, uint64_t rows, uint64_t cols, uint32_t then_kind,
                   uint32_t then_bits, uint32_t* out) {
  constexpr int ROWS_PER_BLOCK = 256 / THREADS;
  __shared__ uint32_t part[8];
  const int lane_in_row = threadIdx.x % THREADS;
  const int sub = threadIdx.x / THREADS;
  for (uint64_t row0 = (uint64_t)blockIdx.x * ROWS_PER_BLOCK; row0 < rows;
       row0 += (uint64_t)gridDim.x * ROWS_PER_BLOCK) {
    const uint64_t row = row0 + sub;
    uint32_t acc = identity<OP>();
    if (row < rows) {
      const uint64_t base = row * cols;
      const bool vec = !bf16 && (cols % 4 == 0) &&
                       ((reinterpret_cast<uintptr_t>(a) & 15) == 0);
      if (vec) {
        const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const uint32_t*>(a) + base);
        const uint64_t n4 = cols / 4;
        uint32_t a0 = identity<OP>(), a1 = a0, a2 = a0, a3 = a0;
        for (uint64_t i = lane_in_row; i < n4; i += THREADS) {
          const uint4 v = __ldcs(p + i);
          a0 = combine<OP>(a0, v.x); a1 = combine<OP>(a1, v.y);
          a2 = combine<OP>(a2, v.z); a3 = combine<OP>(a3, v.w);
        }
        acc = combine<OP>(combine<OP>(a0, a1), combine<OP>(a2, a3));
      } else {
        for (uint64_t i = lane_in_row; i < cols; i += THREADS)
          acc = combine<OP>(acc, ld_word(a, bf16, base + i));
      }
    }
    acc = warp_reduce<OP>(acc);
    if constexpr (THREADS == 32) {
      if (lane_in_row == 0 && row < rows) out[row] = apply_then(acc, then_kind, then_bits);
    } else {
      if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
      __syncthreads();
      if (threadIdx.x == 0) {
        uint32_t t = part[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) t = combine<OP>(t, part[w]);
        out[row] = apply_then(t, then_kind, then_bits);
      }
      __syncthreads();
    }
  }
}

template <int OP>
cudaError_t launch_reduce_op(const void* a, int bf16, uint64_t rows, uint64_t cols, int axis,
                             uint32_t tk, uint32_t tb, void* out, cudaStream_t s) {
  uint32_t* o = reinterpret_cast<uint32_t*>(out);
  if (axis == 0) {
    reduce_rows_kernel<OP><<<(unsigned)((cols + 127) / 128), 128, 0, s>>>(a, bf16, rows, cols, tk, tb, o);
  } else if (cols >= 2048) {
    uint64_t grid = rows < 148ull * 16 ? rows : 148ull * 16;
    reduce_cols_kernel<OP, 256><<<(unsigned)grid, 256, 0, s>>>(a, bf16, rows, cols, tk, tb, o);
  } else {
    uint64_t grid = (rows + 7) / 8;
    if (grid > 148ull * 16) grid = 148ull * 16;
    reduce_cols_kernel<OP, 32><<<(unsigned)grid, 256, 0, s>>>(a, bf16, rows, cols, tk, tb, o);
  }
  return cudaGetLastError();
}

// ---- full sum -----------------------------------------------------------------
constexpr int FULL_BLOCKS = 148 * 8;
constexpr int FULL_THREADS = 256;

__device__ __forceinline__ float block_sum_256(float v, float* sm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = v + __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  if (threadIdx.x == 0) {
    t = sm[0];
    for (int w = 1; w < FULL_THREADS / 32; ++w) t = t + sm[w];
  }
  __syncthreads();
  return t;  // valid in thread 0
}

// One launch: every block leaves its partial, and the block that takes the last ticket adds the
// partials in index order (so the bits do not depend on which block that is) and resets the
// ticket.  scratch: FULL_BLOCKS partials, then the ticket word, which must be zero at entry.
__global__ void __launch_bounds__(FULL_THREADS)
full_sum_fused(const float* __restrict__ a, uint64_t n, int mean, float* __restrict__ scratch,
               float* __restrict__ out) {
  __shared__ float sm[FULL_THREADS / 32];
  __shared__ int is_last;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  const bool vec = (reinterpret_cast<uintptr_t>(a) & 15) == 0;
  const uint64_t n4 = vec ? n / 4 : 0;
  const float4* p = reinterpret_cast<const float4*>(a);
  const uint64_t stride = (uint64_t)gridDim.x * FULL_THREADS;
  uint64_t i = (uint64_t)blockIdx.x * FULL_THREADS + threadIdx.x;
  for (; i + 3 * stride < n4; i += 4 * stride) {
    const float4 v0 = __ldcs(p + i), v1 = __ldcs(p + i + stride), v2 = __ldcs(p + i + 2 * stride),
                 v3 = __ldcs(p + i + 3 * stride);
    s0 = s0 + ((v0.x + v0.y) + (v0.z + v0.w));
    s1 = s1 + ((v1.x + v1.y) + (v1.z + v1.w));
    s2 = s2 + ((v2.x + v2.y) + (v2.z + v2.w));
    s3 = s3 + ((v3.x + v3.y) + (v3.z + v3.w));
  }
  for (; i < n4; i += stride) {
    const float4 v0 = __ldcs(p + i);
    s0 = s0 + ((v0.x + v0.y) + (v0.z + v0.w));
  }
  for (uint64_t j = n4 * 4 + (uint64_t)blockIdx.x * FULL_THREADS + threadIdx.x; j < n; j += stride)
    s1 = s1 + a[j];
  const float t = block_sum_256((s0 + s1) + (s2 + s3), sm);
  unsigned int* ticket = reinterpret_cast<unsigned int*>(scratch + FULL_BLOCKS);
  if (threadIdx.x == 0) {
    scratch[blockIdx.x] = t;
    __threadfence();
    is_last = (atomicAdd(ticket, 1u) == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  float s = 0.f;
  for (int k = threadIdx.x; k < FULL_BLOCKS; k += FULL_THREADS) s = s + __ldcg(scratch + k);
  const float total = block_sum_256(s, sm);
  if (threadIdx.x == 0) {
    out[0] = mean ? total / (float)n : total;  // sum DIV_SCALAR n (ops.rs:3260-3270)
    *ticket = 0u;
  }
}

// ---- softmax rows -----------------------------------------------------------------
__device__ __forceinline__ float nan_max(float a, float b) {
  return (a != a) ? a : ((b != b) ? b : fmaxf(a, b));
}
// The maximum ignores NaNs (fmaxf): a NaN in a row reaches every output of the row anyway,
// through exp(NaN - m) and the sum, which is what a NaN-propagating maximum would give.
template <int THREADS> __device__ __forceinline__ float block_max(float v, float* sm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if constexpr (THREADS == 32) return v;
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = sm[0];
  for (int w = 1; w < THREADS / 32; ++w) t = fmaxf(t, sm[w]);
  __syncthreads();
  return t;
}
template <int THREADS> __device__ __forceinline__ float block_add(float v, float* sm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = v + __shfl_xor_sync(0xffffffffu, v, o);
  if constexpr (THREADS == 32) return v;
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = sm[0];
  for (int w = 1; w < THREADS / 32; ++w) t = t + sm[w];
  __syncthreads();
  return t;
}

// Four results of a row at float4 index i: F32, or rounded once to BF16.
__device__ __forceinline__ void store4(void* row, uint32_t i, float4 t, int bf16) {
  if (bf16) {
    uint2 o;
    o.x = (uint32_t)f32_to_bf16_bits(__float_as_uint(t.x)) | ((uint32_t)f32_to_bf16_bits(__float_as_uint(t.y)) << 16);
    o.y = (uint32_t)f32_to_bf16_bits(__float_as_uint(t.z)) | ((uint32_t)f32_to_bf16_bits(__float_as_uint(t.w)) << 16);
    __stcs(reinterpret_cast<uint2*>(row) + i, o);
  } else {
    __stcs(reinterpret_cast<float4*>(row) + i, t);
  }
}
__device__ __forceinline__ void store1(void* row, uint64_t i, float v, int bf16) {
  if (bf16) reinterpret_cast<uint16_t*>(row)[i] = f32_to_bf16_bits(__float_as_uint(v));
  else reinterpret_cast<float*>(row)[i] = v;
}

__device__ __forceinline__ float scaled_masked(float x, uint32_t m, float scale, bool has_scale) {
  const float s = has_scale ? x * scale : x;
  return m ? -INFINITY : s;
}

// One block a row; the row lives in registers: VPT float4 per thread.
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
softmax_block_kernel(const float* __restrict__ x, const uint32_t* __restrict__ mask, uint64_t mask_rows,
                     float scale, int log_form, void* __restrict__ out, int out_bf16, uint64_t rows, uint32_t cols) {
  __shared__ float sm[32];
  const uint32_t n4 = cols / 4;
  const bool has_scale = scale != 1.0f;
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float4* xr = reinterpret_cast<const float4*>(x + row * cols);
    const uint4* mr = mask ? reinterpret_cast<const uint4*>(mask + (row % mask_rows) * cols) : nullptr;
    float4 v[VPT];
    float m = -INFINITY;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const uint32_t i = threadIdx.x + u * THREADS;
      if (i < n4) {
        float4 t = __ldcs(xr + i);
        if (mr || has_scale) {
          uint4 k = mr ? __ldg(mr + i) : make_uint4(0, 0, 0, 0);
          t.x = scaled_masked(t.x, k.x, scale, has_scale);
          t.y = scaled_masked(t.y, k.y, scale, has_scale);
          t.z = scaled_masked(t.z, k.z, scale, has_scale);
          t.w = scaled_masked(t.w, k.w, scale, has_scale);
        }
        v[u] = t;
        m = fmaxf(m, fmaxf(fmaxf(t.x, t.y), fmaxf(t.z, t.w)));
      }
    }
    m = block_max<THREADS>(m, sm);
    m = (m < -FLT_MAX) ? -FLT_MAX : m;  // clamp: a fully masked row (sfpu/softmax.rs:37-43)
    float s = 0.f;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const uint32_t i = threadIdx.x + u * THREADS;
      if (i < n4) {
        float4 t = v[u];
        if (log_form) {
          t.x = t.x - m; t.y = t.y - m; t.z = t.z - m; t.w = t.w - m;
          v[u] = t;
          s = s + ((expf(t.x) + expf(t.y)) + (expf(t.z) + expf(t.w)));
        } else {
          t.x = expf(t.x - m); t.y = expf(t.y - m); t.z = expf(t.z - m); t.w = expf(t.w - m);
          v[u] = t;
          s = s + ((t.x + t.y) + (t.z + t.w));
        }
      }
    }
    s = block_add<THREADS>(s, sm);
    void* orow = reinterpret_cast<char*>(out) + row * cols * (out_bf16 ? 2 : 4);
    if (log_form) {
      const float l = logf(s);
#pragma unroll
      for (int u = 0; u < VPT; ++u) {
        const uint32_t i = threadIdx.x + u * THREADS;
        if (i < n4) {
          float4 t = v[u];
          t.x = t.x - l; t.y = t.y - l; t.z = t.z - l; t.w = t.w - l;
          store4(orow, i, t, out_bf16);
        }
      }
    } else {
      s = (s < FLT_MIN) ? FLT_MIN : s;
      const float inv = 1.0f / s;  // one division a row, then products: 1.5 u against DIV's 0.5 u
#pragma unroll
      for (int u = 0; u < VPT; ++u) {
        const uint32_t i = threadIdx.x + u * THREADS;
        if (i < n4) {
          float4 t = v[u];
          t.x = t.x * inv; t.y = t.y * inv; t.z = t.z * inv; t.w = t.w * inv;
          store4(orow, i, t, out_bf16);
        }
      }
    }
  }
}

// Wide rows: a thread-block cluster a row.  Each of the C CTAs (256 threads) keeps its
// share of the row in registers and the CTAs exchange their partial maximum and sum through
// distributed shared memory, combined in rank order so every CTA holds the same bits.
// Several clusters are resident per SM at different phases, so one row's loads overlap
// another's exponentials and stores; a single 1024-thread block a row cannot do that.
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
softmax_cluster_kernel(const float* __restrict__ x, const uint32_t* __restrict__ mask, uint64_t mask_rows,
                       float scale, int log_form, void* __restrict__ out, int out_bf16, uint64_t rows, uint32_t cols) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned csize = cluster.num_blocks();
  const unsigned crank = cluster.block_rank();
  __shared__ float sm[32];
  __shared__ float xchg[2][2];  // [row parity][0 max, 1 sum], read by the peers
  const uint32_t n4 = cols / 4;
  const uint32_t share = (n4 + csize - 1) / csize;
  const uint32_t first = crank * share;
  const uint32_t last = (first + share < n4) ? first + share : n4;
  const bool has_scale = scale != 1.0f;
  const uint64_t n_clusters = gridDim.x / csize;
  int par = 0;
  for (uint64_t row = blockIdx.x / csize; row < rows; row += n_clusters, par ^= 1) {
    const float4* xr = reinterpret_cast<const float4*>(x + row * cols);
    const uint4* mr = mask ? reinterpret_cast<const uint4*>(mask + (row % mask_rows) * cols) : nullptr;
    float4 v[VPT];
    float m = -INFINITY;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const uint32_t i = first + threadIdx.x + u * THREADS;
      if (i < last) {
        float4 t = __ldcs(xr + i);
        if (mr || has_scale) {
          uint4 k = mr ? __ldg(mr + i) : make_uint4(0, 0, 0, 0);
          t.x = scaled_masked(t.x, k.x, scale, has_scale);
          t.y = scaled_masked(t.y, k.y, scale, has_scale);
          t.z = scaled_masked(t.z, k.z, scale, has_scale);
          t.w = scaled_masked(t.w, k.w, scale, has_scale);
        }
        v[u] = t;
        m = fmaxf(m, fmaxf(fmaxf(t.x, t.y), fmaxf(t.z, t.w)));
      }
    }
    m = block_max<THREADS>(m, sm);
    if (csize > 1) {
      if (threadIdx.x == 0) xchg[par][0] = m;
      cluster.sync();
      m = *cluster.map_shared_rank(&xchg[par][0], 0);
      for (unsigned r = 1; r < csize; ++r) m = fmaxf(m, *cluster.map_shared_rank(&xchg[par][0], r));
    }
    m = (m < -FLT_MAX) ? -FLT_MAX : m;
    float s = 0.f;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const uint32_t i = first + threadIdx.x + u * THREADS;
      if (i < last) {
        float4 t = v[u];
        if (log_form) {
          t.x = t.x - m; t.y = t.y - m; t.z = t.z - m; t.w = t.w - m;
          v[u] = t;
          s = s + ((expf(t.x) + expf(t.y)) + (expf(t.z) + expf(t.w)));
        } else {
          t.x = expf(t.x - m); t.y = expf(t.y - m); t.z = expf(t.z - m); t.w = expf(t.w - m);
          v[u] = t;
          s = s + ((t.x + t.y) + (t.z + t.w));
        }
      }
    }
    s = block_add<THREADS>(s, sm);
    if (csize > 1) {
      if (threadIdx.x == 0) xchg[par][1] = s;
      cluster.sync();
      s = *cluster.map_shared_rank(&xchg[par][1], 0);
      for (unsigned r = 1; r < csize; ++r) s = s + *cluster.map_shared_rank(&xchg[par][1], r);
    }
    void* orow = reinterpret_cast<char*>(out) + row * cols * (out_bf16 ? 2 : 4);
    if (log_form) {
      const float l = logf(s);
#pragma unroll
      for (int u = 0; u < VPT; ++u) {
        const uint32_t i = first + threadIdx.x + u * THREADS;
        if (i < last) {
          float4 t = v[u];
          t.x = t.x - l; t.y = t.y - l; t.z = t.z - l; t.w = t.w - l;
          store4(orow, i, t, out_bf16);
        }
      }
    } else {
      s = (s < FLT_MIN) ? FLT_MIN : s;
      const float inv = 1.0f / s;
#pragma unroll
      for (int u = 0; u < VPT; ++u) {
        const uint32_t i = first + threadIdx.x + u * THREADS;
        if (i < last) {
          float4 t = v[u];
          t.x = t.x * inv; t.y = t.y * inv; t.z = t.z * inv; t.w = t.w * inv;
          store4(orow, i, t, out_bf16);
        }
      }
    }
  }
  if (csize > 1) cluster.sync();  // no CTA leaves while a peer may still read its exchange slots
}

// Rows of 4,097..32,768 columns: a persistent block of 512 threads an SM, split into workers of T
// threads (T = 128, 256 or 512: the smallest with 16 float4 a thread covering the row).  A worker
// keeps its row in registers; shared memory holds the NEXT row, fetched by cp.async while this one
// is reduced, exponentiated and stored, so loads never wait for arithmetic.  Each thread reads and
// refills only its own shared-memory slots: the only synchronisation is the worker's two
// reductions (named barriers).
template <int T>
__global__ void __launch_bounds__(512, 1)
softmax_workers_kernel(const float* __restrict__ x, const uint32_t* __restrict__ mask, uint64_t mask_rows,
                       float scale, int log_form, void* __restrict__ out, int out_bf16, uint64_t rows, uint32_t cols) {
  constexpr int G = 512 / T, WARPS = T / 32, VPT = 16;
  extern __shared__ float4 ring[];               // [G][VPT][T]
  __shared__ float red[2][G][WARPS];
  const int g = threadIdx.x / T, t = threadIdx.x % T, wl = t >> 5;
  float4* mine = ring + (size_t)g * VPT * T + t;
  const uint32_t n4 = cols / 4;
  const bool has_scale = scale != 1.0f;
  const uint64_t nworkers = (uint64_t)gridDim.x * G;
  auto worker_reduce = [&](float v, bool is_max, int which) -> float {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float w = __shfl_xor_sync(0xffffffffu, v, o);
      v = is_max ? fmaxf(v, w) : v + w;
    }
    if ((t & 31) == 0) red[which][g][wl] = v;
    asm volatile("bar.sync %0, %1;" ::"r"(g + 1), "r"(T) : "memory");
    float r = red[which][g][0];
#pragma unroll
    for (int w = 1; w < WARPS; ++w) r = is_max ? fmaxf(r, red[which][g][w]) : r + red[which][g][w];
    return r;  // red[which] is not rewritten before the worker's next barrier on the other slot
  };
  auto prefetch = [&](uint64_t row) {
    const float4* xr = reinterpret_cast<const float4*>(x + row * cols) + t;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      if (t + u * T < n4) {
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(mine + u * T);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(xr + u * T) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  uint64_t row = (uint64_t)blockIdx.x * G + g;
  if (row < rows) prefetch(row);
  for (; row < rows; row += nworkers) {
    const uint4* mr = mask ? reinterpret_cast<const uint4*>(mask + (row % mask_rows) * cols) : nullptr;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    float4 v[VPT];
    float m = -INFINITY;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const uint32_t i = t + u * T;
      if (i < n4) {
        float4 q = mine[u * T];
        if (mr || has_scale) {
          const uint4 k = mr ? __ldg(mr + i) : make_uint4(0, 0, 0, 0);
          q.x = scaled_masked(q.x, k.x, scale, has_scale); q.y = scaled_masked(q.y, k.y, scale, has_scale);
          q.z = scaled_masked(q.z, k.z, scale, has_scale); q.w = scaled_masked(q.w, k.w, scale, has_scale);
        }
        v[u] = q;
        m = fmaxf(m, fmaxf(fmaxf(q.x, q.y), fmaxf(q.z, q.w)));
      }
    }
    // every slot of this thread has been read (m depends on all of them): refill them
    asm volatile("" ::"f"(m) : "memory");
    if (row + nworkers < rows) prefetch(row + nworkers);
    m = worker_reduce(m, true, 0);
    m = (m < -FLT_MAX) ? -FLT_MAX : m;
    float sum = 0.f;
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      if (t + u * T < n4) {
        float4 q = v[u];
        if (log_form) {
          q.x -= m; q.y -= m; q.z -= m; q.w -= m;
          sum = sum + ((expf(q.x) + expf(q.y)) + (expf(q.z) + expf(q.w)));
        } else {
          q.x = expf(q.x - m); q.y = expf(q.y - m); q.z = expf(q.z - m); q.w = expf(q.w - m);
          sum = sum + ((q.x + q.y) + (q.z + q.w));
        }
        v[u] = q;
      }
    }
    sum = worker_reduce(sum, false, 1);
    void* orow = reinterpret_cast<char*>(out) + row * cols * (out_bf16 ? 2 : 4);
    const float l = log_form ? logf(sum) : 0.f;
    const float inv = 1.0f / ((sum < FLT_MIN) ? FLT_MIN : sum);
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
      const uint32_t i = t + u * T;
      if (i < n4) {
        float4 q = v[u];
        if (log_form) { q.x -= l; q.y -= l; q.z -= l; q.w -= l; }
        else { q.x *= inv; q.y *= inv; q.z *= inv; q.w *= inv; }
        store4(orow, i, q, out_bf16);
      }
    }
  }
}

// Any width: a block a row, three passes over global memory (the second and third
// mostly from L2).  Rows too short or ragged for the register kernel, or too long.
__global__ void __launch_bounds__(256)
softmax_stream_kernel(const float* __restrict__ x, const uint32_t* __restrict__ mask, uint64_t mask_rows,
                      float scale, int log_form, void* __restrict__ out, int out_bf16, uint64_t rows, uint64_t cols) {
  __shared__ float sm[32];
  const bool has_scale = scale != 1.0f;
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * cols;
    const uint32_t* mr = mask ? mask + (row % mask_rows) * cols : nullptr;
    float m = -INFINITY;
    for (uint64_t i = threadIdx.x; i < cols; i += 256)
      m = fmaxf(m, scaled_masked(xr[i], mr ? mr[i] : 0u, scale, has_scale));
    m = block_max<256>(m, sm);
    m = (m < -FLT_MAX) ? -FLT_MAX : m;
    float s = 0.f;
    for (uint64_t i = threadIdx.x; i < cols; i += 256)
      s = s + expf(scaled_masked(xr[i], mr ? mr[i] : 0u, scale, has_scale) - m);
    s = block_add<256>(s, sm);
    void* orow = reinterpret_cast<char*>(out) + row * cols * (out_bf16 ? 2 : 4);
    if (log_form) {
      const float l = logf(s);
      for (uint64_t i = threadIdx.x; i < cols; i += 256)
        store1(orow, i, (scaled_masked(xr[i], mr ? mr[i] : 0u, scale, has_scale) - m) - l, out_bf16);
    } else {
      s = (s < FLT_MIN) ? FLT_MIN : s;
      for (uint64_t i = threadIdx.x; i < cols; i += 256)
        store1(orow, i, expf(scaled_masked(xr[i], mr ? mr[i] : 0u, scale, has_scale) - m) / s, out_bf16);
    }
  }
}

// ---- rms / rms_norm -------------------------------------------------------------
__device__ __forceinline__ float ld_f(const void* p, int bf16, uint64_t i) {
  return __uint_as_float(ld_word(p, bf16, i));
}

// One warp a row.  stat = sqrt(sumsq * (1/n) + eps): MUL_SCALAR, ADD_SCALAR, SQRT (norm.rs:45-60).
__global__ void __launch_bounds__(256)
rms_norm_kernel(const void* a, int a_bf16, const void* b, int b_bf16, const void* gamma, int g_bf16,
                float eps, void* sum_out, int sum_bf16, void* norm_out, int norm_bf16, float* stat_out,
                uint64_t rows, uint64_t cols) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint64_t nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  const float inv = 1.0f / (float)cols;
  for (uint64_t row = warp; row < rows; row += nwarps) {
    const uint64_t base = row * cols;
    float ss = 0.f;
    for (uint64_t i = lane; i < cols; i += 32) {
      float v = ld_f(a, a_bf16, base + i);
      if (b) {
        v = v + ld_f(b, b_bf16, base + i);
        if (sum_out) {
          if (sum_bf16) {
            const uint16_t h = f32_to_bf16_bits(__float_as_uint(v));
            reinterpret_cast<uint16_t*>(sum_out)[base + i] = h;
            v = bf16_bits_to_f32(h);  // the norm reads the sum as it was stored
          } else {
            reinterpret_cast<float*>(sum_out)[base + i] = v;
          }
        }
      }
      ss = ss + v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss = ss + __shfl_xor_sync(0xffffffffu, ss, o);
    const float stat = sqrtf(ss * inv + eps);
    if (stat_out) { if (lane == 0) stat_out[row] = stat; }
    if (norm_out) {
      for (uint64_t i = lane; i < cols; i += 32) {
        float v;
        if (b && sum_out) v = ld_f(sum_out, sum_bf16, base + i);
        else if (b) v = ld_f(a, a_bf16, base + i) + ld_f(b, b_bf16, base + i);
        else v = ld_f(a, a_bf16, base + i);
        float r = v / stat;
        if (gamma) r = r * ld_f(gamma, g_bf16, i);
        if (norm_bf16) reinterpret_cast<uint16_t*>(norm_out)[base + i] = f32_to_bf16_bits(__float_as_uint(r));
        else reinterpret_cast<float*>(norm_out)[base + i] = r;
      }
    }
  }
}

// F32 rows of up to 1024 columns, no residual: a warp a row, the row kept in registers between
// the sum of squares and the division (one read, one write).  Same roundings as the general kernel.
// ADD: the row is a + b (one rounding), also written to sum_out.
template <int V, bool ADD>
__global__ void __launch_bounds__(256)
rms_norm_rows_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ sum_out,
                     const void* __restrict__ gamma, int g_bf16, float eps,
                     void* __restrict__ out, int out_bf16, uint64_t rows, uint32_t cols) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint64_t nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  const uint32_t n4 = cols / 4;
  const float inv = 1.0f / (float)cols;
  for (uint64_t row = warp; row < rows; row += nwarps) {
    const float4* p = reinterpret_cast<const float4*>(a + row * cols);
    float4 v[V];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < V; ++u) {
      const uint32_t i = lane + u * 32;
      if (i < n4) {
        v[u] = p[i];
        if constexpr (ADD) {
          const float4 w = reinterpret_cast<const float4*>(b + row * cols)[i];
          v[u].x = v[u].x + w.x; v[u].y = v[u].y + w.y; v[u].z = v[u].z + w.z; v[u].w = v[u].w + w.w;
          reinterpret_cast<float4*>(sum_out + row * cols)[i] = v[u];
        }
        ss = ss + ((v[u].x * v[u].x + v[u].y * v[u].y) + (v[u].z * v[u].z + v[u].w * v[u].w));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss = ss + __shfl_xor_sync(0xffffffffu, ss, o);
    const float stat = sqrtf(ss * inv + eps);
    void* orow = reinterpret_cast<char*>(out) + row * cols * (out_bf16 ? 2 : 4);
#pragma unroll
    for (int u = 0; u < V; ++u) {
      const uint32_t i = lane + u * 32;
      if (i < n4) {
        float4 t = v[u];
        t.x = t.x / stat; t.y = t.y / stat; t.z = t.z / stat; t.w = t.w / stat;
        if (gamma) {
          float4 g;
          if (g_bf16) {
            const uint2 h = reinterpret_cast<const uint2*>(gamma)[i];
            g.x = __uint_as_float(h.x << 16); g.y = __uint_as_float(h.x & 0xffff0000u);
            g.z = __uint_as_float(h.y << 16); g.w = __uint_as_float(h.y & 0xffff0000u);
          } else {
            g = reinterpret_cast<const float4*>(gamma)[i];
          }
          t.x = t.x * g.x; t.y = t.y * g.y; t.z = t.z * g.z; t.w = t.w * g.w;
        }
        if (out_bf16) {
          uint2 o2;
          o2.x = (uint32_t)f32_to_bf16_bits(__float_as_uint(t.x)) | ((uint32_t)f32_to_bf16_bits(__float_as_uint(t.y)) << 16);
          o2.y = (uint32_t)f32_to_bf16_bits(__float_as_uint(t.z)) | ((uint32_t)f32_to_bf16_bits(__float_as_uint(t.w)) << 16);
          reinterpret_cast<uint2*>(orow)[i] = o2;
        } else {
          reinterpret_cast<float4*>(orow)[i] = t;
        }
      }
    }
  }
}

// ---- argmax ---------------------------------------------------------------------
struct Best { float v; uint32_t i; };
__device__ __forceinline__ bool better(float v, uint32_t i, float bv, uint32_t bi) {
  const bool vn = v != v, bn = bv != bv;
  if (vn || bn) return vn && (!bn || i < bi);
  return v > bv || (v == bv && i < bi);
}
__global__ void __launch_bounds__(1024)
argmax_rows_kernel(const float* __restrict__ a, uint64_t rows, uint64_t cols, int32_t* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ uint32_t si[32];
  for (uint64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* p = a + row * cols;
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;
    // eight of a thread's values asked for before the first is compared: one block reads a row, so a load a compare
    // made a 49,152-column row (a decode step's logits) 48 trips to memory one after the other
    for (uint64_t base = threadIdx.x; base < cols; base += 8ull * blockDim.x) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint64_t i = base + (uint64_t)u * blockDim.x;
        v[u] = i < cols ? p[i] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint64_t i = base + (uint64_t)u * blockDim.x;
        if (i < cols && better(v[u], (uint32_t)i, bv, bi)) { bv = v[u]; bi = (uint32_t)i; }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      const int nw = (blockDim.x + 31) / 32;
      for (int w = 1; w < nw; ++w)
        if (better(sv[w], si[w], bv, bi)) { bv = sv[w]; bi = si[w]; }
      out[row] = (int32_t)bi;
    }
    __syncthreads();
  }
}

// A few long rows (a decode step's logits: one to four rows of 49,152): one block a row read the row at a single SM's rate
// (10.5 us for 196 KB).  Here the eight blocks of a thread-block cluster take an eighth of the row each, hand their best
// (value, index) to the first block's shared memory and meet at the cluster barrier (every block arrives whatever it
// found, so it cannot stall); the first block joins them in rank order.  `better` orders by value, then index, so the
// result does not depend on how the row was cut.
constexpr int ARGMAX_CLUSTER = 8;
__global__ void __launch_bounds__(512)
argmax_rows_cluster_kernel(const float* __restrict__ a, uint64_t rows, uint64_t cols, int32_t* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ uint32_t si[32];
  __shared__ float pv[ARGMAX_CLUSTER];
  __shared__ uint32_t pi[ARGMAX_CLUSTER];
  uint32_t rank, csize;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(csize));
  const uint64_t row = blockIdx.x / csize;
  const uint64_t seg = ((cols + csize - 1) / csize + 3) / 4 * 4, c0 = rank * seg, c1 = c0 + seg < cols ? c0 + seg : cols;
  const float* p = a + row * cols;
  float bv = -INFINITY;
  uint32_t bi = 0xffffffffu;
  for (uint64_t base = c0 + threadIdx.x; base < c1; base += 8ull * blockDim.x) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint64_t i = base + (uint64_t)u * blockDim.x;
      v[u] = i < c1 ? p[i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint64_t i = base + (uint64_t)u * blockDim.x;
      if (i < c1 && better(v[u], (uint32_t)i, bv, bi)) { bv = v[u]; bi = (uint32_t)i; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int nw = (blockDim.x + 31) / 32;
    for (int w = 1; w < nw; ++w)
      if (better(sv[w], si[w], bv, bi)) { bv = sv[w]; bi = si[w]; }
    // this block's best into the first block's shared memory
    uint32_t rv, ri;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rv) : "r"((uint32_t)__cvta_generic_to_shared(&pv[rank])), "r"(0));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ri) : "r"((uint32_t)__cvta_generic_to_shared(&pi[rank])), "r"(0));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(rv), "f"(bv) : "memory");
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(ri), "r"(bi) : "memory");
  }
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (rank == 0 && threadIdx.x == 0 && row < rows) {
    float fv = pv[0];
    uint32_t fi = pi[0];
    for (uint32_t r = 1; r < csize; ++r)
      if (better(pv[r], pi[r], fv, fi)) { fv = pv[r]; fi = pi[r]; }
    out[row] = (int32_t)fi;
  }
}

}  // namespace

cudaError_t launch_reduce(const void* a, int a_bf16, uint64_t rows, uint64_t cols, int op, int axis,
                          uint32_t tk, uint32_t tb, void* out, cudaStream_t s) {
  if (rows == 0 || cols == 0) return cudaSuccess;
  switch (op) {
    case SUM: return launch_reduce_op<SUM>(a, a_bf16, rows, cols, axis, tk, tb, out, s);
    case MAX: return launch_reduce_op<MAX>(a, a_bf16, rows, cols, axis, tk, tb, out, s);
    case PROD: return launch_reduce_op<PROD>(a, a_bf16, rows, cols, axis, tk, tb, out, s);
    case ALL: return launch_reduce_op<ALL>(a, a_bf16, rows, cols, axis, tk, tb, out, s);
    case ANY: return launch_reduce_op<ANY>(a, a_bf16, rows, cols, axis, tk, tb, out, s);
    case BITOR: return launch_reduce_op<BITOR>(a, a_bf16, rows, cols, axis, tk, tb, out, s);
    case SUM_I32: return launch_reduce_op<SUM_I32>(a, a_bf16, rows, cols, axis, tk, tb, out, s);
    case PROD_I32: return launch_reduce_op<PROD_I32>(a, a_bf16, rows, cols, axis, tk, tb, out, s);
    case MIN_I32: return launch_reduce_op<MIN_I32>(a, a_bf16, rows, cols, axis, tk, tb, out, s);
    case MAX_I32: return launch_reduce_op<MAX_I32>(a, a_bf16, rows, cols, axis, tk, tb, out, s);
    default: return cudaErrorNotSupported;
  }
}

uint64_t full_sum_scratch_floats() { return FULL_BLOCKS + 8; }

cudaError_t launch_full_sum(const float* a, uint64_t n, int mean, float* scratch, float* out,
                            cudaStream_t s) {
  full_sum_fused<<<FULL_BLOCKS, FULL_THREADS, 0, s>>>(a, n, mean, scratch, out);
  return cudaGetLastError();
}

}  // namespace b200

// ---- full sum for callers that cannot allocate -------------------------------------
// Some hosts of this library must not call cudaMalloc at all: a process whose device memory
// is owned and budgeted by another runtime (a serving stack that hands out fixed arenas and
// treats any allocation of its own as a leak), or code that runs where allocating would
// synchronise the device at the wrong moment.  For them the two-stage sum's per-block
// partials live in a fixed array inside the library image instead of in a buffer the
// engine allocates.  Every GPU that loads the library holds these 4,768 bytes until exit.
namespace {
constexpr uint64_t NOALLOC_MAX_ELEMS = 1ull << 31;  // the largest input accepted (8 GiB of F32)
constexpr int NOALLOC_MAX_DEVICES = 64;
static __device__ __align__(256) float g_full_sum_partials[b200::FULL_BLOCKS + 8];  // partials, then the ticket word
float* g_partials_addr[NOALLOC_MAX_DEVICES] = {};
std::mutex g_partials_lock;
}  // namespace

// No counterpart in the reference.  See include/b200tt.h for the contract.
extern "C" __attribute__((visibility("default")))
int32_t b200_full_sum_noalloc(const float* device_values, uint64_t n, int32_t mean, float* device_out,
                              void* cuda_stream) {
  if (!device_values || !device_out) {
    b200::set_global_error("full_sum_noalloc: a null device pointer");
    return 2;
  }
  if (n > NOALLOC_MAX_ELEMS) {
    char msg[160];
    snprintf(msg, sizeof msg, "full_sum_noalloc: %llu elements exceed the limit of %llu",
             (unsigned long long)n, (unsigned long long)NOALLOC_MAX_ELEMS);
    b200::set_global_error(msg);
    return 2;
  }
  if (n == 0 && mean) {   // 0 / 0: refused rather than a NaN handed back without a word
    b200::set_global_error("full_sum_noalloc: the mean of no elements is undefined");
    return 2;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) {
    b200::set_global_error("full_sum_noalloc: no current CUDA device");
    return 3;
  }
  float* partials = nullptr;
  {
    // Set-up, once per device, with that device current: in host code the array's name is
    // only a stand-in, so ask the runtime for the address the kernels must be given.
    std::lock_guard<std::mutex> hold(g_partials_lock);
    if (!g_partials_addr[dev]) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_full_sum_partials);
      if (e != cudaSuccess || !p) {
        cudaGetLastError();
        b200::set_global_error((std::string("full_sum_noalloc: cudaGetSymbolAddress: ") + cudaGetErrorString(e)).c_str());
        return 3;
      }
      g_partials_addr[dev] = static_cast<float*>(p);
    }
    partials = g_partials_addr[dev];
  }
  // Every partial is rewritten before it is read, so the last call's partials do not matter.  The
  // one word that must start at zero is the ticket after them.  The block that finishes a call puts
  // it back to zero, but a launch that died half-way, or two calls that overlapped, can leave it
  // counting; so it is cleared here, on the caller's stream ahead of the kernel (a memset node, no
  // allocation), and one bad call cannot spoil the ones after it.
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  e = cudaMemsetAsync(partials + b200::FULL_BLOCKS, 0, 8 * sizeof(float), s);
  if (e != cudaSuccess) {
    b200::set_global_error((std::string("full_sum_noalloc: clearing the ticket: ") + cudaGetErrorString(e)).c_str());
    return 3;
  }
  b200::full_sum_fused<<<b200::FULL_BLOCKS, b200::FULL_THREADS, 0, s>>>(device_values, n, mean, partials, device_out);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    b200::set_global_error((std::string("full_sum_noalloc: launch: ") + cudaGetErrorString(e)).c_str());
    return 3;
  }
  return 0;
}

namespace b200 {

cudaError_t launch_softmax_rows(const float* x, const uint32_t* mask, uint64_t mask_rows, float scale,
                                int log_form, void* out, int out_bf16, uint64_t rows, uint64_t cols,
                                cudaStream_t s) {
  if (rows == 0 || cols == 0) return cudaSuccess;
  const bool al = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) |
                    reinterpret_cast<uintptr_t>(mask)) & 15) == 0;
  const uint64_t n4 = cols / 4;
  const uint64_t grid = rows < 148ull * 64 ? rows : 148ull * 64;
#define SM_LAUNCH(T, V)                                                                         \
  softmax_block_kernel<T, V><<<(unsigned)(rows < (148ull * (2048 / T)) ? rows : 148ull * (2048 / T)), \
                               T, 0, s>>>(x, mask, mask_rows, scale, log_form, out, out_bf16, rows, (uint32_t)cols)
  // Measured on a B200 (2 x rows x cols x 4 bytes over the launch time, 512 MB of scores): the
  // workers kernel reaches 5.6-6.0 TB/s from 2,048 to 32,768 columns; a block a row stays ahead
  // only up to 1,024 columns.
  const uint64_t workers_from = 256;
  if (al && cols % 4 == 0 && cols >= 128 && n4 <= workers_from) {
    if (n4 <= 32) SM_LAUNCH(32, 1);
    else if (n4 <= 64) SM_LAUNCH(64, 1);
    else if (n4 <= 128) SM_LAUNCH(128, 1);
    else if (n4 <= 256) SM_LAUNCH(128, 2);
    else if (n4 <= 512) SM_LAUNCH(256, 2);
    else if (n4 <= 1024) SM_LAUNCH(256, 4);
  } else if (al && cols % 4 == 0 && n4 > workers_from && n4 <= 8192) {
    // T threads a worker, 16 float4 a thread: the smallest T that covers the row
    const int threads = n4 <= 512 ? 32 : (n4 <= 1024 ? 64 : (n4 <= 2048 ? 128 : (n4 <= 4096 ? 256 : 512)));
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t smem = 512 * 16 * sizeof(float4);
    const uint64_t workers = 512 / threads;
    const unsigned gridw = (unsigned)((rows + workers - 1) / workers < (uint64_t)sms ? (rows + workers - 1) / workers : (uint64_t)sms);
#define SW(TT)                                                                                                  \
    do {                                                                                                          \
      {                                                                                                           \
        const cudaError_t e = ensure_dynamic_smem((const void*)softmax_workers_kernel<TT>, smem);                 \
        if (e != cudaSuccess) return e;                                                                           \
      }                                                                                                           \
      softmax_workers_kernel<TT><<<gridw, 512, smem, s>>>(x, mask, mask_rows, scale, log_form, out, out_bf16, rows, (uint32_t)cols); \
    } while (0)
    if (threads == 32) SW(32); else if (threads == 64) SW(64); else if (threads == 128) SW(128);
    else if (threads == 256) SW(256); else SW(512);
#undef SW
  } else if (al && cols % 4 == 0 && n4 <= 4096ull * 8) {
    // n4 in (8192, 32768]: 2..8 blocks of 512 threads a row, exchanging max and sum through
    // distributed shared memory.
    const int threads = 512;
    unsigned csize = 1;
    while ((n4 + csize - 1) / csize > (uint64_t)threads * 8) csize <<= 1;
    uint64_t clusters = rows < (1ull << 20) ? rows : (1ull << 20);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(clusters * csize), 1, 1);
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    const uint32_t cols32 = (uint32_t)cols;
    return cudaLaunchKernelEx(&cfg, softmax_cluster_kernel<512, 8>, x, mask, mask_rows, scale, log_form, out, out_bf16, rows, cols32);
  } else {
    softmax_stream_kernel<<<(unsigned)grid, 256, 0, s>>>(x, mask, mask_rows, scale, log_form, out, out_bf16, rows, cols);
  }
#undef SM_LAUNCH
  return cudaGetLastError();
}

cudaError_t launch_rms(const float* a, uint64_t rows, uint64_t cols, float eps, float* out,
                       cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  uint64_t grid = (rows + 7) / 8;
  if (grid > 148ull * 16) grid = 148ull * 16;
  rms_norm_kernel<<<(unsigned)grid, 256, 0, s>>>(a, 0, nullptr, 0, nullptr, 0, eps, nullptr, 0, nullptr, 0,
                                                 out, rows, cols);
  return cudaGetLastError();
}

cudaError_t launch_rms_norm(const void* a, int a_bf16, const void* b, int b_bf16, const void* gamma,
                            int gamma_bf16, float eps, void* sum_out, int sum_bf16, void* norm_out,
                            int norm_bf16, uint64_t rows, uint64_t cols, cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  uint64_t grid = (rows + 7) / 8;
  if (grid > 148ull * 16) grid = 148ull * 16;
  const bool plain = !b && !sum_out;
  const bool added = b && !b_bf16 && sum_out && !sum_bf16;
  if (!a_bf16 && (plain || added) && norm_out && cols % 4 == 0 && cols <= 1024 &&
      ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(sum_out) |
        reinterpret_cast<uintptr_t>(norm_out) | reinterpret_cast<uintptr_t>(gamma)) & 15) == 0) {
    const float* af = (const float*)a;
    const float* bf = (const float*)b;
    float* sf = (float*)sum_out;
    const uint32_t c32 = (uint32_t)cols;
    const int v = (int)((cols / 4 + 31) / 32);
#define RN(V)                                                                                                              \
  do {                                                                                                                     \
    if (added) launch_pdl(rms_norm_rows_kernel<V, true>, dim3((unsigned)grid), dim3(256), 0, s, af, bf, sf, gamma, gamma_bf16, eps, norm_out, norm_bf16, rows, c32); \
    else launch_pdl(rms_norm_rows_kernel<V, false>, dim3((unsigned)grid), dim3(256), 0, s, af, (const float*)nullptr, (float*)nullptr, gamma, gamma_bf16, eps, norm_out, norm_bf16, rows, c32); \
  } while (0)
    if (v <= 1) RN(1); else if (v <= 2) RN(2); else if (v <= 4) RN(4); else if (v <= 5) RN(5); else RN(8);
#undef RN
    return cudaGetLastError();
  }
  rms_norm_kernel<<<(unsigned)grid, 256, 0, s>>>(a, a_bf16, b, b_bf16, gamma, gamma_bf16, eps, sum_out,
                                                 sum_bf16, norm_out, norm_bf16, nullptr, rows, cols);
  return cudaGetLastError();
}

cudaError_t launch_argmax_rows(const float* a, uint64_t rows, uint64_t cols, int32_t* out,
                               cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  if (rows <= 64 && cols >= 16384 && cols < (1ull << 32)) {   // a few long rows: a cluster of eight blocks a row
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rows * ARGMAX_CLUSTER); cfg.blockDim = dim3(512); cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = ARGMAX_CLUSTER; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, argmax_rows_cluster_kernel, a, rows, cols, out);
  }
  // sixteen and more values a thread: a block of 1,024 threads over a 4,096-column row spent its time being scheduled
  const unsigned threads = cols >= 32768 ? 1024 : (cols >= 8192 ? 512 : (cols >= 2048 ? 256 : (cols >= 512 ? 128 : 64)));
  argmax_rows_kernel<<<(unsigned)(rows < 65535 ? rows : 65535), threads, 0, s>>>(a, rows, cols, out);
  return cudaGetLastError();
}

}  // namespace b200
