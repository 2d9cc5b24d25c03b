// Attention for a few query rows a key/value head (a decode step's) as one op: the device side
// of `Engine::attention_rows` (crates/burn-tt/src/server.rs:257; the reference kernel's contract
// is crates/tt-kernels/src/attention.rs:360-372).  For head i of `items`:
//     out_i = softmax(scale * q_i K_i^T, masked) V_i,   q_i [m, d], K_i [l, d], V_i [l, dv]
// with the composition's steps in the composition's order: the product, `SCALE_MASK_FILL`
// (x * scale, then -inf where the mask is set), the row maximum clamped to -FLT_MAX, exp(x - max),
// the row sum clamped to FLT_MIN, the division, and the product with V.
//
// The work is reading K and V once, so the bound is HBM: a head's positions are split over
// `splits` blocks when there are too few heads to fill the SMs (each block keeps its own maximum,
// sum and unnormalised rows, and a second small kernel joins them), and the scores never leave
// shared memory.
#include <cfloat>
#include <cstdint>
#include <cuda_runtime.h>

#include "kernels.h"

namespace b200 {
namespace {

constexpr int THREADS = 256;
constexpr int ROW_TILE = 8;     // query rows accumulated at once in the product with V

__device__ __forceinline__ float4 ld4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 ld4(const uint16_t* p) {
  const uint2 w = __ldg(reinterpret_cast<const uint2*>(p));
  return make_float4(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xffff0000u),
                     __uint_as_float(w.y << 16), __uint_as_float(w.y & 0xffff0000u));
}

// grid (splits, items).  Shared memory: q [m][d], s [m][lc], red [THREADS * 4 * ROW_TILE].
template <typename KV>
__global__ void __launch_bounds__(THREADS)
attention_rows_kernel(const float* __restrict__ q, uint64_t q_ld, const KV* __restrict__ k, uint64_t k_ld,
                      const KV* __restrict__ v, uint64_t v_ld, const uint32_t* __restrict__ mask,
                      const AttnItem* __restrict__ items, int m, int d, int l, int dv, int lc, float scale,
                      float* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ms) {
  extern __shared__ float smem[];
  float* qs = smem;                       // [m][d]
  float* s = qs + (size_t)m * d;          // [m][lc]
  float* red = s + (size_t)m * lc;        // [THREADS / (dv/4)][ROW_TILE][dv]
  const int item = blockIdx.y, split = blockIdx.x, splits = gridDim.x;
  const AttnItem it = items[item];
  const int j0 = split * lc;
  const int n = min(lc, l - j0);          // this block's positions
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int i = tid; i < m * d; i += THREADS) qs[i] = q[it.q_off + (uint64_t)(i / d) * q_ld + (i % d)];
  __syncthreads();

  // ---- scores: 8 lanes a key, each lane d/32 float4 of it; a warp pass is 8 keys (two a lane
  // group), whose loads are all issued before the first multiply
  {
    const int sub = lane & 7, kg = lane >> 3;
    const unsigned gmask = 0xffu << (kg * 8);
    const int per = d / 32;               // float4 a lane a key (d is a multiple of 32)
    for (int jb = warp * 8; jb < n; jb += (THREADS / 32) * 8) {
      const int ja = jb + kg, jc = jb + 4 + kg;
      const bool has_a = ja < n, has_c = jc < n;   // whole 8-lane groups agree
      const KV* ka = k + it.k_off + (uint64_t)(j0 + (has_a ? ja : 0)) * k_ld;
      const KV* kc = k + it.k_off + (uint64_t)(j0 + (has_c ? jc : 0)) * k_ld;
      for (int r0 = 0; r0 < m; r0 += ROW_TILE) {
        float acc_a[ROW_TILE], acc_c[ROW_TILE];
#pragma unroll
        for (int r = 0; r < ROW_TILE; ++r) { acc_a[r] = 0.f; acc_c[r] = 0.f; }
        for (int tb = 0; tb < per; tb += 4) {
          float4 xa[4], xc[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int e = (sub + 8 * (tb + u)) * 4;
            const bool in = tb + u < per;
            xa[u] = (in && has_a) ? ld4(ka + e) : make_float4(0.f, 0.f, 0.f, 0.f);
            xc[u] = (in && has_c) ? ld4(kc + e) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (tb + u < per) {
              const int e = (sub + 8 * (tb + u)) * 4;
#pragma unroll
              for (int r = 0; r < ROW_TILE; ++r) {
                if (r0 + r < m) {
                  const float4 qq = *reinterpret_cast<const float4*>(qs + (size_t)(r0 + r) * d + e);
                  acc_a[r] = fmaf(xa[u].x, qq.x, fmaf(xa[u].y, qq.y, fmaf(xa[u].z, qq.z, fmaf(xa[u].w, qq.w, acc_a[r]))));
                  acc_c[r] = fmaf(xc[u].x, qq.x, fmaf(xc[u].y, qq.y, fmaf(xc[u].z, qq.z, fmaf(xc[u].w, qq.w, acc_c[r]))));
                }
              }
            }
          }
        }
#pragma unroll
        for (int r = 0; r < ROW_TILE; ++r) {
          float a = acc_a[r], c = acc_c[r];
          a += __shfl_xor_sync(gmask, a, 4, 8); c += __shfl_xor_sync(gmask, c, 4, 8);
          a += __shfl_xor_sync(gmask, a, 2, 8); c += __shfl_xor_sync(gmask, c, 2, 8);
          a += __shfl_xor_sync(gmask, a, 1, 8); c += __shfl_xor_sync(gmask, c, 1, 8);
          if (sub == 0 && r0 + r < m) {
            if (has_a) s[(size_t)(r0 + r) * lc + ja] = mask[j0 + ja] ? -INFINITY : a * scale;
            if (has_c) s[(size_t)(r0 + r) * lc + jc] = mask[j0 + jc] ? -INFINITY : c * scale;
          }
        }
      }
    }
  }
  __syncthreads();

  // ---- a warp a row: maximum, exponentials, sum
  for (int r = warp; r < m; r += THREADS / 32) {
    float* sr = s + (size_t)r * lc;
    float mx = -INFINITY;
    for (int j = lane; j < n; j += 32) mx = fmaxf(mx, sr[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mx = (mx < -FLT_MAX) ? -FLT_MAX : mx;
    float sum = 0.f;
    for (int j = lane; j < n; j += 32) {
      const float p = expf(sr[j] - mx);
      sr[j] = p;
      sum += p;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (splits == 1) {
      const float den = (sum < FLT_MIN) ? FLT_MIN : sum;
      for (int j = lane; j < n; j += 32) sr[j] = sr[j] / den;
    } else if (lane == 0) {
      float* ms = part_ms + (((size_t)item * splits + split) * m + r) * 2;
      ms[0] = mx;
      ms[1] = sum;
    }
  }
  __syncthreads();

  // ---- rows x V: thread = (slice of positions, float4 column); ROW_TILE rows at a time
  {
    const int c4n = dv / 4;                       // float4 columns
    const int lanes_c = c4n < THREADS ? c4n : THREADS;
    const int nsl = THREADS / lanes_c;            // position slices (dv <= 1024)
    const int sl = tid / lanes_c, c4 = tid % lanes_c;
    const bool active = sl < nsl;
    for (int r0 = 0; r0 < m; r0 += ROW_TILE) {
      for (int cb = 0; cb < c4n; cb += lanes_c) {
        const int c = (cb + c4) * 4;
        float4 acc[ROW_TILE];
#pragma unroll
        for (int r = 0; r < ROW_TILE; ++r) acc[r] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (active && cb + c4 < c4n) {
          for (int j = sl; j < n; j += nsl * 4) {
            float4 vv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int jj = j + u * nsl;
              vv[u] = jj < n ? ld4(v + it.v_off + (uint64_t)(j0 + jj) * v_ld + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int jj = j + u * nsl;
              if (jj < n) {
#pragma unroll
                for (int r = 0; r < ROW_TILE; ++r) {
                  if (r0 + r < m) {
                    const float p = s[(size_t)(r0 + r) * lc + jj];
                    acc[r].x = fmaf(p, vv[u].x, acc[r].x); acc[r].y = fmaf(p, vv[u].y, acc[r].y);
                    acc[r].z = fmaf(p, vv[u].z, acc[r].z); acc[r].w = fmaf(p, vv[u].w, acc[r].w);
                  }
                }
              }
            }
          }
        }
        // join the slices in a fixed order
        __syncthreads();
        if (active) {
#pragma unroll
          for (int r = 0; r < ROW_TILE; ++r)
            *reinterpret_cast<float4*>(red + ((size_t)(sl * ROW_TILE + r) * lanes_c + c4) * 4) = acc[r];
        }
        __syncthreads();
        for (int i = tid; i < ROW_TILE * lanes_c; i += THREADS) {
          const int r = i / lanes_c, cc = i % lanes_c;
          if (r0 + r < m && cb + cc < c4n) {
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int z = 0; z < nsl; ++z) {
              const float4 w = *reinterpret_cast<const float4*>(red + ((size_t)(z * ROW_TILE + r) * lanes_c + cc) * 4);
              t.x += w.x; t.y += w.y; t.z += w.z; t.w += w.w;
            }
            float* dst = (splits == 1 ? out + ((size_t)item * m + (r0 + r)) * dv
                                      : part_o + (((size_t)item * splits + split) * m + (r0 + r)) * dv) + (cb + cc) * 4;
            *reinterpret_cast<float4*>(dst) = t;
          }
        }
      }
    }
  }
}

// Joins the splits of a head: M = max of the maxima, L = sum of sums * exp(max_s - M) (clamped),
// row = sum of rows_s * exp(max_s - M) / L.  grid = items * m, a thread a column.
__global__ void __launch_bounds__(128)
attention_join_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ms, int splits, int m, int dv,
                      float* __restrict__ out) {
  const size_t row = blockIdx.x;            // item * m + r
  const size_t item = row / m, r = row % m;
  float mx = -FLT_MAX;
  for (int z = 0; z < splits; ++z) mx = fmaxf(mx, part_ms[((item * splits + z) * m + r) * 2]);
  float den = 0.f;
  for (int z = 0; z < splits; ++z) {
    const float* ms = part_ms + ((item * splits + z) * m + r) * 2;
    den += ms[1] * expf(ms[0] - mx);
  }
  den = (den < FLT_MIN) ? FLT_MIN : den;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float t = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float w = expf(part_ms[((item * splits + z) * m + r) * 2] - mx);
      t += part_o[((item * splits + z) * m + r) * dv + c] * w;
    }
    out[row * dv + c] = t / den;
  }
}

}  // namespace

// How a head's positions are split: enough blocks for two a SM, chunks of at least 256 positions,
// and a chunk's scores within 96 KB of shared memory.
void attention_rows_plan(uint64_t n_items, int m, int l, int sms, int* splits, int* lc) {
  if (sms <= 0) {
    int dev = 0;
    sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int lc_max = ((96 * 1024 / 4) / m) / 32 * 32;
  uint64_t want = (2ull * (uint64_t)sms + n_items - 1) / n_items;
  const uint64_t by_len = (uint64_t)(l / 256 > 1 ? l / 256 : 1);
  if (want > by_len) want = by_len;
  const uint64_t need = ((uint64_t)l + lc_max - 1) / lc_max;
  if (want < need) want = need;
  int c = (int)((l + want - 1) / want);
  c = (c + 31) / 32 * 32;
  *lc = c;
  *splits = (l + c - 1) / c;
}

size_t attention_rows_scratch_floats(uint64_t n_items, int m, int dv, int splits) {
  return splits > 1 ? (size_t)n_items * splits * m * (dv + 2) : 0;
}

cudaError_t launch_attention_rows(const float* q, uint64_t q_ld, const void* k, uint64_t k_ld, const void* v,
                                  uint64_t v_ld, int kv_bf16, const uint32_t* mask, const AttnItem* items,
                                  uint64_t n_items, int m, int d, int l, int dv, float scale, int splits, int lc,
                                  float* scratch, float* out, int* launches, cudaStream_t stream) {
  *launches = 0;
  if (n_items == 0) return cudaSuccess;
  if (n_items > 65535) return cudaErrorNotSupported;
  const int c4n = dv / 4;
  const int lanes_c = c4n < THREADS ? c4n : THREADS;
  const size_t red = (size_t)(THREADS / lanes_c) * ROW_TILE * lanes_c * 4;
  const size_t smem = ((size_t)m * d + (size_t)m * lc + red) * sizeof(float);
  if (smem > 200 * 1024) return cudaErrorNotSupported;
  float* part_o = scratch;
  float* part_ms = scratch ? scratch + (size_t)n_items * splits * m * dv : nullptr;
  const dim3 grid((unsigned)splits, (unsigned)n_items, 1);
  cudaError_t e;
  if (kv_bf16) {
    static bool set = false;
    if (!set) {
      e = cudaFuncSetAttribute(attention_rows_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (e != cudaSuccess) return e;
      set = true;
    }
    attention_rows_kernel<uint16_t><<<grid, THREADS, smem, stream>>>(
        q, q_ld, (const uint16_t*)k, k_ld, (const uint16_t*)v, v_ld, mask, items, m, d, l, dv, lc, scale, out, part_o, part_ms);
  } else {
    static bool set = false;
    if (!set) {
      e = cudaFuncSetAttribute(attention_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (e != cudaSuccess) return e;
      set = true;
    }
    attention_rows_kernel<float><<<grid, THREADS, smem, stream>>>(
        q, q_ld, (const float*)k, k_ld, (const float*)v, v_ld, mask, items, m, d, l, dv, lc, scale, out, part_o, part_ms);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  *launches = 1;
  if (splits > 1) {
    attention_join_kernel<<<(unsigned)(n_items * m), 128, 0, stream>>>(part_o, part_ms, splits, m, dv, out);
    e = cudaGetLastError();
    if (e == cudaSuccess) *launches = 2;
  }
  return e;
}

}  // namespace b200
