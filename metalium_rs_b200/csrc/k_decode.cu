// One token a sequence through every layer of a Llama-architecture decoder in ONE launch: the device side of the
// reference's traced generation step (crates/tt-models/src/generate.rs:781; layer crates/tt-models/src/llama.rs:371-507;
// cache crates/tt-models/src/kv_cache.rs:185-330).  The composed step is eleven small launches a layer whose device
// work (a layer's 9 MB of weights) takes far less time than their launch latencies; here one launch walks the layers
// with five exchanges a layer instead.  Three forms of the same five phases, chosen at the call (`cluster_form_of`):
// a cooperative grid of persistent blocks that exchange partial sums through global memory and wait at a counter
// (described first); ONE thread-block cluster of sixteen blocks that hand results on through distributed shared memory,
// by copies that complete on the receivers' transaction barriers, and stream their weights through a ring of TMA copies
// (further down); and two to four such clusters that share a layer's heads and ff the way tensor-parallel ranks do and
// exchange their partial sums as tagged words in global memory (last; the form a step takes where the shape divides).
//
// A layer, for `B` <= 4 rows (one token of each sequence), in five phases.  Between phases stand grid barriers; the
// residual stream lives redundantly in every block's shared memory, so no phase waits for one block to publish it.
//   1  x = x_prev + down (the partial sums of the layer before, added in a fixed order); n1 = RMSNorm(x) as BF16;
//      the fused QKV projection as work items of (64 columns, a slice of k), each leaving a partial sum.
//   2  attention: an item is (sequence, key/value head, 64 cache positions).  It sums the projection's partials for
//      its heads, rounds them to BF16 as the product would, rotates queries and the key (RoPE, F32, separate
//      roundings), and -- the one item whose positions include the step's -- writes the key (rounded once to BF16) and
//      the value into the cache.  Scores with the scale, positions later than the step's masked, a chunk-local
//      softmax, P V; the chunks' (o, max, sum) are joined in phase 3.
//   3  every block joins the chunks (fixed order), rounds to BF16; the output projection as items.
//   4  x2 = x + o; n2 = RMSNorm(x2) as BF16; the gate|up projection as items.
//   5  an item of the down projection forms silu(gate) * up for its slice of k only (both halves rounded to BF16 as
//      the product would, SILU_MUL's separate roundings, BF16), multiplies, leaves a partial sum.
// After the last layer block 0 adds the last partials and writes the final RMSNorm as BF16: the head product's input.
//
// Weights are BF16 or BFP8 (decoded in the load path: csrc/k_bfp.cu), read as stored [k, n]; a thread's load is one
// 16-byte (8-byte) group of 8 columns.  What a phase reads that no earlier phase of the step writes -- its first item's
// weight tile, the cache rows of earlier positions -- is fetched into shared memory (cp.async) BEFORE the barrier the
// phase waits at, so the fetch runs under the phase before and under the barrier itself.  Every sum has a fixed order, so a step's bits do not depend on the launch.
// Every spin of the barrier is bounded by the engine's wait limit: when it runs out the error word becomes TIMEOUT,
// a flag tells the other blocks, and every block returns.
#include <cooperative_groups.h>
#include <cstdint>
#include <cstdlib>
#include <cuda_runtime.h>

#include "device_math.cuh"
#include "kernels.h"
#include "tc_common.cuh"

namespace b200 {
namespace {

constexpr int DT = 256;            // threads a block
constexpr int DCOLS = 64;          // columns of a product item
constexpr int DCH = 64;            // cache positions of an attention item
constexpr int HD = 64;             // head width the kernel is written for
constexpr int TIMEOUT_CODE = 4;
constexpr long long DEFAULT_WAIT = 4000000000ll;

__device__ __forceinline__ float bf16_round(float v) { return __uint_as_float((uint32_t)f32_to_bf16_bits(__float_as_uint(v)) << 16); }
__device__ __forceinline__ float bf16_at(const void* p, uint64_t i) { return __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(p)[i] << 16); }

constexpr int WT_ROWS = 256;       // k-rows of a product item at most (a slice of k)
struct Shared {
  float* xres;    // [MT][hidden]  the residual stream
  float* vec;     // [MT][vec_cols] a product's A operand
  float* red;     // [8][MT][64]
  uint4* ksm;     // [64][8] a chunk of keys: 128-byte rows of BF16, the 16-byte units of row j stored at u ^ (j & 7)
  uint4* vsm;     // [64][8] a chunk of values, the same layout
  float* qs;      // [4][64] rotated queries of a group
  float* ps;      // [4][64] probabilities
  float* stat;    // [16] small reductions
  uint8_t* wt;    // a product item's weight tile fetched ahead: [rows][64] BF16, or [rows][64] datums then [rows][4] exponents
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Fetch ahead the weight tile of a product item: k rows [k0, k0 + len) x columns [c0, c0 + 64) of W [k, n].
__device__ __forceinline__ void fetch_tile(uint8_t* wt, const void* w, int bfp, uint64_t k_total, uint64_t n, uint32_t k0, uint32_t len,
                                           uint32_t c0) {
  if (!bfp) {
    const uint16_t* src = reinterpret_cast<const uint16_t*>(w) + (uint64_t)k0 * n + c0;
    for (uint32_t i = threadIdx.x; i < len * 8; i += DT) cp_async16(wt + (size_t)i * 16, src + (uint64_t)(i >> 3) * n + (i & 7) * 8);
  } else {
    const uint8_t* datums = reinterpret_cast<const uint8_t*>(w);
    const uint8_t* src = datums + (uint64_t)k0 * n + c0;
    const uint8_t* ex = datums + k_total * n + (uint64_t)k0 * (n / 16) + c0 / 16;
    for (uint32_t i = threadIdx.x; i < len * 4; i += DT) cp_async16(wt + (size_t)i * 16, src + (uint64_t)(i >> 2) * n + (i & 3) * 16);
    for (uint32_t i = threadIdx.x; i < len; i += DT) cp_async4(wt + (size_t)WT_ROWS * 64 + (size_t)i * 4, ex + (uint64_t)i * (n / 16));
  }
}

// Bounded grid barrier: the `index`-th one of the launch.
__device__ __forceinline__ bool grid_barrier(unsigned* bar, unsigned index, long long limit, int* err, int* ok_word) {
  __syncthreads();
  if (threadIdx.x == 0) {
    volatile unsigned* counter = bar;
    volatile unsigned* abort_word = bar + 1;
    __threadfence();
    atomicAdd(bar, 1u);
    const unsigned target = (index + 1u) * gridDim.x;
    const long long t0 = clock64();
    int ok = 1;
    while (*counter < target) {
      if (*abort_word || clock64() - t0 > limit) { ok = 0; break; }
    }
    if (!ok) { atomicCAS(err, 0, TIMEOUT_CODE); *abort_word = 1u; }
    __threadfence();
    *ok_word = ok;
  }
  __syncthreads();
  return *ok_word != 0;
}

// sum over the block of one value a thread; the result in every thread
__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < DT / 32; ++w) t += scratch[w];
  return t;
}

// One product item: C[r, c0 .. c0+64) partial over k rows [k0, k0 + len) of W [k, n]; A's rows are `a` (shared memory,
// row pitch lda, already offset to k0).  A thread owns 8 columns and every 32nd k-row.
// `emit(r, column, value)` receives the item's results; `wt` holds the item's first `wt_rows` k-rows, fetched ahead (0: none).
template <int MT, class Emit>
__device__ __forceinline__ void product_item(const float* a, uint32_t lda, const void* w, int bfp, uint64_t k_total, uint64_t n,
                                             uint32_t k0, uint32_t len, uint32_t c0, float* red, const uint8_t* wt, uint32_t wt_rows,
                                             Emit emit) {
  const int tid = threadIdx.x, cg = tid & 7, kr = tid >> 3, warp = tid >> 5, lane = tid & 31;
  float acc[MT][8];
#pragma unroll
  for (int r = 0; r < MT; ++r)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[r][e] = 0.f;
  const uint64_t col = (uint64_t)c0 + cg * 8;
  if (wt_rows > len) wt_rows = len;
  if (col < n && wt_rows) {
    // rows fetched ahead into shared memory: the same rows, the same order of additions as the loads from global memory below
    for (uint32_t kk = kr; kk < wt_rows; kk += 32) {
      float x[8];
      if (!bfp) {
        const uint4 raw = *reinterpret_cast<const uint4*>(wt + ((size_t)kk * 8 + cg) * 16);
        x[0] = __uint_as_float(raw.x << 16); x[1] = __uint_as_float(raw.x & 0xffff0000u);
        x[2] = __uint_as_float(raw.y << 16); x[3] = __uint_as_float(raw.y & 0xffff0000u);
        x[4] = __uint_as_float(raw.z << 16); x[5] = __uint_as_float(raw.z & 0xffff0000u);
        x[6] = __uint_as_float(raw.w << 16); x[7] = __uint_as_float(raw.w & 0xffff0000u);
      } else {
        const uint2 raw = *reinterpret_cast<const uint2*>(wt + (size_t)kk * 64 + cg * 8);
        const uint32_t ex = wt[(size_t)WT_ROWS * 64 + (size_t)kk * 4 + (cg >> 1)];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          x[e] = bfp8_value((raw.x >> (e * 8)) & 0xffu, ex);
          x[4 + e] = bfp8_value((raw.y >> (e * 8)) & 0xffu, ex);
        }
      }
#pragma unroll
      for (int r = 0; r < MT; ++r) {
        const float av = a[(size_t)r * lda + kk];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[r][e] = fmaf(av, x[e], acc[r][e]);
      }
    }
  }
  if (col < n && wt_rows < len) {                     // wt_rows is a multiple of 32 here: a thread goes on with its next row
    if (!bfp) {
      const uint16_t* bp = reinterpret_cast<const uint16_t*>(w) + (uint64_t)k0 * n + col;
      for (uint32_t kk0 = wt_rows + kr; kk0 < len; kk0 += 32 * 4) {
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t kk = kk0 + u * 32;
          if (kk < len) raw[u] = __ldg(reinterpret_cast<const uint4*>(bp + (uint64_t)kk * n));
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t kk = kk0 + u * 32;
          if (kk < len) {
            float x[8];
            x[0] = __uint_as_float(raw[u].x << 16); x[1] = __uint_as_float(raw[u].x & 0xffff0000u);
            x[2] = __uint_as_float(raw[u].y << 16); x[3] = __uint_as_float(raw[u].y & 0xffff0000u);
            x[4] = __uint_as_float(raw[u].z << 16); x[5] = __uint_as_float(raw[u].z & 0xffff0000u);
            x[6] = __uint_as_float(raw[u].w << 16); x[7] = __uint_as_float(raw[u].w & 0xffff0000u);
#pragma unroll
            for (int r = 0; r < MT; ++r) {
              const float av = a[(size_t)r * lda + kk];
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[r][e] = fmaf(av, x[e], acc[r][e]);
            }
          }
        }
      }
    } else {
      const uint8_t* datums = reinterpret_cast<const uint8_t*>(w);
      const uint8_t* exps = datums + k_total * n;
      const uint8_t* bp = datums + (uint64_t)k0 * n + col;
      const uint8_t* ep = exps + (uint64_t)k0 * (n / 16) + col / 16;
      for (uint32_t kk0 = wt_rows + kr; kk0 < len; kk0 += 32 * 4) {
        uint2 raw[4];
        uint32_t ex[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t kk = kk0 + u * 32;
          if (kk < len) {
            raw[u] = __ldg(reinterpret_cast<const uint2*>(bp + (uint64_t)kk * n));
            ex[u] = __ldg(ep + (uint64_t)kk * (n / 16));
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t kk = kk0 + u * 32;
          if (kk < len) {
            float x[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              x[e] = bfp8_value((raw[u].x >> (e * 8)) & 0xffu, ex[u]);
              x[4 + e] = bfp8_value((raw[u].y >> (e * 8)) & 0xffu, ex[u]);
            }
#pragma unroll
            for (int r = 0; r < MT; ++r) {
              const float av = a[(size_t)r * lda + kk];
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[r][e] = fmaf(av, x[e], acc[r][e]);
            }
          }
        }
      }
    }
  }
  // a warp holds four k-rows of the same eight column groups: lanes 8 and 16 apart
#pragma unroll
  for (int r = 0; r < MT; ++r)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float v = acc[r][e];
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      acc[r][e] = v;
    }
  __syncthreads();   // `red` may still be read by the item before
  if (lane < 8) {
#pragma unroll
    for (int r = 0; r < MT; ++r)
#pragma unroll
      for (int e = 0; e < 8; ++e) red[((size_t)warp * MT + r) * DCOLS + lane * 8 + e] = acc[r][e];
  }
  __syncthreads();
  for (int i = tid; i < MT * DCOLS; i += DT) {
    const int r = i / DCOLS, cc = i - r * DCOLS;
    const uint64_t oc = (uint64_t)c0 + cc;
    if (oc < n) {
      float t = 0.f;
#pragma unroll
      for (int wv = 0; wv < DT / 32; ++wv) t += red[((size_t)wv * MT + r) * DCOLS + cc];
      emit(r, (uint32_t)oc, t);
    }
  }
}

// vec[r][:] = BF16(RMSNorm(x[r][:]) * gamma): x / sqrt(mean(x^2) + eps), times the gain, rounded once
// (crates/tt-kernels/src/sfpu/norm.rs:3-5; `rms_norm_as`, crates/burn-tt/src/server.rs:449).
template <int MT>
__device__ __forceinline__ void norm_rows(const float* x, uint32_t cols, const void* gamma, float eps, float* vec, uint32_t vec_pitch,
                                          float* scratch) {
  const float inv_n = 1.0f / (float)cols;
  for (int r = 0; r < MT; ++r) {
    float ss = 0.f;
    for (uint32_t c = threadIdx.x; c < cols; c += DT) ss = fmaf(x[(size_t)r * cols + c], x[(size_t)r * cols + c], ss);
    const float total = block_sum(ss, scratch);
    const float stat = sqrtf(__fadd_rn(__fmul_rn(total, inv_n), eps));
    for (uint32_t c = threadIdx.x; c < cols; c += DT) {
      const float t = __fdiv_rn(x[(size_t)r * cols + c], stat);
      vec[(size_t)r * vec_pitch + c] = bf16_round(__fmul_rn(t, bf16_at(gamma, c)));
    }
  }
  __syncthreads();
}

// The same with the gains already in shared memory as F32 (exact: they are BF16 values), the result stored as BF16 bits,
// and the rows taken side by side: 8 / MT warps a row, a warp's partial sum of squares in `scratch`, a row's partials added
// in warp order by every thread of the row -- two block barriers whatever MT (a row after the other cost two each).
template <int MT>
__device__ __forceinline__ void norm_rows_sm(const float* x, uint32_t cols, const float* gains, float eps, uint16_t* vec, uint32_t vec_pitch,
                                             float* scratch) {
  constexpr int W = (DT / 32) / MT;                    // warps a row
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, r = warp / W, sub = warp - r * W;
  const float* xr = x + (size_t)r * cols;
  float ss = 0.f;
#pragma unroll (MT == 1 ? 1 : 4)                       // (one row: eight warps share it, and short code beats unrolled; several: a thread has nine divisions in a row)
  for (uint32_t c = sub * 32 + lane; c < cols; c += W * 32) ss = fmaf(xr[c], xr[c], ss);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  __syncthreads();                                     // `scratch` is free
  if (lane == 0) scratch[warp] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < W; ++w) total += scratch[r * W + w];
  const float stat = sqrtf(__fadd_rn(__fmul_rn(total, 1.0f / (float)cols), eps));
#pragma unroll (MT == 1 ? 1 : 4)
  for (uint32_t c = sub * 32 + lane; c < cols; c += W * 32)
    vec[(size_t)r * vec_pitch + c] = f32_to_bf16_bits(__float_as_uint(__fmul_rn(__fdiv_rn(xr[c], stat), gains[c])));
  __syncthreads();
}

struct DecodeLayerDev {
  const void* norm1; const void* qkv; const void* o; const void* norm2; const void* gate_up; const void* down;
  void* kc; void* vc;
  uint32_t bfp;        // bit 0 qkv, 1 o, 2 gate_up, 3 down: the matrix is BFP8
  uint32_t pad;
};

struct DecodeParams {
  const DecodeLayerDev* layers;
  uint32_t n_layers, rows, hidden, heads, kv_heads, ff, max_len, attend;
  float eps, scale;
  const float* x0;          // [rows, hidden] F32
  const void* final_norm;   // BF16 gains
  const float* cos;         // [max_len, 64]
  const float* sin;         // [max_len, 64]: [-sin, sin]
  const int32_t* pos;
  uint16_t* out;            // [rows, hidden] BF16
  float* part_qkv; float* part_att; float* part_o; float* part_gu; float* part_dn;
  unsigned* bar;
  int* err;
  uint32_t ks_qkv, sl_qkv, ks_o, sl_o, ks_gu, sl_gu, ks_dn, sl_dn;
  uint32_t vec_cols;
};

// Which item of a phase a block takes first, and where its weight tile lies.
struct Item { uint32_t cb, ks, k0, len; bool any; };
__device__ __forceinline__ Item first_item(uint32_t col_blocks, uint32_t ks_count, uint32_t slice, uint32_t k) {
  Item it{};
  it.any = blockIdx.x < col_blocks * ks_count;
  it.cb = blockIdx.x % col_blocks;
  it.ks = blockIdx.x / col_blocks;
  it.k0 = it.ks * slice;
  it.len = it.k0 + slice <= k ? slice : k - it.k0;
  return it;
}

template <int MT>
__global__ void __launch_bounds__(DT, 1) decode_layers_kernel(const DecodeParams p) {
  extern __shared__ __align__(16) float smem[];
  __shared__ int ok_word;
  Shared s;
  s.wt = reinterpret_cast<uint8_t*>(smem);                                     // 16-byte aligned pieces first
  s.ksm = reinterpret_cast<uint4*>(s.wt + WT_ROWS * 64 * 2);
  s.vsm = s.ksm + DCH * 8;
  s.xres = reinterpret_cast<float*>(s.vsm + DCH * 8);
  s.vec = s.xres + (size_t)MT * p.hidden;
  s.red = s.vec + (size_t)MT * p.vec_cols;
  s.qs = s.red + 8 * MT * DCOLS;
  s.ps = s.qs + 4 * HD;
  s.stat = s.ps + 4 * DCH;

  const int tid = threadIdx.x;
  const uint32_t H = p.hidden, QC = p.heads * HD, KC = p.kv_heads * HD, NQKV = QC + 2 * KC, FF = p.ff;
  const uint32_t group = p.heads / p.kv_heads;
  const uint32_t chunks = p.attend / DCH;
  const uint32_t att_pitch = 4 * (HD + 2);            // an attention item's partial: up to four heads of (o[64], max, sum)
  long long limit = *reinterpret_cast<const volatile long long*>(p.err + 2);
  if (limit <= 0) limit = DEFAULT_WAIT;
  const int32_t pos = *p.pos;
  if (pos < 0 || (uint32_t)pos >= p.max_len || (uint32_t)pos >= p.attend) {   // outside the cache: DOMAIN, nothing is touched
    if (tid == 0) atomicCAS(p.err, 0, 6);
    return;
  }
  unsigned barrier_index = 0;
  const uint32_t nb_qkv = NQKV / DCOLS, nb_h = H / DCOLS, nb_gu = 2 * FF / DCOLS;
  const uint32_t att_items = p.rows * p.kv_heads * chunks;

  // the first layer's QKV tile, fetched under the embedding's norm
  {
    const Item it = first_item(nb_qkv, p.ks_qkv, p.sl_qkv, H);
    if (it.any) fetch_tile(s.wt, p.layers[0].qkv, p.layers[0].bfp & 1, H, NQKV, it.k0, it.len, it.cb * DCOLS);
    cp_async_commit();
  }

  for (uint32_t l = 0; l < p.n_layers; ++l) {
    const DecodeLayerDev L = p.layers[l];
    // ---- phase 1: the residual stream, its norm, the QKV projection ------------------------------------------------
    for (uint32_t i = tid; i < (uint32_t)MT * H; i += DT) {
      const uint32_t r = i / H, c = i - r * H;
      float v;
      if (l == 0) {
        v = r < p.rows ? p.x0[(size_t)r * H + c] : 0.f;
      } else {
        float d = 0.f;
        for (uint32_t k = 0; k < p.ks_dn; ++k) d += p.part_dn[((size_t)k * MT + r) * H + c];
        v = __fadd_rn(s.xres[i], d);                   // x2 + down (llama.rs:505)
      }
      s.xres[i] = v;
    }
    __syncthreads();
    norm_rows<MT>(s.xres, H, L.norm1, p.eps, s.vec, p.vec_cols, s.stat);
    cp_async_wait_all();
    __syncthreads();
    {
      const uint32_t items = nb_qkv * p.ks_qkv;
      for (uint32_t it = blockIdx.x; it < items; it += gridDim.x) {
        const uint32_t cb = it % nb_qkv, ks = it / nb_qkv, k0 = ks * p.sl_qkv;
        const uint32_t len = k0 + p.sl_qkv <= H ? p.sl_qkv : H - k0;
        float* out = p.part_qkv + (size_t)ks * MT * NQKV;
        product_item<MT>(s.vec + k0, p.vec_cols, L.qkv, L.bfp & 1, H, NQKV, k0, len, cb * DCOLS, s.red, s.wt, it == blockIdx.x ? len : 0,
                         [&](int r, uint32_t c, float t) { out[(size_t)r * NQKV + c] = t; });
      }
    }
    __syncthreads();
    // fetched under phase 2 and its barriers: the output projection's tile; under barrier 1: the cache rows of the
    // block's first attention item (earlier steps wrote them; the step's own row is patched in after the barrier)
    {
      const Item it = first_item(nb_h, p.ks_o, p.sl_o, QC);
      if (it.any) fetch_tile(s.wt, L.o, (L.bfp >> 1) & 1, QC, H, it.k0, it.len, it.cb * DCOLS);
      if (blockIdx.x < att_items) {
        const uint32_t a = blockIdx.x, ch = a % chunks, kvh = (a / chunks) % p.kv_heads, b = a / (chunks * p.kv_heads);
        if (ch * DCH <= (uint32_t)pos) {
          const uint64_t row0 = (uint64_t)b * p.max_len + (uint64_t)ch * DCH;
          for (uint32_t i = tid; i < DCH * 8; i += DT) {
            const uint32_t j = i >> 3, u = i & 7;
            cp_async16(s.ksm + j * 8 + (u ^ (j & 7)), reinterpret_cast<const uint16_t*>(L.kc) + (row0 + j) * KC + kvh * HD + u * 8);
            cp_async16(s.vsm + j * 8 + (u ^ (j & 7)), reinterpret_cast<const uint16_t*>(L.vc) + (row0 + j) * KC + kvh * HD + u * 8);
          }
        }
      }
      cp_async_commit();
    }
    if (!grid_barrier(p.bar, barrier_index++, limit, p.err, &ok_word)) return;

    // ---- phase 2: RoPE, the cache write, attention over chunks of positions ------------------------------------------
    {
      for (uint32_t it = blockIdx.x; it < att_items; it += gridDim.x) {
        const uint32_t ch = it % chunks, kvh = (it / chunks) % p.kv_heads, b = it / (chunks * p.kv_heads);
        float* part = p.part_att + (size_t)it * att_pitch;
        __syncthreads();
        if (ch * DCH > (uint32_t)pos) {               // every position of the chunk lies after the step's: nothing attended
          for (uint32_t i = tid; i < group * (HD + 2); i += DT) {
            const uint32_t g = i / (HD + 2), j = i - g * (HD + 2);
            part[g * (HD + 2) + j] = j == HD ? -INFINITY : 0.f;
          }
          continue;
        }
        auto qkv_at = [&](uint32_t col) -> float {   // the projection's BF16 result at (b, col)
          float t = 0.f;
          for (uint32_t k = 0; k < p.ks_qkv; ++k) t += p.part_qkv[((size_t)k * MT + b) * NQKV + col];
          return bf16_round(t);
        };
        const float* cs = p.cos + (size_t)pos * HD;
        const float* sn = p.sin + (size_t)pos * HD;
        // rotated queries of the group (F32)
        for (uint32_t i = tid; i < group * HD; i += DT) {
          const uint32_t g = i / HD, j = i - g * HD, base = (kvh * group + g) * HD;
          const float x = qkv_at(base + j), xs = qkv_at(base + (j < HD / 2 ? j + HD / 2 : j - HD / 2));
          s.qs[g * HD + j] = __fadd_rn(__fmul_rn(x, cs[j]), __fmul_rn(xs, sn[j]));
        }
        if (it != blockIdx.x) {                        // not the item fetched ahead: the chunk's rows now
          const uint64_t row0 = (uint64_t)b * p.max_len + (uint64_t)ch * DCH;
          for (uint32_t i = tid; i < DCH * 8; i += DT) {
            const uint32_t j = i >> 3, u = i & 7;
            cp_async16(s.ksm + j * 8 + (u ^ (j & 7)), reinterpret_cast<const uint16_t*>(L.kc) + (row0 + j) * KC + kvh * HD + u * 8);
            cp_async16(s.vsm + j * 8 + (u ^ (j & 7)), reinterpret_cast<const uint16_t*>(L.vc) + (row0 + j) * KC + kvh * HD + u * 8);
          }
          cp_async_commit();
        }
        // NB: the tile of the output projection shares the commit group of the item fetched ahead; waiting for all is right
        cp_async_wait_all();
        __syncthreads();
        // the step's own key (rotated, rounded once to BF16) and value: into the cache, and into the chunk that holds them
        if ((uint32_t)pos / DCH == ch && tid < HD) {
          const uint32_t j = tid, kb = QC + kvh * HD, vb = QC + KC + kvh * HD, jr = (uint32_t)pos % DCH;
          const float x = qkv_at(kb + j), xs = qkv_at(kb + (j < HD / 2 ? j + HD / 2 : j - HD / 2));
          const uint16_t kbits = f32_to_bf16_bits(__float_as_uint(__fadd_rn(__fmul_rn(x, cs[j]), __fmul_rn(xs, sn[j]))));
          const uint16_t vbits = f32_to_bf16_bits(__float_as_uint(qkv_at(vb + j)));
          const uint64_t row = (uint64_t)b * p.max_len + (uint32_t)pos;
          reinterpret_cast<uint16_t*>(L.kc)[row * KC + kvh * HD + j] = kbits;
          reinterpret_cast<uint16_t*>(L.vc)[row * KC + kvh * HD + j] = vbits;
          reinterpret_cast<uint16_t*>(s.ksm + jr * 8 + ((j >> 3) ^ (jr & 7)))[j & 7] = kbits;
          reinterpret_cast<uint16_t*>(s.vsm + jr * 8 + ((j >> 3) ^ (jr & 7)))[j & 7] = vbits;
        }
        __syncthreads();
        // scores: a thread a (head of the group, position)
        const uint32_t g = tid / DCH, j = tid - g * DCH;
        float sc = -INFINITY;
        if (g < group) {
          const uint32_t pj = ch * DCH + j;
          if (pj <= (uint32_t)pos) {
            float t = 0.f;
            const float* q = s.qs + g * HD;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const uint4 kq = s.ksm[j * 8 + (u ^ (j & 7))];
              const uint32_t w4[4] = {kq.x, kq.y, kq.z, kq.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                t = fmaf(q[u * 8 + 2 * e], __uint_as_float(w4[e] << 16), t);
                t = fmaf(q[u * 8 + 2 * e + 1], __uint_as_float(w4[e] & 0xffff0000u), t);
              }
            }
            sc = __fmul_rn(t, p.scale);
          }
        }
        // the chunk's maximum and sum for each head: two warps a head
        float m = sc;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if ((tid & 31) == 0) s.stat[tid >> 5] = m;
        __syncthreads();
        const float mh = g < group ? fmaxf(fmaxf(s.stat[2 * g], s.stat[2 * g + 1]), -3.402823466e38f) : 0.f;
        const float e = g < group ? expf(sc - mh) : 0.f;
        if (g < group) s.ps[g * DCH + j] = e;
        float sum = e;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        __syncthreads();
        if ((tid & 31) == 0) s.stat[8 + (tid >> 5)] = sum;
        __syncthreads();
        // P V: a thread a (head, column)
        if (g < group) {
          const uint32_t d = j;
          float o = 0.f;
          const float* pr = s.ps + g * DCH;
          for (int jj = 0; jj < DCH; ++jj) {
            const uint16_t hv = reinterpret_cast<const uint16_t*>(s.vsm + jj * 8 + ((d >> 3) ^ (jj & 7)))[d & 7];
            o = fmaf(pr[jj], __uint_as_float((uint32_t)hv << 16), o);
          }
          part[g * (HD + 2) + d] = o;
          if (d == 0) {
            part[g * (HD + 2) + HD] = mh;
            part[g * (HD + 2) + HD + 1] = s.stat[8 + 2 * g] + s.stat[8 + 2 * g + 1];
          }
        }
      }
    }
    if (!grid_barrier(p.bar, barrier_index++, limit, p.err, &ok_word)) return;

    // ---- phase 3: join the chunks, the output projection ----------------------------------------------------------------
    for (uint32_t i = tid; i < (uint32_t)MT * QC; i += DT) {
      const uint32_t r = i / QC, c = i - r * QC, h = c / HD, d = c - h * HD, kvh = h / group, g = h - kvh * group;
      float v = 0.f;
      if (r < p.rows) {
        const float* base = p.part_att + (size_t)((r * p.kv_heads + kvh) * chunks) * att_pitch + g * (HD + 2);
        float M = -3.402823466e38f;
        for (uint32_t c2 = 0; c2 < chunks; ++c2) M = fmaxf(M, base[(size_t)c2 * att_pitch + HD]);
        float Lsum = 0.f, O = 0.f;
        for (uint32_t c2 = 0; c2 < chunks; ++c2) {
          const float* q = base + (size_t)c2 * att_pitch;
          const float wgt = expf(q[HD] - M);           // exp(-inf) = 0 for a chunk nothing attended
          Lsum = fmaf(q[HD + 1], wgt, Lsum);
          O = fmaf(q[d], wgt, O);
        }
        v = bf16_round(__fdiv_rn(O, fmaxf(Lsum, 1.175494351e-38f)));   // `attention_rows_as`: the clamped sum, a BF16 result
      }
      s.vec[(size_t)r * p.vec_cols + c] = v;
    }
    cp_async_wait_all();
    __syncthreads();
    {
      const uint32_t items = nb_h * p.ks_o;
      for (uint32_t it = blockIdx.x; it < items; it += gridDim.x) {
        const uint32_t cb = it % nb_h, ks = it / nb_h, k0 = ks * p.sl_o;
        const uint32_t len = k0 + p.sl_o <= QC ? p.sl_o : QC - k0;
        float* out = p.part_o + (size_t)ks * MT * H;
        product_item<MT>(s.vec + k0, p.vec_cols, L.o, (L.bfp >> 1) & 1, QC, H, k0, len, cb * DCOLS, s.red, s.wt, it == blockIdx.x ? len : 0,
                         [&](int r, uint32_t c, float t) { out[(size_t)r * H + c] = t; });
      }
    }
    __syncthreads();
    {
      const Item it = first_item(nb_gu, p.ks_gu, p.sl_gu, H);
      if (it.any) fetch_tile(s.wt, L.gate_up, (L.bfp >> 2) & 1, H, 2 * FF, it.k0, it.len, it.cb * DCOLS);
      cp_async_commit();
    }
    if (!grid_barrier(p.bar, barrier_index++, limit, p.err, &ok_word)) return;

    // ---- phase 4: x2 = x + o, its norm, the gate|up projection ---------------------------------------------------------
    for (uint32_t i = tid; i < (uint32_t)MT * H; i += DT) {
      const uint32_t r = i / H, c = i - r * H;
      float d = 0.f;
      for (uint32_t k = 0; k < p.ks_o; ++k) d += p.part_o[((size_t)k * MT + r) * H + c];
      s.xres[i] = __fadd_rn(s.xres[i], d);
    }
    __syncthreads();
    norm_rows<MT>(s.xres, H, L.norm2, p.eps, s.vec, p.vec_cols, s.stat);
    cp_async_wait_all();
    __syncthreads();
    {
      const uint32_t items = nb_gu * p.ks_gu;
      for (uint32_t it = blockIdx.x; it < items; it += gridDim.x) {
        const uint32_t cb = it % nb_gu, ks = it / nb_gu, k0 = ks * p.sl_gu;
        const uint32_t len = k0 + p.sl_gu <= H ? p.sl_gu : H - k0;
        float* out = p.part_gu + (size_t)ks * MT * 2 * FF;
        product_item<MT>(s.vec + k0, p.vec_cols, L.gate_up, (L.bfp >> 2) & 1, H, 2 * FF, k0, len, cb * DCOLS, s.red, s.wt,
                         it == blockIdx.x ? len : 0, [&](int r, uint32_t c, float t) { out[(size_t)r * 2 * FF + c] = t; });
      }
    }
    __syncthreads();
    {
      const Item it = first_item(nb_h, p.ks_dn, p.sl_dn, FF);
      if (it.any) fetch_tile(s.wt, L.down, (L.bfp >> 3) & 1, FF, H, it.k0, it.len, it.cb * DCOLS);
      cp_async_commit();
    }
    if (!grid_barrier(p.bar, barrier_index++, limit, p.err, &ok_word)) return;

    // ---- phase 5: silu(gate) * up for an item's slice of k, the down projection ------------------------------------------
    {
      const uint32_t items = nb_h * p.ks_dn;
      for (uint32_t it = blockIdx.x; it < items; it += gridDim.x) {
        const uint32_t cb = it % nb_h, ks = it / nb_h, k0 = ks * p.sl_dn;
        const uint32_t len = k0 + p.sl_dn <= FF ? p.sl_dn : FF - k0;
        __syncthreads();
        for (uint32_t i = tid; i < (uint32_t)MT * len; i += DT) {
          const uint32_t r = i / len, kk = i - r * len;
          float gt = 0.f, up = 0.f;
          for (uint32_t k = 0; k < p.ks_gu; ++k) {
            gt += p.part_gu[((size_t)k * MT + r) * 2 * FF + k0 + kk];
            up += p.part_gu[((size_t)k * MT + r) * 2 * FF + FF + k0 + kk];
          }
          const float a = bf16_round(gt), bq = bf16_round(up);
          s.vec[(size_t)r * p.vec_cols + kk] = bf16_round(__fmul_rn(__fmul_rn(a, sigmoid_flex(a)), bq));   // SILU_MUL, BF16 result
        }
        cp_async_wait_all();
        __syncthreads();
        float* out = p.part_dn + (size_t)ks * MT * H;
        product_item<MT>(s.vec, p.vec_cols, L.down, (L.bfp >> 3) & 1, FF, H, k0, len, cb * DCOLS, s.red, s.wt, it == blockIdx.x ? len : 0,
                         [&](int r, uint32_t c, float t) { out[(size_t)r * H + c] = t; });
      }
    }
    __syncthreads();
    if (l + 1 < p.n_layers) {                          // the next layer's QKV tile, under the barrier
      const Item it = first_item(nb_qkv, p.ks_qkv, p.sl_qkv, H);
      if (it.any) fetch_tile(s.wt, p.layers[l + 1].qkv, p.layers[l + 1].bfp & 1, H, NQKV, it.k0, it.len, it.cb * DCOLS);
    }
    cp_async_commit();
    if (!grid_barrier(p.bar, barrier_index++, limit, p.err, &ok_word)) return;
  }
  cp_async_wait_all();

  // ---- the stream's last value and its norm: the head product's input -------------------------------------------------------
  if (blockIdx.x == 0) {
    for (uint32_t i = tid; i < (uint32_t)MT * H; i += DT) {
      const uint32_t r = i / H, c = i - r * H;
      float d = 0.f;
      for (uint32_t k = 0; k < p.ks_dn; ++k) d += p.part_dn[((size_t)k * MT + r) * H + c];
      s.xres[i] = __fadd_rn(s.xres[i], d);
    }
    __syncthreads();
    norm_rows<MT>(s.xres, H, p.final_norm, p.eps, s.vec, p.vec_cols, s.stat);
    for (uint32_t i = tid; i < p.rows * H; i += DT) {
      const uint32_t r = i / H, c = i - r * H;
      p.out[i] = f32_to_bf16_bits(__float_as_uint(s.vec[(size_t)r * p.vec_cols + c]));
    }
  }
}

// ---- the same step on ONE thread-block cluster --------------------------------------------------------------------------
// Sixteen (or eight) blocks of one cluster instead of a grid: what a phase hands to the next travels through
// distributed shared memory -- a block stages its results and the copy engine delivers them into every block's shared
// memory, completing as transaction bytes on the receiver's mbarrier of the phase -- so a block waits for the bytes it
// expects instead of at a counter in global memory after round trips through L2 for the partial sums.  Only the down
// projection slices k (its partial sums are added in a fixed order by every block); the other products give a block
// whole columns.
//
// With so few blocks the step is bound by how many bytes of weights a block keeps in flight, so the weights do not wait
// for the phase that uses them: the tiles a block will multiply by are known from the start (layer after layer, phase
// after phase, item after item), and a ring of shared-memory slots is kept full of the next chunks by TMA (one tiled copy
// a chunk -- 192 k-rows by 64 columns, or 576 for one sequence, where a chunk is a whole item -- completing on the slot's
// mbarrier), across phases and cluster
// barriers: loads issued by threads keep some 16 KB a block in flight, far too little for sixteen blocks to draw the
// device's bandwidth, where the ring holds up to 144 KB a block.  A product waits for its next chunk, multiplies from
// shared memory with tensor-core tiles (`mma.sync`: a warp owns 8 of the item's 64 columns), and refills the slot with
// the chunk that is R chunks ahead.  The form takes BF16 matrices only.
namespace cg = cooperative_groups;

// The several-cluster form's cut of a layer, worked out on the host (a division in the kernel is a hundred cycles, and
// under its register pressure the compiler repeats one wherever its result is used): a cluster takes hq query heads with
// their hk key/value heads and FFl of ff.
struct TpShape {
  uint32_t hq, hk, QCl, KCl, NQl, FFl, nfl, ffb, n_q, n_qs, n_att, nb_h, n_gu, n_dn, off_att, off_o, off_dn, group;
};

struct ClusterParams {
  const DecodeLayerDev* layers;
  uint32_t n_layers, rows, hidden, heads, kv_heads, ff, max_len, attend;
  float eps, scale;
  const float* x0;
  const void* final_norm;
  const float* cos;
  const float* sin;
  const int32_t* pos;
  uint16_t* out;
  int* err;
  uint32_t ks_dn, sl_dn, vec_cols, att_items;
  uint32_t min_width;        // the narrowest cluster the shared-memory plan holds the staging slots of (8 or 16 blocks)
  const CUtensorMap* maps;   // [n_layers][4]: qkv, o, gate|up, down as [k, n] with a box of 64 rows by 64 columns
  // the several-cluster form only
  uint32_t tp;               // clusters a step: each takes 1/tp of the heads and of ff
  uint32_t pbytes[4];        // bytes one tiled copy of a chunk lands, by matrix (the box of that matrix's descriptors)
  // a cluster's partial sums, in global memory, every element an 8-byte word {value, layer + 1}, two copies used by
  // the layers in turn, all words zero at launch
  unsigned long long* part_o;    // [2][tp][MT][hidden]: a cluster's share of the attention output's projection
  unsigned long long* part_dn;   // [2][tp * ks_dn][MT][hidden]: and of the down projection, a slice of k each
  uint32_t ks_q, sl_q;           // the QKV product's k in ks_q slices of sl_q rows: an item a (column block, slice)
  // BFP8 matrices (every matrix of every layer, or none): a chunk lands as its datum bytes [rows][64] by one tiled copy and
  // its exponent bytes [rows][4] by 4-byte copies a thread, and is decoded into BF16 before the tensor-core tiles read it
  uint32_t bfp;
  uint32_t crows[4];             // rows a chunk's copy brings, by matrix
  uint32_t kn[4][2];             // the matrices' [k, n]
  TpShape cut;
  unsigned long long* done;      // [2][blocks]: a block's word {0, layer + 1}: it has finished the layer
  uint32_t skip_done;            // a test's hook: that block never stores its word, so the others' polls run out (no block: ~0)
};

constexpr int CK_ROWS = 192;                           // k-rows of a tiled copy's box (at most 256)
constexpr int GN = 4;                                  // gains a thread fetches ahead: the cluster form takes hidden <= GN * 256
constexpr uint32_t BOX_BYTES = CK_ROWS * 128;          // rows of 64 BF16, 128-byte swizzled as the copy writes them
static_assert(BOX_BYTES % 1024 == 0 && CK_ROWS % 32 == 0 && CK_ROWS <= 256, "a swizzled box starts on 1,024 bytes and has at most 256 rows");
// A chunk -- what one wait, one block barrier and one issue move -- is up to NB boxes on one mbarrier: a wait, a barrier and
// an issue cost some 500 cycles a chunk whatever its size, so one sequence (whose other buffers are small) takes a whole
// 576-row item as one chunk in a ring of two; the wider steps keep single boxes.
template <int MT> struct ChunkBoxes { static constexpr int value = MT == 1 ? 3 : 1; };
template <int MT> struct RingDepth { static constexpr int value = MT == 1 ? 2 : (MT == 2 ? 4 : 2); };
inline uint32_t chunk_rows_of(uint32_t mt) { return (mt == 1 ? 3u : 1u) * CK_ROWS; }

// The chunks of weights a block multiplies by during ONE layer, in the order it uses them: the same list for every layer,
// so it is written once (by one thread, into shared memory) and the step's issue path only reads it.
struct ChunkEnt { uint16_t phase, rows, cb, k0; };     // phase 0 qkv, 1 o, 2 gate|up, 3 down; rows of the chunk; column block; first k-row
constexpr uint32_t SCHED_MAX = 256;

// The several-cluster form's cut of a layer: cluster `cgi` of `tp` takes heads / tp query heads with their key/value
// heads (the QKV columns of those heads, their attention, the rows of the output projection they feed) and ff / tp of the
// MLP (those gate and up columns, the rows of the down projection they feed).  Item j of a phase goes to the block whose
// rank is (j + the phase's offset) mod the cluster's width, so that the phases with fewer items than blocks do not all
// land on the first blocks.
struct TpCut : TpShape {
  uint32_t cgi, heads, kv_heads;
  __device__ TpCut(const ClusterParams& p, uint32_t cgi_) : TpShape(p.cut) { cgi = cgi_; heads = p.heads; kv_heads = p.kv_heads; }
  // the column block (of 64) of the stored matrix that local item j multiplies by
  __device__ uint32_t qkv_cb(uint32_t j) const {
    return j < hq ? cgi * hq + j : (j < hq + hk ? heads + cgi * hk + (j - hq) : heads + kv_heads + cgi * hk + (j - hq - hk));
  }
  __device__ uint32_t gu_cb(uint32_t j) const { return j < nfl ? cgi * nfl + j : ffb + cgi * nfl + (j - nfl); }
  __device__ static uint32_t first(uint32_t me, uint32_t C, uint32_t off) { return (me + C - (off & (C - 1))) & (C - 1); }   // C is 8 or 16
};

struct WeightWalk {
  const ClusterParams* p;
  const ChunkEnt* tab;
  uint32_t cnt, ii, il;                                // the list's length; the next chunk to issue: entry ii of layer il
  uint32_t ic, lc;                                     // the entry being multiplied, of layer lc (the list repeats every layer)
  const DecodeLayerDev* lay;                           // the layers' records in shared memory (the BFP8 form reads the matrices' addresses)
  // thread 0 writes the list; every thread calls this, the caller's __syncthreads publishes it
  __device__ void start(const ClusterParams* pp, ChunkEnt* tab_, uint32_t* cnt_sm, uint32_t me, uint32_t C, uint32_t chunk_rows) {
    p = pp; tab = tab_; ii = 0; il = 0; ic = 0; lc = 0; lay = nullptr;
    if (threadIdx.x == 0) {
      const uint32_t H = pp->hidden, QC = pp->heads * HD, NQKV = QC + 2 * pp->kv_heads * HD, FF = pp->ff, nb_h = H / DCOLS;
      uint32_t c = 0;
      for (uint32_t ph = 0; ph < 4; ++ph) {
        const uint32_t items = ph == 0 ? NQKV / DCOLS : (ph == 1 ? nb_h : (ph == 2 ? 2 * FF / DCOLS : nb_h * pp->ks_dn));
        for (uint32_t item = me; item < items; item += C) {
          const uint32_t kbase = ph == 3 ? (item / nb_h) * pp->sl_dn : 0;
          const uint32_t total = ph == 0 || ph == 2 ? H : (ph == 1 ? QC : (kbase + pp->sl_dn <= FF ? pp->sl_dn : FF - kbase));
          const uint32_t cb = ph == 3 ? item % nb_h : item;
          for (uint32_t k = 0; k < total && c < SCHED_MAX; k += chunk_rows)
            tab_[c++] = ChunkEnt{(uint16_t)ph, (uint16_t)(total - k < chunk_rows ? total - k : chunk_rows), (uint16_t)cb, (uint16_t)(kbase + k)};
        }
      }
      *cnt_sm = c;
    }
  }
  // the same list for a block of the several-cluster form: its cluster's share, in the order of the phases
  __device__ void start_tp(const ClusterParams* pp, ChunkEnt* tab_, uint32_t* cnt_sm, uint32_t me, uint32_t C, const TpCut& cut,
                           uint32_t chunk_rows) {
    p = pp; tab = tab_; ii = 0; il = 0; ic = 0; lc = 0; lay = nullptr;
    if (threadIdx.x == 0) {
      uint32_t c = 0;
      auto put = [&](uint32_t ph, uint32_t cb, uint32_t k0, uint32_t total) {
        for (uint32_t k = 0; k < total && c < SCHED_MAX; k += chunk_rows)
          tab_[c++] = ChunkEnt{(uint16_t)ph, (uint16_t)(total - k < chunk_rows ? total - k : chunk_rows), (uint16_t)cb, (uint16_t)(k0 + k)};
      };
      for (uint32_t j = TpCut::first(me, C, 0); j < cut.n_qs; j += C) {
        const uint32_t k0 = (j / cut.n_q) * pp->sl_q;
        put(0, cut.qkv_cb(j % cut.n_q), k0, k0 + pp->sl_q <= pp->hidden ? pp->sl_q : pp->hidden - k0);
      }
      for (uint32_t j = TpCut::first(me, C, cut.off_o); j < cut.nb_h; j += C) put(1, j, cut.cgi * cut.QCl, cut.QCl);
      for (uint32_t j = TpCut::first(me, C, 0); j < cut.n_gu; j += C) put(2, cut.gu_cb(j), 0, pp->hidden);
      for (uint32_t j = TpCut::first(me, C, cut.off_dn); j < cut.n_dn; j += C) {
        const uint32_t ks = j / cut.nb_h, k0 = ks * pp->sl_dn;
        put(3, j % cut.nb_h, cut.cgi * cut.FFl + k0, k0 + pp->sl_dn <= cut.FFl ? pp->sl_dn : cut.FFl - k0);
      }
      *cnt_sm = c;
    }
  }
  __device__ __forceinline__ void consumed() { if (++ic == cnt) { ic = 0; ++lc; } }
  // issue the copy of the next chunk into `slot` (called by every thread of the block; thread 0 issues), then move on
  __device__ __forceinline__ void issue(uint8_t* slot, uint64_t* bar) {
    if (cnt != 0 && il < p->n_layers) {
      if (p->bfp) {
        // the chunk's exponent bytes: four a row (the item's 64 columns are four groups of sixteen), a 4-byte copy a row,
        // whose completion arrives on the slot's barrier with the tiled copy's bytes (the barrier counts every thread: one warp issuing a chunk's 576 copies held the block up for ~1,000 cycles)
        const ChunkEnt e = tab[ii];
        const uint32_t rows = p->crows[e.phase], K = p->kn[e.phase][0], N = p->kn[e.phase][1];
        const DecodeLayerDev& L = lay[il];
        const uint8_t* w = reinterpret_cast<const uint8_t*>(e.phase == 0 ? L.qkv : (e.phase == 1 ? L.o : (e.phase == 2 ? L.gate_up : L.down)));
        const uint8_t* ex = w + (size_t)K * N + (size_t)e.k0 * (N / 16) + (size_t)e.cb * 4;
        for (uint32_t r = threadIdx.x; r < rows && e.k0 + r < K; r += DT) cp_async4(slot + (size_t)rows * 64 + r * 4, ex + (size_t)r * (N / 16));
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(tc::smem_u32(bar)) : "memory");
      }
      if (threadIdx.x == 0) {
        // one copy a chunk: the matrices are described as [k / 64][64][n], so a box of (chunk rows / 64) x 64 x 64 is the
        // chunk's rows in order (at most 256 a dimension); the whole box counts, rows past the matrix filled with zeros
        const ChunkEnt e = tab[ii];
        tc::mbar_expect_tx(bar, p->pbytes[e.phase]);   // what the matrix's descriptor brings
        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                     ::"r"(tc::smem_u32(slot)), "l"(p->maps + (size_t)il * 4 + e.phase), "r"(tc::smem_u32(bar)), "r"((int32_t)e.cb * DCOLS),
                       "r"(0), "r"((int32_t)(e.k0 / 64)) : "memory");
      }
      if (++ii == cnt) { ii = 0; ++il; }
    }
  }
};

// mbar_wait's abort flag: a product's wait has no other block to hear from, so the flag is the error word itself (set by
// any block of the engine's kernels that gave up)
__device__ __forceinline__ volatile int& dead_flag_of(int* err) { return *reinterpret_cast<volatile int*>(err); }
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One product item fed from the ring: `len` k-rows in chunks of up to ChunkBoxes<MT> boxes of CK_ROWS, A's rows as BF16 in
// shared memory (pitch lda elements, offset to the item's first k-row).  The product is taken transposed on the tensor
// cores, C^T = W^T x^T, so that the 16-row side of `mma.sync.m16n8k16` holds sixteen of the item's 64 columns and the
// 8-column side the step's rows (MT of them fed, the rest zeros): a warp owns sixteen columns and half of a box's
// k-steps (warps 0-3 the first six, warps 4-7 the last six), six MMAs a box where the other orientation -- eight columns
// and all of k a warp -- took twelve; the two halves of k meet in shared memory, added in a fixed order.  The weights'
// fragment comes by `ldmatrix.trans` (the slot is [k][64 columns], 128-byte swizzled as the copy wrote it: the 16-byte
// unit of row k sits at unit ^ (k & 7), so eight rows of one matrix meet eight bank groups).
// With 16 blocks a step the CUDA cores were the products' bound (unpacking and 8 FMA a 16-byte load: 17 k of a block's
// 48 k warp instructions a layer); an eighth of a tensor tile is used and it is still an order less issue.
// BFP8 chunks: eight datums of a row (one 16-byte piece of the BF16 tile) a thread at a time.  A datum is a sign over a
// 7-bit magnitude m, its value m 2^(E - 133) under the group's exponent byte E (crates/tt-isa/src/tile.rs:619-634).  Two
// datums a step on the BF16 pipe: the magnitudes set into the mantissas of two 128.0 give 128 + m exactly, less 128.0 is m,
// times 2^(E - 133) is the value (a power of two: exact), and the sign bits go on top -- the decoder's bits for every
// finite group.  An exponent of 255 (a group that keeps an infinity or a NaN), an exponent below 7 (stored as zeros) and a
// datum 0x80 (the decoder's -infinity) take the decoder itself.
__device__ __forceinline__ uint32_t bfp8_pair(uint32_t two, uint32_t scale2, uint32_t off2) {
  // `two`: a datum in both bytes of each half.  (128 + m) s - 128 s in one rounding: every term a BF16 value, the result exact
  uint32_t r;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"((two & 0x007f007fu) | 0x43004300u), "r"(scale2), "r"(off2));
  return r ^ (two & 0x80008000u);
}
__device__ __forceinline__ bool bfp8_slow(uint2 raw, uint32_t E) {
  const uint32_t x = raw.x ^ 0x80808080u, y = raw.y ^ 0x80808080u;
  return E >= 254u || E < 7u || ((((x - 0x01010101u) & ~x) | ((y - 0x01010101u) & ~y)) & 0x80808080u) != 0;   // (254: 128 s would overflow)
}
__device__ __forceinline__ uint4 bfp8_unit_slow(uint2 raw, uint32_t E) {
  uint32_t w[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint32_t src = q < 2 ? raw.x : raw.y, sh = (q & 1) * 16;
    w[q] = (uint32_t)bfp8_to_bf16_bits((src >> sh) & 0xffu, E) | ((uint32_t)bfp8_to_bf16_bits((src >> (sh + 8)) & 0xffu, E) << 16);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ uint4 bfp8_unit_fast(uint2 raw, uint32_t E) {
  const uint32_t s1 = (E - 6u) << 7, s2 = s1 | (s1 << 16);             // 2^(E - 133) twice
  const uint32_t o1 = ((E + 1u) << 7) | 0x8000u, o2 = o1 | (o1 << 16);  // -128 of them
  uint4 o;
  o.x = bfp8_pair(__byte_perm(raw.x, 0, 0x1100), s2, o2);
  o.y = bfp8_pair(__byte_perm(raw.x, 0, 0x3322), s2, o2);
  o.z = bfp8_pair(__byte_perm(raw.y, 0, 0x1100), s2, o2);
  o.w = bfp8_pair(__byte_perm(raw.y, 0, 0x3322), s2, o2);
  return o;
}

// A landed BFP8 chunk (datum bytes [crows][64], then exponent bytes [crows][4]) into the BF16 tile the tensor-core loads
// expect: row k's 16-byte piece u at piece u ^ (k & 7), as the BF16 form's copies write it.  Every thread; four pieces a
// step, 32 rows apart, so that their chains interleave (`rows` is a multiple of 16).
__device__ __forceinline__ void decode_chunk(const uint8_t* raw, uint32_t crows, uint32_t rows, uint8_t* wbuf) {
  constexpr int NP = 4;                                // pieces a step, 32 rows apart
  const uint32_t tid = threadIdx.x, c8 = tid & 7, r0 = tid >> 3;
  const uint32_t sraw = tc::smem_u32(raw) + c8 * 8, sex = tc::smem_u32(raw) + crows * 64 + (c8 >> 1), sout = tc::smem_u32(wbuf);
  for (uint32_t r = r0; r < rows; r += 32 * NP) {
    uint2 d[NP];
    uint32_t E[NP], rr[NP];
    bool slow = false;
#pragma unroll
    for (int q = 0; q < NP; ++q) {
      rr[q] = r + 32 * q < rows ? r + 32 * q : r;     // (a piece past the chunk decodes the first again and is not stored)
      asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(d[q].x), "=r"(d[q].y) : "r"(sraw + rr[q] * 64));
      asm volatile("ld.shared.u8 %0, [%1];" : "=r"(E[q]) : "r"(sex + rr[q] * 4));
    }
#pragma unroll
    for (int q = 0; q < NP; ++q) slow = slow || bfp8_slow(d[q], E[q]);
    uint4 o[NP];
    if (slow) {
#pragma unroll
      for (int q = 0; q < NP; ++q) o[q] = bfp8_unit_slow(d[q], E[q]);
    } else {
#pragma unroll
      for (int q = 0; q < NP; ++q) o[q] = bfp8_unit_fast(d[q], E[q]);
    }
#pragma unroll
    for (int q = 0; q < NP; ++q)
      if (q == 0 || r + 32 * q < rows)
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(sout + rr[q] * 128 + ((c8 ^ (rr[q] & 7)) << 4)), "r"(o[q].x), "r"(o[q].y),
                     "r"(o[q].z), "r"(o[q].w) : "memory");
  }
}

// The BFP8 form's next chunk taken ahead of its product: waited for, decoded into the (free) BF16 tile, its slot given
// back.  A block calls this when a phase's items are done and sent, before it waits for the other blocks: the decode
// (some 3,000 cycles a 576-row chunk) then runs in time the block would have spent waiting.  `ahead` tells the product
// that its first chunk is already in the tile.
template <int MT, int R>
__device__ __forceinline__ void decode_ahead(uint8_t* ring, uint64_t* bars, uint32_t head, uint32_t& parity, bool& dead, long long limit,
                                             int* err, WeightWalk& walk, uint8_t* wbuf, bool& ahead) {
  constexpr uint32_t SLOT_BYTES = (ChunkBoxes<MT>::value * CK_ROWS * 68 + 1023) / 1024 * 1024;
  if (ahead || walk.cnt == 0 || walk.lc >= walk.p->n_layers) return;
  if (!dead && !tc::mbar_wait(&bars[head], (parity >> head) & 1u, &dead_flag_of(err), limit)) {
    dead = true;
    atomicCAS(err, 0, TIMEOUT_CODE);
  }
  parity ^= 1u << head;
  const ChunkEnt e = walk.tab[walk.ic];
  decode_chunk(ring + (size_t)head * SLOT_BYTES, walk.p->crows[e.phase], ((uint32_t)e.rows + 15) / 16 * 16, wbuf);
  __syncthreads();                                     // the tile is whole, the slot is read
  walk.issue(ring + (size_t)head * SLOT_BYTES, &bars[head]);
  ahead = true;
}

template <int MT, int R, bool BFP = false, class Emit>
__device__ __forceinline__ void product_stream(const uint16_t* a, uint32_t lda, uint32_t len, uint8_t* ring, uint64_t* bars, uint32_t& head,
                                               uint32_t& parity, bool& dead, long long limit, int* err, WeightWalk& walk, float* halves,
                                               Emit emit, uint8_t* wbuf = nullptr, bool* ahead = nullptr) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const uint32_t mblk = warp & 3, khalf = warp >> 2;
  float c[2][4] = {};
  const uint16_t* arow = a + (size_t)(g < MT ? g : 0) * lda;
  // this lane's row and 16-byte unit inside a k-step's sixteen rows, for the load of four 8x8 matrices:
  // matrices 0, 1: rows 0-7, the block's first and second eight columns; 2, 3: rows 8-15
  const uint32_t lrow = (uint32_t)(lane & 7) + ((lane >> 4) << 3), lunit = mblk * 2 + ((lane >> 3) & 1);
  constexpr uint32_t CHUNK_ROWS = ChunkBoxes<MT>::value * CK_ROWS;
  // a slot holds a chunk as the copies land it: BF16 tiles, or datum bytes [rows][64] and exponent bytes [rows][4]
  constexpr uint32_t SLOT_BYTES = BFP ? (CHUNK_ROWS * 68 + 1023) / 1024 * 1024 : ChunkBoxes<MT>::value * BOX_BYTES;
  constexpr int HALF_STEPS = CK_ROWS / 32;             // k-steps of 16 rows a warp takes of a box
  for (uint32_t cbase = 0; cbase < len; cbase += CHUNK_ROWS) {
    const uint32_t boxes = len - cbase < CHUNK_ROWS ? (len - cbase + CK_ROWS - 1) / CK_ROWS : ChunkBoxes<MT>::value;
    if (BFP && *ahead) {
      *ahead = false;                                  // `decode_ahead` waited for this chunk, decoded it and gave its slot back
    } else {
      // the oldest of the R chunks in flight: its tile has landed when the slot's mbarrier flips
      if (!dead && !tc::mbar_wait(&bars[head], (parity >> head) & 1u, &dead_flag_of(err), limit)) {
        dead = true;                                   // recorded; the block walks on without waiting, so that the cluster's barriers are still met
        atomicCAS(err, 0, TIMEOUT_CODE);
      }
      parity ^= 1u << head;
      if (BFP) {
        // decode the chunk into the BF16 tile, then give the slot back: its next chunk travels while this one is multiplied
        const uint32_t crows = walk.p->crows[walk.tab[walk.ic].phase];          // rows the slot's copy brought
        decode_chunk(ring + (size_t)head * SLOT_BYTES, crows, len - cbase < crows ? (len - cbase + 15) / 16 * 16 : crows, wbuf);
        __syncthreads();                               // the tile is whole, the slot is read
        walk.issue(ring + (size_t)head * SLOT_BYTES, &bars[head]);
      }
    }
#pragma unroll
    for (uint32_t bx = 0; bx < boxes; ++bx) {
      const uint32_t base = cbase + bx * CK_ROWS + khalf * (CK_ROWS / 2);     // this warp's first k-row of the box, in the item
      const uint32_t slot = tc::smem_u32(BFP ? wbuf + (size_t)bx * BOX_BYTES : ring + (size_t)head * SLOT_BYTES + (size_t)bx * BOX_BYTES) +
                            khalf * (CK_ROWS / 2) * 128;
      // every load first (six loads of four 8x8 matrices, the rows' values beside them), then six MMAs into two accumulators in turn
      uint32_t wq[HALF_STEPS][4], xq[HALF_STEPS][2];
#pragma unroll
      for (int i = 0; i < HALF_STEPS; ++i) {
        const uint32_t k = i * 16 + lrow;              // row of the warp's half of the box
        ldmatrix_x4_trans(slot + k * 128 + ((lunit ^ (k & 7)) << 4), wq[i][0], wq[i][1], wq[i][2], wq[i][3]);
        const uint32_t kk = base + i * 16 + 2 * t;      // this thread's k columns of the rows' fragment: kk, kk+1 and kk+8, kk+9
        xq[i][0] = (g < MT && kk < len) ? *reinterpret_cast<const uint32_t*>(arow + kk) : 0u;       // a row past the item's k counts as zeros
        xq[i][1] = (g < MT && kk + 8 < len) ? *reinterpret_cast<const uint32_t*>(arow + kk + 8) : 0u;
      }
#pragma unroll
      for (int i = 0; i < HALF_STEPS; ++i)               // (a step past the item's k is no product: its slot rows may be another chunk's)
        if (base + i * 16 < len) mma_bf16_16816(c[i & 1], wq[i][0], wq[i][1], wq[i][2], wq[i][3], xq[i][0], xq[i][1]);
    }
    __syncthreads();                                   // every warp is done with the slot (with the decoded tile): refill it
    if (!BFP) walk.issue(ring + (size_t)head * SLOT_BYTES, &bars[head]);
    walk.consumed();
    head = head + 1 == (uint32_t)R ? 0 : head + 1;
  }
  // a thread holds columns mblk * 16 + g (and + 8) of rows 2t, 2t + 1 for its half of k: halves[khalf][row][column]
  {
    const uint32_t col = mblk * 16 + g;
    const float lo0 = c[0][0] + c[1][0], lo1 = c[0][1] + c[1][1], hi0 = c[0][2] + c[1][2], hi1 = c[0][3] + c[1][3];
    if (2 * t < MT) { halves[(khalf * MT + 2 * t) * DCOLS + col] = lo0; halves[(khalf * MT + 2 * t) * DCOLS + col + 8] = hi0; }
    if (2 * t + 1 < MT) { halves[(khalf * MT + 2 * t + 1) * DCOLS + col] = lo1; halves[(khalf * MT + 2 * t + 1) * DCOLS + col + 8] = hi1; }
  }
  __syncthreads();
  for (int i = tid; i < MT * DCOLS; i += DT) {
    const int r = i / DCOLS, cc = i - r * DCOLS;
    emit(r, cc, halves[r * DCOLS + cc] + halves[(MT + r) * DCOLS + cc]);   // into the block's staging row: the caller sends it on
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // written by threads, read by the copy engine
  __syncthreads();                                     // the staged results are whole
}

// The same delivery by the copy engine: `bytes` staged in this block's shared memory go to the same offset `dst` in the
// shared memory of block `rank`, and complete (as transaction bytes) on that block's mbarrier `bar` -- the receiver waits
// for the bytes it expects of a phase on its own barrier instead of the whole cluster meeting at a barrier whose release
// must first see every store into sixteen shared memories land.
__device__ __forceinline__ void copy_to_block(void* dst, const void* staged, uint32_t bytes, uint64_t* bar, uint32_t rank) {
  uint32_t rd, rb;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rd) : "r"(tc::smem_u32(dst)), "r"(rank));
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rb) : "r"(tc::smem_u32(bar)), "r"(rank));
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(rd), "r"(tc::smem_u32(staged)), "r"(bytes), "r"(rb) : "memory");
}

// Before a block leaves: no copy may still be on its way into the block's shared memory.  After a normal step every
// chunk that was asked for was waited for, and this returns at once; a block that gave up its waits (a timeout anywhere in
// the step) walked on without them, so the last copy armed on each slot may still be in flight: it is waited for here,
// bounded.  Slot r's last armed phase is the one before the parity the block would wait for next.
__device__ __forceinline__ void drain_ring(uint64_t* bars, int slots, uint32_t parity, long long limit) {
  const long long t0 = clock64();
  for (int r = 0; r < slots; ++r)
    while (!tc::mbar_try(&bars[r], ((parity >> r) & 1u) ^ 1u))
      if (clock64() - t0 > limit) return;
}
// The same for what the other blocks of the cluster send into this block: a thread that gave up a wait waits (bounded) for
// the last layer's phase of each of the block's receiving barriers before the block may leave.
__device__ __forceinline__ void drain_received(uint64_t* xb, int n, uint32_t last_layer, bool dead, long long limit) {
  if (!dead) return;                                   // every phase was waited for where it was used
  const long long t0 = clock64();
  for (int k = 0; k < n; ++k)
    while (!tc::mbar_try(&xb[k], last_layer & 1u))
      if (clock64() - t0 > limit) return;
}

template <int MT>
__global__ void __launch_bounds__(DT, 1) decode_cluster_kernel(const ClusterParams p) {
  constexpr int R = RingDepth<MT>::value;
  constexpr uint32_t SLOT_BYTES = ChunkBoxes<MT>::value * BOX_BYTES;
  extern __shared__ __align__(16) float smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t C = cluster.num_blocks(), me = cluster.block_rank();
  const int tid = threadIdx.x;
  const uint32_t H = p.hidden, QC = p.heads * HD, KC = p.kv_heads * HD, NQKV = QC + 2 * KC, FF = p.ff;
  const uint32_t group = p.heads / p.kv_heads, chunks = p.attend / DCH;
  // a bulk copy's issue costs its warp some 70 cycles, so an item's copies (one a block and row) are spread over the eight warps
  const uint32_t cpw = (C * MT + DT / 32 - 1) / (DT / 32), cpa = (C + DT / 32 - 1) / (DT / 32);
  constexpr uint32_t APH = HD + 4;                    // a head's partial of an attention item: 64 sums, the maximum, the sum, two unused (whole 16-byte pieces)
  constexpr uint32_t AP = 4 * APH;                    // an attention item's partial
  // shared memory (the same offsets in every block of the cluster)
  uint8_t* ring = reinterpret_cast<uint8_t*>(((uintptr_t)smem + 1023) & ~(uintptr_t)1023);   // a swizzled tile starts on 1,024 bytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (size_t)R * SLOT_BYTES);             // [16]
  uint4* ksm = reinterpret_cast<uint4*>(bars + 16);
  uint4* vsm = ksm + DCH * 8;
  float* xres = reinterpret_cast<float*>(vsm + DCH * 8);          // [MT][H]
  float* qkv = xres + (size_t)MT * H;                             // [MT][NQKV]   BF16 values, from every block
  float* att = qkv + (size_t)MT * NQKV;                           // [att_items][AP]
  float* osum = att + (size_t)p.att_items * AP;                   // [MT][H]
  float* dn = osum + (size_t)MT * H;                              // [ks_dn][MT][H]
  float* qs = dn + (size_t)p.ks_dn * MT * H;
  float* ps = qs + 4 * HD;
  float* stat = ps + 4 * DCH;
  float* halves = stat + 16;                                      // [2][MT][64] a product item's sums over the two halves of k
  // what the block's items of a phase hand to the copy engine, a slot an item: the engine reads a slot after the block
  // has moved on, and the slot is written again a layer later, when every receiver has long waited for its bytes
  const uint32_t nb_qkv = NQKV / DCOLS, nb_h = H / DCOLS, nb_gu = 2 * FF / DCOLS, nb_dn = nb_h * p.ks_dn;
  float* sq = halves + 2 * MT * DCOLS;                            // [items a block of phase 1][MT][64]
  float* sa = sq + (size_t)((nb_qkv + C - 1) / C) * MT * DCOLS;   // [... of phase 2][AP]
  float* so = sa + (size_t)((p.att_items + C - 1) / C) * AP;      // [... of phase 3][MT][64]
  float* sg = so + (size_t)((nb_h + C - 1) / C) * MT * DCOLS;     // [... of phase 4][MT][64] BF16
  float* sd = sg + (size_t)((nb_gu + C - 1) / C) * MT * DCOLS / 2;   // [... of phase 5][MT][64]
  float* g1 = sd + (size_t)((nb_dn + C - 1) / C) * MT * DCOLS;    // [H] the gains of the next first norm
  float* g2 = g1 + H;                                             // [H] the gains of the next second norm
  float* cs = g2 + H;                                             // [64] the position's row of the cosine table
  float* sn = cs + HD;                                            // [64] and of the sine table
  DecodeLayerDev* lay = reinterpret_cast<DecodeLayerDev*>(sn + HD);   // [n_layers]
  ChunkEnt* tab = reinterpret_cast<ChunkEnt*>(lay + p.n_layers);  // [SCHED_MAX]
  uint32_t* tab_len = reinterpret_cast<uint32_t*>(tab + SCHED_MAX);   // [2]
  uint16_t* gu = reinterpret_cast<uint16_t*>(((uintptr_t)(tab_len + 2) + 15) & ~(uintptr_t)15);   // [MT][2 FF] BF16
  uint16_t* vec = gu + (size_t)MT * 2 * FF;                       // [MT][vec_cols] BF16: a product's A operand

  const int32_t pos = *p.pos;
  if (pos < 0 || (uint32_t)pos >= p.max_len || (uint32_t)pos >= p.attend) {   // every block sees the same position
    if (tid == 0) atomicCAS(p.err, 0, 6);
    return;
  }
  // what every layer needs from global memory and no step changes: read once, so that no phase waits for it
  for (uint32_t i = tid; i < p.n_layers * (uint32_t)(sizeof(DecodeLayerDev) / 8); i += DT)
    reinterpret_cast<uint64_t*>(lay)[i] = reinterpret_cast<const uint64_t*>(p.layers)[i];
  if (tid < HD) { cs[tid] = p.cos[(size_t)pos * HD + tid]; sn[tid] = p.sin[(size_t)pos * HD + tid]; }
  WeightWalk walk;
  walk.start(&p, tab, tab_len, me, C, ChunkBoxes<MT>::value * CK_ROWS);
  __syncthreads();
  walk.cnt = *tab_len;
  for (uint32_t c = tid; c < H; c += DT) g1[c] = bf16_at(lay[0].norm1, c);
  uint32_t head = 0, parity = 0;
  bool dead = false;
  const long long limit = tc::wait_limit_of(p.err);
  // The phases hand their results on by copies that complete, as transaction bytes, on the RECEIVER's mbarrier of the
  // phase: a block waits for the bytes it expects of a phase instead of the cluster meeting at a barrier (whose release
  // must first see every store into sixteen shared memories land: 8,000 of a layer's 42,000 cycles).  Nothing else
  // orders the blocks, and nothing else has to: every block has items in the gate|up and down phases, so no block can be
  // a layer ahead of another -- a buffer is read before the phase that refills it a layer later can have started
  // anywhere, and a barrier is armed for its next use before a byte of that use can have been sent.
  uint64_t* xb = &bars[8];                            // [5]
  const uint32_t expect[5] = {nb_qkv * MT * DCOLS * 4, p.att_items * group * APH * 4, nb_h * MT * DCOLS * 4, nb_gu * MT * DCOLS * 2,
                              nb_dn * MT * DCOLS * 4};
  if (tid == 0) {
    for (int r = 0; r < R; ++r) tc::mbar_init(&bars[r], 1);
    for (int k = 0; k < 5; ++k) tc::mbar_init(&xb[k], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int k = 0; k < 5; ++k) tc::mbar_expect_tx(&xb[k], expect[k]);   // layer 0's
  }
  __syncthreads();
  cluster.sync();                                      // every block's barriers exist before a copy may name them
  for (int r = 0; r < R; ++r) walk.issue(ring + (size_t)r * SLOT_BYTES, &bars[r]);   // the ring starts full

  for (uint32_t l = 0; l < p.n_layers; ++l) {
    const DecodeLayerDev L = lay[l];
    // wait for the bytes this block expects of phase k of this layer, then arm the barrier for the next layer's
    auto arrived = [&](int k) {
      if (!dead && !tc::mbar_wait(&xb[k], l & 1u, &dead_flag_of(p.err), limit)) { dead = true; atomicCAS(p.err, 0, TIMEOUT_CODE); }
      __syncthreads();                                 // every thread is past the wait
      if (tid == 0 && l + 1 < p.n_layers) tc::mbar_expect_tx(&xb[k], expect[k]);
    };
    // the gains of this layer's second norm: asked for now, kept in registers, stored after the products
    float gn[GN];
#pragma unroll
    for (int i = 0; i < GN; ++i) gn[i] = tid + i * DT < H ? bf16_at(L.norm2, tid + i * DT) : 0.f;
    // ---- phase 1 ----
    for (uint32_t i = tid; i < (uint32_t)MT * H; i += DT) {
      const uint32_t r = MT == 1 ? 0u : i / H, c = i - r * H;              // (one sequence: no division)
      float v;
      if (l == 0) {
        v = r < p.rows ? p.x0[(size_t)r * H + c] : 0.f;
      } else {
        float d = 0.f;
        for (uint32_t k = 0; k < p.ks_dn; ++k) d += dn[((size_t)k * MT + r) * H + c];
        v = __fadd_rn(xres[i], d);
      }
      xres[i] = v;
    }
    __syncthreads();
    norm_rows_sm<MT>(xres, H, g1, p.eps, vec, p.vec_cols, stat);
    for (uint32_t it = me; it < nb_qkv; it += C) {
      float* slot = sq + (size_t)((it - me) / C) * MT * DCOLS;
      product_stream<MT, R>(vec, p.vec_cols, H, ring, bars, head, parity, dead, limit, p.err, walk, halves,
                            [&](int r, int cc, float t) { slot[r * DCOLS + cc] = bf16_round(t); });   // the product's BF16 result
      if (const uint32_t ci = (uint32_t)(tid >> 5) * cpw + (tid & 31); (uint32_t)(tid & 31) < cpw && ci < C * MT) {   // a (block, row) pair a thread: 256 bytes each
        const uint32_t d = ci / MT, r = ci - d * MT;
        copy_to_block(qkv + (size_t)r * NQKV + it * DCOLS, slot + r * DCOLS, DCOLS * 4, &xb[0], d);
      }
    }
#pragma unroll
    for (int i = 0; i < GN; ++i)
      if (tid + i * DT < H) g2[tid + i * DT] = gn[i];
    // the first attention item's cache rows (earlier steps wrote them) are asked for before the barrier
    uint4 kreg[2], vreg[2];
    auto load_cache = [&](uint32_t it) {
      const uint32_t ch = it % chunks, kvh = (it / chunks) % p.kv_heads, b = it / (chunks * p.kv_heads);
      if (ch * DCH > (uint32_t)pos) return;
      const uint64_t row0 = (uint64_t)b * p.max_len + (uint64_t)ch * DCH;
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const uint32_t i = tid + h2 * DT, j = i >> 3, u = i & 7;
        kreg[h2] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(L.kc) + (row0 + j) * KC + kvh * HD + u * 8);
        vreg[h2] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(L.vc) + (row0 + j) * KC + kvh * HD + u * 8);
      }
    };
    if (me < p.att_items) load_cache(me);
    arrived(0);                                        // every block's QKV results have landed here

    // ---- phase 2 ----
    for (uint32_t it = me; it < p.att_items; it += C) {
      const uint32_t ch = it % chunks, kvh = (it / chunks) % p.kv_heads, b = it / (chunks * p.kv_heads);
      float* stage = sa + (size_t)((it - me) / C) * AP;
      __syncthreads();
      if (it != me) load_cache(it);
      if (ch * DCH > (uint32_t)pos) {
        for (uint32_t i = tid; i < AP; i += DT) stage[i] = i % APH == HD ? -INFINITY : 0.f;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (const uint32_t ci = (uint32_t)(tid >> 5) * cpa + (tid & 31); (uint32_t)(tid & 31) < cpa && ci < C)
          copy_to_block(att + (size_t)it * AP, stage, group * APH * 4, &xb[1], ci);
        continue;
      }
      const float* qrow = qkv + (size_t)b * NQKV;
      for (uint32_t i = tid; i < group * HD; i += DT) {
        const uint32_t g = i / HD, j = i - g * HD, base = (kvh * group + g) * HD;
        qs[g * HD + j] = __fadd_rn(__fmul_rn(qrow[base + j], cs[j]), __fmul_rn(qrow[base + (j < HD / 2 ? j + HD / 2 : j - HD / 2)], sn[j]));
      }
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const uint32_t i = tid + h2 * DT, j = i >> 3, u = i & 7;
        ksm[j * 8 + (u ^ (j & 7))] = kreg[h2];
        vsm[j * 8 + (u ^ (j & 7))] = vreg[h2];
      }
      __syncthreads();
      if ((uint32_t)pos / DCH == ch && tid < HD) {
        const uint32_t j = tid, kb = QC + kvh * HD, vb = QC + KC + kvh * HD, jr = (uint32_t)pos % DCH;
        const float x = qrow[kb + j], xs = qrow[kb + (j < HD / 2 ? j + HD / 2 : j - HD / 2)];
        const uint16_t kbits = f32_to_bf16_bits(__float_as_uint(__fadd_rn(__fmul_rn(x, cs[j]), __fmul_rn(xs, sn[j]))));
        const uint16_t vbits = f32_to_bf16_bits(__float_as_uint(qrow[vb + j]));
        const uint64_t row = (uint64_t)b * p.max_len + (uint32_t)pos;
        reinterpret_cast<uint16_t*>(L.kc)[row * KC + kvh * HD + j] = kbits;
        reinterpret_cast<uint16_t*>(L.vc)[row * KC + kvh * HD + j] = vbits;
        reinterpret_cast<uint16_t*>(ksm + jr * 8 + ((j >> 3) ^ (jr & 7)))[j & 7] = kbits;
        reinterpret_cast<uint16_t*>(vsm + jr * 8 + ((j >> 3) ^ (jr & 7)))[j & 7] = vbits;
      }
      __syncthreads();
      const uint32_t g = tid / DCH, j = tid - g * DCH;
      float sc = -INFINITY;
      if (g < group && ch * DCH + j <= (uint32_t)pos) {
        float t4[4] = {0.f, 0.f, 0.f, 0.f};            // four chains of sixteen instead of one of 64, joined in a fixed order
        const float* q = qs + g * HD;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const uint4 kq = ksm[j * 8 + (u ^ (j & 7))];
          const uint32_t w4[4] = {kq.x, kq.y, kq.z, kq.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            t4[e] = fmaf(q[u * 8 + 2 * e], __uint_as_float(w4[e] << 16), t4[e]);
            t4[e] = fmaf(q[u * 8 + 2 * e + 1], __uint_as_float(w4[e] & 0xffff0000u), t4[e]);
          }
        }
        sc = __fmul_rn((t4[0] + t4[1]) + (t4[2] + t4[3]), p.scale);
      }
      float m = sc;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      if ((tid & 31) == 0) stat[tid >> 5] = m;
      __syncthreads();
      const float mh = g < group ? fmaxf(fmaxf(stat[2 * g], stat[2 * g + 1]), -3.402823466e38f) : 0.f;
      const float e = g < group ? expf(sc - mh) : 0.f;
      if (g < group) ps[g * DCH + j] = e;
      float sum = e;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      __syncthreads();
      if ((tid & 31) == 0) stat[8 + (tid >> 5)] = sum;
      __syncthreads();
      if (g < group) {
        const uint32_t d = j;
        float o4[4] = {0.f, 0.f, 0.f, 0.f};            // four chains over the positions, joined in a fixed order
        const float* pr = ps + g * DCH;
#pragma unroll 4
        for (int jj = 0; jj < DCH; jj += 4) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint16_t hv = reinterpret_cast<const uint16_t*>(vsm + (jj + e) * 8 + ((d >> 3) ^ ((jj + e) & 7)))[d & 7];
            o4[e] = fmaf(pr[jj + e], __uint_as_float((uint32_t)hv << 16), o4[e]);
          }
        }
        const float o = (o4[0] + o4[1]) + (o4[2] + o4[3]);
        const float lsum = stat[8 + 2 * g] + stat[8 + 2 * g + 1];
        stage[g * APH + d] = o;
        if (d == 0) { stage[g * APH + HD] = mh; stage[g * APH + HD + 1] = lsum; }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncthreads();
      if (const uint32_t ci = (uint32_t)(tid >> 5) * cpa + (tid & 31); (uint32_t)(tid & 31) < cpa && ci < C)
          copy_to_block(att + (size_t)it * AP, stage, group * APH * 4, &xb[1], ci);
    }
    arrived(1);                                        // every chunk's partial has landed here

    // ---- phase 3 ----
    // a (row, head)'s chunk weights exp(m_c - M) and its sum, once (a thread a pair), in the down projection's idle buffer;
    // then every output element is four multiply-adds and a division instead of eight exponentials
    float* mw = dn;                                    // [MT * heads][chunks + 1]
    uint32_t* mbase = reinterpret_cast<uint32_t*>(mw + (size_t)MT * p.heads * (chunks + 1));   // [MT * heads]
    for (uint32_t i = tid; i < (uint32_t)MT * p.heads; i += DT) {
      const uint32_t r = MT == 1 ? 0u : i / p.heads, h = i - r * p.heads, kvh = h / group, g = h - kvh * group;
      const float* base = att + (size_t)((r * p.kv_heads + kvh) * chunks) * AP + g * APH;
      float M = -3.402823466e38f;
      for (uint32_t c2 = 0; c2 < chunks; ++c2) M = fmaxf(M, base[(size_t)c2 * AP + HD]);
      float Lsum = 0.f;
      for (uint32_t c2 = 0; c2 < chunks; ++c2) {
        const float wgt = expf(base[(size_t)c2 * AP + HD] - M);
        mw[(size_t)i * (chunks + 1) + c2] = wgt;
        Lsum = fmaf(base[(size_t)c2 * AP + HD + 1], wgt, Lsum);
      }
      mw[(size_t)i * (chunks + 1) + chunks] = fmaxf(Lsum, 1.175494351e-38f);
      mbase[i] = (uint32_t)((size_t)((r * p.kv_heads + kvh) * chunks) * AP + g * APH);   // where the head's partials start
    }
    __syncthreads();
    for (uint32_t i = tid; i < (uint32_t)MT * QC; i += DT) {
      const uint32_t r = MT == 1 ? 0u : i / QC, c = i - r * QC, h = c / HD, d = c - h * HD;
      float v = 0.f;
      if (r < p.rows) {
        const float* base = att + mbase[r * p.heads + h];
        const float* w = mw + (size_t)(r * p.heads + h) * (chunks + 1);
        float O = 0.f;
        for (uint32_t c2 = 0; c2 < chunks; ++c2) O = fmaf(base[(size_t)c2 * AP + d], w[c2], O);
        v = __fdiv_rn(O, w[chunks]);
      }
      vec[(size_t)r * p.vec_cols + c] = f32_to_bf16_bits(__float_as_uint(v));
    }
    __syncthreads();
    for (uint32_t it = me; it < nb_h; it += C) {
      float* slot = so + (size_t)((it - me) / C) * MT * DCOLS;
      product_stream<MT, R>(vec, p.vec_cols, QC, ring, bars, head, parity, dead, limit, p.err, walk, halves,
                            [&](int r, int cc, float t) { slot[r * DCOLS + cc] = t; });
      if (const uint32_t ci = (uint32_t)(tid >> 5) * cpw + (tid & 31); (uint32_t)(tid & 31) < cpw && ci < C * MT) {
        const uint32_t d = ci / MT, r = ci - d * MT;
        copy_to_block(osum + (size_t)r * H + it * DCOLS, slot + r * DCOLS, DCOLS * 4, &xb[2], d);
      }
    }
    arrived(2);                                        // the attention output's projection, whole

    // ---- phase 4 ----
    for (uint32_t i = tid; i < (uint32_t)MT * H; i += DT) xres[i] = __fadd_rn(xres[i], osum[i]);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < GN; ++i) gn[i] = l + 1 < p.n_layers && tid + i * DT < H ? bf16_at(lay[l + 1].norm1, tid + i * DT) : 0.f;
    norm_rows_sm<MT>(xres, H, g2, p.eps, vec, p.vec_cols, stat);
    for (uint32_t it = me; it < nb_gu; it += C) {
      uint16_t* slot = reinterpret_cast<uint16_t*>(sg) + (size_t)((it - me) / C) * MT * DCOLS;
      product_stream<MT, R>(vec, p.vec_cols, H, ring, bars, head, parity, dead, limit, p.err, walk, halves, [&](int r, int cc, float t) {
        slot[r * DCOLS + cc] = f32_to_bf16_bits(__float_as_uint(t));   // the product's BF16 result
      });
      if (const uint32_t ci = (uint32_t)(tid >> 5) * cpw + (tid & 31); (uint32_t)(tid & 31) < cpw && ci < C * MT) {
        const uint32_t d = ci / MT, r = ci - d * MT;
        copy_to_block(gu + (size_t)r * 2 * FF + it * DCOLS, slot + r * DCOLS, DCOLS * 2, &xb[3], d);
      }
    }
#pragma unroll
    for (int i = 0; i < GN; ++i)
      if (tid + i * DT < H) g1[tid + i * DT] = gn[i];
    arrived(3);                                        // gate|up, whole

    // ---- phase 5 ----
    for (uint32_t it = me; it < nb_dn; it += C) {
      const uint32_t cb = it % nb_h, ks = it / nb_h, k0 = ks * p.sl_dn;
      const uint32_t len = k0 + p.sl_dn <= FF ? p.sl_dn : FF - k0;
      __syncthreads();
      for (uint32_t i = tid; i < (uint32_t)MT * len; i += DT) {
        const uint32_t r = MT == 1 ? 0u : i / len, kk = i - r * len;
        const float a = __uint_as_float((uint32_t)gu[(size_t)r * 2 * FF + k0 + kk] << 16);
        const float bq = __uint_as_float((uint32_t)gu[(size_t)r * 2 * FF + FF + k0 + kk] << 16);
        vec[(size_t)r * p.vec_cols + kk] = f32_to_bf16_bits(__float_as_uint(__fmul_rn(__fmul_rn(a, sigmoid_flex(a)), bq)));
      }
      __syncthreads();
      float* slot = sd + (size_t)((it - me) / C) * MT * DCOLS;
      product_stream<MT, R>(vec, p.vec_cols, len, ring, bars, head, parity, dead, limit, p.err, walk, halves,
                            [&](int r, int cc, float t) { slot[r * DCOLS + cc] = t; });
      if (const uint32_t ci = (uint32_t)(tid >> 5) * cpw + (tid & 31); (uint32_t)(tid & 31) < cpw && ci < C * MT) {
        const uint32_t d = ci / MT, r = ci - d * MT;
        copy_to_block(dn + ((size_t)ks * MT + r) * H + cb * DCOLS, slot + r * DCOLS, DCOLS * 4, &xb[4], d);
      }
    }
    arrived(4);                                        // the down projection's partial sums, all of them
  }
  if (me == 0) {
    for (uint32_t i = tid; i < (uint32_t)MT * H; i += DT) {
      const uint32_t r = MT == 1 ? 0u : i / H, c = i - r * H;
      float d = 0.f;
      for (uint32_t k = 0; k < p.ks_dn; ++k) d += dn[((size_t)k * MT + r) * H + c];
      xres[i] = __fadd_rn(xres[i], d);
    }
    __syncthreads();
    norm_rows<MT>(xres, H, p.final_norm, p.eps, osum, H, stat);   // `osum` is free: the norm's BF16 values as F32
    for (uint32_t i = tid; i < p.rows * H; i += DT) p.out[i] = f32_to_bf16_bits(__float_as_uint(osum[i]));
  }
  drain_ring(bars, R, parity, limit);
  drain_received(xb, 5, p.n_layers - 1, dead, limit);
  cluster.sync();   // no block leaves while another may still store into its shared memory
}


// ---- The several-cluster form ----
// One cluster draws its weights through one GPC's port to the L2, so sixteen blocks stream a step's 213 MB of BF16 weights
// no faster than some 0.3 ms whatever else they do, and a phase with fewer items than blocks leaves blocks idle.  Here `tp`
// clusters share a step the way tensor-parallel ranks share a layer: cluster c takes heads / tp of the query heads with their
// key/value heads and ff / tp of the MLP.  QKV, the attention and its merge, gate|up and the activation stay inside a
// cluster (results handed on by copies onto the receivers' transaction barriers, as in the one-cluster form); the output
// projection and the down projection give one partial sum a cluster (and slice of k), which every block of every cluster
// needs.  Those go through global memory, and a trip to the L2 and back costs some 2,000 cycles here (the two dies), so an
// exchange is ONE trip after the data is there: an element travels as an 8-byte word {value, layer + 1}, stored and loaded
// whole, and a reader polls the very words it needs until each carries the layer's tag -- no counter to wait for and then
// the data to fetch, no fence.  What orders the blocks is one more such word a block: at the end of a layer a block stores
// {0, layer + 1} in its own place, and the poll that opens the next layer (for the down partials) also waits for every
// block's word -- so nothing of layer l + 1 is sent anywhere before every block has read what layer l sent it and armed
// its barriers for l + 1.  The words' two copies are used by the layers in turn: a block may still poll layer l's while
// a faster one stores layer l + 1's.  Every poll is bounded.
__device__ __forceinline__ void st_tagged(unsigned long long* dst, float v, uint32_t tag) {
  const unsigned long long w = ((unsigned long long)tag << 32) | __float_as_uint(v);
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(dst), "l"(w) : "memory");
}
// x[i] += parts[0][i] + parts[1][i] + ... (in that order) for i < n, once every word carries `tag`.  A thread asks for all
// the words of up to four of its elements at once, so a pass costs one trip to the L2 once the data is there.
template <int E>                                       // elements a thread asks for at once: a trip to the L2 a batch
__device__ __forceinline__ void add_parts_tagged(float* x, uint32_t n, const unsigned long long* parts, uint32_t nparts, size_t stride,
                                                 uint32_t tag, bool& dead, long long limit, int* err,
                                                 const unsigned long long* also = nullptr) {   // one more word this thread waits for
  constexpr int KMAX = 4;
  for (uint32_t base = 0; base < n; base += E * DT) {
    float d[E];
#pragma unroll
    for (int e = 0; e < E; ++e) d[e] = 0.f;
    for (uint32_t k0 = 0; k0 < nparts; k0 += KMAX) {
      unsigned long long w[KMAX][E];
      long long t0 = 0;
      for (uint32_t spins = 0;; ++spins) {
        bool ok = true;
#pragma unroll
        for (int k = 0; k < KMAX; ++k)
#pragma unroll
          for (int e = 0; e < E; ++e) {                 // no load is conditional (an index past the end reads the last word again)
            const uint32_t i = base + e * DT + threadIdx.x, kk = k0 + k < nparts ? k0 + k : nparts - 1;
            asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w[k][e]) : "l"(parts + (size_t)kk * stride + (i < n ? i : n - 1)) : "memory");
          }
        if (also) {
          unsigned long long t;
          asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(t) : "l"(also) : "memory");
          ok = (uint32_t)(t >> 32) == tag;
        }
#pragma unroll
        for (int k = 0; k < KMAX; ++k)
#pragma unroll
          for (int e = 0; e < E; ++e) ok = ok && (uint32_t)(w[k][e] >> 32) == tag;
        if (ok || dead) break;
        if ((spins & 15u) == 15u) {                     // the wait is bounded: by the engine's limit, and by another block's giving up
          if (t0 == 0) t0 = clock64();
          if (dead_flag_of(err) != 0 || clock64() - t0 > limit) { atomicCAS(err, 0, TIMEOUT_CODE); dead = true; }
        }
      }
#pragma unroll
      for (int k = 0; k < KMAX; ++k)
#pragma unroll
        for (int e = 0; e < E; ++e)
          if (k0 + k < nparts) d[e] += __uint_as_float((uint32_t)w[k][e]);
    }
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const uint32_t i = base + e * DT + threadIdx.x;
      if (i < n) x[i] = __fadd_rn(x[i], d[e]);
    }
  }
}

template <int MT, bool BFP>
__global__ void __launch_bounds__(DT, 1) decode_tp_kernel(const ClusterParams p) {
  constexpr int R = RingDepth<MT>::value;
  constexpr uint32_t CHUNK_ROWS = ChunkBoxes<MT>::value * CK_ROWS;
  constexpr uint32_t SLOT_BYTES = BFP ? (CHUNK_ROWS * 68 + 1023) / 1024 * 1024 : ChunkBoxes<MT>::value * BOX_BYTES;   // as `product_stream` has it
  constexpr uint32_t WBUF_BYTES = BFP ? CHUNK_ROWS * 128 : 0;   // the BF16 tile a BFP8 chunk is decoded into
  extern __shared__ __align__(16) float smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t C = cluster.num_blocks(), me = cluster.block_rank(), lgC = 31 - __clz(C), cgi = blockIdx.x >> lgC;   // C is 8 or 16
  const int tid = threadIdx.x;
  const TpCut cut(p, cgi);
  const uint32_t H = p.hidden, KC = p.kv_heads * HD, QCl = cut.QCl, KCl = cut.KCl, NQl = cut.NQl, FFl = cut.FFl;
  const uint32_t group = cut.group, chunks = p.attend / DCH, att_l = cut.n_att, nparts_dn = p.tp * p.ks_dn;
  constexpr uint32_t APH = HD + 4, AP = 4 * APH;      // as in the one-cluster form
  constexpr int PE = MT == 1 ? 4 : (MT == 2 ? 5 : 9);   // elements of the residual a thread fetches at once (hidden 576: all of them)
  auto per = [&](uint32_t items) { return (items + C - 1) >> lgC; };
  // a bulk copy's issue costs its warp some 70 cycles, so an item's copies (one a block and row) are spread over the eight warps
  const uint32_t cpw = (C * MT + DT / 32 - 1) / (DT / 32), cpa = (C + DT / 32 - 1) / (DT / 32);
  // shared memory (the same offsets in every block of a cluster); every piece is a whole number of 16 bytes
  uint8_t* ring = reinterpret_cast<uint8_t*>(((uintptr_t)smem + 1023) & ~(uintptr_t)1023);
  uint8_t* wbuf = ring + (size_t)R * SLOT_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(wbuf + WBUF_BYTES);                         // [16]
  uint4* ksm = reinterpret_cast<uint4*>(bars + 16);
  uint4* vsm = ksm + DCH * 8;
  float* xres = reinterpret_cast<float*>(vsm + DCH * 8);          // [MT][H]
  float* qkv = xres + (size_t)MT * H;                             // [MT][NQl]: the cluster's heads, q | k | v
  float* qkvp = qkv + (size_t)MT * NQl;                           // [ks_q][MT][NQl]: their sums over the slices of k, from every block
  float* att = qkvp + (size_t)p.ks_q * MT * NQl;                  // [att_l][AP]
  float* osum = att + (size_t)att_l * AP;                         // [MT][H]: the last norm's values
  float* mw = osum + (size_t)MT * H;                              // [MT * hq][chunks + 1] and [MT * hq] offsets
  float* qs = mw + (((size_t)MT * cut.hq * (chunks + 2) + 3) & ~(size_t)3);
  float* ps = qs + 4 * HD;
  float* stat = ps + 4 * DCH;
  float* halves = stat + 16;                                      // [2][MT][64]
  float* sq = halves + 2 * MT * DCOLS;                            // staging, a slot an item of the block: QKV
  float* sa = sq + (size_t)per(cut.n_qs) * MT * DCOLS;            // attention partials
  float* sg = sa + (size_t)per(att_l) * AP;                       // gate|up, BF16
  float* g1 = sg + (size_t)per(cut.n_gu) * MT * DCOLS / 2;
  float* g2 = g1 + H;
  float* cs = g2 + H;
  float* sn = cs + HD;
  DecodeLayerDev* lay = reinterpret_cast<DecodeLayerDev*>(sn + HD);   // [n_layers]
  ChunkEnt* tab = reinterpret_cast<ChunkEnt*>(lay + p.n_layers);  // [SCHED_MAX]
  uint32_t* tab_len = reinterpret_cast<uint32_t*>(tab + SCHED_MAX);   // [2]
  // the block's items of the phases whose items take divisions to name, worked out once: {column block or chunk, slice or
  // key/value head, first k-row or sequence, rows}
  uint4* it_q = reinterpret_cast<uint4*>(((uintptr_t)(tab_len + 2) + 15) & ~(uintptr_t)15);   // QKV
  uint4* it_a = it_q + per(cut.n_qs);                             // attention
  uint4* it_d = it_a + per(att_l);                                // down
  uint16_t* gu = reinterpret_cast<uint16_t*>(it_d + per(cut.n_dn));   // [MT][2 FFl] BF16: gate | up of the cluster's slice
  uint16_t* vec = gu + (size_t)MT * 2 * FFl;                      // [MT][vec_cols] BF16: a product's A operand

  const int32_t pos = *p.pos;
  if (pos < 0 || (uint32_t)pos >= p.max_len || (uint32_t)pos >= p.attend) {   // every block sees the same position
    if (tid == 0) atomicCAS(p.err, 0, 6);
    return;
  }
  for (uint32_t i = tid; i < p.n_layers * (uint32_t)(sizeof(DecodeLayerDev) / 8); i += DT)
    reinterpret_cast<uint64_t*>(lay)[i] = reinterpret_cast<const uint64_t*>(p.layers)[i];
  if (tid < HD) { cs[tid] = p.cos[(size_t)pos * HD + tid]; sn[tid] = p.sin[(size_t)pos * HD + tid]; }
  WeightWalk walk;
  walk.start_tp(&p, tab, tab_len, me, C, cut, ChunkBoxes<MT>::value * CK_ROWS);
  const uint32_t j0q = TpCut::first(me, C, 0), it0 = TpCut::first(me, C, cut.off_att), j0o = TpCut::first(me, C, cut.off_o),
                 j0d = TpCut::first(me, C, cut.off_dn);
  for (uint32_t i = tid, j = j0q + tid * C; j < cut.n_qs; i += DT, j += DT * C) {
    const uint32_t ks = j / cut.n_q, k0 = ks * p.sl_q;
    it_q[i] = make_uint4(j - ks * cut.n_q, ks, k0, k0 + p.sl_q <= H ? p.sl_q : H - k0);
  }
  for (uint32_t i = tid, it = it0 + tid * C; it < att_l; i += DT, it += DT * C) {
    const uint32_t q = it / chunks, b = q / cut.hk;
    it_a[i] = make_uint4(it - q * chunks, q - b * cut.hk, b, 0);
  }
  for (uint32_t i = tid, j = j0d + tid * C; j < cut.n_dn; i += DT, j += DT * C) {
    const uint32_t ks = j / cut.nb_h, k0 = ks * p.sl_dn;
    it_d[i] = make_uint4(j - ks * cut.nb_h, ks, k0, k0 + p.sl_dn <= FFl ? p.sl_dn : FFl - k0);
  }
  __syncthreads();
  walk.cnt = *tab_len;
  walk.lay = lay;
  for (uint32_t c = tid; c < H; c += DT) g1[c] = bf16_at(lay[0].norm1, c);
  uint32_t head = 0, parity = 0;
  bool dead = false, ahead = false;                    // (BFP8: the next chunk is already decoded into the tile)
  const long long limit = tc::wait_limit_of(p.err);
  uint64_t* xb = &bars[8];                            // [3]: QKV, attention partials, gate|up
  const uint32_t expect[3] = {cut.n_qs * MT * DCOLS * 4, att_l * group * APH * 4, cut.n_gu * MT * DCOLS * 2};
  if (tid == 0) {
    for (int r = 0; r < R; ++r) tc::mbar_init(&bars[r], BFP ? 1 + DT : 1);   // (a BFP8 chunk's exponent bytes: every thread's copies arrive)
    for (int k = 0; k < 3; ++k) tc::mbar_init(&xb[k], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int k = 0; k < 3; ++k) tc::mbar_expect_tx(&xb[k], expect[k]);   // layer 0's
  }
  __syncthreads();
  cluster.sync();                                      // every block's barriers exist before a copy may name them
  for (int r = 0; r < R; ++r) walk.issue(ring + (size_t)r * SLOT_BYTES, &bars[r]);

  for (uint32_t l = 0; l < p.n_layers; ++l) {
    const DecodeLayerDev L = lay[l];
    auto arrived = [&](int k) {
      if (!dead && !tc::mbar_wait(&xb[k], l & 1u, &dead_flag_of(p.err), limit)) { dead = true; atomicCAS(p.err, 0, TIMEOUT_CODE); }
      __syncthreads();
      if (tid == 0 && l + 1 < p.n_layers) tc::mbar_expect_tx(&xb[k], expect[k]);
    };
    float gn[GN];
#pragma unroll
    for (int i = 0; i < GN; ++i) gn[i] = tid + i * DT < H ? bf16_at(L.norm2, tid + i * DT) : 0.f;
    // ---- phase 1: the residual (the clusters' down partials of the layer before, in a fixed order), norm, QKV of the cluster's heads ----
    if (l == 0) {
      for (uint32_t i = tid; i < (uint32_t)MT * H; i += DT) xres[i] = i < p.rows * H ? p.x0[i] : 0.f;
    } else {
      // (thread t also waits for block t's word: every block has finished layer l - 1)
      add_parts_tagged<PE>(xres, MT * H, p.part_dn + (size_t)((l - 1) & 1u) * nparts_dn * MT * H, nparts_dn, (size_t)MT * H, l, dead, limit, p.err,
                       (uint32_t)tid < gridDim.x ? p.done + (size_t)((l - 1) & 1u) * gridDim.x + tid : nullptr);
    }
    __syncthreads();
    norm_rows_sm<MT>(xres, H, g1, p.eps, vec, p.vec_cols, stat);
    {
      for (uint32_t j = j0q, idx = 0; j < cut.n_qs; j += C, ++idx) {   // an item a (column block, slice of k): the slices' sums meet at the receivers
        const uint4 e = it_q[idx];
        const uint32_t jc = e.x, ks = e.y, k0 = e.z, len = e.w;
        float* slot = sq + (size_t)idx * MT * DCOLS;
        const bool whole = p.ks_q == 1;                  // one slice: the sender rounds, the receivers take the values as they come
        product_stream<MT, R, BFP>(vec + k0, p.vec_cols, len, ring, bars, head, parity, dead, limit, p.err, walk, halves,
                              [&](int r, int cc, float t) { slot[r * DCOLS + cc] = whole ? bf16_round(t) : t; }, wbuf, &ahead);
        if (const uint32_t ci = (uint32_t)(tid >> 5) * cpw + (tid & 31); (uint32_t)(tid & 31) < cpw && ci < C * MT) {
          const uint32_t d = ci / MT, r = ci - d * MT;
          copy_to_block((whole ? qkv : qkvp + (size_t)ks * MT * NQl) + (size_t)r * NQl + jc * DCOLS, slot + r * DCOLS, DCOLS * 4, &xb[0], d);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < GN; ++i)
      if (tid + i * DT < H) g2[tid + i * DT] = gn[i];
    uint4 kreg[2], vreg[2];
    auto load_cache = [&](uint32_t idx) {
      const uint4 e = it_a[idx];
      const uint32_t ch = e.x, kvh = cgi * cut.hk + e.y, b = e.z;
      if (ch * DCH > (uint32_t)pos) return;
      const uint64_t row0 = (uint64_t)b * p.max_len + (uint64_t)ch * DCH;
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const uint32_t i = tid + h2 * DT, j = i >> 3, u = i & 7;
        kreg[h2] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(L.kc) + (row0 + j) * KC + kvh * HD + u * 8);
        vreg[h2] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(L.vc) + (row0 + j) * KC + kvh * HD + u * 8);
      }
    };
    if (it0 < att_l) load_cache(0);
    if constexpr (BFP) decode_ahead<MT, R>(ring, bars, head, parity, dead, limit, p.err, walk, wbuf, ahead);
    arrived(0);

    // ---- phase 2: the attention of the cluster's heads, an item a (sequence, key/value head, 64 positions) ----
    if (it0 < att_l && p.ks_q > 1)                     // the product's BF16 result: the slices' sums in order, rounded once
      for (uint32_t i = tid; i < (uint32_t)MT * NQl; i += DT) {
        float t = qkvp[i];
        for (uint32_t k = 1; k < p.ks_q; ++k) t += qkvp[(size_t)k * MT * NQl + i];
        qkv[i] = bf16_round(t);
      }
    for (uint32_t it = it0, idx = 0; it < att_l; it += C, ++idx) {
      const uint4 e4 = it_a[idx];
      const uint32_t ch = e4.x, kvl = e4.y, kvh = cgi * cut.hk + kvl, b = e4.z;
      float* stage = sa + (size_t)idx * AP;
      __syncthreads();
      if (idx != 0) load_cache(idx);
      if (ch * DCH > (uint32_t)pos) {
        for (uint32_t i = tid; i < AP; i += DT) stage[i] = i % APH == HD ? -INFINITY : 0.f;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (const uint32_t ci = (uint32_t)(tid >> 5) * cpa + (tid & 31); (uint32_t)(tid & 31) < cpa && ci < C)
          copy_to_block(att + (size_t)it * AP, stage, group * APH * 4, &xb[1], ci);
        continue;
      }
      const float* qrow = qkv + (size_t)b * NQl;
      for (uint32_t i = tid; i < group * HD; i += DT) {
        const uint32_t g = i / HD, j = i - g * HD, base = (kvl * group + g) * HD;
        qs[g * HD + j] = __fadd_rn(__fmul_rn(qrow[base + j], cs[j]), __fmul_rn(qrow[base + (j < HD / 2 ? j + HD / 2 : j - HD / 2)], sn[j]));
      }
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const uint32_t i = tid + h2 * DT, j = i >> 3, u = i & 7;
        ksm[j * 8 + (u ^ (j & 7))] = kreg[h2];
        vsm[j * 8 + (u ^ (j & 7))] = vreg[h2];
      }
      __syncthreads();
      if ((uint32_t)pos / DCH == ch && tid < HD) {
        const uint32_t j = tid, kb = QCl + kvl * HD, vb = QCl + KCl + kvl * HD, jr = (uint32_t)pos % DCH;
        const float x = qrow[kb + j], xs = qrow[kb + (j < HD / 2 ? j + HD / 2 : j - HD / 2)];
        const uint16_t kbits = f32_to_bf16_bits(__float_as_uint(__fadd_rn(__fmul_rn(x, cs[j]), __fmul_rn(xs, sn[j]))));
        const uint16_t vbits = f32_to_bf16_bits(__float_as_uint(qrow[vb + j]));
        const uint64_t row = (uint64_t)b * p.max_len + (uint32_t)pos;
        reinterpret_cast<uint16_t*>(L.kc)[row * KC + kvh * HD + j] = kbits;
        reinterpret_cast<uint16_t*>(L.vc)[row * KC + kvh * HD + j] = vbits;
        reinterpret_cast<uint16_t*>(ksm + jr * 8 + ((j >> 3) ^ (jr & 7)))[j & 7] = kbits;
        reinterpret_cast<uint16_t*>(vsm + jr * 8 + ((j >> 3) ^ (jr & 7)))[j & 7] = vbits;
      }
      __syncthreads();
      const uint32_t g = tid / DCH, j = tid - g * DCH;
      float sc = -INFINITY;
      if (g < group && ch * DCH + j <= (uint32_t)pos) {
        float t4[4] = {0.f, 0.f, 0.f, 0.f};
        const float* q = qs + g * HD;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const uint4 kq = ksm[j * 8 + (u ^ (j & 7))];
          const uint32_t w4[4] = {kq.x, kq.y, kq.z, kq.w};
          const float4 qa = *reinterpret_cast<const float4*>(q + u * 8), qb = *reinterpret_cast<const float4*>(q + u * 8 + 4);
          const float q8[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            t4[e] = fmaf(q8[2 * e], __uint_as_float(w4[e] << 16), t4[e]);
            t4[e] = fmaf(q8[2 * e + 1], __uint_as_float(w4[e] & 0xffff0000u), t4[e]);
          }
        }
        sc = __fmul_rn((t4[0] + t4[1]) + (t4[2] + t4[3]), p.scale);
      }
      float m = sc;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      if ((tid & 31) == 0) stat[tid >> 5] = m;
      __syncthreads();
      const float mh = g < group ? fmaxf(fmaxf(stat[2 * g], stat[2 * g + 1]), -3.402823466e38f) : 0.f;
      const float e = g < group ? expf(sc - mh) : 0.f;
      if (g < group) ps[g * DCH + j] = e;
      float sum = e;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      __syncthreads();
      if ((tid & 31) == 0) stat[8 + (tid >> 5)] = sum;
      __syncthreads();
      // P.V: a head's two warps take half of the positions each, a lane two columns (one 4-byte load a position: a row of V
      // is the warp's 128 bytes), the probabilities by 16-byte loads; the halves meet in the query's idle buffer.  A load a
      // position and column, as before, kept the load pipe busy for most of the phase.
      if (g < group) {
        const uint32_t half = (j >> 5) & 1u, dp = j & 31u;
        float oa[2] = {0.f, 0.f}, ob[2] = {0.f, 0.f};    // two chains a column, joined in a fixed order
        const float* pr = ps + g * DCH + half * 32;
#pragma unroll 2
        for (int jj = 0; jj < 32; jj += 4) {
          const float4 p4 = *reinterpret_cast<const float4*>(pr + jj);
          const float pe[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
          for (int e2 = 0; e2 < 4; ++e2) {
            const uint32_t row = half * 32 + jj + e2;
            const uint32_t w2 = reinterpret_cast<const uint32_t*>(vsm + row * 8 + ((dp >> 2) ^ (row & 7)))[dp & 3];
            oa[e2 & 1] = fmaf(pe[e2], __uint_as_float(w2 << 16), oa[e2 & 1]);
            ob[e2 & 1] = fmaf(pe[e2], __uint_as_float(w2 & 0xffff0000u), ob[e2 & 1]);
          }
        }
        const float o_lo = oa[0] + oa[1], o_hi = ob[0] + ob[1];
        if (half) { qs[g * HD + 2 * dp] = o_lo; qs[g * HD + 2 * dp + 1] = o_hi; }
        __syncthreads();
        if (!half) {
          stage[g * APH + 2 * dp] = o_lo + qs[g * HD + 2 * dp];
          stage[g * APH + 2 * dp + 1] = o_hi + qs[g * HD + 2 * dp + 1];
          if (dp == 0) { stage[g * APH + HD] = mh; stage[g * APH + HD + 1] = stat[8 + 2 * g] + stat[8 + 2 * g + 1]; }
        }
      } else {
        __syncthreads();
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncthreads();
      if (const uint32_t ci = (uint32_t)(tid >> 5) * cpa + (tid & 31); (uint32_t)(tid & 31) < cpa && ci < C)
        copy_to_block(att + (size_t)it * AP, stage, group * APH * 4, &xb[1], ci);
    }
    if constexpr (BFP) decode_ahead<MT, R>(ring, bars, head, parity, dead, limit, p.err, walk, wbuf, ahead);
    arrived(1);

    // ---- phase 3: the merge of the cluster's heads, and their rows of the output projection: a partial sum a cluster ----
    uint32_t* mbase = reinterpret_cast<uint32_t*>(mw + (size_t)MT * cut.hq * (chunks + 1));   // [MT * hq]
    for (uint32_t i = tid; i < (uint32_t)MT * cut.hq; i += DT) {
      const uint32_t r = MT == 1 ? 0u : i / cut.hq, h = i - r * cut.hq, kvl = h / group, g = h - kvl * group;
      const float* base = att + (size_t)((r * cut.hk + kvl) * chunks) * AP + g * APH;
      float M = -3.402823466e38f;
      for (uint32_t c2 = 0; c2 < chunks; ++c2) M = fmaxf(M, base[(size_t)c2 * AP + HD]);
      float Lsum = 0.f;
      for (uint32_t c2 = 0; c2 < chunks; ++c2) {
        const float wgt = expf(base[(size_t)c2 * AP + HD] - M);
        mw[(size_t)i * (chunks + 1) + c2] = wgt;
        Lsum = fmaf(base[(size_t)c2 * AP + HD + 1], wgt, Lsum);
      }
      mw[(size_t)i * (chunks + 1) + chunks] = fmaxf(Lsum, 1.175494351e-38f);
      mbase[i] = (uint32_t)((size_t)((r * cut.hk + kvl) * chunks) * AP + g * APH);
    }
    __syncthreads();
    for (uint32_t i = tid; i < (uint32_t)MT * QCl; i += DT) {
      const uint32_t r = MT == 1 ? 0u : i / QCl, c = i - r * QCl, h = c / HD, d = c - h * HD;
      float v = 0.f;
      if (r < p.rows) {
        const float* base = att + mbase[r * cut.hq + h];
        const float* w = mw + (size_t)(r * cut.hq + h) * (chunks + 1);
        float O = 0.f;
        for (uint32_t c2 = 0; c2 < chunks; ++c2) O = fmaf(base[(size_t)c2 * AP + d], w[c2], O);
        v = __fdiv_rn(O, w[chunks]);
      }
      vec[(size_t)r * p.vec_cols + c] = f32_to_bf16_bits(__float_as_uint(v));
    }
    __syncthreads();
    for (uint32_t j = j0o; j < cut.nb_h; j += C) {
      unsigned long long* dst = p.part_o + ((size_t)(l & 1u) * p.tp + cgi) * MT * H + j * DCOLS;
      product_stream<MT, R, BFP>(vec, p.vec_cols, QCl, ring, bars, head, parity, dead, limit, p.err, walk, halves,
                            [&](int r, int cc, float t) { st_tagged(dst + (size_t)r * H + cc, t, l + 1); }, wbuf, &ahead);
    }

    // ---- phase 4: the residual, norm, the cluster's gate and up columns ----
    if constexpr (BFP) decode_ahead<MT, R>(ring, bars, head, parity, dead, limit, p.err, walk, wbuf, ahead);
    // (the next layer's first gains are asked for before the poll, whose wait hides their trip)
    uint16_t gnb[GN];
#pragma unroll
    for (int i = 0; i < GN; ++i)
      gnb[i] = l + 1 < p.n_layers && tid + i * DT < H ? reinterpret_cast<const uint16_t*>(lay[l + 1].norm1)[tid + i * DT] : (uint16_t)0;
    add_parts_tagged<PE>(xres, MT * H, p.part_o + (size_t)(l & 1u) * p.tp * MT * H, p.tp, (size_t)MT * H, l + 1, dead, limit, p.err);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < GN; ++i) gn[i] = __uint_as_float((uint32_t)gnb[i] << 16);
    norm_rows_sm<MT>(xres, H, g2, p.eps, vec, p.vec_cols, stat);
    {
      for (uint32_t j = j0q, idx = 0; j < cut.n_gu; j += C, ++idx) {
        uint16_t* slot = reinterpret_cast<uint16_t*>(sg) + (size_t)idx * MT * DCOLS;
        product_stream<MT, R, BFP>(vec, p.vec_cols, H, ring, bars, head, parity, dead, limit, p.err, walk, halves, [&](int r, int cc, float t) {
          slot[r * DCOLS + cc] = f32_to_bf16_bits(__float_as_uint(t));
        }, wbuf, &ahead);
        if (const uint32_t ci = (uint32_t)(tid >> 5) * cpw + (tid & 31); (uint32_t)(tid & 31) < cpw && ci < C * MT) {
          const uint32_t d = ci / MT, r = ci - d * MT;
          copy_to_block(gu + (size_t)r * 2 * FFl + j * DCOLS, slot + r * DCOLS, DCOLS * 2, &xb[2], d);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < GN; ++i)
      if (tid + i * DT < H) g1[tid + i * DT] = gn[i];
    if constexpr (BFP) decode_ahead<MT, R>(ring, bars, head, parity, dead, limit, p.err, walk, wbuf, ahead);
    arrived(2);

    // ---- phase 5: the activation of the cluster's slice of ff and its rows of the down projection: a partial a (cluster, slice) ----
    for (uint32_t j = j0d, idx = 0; j < cut.n_dn; j += C, ++idx) {
      const uint4 e = it_d[idx];
      const uint32_t cb = e.x, ks = e.y, k0 = e.z, len = e.w;
      __syncthreads();
      for (uint32_t i = tid; i < (uint32_t)MT * len; i += DT) {
        const uint32_t r = MT == 1 ? 0u : i / len, kk = i - r * len;
        const float a = __uint_as_float((uint32_t)gu[(size_t)r * 2 * FFl + k0 + kk] << 16);
        const float bq = __uint_as_float((uint32_t)gu[(size_t)r * 2 * FFl + FFl + k0 + kk] << 16);
        vec[(size_t)r * p.vec_cols + kk] = f32_to_bf16_bits(__float_as_uint(__fmul_rn(__fmul_rn(a, sigmoid_flex(a)), bq)));
      }
      __syncthreads();
      unsigned long long* dst = p.part_dn + ((size_t)(l & 1u) * nparts_dn + (size_t)cgi * p.ks_dn + ks) * MT * H + cb * DCOLS;
      product_stream<MT, R, BFP>(vec, p.vec_cols, len, ring, bars, head, parity, dead, limit, p.err, walk, halves,
                            [&](int r, int cc, float t) { st_tagged(dst + (size_t)r * H + cc, t, l + 1); }, wbuf, &ahead);
    }
    // every thread of the block is past its last read of what the layer sent it (each path here ends in a block barrier)
    if (tid == 0 && blockIdx.x != p.skip_done) st_tagged(p.done + (size_t)(l & 1u) * gridDim.x + blockIdx.x, 0.f, l + 1);
    if constexpr (BFP) decode_ahead<MT, R>(ring, bars, head, parity, dead, limit, p.err, walk, wbuf, ahead);
  }
  if (blockIdx.x == 0) {
    add_parts_tagged<PE>(xres, MT * H, p.part_dn + (size_t)((p.n_layers - 1) & 1u) * nparts_dn * MT * H, nparts_dn, (size_t)MT * H, p.n_layers,
                     dead, limit, p.err);
    __syncthreads();
    norm_rows<MT>(xres, H, p.final_norm, p.eps, osum, H, stat);
    for (uint32_t i = tid; i < p.rows * H; i += DT) p.out[i] = f32_to_bf16_bits(__float_as_uint(osum[i]));
  }
  drain_ring(bars, R, parity, limit);
  drain_received(xb, 3, p.n_layers - 1, dead, limit);
  cluster.sync();   // no block leaves while another may still store into its shared memory
}

template <int MT>
cudaError_t launch_cluster(const ClusterParams& p, size_t smem, int* cluster_blocks, cudaStream_t stream) {
  // the widest cluster the device will schedule: sixteen blocks (beyond the portable eight), else eight
  cudaError_t e = ensure_dynamic_smem((const void*)decode_cluster_kernel<MT>, smem);
  if (e != cudaSuccess) return e;
  int width = 0;
  if (!device_value_get((const void*)decode_cluster_kernel<MT>, &width)) {
    width = -1;
    for (int c : {16, 8}) {
      if ((uint32_t)c < p.min_width) continue;
      if (c > 8 && cudaFuncSetAttribute((const void*)decode_cluster_kernel<MT>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
        cudaGetLastError();
        continue;
      }
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(c); cfg.blockDim = dim3(DT); cfg.dynamicSmemBytes = smem;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = c; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
      cfg.attrs = at; cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, decode_cluster_kernel<MT>, &cfg) == cudaSuccess && n >= 1) { width = c; break; }
      cudaGetLastError();
    }
    device_value_set((const void*)decode_cluster_kernel<MT>, width);
  }
  if (width < 8 || (uint32_t)width < p.min_width) return cudaErrorNotSupported;
  *cluster_blocks = width;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(width); cfg.blockDim = dim3(DT); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = width; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, decode_cluster_kernel<MT>, p);
}

// The several-cluster form's launch: `p.tp` clusters of the widest width the device holds all at once (every block meets
// every other twice a layer, so the launch is made only where the occupancy figure says they are resident together;
// the meetings' waits are bounded all the same).
template <int MT, bool BFP>
cudaError_t launch_tp(const ClusterParams& p, size_t smem, int* cluster_blocks, cudaStream_t stream) {
  cudaError_t e = ensure_dynamic_smem((const void*)decode_tp_kernel<MT, BFP>, smem);
  if (e != cudaSuccess) return e;
  int found = 0;                                       // width * 256 + clusters the device holds at once
  if (!device_value_get((const void*)decode_tp_kernel<MT, BFP>, &found)) {
    found = 0;
    for (int c : {16, 8}) {
      if ((uint32_t)c < p.min_width) continue;
      if (c > 8 && cudaFuncSetAttribute((const void*)decode_tp_kernel<MT, BFP>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
        cudaGetLastError();
        continue;
      }
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(c * p.tp); cfg.blockDim = dim3(DT); cfg.dynamicSmemBytes = smem;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = c; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
      cfg.attrs = at; cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, decode_tp_kernel<MT, BFP>, &cfg) == cudaSuccess && n >= (int)p.tp) { found = c * 256 + (n > 255 ? 255 : n); break; }
      cudaGetLastError();
    }
    device_value_set((const void*)decode_tp_kernel<MT, BFP>, found);
  }
  const int width = found / 256, held = found % 256;
  if (width < 8 || (uint32_t)width < p.min_width || held < (int)p.tp) return cudaErrorNotSupported;
  *cluster_blocks = width;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(width * p.tp); cfg.blockDim = dim3(DT); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = width; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, decode_tp_kernel<MT, BFP>, p);
}

uint32_t slices_for(uint32_t col_blocks, uint32_t k, uint32_t grid, uint32_t* slice_len) {
  // Slices of k so that a phase's items (column blocks x slices) come to about one a block: as many slices as fit the
  // grid, at least as many as keep a slice within the tile fetched ahead, at most 8; slices of whole 32-row steps.
  uint32_t ks = grid / col_blocks;
  if (ks < 1) ks = 1;
  if (ks > 8) ks = 8;
  const uint32_t need = (k + WT_ROWS - 1) / WT_ROWS;
  if (ks < need) ks = need;
  uint32_t len = ((k + ks - 1) / ks + 31) / 32 * 32;
  if (len > k) len = k;
  *slice_len = len;
  return (k + len - 1) / len;
}

}  // namespace

namespace {
// What the cluster form needs of a shape: its buffers in a block's shared memory, its per-layer list of chunks within the
// table, hidden within what a thread fetches ahead.  Fills the shape-derived fields of `c`.
bool cluster_plan(const DecodeShape& sh, ClusterParams& c, size_t* smem) {
  const uint32_t MTc = sh.rows <= 1 ? 1 : (sh.rows <= 2 ? 2 : 4);
  const uint32_t QCc = sh.heads * HD, NQ = QCc + 2 * sh.kv_heads * HD, att_items = sh.rows * sh.kv_heads * (sh.attend / DCH);
  c.n_layers = sh.layers; c.rows = sh.rows; c.hidden = sh.hidden; c.heads = sh.heads; c.kv_heads = sh.kv_heads; c.ff = sh.ff;
  c.max_len = sh.max_len; c.attend = sh.attend; c.eps = sh.eps; c.scale = sh.scale;
  // the down projection's k in slices of about a chunk's rows (one sequence: 576, three slices and 27 items for SmolLM2-135M; else 768)
  const uint32_t want_rows = MTc == 1 ? 576u : 768u;
  c.ks_dn = (sh.ff + want_rows - 1) / want_rows;
  if (c.ks_dn < 1) c.ks_dn = 1;
  c.sl_dn = ((sh.ff + c.ks_dn - 1) / c.ks_dn + 63) / 64 * 64;   // a slice starts at a multiple of 64 rows: the copies address k in 64s
  c.ks_dn = (sh.ff + c.sl_dn - 1) / c.sl_dn;
  uint32_t vc = sh.hidden > QCc ? sh.hidden : QCc;
  if (c.sl_dn > vc) vc = c.sl_dn;
  vc = (vc + 7) / 8 * 8;
  c.vec_cols = vc;
  c.att_items = att_items;
  for (int i = 0; i < 4; ++i) c.pbytes[i] = chunk_rows_of(MTc) * 128;
  const size_t ring_slots = MTc == 1 ? RingDepth<1>::value : (MTc == 2 ? RingDepth<2>::value : RingDepth<4>::value);
  const uint32_t chunk_rows = chunk_rows_of(MTc);
  const size_t SLOT_BYTES = (size_t)chunk_rows * 128;
  // the items' staging slots, sized for a cluster of eight blocks where that fits, else of sixteen
  const uint64_t nbq = NQ / DCOLS, nbh = sh.hidden / DCOLS, nbg = 2 * sh.ff / DCOLS, nbd = nbh * c.ks_dn;
  for (uint32_t width : {8u, 16u}) {
    auto per = [&](uint64_t items) { return (items + width - 1) / width; };
    const size_t stage = (per(nbq) + per(nbh) + per(nbd)) * MTc * DCOLS + per(att_items) * 4 * (HD + 4) + per(nbg) * MTc * DCOLS / 2;
    *smem = 1024 + ring_slots * SLOT_BYTES + 16 * sizeof(uint64_t) + 2 * DCH * 8 * sizeof(uint4) +
            ((size_t)MTc * sh.hidden * 2 + (size_t)MTc * NQ + (size_t)att_items * 4 * (HD + 4) +
             (size_t)c.ks_dn * MTc * sh.hidden + 4 * HD + 4 * DCH + 16 + stage + 2 * MTc * DCOLS + 2 * sh.hidden + 2 * HD) * sizeof(float) +
            (size_t)sh.layers * sizeof(DecodeLayerDev) + SCHED_MAX * sizeof(ChunkEnt) + 8 + 16 +
            ((size_t)MTc * 2 * sh.ff + (size_t)MTc * vc) * sizeof(uint16_t);
    c.min_width = width;
    if (*smem <= 224 * 1024) break;
  }
  // the longest list of chunks a block of an eight-block cluster walks in a layer (block 0's)
  auto chunks_of = [&](uint32_t items, uint32_t rows) { return (uint64_t)((items + 7) / 8) * ((rows + chunk_rows - 1) / chunk_rows); };
  const uint64_t sched = chunks_of(NQ / DCOLS, sh.hidden) + chunks_of(sh.hidden / DCOLS, QCc) + chunks_of(2 * sh.ff / DCOLS, sh.hidden) +
                         chunks_of(sh.hidden / DCOLS * c.ks_dn, c.sl_dn);
  const uint64_t merge_words = (uint64_t)sh.heads * (sh.attend / DCH + 2);   // a row's chunk weights (and where its partials start) wait in the down projection's buffer
  return *smem <= 224 * 1024 && sh.hidden <= (uint32_t)GN * DT && sched <= SCHED_MAX && sh.ff < 65536 && 2 * sh.ff / DCOLS < 65536 &&
         merge_words <= (uint64_t)c.ks_dn * sh.hidden &&
         nbg >= 16 && nbd >= 16;                         // every block has gate|up and down items: what orders the blocks (see the kernel)
}

// The several-cluster form's plan: how many clusters share a step (the most of 4, 3, 2 that cut the heads, the key/value
// heads and ff's 64-column blocks evenly), the down projection's slices of a cluster's share of ff, the rows a chunk's copy
// brings of each matrix, and a block's shared memory.  False where no cut or no plan fits.
struct TpPlan { uint32_t G, ks, sl, ks_q, sl_q, vc, att_items, min_width, cr[4]; size_t smem; };
bool tp_plan(const DecodeShape& sh, TpPlan* t) {
  const uint32_t MTc = sh.rows <= 1 ? 1 : (sh.rows <= 2 ? 2 : 4);
  const char* e = getenv("B200TT_DECODE_TP");          // a development switch: that many clusters, or none (1)
  const uint32_t forced = e ? (uint32_t)atoi(e) : 0;
  uint32_t G = 0;
  for (uint32_t g : {4u, 3u, 2u}) {
    if (forced && g != forced) continue;
    if (sh.heads % g == 0 && sh.kv_heads % g == 0 && sh.ff % (DCOLS * g) == 0) { G = g; break; }
  }
  if (!G || sh.hidden % DCOLS) return false;
  const uint32_t hq = sh.heads / G, hk = sh.kv_heads / G, QCl = hq * HD, NQl = QCl + 2 * hk * HD, FFl = sh.ff / G, chunks = sh.attend / DCH;
  const uint32_t att_l = sh.rows * hk * chunks;
  const uint32_t want_rows = MTc == 1 ? 576u : 768u;
  uint32_t ks = (FFl + want_rows - 1) / want_rows;
  if (ks < 1) ks = 1;
  const uint32_t sl = ((FFl + ks - 1) / ks + 63) / 64 * 64;
  ks = (FFl + sl - 1) / sl;
  uint32_t vc = sh.hidden > QCl ? sh.hidden : QCl;
  if (sl > vc) vc = sl;
  vc = (vc + 7) / 8 * 8;
  const uint32_t chunk_rows = chunk_rows_of(MTc);
  // the QKV product's k in slices of whole boxes, as many as spread a cluster's few column blocks over sixteen blocks
  uint32_t ks_q = 16 / (hq + 2 * hk);
  const uint32_t boxes_q = (sh.hidden + CK_ROWS - 1) / CK_ROWS;
  if (ks_q > boxes_q) ks_q = boxes_q;
  if (MTc == 1) ks_q = 1;                              // one sequence takes a 576-row item as one chunk: slices did not pay (0.50 against 0.49 ms)
  if (ks_q < 1) ks_q = 1;
  const uint32_t sl_q = (boxes_q + ks_q - 1) / ks_q * CK_ROWS;
  ks_q = (sh.hidden + sl_q - 1) / sl_q;
  t->ks_q = ks_q; t->sl_q = sl_q;
  const uint32_t rows_of[4] = {sl_q < sh.hidden ? sl_q : sh.hidden, QCl, sh.hidden, sl};
  for (int i = 0; i < 4; ++i) {
    const uint32_t r64 = (rows_of[i] + 63) / 64 * 64;
    t->cr[i] = r64 < chunk_rows ? r64 : chunk_rows;
  }
  t->G = G; t->ks = ks; t->sl = sl; t->vc = vc; t->att_items = att_l;
  const size_t ring_slots = MTc == 1 ? RingDepth<1>::value : (MTc == 2 ? RingDepth<2>::value : RingDepth<4>::value);
  const bool bfp = sh.weights == 1;                    // datum and exponent bytes in the slots, and the BF16 tile a chunk is decoded into
  const size_t SLOT_BYTES = bfp ? ((size_t)chunk_rows * 68 + 1023) / 1024 * 1024 + (size_t)chunk_rows * 128 / ring_slots : (size_t)chunk_rows * 128;
  const uint64_t n_q = (uint64_t)(hq + 2 * hk) * ks_q, nb_h = sh.hidden / DCOLS, n_gu = 2 * FFl / DCOLS, n_dn = nb_h * ks;
  constexpr uint64_t AP = 4 * (HD + 4);
  for (uint32_t width : {8u, 16u}) {
    auto per = [&](uint64_t items) { return (items + width - 1) / width; };
    const size_t stage = per(n_q) * MTc * DCOLS + per(att_l) * AP + per(n_gu) * MTc * DCOLS / 2;
    t->smem = 1024 + ring_slots * SLOT_BYTES + 16 * sizeof(uint64_t) + 2 * DCH * 8 * sizeof(uint4) +
              ((size_t)MTc * sh.hidden * 2 + (size_t)(1 + ks_q) * MTc * NQl + (size_t)att_l * AP + (((size_t)MTc * hq * (chunks + 2) + 3) & ~(size_t)3) +
               4 * HD + 4 * DCH + 16 + 2 * MTc * DCOLS + stage + 2 * sh.hidden + 2 * HD) * sizeof(float) +
              (size_t)sh.layers * sizeof(DecodeLayerDev) + SCHED_MAX * sizeof(ChunkEnt) + 8 + 16 +
              (per(n_q) + per(att_l) + per(n_dn)) * sizeof(uint4) +
              ((size_t)MTc * 2 * FFl + (size_t)MTc * vc) * sizeof(uint16_t);
    t->min_width = width;
    if (t->smem <= 224 * 1024) break;
  }
  auto chunks_of = [&](uint64_t items, uint32_t rows) { return (uint64_t)((items + 7) / 8) * ((rows + chunk_rows - 1) / chunk_rows); };
  const uint64_t sched = chunks_of(n_q, rows_of[0]) + chunks_of(nb_h, QCl) + chunks_of(n_gu, sh.hidden) + chunks_of(n_dn, sl);
  return t->smem <= 224 * 1024 && sh.hidden <= (uint32_t)GN * DT && sched <= SCHED_MAX && sh.ff < 65536 && 2 * sh.ff / DCOLS < 65536 &&
         16 * G <= (uint32_t)DT;                         // a thread a block waits for that block's word
}

// Which form a step of BF16 matrices takes: 2 several clusters, 1 one cluster, 0 the grid.  B200TT_DECODE=grid and
// B200TT_DECODE=one force the grid and the one-cluster form (development switches; the tests run all three).
int cluster_form_of(const DecodeShape& sh, TpPlan* t) {
  const char* form = getenv("B200TT_DECODE");
  if ((form && form[0] == 'g') || sh.weights == 2) return 0;   // (BF16 and BFP8 matrices mixed: the grid form takes each as it is)
  if (!(form && form[0] == 'o') && tp_plan(sh, t)) return 2;
  if (sh.weights != 0) return 0;                       // the one-cluster form multiplies BF16 tiles where they land
  ClusterParams c{};
  size_t smem = 0;
  return cluster_plan(sh, c, &smem) ? 1 : 0;
}
}  // namespace

bool decode_layers_supported(const DecodeShape& sh, const char** why) {
  *why = "";
  if (sh.rows < 1 || sh.rows > 4) { *why = "one to four sequences a step"; return false; }
  if (sh.head_dim != HD) { *why = "heads of 64 columns"; return false; }
  if (sh.heads == 0 || sh.kv_heads == 0 || sh.heads % sh.kv_heads || sh.heads / sh.kv_heads > 4) { *why = "one to four query heads a key/value head"; return false; }
  if (sh.hidden % 64 || sh.ff % 64 || sh.hidden == 0 || sh.ff == 0) { *why = "hidden and ff in whole 64-column blocks"; return false; }
  if (sh.attend == 0 || sh.attend % DCH || sh.attend > sh.max_len) { *why = "attended positions in whole chunks of 64 inside the cache"; return false; }
  return true;
}

DecodeScratch decode_layers_scratch(const DecodeShape& sh, int grid) {
  DecodeScratch d{};
  const uint32_t MT = sh.rows <= 1 ? 1 : (sh.rows <= 2 ? 2 : 4);
  const uint32_t QC = sh.heads * HD, KC = sh.kv_heads * HD, NQKV = QC + 2 * KC;
  d.ks_qkv = slices_for(NQKV / DCOLS, sh.hidden, grid, &d.sl_qkv);
  d.ks_o = slices_for(sh.hidden / DCOLS, QC, grid, &d.sl_o);
  d.ks_gu = slices_for(2 * sh.ff / DCOLS, sh.hidden, grid, &d.sl_gu);
  d.ks_dn = slices_for(sh.hidden / DCOLS, sh.ff, grid, &d.sl_dn);
  uint64_t off = 0;
  auto take = [&](uint64_t floats) { const uint64_t at = off; off += (floats + 63) / 64 * 64; return at; };
  d.off_qkv = take((uint64_t)d.ks_qkv * MT * NQKV);
  d.off_att = take((uint64_t)sh.rows * sh.kv_heads * (sh.attend / DCH) * 4 * (HD + 2));
  d.off_o = take((uint64_t)d.ks_o * MT * sh.hidden);
  d.off_gu = take((uint64_t)d.ks_gu * MT * 2 * sh.ff);
  d.off_dn = take((uint64_t)d.ks_dn * MT * sh.hidden);
  d.off_bar = take(64);
  TpPlan t{};                                          // the several-cluster form's partial sums: 8-byte words, two copies of each
  d.tp_floats = tp_plan(sh, &t) ? 2 * ((uint64_t)2 * t.G * MT * sh.hidden + (uint64_t)2 * t.G * t.ks * MT * sh.hidden + 2 * 16 * t.G) : 0;
  d.off_tp = take(d.tp_floats);
  d.floats = off;
  return d;
}

// The tiled-copy descriptors of the layers' matrices, for the cluster form: four a layer, each over the stored [k, n]
// (BF16) as [k / 64][64][n] with a box of a chunk's rows by 64 columns, 128-byte swizzled.  False where the driver has no encoder.
size_t decode_layers_maps_bytes(const DecodeShape& sh) { return (size_t)sh.layers * 4 * sizeof(CUtensorMap); }
bool decode_layers_make_maps(const DecodeShape& sh, const DecodeLayerPtrs* recs, void* maps_host) {
  const uint32_t MTm = sh.rows <= 1 ? 1 : (sh.rows <= 2 ? 2 : 4);
  TpPlan t{};
  const int form = cluster_form_of(sh, &t);            // the several-cluster form's chunks are as deep as its items' k
  tc::EncodeTiledFn fn = tc::encode_fn();
  if (!fn) return false;
  CUtensorMap* maps = reinterpret_cast<CUtensorMap*>(maps_host);
  const uint64_t H = sh.hidden, QC = (uint64_t)sh.heads * HD, KC = (uint64_t)sh.kv_heads * HD, FF = sh.ff;
  const uint64_t kn[4][2] = {{H, QC + 2 * KC}, {QC, H}, {H, 2 * FF}, {FF, H}};
  for (uint32_t l = 0; l < sh.layers; ++l) {
    const void* w[4] = {recs[l].qkv, recs[l].o, recs[l].gate_up, recs[l].down};
    for (int i = 0; i < 4; ++i) {
      const bool bfp = (recs[l].bfp >> i) & 1u;
      if (bfp != (sh.weights == 1) || (bfp && form != 2)) return false;   // every matrix as the shape says; BFP8 only in the several-cluster form
      if (kn[i][0] % 64) return false;
      const uint64_t eb = bfp ? 1 : 2;                 // BFP8: the datum bytes [k, n] (the exponent bytes behind them travel by plain copies)
      // [k, n] seen as [k / 64][64][n]: a box of (a chunk's rows / 64) x 64 rows x 64 columns lands as the chunk's rows in order
      const cuuint64_t dims[3] = {kn[i][1], 64, (kn[i][0] + 63) / 64};
      const cuuint64_t strides[2] = {kn[i][1] * eb, kn[i][1] * eb * 64u};
      const cuuint32_t box[3] = {(cuuint32_t)DCOLS, 64u, (cuuint32_t)((form == 2 ? t.cr[i] : chunk_rows_of(MTm)) / 64)};
      const cuuint32_t estr[3] = {1, 1, 1};
      if (fn(&maps[(size_t)l * 4 + i], bfp ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(w[i]),
             dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, bfp ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    }
  }
  return true;
}

int decode_layers_grid() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const char* e = getenv("B200TT_DECODE_GRID");   // a development switch
  const int want = e ? atoi(e) : 128;            // measured on SmolLM2-135M's shape: 64, 96, 128 blocks give 1.12, 1.05, 0.98 ms a step
  return want >= 1 && want <= sms ? want : (sms < 128 ? sms : 128);
}


// Which form a step takes.  The cluster form where its plan fits and every matrix is BF16 (its products are tensor-core
// tiles of BF16 as the copies land them); with BFP8 weights every datum is decoded on the ALUs, and the grid's 128 blocks
// do that twice as fast as sixteen (measured 1.33 against 2.66 ms a step).  B200TT_DECODE=grid forces the grid form (a
// development switch; the tests run both).
bool decode_layers_cluster_wanted(const DecodeShape& sh, bool any_bfp) {
  TpPlan t{};
  return (!any_bfp || sh.weights == 1) && cluster_form_of(sh, &t) != 0;
}

cudaError_t launch_decode_layers(const DecodeShape& sh, const DecodeLayerPtrs* layers_dev, const float* x0, const void* final_norm,
                                 const float* cos_t, const float* sin_t, const int32_t* pos, uint16_t* out, float* scratch,
                                 const DecodeScratch& d, int grid, const void* maps_dev, int* err, cudaStream_t stream, const char** form) {
  static_assert(sizeof(DecodeLayerPtrs) == sizeof(DecodeLayerDev), "the host's layer record is the kernel's");
  // One cluster when the caller built its descriptors (`decode_layers_cluster_wanted`) and the device schedules one; the
  // grid form otherwise.
  ClusterParams c{};
  size_t smem_c = 0;
  TpPlan t{};
  const int want = maps_dev ? cluster_form_of(sh, &t) : 0;
  if (want == 2) {
    const uint32_t MTc = sh.rows <= 1 ? 1 : (sh.rows <= 2 ? 2 : 4);
    c.n_layers = sh.layers; c.rows = sh.rows; c.hidden = sh.hidden; c.heads = sh.heads; c.kv_heads = sh.kv_heads; c.ff = sh.ff;
    c.max_len = sh.max_len; c.attend = sh.attend; c.eps = sh.eps; c.scale = sh.scale;
    c.ks_dn = t.ks; c.sl_dn = t.sl; c.vec_cols = t.vc; c.att_items = t.att_items; c.min_width = t.min_width; c.tp = t.G; c.ks_q = t.ks_q; c.sl_q = t.sl_q;
    {
      TpShape& u = c.cut;
      u.hq = sh.heads / t.G; u.hk = sh.kv_heads / t.G; u.QCl = u.hq * HD; u.KCl = u.hk * HD; u.NQl = u.QCl + 2 * u.KCl;
      u.FFl = sh.ff / t.G; u.nfl = u.FFl / DCOLS; u.ffb = sh.ff / DCOLS;
      u.n_q = u.hq + 2 * u.hk; u.n_qs = u.n_q * t.ks_q; u.n_att = sh.rows * u.hk * (sh.attend / DCH); u.nb_h = sh.hidden / DCOLS;
      u.n_gu = 2 * u.nfl; u.n_dn = u.nb_h * t.ks;
      u.off_att = u.n_qs; u.off_o = u.off_att + u.n_att; u.off_dn = u.off_o + u.nb_h; u.group = sh.heads / sh.kv_heads;
    }
    const bool bfp = sh.weights == 1;
    c.bfp = bfp ? 1u : 0u;
    const char* skip = getenv("B200TT_DEBUG_DECODE_SKIP_DONE");   // a test's hook (see `skip_done`)
    c.skip_done = skip ? (uint32_t)atoi(skip) : ~0u;
    for (int i = 0; i < 4; ++i) { c.crows[i] = t.cr[i]; c.pbytes[i] = t.cr[i] * (bfp ? 64 : 128); }
    {
      const uint32_t QCg = sh.heads * HD, NQg = QCg + 2 * sh.kv_heads * HD;
      const uint32_t kn[4][2] = {{sh.hidden, NQg}, {QCg, sh.hidden}, {sh.hidden, 2 * sh.ff}, {sh.ff, sh.hidden}};
      for (int i = 0; i < 4; ++i) { c.kn[i][0] = kn[i][0]; c.kn[i][1] = kn[i][1]; }
    }
    c.layers = reinterpret_cast<const DecodeLayerDev*>(layers_dev);
    c.x0 = x0; c.final_norm = final_norm; c.cos = cos_t; c.sin = sin_t; c.pos = pos; c.out = out; c.err = err;
    c.maps = reinterpret_cast<const CUtensorMap*>(maps_dev);
    // the partials' words (two copies of each) follow the grid form's scratch; a word's tag is the layer's, so all start at zero
    const size_t words_o = (size_t)2 * t.G * MTc * sh.hidden, words_dn = (size_t)2 * t.G * t.ks * MTc * sh.hidden;
    const size_t words_done = (size_t)2 * 16 * t.G;
    if (d.tp_floats < 2 * (words_o + words_dn + words_done)) return cudaErrorInvalidValue;
    c.part_o = reinterpret_cast<unsigned long long*>(scratch + d.off_tp);
    c.part_dn = c.part_o + words_o;
    c.done = c.part_dn + words_dn;
    cudaError_t ce = cudaMemsetAsync(c.part_o, 0, (words_o + words_dn + words_done) * sizeof(unsigned long long), stream);
    if (ce != cudaSuccess) return ce;
    int width = 0;
    if (bfp)
      ce = MTc == 1 ? launch_tp<1, true>(c, t.smem, &width, stream)
                    : (MTc == 2 ? launch_tp<2, true>(c, t.smem, &width, stream) : launch_tp<4, true>(c, t.smem, &width, stream));
    else
      ce = MTc == 1 ? launch_tp<1, false>(c, t.smem, &width, stream)
                    : (MTc == 2 ? launch_tp<2, false>(c, t.smem, &width, stream) : launch_tp<4, false>(c, t.smem, &width, stream));
    if (ce != cudaErrorNotSupported) {
      static const char* const names[2][3] = {{"cluster8x2", "cluster8x3", "cluster8x4"}, {"cluster16x2", "cluster16x3", "cluster16x4"}};
      *form = names[width == 16][t.G - 2];
      return ce;
    }
    // (the descriptors were built for this form's chunks: the one-cluster form cannot use them, the grid form needs none)
  }
  if (want == 1 && cluster_plan(sh, c, &smem_c)) {
    const uint32_t MTc = sh.rows <= 1 ? 1 : (sh.rows <= 2 ? 2 : 4);
    c.layers = reinterpret_cast<const DecodeLayerDev*>(layers_dev);
    c.x0 = x0; c.final_norm = final_norm; c.cos = cos_t; c.sin = sin_t; c.pos = pos; c.out = out; c.err = err;
    c.maps = reinterpret_cast<const CUtensorMap*>(maps_dev);
    int width = 0;
    cudaError_t ce = MTc == 1 ? launch_cluster<1>(c, smem_c, &width, stream)
                              : (MTc == 2 ? launch_cluster<2>(c, smem_c, &width, stream) : launch_cluster<4>(c, smem_c, &width, stream));
    if (ce != cudaErrorNotSupported) {
      *form = width == 16 ? "cluster16" : "cluster8";
      return ce;
    }
  }
  *form = "grid";
  DecodeParams p{};
  p.layers = reinterpret_cast<const DecodeLayerDev*>(layers_dev);
  p.n_layers = sh.layers; p.rows = sh.rows; p.hidden = sh.hidden; p.heads = sh.heads; p.kv_heads = sh.kv_heads; p.ff = sh.ff;
  p.max_len = sh.max_len; p.attend = sh.attend; p.eps = sh.eps; p.scale = sh.scale;
  p.x0 = x0; p.final_norm = final_norm; p.cos = cos_t; p.sin = sin_t; p.pos = pos; p.out = out;
  p.part_qkv = scratch + d.off_qkv; p.part_att = scratch + d.off_att; p.part_o = scratch + d.off_o;
  p.part_gu = scratch + d.off_gu; p.part_dn = scratch + d.off_dn;
  p.bar = reinterpret_cast<unsigned*>(scratch + d.off_bar);
  p.err = err;
  p.ks_qkv = d.ks_qkv; p.sl_qkv = d.sl_qkv; p.ks_o = d.ks_o; p.sl_o = d.sl_o;
  p.ks_gu = d.ks_gu; p.sl_gu = d.sl_gu; p.ks_dn = d.ks_dn; p.sl_dn = d.sl_dn;
  const uint32_t MT = sh.rows <= 1 ? 1 : (sh.rows <= 2 ? 2 : 4);
  const uint32_t QC = sh.heads * HD;
  uint32_t vc = sh.hidden > QC ? sh.hidden : QC;
  if (d.sl_dn > vc) vc = d.sl_dn;
  p.vec_cols = vc;
  const size_t smem = (size_t)WT_ROWS * 64 * 2 + 2 * DCH * 8 * sizeof(uint4) +
                      ((size_t)MT * sh.hidden + (size_t)MT * vc + 8 * MT * DCOLS + 4 * HD + 4 * DCH + 16) * sizeof(float);
  cudaError_t e = cudaMemsetAsync(p.bar, 0, 64 * sizeof(float), stream);   // the barrier's counter and its abort flag start at zero
  if (e != cudaSuccess) return e;
  void* args[] = {(void*)&p};
#define GO(M)                                                                                         \
  do {                                                                                                \
    e = ensure_dynamic_smem((const void*)decode_layers_kernel<M>, smem);                              \
    if (e != cudaSuccess) return e;                                                                   \
    e = cudaLaunchCooperativeKernel((const void*)decode_layers_kernel<M>, dim3(grid), dim3(DT), args, smem, stream); \
  } while (0)
  if (MT == 1) GO(1); else if (MT == 2) GO(2); else GO(4);
#undef GO
  return e;
}

}  // namespace b200
