// One token a sequence through every layer of a Llama-architecture decoder in ONE launch: the device side of the
// reference's traced generation step (crates/tt-models/src/generate.rs:781; layer crates/tt-models/src/llama.rs:371-507;
// cache crates/tt-models/src/kv_cache.rs:185-330).  The composed step is eleven small launches a layer whose device
// work (a layer's 9 MB of weights) takes far less time than their launch latencies; here a cooperative grid of
// persistent blocks walks the layers with five grid-wide barriers a layer instead.
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
// 16-byte (8-byte) group of 8 columns.  Every sum has a fixed order, so a step's bits do not depend on the launch.
// Every spin of the barrier is bounded by the engine's wait limit: when it runs out the error word becomes TIMEOUT,
// a flag tells the other blocks, and every block returns.
#include <cooperative_groups.h>
#include <cstdint>
#include <cuda_runtime.h>

#include "device_math.cuh"
#include "kernels.h"

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

struct Shared {
  float* xres;    // [MT][hidden]  the residual stream
  float* vec;     // [MT][vec_cols] a product's A operand
  float* red;     // [8][MT][64]
  uint32_t* ksm;  // [64][33] a chunk of keys (BF16 pairs), padded
  uint32_t* vsm;  // [64][33] a chunk of values
  float* qs;      // [4][64] rotated queries of a group
  float* ps;      // [4][64] probabilities
  float* stat;    // [16] small reductions
};

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
template <int MT>
__device__ __forceinline__ void product_item(const float* a, uint32_t lda, const void* w, int bfp, uint64_t k_total, uint64_t n,
                                             uint32_t k0, uint32_t len, uint32_t c0, float* out /* [MT][n] */, float* red) {
  const int tid = threadIdx.x, cg = tid & 7, kr = tid >> 3, warp = tid >> 5, lane = tid & 31;
  float acc[MT][8];
#pragma unroll
  for (int r = 0; r < MT; ++r)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[r][e] = 0.f;
  const uint64_t col = (uint64_t)c0 + cg * 8;
  if (col < n) {
    if (!bfp) {
      const uint16_t* bp = reinterpret_cast<const uint16_t*>(w) + (uint64_t)k0 * n + col;
      for (uint32_t kk0 = kr; kk0 < len; kk0 += 32 * 4) {
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
      for (uint32_t kk0 = kr; kk0 < len; kk0 += 32 * 4) {
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
      out[(uint64_t)r * n + oc] = t;
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

template <int MT>
__global__ void __launch_bounds__(DT, 1) decode_layers_kernel(const DecodeParams p) {
  extern __shared__ float smem[];
  __shared__ int ok_word;
  Shared s;
  s.xres = smem;
  s.vec = s.xres + (size_t)MT * p.hidden;
  s.red = s.vec + (size_t)MT * p.vec_cols;
  s.ksm = reinterpret_cast<uint32_t*>(s.red + 8 * MT * DCOLS);
  s.vsm = s.ksm + DCH * 33;
  s.qs = reinterpret_cast<float*>(s.vsm + DCH * 33);
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
    {
      const uint32_t nb = NQKV / DCOLS, items = nb * p.ks_qkv;
      for (uint32_t it = blockIdx.x; it < items; it += gridDim.x) {
        const uint32_t cb = it % nb, ks = it / nb, k0 = ks * p.sl_qkv;
        const uint32_t len = k0 + p.sl_qkv <= H ? p.sl_qkv : H - k0;
        product_item<MT>(s.vec + k0, p.vec_cols, L.qkv, L.bfp & 1, H, NQKV, k0, len, cb * DCOLS, p.part_qkv + (size_t)ks * MT * NQKV, s.red);
      }
    }
    if (!grid_barrier(p.bar, barrier_index++, limit, p.err, &ok_word)) return;

    // ---- phase 2: RoPE, the cache write, attention over chunks of positions ------------------------------------------
    {
      const uint32_t items = p.rows * p.kv_heads * chunks;
      for (uint32_t it = blockIdx.x; it < items; it += gridDim.x) {
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
        // rotated queries of the group (F32), and the step's key and value for this head
        for (uint32_t i = tid; i < group * HD; i += DT) {
          const uint32_t g = i / HD, j = i - g * HD, base = (kvh * group + g) * HD;
          const float x = qkv_at(base + j), xs = qkv_at(base + (j < HD / 2 ? j + HD / 2 : j - HD / 2));
          s.qs[g * HD + j] = __fadd_rn(__fmul_rn(x, cs[j]), __fmul_rn(xs, sn[j]));
        }
        const bool writer = (uint32_t)pos / DCH == ch;
        if (writer && tid < HD) {
          const uint32_t j = tid, kb = QC + kvh * HD, vb = QC + KC + kvh * HD;
          const float x = qkv_at(kb + j), xs = qkv_at(kb + (j < HD / 2 ? j + HD / 2 : j - HD / 2));
          const float kr = __fadd_rn(__fmul_rn(x, cs[j]), __fmul_rn(xs, sn[j]));
          const uint64_t row = (uint64_t)b * p.max_len + (uint32_t)pos;
          reinterpret_cast<uint16_t*>(L.kc)[row * KC + kvh * HD + j] = f32_to_bf16_bits(__float_as_uint(kr));
          reinterpret_cast<uint16_t*>(L.vc)[row * KC + kvh * HD + j] = f32_to_bf16_bits(__float_as_uint(qkv_at(vb + j)));
        }
        __syncthreads();                               // the step's own row is visible to this block
        // the chunk's keys and values into shared memory: 64 rows of 128 bytes each
        {
          const uint64_t row0 = (uint64_t)b * p.max_len + (uint64_t)ch * DCH;
          for (uint32_t i = tid; i < DCH * 8; i += DT) {
            const uint32_t j = i >> 3, u = i & 7;
            const uint4 kq = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(L.kc) + (row0 + j) * KC + kvh * HD + u * 8);
            const uint4 vq = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(L.vc) + (row0 + j) * KC + kvh * HD + u * 8);
            uint32_t* kd = s.ksm + j * 33 + u * 4;
            uint32_t* vd = s.vsm + j * 33 + u * 4;
            kd[0] = kq.x; kd[1] = kq.y; kd[2] = kq.z; kd[3] = kq.w;
            vd[0] = vq.x; vd[1] = vq.y; vd[2] = vq.z; vd[3] = vq.w;
          }
        }
        __syncthreads();
        // scores: a thread a (head of the group, position)
        const uint32_t g = tid / DCH, j = tid - g * DCH;
        float sc = -INFINITY;
        if (g < group) {
          const uint32_t pj = ch * DCH + j;
          if (pj <= (uint32_t)pos) {
            float t = 0.f;
            const uint32_t* kr = s.ksm + j * 33;
            const float* q = s.qs + g * HD;
#pragma unroll 8
            for (int d2 = 0; d2 < HD / 2; ++d2) {
              const uint32_t w2 = kr[d2];
              t = fmaf(q[2 * d2], __uint_as_float(w2 << 16), t);
              t = fmaf(q[2 * d2 + 1], __uint_as_float(w2 & 0xffff0000u), t);
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
            const uint32_t w2 = s.vsm[jj * 33 + (d >> 1)];
            o = fmaf(pr[jj], __uint_as_float((d & 1) ? (w2 & 0xffff0000u) : (w2 << 16)), o);
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
    __syncthreads();
    {
      const uint32_t nb = H / DCOLS, items = nb * p.ks_o;
      for (uint32_t it = blockIdx.x; it < items; it += gridDim.x) {
        const uint32_t cb = it % nb, ks = it / nb, k0 = ks * p.sl_o;
        const uint32_t len = k0 + p.sl_o <= QC ? p.sl_o : QC - k0;
        product_item<MT>(s.vec + k0, p.vec_cols, L.o, (L.bfp >> 1) & 1, QC, H, k0, len, cb * DCOLS, p.part_o + (size_t)ks * MT * H, s.red);
      }
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
    {
      const uint32_t nb = 2 * FF / DCOLS, items = nb * p.ks_gu;
      for (uint32_t it = blockIdx.x; it < items; it += gridDim.x) {
        const uint32_t cb = it % nb, ks = it / nb, k0 = ks * p.sl_gu;
        const uint32_t len = k0 + p.sl_gu <= H ? p.sl_gu : H - k0;
        product_item<MT>(s.vec + k0, p.vec_cols, L.gate_up, (L.bfp >> 2) & 1, H, 2 * FF, k0, len, cb * DCOLS, p.part_gu + (size_t)ks * MT * 2 * FF, s.red);
      }
    }
    if (!grid_barrier(p.bar, barrier_index++, limit, p.err, &ok_word)) return;

    // ---- phase 5: silu(gate) * up for an item's slice of k, the down projection ------------------------------------------
    {
      const uint32_t nb = H / DCOLS, items = nb * p.ks_dn;
      for (uint32_t it = blockIdx.x; it < items; it += gridDim.x) {
        const uint32_t cb = it % nb, ks = it / nb, k0 = ks * p.sl_dn;
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
        __syncthreads();
        product_item<MT>(s.vec, p.vec_cols, L.down, (L.bfp >> 3) & 1, FF, H, k0, len, cb * DCOLS, p.part_dn + (size_t)ks * MT * H, s.red);
      }
    }
    if (!grid_barrier(p.bar, barrier_index++, limit, p.err, &ok_word)) return;
  }

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

uint32_t slices_for(uint32_t col_blocks, uint32_t k, uint32_t grid, uint32_t* slice_len) {
  // as many slices of k as it takes to give every block an item, in slices of whole 32-row steps, at most 8
  uint32_t ks = (grid + col_blocks - 1) / col_blocks;
  if (ks < 1) ks = 1;
  if (ks > 8) ks = 8;
  uint32_t len = ((k + ks - 1) / ks + 31) / 32 * 32;
  if (len > k) len = k;
  ks = (k + len - 1) / len;
  *slice_len = len;
  return ks;
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
  d.floats = off;
  return d;
}

int decode_layers_grid() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms < 64 ? sms : 64;   // the phases have 27 to 96 items; more blocks only lengthen the barriers
}

cudaError_t launch_decode_layers(const DecodeShape& sh, const DecodeLayerPtrs* layers_dev, const float* x0, const void* final_norm,
                                 const float* cos_t, const float* sin_t, const int32_t* pos, uint16_t* out, float* scratch,
                                 const DecodeScratch& d, int grid, int* err, cudaStream_t stream) {
  static_assert(sizeof(DecodeLayerPtrs) == sizeof(DecodeLayerDev), "the host's layer record is the kernel's");
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
  const size_t smem = ((size_t)MT * sh.hidden + (size_t)MT * vc + 8 * MT * DCOLS + 4 * HD + 4 * DCH + 16) * sizeof(float) +
                      2 * DCH * 33 * sizeof(uint32_t);
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
