// Attention for a few query rows a key/value head (a decode step's) as one op: the device side
// of `Engine::attention_rows` (crates/burn-tt/src/server.rs:257; the reference kernel's contract
// is crates/tt-kernels/src/attention.rs:360-372).  For head i of `items`:
//     out_i = softmax(scale * q_i K_i^T, masked) V_i,   q_i [m, d], K_i [l, d], V_i [l, dv]
// with the composition's steps in the composition's order: the product, `SCALE_MASK_FILL`
// (x * scale, then -inf where the mask is set), the row maximum clamped to -FLT_MAX, exp(x - max),
// the row sum clamped to FLT_MIN, the division, and the product with V.
//
// The work is reading K and V once, so the bound is HBM.  The host groups the heads that share a
// key/value block (grouped-query attention) into jobs of up to 8 query rows, so K and V are read
// once for all of them.  A job's positions are split over `splits` blocks when there are too few
// jobs to fill the SMs (each block keeps its own maximum, sum and unnormalised rows, and a second
// small kernel joins them).  The scores never leave shared memory.
//   scores: eight lanes a key, a lane a 16-byte unit (whole 128-byte lines a warp load), the partial sums of
//           several keys joined by a butterfly of shuffles; for head widths that are not whole groups, a lane
//           a key walking its row in 32-byte steps against the query rows broadcast from shared memory;
//   softmax: the whole block a row;
//   rows x V: a thread a 16-byte column group and a slice of positions, rows in registers.
#include <cfloat>
#include <cstdint>
#include <cstdlib>
#include <cuda_runtime.h>

#include "device_math.cuh"
#include "kernels.h"
#include "pdl.cuh"

namespace b200 {
namespace {

constexpr int THREADS = 256;
constexpr int WARPS = THREADS / 32;

// A 16-byte piece of a row: loaded raw (it waits in four registers) and widened where it is used.
template <typename KV> struct Unit;
template <> struct Unit<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ uint4 load(const float* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
  static __device__ __forceinline__ void widen(const uint4& w, float* f) {
    f[0] = __uint_as_float(w.x); f[1] = __uint_as_float(w.y); f[2] = __uint_as_float(w.z); f[3] = __uint_as_float(w.w);
  }
};
template <> struct Unit<uint16_t> {
  static constexpr int N = 8;
  static __device__ __forceinline__ uint4 load(const uint16_t* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
  static __device__ __forceinline__ void widen(const uint4& w, float* f) {
    f[0] = __uint_as_float(w.x << 16); f[1] = __uint_as_float(w.x & 0xffff0000u);
    f[2] = __uint_as_float(w.y << 16); f[3] = __uint_as_float(w.y & 0xffff0000u);
    f[4] = __uint_as_float(w.z << 16); f[5] = __uint_as_float(w.z & 0xffff0000u);
    f[6] = __uint_as_float(w.w << 16); f[7] = __uint_as_float(w.w & 0xffff0000u);
  }
};

// the result element: F32, or rounded once to BF16 (what `cast_float` would make of it)
__device__ __forceinline__ void put(void* out, int bf16, uint64_t i, float v) {
  if (bf16) reinterpret_cast<uint16_t*>(out)[i] = f32_to_bf16_bits(__float_as_uint(v));
  else reinterpret_cast<float*>(out)[i] = v;
}

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float w = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, w) : v + w;
  }
  __syncthreads();                       // sh is free again
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = sh[0];
#pragma unroll
  for (int w = 1; w < WARPS; ++w) r = is_max ? fmaxf(r, sh[w]) : r + sh[w];
  return r;
}

// grid (splits, jobs).  Shared memory: q [RT][d], s [RT][lc], red [slices][dv or less].
template <typename KV, int RT, bool GROUPED>
__global__ void __launch_bounds__(THREADS, RT >= 8 ? 2 : (RT >= 4 ? 3 : 4))
attention_rows_kernel(const float* __restrict__ q, const KV* __restrict__ k, uint64_t k_ld, const KV* __restrict__ v,
                      uint64_t v_ld, const uint32_t* __restrict__ mask, const AttnJob* __restrict__ jobs,
                      const AttnRow* __restrict__ rows, int d, int l, int dv, int lc, float scale,
                      void* __restrict__ out, int out_bf16, float* __restrict__ part_o, float* __restrict__ part_ms) {
  constexpr int UN = Unit<KV>::N;
  extern __shared__ float smem[];
  __shared__ float sh[WARPS];
  pdl_enter();
  float* qs = smem;                        // [RT][d]
  float* s = qs + (size_t)RT * d;          // [RT][lc]
  float* red = s + (size_t)RT * lc;        // [nsl][lanes_c * UN]: one row's slices
  const int job_i = blockIdx.y, split = blockIdx.x, splits = gridDim.x;
  const AttnJob job = jobs[job_i];
  const AttnRow* jr = rows + job.row_start;
  const int nrows = job.nrows;
  const int j0 = split * lc;
  const int n = min(lc, l - j0);           // this block's positions
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int i = tid; i < RT * d; i += THREADS) {
    const int r = i / d, e = i % d;
    qs[i] = r < nrows ? q[jr[r].q_off + e] : 0.f;
  }
  __syncthreads();

  // ---- scores, grouped form: eight lanes a key, a lane a 16-byte unit of it, so a warp's load is four keys'
  // whole 128-byte lines (a lane a key makes it 32 lines of 32 bytes, and the line lookups then bound the loads).
  // A lane keeps its partial dot products for KB keys; a butterfly over the group's eight lanes adds them and
  // leaves key kb's score in lane 8 kb / KB of the group.
  if constexpr (GROUPED) {
    constexpr int G = 8, NG = 32 / G, KB = RT >= 2 ? 4 : 8, LD = 4;
    const int cg = lane & (G - 1), grp = lane / G;
    const int iters = d / (G * UN);           // d / UN is a multiple of 8 on this path
    for (int wb = warp * NG * KB; wb < n; wb += WARPS * NG * KB) {     // the same trip count for a warp's lanes
      const int jb = wb + grp * KB;
      float acc[RT][KB];
#pragma unroll
      for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int b = 0; b < KB; ++b) acc[r][b] = 0.f;
      for (int it = 0; it < iters; ++it) {
        const int eoff = (cg + it * G) * UN;
        const float* qp = qs + eoff;
#pragma unroll
        for (int b0 = 0; b0 < KB; b0 += LD) {
          uint4 raw[LD];
#pragma unroll
          for (int u = 0; u < LD; ++u) {
            const int j = jb + b0 + u;
            raw[u] = Unit<KV>::load(k + job.k_off + (uint64_t)(j0 + (j < n ? j : 0)) * k_ld + eoff);
          }
#pragma unroll
          for (int u = 0; u < LD; ++u) {
            float x[UN];
            Unit<KV>::widen(raw[u], x);
#pragma unroll
            for (int r = 0; r < RT; ++r) {
              float a = acc[r][b0 + u];
#pragma unroll
              for (int e4 = 0; e4 < UN; e4 += 4) {
                const float4 qq = *reinterpret_cast<const float4*>(qp + (size_t)r * d + e4);
                a = fmaf(x[e4], qq.x, a); a = fmaf(x[e4 + 1], qq.y, a);
                a = fmaf(x[e4 + 2], qq.z, a); a = fmaf(x[e4 + 3], qq.w, a);
              }
              acc[r][b0 + u] = a;
            }
          }
        }
      }
#pragma unroll
      for (int r = 0; r < RT; ++r) {
        // halving stages: a lane keeps the half of the keys its bit names and takes the partner's sums for them
        int vals = KB;
#pragma unroll
        for (int off = G / 2; off >= 1; off >>= 1) {
          const bool upper = (cg & off) != 0;
          if (vals > 1) {
            const int half = vals / 2;
#pragma unroll
            for (int i = 0; i < KB / 2; ++i) {
              if (i < half) {
                const float send = upper ? acc[r][i] : acc[r][i + half];
                const float keep = upper ? acc[r][i + half] : acc[r][i];
                acc[r][i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
              }
            }
            vals = half;
          } else {
            acc[r][0] += __shfl_xor_sync(0xffffffffu, acc[r][0], off);
          }
        }
      }
      // lane cg holds key cg * KB / G (every lane of a run of G / KB lanes the same sum)
      const int kb = cg / (G / KB);
      const int j = jb + kb;
      if ((cg % (G / KB)) == 0 && j < n) {
        const bool off = mask[j0 + j] != 0;
#pragma unroll
        for (int r = 0; r < RT; ++r) s[(size_t)r * lc + j] = off ? -INFINITY : acc[r][0] * scale;
      }
    }
  } else
  // ---- scores: a lane a key; 32 bytes of the key a step, four steps in flight
  {
    const int steps = d / (2 * UN);         // d is a multiple of 32
    for (int jb = warp * 32; jb < n; jb += THREADS) {
      const int j = jb + lane;
      const bool has = j < n;
      const KV* kr = k + job.k_off + (uint64_t)(j0 + (has ? j : 0)) * k_ld;
      float acc[RT][2];
#pragma unroll
      for (int r = 0; r < RT; ++r) { acc[r][0] = 0.f; acc[r][1] = 0.f; }
      for (int sb = 0; sb < steps; sb += 4) {
        uint4 raw[4][2];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (sb + u < steps) {
            raw[u][0] = Unit<KV>::load(kr + (sb + u) * 2 * UN);
            raw[u][1] = Unit<KV>::load(kr + (sb + u) * 2 * UN + UN);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (sb + u < steps) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              float x[UN];
              Unit<KV>::widen(raw[u][hf], x);
              const float* qp = qs + (sb + u) * 2 * UN + hf * UN;
#pragma unroll
              for (int r = 0; r < RT; ++r) {
#pragma unroll
                for (int e4 = 0; e4 < UN; e4 += 4) {
                  const float4 qq = *reinterpret_cast<const float4*>(qp + (size_t)r * d + e4);
                  float& a = acc[r][(UN == 4 ? hf : (e4 >> 2)) & 1];
                  a = fmaf(x[e4], qq.x, a); a = fmaf(x[e4 + 1], qq.y, a);
                  a = fmaf(x[e4 + 2], qq.z, a); a = fmaf(x[e4 + 3], qq.w, a);
                }
              }
            }
          }
        }
      }
      if (has) {
        const bool off = mask[j0 + j] != 0;
#pragma unroll
        for (int r = 0; r < RT; ++r) s[(size_t)r * lc + j] = off ? -INFINITY : (acc[r][0] + acc[r][1]) * scale;
      }
    }
  }
  __syncthreads();

  // ---- the whole block a row: maximum, exponentials, sum
#pragma unroll 1
  for (int r = 0; r < RT; ++r) {
    if (r >= nrows) break;                 // the same for every thread
    float* sr = s + (size_t)r * lc;
    float mx = -INFINITY;
    for (int j = tid; j < n; j += THREADS) mx = fmaxf(mx, sr[j]);
    mx = block_reduce(mx, true, sh);
    mx = (mx < -FLT_MAX) ? -FLT_MAX : mx;
    float sum = 0.f;
    for (int j = tid; j < n; j += THREADS) {
      const float p = expf(sr[j] - mx);
      sr[j] = p;
      sum += p;
    }
    sum = block_reduce(sum, false, sh);
    if (splits == 1) {
      const float den = (sum < FLT_MIN) ? FLT_MIN : sum;
      for (int j = tid; j < n; j += THREADS) sr[j] = sr[j] / den;
    } else if (tid == 0) {
      float* ms = part_ms + (((size_t)job_i * splits + split) * RT + r) * 2;
      ms[0] = mx;
      ms[1] = sum;
    }
  }
  __syncthreads();

  // ---- rows x V: thread = (16-byte column group, slice of positions); four positions in flight
  {
    const int cgn = dv / UN;                          // column groups a row
    const int lanes_c = cgn < THREADS ? cgn : THREADS;
    const int nsl = THREADS / lanes_c;                // position slices
    const int sl = tid / lanes_c, cg = tid % lanes_c;
    const bool active = sl < nsl;
    for (int cb = 0; cb < cgn; cb += lanes_c) {
      const bool mine = active && cb + cg < cgn;
      const int c = (cb + cg) * UN;
      float acc[RT][UN];
#pragma unroll
      for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int e = 0; e < UN; ++e) acc[r][e] = 0.f;
      if (mine) {
        const KV* vb = v + job.v_off + (uint64_t)j0 * v_ld + c;
        for (int j = sl; j < n; j += nsl * 4) {
          uint4 raw[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int jj = j + u * nsl;
            if (jj < n) raw[u] = Unit<KV>::load(vb + (uint64_t)jj * v_ld);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int jj = j + u * nsl;
            if (jj < n) {
              float x[UN];
              Unit<KV>::widen(raw[u], x);
#pragma unroll
              for (int r = 0; r < RT; ++r) {
                const float p = s[(size_t)r * lc + jj];
#pragma unroll
                for (int e = 0; e < UN; ++e) acc[r][e] = fmaf(p, x[e], acc[r][e]);
              }
            }
          }
        }
      }
      // join the slices in a fixed order, a row at a time: slot [sl][cg][e]
#pragma unroll
      for (int r = 0; r < RT; ++r) {
        if (r >= nrows) break;               // the same for every thread
        __syncthreads();
        if (active) {
#pragma unroll
          for (int e = 0; e < UN; ++e) red[((size_t)sl * lanes_c + cg) * UN + e] = acc[r][e];
        }
        __syncthreads();
        for (int w = tid; w < lanes_c * UN; w += THREADS) {
          const int col = cb * UN + w;
          if (col < dv) {
            float t = 0.f;
            for (int z = 0; z < nsl; ++z) t += red[(size_t)z * lanes_c * UN + w];
            if (splits == 1) put(out, out_bf16, jr[r].out_off + col, t);
            else part_o[(((size_t)job_i * splits + split) * RT + r) * dv + col] = t;
          }
        }
      }
    }
  }
}

// Joins the splits of a job's row: M = max of the maxima, L = sum of sums * exp(max_s - M) (clamped),
// row = sum of rows_s * exp(max_s - M) / L.  grid (rt, jobs), a thread a column.
__global__ void __launch_bounds__(128)
attention_join_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ms, const AttnJob* __restrict__ jobs,
                      const AttnRow* __restrict__ rows, int splits, int rt, int dv, void* __restrict__ out, int out_bf16) {
  pdl_enter();
  const size_t job_i = blockIdx.y, r = blockIdx.x;
  const AttnJob job = jobs[job_i];
  if ((int)r >= job.nrows) return;
  const float* ms0 = part_ms + ((job_i * splits) * rt + r) * 2;
  const size_t stride = (size_t)rt * 2;
  float mx = -FLT_MAX;
  for (int z = 0; z < splits; ++z) mx = fmaxf(mx, ms0[z * stride]);
  float den = 0.f;
  for (int z = 0; z < splits; ++z) den += ms0[z * stride + 1] * expf(ms0[z * stride] - mx);
  den = (den < FLT_MIN) ? FLT_MIN : den;
  const uint64_t dst = rows[job.row_start + r].out_off;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float t = 0.f;
    for (int z = 0; z < splits; ++z)
      t += part_o[((job_i * splits + z) * rt + r) * dv + c] * expf(ms0[z * stride] - mx);
    put(out, out_bf16, dst + c, t / den);
  }
}

size_t smem_floats(int rt, int d, int lc, int dv, int kv_bf16) {
  const int un = kv_bf16 ? 8 : 4;
  const int cgn = dv / un;
  const int lanes_c = cgn < THREADS ? cgn : THREADS;
  const int nsl = THREADS / lanes_c;
  return (size_t)rt * d + (size_t)rt * lc + (size_t)nsl * lanes_c * un;
}

template <typename KV, int RT, bool GROUPED>
cudaError_t launch_rt(const float* q, const KV* k, uint64_t k_ld, const KV* v, uint64_t v_ld, const uint32_t* mask,
                      const AttnJob* jobs, const AttnRow* rows, uint64_t n_jobs, int d, int l, int dv, float scale,
                      int splits, int lc, size_t smem, void* out, int out_bf16, float* part_o, float* part_ms, cudaStream_t stream) {
  {
    const cudaError_t e = ensure_dynamic_smem((const void*)attention_rows_kernel<KV, RT, GROUPED>, 200 * 1024);
    if (e != cudaSuccess) return e;
  }
  launch_pdl(attention_rows_kernel<KV, RT, GROUPED>, dim3((unsigned)splits, (unsigned)n_jobs, 1), dim3(THREADS), smem, stream,
             q, k, k_ld, v, v_ld, mask, jobs, rows, d, l, dv, lc, scale, out, out_bf16, part_o, part_ms);
  return cudaGetLastError();
}

template <typename KV>
cudaError_t launch_kv(int rt, const float* q, const KV* k, uint64_t k_ld, const KV* v, uint64_t v_ld, const uint32_t* mask,
                      const AttnJob* jobs, const AttnRow* rows, uint64_t n_jobs, int d, int l, int dv, float scale,
                      int splits, int lc, size_t smem, void* out, int out_bf16, float* part_o, float* part_ms, cudaStream_t stream) {
  // the grouped scores want whole groups of eight 16-byte units a key (d a multiple of 64 for BF16, of 32 for F32);
  // B200TT_ATTN_SCORES=lane keeps the lane-a-key form for comparison
  static int lane_form = -1;
  if (lane_form < 0) { const char* e = getenv("B200TT_ATTN_SCORES"); lane_form = (e && e[0] == 'l') ? 1 : 0; }
  const bool grouped = !lane_form && (d / Unit<KV>::N) % 8 == 0;
#define GO(R) return grouped ? launch_rt<KV, R, true>(q, k, k_ld, v, v_ld, mask, jobs, rows, n_jobs, d, l, dv, scale, splits, lc, smem, out, out_bf16, part_o, part_ms, stream) \
                             : launch_rt<KV, R, false>(q, k, k_ld, v, v_ld, mask, jobs, rows, n_jobs, d, l, dv, scale, splits, lc, smem, out, out_bf16, part_o, part_ms, stream)
  if (rt <= 1) GO(1);
  if (rt <= 2) GO(2);
  if (rt <= 4) GO(4);
  GO(8);
#undef GO
}

}  // namespace

int attention_rows_tile(int rows) { return rows <= 1 ? 1 : (rows <= 2 ? 2 : (rows <= 4 ? 4 : 8)); }

// How a job's positions are split over blocks.  The kernel reads K and V once, so the step's time is the time of the
// longest chain of blocks an SM runs: with R blocks resident on the device at once (the kernel's blocks an SM by its row
// tile, fewer where a chunk's scores fill shared memory), s splits make ceil(jobs * s / R) rounds of blocks of l / s
// positions (plus a block's fixed part, taken as 96 positions).  The split count with the least rounds x length wins:
// 256 jobs of 4096 positions took 1,280 blocks in three rounds (114 us) where 1,024 in two take 99; 64 grouped jobs took
// 512 blocks in two rounds (62 us) where 384 in one take 44.  A chunk is at least `B200TT_ATTN_CHUNK` positions
// (default 256) and its scores stay within 64 KB of shared memory.  rt = the rows a job is built for (1, 2, 4, 8).
void attention_rows_plan(uint64_t n_jobs, int rt, int l, int sms, int* splits, int* lc) {
  if (sms <= 0) {
    int dev = 0;
    sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int lc_max = ((64 * 1024 / 4) / rt) / 32 * 32;
  static int chunk = 0;
  if (!chunk) { const char* e = getenv("B200TT_ATTN_CHUNK"); chunk = e ? atoi(e) : 256; if (chunk < 32) chunk = 256; }
  const uint64_t need = ((uint64_t)l + lc_max - 1) / lc_max;          // fewest splits: a chunk's scores fit
  uint64_t most = (uint64_t)(l / chunk > 1 ? l / chunk : 1);            // most splits: a chunk is not too short
  if (most < need) most = need;
  if (most > 64) most = 64;
  const int by_bounds = rt >= 8 ? 2 : (rt >= 4 ? 3 : 4);                // the kernel's launch bounds
  uint64_t best = need, best_cost = ~0ull;
  for (uint64_t s = need; s <= most; ++s) {
    int c = (int)((l + s - 1) / s);
    c = (c + 31) / 32 * 32;
    const uint64_t real = ((uint64_t)l + c - 1) / c;                    // the splits that chunk length makes
    const uint64_t smem = (uint64_t)rt * (128 + c) * 4 + 8 * 1024;       // about a block's shared memory (heads of 128 columns)
    uint64_t occ = (220ull * 1024) / smem;
    if (occ > (uint64_t)by_bounds) occ = by_bounds;
    if (occ < 1) occ = 1;
    const uint64_t resident = occ * (uint64_t)sms, blocks = n_jobs * real;
    const uint64_t cost = ((blocks + resident - 1) / resident) * (uint64_t)(c + 96);
    if (cost < best_cost) { best_cost = cost; best = s; }
  }
  int c = (int)((l + best - 1) / best);
  c = (c + 31) / 32 * 32;
  *lc = c;
  *splits = (l + c - 1) / c;
}

size_t attention_rows_scratch_floats(uint64_t n_jobs, int rt, int dv, int splits) {
  return splits > 1 ? (size_t)n_jobs * splits * rt * (dv + 2) : 0;
}

cudaError_t launch_attention_rows(const float* q, const void* k, uint64_t k_ld, const void* v, uint64_t v_ld, int kv_bf16,
                                  const uint32_t* mask, const AttnJob* jobs, const AttnRow* rows, uint64_t n_jobs, int rt,
                                  int d, int l, int dv, float scale, int splits, int lc, float* scratch, void* out,
                                  int out_bf16, int* launches, cudaStream_t stream) {
  *launches = 0;
  if (n_jobs == 0) return cudaSuccess;
  if (n_jobs > 65535 || rt > 8) return cudaErrorNotSupported;
  rt = attention_rows_tile(rt);
  const size_t smem = smem_floats(rt, d, lc, dv, kv_bf16) * sizeof(float);
  if (smem > 200 * 1024) return cudaErrorNotSupported;
  float* part_o = scratch;
  float* part_ms = scratch ? scratch + (size_t)n_jobs * splits * rt * dv : nullptr;
  cudaError_t e = kv_bf16
      ? launch_kv<uint16_t>(rt, q, (const uint16_t*)k, k_ld, (const uint16_t*)v, v_ld, mask, jobs, rows, n_jobs, d, l, dv, scale,
                            splits, lc, smem, out, out_bf16, part_o, part_ms, stream)
      : launch_kv<float>(rt, q, (const float*)k, k_ld, (const float*)v, v_ld, mask, jobs, rows, n_jobs, d, l, dv, scale,
                         splits, lc, smem, out, out_bf16, part_o, part_ms, stream);
  if (e != cudaSuccess) return e;
  *launches = 1;
  if (splits > 1) {
    launch_pdl(attention_join_kernel, dim3((unsigned)rt, (unsigned)n_jobs, 1), dim3(128), 0, stream, (const float*)part_o, (const float*)part_ms,
               jobs, rows, splits, rt, dv, out, out_bf16);
    e = cudaGetLastError();
    if (e == cudaSuccess) *launches = 2;
  }
  return e;
}

}  // namespace b200
