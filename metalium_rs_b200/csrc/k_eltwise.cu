// Element-wise kernels: every `Eltwise` kind of the reference
// (crates/tt-kernels/src/sfpu/ops.rs:24-251, crates/tt-kernels/src/kind.rs:12-26)
// over 32-bit words (F32 / I32 / Bool) or BF16 storage, with the reference's
// broadcast forms (crates/tt-kernels/src/tensor.rs:3799-3859).
//
// Memory-bound: the fast path moves 128-bit vectors, four per thread in flight,
// coalesced; the generic path handles blocks of buffers, BF16 and odd widths.
// Compiled with -fmad=false: every kind that the reference defines as separate
// roundings (MUL_ADD, HARD_SIGMOID, SILU_MUL ...) keeps them.
#include "eltwise_ev.cuh"
#include "kernels.h"
#include "pdl.cuh"

namespace b200 {
namespace {

// ---- fast path: contiguous 32-bit words, cols % 4 == 0 -------------------------
// BM: 0 no b, 1 b of a's shape, 2 b one row, 3 b one column.
template <uint32_t K, int BM>
__global__ void __launch_bounds__(256)
elt_vec4(const uint4* __restrict__ a, const uint32_t* __restrict__ b, uint4* __restrict__ out,
         uint64_t n4, uint32_t cols4, float s1, float s2, int* err, int streaming) {
  constexpr int U = 4;
  pdl_enter();
  const uint64_t base = (uint64_t)blockIdx.x * (256 * U) + threadIdx.x;
  uint4 va[U], vb[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const uint64_t i = base + (uint64_t)u * 256;
    if (i < n4) {
      va[u] = streaming ? __ldcs(a + i) : a[i];
      if constexpr (BM == 1) {
        vb[u] = streaming ? __ldcs(reinterpret_cast<const uint4*>(b) + i)
                          : reinterpret_cast<const uint4*>(b)[i];
      } else if constexpr (BM == 2) {
        vb[u] = __ldg(reinterpret_cast<const uint4*>(b) + (i % cols4));
      } else if constexpr (BM == 3) {
        uint32_t w = __ldg(b + (i / cols4));
        vb[u] = make_uint4(w, w, w, w);
      } else {
        vb[u] = make_uint4(0, 0, 0, 0);
      }
    }
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const uint64_t i = base + (uint64_t)u * 256;
    if (i < n4) {
      uint4 r;
      r.x = ev<K>(va[u].x, vb[u].x, 0u, s1, s2, err);
      r.y = ev<K>(va[u].y, vb[u].y, 0u, s1, s2, err);
      r.z = ev<K>(va[u].z, vb[u].z, 0u, s1, s2, err);
      r.w = ev<K>(va[u].w, vb[u].w, 0u, s1, s2, err);
      if (streaming) __stcs(out + i, r); else out[i] = r;
    }
  }
}

// ---- generic path ------------------------------------------------------------
__device__ __forceinline__ uint32_t load_word(const Mat& m, uint64_t r, uint64_t c) {
  const uint64_t rr = (m.rows == 1) ? 0 : (r % m.rows);
  const uint64_t cc = (m.cols == 1) ? 0 : (c % m.cols);
  const uint64_t off = rr * m.ld + cc;
  if (m.bf16) return (uint32_t)reinterpret_cast<const uint16_t*>(m.p)[off] << 16;
  return reinterpret_cast<const uint32_t*>(m.p)[off];
}

template <uint32_t K>
__global__ void __launch_bounds__(256) elt_generic(EltwiseArgs g) {
  const uint64_t n = g.rows * g.cols;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    uint64_t r, c;
    if (n <= 0xffffffffull) {
      r = (uint32_t)i / (uint32_t)g.cols;
      c = (uint32_t)i - (uint32_t)r * (uint32_t)g.cols;
    } else {
      r = i / g.cols;
      c = i - r * g.cols;
    }
    const uint32_t ua = load_word(g.a, r, c);
    const uint32_t ub = g.b.p ? load_word(g.b, r, c) : 0u;
    const uint32_t uc = g.c.p ? load_word(g.c, r, c) : 0u;
    const uint32_t res = ev<K>(ua, ub, uc, g.s1, g.s2, g.err);
    const uint64_t o = r * g.out_ld + c;
    if (g.out_bf16) reinterpret_cast<uint16_t*>(g.out)[o] = f32_to_bf16_bits(res);
    else reinterpret_cast<uint32_t*>(g.out)[o] = res;
  }
}

// ---- block / BF16 fast path: eight consecutive columns a thread ---------------------
// Operands may be blocks of wider buffers (ld > cols), F32 or BF16, and b may be a's shape, one
// row, whole rows repeated, or one column.  Needs cols % 8 == 0 and 16-byte aligned rows.
struct Word8 { uint32_t w[8]; };

__device__ __forceinline__ Word8 load8(const Mat& m, uint64_t r, uint32_t c) {
  Word8 o;
  // the division only for a repeated block, and in 32 bits when the numbers fit
  const uint64_t rr = (m.rows == 1) ? 0 : (r < m.rows ? r : (((r | m.rows) >> 32) == 0 ? (uint64_t)((uint32_t)r % (uint32_t)m.rows) : r % m.rows));
  if (m.cols == 1) {
    const uint32_t v = m.bf16 ? (uint32_t)reinterpret_cast<const uint16_t*>(m.p)[rr * m.ld] << 16
                              : reinterpret_cast<const uint32_t*>(m.p)[rr * m.ld];
#pragma unroll
    for (int i = 0; i < 8; ++i) o.w[i] = v;
    return o;
  }
  const uint64_t off = rr * m.ld + c;
  if (m.bf16) {
    const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(m.p) + off);
    o.w[0] = v.x << 16; o.w[1] = v.x & 0xffff0000u; o.w[2] = v.y << 16; o.w[3] = v.y & 0xffff0000u;
    o.w[4] = v.z << 16; o.w[5] = v.z & 0xffff0000u; o.w[6] = v.w << 16; o.w[7] = v.w & 0xffff0000u;
  } else {
    const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const uint32_t*>(m.p) + off);
    const uint4 v0 = p[0], v1 = p[1];
    o.w[0] = v0.x; o.w[1] = v0.y; o.w[2] = v0.z; o.w[3] = v0.w;
    o.w[4] = v1.x; o.w[5] = v1.y; o.w[6] = v1.z; o.w[7] = v1.w;
  }
  return o;
}

__device__ __forceinline__ void store8(void* out, uint64_t off, int bf16, const Word8& v) {
  if (bf16) {
    uint4 o;
    o.x = (uint32_t)f32_to_bf16_bits(v.w[0]) | ((uint32_t)f32_to_bf16_bits(v.w[1]) << 16);
    o.y = (uint32_t)f32_to_bf16_bits(v.w[2]) | ((uint32_t)f32_to_bf16_bits(v.w[3]) << 16);
    o.z = (uint32_t)f32_to_bf16_bits(v.w[4]) | ((uint32_t)f32_to_bf16_bits(v.w[5]) << 16);
    o.w = (uint32_t)f32_to_bf16_bits(v.w[6]) | ((uint32_t)f32_to_bf16_bits(v.w[7]) << 16);
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out) + off) = o;
  } else {
    uint4* p = reinterpret_cast<uint4*>(reinterpret_cast<uint32_t*>(out) + off);
    p[0] = make_uint4(v.w[0], v.w[1], v.w[2], v.w[3]);
    p[1] = make_uint4(v.w[4], v.w[5], v.w[6], v.w[7]);
  }
}

// Eight columns a thread; two such pieces in flight a thread.  I is the index type: 32-bit
// arithmetic (no 64-bit division) whenever the piece count fits.
template <uint32_t K, typename I>
__global__ void __launch_bounds__(256) elt_rows8(EltwiseArgs g) {
  pdl_enter();
  const I c8 = (I)(g.cols / 8);
  const I n8 = (I)(g.rows * (g.cols / 8));
  const I stride = (I)gridDim.x * blockDim.x;
  for (I i = (I)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += 2 * stride) {
    const I i2 = i + stride;
    const bool two = i2 < n8 && i2 > i;   // (i2 > i: no wrap of a 32-bit index)
    const I r0 = i / c8, r1 = two ? i2 / c8 : r0;
    const uint32_t c0 = (uint32_t)(i - r0 * c8) * 8, c1 = two ? (uint32_t)(i2 - r1 * c8) * 8 : c0;
    Word8 a0 = load8(g.a, r0, c0), a1, b0, b1, cc0, cc1, o;
    if (two) a1 = load8(g.a, r1, c1);
    if (g.b.p) { b0 = load8(g.b, r0, c0); if (two) b1 = load8(g.b, r1, c1); }
    if (g.c.p) { cc0 = load8(g.c, r0, c0); if (two) cc1 = load8(g.c, r1, c1); }
#pragma unroll
    for (int j = 0; j < 8; ++j) o.w[j] = ev<K>(a0.w[j], g.b.p ? b0.w[j] : 0u, g.c.p ? cc0.w[j] : 0u, g.s1, g.s2, g.err);
    store8(g.out, (uint64_t)r0 * g.out_ld + c0, g.out_bf16, o);
    if (two) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o.w[j] = ev<K>(a1.w[j], g.b.p ? b1.w[j] : 0u, g.c.p ? cc1.w[j] : 0u, g.s1, g.s2, g.err);
      store8(g.out, (uint64_t)r1 * g.out_ld + c1, g.out_bf16, o);
    }
  }
}

inline bool mat_ok8(const Mat& m, uint64_t rows, uint64_t cols) {
  if (!m.p) return true;
  const uintptr_t a = reinterpret_cast<uintptr_t>(m.p);
  if (m.cols == 1) return m.rows == rows || m.rows == 1;
  const uint64_t eb = m.bf16 ? 2 : 4;
  return m.cols == cols && (a % 16 == 0) && ((m.ld * eb) % 16 == 0) && (m.rows == rows || m.rows == 1 || rows % m.rows == 0);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <uint32_t K>
cudaError_t launch_kind(const EltwiseArgs& g, cudaStream_t stream) {
  const uint64_t n = g.rows * g.cols;
  if (n == 0) return cudaSuccess;
  // Which broadcast form b takes, if the fast path can serve it.
  int bm = -1;
  const bool plain = !g.a.bf16 && !g.out_bf16 && !g.c.p && g.a.ld == g.cols && g.out_ld == g.cols &&
                     g.a.rows == g.rows && g.a.cols == g.cols && (g.cols % 4 == 0) &&
                     aligned16(g.a.p) && aligned16(g.out) && (g.cols / 4) <= 0xffffffffull;
  if (plain) {
    if (!g.b.p) bm = 0;
    else if (!g.b.bf16 && g.b.rows == g.rows && g.b.cols == g.cols && g.b.ld == g.cols && aligned16(g.b.p)) bm = 1;
    else if (!g.b.bf16 && g.b.rows == 1 && g.b.cols == g.cols && aligned16(g.b.p)) bm = 2;
    else if (!g.b.bf16 && g.b.cols == 1 && g.b.rows == g.rows && g.b.ld == 1) bm = 3;
  }
  if (bm >= 0) {
    const uint64_t n4 = n / 4;
    const uint32_t cols4 = (uint32_t)(g.cols / 4);
    const unsigned grid = (unsigned)((n4 + 1023) / 1024);
    const int streaming = n * 4 > (64ull << 20);
    auto a = reinterpret_cast<const uint4*>(g.a.p);
    auto b = reinterpret_cast<const uint32_t*>(g.b.p);
    auto o = reinterpret_cast<uint4*>(g.out);
    switch (bm) {
      case 0: launch_pdl(elt_vec4<K, 0>, dim3(grid), dim3(256), 0, stream, a, b, o, n4, cols4, g.s1, g.s2, g.err, streaming); break;
      case 1: launch_pdl(elt_vec4<K, 1>, dim3(grid), dim3(256), 0, stream, a, b, o, n4, cols4, g.s1, g.s2, g.err, streaming); break;
      case 2: launch_pdl(elt_vec4<K, 2>, dim3(grid), dim3(256), 0, stream, a, b, o, n4, cols4, g.s1, g.s2, g.err, streaming); break;
      default: launch_pdl(elt_vec4<K, 3>, dim3(grid), dim3(256), 0, stream, a, b, o, n4, cols4, g.s1, g.s2, g.err, streaming); break;
    }
    return cudaGetLastError();
  }
  if (g.cols % 8 == 0 && g.a.rows == g.rows && mat_ok8(g.a, g.rows, g.cols) && g.a.cols == g.cols &&
      mat_ok8(g.b, g.rows, g.cols) && mat_ok8(g.c, g.rows, g.cols) && (!g.c.p || g.c.cols == g.cols) &&
      (reinterpret_cast<uintptr_t>(g.out) % 16 == 0) && ((g.out_ld * (g.out_bf16 ? 2 : 4)) % 16 == 0) && g.cols / 8 <= 0xffffffffull) {
    uint64_t blocks = (n / 16 + 255) / 256;
    if (blocks == 0) blocks = 1;
    if (blocks > 148ull * 32) blocks = 148ull * 32;
    if (n / 8 + 2ull * blocks * 256 < 0xffffffffull) launch_pdl(elt_rows8<K, uint32_t>, dim3((unsigned)blocks), dim3(256), 0, stream, g);
    else launch_pdl(elt_rows8<K, uint64_t>, dim3((unsigned)blocks), dim3(256), 0, stream, g);
    return cudaGetLastError();
  }
  uint64_t blocks = (n + 255) / 256;
  if (blocks > 148ull * 32) blocks = 148ull * 32;
  elt_generic<K><<<(unsigned)blocks, 256, 0, stream>>>(g);
  return cudaGetLastError();
}

// ---- RoPE -------------------------------------------------------------------
// out = fl(fl(x cos) + fl(swap(x) sin)): the product, the product and the sum
// (crates/tt-kernels/src/tensor.rs:5545-5552).
__global__ void __launch_bounds__(256)
rope_kernel(Mat x, Mat cs, Mat sn, uint64_t head, void* out, uint64_t out_ld, int out_bf16,
            uint64_t rows, uint64_t cols) {
  const uint64_t n = rows * cols;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t half = head / 2;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const uint64_t r = i / cols, c = i - r * cols;
    const uint64_t h = c / head, j = c - h * head;
    const uint64_t cswap = h * head + (j < half ? j + half : j - half);
    const float xv = __uint_as_float(load_word(x, r, c));
    const float xs = __uint_as_float(load_word(x, r, cswap));
    const float co = __uint_as_float(load_word(cs, r, cs.cols == head ? j : c));
    const float si = __uint_as_float(load_word(sn, r, sn.cols == head ? j : c));
    const float p1 = xv * co;
    const float p2 = xs * si;
    const uint32_t res = __float_as_uint(p1 + p2);
    const uint64_t o = r * out_ld + c;
    if (out_bf16) reinterpret_cast<uint16_t*>(out)[o] = f32_to_bf16_bits(res);
    else reinterpret_cast<uint32_t*>(out)[o] = res;
  }
}

// Eight consecutive columns a thread (they lie in one half of one head when head/2 % 8 == 0).
__global__ void __launch_bounds__(256)
rope_kernel8(Mat x, Mat cs, Mat sn, uint32_t head, void* out, uint64_t out_ld, int out_bf16,
             uint64_t rows, uint32_t cols) {
  pdl_enter();
  const uint32_t c8 = cols / 8, half = head / 2;
  const uint64_t n8 = rows * c8;
  const bool small = n8 <= 0xffffffffull;     // 32-bit divisions
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t r = small ? (uint64_t)((uint32_t)i / c8) : i / c8;
    const uint32_t c = (uint32_t)(i - r * c8) * 8;
    const uint32_t h = c / head, j = c - h * head;
    const uint32_t cswap = h * head + (j < half ? j + half : j - half);
    const Word8 xv = load8(x, r, c), xs = load8(x, r, cswap);
    const Word8 co = load8(cs, r, cs.cols == head ? j : c), si = load8(sn, r, sn.cols == head ? j : c);
    Word8 o;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float p1 = __uint_as_float(xv.w[q]) * __uint_as_float(co.w[q]);
      const float p2 = __uint_as_float(xs.w[q]) * __uint_as_float(si.w[q]);
      o.w[q] = __float_as_uint(p1 + p2);
    }
    store8(out, r * out_ld + c, out_bf16, o);
  }
}

// RoPE on heads of 64 columns of a BF16 matrix with F32 tables of 64 columns (a Llama layer's query and key heads,
// crates/tt-models/src/rope.rs:19-60): a warp a row.  A lane takes four consecutive columns j of the low half of a head and
// the four at j + 32, of one head in four, so a warp's load is four heads' two 64-byte halves; the row's table entries for
// those columns wait in registers for all of the row's heads (the general kernel fetches them again for every eight
// outputs: a 4096 x 768 block moved 38 MB through the load pipe for 12.6 MB of heads).  The steps are the general
// kernel's: fl(fl(x cos) + fl(x' sin)) with x' the element 32 columns across, rounded once to BF16.
__device__ __forceinline__ uint2 rope_bf16x4(float t0, float t1, float t2, float t3) {
  // `f32_to_bf16_bits` of four values: the hardware's conversion is that rounding for every number that is zero or at
  // least 2^-126 in magnitude; the others, and NaNs, take the integer rule
  const uint32_t a0 = __float_as_uint(t0) & 0x7fffffffu, a1 = __float_as_uint(t1) & 0x7fffffffu;
  const uint32_t a2 = __float_as_uint(t2) & 0x7fffffffu, a3 = __float_as_uint(t3) & 0x7fffffffu;
  const uint32_t lo = min(min(a0 - 1u, a1 - 1u), min(a2 - 1u, a3 - 1u)), hi = max(max(a0, a1), max(a2, a3));
  uint2 o;
  if (lo < 0x007fffffu || hi > 0x7f800000u) {
    o.x = (uint32_t)f32_to_bf16_bits(__float_as_uint(t0)) | ((uint32_t)f32_to_bf16_bits(__float_as_uint(t1)) << 16);
    o.y = (uint32_t)f32_to_bf16_bits(__float_as_uint(t2)) | ((uint32_t)f32_to_bf16_bits(__float_as_uint(t3)) << 16);
  } else {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o.x) : "f"(t1), "f"(t0));
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o.y) : "f"(t3), "f"(t2));
  }
  return o;
}
__global__ void __launch_bounds__(256)
rope_rows64_kernel(const uint16_t* __restrict__ x, uint64_t x_ld, const float* __restrict__ cs, uint64_t cs_ld,
                   const float* __restrict__ sn, uint64_t sn_ld, uint64_t table_rows, uint16_t* __restrict__ out, uint64_t out_ld,
                   uint64_t rows, uint32_t heads) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const uint32_t j0 = (lane & 7) * 4, hg = lane >> 3;
  const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  for (uint64_t r = warp; r < rows; r += nwarps) {
    const uint64_t tr = r < table_rows ? r : r % table_rows;
    const float4 cl = *reinterpret_cast<const float4*>(cs + tr * cs_ld + j0), ch = *reinterpret_cast<const float4*>(cs + tr * cs_ld + 32 + j0);
    const float4 sl = *reinterpret_cast<const float4*>(sn + tr * sn_ld + j0), sh = *reinterpret_cast<const float4*>(sn + tr * sn_ld + 32 + j0);
    const uint16_t* xr = x + r * x_ld;
    uint16_t* orow = out + r * out_ld;
    for (uint32_t h = hg; h < heads; h += 4) {
      const uint2 lo = *reinterpret_cast<const uint2*>(xr + h * 64 + j0), hi = *reinterpret_cast<const uint2*>(xr + h * 64 + 32 + j0);
      const float a0 = __uint_as_float(lo.x << 16), a1 = __uint_as_float(lo.x & 0xffff0000u);
      const float a2 = __uint_as_float(lo.y << 16), a3 = __uint_as_float(lo.y & 0xffff0000u);
      const float b0 = __uint_as_float(hi.x << 16), b1 = __uint_as_float(hi.x & 0xffff0000u);
      const float b2 = __uint_as_float(hi.y << 16), b3 = __uint_as_float(hi.y & 0xffff0000u);
      *reinterpret_cast<uint2*>(orow + h * 64 + j0) =
          rope_bf16x4(__fadd_rn(__fmul_rn(a0, cl.x), __fmul_rn(b0, sl.x)), __fadd_rn(__fmul_rn(a1, cl.y), __fmul_rn(b1, sl.y)),
                      __fadd_rn(__fmul_rn(a2, cl.z), __fmul_rn(b2, sl.z)), __fadd_rn(__fmul_rn(a3, cl.w), __fmul_rn(b3, sl.w)));
      *reinterpret_cast<uint2*>(orow + h * 64 + 32 + j0) =
          rope_bf16x4(__fadd_rn(__fmul_rn(b0, ch.x), __fmul_rn(a0, sh.x)), __fadd_rn(__fmul_rn(b1, ch.y), __fmul_rn(a1, sh.y)),
                      __fadd_rn(__fmul_rn(b2, ch.z), __fmul_rn(a2, sh.z)), __fadd_rn(__fmul_rn(b3, ch.w), __fmul_rn(a3, sh.w)));
    }
  }
}

// ---- casts ---------------------------------------------------------------------
__global__ void __launch_bounds__(256)
cast_to_bf16(const uint32_t* __restrict__ in, uint16_t* __restrict__ out, uint64_t n) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x * 4;
  for (uint64_t i = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 3 < n && ((reinterpret_cast<uintptr_t>(in) & 15) == 0) && ((reinterpret_cast<uintptr_t>(out) & 7) == 0)) {
      const uint4 v = *reinterpret_cast<const uint4*>(in + i);
      uint2 o;
      o.x = (uint32_t)f32_to_bf16_bits(v.x) | ((uint32_t)f32_to_bf16_bits(v.y) << 16);
      o.y = (uint32_t)f32_to_bf16_bits(v.z) | ((uint32_t)f32_to_bf16_bits(v.w) << 16);
      *reinterpret_cast<uint2*>(out + i) = o;
    } else {
      for (uint64_t j = i; j < n && j < i + 4; ++j) out[j] = f32_to_bf16_bits(in[j]);
    }
  }
}
__global__ void __launch_bounds__(256)
cast_from_bf16(const uint16_t* __restrict__ in, uint32_t* __restrict__ out, uint64_t n) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = (uint32_t)in[i] << 16;
}

}  // namespace

bool eltwise_kind_known(uint32_t k) { return kind::arity(k) != 0; }

cudaError_t launch_eltwise(const EltwiseArgs& g, cudaStream_t stream) {
  switch (g.kind) {
#define B200_CASE(name, value, ar) case value: return launch_kind<value>(g, stream);
    B200_KINDS(B200_CASE)
#undef B200_CASE
    default: return cudaErrorNotSupported;
  }
}

cudaError_t launch_rope(const Mat& x, const Mat& cs, const Mat& sn, uint64_t head, void* out,
                        uint64_t out_ld, int out_bf16, uint64_t rows, uint64_t cols,
                        cudaStream_t stream) {
  const uint64_t n = rows * cols;
  if (n == 0) return cudaSuccess;
  auto ok8 = [&](const Mat& m, uint64_t want_cols) {
    const uint64_t eb = m.bf16 ? 2 : 4;
    return m.cols == want_cols && reinterpret_cast<uintptr_t>(m.p) % 16 == 0 && (m.ld * eb) % 16 == 0;
  };
  // heads of 64 columns, BF16 in and out, F32 tables a head wide: a warp a row, the row's table entries kept for all its heads
  static int rows_form = -1;
  if (rows_form < 0) { const char* e = getenv("B200TT_ROPE_ROWS"); rows_form = (e && e[0] == '0') ? 0 : 1; }   // a development switch
  if (rows_form && head == 64 && x.bf16 && out_bf16 && !cs.bf16 && !sn.bf16 && cs.cols == 64 && sn.cols == 64 && cs.rows == sn.rows && cs.rows > 0 &&
      cols % 64 == 0 && cols / 64 < (1ull << 31) && x.cols == cols && x.rows == rows && x.ld % 4 == 0 && out_ld % 4 == 0 && cs.ld % 4 == 0 &&
      sn.ld % 4 == 0 && reinterpret_cast<uintptr_t>(x.p) % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 8 == 0 &&
      reinterpret_cast<uintptr_t>(cs.p) % 16 == 0 && reinterpret_cast<uintptr_t>(sn.p) % 16 == 0) {
    uint64_t blocks = (rows + 7) / 8;
    if (blocks > 148ull * 32) blocks = 148ull * 32;
    launch_pdl(rope_rows64_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, (const uint16_t*)x.p, x.ld, (const float*)cs.p, cs.ld,
               (const float*)sn.p, sn.ld, cs.rows, (uint16_t*)out, out_ld, rows, (uint32_t)(cols / 64));
    return cudaGetLastError();
  }
  if ((head / 2) % 8 == 0 && cols <= 0xffffffffull && ok8(x, cols) && (ok8(cs, head) || ok8(cs, cols)) &&
      (ok8(sn, head) || ok8(sn, cols)) && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
      (out_ld * (out_bf16 ? 2 : 4)) % 16 == 0) {
    uint64_t b8 = (n / 8 + 255) / 256;
    if (b8 > 148ull * 32) b8 = 148ull * 32;
    launch_pdl(rope_kernel8, dim3((unsigned)b8), dim3(256), 0, stream, x, cs, sn, (uint32_t)head, out, out_ld, out_bf16, rows, (uint32_t)cols);
    return cudaGetLastError();
  }
  uint64_t blocks = (n + 255) / 256;
  if (blocks > 148ull * 32) blocks = 148ull * 32;
  rope_kernel<<<(unsigned)blocks, 256, 0, stream>>>(x, cs, sn, head, out, out_ld, out_bf16, rows, cols);
  return cudaGetLastError();
}

cudaError_t launch_cast(const void* in, void* out, uint64_t n, int to_bf16, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  uint64_t blocks = to_bf16 ? (n / 4 + 255) / 256 + 1 : (n + 255) / 256;
  if (blocks > 148ull * 64) blocks = 148ull * 64;
  if (to_bf16)
    cast_to_bf16<<<(unsigned)blocks, 256, 0, stream>>>((const uint32_t*)in, (uint16_t*)out, n);
  else
    cast_from_bf16<<<(unsigned)blocks, 256, 0, stream>>>((const uint16_t*)in, (uint32_t*)out, n);
  return cudaGetLastError();
}

}  // namespace b200
