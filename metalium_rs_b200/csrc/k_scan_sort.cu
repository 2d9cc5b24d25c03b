// Inclusive scans down the rows of a matrix and the sort of a planes matrix.
//
// Scan: `Engine::scan` (crates/burn-tt/src/server.rs:414; the op list and its scalar model
// crates/tt-kernels/src/sfpu/scan.rs:19-41, 196-231).  Every column is scanned from its first row to its
// last, starting from the op's identity: out[r] = step(out[r-1], x[r]).  F32 `Sum` and `Prod` are left
// folds in row order (the sum starts from +0.0, the product from 1.0), so their bits are those of a
// sequential loop and the rows of a column cannot be split; the selecting ops (raw total-order Min/Max,
// the NaN-taking MinNan/MaxNan where the earlier element wins a tie and a later NaN replaces an earlier
// one) and the wrapping I32 ops are associative over row segments, so few-column inputs are cut into row
// chunks: fold each chunk, fold the chunk totals before it, then scan the chunk from that prefix.
//
// Sort: `Engine::sort_planes` (server.rs:758; crates/tt-kernels/src/sfpu/sort.rs:1-66, 196-228).  The
// input holds problem q's axis position e at the planes coordinate of sort.rs:198: a 32x32 tile holds 32
// problems by 32 positions, one tile row being eight problems (those with the same q % 32 / 8) by four
// positions.  The order is the total order on (key, original index): `total_cmp` for F32, two's
// complement for I32, reversed keys for a descending sort with ties still in ascending index.  Positions
// at or past n are sentinels that sort last and are never returned as one of the first n.  A block takes
// the eight problems of one tile row pattern, reads whole 128-byte rows into shared memory, runs a
// bitonic network over (ordered key, index) words, which never tie, and writes keys (and indices) back
// in the same layout.
#include <cstdint>
#include <cuda_runtime.h>

#include "kernels.h"
#include "pdl.cuh"

namespace b200 {
namespace {

enum { S_SUM, S_PROD, S_MIN, S_MAX, S_MINNAN, S_MAXNAN, S_ISUM, S_IPROD, S_IMIN, S_IMAX };

__device__ __forceinline__ int32_t total_key(uint32_t x) { return (int32_t)(x ^ (((uint32_t)((int32_t)x >> 31)) >> 1)); }

template <int OP>
__device__ __forceinline__ uint32_t scan_identity() {
  switch (OP) {
    case S_SUM: case S_ISUM: return 0u;
    case S_PROD: return 0x3f800000u;
    case S_IPROD: return 1u;
    case S_MIN: return 0x7fffffffu;
    case S_MAX: return 0xffffffffu;
    case S_MINNAN: return 0x7f800000u;
    case S_MAXNAN: return 0xff800000u;
    case S_IMIN: return 0x7fffffffu;
    default: return 0x80000000u;
  }
}

template <int OP>
__device__ __forceinline__ uint32_t scan_step(uint32_t acc, uint32_t x) {
  switch (OP) {
    case S_SUM: return __float_as_uint(__fadd_rn(__uint_as_float(x), __uint_as_float(acc)));
    case S_PROD: return __float_as_uint(__fmul_rn(__uint_as_float(acc), __uint_as_float(x)));
    case S_MIN: return total_key(x) < total_key(acc) ? x : acc;
    case S_MAX: return total_key(x) > total_key(acc) ? x : acc;
    case S_MINNAN: { const float v = __uint_as_float(x), a = __uint_as_float(acc); return (v != v || v < a) ? x : acc; }
    case S_MAXNAN: { const float v = __uint_as_float(x), a = __uint_as_float(acc); return (v != v || v > a) ? x : acc; }
    case S_ISUM: return acc + x;
    case S_IPROD: return acc * x;
    case S_IMIN: return (int32_t)x < (int32_t)acc ? x : acc;
    default: return (int32_t)x > (int32_t)acc ? x : acc;
  }
}

// A thread a column, rows [r0, r1) of it; `carry` (chunk totals, [chunks][cols]) gives the prefix of the
// chunks before this one when MODE == 2; MODE == 1 only folds the chunk and stores its total.
template <int OP, int MODE>
__global__ void __launch_bounds__(128)
scan_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, uint64_t rows, uint64_t cols, uint64_t chunk_rows,
            uint32_t* __restrict__ carry) {
  pdl_enter();
  const uint64_t c = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const uint64_t chunk = blockIdx.y, r0 = chunk * chunk_rows;
  const uint64_t r1 = r0 + chunk_rows < rows ? r0 + chunk_rows : rows;
  uint32_t acc = scan_identity<OP>();
  if (MODE == 2)
    for (uint64_t k = 0; k < chunk; ++k) acc = scan_step<OP>(acc, carry[k * cols + c]);
  const uint32_t* p = in + r0 * cols + c;
  uint32_t* q = out + r0 * cols + c;
  uint64_t r = r0;
  for (; r + 8 <= r1; r += 8) {                 // eight independent loads in flight a thread
    uint32_t x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) x[u] = __ldg(p + (uint64_t)u * cols);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      acc = scan_step<OP>(acc, x[u]);
      if (MODE != 1) q[(uint64_t)u * cols] = acc;
    }
    p += 8 * cols; q += 8 * cols;
  }
  for (; r < r1; ++r) {
    acc = scan_step<OP>(acc, __ldg(p));
    if (MODE != 1) *q = acc;
    p += cols; q += cols;
  }
  if (MODE == 1) carry[chunk * cols + c] = acc;
}

// The scanning form for whole launches: a block owns a strip of 32 columns (one 128-byte line a row) and walks
// its rows in tiles kept in a ring of four shared-memory slots.  Its warps are specialised: warp 0 scans (a lane
// a column; the serial chain is an add or a select a row with its operand already on chip) and three mover
// warps, while tile t is scanned, store tile t - 1 and bring tile t + 2 in with cp.async -- sixteen bytes a
// lane, so one instruction moves four rows of the strip, the addresses advanced by additions only.  One barrier
// a tile.  What the forms before this one measured on a [8192, 8192] row-order sum: a thread a column over
// global memory, 1.3 TB/s of bytes moved (only what a thread has in flight is ahead of the chain); all warps
// fetching, scanning and storing in turn, four bytes a lane, 3.1 TB/s (instruction latencies of the one warp
// that does everything); this form, 4.9 TB/s.
constexpr int SCAN_SLOTS = 4;
constexpr int SCAN_MOVERS = 3;           // mover warps a block
constexpr int SCAN_THREADS = 32 * (1 + SCAN_MOVERS);

__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// VEC: the strip's rows are whole 16-byte pieces at 16-byte addresses (cols % 4 == 0, aligned bases).
template <int OP, int MODE, bool VEC>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_tiled_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, uint64_t rows, uint64_t cols, uint64_t chunk_rows,
                  int tile_rows, const uint32_t* __restrict__ carry) {
  extern __shared__ __align__(16) uint32_t tiles[];        // SCAN_SLOTS tiles of [tile_rows][32]
  pdl_enter();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint64_t c0 = (uint64_t)blockIdx.x * 32;
  const uint64_t chunk = blockIdx.y, r0 = chunk * chunk_rows;
  const uint64_t r1 = r0 + chunk_rows < rows ? r0 + chunk_rows : rows;
  const int tile_words = tile_rows * 32;
  const int n_tiles = (int)((r1 - r0 + tile_rows - 1) / tile_rows);
  auto rows_of = [&](int t) {
    const uint64_t row0 = r0 + (uint64_t)t * tile_rows;
    return (int)(r1 - row0 < (uint64_t)tile_rows ? r1 - row0 : tile_rows);
  };
  if (warp == 0) {
    // ---- the scanning warp: tile t between the barriers of iteration t
    const bool live = c0 + lane < cols;
    uint32_t acc = scan_identity<OP>();
    if (MODE == 2 && live)
      for (uint64_t k = 0; k < chunk; ++k) acc = scan_step<OP>(acc, carry[k * cols + c0 + lane]);
    __syncthreads();                                       // tile 0 has landed
    for (int t = 0; t <= n_tiles; ++t) {
      if (t < n_tiles && live) {
        uint32_t* col = tiles + (t & (SCAN_SLOTS - 1)) * tile_words + lane;
        const int n = rows_of(t);
        int r = 0;
        if (n >= 8) {                                      // eight rows read ahead of the eight being folded
          uint32_t x[8], y[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) x[u] = col[u * 32];
          for (; r + 16 <= n; r += 8) {
#pragma unroll
            for (int u = 0; u < 8; ++u) y[u] = col[(8 + u) * 32];
#pragma unroll
            for (int u = 0; u < 8; ++u) { acc = scan_step<OP>(acc, x[u]); col[u * 32] = acc; }
#pragma unroll
            for (int u = 0; u < 8; ++u) x[u] = y[u];
            col += 8 * 32;
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) { acc = scan_step<OP>(acc, x[u]); col[u * 32] = acc; }
          col += 8 * 32;
          r += 8;
        }
        for (; r < n; ++r) { acc = scan_step<OP>(acc, col[0]); col[0] = acc; col += 32; }
      }
      __syncthreads();
    }
  } else {
    // ---- a mover warp: in iteration t it stores tile t - 1, then fetches tile t + 2 into the slot tile t - 2 left
    // (stored in iteration t - 1, before that iteration's barrier), and waits until tile t + 1 has landed
    const int mw = warp - 1;
    // VEC: a lane moves piece `pc` (four columns) of row 4 i + `sub`; else a lane a column of row i
    const int sub = lane >> 3, pc = (lane & 7) * 4;
    const bool has = VEC ? c0 + pc < cols : c0 + lane < cols;
    auto fetch = [&](int t) {
      if (t < n_tiles && has) {
        const uint64_t row0 = r0 + (uint64_t)t * tile_rows;
        const int n = rows_of(t);
        uint32_t* buf = tiles + (t & (SCAN_SLOTS - 1)) * tile_words;
        if (VEC) {
          const uint32_t* src = in + (row0 + 4 * mw + sub) * cols + c0 + pc;
          uint32_t* dst = buf + (4 * mw + sub) * 32 + pc;
          for (int r = 4 * mw + sub; r < n; r += 4 * SCAN_MOVERS) {
            cp_async16(dst, src);
            src += 4 * SCAN_MOVERS * cols; dst += 4 * SCAN_MOVERS * 32;
          }
        } else {
          const uint32_t* src = in + (row0 + mw) * cols + c0 + lane;
          uint32_t* dst = buf + mw * 32 + lane;
          for (int r = mw; r < n; r += SCAN_MOVERS) { cp_async4(dst, src); src += SCAN_MOVERS * cols; dst += SCAN_MOVERS * 32; }
        }
      }
      cp_async_commit();                                   // a group a tile slot, empty past the last tile
    };
    fetch(0); fetch(1);
    cp_async_wait<1>();
    __syncthreads();                                       // tile 0 has landed
    for (int t = 0; t <= n_tiles; ++t) {
      if (t >= 1 && has) {
        const uint64_t row0 = r0 + (uint64_t)(t - 1) * tile_rows;
        const int n = rows_of(t - 1);
        const uint32_t* buf = tiles + ((t - 1) & (SCAN_SLOTS - 1)) * tile_words;
        if (VEC) {
          uint32_t* dst = out + (row0 + 4 * mw + sub) * cols + c0 + pc;
          const uint32_t* src = buf + (4 * mw + sub) * 32 + pc;
          for (int r = 4 * mw + sub; r < n; r += 4 * SCAN_MOVERS) {
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
            dst += 4 * SCAN_MOVERS * cols; src += 4 * SCAN_MOVERS * 32;
          }
        } else {
          uint32_t* dst = out + (row0 + mw) * cols + c0 + lane;
          const uint32_t* src = buf + mw * 32 + lane;
          for (int r = mw; r < n; r += SCAN_MOVERS) { *dst = *src; dst += SCAN_MOVERS * cols; src += SCAN_MOVERS * 32; }
        }
      }
      fetch(t + 2);
      cp_async_wait<1>();                                  // all but the newest group: tile t + 1 is in
      __syncthreads();
    }
  }
}

template <int OP>
cudaError_t scan_go(const uint32_t* in, uint32_t* out, uint64_t rows, uint64_t cols, uint64_t chunks, uint64_t chunk_rows,
                    uint32_t* carry, cudaStream_t s) {
  const dim3 block(128);
  const unsigned gx = (unsigned)((cols + 127) / 128);
  const unsigned strips = (unsigned)((cols + 31) / 32);
  // every block resident at once: the tiles are as deep as the shared memory of an SM, shared by the blocks that
  // land on it, allows (few blocks: deep tiles, so that what a block has in flight hides the latency)
  const uint64_t per_sm = ((uint64_t)strips * chunks + 147) / 148;
  int tile_rows = 256;
  while (tile_rows > 16 && per_sm * SCAN_SLOTS * tile_rows * 128 > 200 * 1024) tile_rows >>= 1;
  const size_t smem = (size_t)SCAN_SLOTS * tile_rows * 128;
  const bool vec = cols % 4 == 0 && reinterpret_cast<uintptr_t>(in) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
  {
    const void* fn = chunks > 1 ? (vec ? (const void*)scan_tiled_kernel<OP, 2, true> : (const void*)scan_tiled_kernel<OP, 2, false>)
                                : (vec ? (const void*)scan_tiled_kernel<OP, 0, true> : (const void*)scan_tiled_kernel<OP, 0, false>);
    const cudaError_t e = ensure_dynamic_smem(fn, smem);
    if (e != cudaSuccess) return e;
  }
  if (chunks <= 1) {
    if (vec) launch_pdl(scan_tiled_kernel<OP, 0, true>, dim3(strips, 1), dim3(SCAN_THREADS), smem, s, in, out, rows, cols, rows, tile_rows, (const uint32_t*)nullptr);
    else launch_pdl(scan_tiled_kernel<OP, 0, false>, dim3(strips, 1), dim3(SCAN_THREADS), smem, s, in, out, rows, cols, rows, tile_rows, (const uint32_t*)nullptr);
  } else {
    launch_pdl(scan_kernel<OP, 1>, dim3(gx, (unsigned)chunks), block, 0, s, in, out, rows, cols, chunk_rows, carry);
    if (vec) launch_pdl(scan_tiled_kernel<OP, 2, true>, dim3(strips, (unsigned)chunks), dim3(SCAN_THREADS), smem, s, in, out, rows, cols, chunk_rows, tile_rows, (const uint32_t*)carry);
    else launch_pdl(scan_tiled_kernel<OP, 2, false>, dim3(strips, (unsigned)chunks), dim3(SCAN_THREADS), smem, s, in, out, rows, cols, chunk_rows, tile_rows, (const uint32_t*)carry);
  }
  return cudaGetLastError();
}

// ---- sort ----------------------------------------------------------------------------------------------
constexpr int SORT_THREADS = 256;

__device__ __forceinline__ uint32_t ordered(uint32_t x, int is_i32, int descending) {
  uint32_t u = is_i32 ? (x ^ 0x80000000u) : ((x & 0x80000000u) ? ~x : (x | 0x80000000u));
  return descending ? ~u : u;
}
__device__ __forceinline__ uint32_t unordered(uint32_t u, int is_i32, int descending) {
  if (descending) u = ~u;
  return is_i32 ? (u ^ 0x80000000u) : ((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

// A wire's place in shared memory: one word of padding every eight, so that a thread reading eight consecutive
// wires (72 bytes from its neighbour's) meets no bank conflict.
__device__ __forceinline__ uint32_t wire_at(uint32_t i) { return i + (i >> 3); }
__device__ __forceinline__ void exchange(unsigned long long& a, unsigned long long& b, bool up) {
  if ((a > b) == up) { const unsigned long long t = a; a = b; b = t; }
}

// grid (column blocks, 4): block (cb, j) sorts problems 32 cb + 8 j + c, c = 0..7, over N = `rows` wires.  The
// network's stages whose partners are less than eight wires apart (the first six stages, and the last three of
// every later merge) run in registers, eight wires a thread; the others are one pass over shared memory each.
__global__ void __launch_bounds__(SORT_THREADS)
sort_planes_kernel(const uint32_t* __restrict__ in, uint64_t rows, uint64_t cols, uint32_t n, int is_i32, int descending,
                   uint32_t* __restrict__ keys, uint32_t* __restrict__ indices) {
  extern __shared__ unsigned long long wires[];          // [8][N + N / 8]
  pdl_enter();
  const uint32_t N = (uint32_t)rows, NP = N + N / 8, cb = blockIdx.x, j = blockIdx.y, tid = threadIdx.x;
  const uint32_t word = tid & 31;                         // a column of the tile row: (face % 2, c, odd)
  const uint32_t fl = word >> 4, c = (word >> 1) & 7, odd = word & 1;
  // tile rows this block owns: row = 32 tr + 16 fh + 4 g + j
  for (uint32_t rr = tid >> 5; rr < N / 4; rr += SORT_THREADS / 32) {
    const uint32_t tr = rr >> 3, fh = (rr >> 2) & 1, g = rr & 3;
    const uint64_t row = 32ull * tr + 16 * fh + 4 * g + j;
    const uint32_t e = 32 * tr + 8 * (2 * fh + fl) + 2 * g + odd;
    const uint32_t x = in[row * cols + 32ull * cb + word];
    const uint32_t u = e < n ? ordered(x, is_i32, descending) : 0xffffffffu;
    wires[c * NP + wire_at(e)] = ((unsigned long long)u << 32) | e;
  }
  __syncthreads();
  const uint32_t half_lg = 30 - __clz(N);                  // log2(N / 2)
  const uint32_t group_lg = half_lg - 2;                   // log2(N / 8): groups of eight wires a problem
  // the stages inside a group of eight: all of k = 2, 4, 8 (`first`), or s = 4, 2, 1 of merge k
  auto in_registers = [&](uint32_t k, bool first) {
    for (uint32_t g = tid; g < N; g += SORT_THREADS) {     // 8 problems x N / 8 groups
      const uint32_t prob = g >> group_lg, base = (g & ((N >> 3) - 1)) << 3;
      unsigned long long* w = wires + prob * NP + wire_at(base);
      unsigned long long v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = w[i];
      if (first) {
#pragma unroll
        for (int kk = 2; kk <= 8; kk <<= 1)
#pragma unroll
          for (int ss = kk >> 1; ss >= 1; ss >>= 1)
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (!(i & ss)) exchange(v[i], v[i | ss], ((base + i) & kk) == 0);
      } else {
        const bool up = (base & k) == 0;
#pragma unroll
        for (int ss = 4; ss >= 1; ss >>= 1)
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (!(i & ss)) exchange(v[i], v[i | ss], up);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) w[i] = v[i];
    }
    __syncthreads();
  };
  in_registers(8, true);
  for (uint32_t k = 16; k <= N; k <<= 1) {
    for (uint32_t s = k >> 1; s >= 8; s >>= 1) {
      for (uint32_t t = tid; t < 4 * N; t += SORT_THREADS) {     // 8 problems x N/2 exchanges
        const uint32_t prob = t >> half_lg, i = t & (N / 2 - 1);     // N is a power of two
        const uint32_t lo = ((i & ~(s - 1)) << 1) | (i & (s - 1)), hi = lo | s;
        unsigned long long* w = wires + prob * NP;
        const unsigned long long a = w[wire_at(lo)], b = w[wire_at(hi)];
        const bool up = (lo & k) == 0;
        if ((a > b) == up) { w[wire_at(lo)] = b; w[wire_at(hi)] = a; }
      }
      __syncthreads();
    }
    in_registers(k, false);
  }
  for (uint32_t rr = tid >> 5; rr < N / 4; rr += SORT_THREADS / 32) {
    const uint32_t tr = rr >> 3, fh = (rr >> 2) & 1, g = rr & 3;
    const uint64_t row = 32ull * tr + 16 * fh + 4 * g + j;
    const uint32_t e = 32 * tr + 8 * (2 * fh + fl) + 2 * g + odd;
    const unsigned long long w = wires[c * NP + wire_at(e)];
    keys[row * cols + 32ull * cb + word] = unordered((uint32_t)(w >> 32), is_i32, descending);
    if (indices) indices[row * cols + 32ull * cb + word] = (uint32_t)w;
  }
}

}  // namespace

uint64_t scan_chunks(int op, uint64_t rows, uint64_t cols) {
  if (op == S_SUM || op == S_PROD) return 1;                 // a left fold in row order: the rows stay together
  const uint64_t strips = (cols + 31) / 32;                  // blocks of the scanning kernel a chunk
  if (strips >= 148 || rows < 512) return 1;
  uint64_t chunks = (148 * 2 + strips - 1) / strips;
  if (chunks > rows / 256) chunks = rows / 256;
  if (chunks > 256) chunks = 256;
  return chunks < 2 ? 1 : chunks;
}

cudaError_t launch_scan(const uint32_t* in, uint32_t* out, uint64_t rows, uint64_t cols, int op, uint32_t* carry, cudaStream_t s) {
  if (rows == 0 || cols == 0) return cudaSuccess;
  uint64_t chunks = carry ? scan_chunks(op, rows, cols) : 1;
  const uint64_t chunk_rows = (rows + chunks - 1) / chunks;
  chunks = (rows + chunk_rows - 1) / chunk_rows;
  switch (op) {
#define GO(OP) case OP: return scan_go<OP>(in, out, rows, cols, chunks, chunk_rows, carry, s);
    GO(S_SUM) GO(S_PROD) GO(S_MIN) GO(S_MAX) GO(S_MINNAN) GO(S_MAXNAN) GO(S_ISUM) GO(S_IPROD) GO(S_IMIN) GO(S_IMAX)
#undef GO
    default: return cudaErrorNotSupported;
  }
}

cudaError_t launch_sort_planes(const uint32_t* in, uint64_t rows, uint64_t cols, uint32_t n, int is_i32, int descending,
                               uint32_t* keys, uint32_t* indices, cudaStream_t s) {
  if (rows == 0 || cols == 0) return cudaSuccess;
  const size_t smem = (size_t)8 * (rows + rows / 8) * sizeof(unsigned long long);
  {
    const cudaError_t e = ensure_dynamic_smem((const void*)sort_planes_kernel, smem);
    if (e != cudaSuccess) return e;
  }
  launch_pdl(sort_planes_kernel, dim3((unsigned)(cols / 32), 4), dim3(SORT_THREADS), smem, s, in, rows, cols, n, is_i32, descending,
             keys, indices);
  return cudaGetLastError();
}

}  // namespace b200
