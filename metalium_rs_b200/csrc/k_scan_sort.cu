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
#include <cstdlib>
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
// its rows in tiles of `tile_rows` rows.  All of its warps bring the next tile into shared memory with
// cp.async while warp 0 scans the current one in place (a lane a column, the serial chain now an add or a
// select a row with its operand already on chip), then all warps store the scanned tile in whole lines.  The
// loads in flight no longer depend on the chain, which is what a thread-a-column loop over global memory
// cannot give (a [8192, 8192] row-order sum: 1.3 TB/s of bytes moved that way, 3.1 TB/s with two tiles a block).
constexpr int SCAN_THREADS = 128;

__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int SCAN_STAGES = 4;          // tiles a block keeps in shared memory: three in flight behind the one being scanned

template <int OP, int MODE>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_tiled_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, uint64_t rows, uint64_t cols, uint64_t chunk_rows,
                  int tile_rows, int strip, const uint32_t* __restrict__ carry) {
  extern __shared__ uint32_t tiles[];                      // SCAN_STAGES tiles of [tile_rows][strip]
  pdl_enter();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int segs = strip / 32;                             // 32-column segments a row of the strip: a scanning warp each
  const uint64_t c0 = (uint64_t)blockIdx.x * strip;
  const uint64_t chunk = blockIdx.y, r0 = chunk * chunk_rows;
  const uint64_t r1 = r0 + chunk_rows < rows ? r0 + chunk_rows : rows;
  const bool scans = warp < segs && c0 + warp * 32 + lane < cols;
  uint32_t acc = scan_identity<OP>();
  if (MODE == 2 && scans)
    for (uint64_t k = 0; k < chunk; ++k) acc = scan_step<OP>(acc, carry[k * cols + c0 + warp * 32 + lane]);
  const int warps = SCAN_THREADS / 32;
  const size_t tile_words = (size_t)tile_rows * strip;
  const uint64_t n_tiles = (r1 - r0 + tile_rows - 1) / tile_rows;
  // every thread commits one group a tile slot, empty past the last tile, so "all but the newest
  // SCAN_STAGES - 1 groups are complete" always means "tile t has landed"
  auto fetch = [&](uint64_t t) {
    if (t < n_tiles) {
      const uint64_t row0 = r0 + t * tile_rows;
      const int n = (int)(r1 - row0 < (uint64_t)tile_rows ? r1 - row0 : tile_rows);
      uint32_t* buf = tiles + (t % SCAN_STAGES) * tile_words;
      for (int i = warp; i < n * segs; i += warps) {         // whole 128-byte segments, a row's side by side
        const int r = i / segs, sg = i - r * segs;
        if (c0 + sg * 32 + lane < cols) cp_async4(buf + r * strip + sg * 32 + lane, in + (row0 + r) * cols + c0 + sg * 32 + lane);
      }
    }
    cp_async_commit();
  };
  for (int t = 0; t < SCAN_STAGES - 1; ++t) fetch(t);
  for (uint64_t t = 0; t < n_tiles; ++t) {
    uint32_t* cur = tiles + (t % SCAN_STAGES) * tile_words;
    const uint64_t row0 = r0 + t * tile_rows;
    const int n = (int)(r1 - row0 < (uint64_t)tile_rows ? r1 - row0 : tile_rows);
    // the slot this fetch fills held tile t - 1, which every thread stored at the end of the iteration before
    // (a thread refills only words it stored itself: the two loops deal the segments to the warps alike)
    fetch(t + SCAN_STAGES - 1);
    cp_async_wait<SCAN_STAGES - 1>();
    __syncthreads();
    if (scans) {
      uint32_t* col = cur + warp * 32 + lane;
      int r = 0;
      for (; r + 8 <= n; r += 8) {
        uint32_t x[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) x[u] = col[(r + u) * strip];
#pragma unroll
        for (int u = 0; u < 8; ++u) { acc = scan_step<OP>(acc, x[u]); col[(r + u) * strip] = acc; }
      }
      for (; r < n; ++r) { acc = scan_step<OP>(acc, col[r * strip]); col[r * strip] = acc; }
    }
    __syncthreads();
    for (int i = warp; i < n * segs; i += warps) {
      const int r = i / segs, sg = i - r * segs;
      if (c0 + sg * 32 + lane < cols) out[(row0 + r) * cols + c0 + sg * 32 + lane] = cur[r * strip + sg * 32 + lane];
    }
  }
}

template <int OP>
cudaError_t scan_go(const uint32_t* in, uint32_t* out, uint64_t rows, uint64_t cols, uint64_t chunks, uint64_t chunk_rows,
                    uint32_t* carry, cudaStream_t s) {
  const dim3 block(128);
  const unsigned gx = (unsigned)((cols + 127) / 128);
  // A block's strip is 32, 64 or 128 columns (one to four scanning warps): wider strips make longer contiguous
  // reads a row (HBM pages stay open) as long as enough blocks remain to fill the device.
  static int forced = -1;
  if (forced < 0) { const char* e = getenv("B200TT_SCAN_STRIP"); forced = e ? atoi(e) : 0; }
  int strip = 128;
  while (strip > 32 && ((cols + strip - 1) / strip) * chunks < 64) strip >>= 1;
  if (forced == 32 || forced == 64 || forced == 128) strip = forced;
  const unsigned strips = (unsigned)((cols + strip - 1) / strip);
  // every block resident at once: the tiles are as deep as the shared memory of an SM, shared by the blocks that
  // land on it, allows (few blocks: deep tiles, so that what a block has in flight hides the latency)
  const uint64_t per_sm = ((uint64_t)strips * chunks + 147) / 148;
  int tile_rows = 256;
  while (tile_rows > 16 && per_sm * SCAN_STAGES * tile_rows * strip * 4 > 200 * 1024) tile_rows >>= 1;
  const size_t smem = (size_t)SCAN_STAGES * tile_rows * strip * sizeof(uint32_t);
  static size_t set0 = 0, set2 = 0;
  if (smem > 48 * 1024) {
    if (chunks <= 1 && smem > set0) {
      cudaError_t e = cudaFuncSetAttribute(scan_tiled_kernel<OP, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      set0 = smem;
    }
    if (chunks > 1 && smem > set2) {
      cudaError_t e = cudaFuncSetAttribute(scan_tiled_kernel<OP, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      set2 = smem;
    }
  }
  if (chunks <= 1) {
    launch_pdl(scan_tiled_kernel<OP, 0>, dim3(strips, 1), dim3(SCAN_THREADS), smem, s, in, out, rows, cols, rows, tile_rows, strip,
               (const uint32_t*)nullptr);
  } else {
    launch_pdl(scan_kernel<OP, 1>, dim3(gx, (unsigned)chunks), block, 0, s, in, out, rows, cols, chunk_rows, carry);
    launch_pdl(scan_tiled_kernel<OP, 2>, dim3(strips, (unsigned)chunks), dim3(SCAN_THREADS), smem, s, in, out, rows, cols, chunk_rows,
               tile_rows, strip, (const uint32_t*)carry);
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

// grid (column blocks, 4): block (cb, j) sorts problems 32 cb + 8 j + c, c = 0..7, over N = `rows` wires.
__global__ void __launch_bounds__(SORT_THREADS)
sort_planes_kernel(const uint32_t* __restrict__ in, uint64_t rows, uint64_t cols, uint32_t n, int is_i32, int descending,
                   uint32_t* __restrict__ keys, uint32_t* __restrict__ indices) {
  extern __shared__ unsigned long long wires[];          // [8][N]
  pdl_enter();
  const uint32_t N = (uint32_t)rows, cb = blockIdx.x, j = blockIdx.y, tid = threadIdx.x;
  const uint32_t word = tid & 31;                         // a column of the tile row: (face % 2, c, odd)
  const uint32_t fl = word >> 4, c = (word >> 1) & 7, odd = word & 1;
  // tile rows this block owns: row = 32 tr + 16 fh + 4 g + j
  for (uint32_t rr = tid >> 5; rr < N / 4; rr += SORT_THREADS / 32) {
    const uint32_t tr = rr >> 3, fh = (rr >> 2) & 1, g = rr & 3;
    const uint64_t row = 32ull * tr + 16 * fh + 4 * g + j;
    const uint32_t e = 32 * tr + 8 * (2 * fh + fl) + 2 * g + odd;
    const uint32_t x = in[row * cols + 32ull * cb + word];
    const uint32_t u = e < n ? ordered(x, is_i32, descending) : 0xffffffffu;
    wires[c * N + e] = ((unsigned long long)u << 32) | e;
  }
  __syncthreads();
  const uint32_t half_lg = 30 - __clz(N);                  // log2(N / 2)
  for (uint32_t k = 2; k <= N; k <<= 1) {
    for (uint32_t s = k >> 1; s > 0; s >>= 1) {
      for (uint32_t t = tid; t < 4 * N; t += SORT_THREADS) {     // 8 problems x N/2 exchanges
        const uint32_t prob = t >> half_lg, i = t & (N / 2 - 1);     // N is a power of two
        const uint32_t lo = ((i & ~(s - 1)) << 1) | (i & (s - 1)), hi = lo | s;
        unsigned long long* w = wires + prob * N;
        const unsigned long long a = w[lo], b = w[hi];
        const bool up = (lo & k) == 0;
        if ((a > b) == up) { w[lo] = b; w[hi] = a; }
      }
      __syncthreads();
    }
  }
  for (uint32_t rr = tid >> 5; rr < N / 4; rr += SORT_THREADS / 32) {
    const uint32_t tr = rr >> 3, fh = (rr >> 2) & 1, g = rr & 3;
    const uint64_t row = 32ull * tr + 16 * fh + 4 * g + j;
    const uint32_t e = 32 * tr + 8 * (2 * fh + fl) + 2 * g + odd;
    const unsigned long long w = wires[c * N + e];
    keys[row * cols + 32ull * cb + word] = unordered((uint32_t)(w >> 32), is_i32, descending);
    if (indices) indices[row * cols + 32ull * cb + word] = (uint32_t)w;
  }
}

}  // namespace

uint64_t scan_chunks(int op, uint64_t rows, uint64_t cols) {
  if (op == S_SUM || op == S_PROD) return 1;                 // a left fold in row order: the rows stay together
  const uint64_t col_blocks = (cols + 127) / 128;
  if (col_blocks >= 148 * 2 || rows < 512) return 1;
  uint64_t chunks = (148 * 4 + col_blocks - 1) / col_blocks;
  if (chunks > rows / 64) chunks = rows / 64;
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
  const size_t smem = (size_t)8 * rows * sizeof(unsigned long long);
  static size_t set = 0;
  if (smem > 48 * 1024 && smem > set) {
    cudaError_t e = cudaFuncSetAttribute(sort_planes_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    set = smem;
  }
  launch_pdl(sort_planes_kernel, dim3((unsigned)(cols / 32), 4), dim3(SORT_THREADS), smem, s, in, rows, cols, n, is_i32, descending,
             keys, indices);
  return cudaGetLastError();
}

}  // namespace b200
