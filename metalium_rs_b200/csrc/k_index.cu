// Indexing and copy kernels: every one moves raw bits (crates/tt-kernels/src/index.rs,
// crates/tt-kernels/src/session.rs:7978-8396).  A datum's sign of zero, NaN payload and
// denormal bits survive.  An index outside its table sets the engine's error word to
// DOMAIN and the access is skipped (crates/burn-tt/src/ops.rs:1177 "checked indices").
#include "device_math.cuh"
#include "kernels.h"
#include "pdl.cuh"

namespace b200 {
namespace {

constexpr int DOMAIN = 6;
__device__ __forceinline__ void set_err(int* err, int code) { if (err) atomicCAS(err, 0, code); }

// Copy `bytes` (a multiple of elem size) from src to dst with the widest aligned vector.
__device__ __forceinline__ void copy_row(const char* src, char* dst, uint64_t bytes, int lane, int lanes) {
  if ((((uintptr_t)src | (uintptr_t)dst | bytes) & 15) == 0) {
    const uint4* s = (const uint4*)src; uint4* d = (uint4*)dst;
    for (uint64_t i = lane; i < bytes / 16; i += lanes) d[i] = s[i];
  } else if ((((uintptr_t)src | (uintptr_t)dst | bytes) & 3) == 0) {
    const uint32_t* s = (const uint32_t*)src; uint32_t* d = (uint32_t*)dst;
    for (uint64_t i = lane; i < bytes / 4; i += lanes) d[i] = s[i];
  } else {
    const uint16_t* s = (const uint16_t*)src; uint16_t* d = (uint16_t*)dst;
    for (uint64_t i = lane; i < bytes / 2; i += lanes) d[i] = s[i];
  }
}

// out[i,:] = table[idx[i],:]; a warp a row.
__global__ void __launch_bounds__(256)
select_rows_kernel(const char* table, uint64_t t_rows, uint64_t row_bytes, const int32_t* idx, uint64_t n,
                   char* out, int* err) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint64_t nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  for (uint64_t i = warp; i < n; i += nwarps) {
    const int64_t r = idx[i];
    if (r < 0 || (uint64_t)r >= t_rows) { if (lane == 0) set_err(err, DOMAIN); continue; }
    copy_row(table + (uint64_t)r * row_bytes, out + i * row_bytes, row_bytes, lane, 32);
  }
}

__global__ void pick_columns_kernel(const uint32_t* x, uint64_t rows, uint64_t cols, const int32_t* idx,
                                    uint32_t* out, int* err) {
  const uint64_t r = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int64_t c = idx[r];
  if (c < 0 || (uint64_t)c >= cols) { set_err(err, DOMAIN); out[r] = 0; return; }
  out[r] = x[r * cols + c];
}

// t (a copy of the input) gets v[r] added at (r, idx[r]): one add a row, every other
// datum untouched (crates/burn-tt/src/ops.rs:1043).
__global__ void scatter_add_columns_kernel(float* t, uint64_t rows, uint64_t cols, const int32_t* idx,
                                           const float* v, int* err) {
  const uint64_t r = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int64_t c = idx[r];
  if (c < 0 || (uint64_t)c >= cols) { set_err(err, DOMAIN); return; }
  t[r * cols + c] = t[r * cols + c] + v[r];
}

// out[idx[i],:] += value[i,:], i ascending: a thread owns a column and walks the index
// list in order, so rows named twice are added in index order (server.rs:358).
__global__ void __launch_bounds__(128)
select_add_rows_kernel(float* out, uint64_t t_rows, uint64_t cols, const int32_t* idx, uint64_t n,
                       const float* value, int* err) {
  const uint64_t c = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  for (uint64_t i = 0; i < n; ++i) {
    const int64_t r = idx[i];
    if (r < 0 || (uint64_t)r >= t_rows) { if (c == 0) set_err(err, DOMAIN); continue; }
    out[(uint64_t)r * cols + c] = out[(uint64_t)r * cols + c] + value[i * cols + c];
  }
}

// out[idx[i],:] = values[i,:]; a thread owns a column and walks the list in order, so the
// last assignment to a row wins whatever the launch (server.rs:379).
__global__ void __launch_bounds__(128)
scatter_rows_kernel(uint32_t* out, uint64_t t_rows, uint64_t cols, const int32_t* idx, uint64_t n,
                    const uint32_t* values, int* err) {
  const uint64_t c = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  for (uint64_t i = 0; i < n; ++i) {
    const int64_t r = idx[i];
    if (r < 0 || (uint64_t)r >= t_rows) { if (c == 0) set_err(err, DOMAIN); continue; }
    out[(uint64_t)r * cols + c] = values[i * cols + c];
  }
}

// scatter_rows into the table itself (server.rs:389): table[idx[i], :] = the block's row i, for a
// table of 16- or 32-bit elements and values that are a block of a wider buffer.  A thread a
// column, the rows in order, so the last assignment to a row wins whatever the launch.
template <typename E>
__global__ void __launch_bounds__(128)
scatter_rows_into_kernel(E* table, uint64_t t_rows, uint64_t cols, const int32_t* idx, uint64_t n,
                         const E* values, uint64_t v_ld, int* err) {
  pdl_enter();
  const uint64_t c = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  for (uint64_t i = 0; i < n; ++i) {
    const int64_t r = idx[i];
    if (r < 0 || (uint64_t)r >= t_rows) { if (c == 0) set_err(err, DOMAIN); continue; }
    table[(uint64_t)r * cols + c] = values[i * v_ld + c];
  }
}

// A [rows, row_bytes] block copied into the same place of up to eight matrices (this GPU's or, through
// IPC mappings, its peers'): what an all-gather of column slices is when every rank stores its own
// slice everywhere.  16-byte pieces, consecutive threads on consecutive pieces of a row.
struct ManyDst { char* p[8]; int n; int multicast; };
__global__ void __launch_bounds__(256)
store_block_many_kernel(const char* __restrict__ src, uint64_t src_pitch, ManyDst dst, uint64_t dst_pitch, uint64_t rows,
                        uint64_t row_bytes) {
  const uint64_t units = row_bytes / 16, total = rows * units;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t r = i / units, u = i - r * units;
    const uint4 w = *reinterpret_cast<const uint4*>(src + r * src_pitch + u * 16);
    if (dst.multicast) st_multicast_16(dst.p[0] + r * dst_pitch + u * 16, w);   // one store, delivered to every GPU of the group
    else for (int d = 0; d < dst.n; ++d) *reinterpret_cast<uint4*>(dst.p[d] + r * dst_pitch + u * 16) = w;
  }
}

__global__ void __launch_bounds__(128)
scatter_rows_narrow_kernel(uint16_t* table, uint64_t t_rows, uint64_t cols, const int32_t* idx, uint64_t n,
                           const uint32_t* values, uint64_t v_ld, int* err) {
  pdl_enter();
  const uint64_t c = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  for (uint64_t i = 0; i < n; ++i) {
    const int64_t r = idx[i];
    if (r < 0 || (uint64_t)r >= t_rows) { if (c == 0) set_err(err, DOMAIN); continue; }
    table[(uint64_t)r * cols + c] = f32_to_bf16_bits(values[i * v_ld + c]);
  }
}

// out[r, j] = x[r, idx[r, j]]  (Burn's gather along the last dim)
__global__ void gather_indexed_kernel(const uint32_t* x, uint64_t rows, uint64_t cols, const int32_t* idx,
                                      uint64_t i_cols, uint32_t* out, int* err) {
  const uint64_t n = rows * i_cols;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t r = i / i_cols;
    const int64_t c = idx[i];
    if (c < 0 || (uint64_t)c >= cols) { set_err(err, DOMAIN); out[i] = 0; continue; }
    out[i] = x[r * cols + c];
  }
}

__global__ void __launch_bounds__(256)
gather_row_ptrs_kernel(const void* const* row_ptrs, uint64_t n_rows, uint64_t row_bytes, char* out) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint64_t nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  for (uint64_t i = warp; i < n_rows; i += nwarps)
    copy_row((const char*)row_ptrs[i], out + i * row_bytes, row_bytes, lane, 32);
}

// A thread owns a column and applies the pairs in order: a row assigned twice keeps the last.
__global__ void __launch_bounds__(128)
assign_rows_kernel(char* out, const char* value, uint64_t cols, int elem_bytes, const uint64_t* pairs,
                   uint64_t n) {
  const uint64_t c = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  for (uint64_t i = 0; i < n; ++i) {
    const uint64_t d = pairs[2 * i], s = pairs[2 * i + 1];
    if (elem_bytes == 4)
      ((uint32_t*)out)[d * cols + c] = ((const uint32_t*)value)[s * cols + c];
    else
      ((uint16_t*)out)[d * cols + c] = ((const uint16_t*)value)[s * cols + c];
  }
}

// One block of a copy_blocks call: blockIdx.z = move, 32x32 tiles through shared memory so
// both the read and the write are coalesced whether or not the block is transposed.
template <typename T>
__global__ void __launch_bounds__(256)
copy_blocks_kernel(const T* src, uint64_t src_ld, T* dst, uint64_t dst_ld, const MoveDev* moves) {
  __shared__ T tile[32][33];
  const MoveDev mv = moves[blockIdx.z];
  // output block extent is mv.rows x mv.cols at (to_r, to_c)
  const uint64_t tiles_c = (mv.cols + 31) / 32, tiles_r = (mv.rows + 31) / 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (uint64_t t = blockIdx.x; t < tiles_c * tiles_r; t += gridDim.x) {
    const uint64_t tr = t / tiles_c, tc = t % tiles_c;
    if (!mv.transposed) {
      for (int j = ty; j < 32; j += 8) {
        const uint64_t r = tr * 32 + j, c = tc * 32 + tx;
        if (r < mv.rows && c < mv.cols)
          dst[(mv.to_r + r) * dst_ld + mv.to_c + c] = src[(mv.from_r + r) * src_ld + mv.from_c + c];
      }
    } else {
      // source block is cols x rows; out[r][c] = src[c][r]
      for (int j = ty; j < 32; j += 8) {
        const uint64_t sr = tc * 32 + j, sc = tr * 32 + tx;  // source row (= out col), source col (= out row)
        if (sr < mv.cols && sc < mv.rows)
          tile[j][tx] = src[(mv.from_r + sr) * src_ld + mv.from_c + sc];
      }
      __syncthreads();
      for (int j = ty; j < 32; j += 8) {
        const uint64_t r = tr * 32 + j, c = tc * 32 + tx;
        if (r < mv.rows && c < mv.cols) dst[(mv.to_r + r) * dst_ld + mv.to_c + c] = tile[tx][j];
      }
      __syncthreads();
    }
  }
}

template <typename T>
__global__ void repack_kernel(const T* src, uint64_t src_ld, const uint64_t* pairs, uint64_t n, T* out) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (uint64_t)gridDim.x * blockDim.x)
    out[i] = src[pairs[2 * i] * src_ld + pairs[2 * i + 1]];
}

// out[i] = the datum at addrs[i]: `Engine::repack_many` (crates/burn-tt/src/server.rs:317,
// crates/tt-kernels/src/tensor.rs:6791), one source a result element out of several buffers; the host
// resolves (buffer, row, column) to an address, so the kernel is one gather.
template <typename T>
__global__ void gather_addrs_kernel(const uint64_t* __restrict__ addrs, uint64_t n, T* __restrict__ out) {
  pdl_enter();
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
    out[i] = *reinterpret_cast<const T*>(addrs[i]);
}

// `Engine::select_taps` (server.rs:309; crates/tt-kernels/src/index.rs:136-160): row i of the result holds,
// for each tap t, row idx[t][i] of the table from column t * pitch (pitch = the table's columns rounded
// up to 32; the last tap takes the table's own columns only).  The columns between a tap's end and the
// next tap's start are zero, and with `zero_row` an index equal to the table's rows reads zeros (a
// convolution's padding tap).  A warp a (row, tap).
__global__ void __launch_bounds__(256)
select_taps_kernel(const char* __restrict__ table, uint64_t t_rows, uint64_t cols, int eb, const int32_t* __restrict__ idx,
                   uint64_t taps, uint64_t n, int zero_row, char* __restrict__ out, uint64_t out_cols, uint64_t pitch, int lanes_per,
                   int* err) {
  pdl_enter();
  // a (row, tap) takes `lanes_per` lanes (a power of two: enough 16-byte pieces for a tap's columns), so a warp
  // moves 32 / lanes_per of them at once
  const int lane = threadIdx.x & 31, sub = lane / lanes_per, ln = lane % lanes_per, per = 32 / lanes_per;
  const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint64_t nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  for (uint64_t w = warp * per + sub; w < n * taps; w += nwarps * per) {
    const uint64_t i = w / taps, t = w - i * taps;
    const int64_t r = idx[t * n + i];
    char* dst = out + (i * out_cols + t * pitch) * eb;
    const uint64_t width = (t + 1 < taps ? pitch : cols);          // this tap's columns of the result
    const bool zero = zero_row && r == (int64_t)t_rows;
    if (!zero && (r < 0 || (uint64_t)r >= t_rows)) { if (ln == 0) set_err(err, DOMAIN); continue; }
    if (zero) {
      for (uint64_t b = ln * 2; b < width * eb; b += 2 * lanes_per) *reinterpret_cast<uint16_t*>(dst + b) = 0;
    } else {
      copy_row(table + (uint64_t)r * cols * eb, dst, cols * eb, ln, lanes_per);
      for (uint64_t b = cols * eb + ln * 2; b < width * eb; b += 2 * lanes_per) *reinterpret_cast<uint16_t*>(dst + b) = 0;
    }
  }
}

inline unsigned cap_grid(uint64_t blocks) { return (unsigned)(blocks < 148ull * 32 ? (blocks ? blocks : 1) : 148ull * 32); }

}  // namespace

cudaError_t launch_select_rows(const void* table, uint64_t t_rows, uint64_t cols, int elem_bytes,
                               const int32_t* idx, uint64_t n, void* out, int* err, cudaStream_t s) {
  if (n == 0 || cols == 0) return cudaSuccess;
  select_rows_kernel<<<cap_grid((n + 7) / 8), 256, 0, s>>>((const char*)table, t_rows, cols * elem_bytes, idx, n,
                                                           (char*)out, err);
  return cudaGetLastError();
}
cudaError_t launch_pick_columns(const uint32_t* x, uint64_t rows, uint64_t cols, const int32_t* idx,
                                uint32_t* out, int* err, cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  pick_columns_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, s>>>(x, rows, cols, idx, out, err);
  return cudaGetLastError();
}
cudaError_t launch_scatter_add_columns(float* t, uint64_t rows, uint64_t cols, const int32_t* idx,
                                       const float* v, int* err, cudaStream_t s) {
  if (rows == 0) return cudaSuccess;
  scatter_add_columns_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, s>>>(t, rows, cols, idx, v, err);
  return cudaGetLastError();
}
cudaError_t launch_select_add_rows(float* out, uint64_t t_rows, uint64_t cols, const int32_t* idx,
                                   uint64_t n, const float* value, int* err, cudaStream_t s) {
  if (n == 0 || cols == 0) return cudaSuccess;
  select_add_rows_kernel<<<(unsigned)((cols + 127) / 128), 128, 0, s>>>(out, t_rows, cols, idx, n, value, err);
  return cudaGetLastError();
}
cudaError_t launch_scatter_rows(uint32_t* out, uint64_t t_rows, uint64_t cols, const int32_t* idx,
                                uint64_t n, const uint32_t* values, int* err, cudaStream_t s) {
  if (n == 0 || cols == 0) return cudaSuccess;
  scatter_rows_kernel<<<(unsigned)((cols + 127) / 128), 128, 0, s>>>(out, t_rows, cols, idx, n, values, err);
  return cudaGetLastError();
}
cudaError_t launch_scatter_rows_into(void* table, uint64_t t_rows, uint64_t cols, int elem_bytes, const int32_t* idx,
                                     uint64_t n, const void* values, uint64_t v_ld, int* err, cudaStream_t s) {
  if (n == 0 || cols == 0) return cudaSuccess;
  const unsigned grid = (unsigned)((cols + 127) / 128);
  if (elem_bytes == -2)   // a BF16 table, F32 values: each rounded once (what `cast_float` would store)
    launch_pdl(scatter_rows_narrow_kernel, dim3(grid), dim3(128), 0, s, (uint16_t*)table, t_rows, cols, idx, n, (const uint32_t*)values, v_ld, err);
  else if (elem_bytes == 2)
    launch_pdl(scatter_rows_into_kernel<uint16_t>, dim3(grid), dim3(128), 0, s, (uint16_t*)table, t_rows, cols, idx, n, (const uint16_t*)values, v_ld, err);
  else
    launch_pdl(scatter_rows_into_kernel<uint32_t>, dim3(grid), dim3(128), 0, s, (uint32_t*)table, t_rows, cols, idx, n, (const uint32_t*)values, v_ld, err);
  return cudaGetLastError();
}
cudaError_t launch_store_block_many(const void* src, uint64_t src_pitch, void* const* dst, int n_dst, uint64_t dst_pitch,
                                    uint64_t rows, uint64_t row_bytes, int multicast, cudaStream_t s) {
  if (rows == 0 || row_bytes == 0) return cudaSuccess;
  if (n_dst < 1 || n_dst > 8 || row_bytes % 16 || src_pitch % 16 || dst_pitch % 16 || ((uintptr_t)src & 15)) return cudaErrorNotSupported;
  if (multicast && n_dst != 1) return cudaErrorNotSupported;
  ManyDst d;
  d.n = n_dst;
  d.multicast = multicast;
  for (int i = 0; i < 8; ++i) {
    d.p[i] = i < n_dst ? (char*)dst[i] : nullptr;
    if (i < n_dst && ((uintptr_t)dst[i] & 15)) return cudaErrorNotSupported;
  }
  store_block_many_kernel<<<cap_grid((rows * (row_bytes / 16) + 255) / 256), 256, 0, s>>>((const char*)src, src_pitch, d, dst_pitch, rows, row_bytes);
  return cudaGetLastError();
}
cudaError_t launch_gather_indexed(const uint32_t* x, uint64_t rows, uint64_t cols, const int32_t* idx,
                                  uint64_t i_cols, uint32_t* out, int* err, cudaStream_t s) {
  if (rows * i_cols == 0) return cudaSuccess;
  gather_indexed_kernel<<<cap_grid((rows * i_cols + 255) / 256), 256, 0, s>>>(x, rows, cols, idx, i_cols, out, err);
  return cudaGetLastError();
}
cudaError_t launch_gather_row_ptrs(const void* const* row_ptrs, uint64_t n_rows, uint64_t cols,
                                   int elem_bytes, void* out, cudaStream_t s) {
  if (n_rows == 0 || cols == 0) return cudaSuccess;
  gather_row_ptrs_kernel<<<cap_grid((n_rows + 7) / 8), 256, 0, s>>>(row_ptrs, n_rows, cols * elem_bytes, (char*)out);
  return cudaGetLastError();
}
cudaError_t launch_assign_rows(void* out, const void* value, uint64_t cols, int elem_bytes,
                               const uint64_t* pairs, uint64_t n, cudaStream_t s) {
  if (n == 0 || cols == 0) return cudaSuccess;
  assign_rows_kernel<<<(unsigned)((cols + 127) / 128), 128, 0, s>>>((char*)out, (const char*)value, cols, elem_bytes, pairs, n);
  return cudaGetLastError();
}
cudaError_t launch_copy_blocks(const void* src, uint64_t src_ld, void* dst, uint64_t dst_ld,
                               int elem_bytes, const MoveDev* moves_dev, uint64_t n_moves,
                               uint64_t max_rows, uint64_t max_cols, cudaStream_t s) {
  if (n_moves == 0) return cudaSuccess;
  uint64_t tiles = ((max_rows + 31) / 32) * ((max_cols + 31) / 32);
  if (tiles == 0) return cudaSuccess;
  if (tiles > 4096) tiles = 4096;
  for (uint64_t z0 = 0; z0 < n_moves; z0 += 65535) {
    const unsigned nz = (unsigned)((n_moves - z0) < 65535 ? (n_moves - z0) : 65535);
    dim3 grid((unsigned)tiles, 1, nz);
    if (elem_bytes == 4)
      copy_blocks_kernel<uint32_t><<<grid, 256, 0, s>>>((const uint32_t*)src, src_ld, (uint32_t*)dst, dst_ld, moves_dev + z0);
    else
      copy_blocks_kernel<uint16_t><<<grid, 256, 0, s>>>((const uint16_t*)src, src_ld, (uint16_t*)dst, dst_ld, moves_dev + z0);
  }
  return cudaGetLastError();
}
cudaError_t launch_repack(const void* src, uint64_t src_ld, int elem_bytes, const uint64_t* pairs_dev,
                          uint64_t n, void* out, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  if (elem_bytes == 4)
    repack_kernel<uint32_t><<<cap_grid((n + 255) / 256), 256, 0, s>>>((const uint32_t*)src, src_ld, pairs_dev, n, (uint32_t*)out);
  else
    repack_kernel<uint16_t><<<cap_grid((n + 255) / 256), 256, 0, s>>>((const uint16_t*)src, src_ld, pairs_dev, n, (uint16_t*)out);
  return cudaGetLastError();
}

cudaError_t launch_gather_addrs(const uint64_t* addrs_dev, uint64_t n, int elem_bytes, void* out, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  if (elem_bytes == 4) launch_pdl(gather_addrs_kernel<uint32_t>, dim3(cap_grid((n + 255) / 256)), dim3(256), 0, s, addrs_dev, n, (uint32_t*)out);
  else launch_pdl(gather_addrs_kernel<uint16_t>, dim3(cap_grid((n + 255) / 256)), dim3(256), 0, s, addrs_dev, n, (uint16_t*)out);
  return cudaGetLastError();
}
cudaError_t launch_select_taps(const void* table, uint64_t t_rows, uint64_t cols, int elem_bytes, const int32_t* idx,
                               uint64_t taps, uint64_t n, int zero_row, void* out, uint64_t out_cols, int* err, cudaStream_t s) {
  if (n == 0 || taps == 0 || cols == 0) return cudaSuccess;
  const uint64_t pitch = (cols + 31) / 32 * 32;
  int lanes_per = 1;
  while (lanes_per < 32 && (uint64_t)lanes_per * 16 < pitch * elem_bytes) lanes_per <<= 1;
  const uint64_t per_block = 8 * (32 / lanes_per);
  launch_pdl(select_taps_kernel, dim3(cap_grid((n * taps + per_block - 1) / per_block)), dim3(256), 0, s, (const char*)table, t_rows, cols,
             elem_bytes, idx, taps, n, zero_row, (char*)out, out_cols, pitch, lanes_per, err);
  return cudaGetLastError();
}

}  // namespace b200
