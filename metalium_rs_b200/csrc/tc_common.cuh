// Shared pieces of the tcgen05 product kernels: mbarrier and TMA wrappers with bounded waits,
// the sm_100 shared-memory matrix descriptor, TMEM loads, the tile order, and the host-side
// tensor-map encoder (resolved from the driver at run time, so the library links no libcuda).
#pragma once
#include <cuda.h>
#include <stdlib.h>

#include "device_math.cuh"
#include "kernels.h"

namespace b200 {
namespace tc {

constexpr int BM = 128;
constexpr int BK = 64;            // bf16 elements: one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;  // 6 warps
constexpr int TIMEOUT_CODE = 4;
constexpr long long WAIT_CYCLES = 4000000000ll;  // ~2 s: far beyond any healthy wait (the default limit)

struct TcParams {
  uint64_t m, n, k;
  uint64_t lda, ldb, ldc;
  uint32_t tiles_m, tiles_n;
  uint64_t batch;
  const GemmBatch* batches;  // device, or nullptr
  void* c;
  void* c_more[7];           // further copies of C with c's pitch (a peer GPU's memory among them), or none
  int n_more;
  int epi_mode;              // 0: store the product; 1: silu(gate) * up of a tile's two 128-column halves (BN 256);
                             // 2: RoPE on the 64-column heads below rope_cols (BF16 result)
  const float* rope_cos;     // [rope_rows, 64] F32, pitch rope_ld: product row r uses table row r % rope_rows
  const float* rope_sin;     // [-sin, sin]
  uint32_t rope_rows, rope_ld, rope_cols;
  int staged;                // the epilogue may go through shared memory (pointers and pitch are 16-byte aligned)
  int out_bf16;
  int multicast;             // c is a multicast address (stored once with multimem.st, every row piece whole: no ragged edges)
  int* err;
  uint32_t mn_lbo, mn_sbo;   // byte offsets of an MN-major operand's descriptor
  uint32_t group;            // tile rows walked together (see tile_coords); 0: the default
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// The engine keeps its wait limit (clock cycles, `b200_config.wait_limit_cycles`) in the two words
// that follow its device error word; a kernel reads it once.  0 or less: the default.
__device__ __forceinline__ long long wait_limit_of(const int* err) {
  const long long v = *reinterpret_cast<const volatile long long*>(err + 2);
  return v > 0 ? v : WAIT_CYCLES;
}
// Bounded wait: false when it ran out (the caller abandons its role).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, long long limit) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > limit) return false;
  }
}

// The same wait by polling (`test_wait` never suspends the thread): the shortest wake-up after the
// arrival, for hand-offs that sit on a kernel's critical path, at the price of issue slots.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, volatile int* abort_flag, long long limit) {
  if (mbar_test(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 256; ++i)
      if (mbar_test(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > limit) return false;
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

// Shared-memory matrix descriptor (sm_100 UMMA): start address, leading / stride byte
// offsets (all >> 4), version 1, 128-byte swizzle.
// layout: 2 = 128-byte swizzle (16-byte atoms), 1 = 128-byte swizzle with 32-byte atoms (the only
// layout an MN-major 32-bit operand may use).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout = 2) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fff);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= 1ull << 46;  // descriptor version
  d |= (uint64_t)layout << 61;
  return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr) : "memory");
}

// ---- epilogue ---------------------------------------------------------------------------------
// A warp owns 32 rows of the accumulator (a lane a row).  Stored straight from registers a warp
// instruction would touch 32 rows with 16 bytes each; a peer GPU's memory takes such stores at a
// few percent of NVLink's rate.  So 128 bytes of each row are staged in shared memory (EPI_PITCH:
// 128 + 16 of padding, conflict-free both ways) and written back four rows of 128 contiguous bytes
// an instruction, to every copy of C.
constexpr uint32_t EPI_PITCH = 144;
constexpr uint32_t EPI_WARP_BYTES = 32 * EPI_PITCH;
constexpr uint32_t EPI_BYTES = 4 * EPI_WARP_BYTES;

__device__ __forceinline__ void epi_store_rows(const uint8_t* stage, const TcParams& p, uint64_t byte_off_row0,
                                               uint64_t pitch_bytes, uint64_t row0, int lane) {
  const int sub = lane >> 3, unit = lane & 7;
  if (p.multicast) {
    char* base = (char*)p.c + byte_off_row0 + unit * 16;
#pragma unroll
    for (int r = 0; r < 32; r += 4) {
      const int rr = r + sub;
      if (row0 + rr < p.m) st_multicast_16(base + (uint64_t)rr * pitch_bytes, *reinterpret_cast<const uint4*>(stage + rr * EPI_PITCH + unit * 16));
    }
    return;
  }
  for (int dsti = -1; dsti < p.n_more; ++dsti) {
    char* base = (char*)(dsti < 0 ? p.c : p.c_more[dsti]) + byte_off_row0 + unit * 16;
#pragma unroll
    for (int r = 0; r < 32; r += 4) {
      const int rr = r + sub;
      if (row0 + rr < p.m)
        *reinterpret_cast<uint4*>(base + (uint64_t)rr * pitch_bytes) = *reinterpret_cast<const uint4*>(stage + rr * EPI_PITCH + unit * 16);
    }
  }
}

// 32 columns of this lane's row straight from registers (ragged edges, unaligned pitches).
__device__ __forceinline__ void epi_store_direct(const TcParams& p, const uint32_t* v, uint64_t o, uint64_t col) {
  if (p.multicast) return;   // the host refuses a multicast product with ragged pieces; never a plain store to that address
  for (int dsti = -1; dsti < p.n_more; ++dsti) {
    void* const cbase = dsti < 0 ? p.c : p.c_more[dsti];
    if (p.out_bf16) {
      uint16_t* dst = (uint16_t*)cbase + o;
      if (col + 32 <= p.n && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 w;
          w.x = (uint32_t)f32_to_bf16_bits(v[q * 8 + 0]) | ((uint32_t)f32_to_bf16_bits(v[q * 8 + 1]) << 16);
          w.y = (uint32_t)f32_to_bf16_bits(v[q * 8 + 2]) | ((uint32_t)f32_to_bf16_bits(v[q * 8 + 3]) << 16);
          w.z = (uint32_t)f32_to_bf16_bits(v[q * 8 + 4]) | ((uint32_t)f32_to_bf16_bits(v[q * 8 + 5]) << 16);
          w.w = (uint32_t)f32_to_bf16_bits(v[q * 8 + 6]) | ((uint32_t)f32_to_bf16_bits(v[q * 8 + 7]) << 16);
          *reinterpret_cast<uint4*>(dst + q * 8) = w;
        }
      } else {
        for (int j = 0; j < 32 && col + j < p.n; ++j) dst[j] = f32_to_bf16_bits(v[j]);
      }
    } else {
      uint32_t* dst = (uint32_t*)cbase + o;
      if (col + 32 <= p.n && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<uint4*>(dst + q * 4) = make_uint4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
      } else {
        for (int j = 0; j < 32 && col + j < p.n; ++j) dst[j] = v[j];
      }
    }
  }
}

// One accumulator's 32 rows x BN_ columns (TMEM address `tacc`: this warp's lane quarter, the
// accumulator's first column) to every copy of C.  row0: the warp's first row; n0: the tile's first
// column; c_off: the product's element offset in C.  stage: this warp's EPI_WARP_BYTES.
template <int BN_>
__device__ __forceinline__ void epilogue_warp(const TcParams& p, uint32_t tacc, uint64_t c_off, uint64_t row0, uint64_t n0,
                                              int lane, uint8_t* stage) {
  const uint64_t row = row0 + lane;
  const bool row_ok = row < p.m;
  const uint64_t eb = p.out_bf16 ? 2 : 4;
  const bool staged = p.staged && ((c_off * eb) & 15) == 0;
  if (p.out_bf16) {
#pragma unroll 1
    for (int cb = 0; cb < BN_ / 32; cb += 2) {
      uint32_t v[64];
      tmem_ld32(tacc + cb * 32, v);
      tmem_ld32(tacc + cb * 32 + 32, v + 32);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      const uint64_t col = n0 + cb * 32;
      if (p.epi_mode == 2 && col + 64 <= p.rope_cols) {   // the same for the whole warp: these 64 columns are one head
        // the composition's steps (crates/tt-models/src/rope.rs:19-60 through `rope_blocks`, crates/tt-kernels/src/tensor.rs:5545-5552):
        // the product rounded to BF16 as its result would be, then fl(fl(x cos) + fl(swap(x) sin)) with swap(j) = j +- 32;
        // the store below rounds that once more to BF16, as `rope_blocks` with a BF16 result does
        const uint64_t tr = (row_ok ? row : 0) % p.rope_rows;
        const float4* co = reinterpret_cast<const float4*>(p.rope_cos + tr * p.rope_ld);
        const float4* si = reinterpret_cast<const float4*>(p.rope_sin + tr * p.rope_ld);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float4 c_lo = co[q], c_hi = co[q + 8], s_lo = si[q], s_hi = si[q + 8];
          const float cl[4] = {c_lo.x, c_lo.y, c_lo.z, c_lo.w}, ch[4] = {c_hi.x, c_hi.y, c_hi.z, c_hi.w};
          const float sl[4] = {s_lo.x, s_lo.y, s_lo.z, s_lo.w}, sh[4] = {s_hi.x, s_hi.y, s_hi.z, s_hi.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = q * 4 + e;
            const float x0 = bf16_bits_to_f32(f32_to_bf16_bits(v[j])), x1 = bf16_bits_to_f32(f32_to_bf16_bits(v[j + 32]));
            v[j] = __float_as_uint(__fadd_rn(__fmul_rn(x0, cl[e]), __fmul_rn(x1, sl[e])));
            v[j + 32] = __float_as_uint(__fadd_rn(__fmul_rn(x1, ch[e]), __fmul_rn(x0, sh[e])));
          }
        }
      }
      if (staged && col + 64 <= p.n) {          // the same for the whole warp
        uint8_t* mine = stage + lane * EPI_PITCH;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          uint4 w;
          w.x = (uint32_t)f32_to_bf16_bits(v[q * 8 + 0]) | ((uint32_t)f32_to_bf16_bits(v[q * 8 + 1]) << 16);
          w.y = (uint32_t)f32_to_bf16_bits(v[q * 8 + 2]) | ((uint32_t)f32_to_bf16_bits(v[q * 8 + 3]) << 16);
          w.z = (uint32_t)f32_to_bf16_bits(v[q * 8 + 4]) | ((uint32_t)f32_to_bf16_bits(v[q * 8 + 5]) << 16);
          w.w = (uint32_t)f32_to_bf16_bits(v[q * 8 + 6]) | ((uint32_t)f32_to_bf16_bits(v[q * 8 + 7]) << 16);
          *reinterpret_cast<uint4*>(mine + q * 16) = w;
        }
        __syncwarp();
        epi_store_rows(stage, p, (c_off + row0 * p.ldc + col) * 2, p.ldc * 2, row0, lane);
        __syncwarp();
      } else if (row_ok) {
        if (col < p.n) epi_store_direct(p, v, c_off + row * p.ldc + col, col);
        if (col + 32 < p.n) epi_store_direct(p, v + 32, c_off + row * p.ldc + col + 32, col + 32);
      }
    }
  } else {
#pragma unroll 1
    for (int cb = 0; cb < BN_ / 32; ++cb) {
      uint32_t v[32];
      tmem_ld32(tacc + cb * 32, v);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      const uint64_t col = n0 + cb * 32;
      if (staged && col + 32 <= p.n) {
        uint8_t* mine = stage + lane * EPI_PITCH;
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<uint4*>(mine + q * 16) = make_uint4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
        __syncwarp();
        epi_store_rows(stage, p, (c_off + row0 * p.ldc + col) * 4, p.ldc * 4, row0, lane);
        __syncwarp();
      } else if (row_ok && col < p.n) {
        epi_store_direct(p, v, c_off + row * p.ldc + col, col);
      }
    }
  }
}

// The gated-activation epilogue (epi_mode 1): B's columns come in groups of 256, gate columns
// 128t.. in the first half and the matching up columns in the second, so a 256-wide tile holds
// both; the tile stores 128 columns of silu(gate) * up.  The steps are the composition's
// (crates/tt-models/src/llama.rs:498: the BF16 product, then `SILU_MUL`, crates/tt-kernels/src/sfpu/ops.rs:772):
// each accumulator rounded to BF16 as the product's result would be, g * sigmoid(g) rounded, times u
// rounded, BF16.  C is [m, n / 2] with pitch ldc.
__device__ __forceinline__ uint32_t silu_mul_pair(uint32_t g0, uint32_t u0, uint32_t g1, uint32_t u1) {
  const float a0 = bf16_bits_to_f32(f32_to_bf16_bits(g0)), b0 = bf16_bits_to_f32(f32_to_bf16_bits(u0));
  const float a1 = bf16_bits_to_f32(f32_to_bf16_bits(g1)), b1 = bf16_bits_to_f32(f32_to_bf16_bits(u1));
  const float r0 = __fmul_rn(__fmul_rn(a0, sigmoid_flex(a0)), b0);
  const float r1 = __fmul_rn(__fmul_rn(a1, sigmoid_flex(a1)), b1);
  return (uint32_t)f32_to_bf16_bits(__float_as_uint(r0)) | ((uint32_t)f32_to_bf16_bits(__float_as_uint(r1)) << 16);
}

// One pass of the gated epilogue: 64 output columns, from gate chunks cb, cb+1 and up chunks 4+cb, 4+cb+1 (cb 0 or 2).
__device__ __forceinline__ void silu_mul_pass(const TcParams& p, uint32_t tacc, uint64_t row0, uint64_t tile_n, int lane,
                                              uint8_t* stage, int cb) {
  const uint64_t row = row0 + lane;
  const bool row_ok = row < p.m;
  const uint64_t out_n = p.n / 2;
  {
    uint32_t g[64], u[64];
    tmem_ld32(tacc + cb * 32, g);
    tmem_ld32(tacc + cb * 32 + 32, g + 32);
    tmem_ld32(tacc + 128 + cb * 32, u);
    tmem_ld32(tacc + 128 + cb * 32 + 32, u + 32);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    const uint64_t col = tile_n * 128 + cb * 32;  // first output column of this pass
    uint32_t w[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) w[j] = silu_mul_pair(g[2 * j], u[2 * j], g[2 * j + 1], u[2 * j + 1]);
    if (p.staged && col + 64 <= out_n) {
      uint8_t* mine = stage + lane * EPI_PITCH;
#pragma unroll
      for (int q = 0; q < 8; ++q) *reinterpret_cast<uint4*>(mine + q * 16) = make_uint4(w[q * 4], w[q * 4 + 1], w[q * 4 + 2], w[q * 4 + 3]);
      __syncwarp();
      epi_store_rows(stage, p, (row0 * p.ldc + col) * 2, p.ldc * 2, row0, lane);
      __syncwarp();
    } else if (row_ok) {
      for (int dsti = -1; dsti < p.n_more; ++dsti) {
        uint16_t* dst = (uint16_t*)(dsti < 0 ? p.c : p.c_more[dsti]) + row * p.ldc + col;
        for (int j = 0; j < 64 && col + j < out_n; ++j) dst[j] = (uint16_t)(w[j >> 1] >> ((j & 1) * 16));
      }
    }
  }
}
// Four epilogue warps a CTA: a warp takes both passes of its 32 rows.  Eight: two warps share the rows, a pass each
// (the activation's exponentials and divisions on four warps outlast a tile of nine k-blocks; on eight they do not).
__device__ __forceinline__ void epilogue_warp_silu_mul(const TcParams& p, uint32_t tacc, uint64_t row0, uint64_t tile_n,
                                                       int lane, uint8_t* stage) {
#pragma unroll 1
  for (int cb = 0; cb < 4; cb += 2) silu_mul_pass(p, tacc, row0, tile_n, lane, stage, cb);
}

// Tile order: groups of G tile rows walked column by column, so the CTAs running at one
// time share A rows and B columns in L2, and a group's A rows stay in L2 from one wave of tiles to the next.
constexpr uint32_t TILE_GROUP = 16;       // the single-CTA kernels' (128-row tiles)
constexpr uint32_t TILE_GROUP_PAIR = 8;   // the pair kernel's (256-row tiles): 8 x 9 tiles a wave of 74 clusters, and the group's eight
                                          // A row panels (34 MB at k = 8192) stay in L2 from wave to wave.  Measured at 8192^3, same box:
                                          // groups of 2 / 4 / 8 / 16 / 32 rows give 1,470 / 1,530 / 1,555 / 1,521 / 1,430 TFLOP/s
__device__ __forceinline__ void tile_coords(uint64_t t, uint32_t tiles_m, uint32_t tiles_n, uint64_t* batch,
                                            uint32_t* tm, uint32_t* tn, uint32_t G = TILE_GROUP) {
  const uint64_t per = (uint64_t)tiles_m * tiles_n;
  *batch = t / per;
  const uint32_t r = (uint32_t)(t - *batch * per);
  const uint32_t group = r / (G * tiles_n);
  const uint32_t first = group * G;
  const uint32_t rows = (tiles_m - first < G) ? (tiles_m - first) : G;
  const uint32_t in = r - group * G * tiles_n;
  *tm = first + in % rows;
  *tn = in / rows;
}

// The tile-row group of the pair kernel: B200TT_TILE_GROUP overrides (a development switch).
inline uint32_t tile_group_setting(uint32_t dflt) {
  const char* e = getenv("B200TT_TILE_GROUP");
  const long v = e ? atol(e) : 0;
  return v > 0 ? (uint32_t)v : dflt;
}

// Whether every copy of C can take 16-byte stores at every row start.
inline int epilogue_staged(const void* c, void* const* c_more, int n_more, uint64_t ldc, int out_bf16) {
  const char* e = getenv("B200TT_EPILOGUE");
  if (e && e[0] == 'd') return 0;   // "direct": stores straight from registers
  uintptr_t bits = (uintptr_t)c | (uintptr_t)(ldc * (out_bf16 ? 2 : 4));
  for (int i = 0; i < n_more; ++i) bits |= (uintptr_t)c_more[i];
  return (bits & 15) == 0;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  // a function-local static's initialiser runs once, and other threads wait for it: no caller ever
  // sees the "tried" state without the pointer
  static const EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      return (EncodeTiledFn)sym;
    return nullptr;
  }();
  return fn;
}

// A 2-D tensor map over a stored [rows, cols] matrix of 2-byte (BF16) or 4-byte (F32) elements,
// box [box_rows, 128 bytes of columns], 128-byte swizzle.
inline bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                     int elem_bytes = 2, bool atom32 = false) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {ld * (uint64_t)elem_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
            const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tc
}  // namespace b200
