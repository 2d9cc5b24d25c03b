// F32 product on the tensor cores at F32 accuracy: each operand is split in two TF32 numbers,
// a = a_hi + a_lo (a_hi the top 19 bits of a, a_lo the top 19 bits of a - a_hi, both exactly
// representable in TF32), and C = a_lo b_hi + a_hi b_lo + a_hi b_hi is accumulated in FP32 in
// tensor memory.  The dropped a_lo b_lo term is below 2^-22 of |a||b|, so the result holds the
// 1e-5 relative bound an F32 product is held to (the reference's own F32 product is only
// TF32-grade: crates/tt-tests/tests/step11_burn.rs:15-32).
// Boundary: `Engine::matmul_dram` on F32 buffers (crates/burn-tt/src/server.rs:178).
//
// Same structure as the BF16 kernel (persistent CTAs, TMA producer warp, one MMA-issuing
// thread, four epilogue warps, two TMEM accumulators, bounded waits); a stage holds four
// tiles (A_hi, A_lo, B_hi, B_lo) of a 32-element k-block and feeds twelve
// tcgen05.mma.kind::tf32 (M 128, N 256, K 8).  No load uses cluster multicast.
#include "tc_common.cuh"

namespace b200 {
namespace {

using namespace tc;

constexpr int TBK = 32;  // F32 elements a k-block: one 128-byte swizzle row
constexpr int TBN = 256;
constexpr int TSTAGES = 2;

// hi = a with its low 13 bits cleared; lo = (a - hi) with its low 13 bits cleared.
__global__ void __launch_bounds__(256)
split_tf32_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ hi, uint32_t* __restrict__ lo, uint64_t n) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x * 4;
  for (uint64_t i = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 3 < n) {
      const uint4 v = *reinterpret_cast<const uint4*>(in + i);
      uint4 h, l;
      h.x = v.x & 0xffffe000u; h.y = v.y & 0xffffe000u; h.z = v.z & 0xffffe000u; h.w = v.w & 0xffffe000u;
      l.x = __float_as_uint(__uint_as_float(v.x) - __uint_as_float(h.x)) & 0xffffe000u;
      l.y = __float_as_uint(__uint_as_float(v.y) - __uint_as_float(h.y)) & 0xffffe000u;
      l.z = __float_as_uint(__uint_as_float(v.z) - __uint_as_float(h.z)) & 0xffffe000u;
      l.w = __float_as_uint(__uint_as_float(v.w) - __uint_as_float(h.w)) & 0xffffe000u;
      *reinterpret_cast<uint4*>(hi + i) = h;
      *reinterpret_cast<uint4*>(lo + i) = l;
    } else {
      for (uint64_t j = i; j < n; ++j) {
        const uint32_t h = in[j] & 0xffffe000u;
        hi[j] = h;
        lo[j] = __float_as_uint(__uint_as_float(in[j]) - __uint_as_float(h)) & 0xffffe000u;
      }
    }
  }
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

struct Tf32Maps { CUtensorMap a_hi, a_lo, b_hi, b_lo; };

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tf32_kernel(const __grid_constant__ Tf32Maps maps, const TcParams p) {
  constexpr uint32_t A_BYTES = BM * 128, B_BYTES = TBN * 128, STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
  constexpr uint32_t CHUNK_BYTES = TBK * 128;  // an MN-major chunk: 32 k-rows of 128 bytes (32 columns)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + TSTAGES * STAGE_BYTES);
  uint64_t* empty = full + TSTAGES;
  uint64_t* acc_full = empty + TSTAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < TSTAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const long long wait_limit = wait_limit_of(p.err);

  const uint64_t total_tiles = (uint64_t)p.tiles_m * p.tiles_n;
  const uint32_t num_kb = (uint32_t)((p.k + TBK - 1) / TBK);

  if (warp == 0) {
    if (lane == 0) {  // ---------------- TMA producer ----------------
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (uint64_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        uint64_t b; uint32_t tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, &b, &tm, &tn);
        const int32_t m0 = (int32_t)(tm * BM), n0 = (int32_t)(tn * TBN);
        for (uint32_t kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, wait_limit)) { ok = false; break; }
          uint8_t* sah = smem + stage * STAGE_BYTES;
          uint8_t* sal = sah + A_BYTES;
          uint8_t* sbh = sal + A_BYTES;
          uint8_t* sbl = sbh + B_BYTES;
          mbar_expect_tx(&full[stage], STAGE_BYTES);
          const int32_t k0 = (int32_t)(kb * TBK);
          if constexpr (!A_MN) {
            tma_load_2d(sah, &maps.a_hi, &full[stage], k0, m0);
            tma_load_2d(sal, &maps.a_lo, &full[stage], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 32; ++j) {
              tma_load_2d(sah + j * CHUNK_BYTES, &maps.a_hi, &full[stage], m0 + j * 32, k0);
              tma_load_2d(sal + j * CHUNK_BYTES, &maps.a_lo, &full[stage], m0 + j * 32, k0);
            }
          }
          if constexpr (!B_MN) {
            tma_load_2d(sbh, &maps.b_hi, &full[stage], k0, n0);
            tma_load_2d(sbl, &maps.b_lo, &full[stage], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < TBN / 32; ++j) {
              tma_load_2d(sbh + j * CHUNK_BYTES, &maps.b_hi, &full[stage], n0 + j * 32, k0);
              tma_load_2d(sbl + j * CHUNK_BYTES, &maps.b_lo, &full[stage], n0 + j * 32, k0);
            }
          }
          if (++stage == TSTAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) { atomicCAS(p.err, 0, TIMEOUT_CODE); *abort_flag = 1; }
      for (int s = 0; s < TSTAGES; ++s) {  // drain: no copy may outlive the CTA
        const uint32_t ph = (s < (int)stage) ? phase : (phase ^ 1);
        const long long t0 = clock64();
        while (!mbar_try(&full[s], ph)) { if (clock64() - t0 > wait_limit) break; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---------------- MMA issuer ----------------
      // c_format F32 (1 << 4), a/b format TF32 (2 << 7, 2 << 10), majors, N >> 3, M >> 4
      constexpr uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                                 ((uint32_t)(TBN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      uint32_t stage = 0, phase = 0, local = 0;
      bool ok = true;
      for (uint64_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
        const uint32_t acc = local & 1, acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, wait_limit)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + acc * TBN;
        for (uint32_t kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, wait_limit)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sah = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sal = sah + A_BYTES, sbh = sal + A_BYTES, sbl = sbh + B_BYTES;
#pragma unroll
          for (int kk = 0; kk < TBK / 8; ++kk) {
            // K-major: 32 bytes a step along the row.  MN-major (128-byte swizzle with 32-byte atoms, four
            // k-rows an atom, 512 bytes between atoms): 8 k-rows (1 KB) a step
            const uint32_t ao = A_MN ? kk * 1024 : kk * 32, bo = B_MN ? kk * 1024 : kk * 32;
            const uint64_t ah = A_MN ? make_desc(sah + ao, CHUNK_BYTES, 512, 1) : make_desc(sah + ao, 16, 1024);
            const uint64_t al = A_MN ? make_desc(sal + ao, CHUNK_BYTES, 512, 1) : make_desc(sal + ao, 16, 1024);
            const uint64_t bh = B_MN ? make_desc(sbh + bo, CHUNK_BYTES, 512, 1) : make_desc(sbh + bo, 16, 1024);
            const uint64_t bl = B_MN ? make_desc(sbl + bo, CHUNK_BYTES, 512, 1) : make_desc(sbl + bo, 16, 1024);
            umma_tf32(d_tmem, al, bh, idesc, (kb | (uint32_t)kk) != 0 ? 1u : 0u);  // small terms first
            umma_tf32(d_tmem, ah, bl, idesc, 1u);
            umma_tf32(d_tmem, ah, bh, idesc, 1u);
          }
          umma_commit(&empty[stage]);
          if (++stage == TSTAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&acc_full[acc]);
      }
      if (!ok) { atomicCAS(p.err, 0, TIMEOUT_CODE); *abort_flag = 1; }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const uint32_t quad = warp & 3;
    uint32_t local = 0;
    bool ok = true;
    for (uint64_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
      uint64_t b; uint32_t tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, &b, &tm, &tn);
      const uint32_t acc = local & 1, acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, wait_limit)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t row = (uint64_t)tm * BM + quad * 32 + lane;
      const uint64_t n0 = (uint64_t)tn * TBN;
      const bool row_ok = row < p.m;
#pragma unroll 1
      for (int cb = 0; cb < TBN / 32; ++cb) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((quad * 32u) << 16) + acc * TBN + cb * 32, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const uint64_t col = n0 + cb * 32;
        if (row_ok && col < p.n) {
          const uint64_t o = row * p.ldc + col;
          if (p.out_bf16) {
            uint16_t* dst = (uint16_t*)p.c + o;
            for (int j = 0; j < 32 && col + j < p.n; ++j) dst[j] = f32_to_bf16_bits(v[j]);
          } else {
            uint32_t* dst = (uint32_t*)p.c + o;
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
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
    }
    if (!ok && lane == 0) { atomicCAS(p.err, 0, TIMEOUT_CODE); *abort_flag = 1; }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace

bool gemm_tf32_supported(const GemmArgs& g, const char** why) {
  *why = "";
  if (g.in_bf16) { *why = "operands are not F32"; return false; }
  if (g.batch > 1) { *why = "batched F32 products take the SIMT kernel"; return false; }
  if (!encode_fn()) { *why = "the driver offers no tensor-map encoder"; return false; }
  if (g.m < 128 || g.n < 128 || g.k < 32) { *why = "a dimension is too small to pay for the split"; return false; }
  if (g.lda % 4 || g.ldb % 4) { *why = "a row pitch is not a multiple of 16 bytes"; return false; }
  if (((uintptr_t)g.a | (uintptr_t)g.b) & 15) { *why = "an operand is not 16-byte aligned"; return false; }
  if (g.m > 0x7fffffffull || g.n > 0x7fffffffull || g.k > 0x7fffffffull) { *why = "a dimension exceeds 2^31"; return false; }
  return true;
}

// a_hi .. b_lo: scratch of the operands' sizes (rows * ld floats each), owned by the caller.
cudaError_t launch_gemm_tf32(const GemmArgs& g, void* a_hi, void* a_lo, void* b_hi, void* b_lo, int* err_word,
                             cudaStream_t stream) {
  const bool a_mn = g.a_trans != 0, b_mn = g.b_trans == 0;
  const uint64_t a_rows = a_mn ? g.k : g.m, a_cols = a_mn ? g.m : g.k;
  const uint64_t b_rows = b_mn ? g.k : g.n, b_cols = b_mn ? g.n : g.k;
  // the stored operands end at their last row's last column (a block of a wider matrix does not own the rest of that row)
  const uint64_t na = (a_rows - 1) * g.lda + a_cols, nb = (b_rows - 1) * g.ldb + b_cols;
  auto grid_for = [](uint64_t n) { uint64_t b = (n / 4 + 255) / 256 + 1; return (unsigned)(b < 148ull * 16 ? b : 148ull * 16); };
  split_tf32_kernel<<<grid_for(na), 256, 0, stream>>>((const uint32_t*)g.a, (uint32_t*)a_hi, (uint32_t*)a_lo, na);
  split_tf32_kernel<<<grid_for(nb), 256, 0, stream>>>((const uint32_t*)g.b, (uint32_t*)b_hi, (uint32_t*)b_lo, nb);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;

  Tf32Maps maps;
  if (!make_map(&maps.a_hi, a_hi, a_rows, a_cols, g.lda, a_mn ? TBK : BM, 4, a_mn) ||
      !make_map(&maps.a_lo, a_lo, a_rows, a_cols, g.lda, a_mn ? TBK : BM, 4, a_mn) ||
      !make_map(&maps.b_hi, b_hi, b_rows, b_cols, g.ldb, b_mn ? TBK : TBN, 4, b_mn) ||
      !make_map(&maps.b_lo, b_lo, b_rows, b_cols, g.ldb, b_mn ? TBK : TBN, 4, b_mn))
    return cudaErrorNotSupported;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  TcParams p{};
  p.m = g.m; p.n = g.n; p.k = g.k;
  p.lda = g.lda; p.ldb = g.ldb; p.ldc = g.ldc;
  p.tiles_m = (uint32_t)((g.m + BM - 1) / BM);
  p.tiles_n = (uint32_t)((g.n + TBN - 1) / TBN);
  p.batch = 1; p.batches = nullptr;
  p.c = g.c; p.out_bf16 = g.out_bf16; p.err = err_word;
  const uint64_t total = (uint64_t)p.tiles_m * p.tiles_n;
  const unsigned grid = (unsigned)(total < (uint64_t)sms ? total : (uint64_t)sms);
  constexpr size_t smem = (size_t)TSTAGES * (2 * BM * 128 + 2 * TBN * 128) + 1024 + 256;
#define TF_LAUNCH(AM, BMJ)                                                                            \
  do {                                                                                                \
    e = ensure_dynamic_smem((const void*)gemm_tf32_kernel<AM, BMJ>, smem);                            \
    if (e != cudaSuccess) return e;                                                                   \
    gemm_tf32_kernel<AM, BMJ><<<grid, NUM_THREADS, smem, stream>>>(maps, p);                          \
  } while (0)
  if (!a_mn && !b_mn) TF_LAUNCH(false, false);
  else if (!a_mn && b_mn) TF_LAUNCH(false, true);
  else if (a_mn && !b_mn) TF_LAUNCH(true, false);
  else TF_LAUNCH(true, true);
#undef TF_LAUNCH
  return cudaGetLastError();
}

}  // namespace b200
