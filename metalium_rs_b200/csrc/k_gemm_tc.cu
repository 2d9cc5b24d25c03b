// Tensor-core product for sm_100a: C = op(A) op(B), BF16 operands, FP32 accumulation in
// tensor memory, the accumulator rounded once to BF16 (or stored F32).
// Boundary: `Engine::matmul_dram_bf16`, `matmul_dram_batched` on BF16 buffers
// (crates/burn-tt/src/server.rs:191,229); arithmetic contract "the F32 product, rounded
// once" (crates/tt-tests/tests/step270_native_bf16.rs:462).
//
// One persistent CTA per SM walks output tiles of 128 x BN.  Warp roles:
//   warp 0      TMA producer: cp.async.bulk.tensor loads of the A and B k-blocks into a
//               ring of shared-memory stages (128-byte swizzle), one mbarrier a stage;
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) from
//               shared-memory descriptors into one of two TMEM accumulators, and
//               tcgen05.commit hands each stage back to the producer;
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (a warp owns the 32 TMEM
//               lanes of its quadrant), round, store; overlaps the next tile's mainloop.
// No load uses cluster multicast: operand reuse comes from L2 through the tile order.
// Either operand may be K-major or MN-major (the stored matrix transposed or not): the
// TMA box and the shared-memory descriptor change, the instruction stays.
// Every wait on an mbarrier is bounded; a wait that runs out sets the engine's error
// word to TIMEOUT and the kernel drains and frees its tensor memory before it returns.
#include "tc_common.cuh"
#include "pdl.cuh"

namespace b200 {
namespace {

using namespace tc;


template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TcParams p) {
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  uint8_t* epi_stage = smem + STAGES * STAGE_BYTES + 256;   // four warps' staging rows for the epilogue

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
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
  // barriers, tensor memory and descriptors are set up: from here on global memory is touched
  pdl_enter();
  const long long wait_limit = wait_limit_of(p.err);

  const uint64_t total_tiles = (uint64_t)p.tiles_m * p.tiles_n * p.batch;
  const uint32_t num_kb = (uint32_t)((p.k + BK - 1) / BK);

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (uint64_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        uint64_t b; uint32_t tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, &b, &tm, &tn);
        uint64_t a_off = 0, b_off = 0;
        if (p.batches) { a_off = p.batches[b].a_off; b_off = p.batches[b].b_off; }
        const int32_t a_r0 = (int32_t)(a_off / p.lda), a_c0 = (int32_t)(a_off % p.lda);
        const int32_t b_r0 = (int32_t)(b_off / p.ldb), b_c0 = (int32_t)(b_off % p.ldb);
        const int32_t m0 = (int32_t)(tm * BM), n0 = (int32_t)(tn * BN);
        for (uint32_t kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, wait_limit)) { ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&full[stage], STAGE_BYTES);
          const int32_t k0 = (int32_t)(kb * BK);
          if constexpr (!A_MN) {
            tma_load_2d(sa, &map_a, &full[stage], a_c0 + k0, a_r0 + m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * 8192, &map_a, &full[stage], a_c0 + m0 + j * 64, a_r0 + k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sb, &map_b, &full[stage], b_c0 + k0, b_r0 + n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * 8192, &map_b, &full[stage], b_c0 + n0 + j * 64, b_r0 + k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        atomicCAS(p.err, 0, TIMEOUT_CODE);
        *abort_flag = 1;
      }
      // Drain: every stage armed above either was consumed (its empty barrier fired) or
      // still has its copy in flight; wait (bounded) until the last armed phase of each
      // stage has landed so no copy outlives the CTA.
      for (int s = 0; s < STAGES; ++s) {
        const uint32_t ph = (s < (int)stage) ? phase : (phase ^ 1);
        // stages before `stage` were armed in the current phase, the rest in the previous
        const long long t0 = clock64();
        while (!mbar_try(&full[s], ph)) {
          if (clock64() - t0 > wait_limit) break;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                                 ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      uint32_t stage = 0, phase = 0, local = 0;
      bool ok = true;
      for (uint64_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
        const uint32_t acc = local & 1, acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, wait_limit)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (uint32_t kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, wait_limit)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t adesc = A_MN ? make_desc(sa + kk * 2048, p.mn_lbo, p.mn_sbo) : make_desc(sa + kk * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_desc(sb + kk * 2048, p.mn_lbo, p.mn_sbo) : make_desc(sb + kk * 32, 16, 1024);
            umma_bf16(d_tmem, adesc, bdesc, idesc, (kb | (uint32_t)kk) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);  // the stage is free once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&acc_full[acc]);
      }
      if (!ok) {
        atomicCAS(p.err, 0, TIMEOUT_CODE);
        *abort_flag = 1;
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const uint32_t quad = warp & 3;  // the TMEM lanes this warp may read
    uint32_t local = 0;
    bool ok = true;
    for (uint64_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
      uint64_t b; uint32_t tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, &b, &tm, &tn);
      const uint32_t acc = local & 1, acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, wait_limit)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t c_off = p.batches ? p.batches[b].c_off : 0;
      const uint64_t n0 = (uint64_t)tn * BN;
      if constexpr (BN == 256) {
        if (p.epi_mode == 1) epilogue_warp_silu_mul(p, tmem_base + ((quad * 32u) << 16) + acc * BN, (uint64_t)tm * BM + quad * 32, tn, lane, epi_stage + quad * EPI_WARP_BYTES);
        else epilogue_warp<BN>(p, tmem_base + ((quad * 32u) << 16) + acc * BN, c_off, (uint64_t)tm * BM + quad * 32, n0, lane, epi_stage + quad * EPI_WARP_BYTES);
      } else {
        epilogue_warp<BN>(p, tmem_base + ((quad * 32u) << 16) + acc * BN, c_off, (uint64_t)tm * BM + quad * 32, n0, lane, epi_stage + quad * EPI_WARP_BYTES);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
    }
    if (!ok && lane == 0) {
      atomicCAS(p.err, 0, TIMEOUT_CODE);
      *abort_flag = 1;
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// A wait nothing ends: the barrier expects bytes no copy was issued for.  The same `mbar_wait` the product
// kernels use runs out at the engine's limit and reports TIMEOUT; the barrier is invalidated before the CTA leaves.
__global__ void __launch_bounds__(32, 1) stalled_wait_kernel(int* err) {
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_expect_tx(&bar, 16);
    if (!mbar_wait(&bar, 0, &abort_word, wait_limit_of(err))) atomicCAS(err, 0, TIMEOUT_CODE);
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
  }
}

// ---- host side -----------------------------------------------------------------

template <int BN, int STAGES>
cudaError_t launch_variant(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, bool a_mn, bool b_mn,
                           unsigned grid, cudaStream_t stream) {
  constexpr size_t smem = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 1024 + 256 + EPI_BYTES;
#define TC_LAUNCH(AM, BMJ)                                                                              \
  do {                                                                                                  \
    {                                                                                                   \
      const cudaError_t e = ensure_dynamic_smem((const void*)gemm_tc_kernel<BN, STAGES, AM, BMJ>, smem); \
      if (e != cudaSuccess) return e;                                                                   \
    }                                                                                                   \
    launch_pdl(gemm_tc_kernel<BN, STAGES, AM, BMJ>, dim3(grid), dim3(NUM_THREADS), smem, stream, ma, mb, p); \
  } while (0)
  if (!a_mn && !b_mn) TC_LAUNCH(false, false);
  else if (!a_mn && b_mn) TC_LAUNCH(false, true);
  else if (a_mn && !b_mn) TC_LAUNCH(true, false);
  else TC_LAUNCH(true, true);
#undef TC_LAUNCH
  return cudaGetLastError();
}

uint32_t env_u32(const char* name, uint32_t dflt) {
  const char* s = getenv(name);
  return s ? (uint32_t)strtoul(s, nullptr, 0) : dflt;
}

}  // namespace

cudaError_t launch_stalled_wait(int* err_word, cudaStream_t stream) {
  stalled_wait_kernel<<<1, 32, 0, stream>>>(err_word);
  return cudaGetLastError();
}

bool gemm_tc_supported(const GemmArgs& g, const char** why) {
  *why = "";
  if (!g.in_bf16) { *why = "operands are not BF16"; return false; }
  if (!encode_fn()) { *why = "the driver offers no tensor-map encoder"; return false; }
  // A short M is served by a 128-row tile whose rows past M are zero-filled by TMA and masked
  // in the epilogue -- only when M is A's outer dimension; an inner extent stays >= one box.
  const bool a_mn = g.batch > 1 ? false : g.a_trans != 0;
  if (g.n < 64 || g.k < 64 || (g.m < 64 && (a_mn || g.batch > 1))) { *why = "a dimension is below 64"; return false; }
  if (g.lda % 8 || g.ldb % 8) { *why = "a row pitch is not a multiple of 16 bytes"; return false; }
  if (((uintptr_t)g.a | (uintptr_t)g.b) & 15) { *why = "an operand is not 16-byte aligned"; return false; }
  if (g.m > 0x7fffffffull || g.n > 0x7fffffffull || g.k > 0x7fffffffull) { *why = "a dimension exceeds 2^31"; return false; }
  if (g.batch > 1 && g.k % BK) { *why = "a batched product's k is not a multiple of 64"; return false; }
  return true;
}

cudaError_t launch_gemm_tc(const GemmArgs& g, const GemmBatch* batches_host, int* err_word, cudaStream_t stream, int* pair_taken) {
  if (pair_taken) *pair_taken = 0;
  if (gemm_tc2_wanted(g)) {
    const cudaError_t e2 = launch_gemm_tc2(g, err_word, stream);
    if (e2 != cudaErrorNotSupported) {
      if (pair_taken) *pair_taken = 1;
      return e2;
    }
  }
  bool a_mn = g.a_trans != 0, b_mn = g.b_trans == 0;
  if (g.batch > 1) {
    a_mn = batches_host[0].a_trans != 0;
    b_mn = batches_host[0].b_trans == 0;
    for (uint64_t i = 0; i < g.batch; ++i) {
      if ((batches_host[i].a_trans != 0) != a_mn || (batches_host[i].b_trans == 0) != b_mn) return cudaErrorNotSupported;
      if (batches_host[i].a_off % 8 || batches_host[i].b_off % 8) return cudaErrorNotSupported;
    }
  }
  // The stored matrices.  For one product they are exactly the operands; for a batched
  // call the maps span the whole buffers and each item adds its block's coordinates.
  uint64_t a_rows, a_cols, b_rows, b_cols;
  if (g.batch > 1) {
    // The engine checked that every block lies inside; rows are not known here beyond
    // that, so cover the blocks' farthest row.
    uint64_t a_last = 0, b_last = 0;
    const uint64_t ar = a_mn ? g.k : g.m, br = b_mn ? g.k : g.n;
    for (uint64_t i = 0; i < g.batch; ++i) {
      a_last = a_last > batches_host[i].a_off / g.lda + ar ? a_last : batches_host[i].a_off / g.lda + ar;
      b_last = b_last > batches_host[i].b_off / g.ldb + br ? b_last : batches_host[i].b_off / g.ldb + br;
    }
    a_rows = a_last; a_cols = g.lda; b_rows = b_last; b_cols = g.ldb;
  } else {
    a_rows = a_mn ? g.k : g.m; a_cols = a_mn ? g.m : g.k;
    b_rows = b_mn ? g.k : g.n; b_cols = b_mn ? g.n : g.k;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (g.sm_limit > 0 && g.sm_limit < sms) sms = g.sm_limit;

  const uint32_t tiles_m = (uint32_t)((g.m + BM - 1) / BM);
  // Tile width: 128, 192 or 256 columns.  A tile costs a fixed part (pipeline fill, epilogue: about
  // what sixteen 128-wide k-blocks cost) plus its k-blocks in proportion to its width; the CTAs run
  // the tiles in waves of one per SM.  Take the width with the least modelled time, so 576 columns
  // run as three 192-wide tiles in one wave instead of five 128-wide ones in two.
  const uint64_t num_kb_host = (g.k + BK - 1) / BK;
  const uint64_t nb = g.batch ? g.batch : 1;
  int bn = 128;
  double best = 1e300;
  for (int cand : {128, 192, 256}) {
    if (cand > 128 && g.n <= 128) continue;
    const uint64_t tiles = (uint64_t)tiles_m * ((g.n + cand - 1) / cand) * nb;
    const uint64_t waves = (tiles + sms - 1) / sms;
    const double cost = (double)waves * (16.0 + (double)num_kb_host * cand / 128.0);
    if (cost < best * 0.999) { best = cost; bn = cand; }
  }
  if (g.epi_mode == 1) bn = 256;   // the gated-activation epilogue reads a tile's two 128-column halves
  const uint32_t tiles_n = (uint32_t)((g.n + bn - 1) / bn);

  CUtensorMap ma, mb;
  if (!make_map(&ma, g.a, a_rows, a_cols, g.lda, a_mn ? 64 : BM)) return cudaErrorNotSupported;
  if (!make_map(&mb, g.b, b_rows, b_cols, g.ldb, b_mn ? 64 : (uint32_t)bn)) return cudaErrorNotSupported;

  TcParams p{};
  p.m = g.m; p.n = g.n; p.k = g.k;
  p.lda = g.lda; p.ldb = g.ldb; p.ldc = g.ldc;
  p.tiles_m = tiles_m; p.tiles_n = tiles_n;
  p.batch = g.batch ? g.batch : 1;
  p.batches = g.batch > 1 ? g.batches_dev : nullptr;
  p.c = g.c; p.out_bf16 = g.out_bf16; p.err = err_word;
  p.n_more = g.n_more;
  p.epi_mode = g.epi_mode;
  p.rope_cos = g.rope_cos; p.rope_sin = g.rope_sin; p.rope_rows = g.rope_rows; p.rope_ld = g.rope_ld; p.rope_cols = g.rope_cols;
  p.multicast = g.multicast;
  p.staged = epilogue_staged(g.c, g.c_more, g.n_more, g.ldc, g.out_bf16);
  for (int i = 0; i < 7; ++i) p.c_more[i] = i < g.n_more ? g.c_more[i] : nullptr;
  p.mn_lbo = env_u32("B200TT_MN_LBO", 8192);
  p.mn_sbo = env_u32("B200TT_MN_SBO", 1024);
  if (g.batch == 1 && g.batches_dev) p.batches = g.batches_dev;

  const uint64_t total = (uint64_t)tiles_m * tiles_n * p.batch;
  const unsigned grid = (unsigned)(total < (uint64_t)sms ? total : (uint64_t)sms);
  if (bn == 256) return launch_variant<256, 4>(ma, mb, p, a_mn, b_mn, grid, stream);
  if (bn == 192) return launch_variant<192, 5>(ma, mb, p, a_mn, b_mn, grid, stream);
  return launch_variant<128, 6>(ma, mb, p, a_mn, b_mn, grid, stream);
}

}  // namespace b200
