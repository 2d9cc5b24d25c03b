// BF16 product on CTA pairs: tcgen05.mma.cta_group::2, one 256 x 256 output tile a pair.
// Same contract as k_gemm_tc.cu (`Engine::matmul_dram_bf16`, crates/burn-tt/src/server.rs:191);
// the engine takes this kernel for one large product and the single-CTA kernel otherwise.
//
// The two CTAs of a cluster each hold 128 rows of A and 128 columns of B for a k-block
// (32 KB a stage instead of 48 KB, so six stages fit and the operand traffic from L2 into an SM
// drops by a third).  The even CTA (the leader) issues every MMA; the instruction reads both
// CTAs' shared memory and writes both CTAs' tensor memory (each CTA ends with its own 128 rows
// of the 256 x 256 tile).  Barriers:
//   full[s]   lives in the leader; both CTAs' TMA loads complete their bytes on it
//             (cp.async.bulk.tensor ... .cta_group::2, no multicast);
//   empty[s]  one in each CTA; the leader's tcgen05.commit arrives on both;
//   acc_full  one in each CTA, also signalled by the leader's commit;
//   acc_empty lives in the leader; the eight epilogue warps of the pair arrive on it.
// Every wait is bounded; on a timeout the engine's error word is set to TIMEOUT and every
// thread still reaches the closing cluster barrier, after which tensor memory is freed.
#include <cooperative_groups.h>

#include "tc_common.cuh"
#include "pdl.cuh"

namespace b200 {
namespace {

using namespace tc;

constexpr int P_BN = 256;     // tile columns of the pair
constexpr int P_HALF = 128;   // B columns a CTA loads
constexpr int P_STAGES = 6;       // with four epilogue warps a CTA; five with eight (their staging rows take a stage's room)

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into this CTA's shared memory; the bytes complete on the barrier at `bar_cluster_addr`
// (the leader's), which .cta_group::2 allows to lie in the peer CTA.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on the barrier at the same offset in both CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

// EW: epilogue warps a CTA.  Four for a plain product; eight for the gated epilogue (`epi_mode` 1), whose activation
// is too much arithmetic for four warps to finish under the next tile's mainloop when k is short.
template <bool A_MN, bool B_MN, int EW = 4>
__global__ void __launch_bounds__(64 + EW * 32, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TcParams p) {
  constexpr int P_STAGES = EW == 8 ? 5 : 6;
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = P_HALF * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + P_STAGES * STAGE_BYTES);
  uint64_t* empty = full + P_STAGES;
  uint64_t* acc_full = empty + P_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  uint8_t* epi_stage = smem + P_STAGES * STAGE_BYTES + 256;   // four warps' staging rows for the epilogue

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();   // 0: leader
  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 2 * EW); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  cluster_sync_all();  // both CTAs' barriers exist before anything remote touches them
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  // barriers, tensor memory and descriptors are set up: from here on global memory is touched
  pdl_enter();
  const long long wait_limit = wait_limit_of(p.err);

  const uint64_t total_tiles = (uint64_t)p.tiles_m * p.tiles_n;  // tiles of 256 x 256
  const uint32_t num_kb = (uint32_t)((p.k + BK - 1) / BK);
  const uint64_t cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;

  if (warp == 0) {
    if (lane == 0) {  // ---------------- TMA producer (both CTAs) ----------------
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (uint64_t t = cluster_id; t < total_tiles && ok; t += n_clusters) {
        uint64_t b; uint32_t tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, &b, &tm, &tn, p.group);
        const int32_t m0 = (int32_t)(tm * 256 + rank * BM), n0 = (int32_t)(tn * P_BN + rank * P_HALF);
        for (uint32_t kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, wait_limit)) { ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          if (rank == 0) mbar_expect_tx(&full[stage], 2 * STAGE_BYTES);  // the pair's bytes
          const uint32_t bar = map_to_rank(smem_u32(&full[stage]), 0);
          const int32_t k0 = (int32_t)(kb * BK);
          if constexpr (!A_MN) {
            tma_load_2d_pair(sa, &map_a, bar, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * 8192, &map_a, bar, m0 + j * 64, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(sb, &map_b, bar, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < P_HALF / 64; ++j) tma_load_2d_pair(sb + j * 8192, &map_b, bar, n0 + j * 64, k0);
          }
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        atomicCAS(p.err, 0, TIMEOUT_CODE);
        *abort_flag = 1;
        const long long t0 = clock64();       // let copies already issued land before the CTA leaves
        while (clock64() - t0 < 2000000ll) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {  // ---------------- MMA issuer (leader only) ----------------
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                                 ((uint32_t)(P_BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
      uint32_t stage = 0, phase = 0, local = 0;
      bool ok = true;
      for (uint64_t t = cluster_id; t < total_tiles && ok; t += n_clusters, ++local) {
        const uint32_t acc = local & 1, acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, wait_limit)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + acc * P_BN;
        for (uint32_t kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, wait_limit)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t adesc = A_MN ? make_desc(sa + kk * 2048, 8192, 1024) : make_desc(sa + kk * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_desc(sb + kk * 2048, 8192, 1024) : make_desc(sb + kk * 32, 16, 1024);
            umma_bf16_pair(d_tmem, adesc, bdesc, idesc, (kb | (uint32_t)kk) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty[stage]);
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(&acc_full[acc]);
      }
      if (!ok) { atomicCAS(p.err, 0, TIMEOUT_CODE); *abort_flag = 1; }
    }
  } else {
    // ---------------- epilogue (warps 2.. of both CTAs; a warp reads the tensor-memory lanes of its quadrant) ----------------
    const uint32_t quad = warp & 3, ew = (uint32_t)warp - 2;
    uint32_t local = 0;
    bool ok = true;
    for (uint64_t t = cluster_id; t < total_tiles && ok; t += n_clusters, ++local) {
      uint64_t b; uint32_t tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, &b, &tm, &tn, p.group);
      const uint32_t acc = local & 1, acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, wait_limit)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t n0 = (uint64_t)tn * P_BN;
      if constexpr (EW == 8) {   // the gated epilogue on eight warps: warps 2..5 take the first 64 output columns, 6..9 the others
        silu_mul_pass(p, tmem_base + ((quad * 32u) << 16) + acc * P_BN, (uint64_t)tm * 256 + rank * BM + quad * 32, tn, lane,
                      epi_stage + ew * EPI_WARP_BYTES, (int)(ew >> 2) * 2);
      } else {
        if (p.epi_mode == 1) epilogue_warp_silu_mul(p, tmem_base + ((quad * 32u) << 16) + acc * P_BN, (uint64_t)tm * 256 + rank * BM + quad * 32, tn, lane, epi_stage + ew * EPI_WARP_BYTES);
        else epilogue_warp<P_BN>(p, tmem_base + ((quad * 32u) << 16) + acc * P_BN, 0, (uint64_t)tm * 256 + rank * BM + quad * 32, n0, lane, epi_stage + ew * EPI_WARP_BYTES);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(map_to_rank(smem_u32(&acc_empty[acc]), 0));
    }
    if (!ok && lane == 0) { atomicCAS(p.err, 0, TIMEOUT_CODE); *abort_flag = 1; }
  }

  // No CTA may leave (or free tensor memory) while its peer can still read its shared memory,
  // write its tensor memory or signal its barriers.
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster_sync_all();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace

// Whether the pair kernel should take this product: one product whose 256 x 256 tiles fill the
// clusters at least once.  B200TT_PAIR=0 / 1 overrides (development switch).
constexpr bool kPairByDefault = true;

bool gemm_tc2_wanted(const GemmArgs& g) {
  static int force = -2;
  if (force == -2) { const char* e = getenv("B200TT_PAIR"); force = e ? atoi(e) : -1; }
  if (g.batch > 1 || g.m < 256 || g.n < 256 || g.k < 64) return false;
  if (force == 0) return false;
  if (force == 1) return true;
  return kPairByDefault && ((g.m + 255) / 256) * ((g.n + 255) / 256) >= 64;
}

cudaError_t launch_gemm_tc2(const GemmArgs& g, int* err_word, cudaStream_t stream) {
  const bool a_mn = g.a_trans != 0, b_mn = g.b_trans == 0;
  const uint64_t a_rows = a_mn ? g.k : g.m, a_cols = a_mn ? g.m : g.k;
  const uint64_t b_rows = b_mn ? g.k : g.n, b_cols = b_mn ? g.n : g.k;
  CUtensorMap ma, mb;
  if (!make_map(&ma, g.a, a_rows, a_cols, g.lda, a_mn ? 64 : BM)) return cudaErrorNotSupported;
  if (!make_map(&mb, g.b, b_rows, b_cols, g.ldb, b_mn ? 64 : P_HALF)) return cudaErrorNotSupported;
  TcParams p{};
  p.m = g.m; p.n = g.n; p.k = g.k;
  p.lda = g.lda; p.ldb = g.ldb; p.ldc = g.ldc;
  p.tiles_m = (uint32_t)((g.m + 255) / 256);
  p.tiles_n = (uint32_t)((g.n + P_BN - 1) / P_BN);
  p.batch = 1; p.batches = nullptr;
  p.c = g.c; p.out_bf16 = g.out_bf16; p.err = err_word;
  p.n_more = g.n_more;
  p.epi_mode = g.epi_mode;
  p.rope_cos = g.rope_cos; p.rope_sin = g.rope_sin; p.rope_rows = g.rope_rows; p.rope_ld = g.rope_ld; p.rope_cols = g.rope_cols;
  p.multicast = g.multicast;
  p.group = tile_group_setting(TILE_GROUP_PAIR);
  p.staged = epilogue_staged(g.c, g.c_more, g.n_more, g.ldc, g.out_bf16);
  for (int i = 0; i < 7; ++i) p.c_more[i] = i < g.n_more ? g.c_more[i] : nullptr;
  // the gated epilogue takes eight epilogue warps a CTA and five stages (B200TT_SILU_WARPS=4: the four-warp form, for comparison)
  static const bool eight = []() { const char* e = getenv("B200TT_SILU_WARPS"); return !(e && e[0] == '4'); }();
  const bool ew8 = g.epi_mode == 1 && eight;
  const size_t smem = ew8 ? (size_t)5 * (BM * BK * 2 + P_HALF * BK * 2) + 1024 + 256 + 2 * EPI_BYTES
                          : (size_t)P_STAGES * (BM * BK * 2 + P_HALF * BK * 2) + 1024 + 256 + EPI_BYTES;
  const uint64_t total = (uint64_t)p.tiles_m * p.tiles_n;

  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(ew8 ? 64 + 8 * 32 : NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaSuccess;
#define TC2_LAUNCH(AM, BMJ, EWJ)                                                                      \
  do {                                                                                                \
    int clusters = 0;   /* clusters of this kernel one device runs at a time: asked once a device */ \
    e = ensure_dynamic_smem((const void*)gemm_tc2_kernel<AM, BMJ, EWJ>, smem);                        \
    if (e != cudaSuccess) return e;                                                                   \
    if (!device_value_get((const void*)gemm_tc2_kernel<AM, BMJ, EWJ>, &clusters)) {                   \
      cfg.gridDim = dim3(148, 1, 1);                                                                  \
      int n = 0;                                                                                      \
      e = cudaOccupancyMaxActiveClusters(&n, gemm_tc2_kernel<AM, BMJ, EWJ>, &cfg);                    \
      if (e != cudaSuccess || n <= 0) { cudaGetLastError(); return cudaErrorNotSupported; }           \
      clusters = n;                                                                                   \
      device_value_set((const void*)gemm_tc2_kernel<AM, BMJ, EWJ>, n);                                \
    }                                                                                                 \
    uint64_t use = total < (uint64_t)clusters ? total : (uint64_t)clusters;                           \
    if (g.sm_limit > 1 && use > (uint64_t)(g.sm_limit / 2)) use = (uint64_t)(g.sm_limit / 2);        \
    cfg.gridDim = dim3((unsigned)(2 * use), 1, 1);                                                    \
    e = cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<AM, BMJ, EWJ>, ma, mb, p);                           \
  } while (0)
  if (ew8) {
    if (!a_mn && !b_mn) TC2_LAUNCH(false, false, 8);
    else if (!a_mn && b_mn) TC2_LAUNCH(false, true, 8);
    else if (a_mn && !b_mn) TC2_LAUNCH(true, false, 8);
    else TC2_LAUNCH(true, true, 8);
  } else {
    if (!a_mn && !b_mn) TC2_LAUNCH(false, false, 4);
    else if (!a_mn && b_mn) TC2_LAUNCH(false, true, 4);
    else if (a_mn && !b_mn) TC2_LAUNCH(true, false, 4);
    else TC2_LAUNCH(true, true, 4);
  }
#undef TC2_LAUNCH
  return e;
}

}  // namespace b200
