// Fused attention over whole sequences on the tensor cores: for each (batch, head) block
//     O = softmax(scale * Q K^T [causal]) V,   Q [sq, d], K [sk, d], V [sk, d]  (BF16), O BF16,
// with the scores and probabilities never written to memory.  It replaces, for prefill-shaped
// work, the reference's composed attention (crates/burn-tt/src/ops.rs:4825 `padded_attention`:
// a batched Q K^T, `SCALE_MASK_FILL`, the row softmax, a batched P V), whose [rows, sk] F32 scores
// are the largest memory cost of the path.
//
// One CTA owns 128 query rows of one block and walks the key tiles (128 keys) ONCE, with a running reference for
// the softmax: S = Q K_j^T on tcgen05 into TMEM; a softmax warp reads its 32 rows (a thread a query row, all 128 keys
// of the tile), P = exp2(S' - ref) rounded to BF16 into shared memory (the 128-byte-swizzled K-major layout the MMA
// reads), O += P V_j accumulated in TMEM, the row sum kept in registers; at the end O / sum is written as BF16.
// The reference is the largest scaled score seen so far, but it is only moved -- and O and the sum rescaled by
// exp2(old - new) -- when a tile's maximum exceeds it by more than 8 (a factor 256: P then stays within BF16's and
// the sum within F32's range), so after the first tiles O is almost never touched; the result is exact whatever the
// reference, since O and the sum carry the same one.  (The kernel once took two passes, the first only for the row
// maxima: Q K^T twice, 1.5x the tensor-core work of this form.)
// Warp 0 lane 0 issues the TMA loads, warp 1 lane 0 the MMAs, warps 2-9 are the softmax: a query row is a TMEM lane,
// a warp reads the lanes of its quadrant, and two threads share a row (keys 0-63 and 64-127 of a tile; they exchange
// their halves' maxima through shared memory every tile and their sums at the end).  S is double-buffered in TMEM so the next tile's product runs under this
// tile's exponentials.  The rescale of O (tcgen05.ld, multiply, tcgen05.st by the row's thread) happens between the
// product with V of the tile before (waited for through that tile's p_empty) and the signal that lets the next one start.
// P is double-buffered in shared memory, so a tile's exponentials run while the tile before is multiplied by V.
// Every wait is bounded; a wait that runs out sets the engine's error word to TIMEOUT and the CTA
// leaves in order (copies drained, TMEM freed).
// sq and sk need not be whole tiles (the reference pads ragged heads, ops.rs:4838-4842): the last query tile's rows
// past sq are computed and not stored, the last key tile's keys past sk are masked by index like the keys a causal
// row may not see.  The rows a tail tile reads past its block are whatever follows in the buffer (zeros past its end):
// scores of such keys never enter a maximum or a sum, and such value rows are weighted by exact zeros.
#include <cfloat>
#include <cstdint>
#include <cuda_runtime.h>

#include "tc_common.cuh"
#include "pdl.cuh"

namespace b200 {
namespace {

using namespace tc;

constexpr uint32_t TILE_BYTES = 128 * 64 * 2;   // a [128 rows, 64 columns] BF16 box
constexpr uint32_t P_BYTES = 2 * TILE_BYTES;    // [128 rows, 128 keys]
constexpr int ATTN_THREADS = 320;               // 10 warps: TMA, MMA, 8 softmax
constexpr int SOFTMAX_THREADS = 256;
constexpr float REF_STEP = 8.0f;                // the reference moves when a tile's maximum exceeds it by more than this (log2 units)

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
        "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}

struct AttnTcParams {
  const AttnBlockDev* items;
  uint32_t q_tiles, k_tiles, n_items;
  uint32_t sq, sk;              // rows of a block's Q and of its K and V (the last tiles may be partial)
  int32_t causal, causal_off;   // a query i sees keys j <= i + causal_off
  float scale_log2;             // scale * log2(e)
  int32_t spin;                 // the S -> P -> O hand-offs wait by polling
  uint16_t* out;
  uint64_t o_ld;
  int* err;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// a in the low half, b in the high half, round to nearest even
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(b), "f"(a));
  return d;
}

template <int D>
__global__ void __launch_bounds__(ATTN_THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const AttnTcParams p) {
  constexpr int CH = D / 64;                       // 64-column chunks of a row of Q, K or V
  constexpr int KS = D == 64 ? 3 : 2;              // stages of K and of V
  constexpr uint32_t OP_BYTES = CH * TILE_BYTES;   // one Q, K or V tile
  constexpr uint32_t S_COLS = 128, O_COL = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + OP_BYTES;
  uint8_t* sV = sK + KS * OP_BYTES;
  uint8_t* sP = sV + KS * OP_BYTES;
  uint64_t* q_full = (uint64_t*)(sP + 2 * P_BYTES);   // P is double-buffered: a tile's probabilities are written while the tile before is multiplied
  uint64_t* k_full = q_full + 1;
  uint64_t* k_empty = k_full + KS;
  uint64_t* v_full = k_empty + KS;
  uint64_t* v_empty = v_full + KS;
  uint64_t* s_full = v_empty + KS;
  uint64_t* s_empty = s_full + 2;
  uint64_t* p_full = s_empty + 2;
  uint64_t* p_empty = p_full + 2;
  uint64_t* o_full = p_empty + 2;
  uint32_t* tmem_slot = (uint32_t*)(o_full + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  float* xmax = (float*)(sP + 2 * P_BYTES + 256);   // [2 halves][128 rows]: the halves' maxima of a tile; at the end their row sums
  long long wait_limit = WAIT_CYCLES;   // the engine's limit, read once global memory may be touched
  auto hand_off = [&](uint64_t* bar, uint32_t parity) -> bool {   // a wait on the chain S -> P -> O
    return p.spin ? mbar_wait_spin(bar, parity, abort_flag, wait_limit) : mbar_wait(bar, parity, abort_flag, wait_limit);
  };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KS; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&s_full[b], 1); mbar_init(&s_empty[b], SOFTMAX_THREADS / 32); }   // a lane a warp arrives
    for (int b = 0; b < 2; ++b) { mbar_init(&p_full[b], SOFTMAX_THREADS / 32); mbar_init(&p_empty[b], 1); }
    mbar_init(o_full, 1);
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
  wait_limit = wait_limit_of(p.err);

  // Heaviest work first: under a causal mask a block's last query tile has the most keys, so the grid
  // runs every block's last tile, then every block's tile before it, ... (the block index is the
  // fastest-varying one), and the short tiles fill the SMs the long ones leave.
  // Without a mask every tile costs the same and a block's query tiles run side by side, sharing its
  // K and V in L2.
  const uint32_t qt = p.causal ? p.q_tiles - 1 - blockIdx.x / p.n_items : blockIdx.x % p.q_tiles;
  const AttnBlockDev it = p.items[p.causal ? blockIdx.x % p.n_items : blockIdx.x / p.q_tiles];
  const int32_t i0 = (int32_t)(qt * 128);
  uint32_t nk = p.k_tiles;
  if (p.causal) {
    const int32_t last = i0 + 127 + p.causal_off;      // the last key any row of this tile sees (>= 0)
    const uint32_t lim = (uint32_t)(last / 128) + 1;
    nk = lim < nk ? lim : nk;
  }

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(q_full, OP_BYTES);
#pragma unroll
      for (int c = 0; c < CH; ++c) tma_load_2d(sQ + c * TILE_BYTES, &map_q, q_full, it.q_c + c * 64, it.q_r + i0);
      uint32_t ks = 0, kph = 0, vs = 0, vph = 0;
      for (uint32_t j = 0; j < nk; ++j) {
        if (!mbar_wait(&k_empty[ks], kph ^ 1, abort_flag, wait_limit)) { ok = false; break; }
        mbar_expect_tx(&k_full[ks], OP_BYTES);
#pragma unroll
        for (int c = 0; c < CH; ++c)
          tma_load_2d(sK + ks * OP_BYTES + c * TILE_BYTES, &map_k, &k_full[ks], it.k_c + c * 64, it.k_r + (int32_t)(j * 128));
        if (++ks == KS) { ks = 0; kph ^= 1; }
        if (!mbar_wait(&v_empty[vs], vph ^ 1, abort_flag, wait_limit)) { ok = false; break; }
        mbar_expect_tx(&v_full[vs], OP_BYTES);
#pragma unroll
        for (int c = 0; c < CH; ++c)
          tma_load_2d(sV + vs * OP_BYTES + c * TILE_BYTES, &map_v, &v_full[vs], it.v_c + c * 64, it.v_r + (int32_t)(j * 128));
        if (++vs == KS) { vs = 0; vph ^= 1; }
      }
      if (!ok) {
        atomicCAS(p.err, 0, TIMEOUT_CODE);
        *abort_flag = 1;
      }
      // Drain: no copy may outlive the CTA.  Stages before the cursor were armed in the current
      // phase, the rest in the previous one (or never: their barrier is then already past it).
      {
        const long long t0 = clock64();
        while (!mbar_try(q_full, 0)) { if (clock64() - t0 > wait_limit) break; }
      }
      for (int s = 0; s < KS; ++s) {
        const uint32_t kp = (s < (int)ks) ? kph : (kph ^ 1);
        const uint32_t vp = (s < (int)vs) ? vph : (vph ^ 1);
        const long long t0 = clock64();
        while (!mbar_try(&k_full[s], kp)) { if (clock64() - t0 > wait_limit) break; }
        while (!mbar_try(&v_full[s], vp)) { if (clock64() - t0 > wait_limit) break; }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // kind::f16: F32 accumulate (bit 4), BF16 A and B (bits 7, 10), B MN-major for P V (bit 16)
      constexpr uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      constexpr uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      bool ok = mbar_wait(q_full, 0, abort_flag, wait_limit);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t ks = 0, kph = 0, vs = 0, vph = 0, t = 0;
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto issue_qk = [&]() -> bool {
        const uint32_t buf = t & 1, sph = (t >> 1) & 1;
        if (!hand_off(&s_empty[buf], sph ^ 1)) return false;
        if (!mbar_wait(&k_full[ks], kph, abort_flag, wait_limit)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t k_addr = smem_u32(sK + ks * OP_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / UMMA_K; ++kk) {
          const uint32_t off = (kk / 4) * TILE_BYTES + (kk % 4) * 32;
          umma_bf16(tmem_base + buf * S_COLS, make_desc(q_addr + off, 16, 1024), make_desc(k_addr + off, 16, 1024), idesc_qk, kk != 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[ks]);
        umma_commit(&s_full[buf]);
        if (++ks == KS) { ks = 0; kph ^= 1; }
        ++t;
        return true;
      };
      if (ok) ok = issue_qk();                                           // tile 0's scores
      for (uint32_t j = 0; j < nk && ok; ++j) {
        if (j + 1 < nk) { ok = issue_qk(); if (!ok) break; }             // the next scores run under these exponentials
        const uint32_t pb = j & 1, pph = (j >> 1) & 1;
        if (!hand_off(&p_full[pb], pph)) { ok = false; break; }
        if (!mbar_wait(&v_full[vs], vph, abort_flag, wait_limit)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t v_addr = smem_u32(sV + vs * OP_BYTES);
#pragma unroll
        for (int kk = 0; kk < 128 / UMMA_K; ++kk) {
          const uint64_t adesc = make_desc(p_addr + pb * P_BYTES + (kk / 4) * TILE_BYTES + (kk % 4) * 32, 16, 1024);
          const uint64_t bdesc = make_desc(v_addr + kk * 2048, TILE_BYTES, 1024);   // 64-column chunks a tile apart
          umma_bf16(tmem_base + O_COL, adesc, bdesc, idesc_pv, (j | (uint32_t)kk) != 0 ? 1u : 0u);
        }
        umma_commit(&v_empty[vs]);
        umma_commit(&p_empty[pb]);
        if (++vs == KS) { vs = 0; vph ^= 1; }
      }
      if (ok) umma_commit(o_full);
      if (!ok) {
        atomicCAS(p.err, 0, TIMEOUT_CODE);
        *abort_flag = 1;
      }
    }
  } else {
    // ---------------- softmax and epilogue (warps 2..9): two threads a query row ----------------
    // A warp reads the TMEM lanes of its quadrant; warps 2-5 take keys 0-63 of a tile and the first half of O's
    // columns, warps 6-9 keys 64-127 and the second half.  The two threads of a row exchange their halves' maxima
    // through shared memory every tile (one named barrier), so both move the row's reference alike.
    const uint32_t quad = warp & 3;
    const uint32_t half = (uint32_t)(warp - 2) >> 2;
    const uint32_t row = quad * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((quad * 32u) << 16);
    const int32_t qi = i0 + (int32_t)row;
    const int32_t seen = p.causal ? qi + p.causal_off : 0x7fffffff;
    const int32_t last_key = seen < (int32_t)p.sk - 1 ? seen : (int32_t)p.sk - 1;   // no key past the block's
    constexpr int OC = D / 2;                       // this thread's columns of O
    bool ok = true;
    float ref = -INFINITY;                          // the row's reference: a scaled score (log2 units), -inf until a key is seen
    float sum = 0.f;                                // this thread's keys only
    for (uint32_t j = 0; j < nk && ok; ++j) {
      const uint32_t buf = j & 1, sph = (j >> 1) & 1;
      if (!hand_off(&s_full[buf], sph)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int32_t key0 = (int32_t)(j * 128 + half * 64);
      const bool edge = key0 + 63 > last_key;        // only a diagonal or tail tile needs the mask
      uint32_t v[64];
      tmem_ld32(lane_addr + buf * S_COLS + half * 64, v);
      tmem_ld32(lane_addr + buf * S_COLS + half * 64 + 32, v + 32);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[buf]);     // one arrival a warp: the scores are in registers
      if (edge) {                                    // a key this row does not see scores -inf: no maximum, and exp2 makes it 0
#pragma unroll
        for (int e = 0; e < 64; ++e)
          if (key0 + e > last_key) v[e] = 0xff800000u;
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;   // four chains instead of one of 64
#pragma unroll
      for (int e = 0; e < 64; e += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(v[e]));
        mx1 = fmaxf(mx1, __uint_as_float(v[e + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(v[e + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(v[e + 3]));
      }
      float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      xmax[half * 128 + row] = mx;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      mx = fmaxf(xmax[row], xmax[128 + row]);
      asm volatile("bar.sync 1, 256;" ::: "memory");   // every thread has read before the next tile (or the sums) overwrite
      // move the reference only when the tile exceeds it by more than REF_STEP (always at the row's first key)
      const float t2 = mx * p.scale_log2;            // scale > 0 keeps the order; -inf when the tile holds no key of this row
      const bool grow = t2 > ref + REF_STEP;         // (-inf + 8 is -inf: the first key always moves it)
      const float alpha = grow ? ex2(ref - t2) : 1.0f;   // 0 when ref was -inf
      if (grow) ref = t2;
      const float m2 = (ref == -INFINITY) ? 0.f : ref;
      const uint32_t pb = j & 1, pph = (j >> 1) & 1;
      if (j > 0 && __any_sync(0xffffffffu, grow)) {  // the whole warp takes the (warp-wide) loads and stores; a row that did not move multiplies by 1
        // O is being accumulated: the product with V of the tile before must be done (its commit on that tile's p_empty)
        if (!hand_off(&p_empty[pb ^ 1], ((j - 1) >> 1) & 1)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
        for (int cb = 0; cb < OC / 32; ++cb) {
          uint32_t o[32];
          tmem_ld32(lane_addr + O_COL + half * OC + cb * 32, o);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          tmem_st32(lane_addr + O_COL + half * OC + cb * 32, o);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      }
      uint32_t pk[32];
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int e = 0; e < 64; e += 2) {
        const float a = ex2(fmaf(__uint_as_float(v[e]), p.scale_log2, -m2));
        const float b = ex2(fmaf(__uint_as_float(v[e + 1]), p.scale_log2, -m2));
        s0 += a;
        s1 += b;
        pk[e / 2] = pack_bf16(a, b);
      }
      sum = fmaf(sum, alpha, s0 + s1);
      // this tile's P buffer: the product with V of the tile two before must have read it
      if (!hand_off(&p_empty[pb], pph ^ 1)) { ok = false; break; }
      uint8_t* prow = sP + pb * P_BYTES + half * TILE_BYTES + row * 128;
#pragma unroll
      for (int u = 0; u < 8; ++u)
        *reinterpret_cast<uint4*>(prow + ((u ^ (row & 7)) << 4)) = make_uint4(pk[u * 4], pk[u * 4 + 1], pk[u * 4 + 2], pk[u * 4 + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes, read by the MMA
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[pb]);
    }
    xmax[half * 128 + row] = sum;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    sum = xmax[row] + xmax[128 + row];
    if (ok && !mbar_wait(o_full, 0, abort_flag, wait_limit)) ok = false;
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool stored = qi < (int32_t)p.sq;          // a row past the block's queries is read with its warp (the
                                                       // tensor-memory loads are warp-wide) and not stored
      const float inv = 1.0f / ((sum < FLT_MIN) ? FLT_MIN : sum);
      uint16_t* dst = p.out + it.o_off + (uint64_t)(i0 + (int32_t)row) * p.o_ld + half * OC;
#pragma unroll
      for (int cb = 0; cb < OC / 32; ++cb) {
        uint32_t v[32];
        tmem_ld32(lane_addr + O_COL + half * OC + cb * 32, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 w;
          w.x = pack_bf16(__uint_as_float(v[q4 * 8 + 0]) * inv, __uint_as_float(v[q4 * 8 + 1]) * inv);
          w.y = pack_bf16(__uint_as_float(v[q4 * 8 + 2]) * inv, __uint_as_float(v[q4 * 8 + 3]) * inv);
          w.z = pack_bf16(__uint_as_float(v[q4 * 8 + 4]) * inv, __uint_as_float(v[q4 * 8 + 5]) * inv);
          w.w = pack_bf16(__uint_as_float(v[q4 * 8 + 6]) * inv, __uint_as_float(v[q4 * 8 + 7]) * inv);
          if (stored) *reinterpret_cast<uint4*>(dst + cb * 32 + q4 * 8) = w;
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
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

template <int D>
cudaError_t launch_d(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnTcParams& p,
                     uint64_t n_items, cudaStream_t stream) {
  constexpr int CH = D / 64, KS = D == 64 ? 3 : 2;
  constexpr size_t smem = (size_t)(1 + 2 * KS) * CH * TILE_BYTES + 2 * P_BYTES + 256 + 1024 + 1024;
  {
    const cudaError_t e = ensure_dynamic_smem((const void*)attention_tc_kernel<D>, smem);
    if (e != cudaSuccess) return e;
  }
  launch_pdl(attention_tc_kernel<D>, dim3((unsigned)(n_items * p.q_tiles), 1, 1), dim3(ATTN_THREADS), smem, stream, mq, mk, mv, p);
  return cudaGetLastError();
}

}  // namespace

bool attention_tc_supported(uint64_t sq, uint64_t d, uint64_t sk, uint64_t dv, float scale, int causal, const char** why) {
  if (!tc::encode_fn()) { *why = "no tensor-map encoder in this driver"; return false; }
  if (!(d == 64 || d == 128) || dv != d) { *why = "head width 64 or 128, the same for keys and values"; return false; }
  if (sq == 0 || sk == 0) { *why = "no queries or no keys"; return false; }
  if (sq > (1u << 30) || sk > (1u << 30)) { *why = "sequence too long"; return false; }
  if (!(scale > 0.f)) { *why = "scale must be positive"; return false; }
  if (causal && sk < sq) { *why = "a causal mask with fewer keys than queries"; return false; }
  return true;
}

cudaError_t launch_attention_tc(const void* q, uint64_t q_rows, uint64_t q_cols, const void* k, uint64_t k_rows,
                                uint64_t k_cols, const void* v, uint64_t v_rows, uint64_t v_cols,
                                const AttnBlockDev* items, uint64_t n_items, uint64_t sq, uint64_t d, uint64_t sk,
                                float scale, int causal, void* out, uint64_t o_ld, int* err, cudaStream_t stream) {
  if (n_items == 0) return cudaSuccess;
  if (n_items * ((sq + 127) / 128) > 0x7fffffffull) return cudaErrorNotSupported;
  CUtensorMap mq, mk, mv;
  if (!tc::make_map(&mq, q, q_rows, q_cols, q_cols, 128) || !tc::make_map(&mk, k, k_rows, k_cols, k_cols, 128) ||
      !tc::make_map(&mv, v, v_rows, v_cols, v_cols, 128))
    return cudaErrorNotSupported;
  AttnTcParams p;
  p.items = items;
  p.q_tiles = (uint32_t)((sq + 127) / 128);
  p.k_tiles = (uint32_t)((sk + 127) / 128);
  p.sq = (uint32_t)sq;
  p.sk = (uint32_t)sk;
  p.n_items = (uint32_t)n_items;
  p.causal = causal ? 1 : 0;
  p.causal_off = (int32_t)(sk - sq);
  p.scale_log2 = scale * 1.4426950408889634f;
  {
    static int spin = -1;
    if (spin < 0) { const char* e = getenv("B200TT_ATTN_SPIN"); spin = (e && e[0] == '0') ? 0 : 1; }
    p.spin = spin;
  }
  p.out = (uint16_t*)out;
  p.o_ld = o_ld;
  p.err = err;
  return d == 64 ? launch_d<64>(mq, mk, mv, p, n_items, stream) : launch_d<128>(mq, mk, mv, p, n_items, stream);
}

}  // namespace b200
