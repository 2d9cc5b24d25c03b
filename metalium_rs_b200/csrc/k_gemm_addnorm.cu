// A projection whose result goes straight into the residual stream and its RMSNorm, as one kernel:
//     sum = resid + A B (F32),   norm = BF16( (sum / sqrt(mean(sum^2) + eps)) * gains )
// what the prefill's layer does after its output projection and after its down projection
// (crates/tt-models/src/llama.rs:371-507: `matmul_dram` into `add_rms_norm`, the trait's
// `Engine::matmul_dram_bf16` crates/burn-tt/src/server.rs:191 and the norm of
// crates/tt-kernels/src/sfpu/reduce.rs through `add_rms_norm_as`).  Composed, the norm is a launch of its own that
// reads the product and the residual back and writes both results: 6 us of a 120 us layer, twice.
//
// The product is the tcgen05 kernel's (k_gemm_tc.cu: TMA ring, one thread issuing M=128 N=192 K=16 MMAs into TMEM),
// one 128 x 192 tile a CTA.  A row's statistic needs the whole row, and 576 and more F32 columns do not fit a CTA's 512
// TMEM columns, so the n / 192 CTAs of a row panel form a thread-block cluster: each adds the residual to its tile
// (fetched by one tiled copy while the product runs), writes `sum`, takes its 192 columns' sum of squares a row, and
// hands that to the other CTAs' shared memory (`st.shared::cluster`, then an arrive with release on the receiver's
// mbarrier); when every CTA's partial has arrived (bounded wait) each adds them in CTA order, so all hold the same
// statistic, and normalises its own tile.  The roundings are the composed ops': the sum is one F32 addition, the
// quotient and the product with the gain separate roundings, BF16 once.  The sum of squares is added in another fixed
// order than the stand-alone norm's (192 columns a CTA, the CTAs in order), so the norm may differ from the composed
// one by a unit in the last place of the statistic; the logits agree as two correct evaluations do.
// No load uses cluster multicast.  Every wait is bounded.
#include "tc_common.cuh"
#include "pdl.cuh"

namespace b200 {
namespace {

using namespace tc;

constexpr int AN_BN = 192;                                      // tile columns
constexpr int AN_STAGES = 3;
constexpr uint32_t AN_A_BYTES = BM * BK * 2, AN_B_BYTES = AN_BN * BK * 2, AN_STAGE_BYTES = AN_A_BYTES + AN_B_BYTES;
constexpr uint32_t AN_TILE_BYTES = BM * AN_BN * 4;              // a tile of F32: the residual's, and the accumulator's
constexpr int AN_MAX_CLUSTER = 8;
static_assert(AN_STAGES * AN_STAGE_BYTES >= AN_TILE_BYTES, "the accumulator's tile reuses the stages");

struct AddNormParams {
  uint64_t m, k;
  uint32_t n;                 // cluster size * 192
  float* sum_out;             // [m, n] F32
  uint16_t* norm_out;         // [m, n] BF16
  const uint16_t* gains;      // [n] BF16
  float eps;
  int* err;
  uint32_t mn_lbo, mn_sbo;
};

__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_size() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ bool mbar_try_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// where 16-byte piece g of row `row` of the accumulator's tile lies: pieces are exchanged inside groups of eight by the
// row's low bits, so a warp's lanes (a row each) writing the same piece meet eight different bank groups
__device__ __forceinline__ uint32_t tile_piece(uint32_t row, uint32_t g) { return row * (AN_BN * 4) + (((g & ~7u) | ((g ^ row) & 7u)) << 4); }

// Four F32 values rounded to BF16 as `f32_to_bf16_bits` rounds them (nearest even; a result below 2^-126 a signed zero; a
// NaN quiet with its payload).  The hardware's conversion is the same rounding for every number that is zero or at least
// 2^-126 in magnitude, so only the others (and NaNs) take the integer rule -- which alone is nine instructions a value.
__device__ __forceinline__ uint2 bf16x4(float t0, float t1, float t2, float t3) {
  const uint32_t a0 = __float_as_uint(t0) & 0x7fffffffu, a1 = __float_as_uint(t1) & 0x7fffffffu;
  const uint32_t a2 = __float_as_uint(t2) & 0x7fffffffu, a3 = __float_as_uint(t3) & 0x7fffffffu;
  // (a - 1) wraps a zero to the top: "0 < a < 2^-126 or a NaN" is "(a - 1) >= 0x7f800000 or (a - 1) < 0x007fffff" without the zeros
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

constexpr int AN_THREADS = 512;                                  // sixteen warps: two also run the copy and MMA roles, all of them the epilogue
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr) : "memory");
}

__global__ void __launch_bounds__(AN_THREADS, 1)
gemm_addnorm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_r, const AddNormParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* rtile = smem + AN_STAGES * AN_STAGE_BYTES;             // [128][192] F32 as the copy lands it
  uint64_t* full = (uint64_t*)(rtile + AN_TILE_BYTES);
  uint64_t* empty = full + AN_STAGES;
  uint64_t* acc_full = empty + AN_STAGES;
  uint64_t* r_full = acc_full + 1;
  uint64_t* x_bar = r_full + 1;                                   // the other CTAs' partial sums have arrived
  uint32_t* tmem_slot = (uint32_t*)(x_bar + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  float* ssum = (float*)(rtile + AN_TILE_BYTES + 256);            // [cluster][128]: every CTA's sum of squares of the panel's rows

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t C = cluster_size(), tn = cluster_rank(), tm = blockIdx.x / C;
  if (threadIdx.x == 0) {
    for (int s = 0; s < AN_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    mbar_init(r_full, 1);
    mbar_init(x_bar, C > 1 ? (C - 1) * 128 : 1);                  // a thread a row of every other CTA arrives once
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  // every CTA's barriers exist before another CTA of the cluster may arrive on them (all arrive here: it cannot stall)
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  pdl_enter();
  const long long wait_limit = wait_limit_of(p.err);
  const uint32_t num_kb = (uint32_t)((p.k + BK - 1) / BK);
  const int32_t m0 = (int32_t)(tm * BM), n0 = (int32_t)(tn * AN_BN);

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    // the residual's tile first: it travels while the product runs
    mbar_expect_tx(r_full, AN_TILE_BYTES);
    tma_load_2d(rtile, &map_r, r_full, n0, m0);
    uint32_t stage = 0, phase = 0;
    bool okp = true;
    for (uint32_t kb = 0; kb < num_kb; ++kb) {
      if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, wait_limit)) { okp = false; break; }
      uint8_t* sa = smem + stage * AN_STAGE_BYTES;
      uint8_t* sb = sa + AN_A_BYTES;
      mbar_expect_tx(&full[stage], AN_STAGE_BYTES);
      const int32_t k0 = (int32_t)(kb * BK);
      tma_load_2d(sa, &map_a, &full[stage], k0, m0);              // A [m, k]: K-major
#pragma unroll
      for (int j = 0; j < AN_BN / 64; ++j) tma_load_2d(sb + j * 8192, &map_b, &full[stage], n0 + j * 64, k0);   // B [k, n]: MN-major
      if (++stage == AN_STAGES) { stage = 0; phase ^= 1; }
    }
    if (!okp) { atomicCAS(p.err, 0, TIMEOUT_CODE); *abort_flag = 1; }
    // drain: no copy may outlive the CTA (the accumulator's tile is written over the stages only after the last MMA read them)
    for (int s = 0; s < AN_STAGES; ++s) {
      const uint32_t ph = (s < (int)stage) ? phase : (phase ^ 1);
      const long long t0 = clock64();
      while (!mbar_try(&full[s], ph))
        if (clock64() - t0 > wait_limit) break;
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (0u << 15) | (1u << 16) | ((uint32_t)(AN_BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    uint32_t stage = 0, phase = 0;
    bool okm = true;
    for (uint32_t kb = 0; kb < num_kb; ++kb) {
      if (!mbar_wait(&full[stage], phase, abort_flag, wait_limit)) { okm = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t sa = smem_u32(smem + stage * AN_STAGE_BYTES), sb = sa + AN_A_BYTES;
#pragma unroll
      for (int kk = 0; kk < BK / UMMA_K; ++kk)
        umma_bf16(tmem_base, make_desc(sa + kk * 32, 16, 1024), make_desc(sb + kk * 2048, p.mn_lbo, p.mn_sbo), idesc, (kb | (uint32_t)kk) != 0 ? 1u : 0u);
      umma_commit(&empty[stage]);
      if (++stage == AN_STAGES) { stage = 0; phase ^= 1; }
    }
    if (okm) umma_commit(acc_full);
    else { atomicCAS(p.err, 0, TIMEOUT_CODE); *abort_flag = 1; }
  }
  __syncwarp();

  // ---------------- epilogue: all sixteen warps ----------------
  // A warp may read the 32 TMEM lanes of its quarter (warp % 4); the four warps of a quarter take 48 columns each.
  const uint32_t quad = warp & 3, cgp = warp >> 2, row_l = quad * 32 + lane;
  const bool second = lane < AN_BN / 4 - 32;
  // (the gains of this lane's columns: asked for now, used in the last pass)
  const uint2 h0 = *reinterpret_cast<const uint2*>(p.gains + n0 + lane * 4);
  const uint2 h1 = second ? *reinterpret_cast<const uint2*>(p.gains + n0 + (lane + 32) * 4) : make_uint2(0, 0);
  bool ok = mbar_wait(acc_full, 0, abort_flag, wait_limit);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (ok) {
#pragma unroll
    for (int c16 = 0; c16 < 3; ++c16) {
      uint32_t v[16];
      tmem_ld16(tmem_base + ((quad * 32u) << 16) + cgp * 48 + c16 * 16, v);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int q = 0; q < 4; ++q)
        *reinterpret_cast<uint4*>(smem + tile_piece(row_l, cgp * 12 + c16 * 4 + q)) = make_uint4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
    }
    ok = mbar_wait(r_full, 0, abort_flag, wait_limit);            // the residual's tile has landed
  }
  __syncthreads();                                                 // the accumulator's tile is whole
  // pass 1, eight rows a warp: sum = residual + product, written out and kept; its squares summed -- a lane takes 16-byte
  // piece `lane` of the row's 48, and piece `lane + 32` where there is one
  float* mysum = ssum + tn * 128;
  if (ok) {
#pragma unroll 1                                       // (the epilogue runs once a CTA, so every instruction is a cold fetch: short code)
    for (int rr = 0; rr < 8; ++rr) {
      const uint32_t row = warp * 8 + rr;
      const uint64_t grow = (uint64_t)m0 + row;
      float ss = 0.f;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (h == 1 && !second) break;
        const uint32_t g = lane + h * 32;
        float4* at = reinterpret_cast<float4*>(smem + tile_piece(row, g));
        const float4 a = *at, r = *reinterpret_cast<const float4*>(rtile + row * (AN_BN * 4) + g * 16);
        float4 v;
        v.x = r.x + a.x; v.y = r.y + a.y; v.z = r.z + a.z; v.w = r.w + a.w;
        *at = v;
        if (grow < p.m) *reinterpret_cast<float4*>(p.sum_out + grow * p.n + n0 + g * 4) = v;
        ss = ss + ((v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w));
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss = ss + __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) mysum[row] = ss;
    }
  } else if (lane < 8) {
    mysum[warp * 8 + lane] = 0.f;
  }
  __syncthreads();                                                 // this CTA's partial sums are whole
  // every other CTA of the cluster gets them: a thread a row stores it there and arrives, with release, on that CTA's barrier
  if (threadIdx.x < 128) {
    const float mine = mysum[threadIdx.x];
    for (uint32_t c = 0; c < C; ++c) {
      if (c == tn) continue;
      uint32_t ra, rb;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(mysum + threadIdx.x)), "r"(c));
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rb) : "r"(smem_u32(x_bar)), "r"(c));
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(ra), "f"(mine) : "memory");
      asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(rb) : "memory");
    }
  }
  // (also a thread that gave up an earlier wait waits here: no CTA may leave while another still stores into its shared memory)
  if (C > 1) {
    const long long t0 = clock64();
    while (!mbar_try_cluster(x_bar, 0)) {
      if (clock64() - t0 > wait_limit) { ok = false; break; }
    }
  }
  // pass 2: the statistic of the whole row (the CTAs' partial sums in CTA order), the quotient, the gain, BF16
  if (ok) {
    const float inv = 1.0f / (float)p.n;
    float g0[4], g1[4];
    {
      g0[0] = __uint_as_float(h0.x << 16); g0[1] = __uint_as_float(h0.x & 0xffff0000u);
      g0[2] = __uint_as_float(h0.y << 16); g0[3] = __uint_as_float(h0.y & 0xffff0000u);
      g1[0] = __uint_as_float(h1.x << 16); g1[1] = __uint_as_float(h1.x & 0xffff0000u);
      g1[2] = __uint_as_float(h1.y << 16); g1[3] = __uint_as_float(h1.y & 0xffff0000u);
    }
#pragma unroll 1
    for (int rr = 0; rr < 8; ++rr) {
      const uint32_t row = warp * 8 + rr;
      const uint64_t grow = (uint64_t)m0 + row;
      float total = ssum[row];
      for (uint32_t c = 1; c < C; ++c) total = total + ssum[c * 128 + row];
      const float stat = sqrtf(total * inv + p.eps);
      if (grow >= p.m) continue;                                   // (the same for the whole warp)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (h == 1 && !second) break;
        const uint32_t g = lane + h * 32;
        const float4 v = *reinterpret_cast<const float4*>(smem + tile_piece(row, g));
        const float* gg = h ? g1 : g0;
        const float t0 = (v.x / stat) * gg[0], t1 = (v.y / stat) * gg[1], t2 = (v.z / stat) * gg[2], t3 = (v.w / stat) * gg[3];
        *reinterpret_cast<uint2*>(p.norm_out + grow * p.n + n0 + g * 4) = bf16x4(t0, t1, t2, t3);
      }
    }
  }
  if (!ok && lane == 0) { atomicCAS(p.err, 0, TIMEOUT_CODE); *abort_flag = 1; }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
  }
}

}  // namespace

bool gemm_addnorm_supported(uint64_t m, uint64_t n, uint64_t k, const char** why) {
  *why = "";
  if (!encode_fn()) { *why = "the driver offers no tensor-map encoder"; return false; }
  if (n % AN_BN || n / AN_BN > AN_MAX_CLUSTER) { *why = "the row is one to eight tiles of 192 columns"; return false; }
  if (m < 64 || k < 64 || k % 8 || m > 0x7fffffffull || k > 0x7fffffffull) { *why = "at least 64 rows and 64 of k, k a multiple of 8"; return false; }
  return true;
}

// sum = resid + A B, norm = RMSNorm(sum) * gains as BF16; A [m, k] BF16, B [k, n] BF16, resid [m, n] F32, gains [n] BF16.
cudaError_t launch_gemm_addnorm(const void* a, const void* b, const float* resid, const void* gains, float eps, float* sum_out,
                                void* norm_out, uint64_t m, uint64_t n, uint64_t k, int* err_word, cudaStream_t stream) {
  using namespace tc;
  const char* why = "";
  if (!gemm_addnorm_supported(m, n, k, &why)) return cudaErrorNotSupported;
  CUtensorMap ma, mb, mr;
  if (!make_map(&ma, a, m, k, k, BM)) return cudaErrorNotSupported;
  if (!make_map(&mb, b, k, n, n, 64)) return cudaErrorNotSupported;
  {
    EncodeTiledFn fn = encode_fn();
    const cuuint64_t dims[2] = {n, m};
    const cuuint64_t strides[1] = {n * 4};
    const cuuint32_t box[2] = {(cuuint32_t)AN_BN, (cuuint32_t)BM};
    const cuuint32_t estr[2] = {1, 1};
    if (fn(&mr, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(resid), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return cudaErrorNotSupported;
  }
  AddNormParams p{};
  p.m = m; p.k = k; p.n = (uint32_t)n;
  p.sum_out = sum_out; p.norm_out = reinterpret_cast<uint16_t*>(norm_out); p.gains = reinterpret_cast<const uint16_t*>(gains);
  p.eps = eps; p.err = err_word;
  p.mn_lbo = 8192; p.mn_sbo = 1024;
  const unsigned C = (unsigned)(n / AN_BN), tiles_m = (unsigned)((m + BM - 1) / BM);
  constexpr size_t smem = (size_t)AN_STAGES * AN_STAGE_BYTES + AN_TILE_BYTES + 256 + AN_MAX_CLUSTER * 128 * 4 + 1024;
  cudaError_t e = ensure_dynamic_smem((const void*)gemm_addnorm_kernel, smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles_m * C); cfg.blockDim = dim3(AN_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = C; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, gemm_addnorm_kernel, ma, mb, mr, p);
}

}  // namespace b200
