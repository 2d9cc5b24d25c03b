// TEST INFRASTRUCTURE: the kernel launch interface (csrc/kernels.h) with every launch a no-op
// that reports success, and the knobs of the fake runtime.  Linked with engine.cu (compiled as
// C++) into tests/_build/libb200tt_fake.so; results are never computed, only the host logic runs.
#include <cstring>
#include "cuda_runtime.h"
#include "kernels.h"
#include "kinds.h"

extern "C" {
uint64_t fake_cuda_memory_limit = 0;
uint64_t fake_cuda_memory_in_use = 0;
int fake_cuda_device_count = 1;
int fake_cuda_capturing = 0;
int fake_cuda_current_device = 0;
int fake_sync_in_capture = 0;
int fake_smem_attr_calls[8] = {0, 0, 0, 0, 0, 0, 0, 0};
int fake_launch_count = 0;        // launches the engine asked for
int fake_tc_supported = 1;        // what gemm_tc_supported answers for BF16 operands
int fake_last_attention_jobs = 0; // jobs of the last attention_rows launch
}

namespace b200 {
#define OK_LAUNCH ++fake_launch_count; return cudaSuccess
cudaError_t launch_eltwise(const EltwiseArgs&, cudaStream_t) { OK_LAUNCH; }
bool eltwise_kind_known(uint32_t k) { return kind::arity(k) != 0; }
cudaError_t launch_rope(const Mat&, const Mat&, const Mat&, uint64_t, void*, uint64_t, int, uint64_t, uint64_t, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_cast(const void*, void*, uint64_t, int, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_reduce(const void*, int, uint64_t, uint64_t, int, int, uint32_t, uint32_t, void*, cudaStream_t) { OK_LAUNCH; }
uint64_t full_sum_scratch_floats() { return 1184; }
cudaError_t launch_full_sum(const float*, uint64_t, int, float*, float*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_softmax_rows(const float*, const uint32_t*, uint64_t, float, int, void*, int, uint64_t, uint64_t, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_rms(const float*, uint64_t, uint64_t, float, float*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_rms_norm(const void*, int, const void*, int, const void*, int, float, void*, int, void*, int, uint64_t, uint64_t, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_argmax_rows(const float*, uint64_t, uint64_t, int32_t*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_select_rows(const void*, uint64_t, uint64_t, int, const int32_t*, uint64_t, void*, int*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_pick_columns(const uint32_t*, uint64_t, uint64_t, const int32_t*, uint32_t*, int*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_scatter_add_columns(float*, uint64_t, uint64_t, const int32_t*, const float*, int*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_select_add_rows(float*, uint64_t, uint64_t, const int32_t*, uint64_t, const float*, int*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_scatter_rows(uint32_t*, uint64_t, uint64_t, const int32_t*, uint64_t, const uint32_t*, int*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_gather_indexed(const uint32_t*, uint64_t, uint64_t, const int32_t*, uint64_t, uint32_t*, int*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_gather_row_ptrs(const void* const*, uint64_t, uint64_t, int, void*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_assign_rows(void*, const void*, uint64_t, int, const uint64_t*, uint64_t, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_copy_blocks(const void*, uint64_t, void*, uint64_t, int, const MoveDev*, uint64_t, uint64_t, uint64_t, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_repack(const void*, uint64_t, int, const uint64_t*, uint64_t, void*, cudaStream_t) { OK_LAUNCH; }
int attention_rows_tile(int rows) { return rows <= 1 ? 1 : (rows <= 2 ? 2 : (rows <= 4 ? 4 : 8)); }
void attention_rows_plan(uint64_t, int, int l, int, int* splits, int* lc) { *splits = l > 256 ? 2 : 1; *lc = l > 256 ? (l / 2 + 31) / 32 * 32 : l; }
size_t attention_rows_scratch_floats(uint64_t n, int rt, int dv, int splits) { return splits > 1 ? (size_t)n * splits * rt * (dv + 2) : 0; }
cudaError_t launch_attention_rows(const float*, const void*, uint64_t, const void*, uint64_t, int, const uint32_t*, const AttnJob*,
                                  const AttnRow*, uint64_t n_jobs, int, int, int, int, float, int splits, int, float*, void*, int,
                                  int* launches, cudaStream_t) { fake_last_attention_jobs = (int)n_jobs; *launches = splits > 1 ? 2 : 1; OK_LAUNCH; }
bool attention_tc_supported(uint64_t sq, uint64_t d, uint64_t sk, uint64_t dv, float scale, int causal, const char** why) {
  *why = "the fake runtime follows the kernel's rules";
  return (d == 64 || d == 128) && dv == d && sq && sk && sq % 128 == 0 && sk % 128 == 0 && scale > 0.f && (!causal || sk >= sq);
}
cudaError_t launch_attention_tc(const void*, uint64_t, uint64_t, const void*, uint64_t, uint64_t, const void*, uint64_t, uint64_t,
                                const AttnBlockDev*, uint64_t, uint64_t, uint64_t, uint64_t, float, int, void*, uint64_t, int*,
                                cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_scatter_rows_into(void*, uint64_t, uint64_t, int, const int32_t*, uint64_t, const void*, uint64_t, int*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_cast_f16(const void*, void*, uint64_t, int, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_cast_block(const void*, uint64_t, void*, uint64_t, uint64_t, int, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_gather_addrs(const uint64_t*, uint64_t, int, void*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_select_taps(const void*, uint64_t, uint64_t, int, const int32_t*, uint64_t, uint64_t, int, void*, uint64_t, int*, cudaStream_t) { OK_LAUNCH; }
uint64_t scan_chunks(int op, uint64_t rows, uint64_t) { return op >= 2 && rows >= 512 ? 4 : 1; }
cudaError_t launch_scan(const uint32_t*, uint32_t*, uint64_t, uint64_t, int, uint32_t*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_sort_planes(const uint32_t*, uint64_t, uint64_t, uint32_t, int, int, uint32_t*, uint32_t*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_random(uint32_t*, uint64_t, int, float, float, int32_t, int32_t, int, uint64_t, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_pool_windows(const uint16_t*, const uint32_t*, const uint32_t*, const float*, uint64_t, float*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_gemm_simt(const GemmArgs&, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_store_block_many(const void*, uint64_t, void* const*, int, uint64_t, uint64_t, uint64_t, int, cudaStream_t) { OK_LAUNCH; }
bool gemm_skinny_supported(const GemmArgs& g) { return g.in_bf16 && g.batch <= 1 && !g.a_trans && !g.b_trans && g.m <= 4 && g.n % 8 == 0; }
cudaError_t launch_gemm_skinny(const GemmArgs&, cudaStream_t) { OK_LAUNCH; }
bool gemm_tc_supported(const GemmArgs& g, const char** why) {
  *why = g.in_bf16 ? "the fake runtime was told to refuse" : "operands are not BF16";
  return g.in_bf16 && fake_tc_supported;
}
// as the real launcher does: the kernel's shared-memory opt-in is asked for on the current device before the launch
static void fake_tc_kernel() {}
cudaError_t launch_gemm_tc(const GemmArgs&, const GemmBatch*, int*, cudaStream_t, int* pair) {
  if (pair) *pair = 0;
  const cudaError_t e = ensure_dynamic_smem((const void*)fake_tc_kernel, 200 * 1024);
  if (e != cudaSuccess) return e;
  OK_LAUNCH;
}
bool gemm_addnorm_supported(uint64_t m, uint64_t n, uint64_t k, const char** why) {
  *why = "the row is one to eight tiles of 192 columns";
  return n % 192 == 0 && n / 192 <= 8 && m >= 64 && k >= 64 && k % 8 == 0;
}
cudaError_t launch_gemm_addnorm(const void*, const void*, const float*, const void*, float, float*, void*, uint64_t, uint64_t, uint64_t, int*,
                                cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_stalled_wait(int*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_bfp8_encode(const void*, int, uint64_t, uint64_t, uint8_t*, uint8_t*, cudaStream_t) { OK_LAUNCH; }
cudaError_t launch_bfp8_decode(const uint8_t*, const uint8_t*, uint64_t, uint64_t, void*, int, cudaStream_t) { OK_LAUNCH; }
bool decode_layers_supported(const DecodeShape& s, const char** why) {
  *why = "heads of 64 columns, one to four sequences, whole 64-column blocks";
  return s.rows >= 1 && s.rows <= 4 && s.head_dim == 64 && s.kv_heads && s.heads % s.kv_heads == 0 && s.hidden % 64 == 0 && s.ff % 64 == 0 &&
         s.attend && s.attend % 64 == 0 && s.attend <= s.max_len;
}
int decode_layers_grid() { return 64; }
DecodeScratch decode_layers_scratch(const DecodeShape&, int) { DecodeScratch d{}; d.floats = 1024; return d; }
cudaError_t launch_decode_layers(const DecodeShape&, const DecodeLayerPtrs*, const float*, const void*, const float*, const float*, const int32_t*,
                                 uint16_t*, float*, const DecodeScratch&, int, const void* maps, int*, cudaStream_t, const char** form) {
  *form = maps ? "cluster16" : "grid";
  OK_LAUNCH;
}
bool decode_layers_cluster_wanted(const DecodeShape&, bool any_bfp) { return !any_bfp; }
size_t decode_layers_maps_bytes(const DecodeShape& s) { return (size_t)s.layers * 4 * 128; }
bool decode_layers_make_maps(const DecodeShape& s, const DecodeLayerPtrs*, void* maps_host) {
  memset(maps_host, 0, decode_layers_maps_bytes(s));
  return true;
}
bool gemm_skinny_bfp_supported(uint64_t m, uint64_t n, uint64_t) { return m >= 1 && m <= 4 && n % 16 == 0; }
cudaError_t launch_gemm_skinny_bfp(const uint16_t*, uint64_t, const uint8_t*, const uint8_t*, void*, uint64_t, int, uint64_t, uint64_t, uint64_t,
                                   cudaStream_t) { OK_LAUNCH; }
bool gemm_tc2_wanted(const GemmArgs&) { return false; }
cudaError_t launch_gemm_tc2(const GemmArgs&, int*, cudaStream_t) { OK_LAUNCH; }
bool gemm_tf32_supported(const GemmArgs& g, const char** why) { *why = "small"; return !g.in_bf16 && g.batch <= 1 && g.m >= 128 && g.n >= 128 && g.k >= 32; }
cudaError_t launch_gemm_tf32(const GemmArgs&, void*, void*, void*, void*, int*, cudaStream_t) { OK_LAUNCH; }
}  // namespace b200

extern "C" int32_t b200_full_sum_noalloc(const float*, uint64_t, int32_t, float*, void*) { return 2; }
