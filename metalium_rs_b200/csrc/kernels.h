// Launch interface between the engine (host logic, engine.cu) and the kernel
// translation units.  Every function enqueues on `stream` and returns the launch
// status; none allocates or synchronises.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// A matrix operand as a kernel sees it: base already moved to the block's
// first element, leading dimension in elements.
struct Mat {
  const void* p = nullptr;
  uint64_t ld = 0;
  uint64_t rows = 0, cols = 0;  // extent of the operand (for broadcast: r % rows, c % cols)
  int bf16 = 0;                 // 0: 32-bit words, 1: bf16
};

struct EltwiseArgs {
  uint32_t kind;
  float s1, s2;
  Mat a, b, c;
  void* out;
  uint64_t out_ld;
  int out_bf16;
  uint64_t rows, cols;  // output extent
  int* err;             // device error word (first failure wins)
};
cudaError_t launch_eltwise(const EltwiseArgs& args, cudaStream_t stream);
bool eltwise_kind_known(uint32_t kind);

// x cos + swap_halves(x) sin, heads of `head` columns (tt-kernels/src/tensor.rs:5545).
cudaError_t launch_rope(const Mat& x, const Mat& cs, const Mat& sn, uint64_t head, void* out,
                        uint64_t out_ld, int out_bf16, uint64_t rows, uint64_t cols,
                        cudaStream_t stream);
cudaError_t launch_cast(const void* in, void* out, uint64_t n, int to_bf16, cudaStream_t stream);

// ---- reductions ------------------------------------------------------------
cudaError_t launch_reduce(const void* a, int a_bf16, uint64_t rows, uint64_t cols, int op, int axis,
                          uint32_t then_kind, uint32_t then_bits, void* out, cudaStream_t stream);
// Full sum (mean): two stages, fixed order.  `scratch` holds >= full_sum_scratch_floats() floats.
uint64_t full_sum_scratch_floats();
cudaError_t launch_full_sum(const float* a, uint64_t n, int mean, float* scratch, float* out,
                            cudaStream_t stream);
cudaError_t launch_softmax_rows(const float* x, const uint32_t* mask, uint64_t mask_rows, float scale,
                                int log_form, void* out, int out_bf16, uint64_t rows, uint64_t cols,
                                cudaStream_t stream);
cudaError_t launch_rms(const float* a, uint64_t rows, uint64_t cols, float eps, float* out,
                       cudaStream_t stream);
// a (+ b) -> optional sum_out, norm_out (f32 or bf16); a/b may be bf16.
cudaError_t launch_rms_norm(const void* a, int a_bf16, const void* b, int b_bf16, const void* gamma,
                            int gamma_bf16, float eps, void* sum_out, int sum_bf16, void* norm_out,
                            int norm_bf16, uint64_t rows, uint64_t cols, cudaStream_t stream);
cudaError_t launch_argmax_rows(const float* a, uint64_t rows, uint64_t cols, int32_t* out,
                               cudaStream_t stream);

// ---- indexing and copies (bit moves; elem_bytes 2 or 4) -----------------------
cudaError_t launch_select_rows(const void* table, uint64_t t_rows, uint64_t cols, int elem_bytes,
                               const int32_t* idx, uint64_t n, void* out, int* err, cudaStream_t);
cudaError_t launch_pick_columns(const uint32_t* x, uint64_t rows, uint64_t cols, const int32_t* idx,
                                uint32_t* out, int* err, cudaStream_t);
cudaError_t launch_scatter_add_columns(float* t_copy, uint64_t rows, uint64_t cols, const int32_t* idx,
                                       const float* v, int* err, cudaStream_t);
// out (already a copy of t) += value rows at idx, duplicates in index order.
cudaError_t launch_select_add_rows(float* out, uint64_t t_rows, uint64_t cols, const int32_t* idx,
                                   uint64_t n, const float* value, int* err, cudaStream_t);
// out (already a copy of table) row idx[i] = values row i; later i wins.
cudaError_t launch_scatter_rows(uint32_t* out, uint64_t t_rows, uint64_t cols, const int32_t* idx,
                                uint64_t n, const uint32_t* values, int* err, cudaStream_t);
cudaError_t launch_gather_indexed(const uint32_t* x, uint64_t rows, uint64_t cols, const int32_t* idx,
                                  uint64_t i_cols, uint32_t* out, int* err, cudaStream_t);
// out[i,:] = *(row_ptrs[i]) for cols elements.
cudaError_t launch_gather_row_ptrs(const void* const* row_ptrs, uint64_t n_rows, uint64_t cols,
                                   int elem_bytes, void* out, cudaStream_t);
// out[dst_row(i), :] = src[src_row(i), :], pairs (dst, src) on the device.
cudaError_t launch_assign_rows(void* out, const void* value, uint64_t cols, int elem_bytes,
                               const uint64_t* pairs, uint64_t n, cudaStream_t);
// attention_rows (k_attention.cu).  A job is up to 8 query rows that share a key block and a
// value block (element offsets); a row is where its query starts in q and its result in out.
struct AttnJob { uint64_t k_off, v_off; int32_t row_start, nrows; };
struct AttnRow { uint64_t q_off, out_off; };
int attention_rows_tile(int rows);   // the rows a job is built for: 1, 2, 4 or 8
void attention_rows_plan(uint64_t n_jobs, int rt, int l, int sms, int* splits, int* lc);
size_t attention_rows_scratch_floats(uint64_t n_jobs, int rt, int dv, int splits);
cudaError_t launch_attention_rows(const float* q, const void* k, uint64_t k_ld, const void* v, uint64_t v_ld, int kv_bf16,
                                  const uint32_t* mask, const AttnJob* jobs, const AttnRow* rows, uint64_t n_jobs, int rt,
                                  int d, int l, int dv, float scale, int splits, int lc, float* scratch, void* out,
                                  int out_bf16, int* launches, cudaStream_t stream);
// fused attention over whole sequences (k_attention_tc.cu): element coordinates of a block's Q, K
// and V (row, column) and the element offset of its output
struct AttnBlockDev { int32_t q_r, q_c, k_r, k_c, v_r, v_c; int32_t pad0, pad1; uint64_t o_off; };
bool attention_tc_supported(uint64_t sq, uint64_t d, uint64_t sk, uint64_t dv, float scale, int causal, const char** why);
cudaError_t launch_attention_tc(const void* q, uint64_t q_rows, uint64_t q_cols, const void* k, uint64_t k_rows,
                                uint64_t k_cols, const void* v, uint64_t v_rows, uint64_t v_cols,
                                const AttnBlockDev* items, uint64_t n_items, uint64_t sq, uint64_t d, uint64_t sk,
                                float scale, int causal, void* out, uint64_t o_ld, int* err, cudaStream_t stream);
cudaError_t launch_scatter_rows_into(void* table, uint64_t t_rows, uint64_t cols, int elem_bytes, const int32_t* idx,
                                     uint64_t n, const void* values, uint64_t v_ld, int* err, cudaStream_t);
// `multicast`: dst[0] is a multicast address and each piece is stored once with multimem.st (n_dst == 1).
cudaError_t launch_store_block_many(const void* src, uint64_t src_pitch, void* const* dst, int n_dst, uint64_t dst_pitch,
                                    uint64_t rows, uint64_t row_bytes, int multicast, cudaStream_t);
struct MoveDev { uint64_t from_r, from_c, to_r, to_c, rows, cols; int32_t transposed; int32_t pad; };
cudaError_t launch_copy_blocks(const void* src, uint64_t src_ld, void* dst, uint64_t dst_ld,
                               int elem_bytes, const MoveDev* moves_dev, uint64_t n_moves,
                               uint64_t max_rows, uint64_t max_cols, cudaStream_t);
// out[i] = src[pairs[2i] * src_ld + pairs[2i+1]]
cudaError_t launch_repack(const void* src, uint64_t src_ld, int elem_bytes, const uint64_t* pairs_dev,
                          uint64_t n, void* out, cudaStream_t);

// ---- products ---------------------------------------------------------------
struct GemmBatch {       // one product of a batched call, element offsets into a / b / c
  uint64_t a_off, b_off, c_off;
  int32_t a_trans, b_trans;
};
struct GemmArgs {
  const void* a; const void* b; void* c;
  int in_bf16;           // operands bf16 (else f32)
  int out_bf16;          // result bf16 (else f32)
  uint64_t m, n, k;
  uint64_t lda, ldb, ldc;  // leading dims of the stored matrices
  int a_trans, b_trans;    // stored matrix is the transpose of the logical operand
  uint64_t batch;          // 1, or number of products
  const GemmBatch* batches_dev;  // device array when batch > 1 (or nullptr for batch 1)
  void* c_more[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  int n_more = 0;          // the tensor-core product also stores C at these addresses (same pitch as c)
  int multicast = 0;       // c is a multicast address: every 16-byte piece is stored once with multimem.st (n_more == 0)
  int epi_mode = 0;        // 1: the tensor-core epilogue stores silu(gate) * up of each 256-column tile's halves (n % 256 == 0)
                           // 2: BF16 result with RoPE applied to the heads of 64 columns that lie below rope_cols
  const float* rope_cos = nullptr;   // [rope_rows, 64] F32 (pitch rope_ld floats): row r of the product uses table row r % rope_rows
  const float* rope_sin = nullptr;   // the same shape, [-sin, sin]
  uint32_t rope_rows = 0, rope_ld = 0, rope_cols = 0;
  int sm_limit = 0;        // > 0: the tensor-core product uses at most this many SMs (the rest stay free for a
                           // collective running beside it)
};
// SIMT (FFMA) path: any shape, any transposes, f32 or bf16 operands, f32 accumulate.
cudaError_t launch_gemm_simt(const GemmArgs& g, cudaStream_t stream);

// tcgen05 path.  Returns cudaErrorNotSupported when the shape cannot take it.
struct TcPlan;  // opaque: tensor maps + grid
bool gemm_tc_supported(const GemmArgs& g, const char** why);
// `pair_taken` (may be null) is set when the CTA-pair kernel ran the product.
// sum = resid + A B (F32) and norm = RMSNorm(sum) * gains (BF16) as one kernel (k_gemm_addnorm.cu): A [m, k] BF16,
// B [k, n] BF16, resid [m, n] F32, gains [n] BF16; n is one to eight tiles of 192 columns.
bool gemm_addnorm_supported(uint64_t m, uint64_t n, uint64_t k, const char** why);
cudaError_t launch_gemm_addnorm(const void* a, const void* b, const float* resid, const void* gains, float eps, float* sum_out,
                                void* norm_out, uint64_t m, uint64_t n, uint64_t k, int* err_word, cudaStream_t stream);
cudaError_t launch_gemm_tc(const GemmArgs& g, const GemmBatch* batches_host, int* err_word,
                           cudaStream_t stream, int* pair_taken = nullptr);
// One CTA that waits, with the kernels' bounded wait and the engine's limit, on an mbarrier whose bytes
// never arrive: the wait runs out, the error word becomes TIMEOUT and the kernel returns.  It exists so
// the time-out path can be exercised without stalling a real product.
cudaError_t launch_stalled_wait(int* err_word, cudaStream_t stream);

// A product of at most 4 rows (a decode step's projections): streams B once on CUDA cores.
bool gemm_skinny_supported(const GemmArgs& g);
cudaError_t launch_gemm_skinny(const GemmArgs& g, cudaStream_t stream);

// CTA-pair (cta_group::2) variant of the BF16 tensor-core product, for one large product.
bool gemm_tc2_wanted(const GemmArgs& g);
cudaError_t launch_gemm_tc2(const GemmArgs& g, int* err_word, cudaStream_t stream);

// Split-TF32 tensor-core path for F32 operands; the four scratch matrices have the operands' sizes.
bool gemm_tf32_supported(const GemmArgs& g, const char** why);
cudaError_t launch_gemm_tf32(const GemmArgs& g, void* a_hi, void* a_lo, void* b_hi, void* b_lo, int* err_word,
                             cudaStream_t stream);

// F32 <-> IEEE binary16 in two-byte storage, and the F32 <-> BF16 cast of a block of a wider buffer.
cudaError_t launch_cast_f16(const void* in, void* out, uint64_t n, int to_f16, cudaStream_t stream);
cudaError_t launch_cast_block(const void* in, uint64_t in_ld, void* out, uint64_t rows, uint64_t cols, int to_bf16,
                              cudaStream_t stream);
// out[i] = the datum at device address addrs[i] (2- or 4-byte datums).
cudaError_t launch_gather_addrs(const uint64_t* addrs_dev, uint64_t n, int elem_bytes, void* out, cudaStream_t stream);
// Rows of a table for each tap of a [taps, n] index matrix, side by side, each tap from a multiple of 32 columns.
cudaError_t launch_select_taps(const void* table, uint64_t t_rows, uint64_t cols, int elem_bytes, const int32_t* idx,
                               uint64_t taps, uint64_t n, int zero_row, void* out, uint64_t out_cols, int* err,
                               cudaStream_t stream);
// Inclusive scan down rows; `op` in the order Sum, Prod, Min, Max, MinNan, MaxNan, ISum, IProd, IMin, IMax.
// `scan_chunks` row chunks need a [chunks, cols] word scratch (`carry`); with none the rows stay together.
uint64_t scan_chunks(int op, uint64_t rows, uint64_t cols);
cudaError_t launch_scan(const uint32_t* in, uint32_t* out, uint64_t rows, uint64_t cols, int op, uint32_t* carry,
                        cudaStream_t stream);
// Sort of every problem of a planes matrix [rows = 32 * a power of two <= 1024, cols % 32 == 0] over its
// first n positions; `indices` may be null.
cudaError_t launch_sort_planes(const uint32_t* in, uint64_t rows, uint64_t cols, uint32_t n, int is_i32, int descending,
                               uint32_t* keys, uint32_t* indices, cudaStream_t stream);
// A seeded draw of n words; `draw` 0 Unit, 1 Uniform(p0, p1; i1 = bits of the float below p1), 2 Bernoulli(p0),
// 3 Normal(mean p0, std p1), 4 IntRange(lo i0, range p0), 5 IntWords.
cudaError_t launch_random(uint32_t* out, uint64_t n, int draw, float p0, float p1, int32_t i0, int32_t i1, int as_int,
                          uint64_t base, cudaStream_t stream);

// Means over host-built windows of a BF16 matrix: window w is flat[offsets[w] .. offsets[w + 1]) (element offsets).
cudaError_t launch_pool_windows(const uint16_t* in, const uint32_t* offsets_dev, const uint32_t* flat_dev,
                                const float* divisors_dev, uint64_t n, float* out, cudaStream_t stream);

// BFP8 storage (k_bfp.cu): [rows, cols] values (cols % 16 == 0) <-> rows * cols datum bytes + rows * cols / 16 exponent bytes.
cudaError_t launch_bfp8_encode(const void* in, int in_bf16, uint64_t rows, uint64_t cols, uint8_t* datums, uint8_t* exps,
                               cudaStream_t stream);
cudaError_t launch_bfp8_decode(const uint8_t* datums, const uint8_t* exps, uint64_t rows, uint64_t cols, void* out, int out_bf16,
                               cudaStream_t stream);
// The few-row product with B read as BFP8 (m <= 4, n a multiple of 16, A BF16 as stored, B as stored).
bool gemm_skinny_bfp_supported(uint64_t m, uint64_t n, uint64_t k);
cudaError_t launch_gemm_skinny_bfp(const uint16_t* a, uint64_t lda, const uint8_t* datums, const uint8_t* exps, void* c, uint64_t ldc,
                                   int out_bf16, uint64_t m, uint64_t n, uint64_t k, cudaStream_t stream);

// One decode step through every layer in one cooperative launch (k_decode.cu).
struct DecodeShape {
  uint32_t layers, rows, hidden, heads, kv_heads, head_dim, ff, max_len, attend;
  float eps, scale;
  uint32_t weights;   // the layers' matrices: 0 every one BF16, 1 every one BFP8, 2 some of each
};
struct DecodeLayerPtrs {          // a layer's operands as device addresses (a device array, one record a layer)
  const void *norm1, *qkv, *o, *norm2, *gate_up, *down;   // gains BF16 [1, hidden]; matrices [k, n] BF16 or BFP8
  void *kc, *vc;                                           // the layer's key and value cache, [rows * max_len, kv_heads * 64] BF16
  uint32_t bfp, pad;                                       // bit 0 qkv, 1 o, 2 gate_up, 3 down: that matrix is BFP8
};
struct DecodeScratch {            // how the step's scratch (F32 words) is cut, and how each product's k is sliced
  uint32_t ks_qkv, sl_qkv, ks_o, sl_o, ks_gu, sl_gu, ks_dn, sl_dn;
  uint64_t off_qkv, off_att, off_o, off_gu, off_dn, off_bar, floats;
  uint64_t off_tp, tp_floats;       // the several-cluster form's partial sums (F32 words; the region starts on 256 bytes)
};
bool decode_layers_supported(const DecodeShape& shape, const char** why);
int decode_layers_grid();
DecodeScratch decode_layers_scratch(const DecodeShape& shape, int grid);
cudaError_t launch_decode_layers(const DecodeShape& shape, const DecodeLayerPtrs* layers_dev, const float* x0, const void* final_norm,
                                 const float* cos_t, const float* sin_t, const int32_t* pos, uint16_t* out, float* scratch,
                                 const DecodeScratch& cut, int grid, const void* maps_dev, int* err, cudaStream_t stream,
                                 const char** form);   // *form: "cluster16x3" (several clusters), "cluster16", "cluster8" or "grid", what was launched
// Whether the step should take the cluster form (then the caller builds the descriptors below and passes them).
bool decode_layers_cluster_wanted(const DecodeShape& shape, bool any_bfp);
// The cluster form's tiled-copy descriptors (four a layer), built on the host from the layers' addresses and uploaded
// beside them; `maps_dev` null sends the step to the grid form.
size_t decode_layers_maps_bytes(const DecodeShape& shape);
bool decode_layers_make_maps(const DecodeShape& shape, const DecodeLayerPtrs* layers_host, void* maps_host);

// Text for `b200_last_error(NULL, ...)`: failures of calls that take no engine.
void set_global_error(const char* text);

// Launch set-up that belongs to a device, not to the process.  A kernel's opt-in to more than 48 KB of
// dynamic shared memory is an attribute of the function ON ONE DEVICE, and engines on different ordinals
// may live in one process and be driven from different threads: the launchers ask here before every
// launch, and the attribute is set once per (current device, kernel, largest size asked so far) under a lock.
cudaError_t ensure_dynamic_smem(const void* kernel, size_t bytes);
// An integer a launcher works out once per device (an occupancy figure), kept under the same lock.
bool device_value_get(const void* key, int* value);
void device_value_set(const void* key, int value);

}  // namespace b200
