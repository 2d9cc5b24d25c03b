/*
 * b200tt.h -- C ABI of the B200 compute engine that stands in for an
 * implementation of metalium-rs's `burn_tt::Engine` trait
 * (crates/burn-tt/src/server.rs:42-786).
 *
 * Every function mirrors one trait method: same argument meaning, same result
 * dims, same refusal behaviour.  A Rust `impl Engine for CudaEngine` binds these
 * one to one (the `rust/` sources beside the package hold that binding).
 *
 * Conventions
 *  - Tensors are opaque `b200_buffer` ids numbered by the engine
 *    (`BufferId = u64`, server.rs:862).  A tensor is a row-major `[rows, cols]`
 *    matrix; rank-N tensors are stored `[prod(leading), last]`
 *    (crates/burn-tt/src/tensor.rs:905).  F32, I32 and Bool are 32-bit words,
 *    BF16 is 16-bit.  Device layout is plain row-major, leading dimension =
 *    cols, base 256-byte aligned.
 *  - Every producing call returns the new id in `*out` and the stored dims in
 *    `out_dims[2]` (`Result<(BufferId, [usize; 2]), TtError>`).
 *  - Every call returns a status: 0 ok, else one of `b200_status` mapping onto
 *    `TtError` (crates/burn-tt/src/error.rs:26-67).  `b200_last_error` gives
 *    the cause text.  Unsupported shapes or dtypes are refused, never computed
 *    on the host.
 *  - Calls are asynchronous: they launch on the engine's stream and return.
 *    `b200_download*` and `b200_sync` are the waits and report any earlier
 *    device-side failure (server.rs:2392-2405).
 *  - One engine is driven by one thread at a time (the reference's server
 *    thread, server.rs:2801-2820); different engines may be driven
 *    concurrently.
 */
#ifndef B200TT_H
#define B200TT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200_engine b200_engine;
typedef uint64_t b200_buffer; /* server.rs:862 `BufferId` */

/* error.rs:26-67 */
enum b200_status {
  B200_OK = 0,
  B200_OUT_OF_MEMORY = 1, /* TtError::OutOfMemory{slots,free,largest} */
  B200_UNSUPPORTED = 2,   /* TtError::Unsupported */
  B200_DEVICE = 3,        /* TtError::Device */
  B200_TIMEOUT = 4,       /* TtError::Timeout */
  B200_STALE = 5,         /* TtError::StaleTensor */
  B200_DOMAIN = 6,        /* TtError::Device("... DOMAIN ..."): bad index, /0 */
  B200_NO_DEVICE = 7      /* TtError::NoDriver / NoSuchCard */
};

/* tt-kernels/src/tensor.rs:751 `Elem` (+ Elem::BF16) */
enum b200_elem { B200_F32 = 0, B200_I32 = 1, B200_BOOL = 2, B200_BF16 = 3,
                 B200_BFP8 = 4 /* Elem::Packed: block-float storage made by b200_cast_bfp, read by a product as its B */ };

/* tt-kernels/src/sfpu/reduce.rs:56 `ReduceOp`, :117 `Axis` */
enum b200_reduce_op {
  B200_SUM = 0, B200_MAX = 1, B200_PROD = 2, B200_ALL = 3, B200_ANY = 4,
  B200_BITOR = 5, B200_SUM_I32 = 6, B200_PROD_I32 = 7, B200_MIN_I32 = 8,
  B200_MAX_I32 = 9
};
enum b200_axis { B200_ROWS = 0 /* -> [1,cols] */, B200_COLS = 1 /* -> [rows,1] */ };

/* tt-kernels/src/tensor.rs:3785 `Eltwise{kind, scalar, scalar2}`; kinds are the
 * reference's numbers (tt-kernels/src/kind.rs:12-26, sfpu/ops.rs:24-251). */
typedef struct { uint32_t kind; float scalar; float scalar2; } b200_eltwise_op;
/* tt-kernels/src/tensor.rs:3479 `Block{at, transposed}` */
typedef struct { uint64_t at[2]; int32_t transposed; int32_t _pad; } b200_block;
/* tt-kernels/src/tensor.rs:6659 `BlockMove` */
typedef struct { uint64_t from[2]; uint64_t to[2]; uint64_t extent[2];
                 int32_t transposed; int32_t _pad; } b200_block_move;
/* burn-tt/src/server.rs:3449 `BlockArg{id, at, dims}` */
typedef struct { b200_buffer id; uint64_t at[2]; uint64_t dims[2]; } b200_block_arg;
/* tt-kernels/src/session.rs:802 `BatchedLayout{lhs_padded, stacked}` */
typedef struct { int32_t lhs_padded; int32_t stacked; } b200_batched_layout;
/* tt-device/src/device.rs:133 `Traffic`, re-read as host<->device copies */
typedef struct {
  uint64_t bytes_h2d, bytes_d2h, h2d_calls, d2h_calls;
  uint64_t launches;        /* kernels this engine launched */
  uint64_t pool_reserved;   /* bytes held from the driver */
  uint64_t pool_in_use;     /* bytes in live buffers */
  uint64_t pool_high_water; /* max of pool_in_use */
} b200_traffic;

/* registry.rs:31 `TtConfig`, reduced to what a GPU engine needs. */
typedef struct {
  int32_t f32_matmul_mode;   /* 0 auto, 1 FFMA only, 2 split-precision tensor cores */
  int32_t bf16_matmul_mode;  /* 0 auto, 1 SIMT only, 2 tcgen05 only (refuse otherwise) */
  uint64_t pool_limit_bytes; /* 0 = no limit beyond the device's */
  int32_t fail_alloc_at;     /* host fault hook: the Nth allocation reports OOM; 0 off */
  int32_t _pad;
  uint64_t wait_limit_cycles; /* how long a kernel of this engine waits on a barrier before it gives up and the
                               * next wait reports B200_TIMEOUT (tt-device/src/transport.rs:208-217 bounds every
                               * device wait the same way), in SM clock cycles; 0 = the default, about 2 s */
} b200_config;
/* One row of a per-op table (crates/burn-tt/src/report.rs:27-55 `OpStat`, reduced to what a GPU engine can
 * say): the label an op ran under (`set_op_label`), how often, the kernels it launched, its device time. */
typedef struct { char op[48]; uint64_t calls; uint64_t launches; double device_ms; } b200_op_stat;

/* --- attach / detach: server.rs:2738 `attach`, :2711 `AttachGuard::drop` --- */
int32_t b200_engine_create(int32_t device_ordinal, const b200_config* cfg, b200_engine** out);
void b200_engine_destroy(b200_engine* eng);
/* server.rs:75 `supports_dram`, :240 `supports_batched_layout`, :53 */
int32_t b200_supports_dram(const b200_engine* eng);
int32_t b200_supports_batched_layout(const b200_engine* eng);
int32_t b200_supports_exact_matmul(const b200_engine* eng);
/* Text of the last failure on this engine (or of a failed create when eng is NULL). */
size_t b200_last_error(const b200_engine* eng, char* buf, size_t len);
/* OutOfMemory's fields for the last B200_OUT_OF_MEMORY: need, free, largest. */
void b200_last_oom(const b200_engine* eng, uint64_t out[3]);

/* --- storage: server.rs:91,104,107,115,160,170,174,285 --- */
int32_t b200_upload_f32(b200_engine*, const float* values, uint64_t rows, uint64_t cols, b200_buffer* out);
int32_t b200_upload_bf16(b200_engine*, const uint16_t* values, uint64_t rows, uint64_t cols, b200_buffer* out);
int32_t b200_upload_bits(b200_engine*, const uint32_t* bits, uint64_t rows, uint64_t cols, int32_t elem, b200_buffer* out);
int32_t b200_download_f32(b200_engine*, b200_buffer id, float* out, uint64_t capacity_elems);
int32_t b200_download_bf16(b200_engine*, b200_buffer id, uint16_t* out, uint64_t capacity_elems);
int32_t b200_download_bits(b200_engine*, b200_buffer id, uint32_t* out, uint64_t capacity_elems);
void    b200_free(b200_engine*, b200_buffer id); /* unknown id: no-op */
int32_t b200_zeros(b200_engine*, uint64_t rows, uint64_t cols, int32_t elem, b200_buffer* out, uint64_t out_dims[2]);
/* dims and elem of a live buffer (the server's `dims_of`, server.rs:2427) */
int32_t b200_dims(const b200_engine*, b200_buffer id, uint64_t out_dims[2], int32_t* elem);
/* Device address of a live buffer, for a collective library that shares the process. */
int32_t b200_device_ptr(const b200_engine*, b200_buffer id, void** ptr, uint64_t* bytes);
/* Register caller-owned device memory as a buffer (never freed by the engine). */
int32_t b200_adopt(b200_engine*, void* device_ptr, uint64_t rows, uint64_t cols, int32_t elem, b200_buffer* out);
/* server.rs:742 `copy_into` */
int32_t b200_copy_into(b200_engine*, b200_buffer src, b200_buffer dst);
/* Overwrite a live buffer from host memory (same dims): steady-state input refresh. */
int32_t b200_write_f32(b200_engine*, b200_buffer id, const float* values, uint64_t n);
int32_t b200_write_bf16(b200_engine*, b200_buffer id, const uint16_t* values, uint64_t n);

/* --- products: server.rs:70,178,191,229,245 --- */
/* `matmul` (host-staged, required by the trait): upload, matmul_dram, download. */
int32_t b200_matmul_host(b200_engine*, const float* a, const float* b, const uint64_t mkn[3], float* out);
/* The same for BF16 operands and a BF16 result (F32 accumulate), its copies overlapped with the product in
 * row panels on two copy streams; returns when `out` is complete.  Pinned host memory gives the overlap. */
int32_t b200_matmul_host_bf16(b200_engine*, const uint16_t* a, const uint16_t* b, const uint64_t mkn[3], uint16_t* out);
/* A gated MLP's first half as one product (an extension, as `b200_attention_blocks` is): out = silu(A Bg) * (A Bu),
 * BF16 [m, n / 2], where B [k, n] holds the gate and up weights interleaved in groups of 128 columns (columns
 * [256t, 256t + 128) are gate columns 128t.., the next 128 the matching up columns; n % 256 == 0).  Bit for bit
 * `matmul_dram_bf16` on [Bg | Bu] then `SILU_MUL` on its halves (crates/tt-models/src/llama.rs:498), with neither
 * the [m, n] product nor a second launch.  Refused unless the tcgen05 path takes the product. */
int32_t b200_matmul_silu_mul(b200_engine*, b200_buffer a, b200_buffer b, b200_buffer* out, uint64_t out_dims[2]);
/* A fused QKV projection with RoPE in the product's epilogue (an extension, as `b200_matmul_silu_mul` is): out =
 * A B as BF16 [m, n] with the heads of 64 columns that lie below `rope_cols` rotated, fl(fl(x cos) + fl(swap(x) sin))
 * on the product's BF16 result, rounded once more to BF16 -- bit for bit `matmul_dram_bf16` then `rope_blocks`
 * (server.rs:566) with a BF16 result on columns [0, rope_cols) (crates/tt-models/src/llama.rs:404-433,
 * crates/tt-models/src/rope.rs:19-60).  cos_ and sin_ are F32 [r, 64] blocks (sin as [-sin, sin]); product row i
 * uses table row i % r.  Refused unless rope_cols is a multiple of 64 within n, r divides m, the tables' rows start
 * at 16-byte addresses, and the tcgen05 path takes the product. */
int32_t b200_matmul_rope(b200_engine*, b200_buffer a, b200_buffer b, const b200_block_arg* cos_, const b200_block_arg* sin_,
                         uint64_t rope_cols, b200_buffer* out, uint64_t out_dims[2]);
/* A projection into the residual stream and its norm as one product (an extension, as `b200_matmul_silu_mul` is):
 * out[0] = resid + A B (F32 [m, n]) and out[1] = RMSNorm(out[0]) * gains rounded once to BF16 -- `matmul_dram` then
 * `add_rms_norm_as(resid, product, gains, eps, 1)` (crates/tt-models/src/llama.rs:371-507) without the product's round
 * trip through memory or the second launch.  out[0] is that composition's bit for bit; out[1] sums the squares in
 * another fixed order (192 columns a CTA of a cluster, the CTAs in order), so it agrees with the composed norm to a
 * unit in the last place of the statistic.  A [m, k] and B [k, n] BF16, resid F32 [m, n], gains BF16 of n values;
 * refused unless n is one to eight tiles of 192 columns, m >= 64, k >= 64 and the driver makes the descriptors. */
int32_t b200_matmul_add_rms_norm(b200_engine*, b200_buffer a, b200_buffer b, b200_buffer resid, b200_buffer gains, float eps,
                                 b200_buffer out[2], uint64_t out_dims[2]);
/* The sharded product's fused step: C = A B (BF16 operands as stored, no transposes) written from the
 * product's epilogue into columns [col_first, col_first + n) of each of the n_dst matrices dst[i]
 * ([dst_rows, dst_cols] row-major, of the result's type) -- this GPU's C and, through b200_ipc_open,
 * every peer's, over NVLink.  No buffer is made.  The caller orders ranks around it (a barrier before a
 * reader touches C).  Refused unless the tcgen05 path takes the product. */
int32_t b200_matmul_into(b200_engine*, b200_buffer a, b200_buffer b, void* const* dst, int32_t n_dst,
                         uint64_t dst_rows, uint64_t dst_cols, uint64_t col_first, int32_t out_bf16);
/* The same for a value no product made (an activation): a block of a buffer stored into columns
 * [col_first, ...) of every dst[i] -- a rank's column slice of an all-gather, written everywhere by its owner. */
int32_t b200_store_block_into(b200_engine*, const b200_block_arg* src, void* const* dst, int32_t n_dst,
                              uint64_t dst_rows, uint64_t dst_cols, uint64_t col_first);
/* Both of the above with the exchange done by the NVSwitch: `multicast_dst` is the address of an NVLS multicast
 * object that maps the destination matrix of every GPU of a group (made by the caller: cuMulticastCreate and its
 * bindings, or a library that wraps them), and each 16-byte piece is stored there once (`multimem.st`); the switch
 * delivers it to every GPU bound to the object, this one included.  A rank's outbound bytes are then its slice
 * once, whatever the number of ranks (crates/tt-kernels/src/shard.rs:348-458 sends the slice to one chip; here every
 * rank ends with the whole C).  Refused unless the slice is whole 128-byte row segments at 16-byte addresses. */
int32_t b200_matmul_into_multicast(b200_engine*, b200_buffer a, b200_buffer b, void* multicast_dst, uint64_t dst_rows,
                                   uint64_t dst_cols, uint64_t col_first, int32_t out_bf16);
int32_t b200_store_block_into_multicast(b200_engine*, const b200_block_arg* src, void* multicast_dst, uint64_t dst_rows,
                                        uint64_t dst_cols, uint64_t col_first);
/* CUDA IPC for that: a 64-byte handle of a buffer's allocation (not of a view), opened in another process
 * as a device address valid there, closed before the owner frees the buffer. */
int32_t b200_ipc_export(b200_engine*, b200_buffer buf, uint8_t handle[64]);
int32_t b200_ipc_open(b200_engine*, const uint8_t handle[64], void** ptr);
int32_t b200_ipc_close(b200_engine*, void* ptr);
/* `matmul_dram` / `matmul_dram_bf16`: C = op(A) op(B).  F32 operands give an F32
 * result; with out_bf16 the F32 accumulator is rounded once to BF16.  BF16
 * operands accumulate in F32.  One F32 operand against one in BF16 storage (a weight kept by
 * `cast_bf16_storage`, server.rs:150) is bit for bit the F32 product with the stored operand widened. */
int32_t b200_matmul(b200_engine*, b200_buffer a, int32_t a_transposed, b200_buffer b, int32_t b_transposed,
                    int32_t out_bf16, b200_buffer* out, uint64_t out_dims[2]);
/* `matmul_dram_batched(_layout)`: one [m,k]x[k,n] product per (Block,Block) pair,
 * read where it lies; output [items*m, n] stacked, or with layout.stacked == 0
 * product i at row i*ceil(m/32)*32 (server.rs:3749-3754).  layout NULL = STACKED. */
int32_t b200_matmul_batched(b200_engine*, b200_buffer a, b200_buffer b, const b200_block* a_blocks,
                            const b200_block* b_blocks, uint64_t items, const uint64_t mkn[3],
                            const b200_batched_layout* layout, int32_t out_bf16,
                            b200_buffer* out, uint64_t out_dims[2]);

/* --- element-wise: server.rs:492,504,519,536,555 --- */
/* `eltwise_op_as`: out = a (kind) b [, c]; b/c may be 0 (absent).  b may be a's
 * shape, [1,cols], [rows,1] or whole rows repeated down a (tensor.rs:3799-3859). */
int32_t b200_eltwise(b200_engine*, const b200_eltwise_op* op, b200_buffer a, b200_buffer b, b200_buffer c,
                     int32_t out_bf16, b200_buffer* out, uint64_t out_dims[2]);
/* `eltwise_blocks_as`: the same over blocks of buffers; b, c may be NULL. */
int32_t b200_eltwise_blocks(b200_engine*, const b200_eltwise_op* op, const b200_block_arg* a,
                            const b200_block_arg* b, const b200_block_arg* c, int32_t out_bf16,
                            b200_buffer* out, uint64_t out_dims[2]);
/* server.rs:128 `cast_float`: F32 <-> BF16. */
int32_t b200_cast_float(b200_engine*, b200_buffer a, int32_t to_bf16, b200_buffer* out, uint64_t out_dims[2]);
/* server.rs:141 `cast_bfp(id, format)`: explicit block-float storage (crates/tt-kernels/src/bfp.rs:60-63: sixteen
 * consecutive values of a row share an 8-bit exponent, a datum is a sign over a 7-bit magnitude).  format 8: an F32 or
 * BF16 [rows, cols] buffer (cols % 16 == 0) -> a B200_BFP8 buffer of 17 bytes for 16 values; format 0 (the trait's
 * `None`): a BFP8 buffer widened to F32; format -16: widened to BF16 (exact: every decoded value is a BF16 value).
 * Decoding is the reference's `bfp8_to_bf16` (crates/tt-isa/src/tile.rs:619-634); encoding rounds |x| 2^(133 - E) to
 * nearest even under the group's largest exponent E, so a decoded value is within half a step 2^(E - 133) of what was
 * stored; -0 and values that round to magnitude 0 are stored +0 (the format has no -0), groups below 2^-119 are stored as
 * zeros, and a group with an infinity or a NaN keeps those and zeroes its finite members.  BFP4 and BFP2 are refused.
 * `b200_matmul` takes a BFP8 buffer as B (not transposed): bit for bit the product with B widened.  Every other op
 * refuses a BFP8 buffer. */
int32_t b200_cast_bfp(b200_engine*, b200_buffer a, int32_t format, b200_buffer* out, uint64_t out_dims[2]);
/* The stored bytes of a BFP8 buffer: rows * cols datums (row-major) and rows * cols / 16 exponents (row-major). */
int32_t b200_download_bfp(b200_engine*, b200_buffer id, uint8_t* datums, uint8_t* exponents, uint64_t capacity_datums);
/* server.rs:566 `rope_blocks` */
int32_t b200_rope_blocks(b200_engine*, const b200_block_arg* x, const b200_block_arg* cos_,
                         const b200_block_arg* sin_, uint64_t head, int32_t out_bf16,
                         b200_buffer* out, uint64_t out_dims[2]);

/* --- reductions: server.rs:80,399,404,423,428,438,449,466,477 --- */
/* `reduce(a, op, axis, then)`: then_kind 0 = none, else an exact unary kind
 * applied to the result with scalar bits then_bits (tensor.rs:6038). */
int32_t b200_reduce(b200_engine*, b200_buffer a, int32_t op, int32_t axis, uint32_t then_kind,
                    uint32_t then_bits, b200_buffer* out, uint64_t out_dims[2]);
int32_t b200_sum_rows(b200_engine*, b200_buffer a, b200_buffer* out, uint64_t out_dims[2]);
/* Burn's `float_sum` / `float_mean` of a resident tensor (ops.rs:3246-3398): [1,1]. */
int32_t b200_full_sum(b200_engine*, b200_buffer a, int32_t mean, b200_buffer* out, uint64_t out_dims[2]);
/* No counterpart in the reference.  The full sum (or mean) of `n` F32 values for a caller
 * that must not allocate device memory -- a host whose GPU memory belongs to another
 * runtime's fixed arenas, or code on a path where an allocation would stall the device.
 * `device_values` and `device_out` (one float) are the caller's device memory; the call
 * launches on `cuda_stream` (a cudaStream_t; NULL is the default stream) of the current
 * device and returns without waiting.  It calls no cudaMalloc or cudaFree: the per-block
 * partial sums go to a fixed 4,768-byte array inside the library image, which every GPU
 * that loads the library holds until exit.
 *  - n may not exceed 2^31 (B200_UNSUPPORTED, text through b200_last_error(NULL, ..)).
 *  - The first call on each device looks the array's address up; make that call before
 *    any stream capture begins.
 *  - All calls share the array and it keeps the last call's contents.  The partials need no
 *    clearing (each is rewritten before it is read); the ticket word behind them is cleared on
 *    `cuda_stream` ahead of every launch, so a call that was cut short leaves nothing behind
 *    for the next one.  Two calls that overlap on one GPU -- different streams, or different
 *    threads -- still race on the array and either may give a wrong sum or none: order them.
 *  - n = 0 gives 0.0 for the sum; the mean of nothing is refused (B200_UNSUPPORTED).
 *  - The result has the same bits as b200_full_sum's on the same values. */
int32_t b200_full_sum_noalloc(const float* device_values, uint64_t n, int32_t mean, float* device_out,
                              void* cuda_stream);
/* `full_reduce(values, dims, mean)`: host values in, scalar out, device arithmetic. */
int32_t b200_full_reduce(b200_engine*, const float* values, const uint64_t dims[2], int32_t mean, float* out);
/* `softmax_rows(x, mask, scale)`: mask 0 = none; Bool words, read for rows r % mask_rows. */
int32_t b200_softmax_rows(b200_engine*, b200_buffer x, b200_buffer mask, float scale,
                          b200_buffer* out, uint64_t out_dims[2]);
/* `softmax_rows` with its result's type named, as the reference's `_as` methods do
 * (`rms_norm_as` server.rs:449, `eltwise_op_as` :519): out_bf16 rounds the F32 probabilities
 * once, bit for bit `softmax_rows` then `cast_float`, with no F32 result written. */
int32_t b200_softmax_rows_as(b200_engine*, b200_buffer x, b200_buffer mask, float scale, int32_t out_bf16,
                             b200_buffer* out, uint64_t out_dims[2]);
/* Burn's `activation::log_softmax` over the last dim (ops.rs:5153-5158). */
int32_t b200_log_softmax_rows(b200_engine*, b200_buffer x, b200_buffer* out, uint64_t out_dims[2]);
int32_t b200_rms(b200_engine*, b200_buffer a, float eps, b200_buffer* out, uint64_t out_dims[2]);
int32_t b200_rms_norm(b200_engine*, b200_buffer a, b200_buffer gamma, float eps, int32_t out_bf16,
                      b200_buffer* out, uint64_t out_dims[2]);
/* `add_rms_norm`: s = a + b and s's RMSNorm: (s, norm). */
int32_t b200_add_rms_norm(b200_engine*, b200_buffer a, b200_buffer b, b200_buffer gamma, float eps,
                          b200_buffer out[2], uint64_t out_dims[2]);
/* `add_rms_norm` with the norm's type named, as `rms_norm_as` (server.rs:449) names it: norm_bf16
 * rounds the F32 norm once, bit for bit `add_rms_norm` then `cast_float` of the norm; s stays in
 * the operands' type. */
int32_t b200_add_rms_norm_as(b200_engine*, b200_buffer a, b200_buffer b, b200_buffer gamma, float eps,
                             int32_t norm_bf16, b200_buffer out[2], uint64_t out_dims[2]);
/* `argmax_row`: a [rows, cols] -> [rows, 1] I32 (the trait passes one row). */
int32_t b200_argmax_row(b200_engine*, b200_buffer a, b200_buffer* out, uint64_t out_dims[2]);

/* --- indexing: server.rs:269,277,293,300,329,339,349,358,368,379,482 --- */
int32_t b200_select_rows(b200_engine*, b200_buffer table, b200_buffer indices, b200_buffer* out, uint64_t out_dims[2]);
int32_t b200_pick_columns(b200_engine*, b200_buffer input, b200_buffer indices, b200_buffer* out, uint64_t out_dims[2]);
/* Burn's scatter-add of a [rows,1] value at (r, idx[r]) into a copy of t (ops.rs:1043). */
int32_t b200_scatter_add_columns(b200_engine*, b200_buffer t, b200_buffer indices, b200_buffer value,
                                 b200_buffer* out, uint64_t out_dims[2]);
int32_t b200_select_add_rows(b200_engine*, b200_buffer t, b200_buffer indices, b200_buffer value,
                             b200_buffer* out, uint64_t out_dims[2]);
int32_t b200_rows_add(b200_engine*, b200_buffer t, const uint64_t* indices, uint64_t n, b200_buffer value,
                      b200_buffer* out, uint64_t out_dims[2]);
int32_t b200_assign_rows(b200_engine*, b200_buffer t, b200_buffer value, const uint64_t* dst_src_pairs,
                         uint64_t n, b200_buffer* out, uint64_t out_dims[2]);
int32_t b200_scatter_rows(b200_engine*, b200_buffer table, b200_buffer indices, b200_buffer values,
                          int32_t column, b200_buffer* out, uint64_t out_dims[2]);
/* `scatter_rows_into` (server.rs:389): `scatter_rows` into `table` itself -- a KV cache's step
 * write.  values is a [n, table cols] block of a buffer of the table's type (F32, I32 or BF16), or of an F32
 * buffer for a BF16 table: each value is then rounded once, as `cast_float` would round it. */
int32_t b200_scatter_rows_into(b200_engine*, b200_buffer table, b200_buffer indices, const b200_block_arg* values,
                               int32_t column);
/* The same words seen as another [rows, cols] (rows * cols unchanged): a view, no copy, the parent
 * kept alive as `slice_rows` keeps it.  burn-tt reshapes contiguous tensors above the trait
 * (`views::Strided`); a caller of this ABI needs it to hand `attention_rows`' result row to a
 * product as [tokens, heads * dv]. */
int32_t b200_reshape(b200_engine*, b200_buffer a, uint64_t rows, uint64_t cols, b200_buffer* out, uint64_t out_dims[2]);
int32_t b200_gather_indexed(b200_engine*, b200_buffer input, b200_buffer indices, b200_buffer* out, uint64_t out_dims[2]);
/* `gather_rows(sources, rows:[(source, row)], cols)` */
int32_t b200_gather_rows(b200_engine*, const b200_buffer* sources, uint64_t n_sources,
                         const uint64_t* source_row_pairs, uint64_t n_rows, uint64_t cols,
                         b200_buffer* out, uint64_t out_dims[2]);
/* `slice_rows`: a view, no copy; the parent stays alive while a view is. */
int32_t b200_slice_rows(b200_engine*, b200_buffer a, uint64_t first, uint64_t rows, b200_buffer* out, uint64_t out_dims[2]);
int32_t b200_copy_blocks(b200_engine*, b200_buffer a, const b200_block_move* moves, uint64_t n,
                         const uint64_t dims[2], b200_buffer* out, uint64_t out_dims[2]);
/* `repack(a, sources:[[row,col]] in output order, dims)` */
int32_t b200_repack(b200_engine*, b200_buffer a, const uint64_t* row_col_pairs, const uint64_t dims[2],
                    b200_buffer* out, uint64_t out_dims[2]);

/* `repack_many(inputs, sources:[(input, [row, col])] in output order, dims)` (server.rs:317;
 * crates/tt-kernels/src/tensor.rs:6791): triples = {input ordinal, row, col} an output element; the inputs
 * share one element type; rows * cols == n_triples and neither is zero, else UNSUPPORTED; a source outside
 * its input is DOMAIN. */
int32_t b200_repack_many(b200_engine*, const b200_buffer* inputs, uint64_t n_inputs, const uint64_t* triples,
                         uint64_t n_triples, const uint64_t dims[2], b200_buffer* out, uint64_t out_dims[2]);
/* `select_taps(table, indices [taps, n] I32, zero_row)` (server.rs:309; crates/tt-kernels/src/index.rs:136-160,
 * crates/tt-kernels/src/session.rs:8068-8084): the result is [n, (taps - 1) * ceil32(cols) + cols]; its row i
 * holds row indices[t][i] of the table from column t * ceil32(cols) for each tap t, and zeros in the columns
 * between one tap's end and the next one's start.  With zero_row an index equal to the table's rows reads a
 * row of zeros.  Any other index outside the table sets DOMAIN on the device. */
int32_t b200_select_taps(b200_engine*, b200_buffer table, b200_buffer indices, int32_t zero_row, b200_buffer* out,
                         uint64_t out_dims[2]);
/* server.rs:137 `cast_block`: `cast_float` of a block of a buffer, a new buffer of the block's dims. */
int32_t b200_cast_block(b200_engine*, const b200_block_arg* a, int32_t to_bf16, b200_buffer* out, uint64_t out_dims[2]);
/* server.rs:779 `cast_f16`: F32 -> IEEE binary16 (ties to even, subnormals kept, NaN quiet with its top ten
 * payload bits) in a two-byte buffer that reads back through `b200_download_bf16`, as the reference keeps FP16
 * in BF16's raw storage (server.rs:2189-2200); or such a buffer widened, exactly, to F32. */
int32_t b200_cast_f16(b200_engine*, b200_buffer a, int32_t to_f16, b200_buffer* out, uint64_t out_dims[2]);
/* server.rs:578 `pow`: x^y as powf; exponent_kind 0 = an F32 buffer of x's shape, 1 = the scalar, 2 = an I32
 * buffer of x's shape (`PowArg`, server.rs:35-39).  The kinds are POW, POW_S and POW_I of `b200_eltwise`. */
int32_t b200_pow(b200_engine*, b200_buffer x, int32_t exponent_kind, b200_buffer y, float scalar, b200_buffer* out,
                 uint64_t out_dims[2]);
/* server.rs:414 `scan`: inclusive scan down the rows of every column (crates/tt-kernels/src/sfpu/scan.rs:19-41).
 * F32 Sum and Prod are left folds in row order from +0.0 and 1.0; Min/Max order raw words by `total_cmp`;
 * MinNan/MaxNan take a NaN, keep the earlier of equal values; the I* ops take and give I32 (wrapping sum and
 * product, signed min and max).  The input's element type must be the op's. */
enum b200_scan_op { B200_SCAN_SUM = 0, B200_SCAN_PROD, B200_SCAN_MIN, B200_SCAN_MAX, B200_SCAN_MIN_NAN,
                    B200_SCAN_MAX_NAN, B200_SCAN_ISUM, B200_SCAN_IPROD, B200_SCAN_IMIN, B200_SCAN_IMAX };
int32_t b200_scan(b200_engine*, b200_buffer a, int32_t op, b200_buffer* out, uint64_t out_dims[2]);
/* server.rs:758 `sort_planes` with `Spec{elem, n, descending, indices}` (crates/tt-kernels/src/sfpu/sort.rs:112-122):
 * `a` is a planes matrix [32 * T, 32 * blocks], T the power of two of 32-position tiles holding n <= 1024
 * positions, problem q's position e at sort.rs:198's coordinate.  keys (a's shape and type) and, when
 * `indices` is not NULL, the original positions (I32) hold each problem's first n positions in the stable
 * order on (key, index): `total_cmp` for F32, two's complement for I32, keys reversed when descending.  What
 * lies past n is unspecified, as in the reference (sort.rs:699-700). */
int32_t b200_sort_planes(b200_engine*, b200_buffer a, int32_t elem, uint64_t n, int32_t descending,
                         b200_buffer* keys, b200_buffer* indices, uint64_t out_dims[2]);
/* server.rs:768 `random_dram(dims, draw, base)`: a tensor drawn on the device from the seed `base`, with no
 * upload.  draw (crates/burn-tt/src/random.rs:73-90): 0 Unit [0,1); 1 Uniform(a, b) -> [a, b); 2 Bernoulli(p = a);
 * 3 Normal(mean a, std b); 4 IntRange(lo, hi) -> [lo, hi), hi - lo <= 2^23; 5 IntWords.  as_int makes Bernoulli
 * and Normal I32 (the normal truncated toward zero).  A datum depends on (base, draw, position) only.  The
 * stream is this engine's own: the reference's differs between its simulator and its silicon and is not a
 * value to match (crates/tt-kernels/src/prng.rs:49-50); the distributions' arithmetic is the reference's. */
int32_t b200_random(b200_engine*, const uint64_t dims[2], int32_t draw, float a, float b, int32_t lo, int32_t hi,
                    int32_t as_int, uint64_t base, b200_buffer* out, uint64_t out_dims[2]);
/* server.rs:118 `pool_bf16(a, windows, divisors, dims)` (crates/tt-kernels/src/fpu.rs:39-132): `a` is BF16; window w
 * is coords[2 * offsets[w] .. 2 * offsets[w + 1]) as [row, col] pairs; the F32 [dims] result holds at element w (row
 * major) the window's sum, taken sixteen values a block with the blocks' partial sums added in order, divided by
 * divisors[w].  Refused as the reference refuses (fpu.rs:48-57): dims[0] * dims[1] != n_windows, no windows, an
 * empty window, a divisor of 0 or above 2^24; a coordinate outside `a` is DOMAIN. */
int32_t b200_pool_bf16(b200_engine*, b200_buffer a, const uint64_t* offsets, const uint64_t* coords, const uint64_t* divisors,
                       uint64_t n_windows, const uint64_t dims[2], b200_buffer* out, uint64_t out_dims[2]);
/* server.rs:95 `metadata`: operation geometry as a resident buffer of words (an upload whose content the
 * engine may keep and share). */
int32_t b200_metadata(b200_engine*, const uint32_t* bits, const uint64_t dims[2], int32_t elem, b200_buffer* out);
/* server.rs:705 `gddr_free_bytes`: (largest block that can be had now, all free bytes) of device memory,
 * the pool's idle blocks included. */
int32_t b200_free_bytes(b200_engine*, uint64_t out[2]);

/* --- attention for a few query rows a key/value head, as one op: server.rs:257 `attention_rows`
 * (kernel contract: crates/tt-kernels/src/attention.rs:360-372).  buffers = [q, k, v, mask]; item i
 * names the top-left element of head i's blocks: q_i [m, d] (F32), K_i [l, d] and V_i [l, dv]
 * (both F32 or both BF16, read as they lie), mask the Bool [1, l] of positions not attended, the
 * same for every row.  dims = [m, d, l, dv].  The result is the F32 [1, n_items * m * dv] row: the
 * heads' rows stacked in row-major order.  out_i = softmax(scale * q_i K_i^T, masked) V_i with the
 * composition's steps (product, scale then mask fill, clamped maximum, exp, clamped sum, division,
 * product).  Refused (UNSUPPORTED) unless 1 <= m <= 32 and d, l, dv are positive multiples of 32
 * (attention.rs:156-171), the key and value blocks start at a column that is a multiple of 4 (F32)
 * or 8 (BF16) in buffers whose width is one, and every block lies inside its buffer.  Heads that
 * name the same key and value blocks (grouped-query attention) read them once. */
typedef struct b200_attention_item { uint64_t q[2], k[2], v[2]; } b200_attention_item;
int32_t b200_attention_rows(b200_engine*, const b200_buffer buffers[4], const b200_attention_item* items,
                            uint64_t n_items, const uint64_t dims[4], float scale,
                            b200_buffer* out, uint64_t out_dims[2]);
/* The same with the result's type named, as the trait's `_as` methods name it (server.rs:449): out_bf16 rounds
 * each F32 result once, bit for bit `attention_rows` then `cast_float` (the projection after it reads BF16). */
int32_t b200_attention_rows_as(b200_engine*, const b200_buffer buffers[4], const b200_attention_item* items,
                               uint64_t n_items, const uint64_t dims[4], float scale, int32_t out_bf16,
                               b200_buffer* out, uint64_t out_dims[2]);

/* --- attention over whole sequences, fused (an extension beyond the `Engine` trait, as
 * `b200_softmax_rows_as` is): what burn-tt composes in `padded_attention` (ops.rs:4825-4960: a
 * batched Q K^T, `SCALE_MASK_FILL` with the causal blocks, the row softmax, a batched P V) as one
 * kernel, the scores never written.  q, k, v are BF16 buffers; block i names the top-left element
 * of its Q [sq, d], K [sk, d] and V [sk, dv] blocks and of its [sq, dv] block of the result.
 * dims = [sq, d, sk, dv].  causal: query row r sees keys 0..r + (sk - sq).  The result is a new
 * BF16 [result_dims] buffer; elements no block covers are zero.  F32 accumulation, the
 * probabilities rounded to BF16 before the product with V (as `b200_softmax_rows_as` + the BF16
 * product do).  sq and sk are any positive lengths (ragged heads are what ops.rs:4838-4842 pads): a tail tile reads
 * the rows that follow its block in the buffer (zeros past the buffer's end) and keeps them out of every maximum and
 * sum; value rows read that way are weighted by exact zeros, so they must be finite.  Refused (UNSUPPORTED) unless
 * d = dv is 64 or 128, scale > 0, sk >= sq when causal, and every column offset and buffer width is a multiple of 8. */
typedef struct b200_attention_block { uint64_t q[2], k[2], v[2], o[2]; } b200_attention_block;
int32_t b200_attention_blocks(b200_engine*, b200_buffer q, b200_buffer k, b200_buffer v,
                              const b200_attention_block* items, uint64_t n_items, const uint64_t dims[4],
                              float scale, int32_t causal, const uint64_t result_dims[2],
                              b200_buffer* out, uint64_t out_dims[2]);

/* --- one generation step through every layer, as one launch (an extension beside the trait, as
 * `b200_attention_blocks` is).  The reference's generation replays a trace of its step (crates/tt-models/src/
 * generate.rs:781); composed from the trait's ops a step is eleven launches a layer whose latencies dwarf the work of
 * reading a layer's weights once, so the layers' device work is also offered as ONE cooperative kernel (five grid
 * barriers a layer, every one bounded: B200_TIMEOUT when one runs out).
 *   x               [rows, hidden] F32: the embedded tokens, one row a sequence (1 <= rows <= 4)
 *   layer_buffers   8 ids a layer: norm1 gain, Wqkv [hidden, (heads + 2 kv_heads) 64], Wo [heads 64, hidden], norm2 gain,
 *                   Wgate|Wup [hidden, 2 ff], Wdown [ff, hidden], key cache, value cache ([rows * max_len, kv_heads 64]
 *                   BF16, position-major as crates/tt-models/src/kv_cache.rs:5-11).  Gains BF16; matrices BF16 or BFP8.
 *   cos/sin tables  F32 [max_len, 64] (sin as [-sin, sin]: crates/tt-models/src/rope.rs:19-60); position: one I32 on the
 *                   device, the step's position in every sequence (a position outside the cache is DOMAIN).
 * Per layer (crates/tt-models/src/llama.rs:371-507): RMSNorm, QKV (rounded to BF16), RoPE in F32, the key (rounded once
 * to BF16) and value written into the cache at `position`, attention over positions 0..position of the first `attend`
 * (scale, mask, softmax, P V; a BF16 result), the output projection, the residual add, RMSNorm, gate|up (BF16),
 * SILU_MUL (BF16), down, the residual add.  The result is the final RMSNorm of the stream as BF16 [rows, hidden]: the
 * head product's input.  The same steps, roundings included, as the composed sequence of trait ops; sums are taken in
 * this kernel's own fixed order, so the two agree to F32 rounding, not bit for bit.  Refused unless head_dim is 64,
 * heads / kv_heads <= 4, hidden and ff are multiples of 64 and attend is a multiple of 64 within max_len. */
typedef struct { uint32_t layers, hidden, heads, kv_heads, head_dim, ff, max_len, attend; float eps, scale; } b200_decode_shape;
int32_t b200_decode_layers(b200_engine*, const b200_decode_shape* shape, b200_buffer x, const b200_buffer* layer_buffers,
                           b200_buffer final_norm, b200_buffer cos_table, b200_buffer sin_table, b200_buffer position,
                           b200_buffer* out, uint64_t out_dims[2]);

/* --- traces: server.rs:591 `begin_trace`, :595 `end_trace`, :650 `run_trace`, :660 `release_trace`.
 * Ops issued between begin and end are captured into a CUDA graph instead of running; a replay
 * runs them again on the same buffers.  Inputs are buffers made before the capture (refresh them
 * with b200_write_* or b200_copy_into), outputs are buffers made during it and still live at
 * end_trace (read them after each replay).  Run the same ops once before capturing, so every
 * kernel is loaded.  No upload, download or sync may be issued inside a capture. */
int32_t b200_begin_trace(b200_engine*);
int32_t b200_end_trace(b200_engine*, uint64_t* trace);
int32_t b200_run_trace(b200_engine*, uint64_t trace);
void    b200_release_trace(b200_engine*, uint64_t trace);
/* server.rs:688 `trace_footprint`: the device bytes a trace holds until it is released (the blocks its capture
 * took; the reference reports stream and program-cache bytes a unit, which a CUDA graph does not have). */
int32_t b200_trace_footprint(const b200_engine*, uint64_t trace, uint64_t* bytes);
/* server.rs:664 `trace_ops`: the ops the trace captured, in order, each with its label and its kernels.
 * Fills at most `capacity` rows; *n is the number of ops. */
int32_t b200_trace_ops(const b200_engine*, uint64_t trace, b200_op_stat* out, uint64_t capacity, uint64_t* n);

/* --- waits and observability: lib.rs:218 `sync`, server.rs:584,663 --- */
int32_t b200_sync(b200_engine*);
/* server.rs:662 `set_op_label`: names the device work queued from here on (the server labels every job before it
 * runs it, server.rs:2370).  The label prefixes error text, is kept with a capture's ops, and keys the profile. */
void    b200_set_op_label(b200_engine*, const char* label);
/* The profile mode (server.rs:672 `profile_mode`, :683 `profile_report`; crates/burn-tt/src/profile.rs:1-48):
 * between start and stop every `b200_set_op_label` puts an event on the stream, and the device time up to the
 * next label is charged to that label.  `b200_profile_stop` is a wait; `b200_profile_read` then gives one row a
 * label in order of first appearance (at most `capacity` rows; *n is the number of labels).  Off by default:
 * an event a label costs about a microsecond of host time. */
int32_t b200_profile_start(b200_engine*);
int32_t b200_profile_stop(b200_engine*);
int32_t b200_profile_read(const b200_engine*, b200_op_stat* out, uint64_t capacity, uint64_t* n);
/* Launches one CTA whose bounded wait can never be satisfied, so that the time-out path (error.rs:40 `Timeout`)
 * runs on a healthy GPU: the wait gives up at `wait_limit_cycles`, the next wait returns B200_TIMEOUT, and the
 * CUDA context stays usable.  Refused unless the engine was made with a limit of at most 2e9 cycles. */
int32_t b200_debug_stalled_wait(b200_engine*);
/* The tensor-core products of this engine use at most `sms` SMs from now on (0 = all): a caller that
 * runs a collective beside a product (the sharded product's all-gather) leaves it SMs to run on. */
void    b200_set_matmul_sm_limit(b200_engine*, int32_t sms);
void    b200_traffic_get(const b200_engine*, b200_traffic* out);
/* Device time of the ops launched between the two marks, in milliseconds
 * (CUDA events on the engine's stream).  `b200_timer_stop` is a wait. */
int32_t b200_timer_start(b200_engine*);
int32_t b200_timer_stop(b200_engine*, float* ms);
/* The engine's stream as a `cudaStream_t`, for a caller that shares the process. */
void*   b200_stream(const b200_engine*);
/* Name of the kernel path the last product took: "tcgen05" (one CTA a tile), "tcgen05-pair" (CTA pairs),
 * "tcgen05-tf32x3", "skinny", "simt". */
const char* b200_last_matmul_path(const b200_engine*);
/* Name of the form the last `b200_decode_layers` took: "cluster16x3" and the like (that many clusters -- 2 to 4 -- of
 * 16 or 8 blocks, sharing a layer's heads and ff), "cluster16" or "cluster8" (one thread-block cluster of that many
 * blocks), "grid" (a cooperative grid), "none" before the first. */
const char* b200_last_decode_form(const b200_engine*);

#ifdef __cplusplus
}
#endif
#endif /* B200TT_H */
