//! Raw FFI of libb200tt (include/b200tt.h), one declaration per C function.
//! Generated from the header; the header's comments name the `burn_tt::Engine` method
//! (crates/burn-tt/src/server.rs) each function stands in for.
//! Shipped as source: it has not met a Rust compiler.
#![allow(non_camel_case_types)]
use std::os::raw::{c_char, c_void};

#[repr(C)] pub struct b200_engine { _private: [u8; 0] }
#[repr(C)] #[derive(Clone, Copy, Default)] pub struct b200_config { pub f32_matmul_mode: i32, pub bf16_matmul_mode: i32, pub pool_limit_bytes: u64, pub fail_alloc_at: i32, pub _pad: i32, pub wait_limit_cycles: u64 }
#[repr(C)] #[derive(Clone, Copy)] pub struct b200_decode_shape { pub layers: u32, pub hidden: u32, pub heads: u32, pub kv_heads: u32, pub head_dim: u32, pub ff: u32, pub max_len: u32, pub attend: u32, pub eps: f32, pub scale: f32 }
#[repr(C)] #[derive(Clone, Copy)] pub struct b200_op_stat { pub op: [c_char; 48], pub calls: u64, pub launches: u64, pub device_ms: f64 }
#[repr(C)] #[derive(Clone, Copy)] pub struct b200_eltwise_op { pub kind: u32, pub scalar: f32, pub scalar2: f32 }
#[repr(C)] #[derive(Clone, Copy)] pub struct b200_block { pub at: [u64; 2], pub transposed: i32, pub _pad: i32 }
#[repr(C)] #[derive(Clone, Copy)] pub struct b200_attention_block { pub q: [u64; 2], pub k: [u64; 2], pub v: [u64; 2], pub o: [u64; 2] }
#[repr(C)] #[derive(Clone, Copy)] pub struct b200_attention_item { pub q: [u64; 2], pub k: [u64; 2], pub v: [u64; 2] }
#[repr(C)] #[derive(Clone, Copy)] pub struct b200_block_move { pub from: [u64; 2], pub to: [u64; 2], pub extent: [u64; 2], pub transposed: i32, pub _pad: i32 }
#[repr(C)] #[derive(Clone, Copy)] pub struct b200_block_arg { pub id: u64, pub at: [u64; 2], pub dims: [u64; 2] }
#[repr(C)] #[derive(Clone, Copy)] pub struct b200_batched_layout { pub lhs_padded: i32, pub stacked: i32 }
#[repr(C)] #[derive(Clone, Copy, Default)] pub struct b200_traffic { pub bytes_h2d: u64, pub bytes_d2h: u64, pub h2d_calls: u64, pub d2h_calls: u64, pub launches: u64, pub pool_reserved: u64, pub pool_in_use: u64, pub pool_high_water: u64 }

extern "C" {
    pub fn b200_engine_create(device_ordinal: i32, cfg: *const b200_config, out: *mut *mut b200_engine) -> i32;
    pub fn b200_engine_destroy(eng: *mut b200_engine);
    pub fn b200_supports_dram(eng: *const b200_engine) -> i32;
    pub fn b200_supports_batched_layout(eng: *const b200_engine) -> i32;
    pub fn b200_supports_exact_matmul(eng: *const b200_engine) -> i32;
    pub fn b200_last_error(eng: *const b200_engine, buf: *mut c_char, len: usize) -> usize;
    pub fn b200_last_oom(eng: *const b200_engine, out: *mut u64);
    pub fn b200_upload_f32(a0: *mut b200_engine, values: *const f32, rows: u64, cols: u64, out: *mut u64) -> i32;
    pub fn b200_upload_bf16(a0: *mut b200_engine, values: *const u16, rows: u64, cols: u64, out: *mut u64) -> i32;
    pub fn b200_upload_bits(a0: *mut b200_engine, bits: *const u32, rows: u64, cols: u64, elem: i32, out: *mut u64) -> i32;
    pub fn b200_download_f32(a0: *mut b200_engine, id: u64, out: *mut f32, capacity_elems: u64) -> i32;
    pub fn b200_download_bf16(a0: *mut b200_engine, id: u64, out: *mut u16, capacity_elems: u64) -> i32;
    pub fn b200_download_bits(a0: *mut b200_engine, id: u64, out: *mut u32, capacity_elems: u64) -> i32;
    pub fn b200_free(a0: *mut b200_engine, id: u64);
    pub fn b200_zeros(a0: *mut b200_engine, rows: u64, cols: u64, elem: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_dims(a0: *const b200_engine, id: u64, out_dims: *mut u64, elem: *mut i32) -> i32;
    pub fn b200_device_ptr(a0: *const b200_engine, id: u64, ptr: *mut *mut c_void, bytes: *mut u64) -> i32;
    pub fn b200_adopt(a0: *mut b200_engine, device_ptr: *mut c_void, rows: u64, cols: u64, elem: i32, out: *mut u64) -> i32;
    pub fn b200_copy_into(a0: *mut b200_engine, src: u64, dst: u64) -> i32;
    pub fn b200_write_f32(a0: *mut b200_engine, id: u64, values: *const f32, n: u64) -> i32;
    pub fn b200_write_bf16(a0: *mut b200_engine, id: u64, values: *const u16, n: u64) -> i32;
    pub fn b200_matmul_host(a0: *mut b200_engine, a: *const f32, b: *const f32, mkn: *const u64, out: *mut f32) -> i32;
    pub fn b200_matmul(a0: *mut b200_engine, a: u64, a_transposed: i32, b: u64, b_transposed: i32, out_bf16: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_matmul_batched(a0: *mut b200_engine, a: u64, b: u64, a_blocks: *const b200_block, b_blocks: *const b200_block, items: u64, mkn: *const u64, layout: *const b200_batched_layout, out_bf16: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_eltwise(a0: *mut b200_engine, op: *const b200_eltwise_op, a: u64, b: u64, c: u64, out_bf16: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_eltwise_blocks(a0: *mut b200_engine, op: *const b200_eltwise_op, a: *const b200_block_arg, b: *const b200_block_arg, c: *const b200_block_arg, out_bf16: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_cast_float(a0: *mut b200_engine, a: u64, to_bf16: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_cast_bfp(a0: *mut b200_engine, a: u64, format: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_download_bfp(a0: *mut b200_engine, id: u64, datums: *mut u8, exponents: *mut u8, capacity_datums: u64) -> i32;
    pub fn b200_rope_blocks(a0: *mut b200_engine, x: *const b200_block_arg, cos_: *const b200_block_arg, sin_: *const b200_block_arg, head: u64, out_bf16: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_reduce(a0: *mut b200_engine, a: u64, op: i32, axis: i32, then_kind: u32, then_bits: u32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_sum_rows(a0: *mut b200_engine, a: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_full_sum(a0: *mut b200_engine, a: u64, mean: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_full_sum_noalloc(device_values: *const f32, n: u64, mean: i32, device_out: *mut f32, cuda_stream: *mut c_void) -> i32;
    pub fn b200_full_reduce(a0: *mut b200_engine, values: *const f32, dims: *const u64, mean: i32, out: *mut f32) -> i32;
    pub fn b200_softmax_rows(a0: *mut b200_engine, x: u64, mask: u64, scale: f32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_softmax_rows_as(a0: *mut b200_engine, x: u64, mask: u64, scale: f32, out_bf16: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_log_softmax_rows(a0: *mut b200_engine, x: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_rms(a0: *mut b200_engine, a: u64, eps: f32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_rms_norm(a0: *mut b200_engine, a: u64, gamma: u64, eps: f32, out_bf16: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_add_rms_norm(a0: *mut b200_engine, a: u64, b: u64, gamma: u64, eps: f32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_add_rms_norm_as(a0: *mut b200_engine, a: u64, b: u64, gamma: u64, eps: f32, norm_bf16: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_argmax_row(a0: *mut b200_engine, a: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_select_rows(a0: *mut b200_engine, table: u64, indices: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_pick_columns(a0: *mut b200_engine, input: u64, indices: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_scatter_add_columns(a0: *mut b200_engine, t: u64, indices: u64, value: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_select_add_rows(a0: *mut b200_engine, t: u64, indices: u64, value: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_rows_add(a0: *mut b200_engine, t: u64, indices: *const u64, n: u64, value: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_assign_rows(a0: *mut b200_engine, t: u64, value: u64, dst_src_pairs: *const u64, n: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_scatter_rows(a0: *mut b200_engine, table: u64, indices: u64, values: u64, column: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_gather_indexed(a0: *mut b200_engine, input: u64, indices: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_gather_rows(a0: *mut b200_engine, sources: *const u64, n_sources: u64, source_row_pairs: *const u64, n_rows: u64, cols: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_slice_rows(a0: *mut b200_engine, a: u64, first: u64, rows: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_copy_blocks(a0: *mut b200_engine, a: u64, moves: *const b200_block_move, n: u64, dims: *const u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_repack(a0: *mut b200_engine, a: u64, row_col_pairs: *const u64, dims: *const u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_repack_many(a0: *mut b200_engine, inputs: *const u64, n_inputs: u64, triples: *const u64, n_triples: u64, dims: *const u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_select_taps(a0: *mut b200_engine, table: u64, indices: u64, zero_row: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_cast_block(a0: *mut b200_engine, a: *const b200_block_arg, to_bf16: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_cast_f16(a0: *mut b200_engine, a: u64, to_f16: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_pow(a0: *mut b200_engine, x: u64, exponent_kind: i32, y: u64, scalar: f32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_scan(a0: *mut b200_engine, a: u64, op: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_sort_planes(a0: *mut b200_engine, a: u64, elem: i32, n: u64, descending: i32, keys: *mut u64, indices: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_random(a0: *mut b200_engine, dims: *const u64, draw: i32, a: f32, b: f32, lo: i32, hi: i32, as_int: i32, base: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_pool_bf16(a0: *mut b200_engine, a: u64, offsets: *const u64, coords: *const u64, divisors: *const u64, n_windows: u64, dims: *const u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_metadata(a0: *mut b200_engine, bits: *const u32, dims: *const u64, elem: i32, out: *mut u64) -> i32;
    pub fn b200_free_bytes(a0: *mut b200_engine, out: *mut u64) -> i32;
    pub fn b200_attention_blocks(a0: *mut b200_engine, q: u64, k: u64, v: u64, items: *const b200_attention_block, n_items: u64, dims: *const u64, scale: f32, causal: i32, result_dims: *const u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_attention_rows(a0: *mut b200_engine, buffers: *const u64, items: *const b200_attention_item, n_items: u64, dims: *const u64, scale: f32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_attention_rows_as(a0: *mut b200_engine, buffers: *const u64, items: *const b200_attention_item, n_items: u64, dims: *const u64, scale: f32, out_bf16: i32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_scatter_rows_into(a0: *mut b200_engine, table: u64, indices: u64, values: *const b200_block_arg, column: i32) -> i32;
    pub fn b200_reshape(a0: *mut b200_engine, a: u64, rows: u64, cols: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_set_matmul_sm_limit(a0: *mut b200_engine, sms: i32);
    pub fn b200_matmul_host_bf16(a0: *mut b200_engine, a: *const u16, b: *const u16, mkn: *const u64, out: *mut u16) -> i32;
    pub fn b200_matmul_silu_mul(a0: *mut b200_engine, a: u64, b: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_matmul_add_rms_norm(a0: *mut b200_engine, a: u64, b: u64, resid: u64, gains: u64, eps: f32, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_matmul_rope(a0: *mut b200_engine, a: u64, b: u64, cos_: *const b200_block_arg, sin_: *const b200_block_arg, rope_cols: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_matmul_into(a0: *mut b200_engine, a: u64, b: u64, dst: *const *mut core::ffi::c_void, n_dst: i32, dst_rows: u64, dst_cols: u64, col_first: u64, out_bf16: i32) -> i32;
    pub fn b200_store_block_into(a0: *mut b200_engine, src: *const b200_block_arg, dst: *const *mut core::ffi::c_void, n_dst: i32, dst_rows: u64, dst_cols: u64, col_first: u64) -> i32;
    pub fn b200_matmul_into_multicast(a0: *mut b200_engine, a: u64, b: u64, multicast_dst: *mut core::ffi::c_void, dst_rows: u64, dst_cols: u64, col_first: u64, out_bf16: i32) -> i32;
    pub fn b200_store_block_into_multicast(a0: *mut b200_engine, src: *const b200_block_arg, multicast_dst: *mut core::ffi::c_void, dst_rows: u64, dst_cols: u64, col_first: u64) -> i32;
    pub fn b200_ipc_export(a0: *mut b200_engine, buf: u64, handle: *mut u8) -> i32;
    pub fn b200_ipc_open(a0: *mut b200_engine, handle: *const u8, ptr: *mut *mut core::ffi::c_void) -> i32;
    pub fn b200_ipc_close(a0: *mut b200_engine, ptr: *mut core::ffi::c_void) -> i32;
    pub fn b200_decode_layers(a0: *mut b200_engine, shape: *const b200_decode_shape, x: u64, layer_buffers: *const u64, final_norm: u64, cos_table: u64, sin_table: u64, position: u64, out: *mut u64, out_dims: *mut u64) -> i32;
    pub fn b200_begin_trace(a0: *mut b200_engine) -> i32;
    pub fn b200_end_trace(a0: *mut b200_engine, trace: *mut u64) -> i32;
    pub fn b200_run_trace(a0: *mut b200_engine, trace: u64) -> i32;
    pub fn b200_release_trace(a0: *mut b200_engine, trace: u64);
    pub fn b200_trace_footprint(a0: *const b200_engine, trace: u64, bytes: *mut u64) -> i32;
    pub fn b200_trace_ops(a0: *const b200_engine, trace: u64, out: *mut b200_op_stat, capacity: u64, n: *mut u64) -> i32;
    pub fn b200_profile_start(a0: *mut b200_engine) -> i32;
    pub fn b200_profile_stop(a0: *mut b200_engine) -> i32;
    pub fn b200_profile_read(a0: *const b200_engine, out: *mut b200_op_stat, capacity: u64, n: *mut u64) -> i32;
    pub fn b200_debug_stalled_wait(a0: *mut b200_engine) -> i32;
    pub fn b200_sync(a0: *mut b200_engine) -> i32;
    pub fn b200_set_op_label(a0: *mut b200_engine, label: *const c_char);
    pub fn b200_traffic_get(a0: *const b200_engine, out: *mut b200_traffic);
    pub fn b200_timer_start(a0: *mut b200_engine) -> i32;
    pub fn b200_timer_stop(a0: *mut b200_engine, ms: *mut f32) -> i32;
    pub fn b200_stream(a0: *const b200_engine) -> *mut c_void;
    pub fn b200_last_matmul_path(a0: *const b200_engine) -> *const c_char;
    pub fn b200_last_decode_form(a0: *const b200_engine) -> *const c_char;
}
