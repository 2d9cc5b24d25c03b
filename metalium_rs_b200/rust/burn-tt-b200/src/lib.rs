//! `impl burn_tt::Engine for CudaEngine`: the B200 engine behind the reference's operator
//! boundary (crates/burn-tt/src/server.rs:42-786).  Attach it with
//! `burn_tt::attach(TtDevice::new(0), cuda_factory(0))` (server.rs:2738) or make it the default
//! with `burn_tt::set_default_engine` (registry.rs:212); nothing above the trait changes.
//!
//! Shipped as source: it has not met a Rust compiler.  A test holds every method of the `impl` below to the
//! trait's parameter and result types by parsing both.
//! Every method is one call of include/b200tt.h through `b200-sys`.
use b200_sys as sys;
use burn_tt::server::{BlockArg, BufferId, Engine, GenericTraceRun, InputPayload, OutputKind, OutputPayload, PowArg, Serve,
                      SortedBuffers, TraceRun};
use burn_tt::TtError;
use tt_kernels::session::BatchedLayout;
use tt_kernels::sfpu::reduce::{Axis, ReduceOp};
use tt_kernels::tensor::{Block, BlockMove, Elem, Eltwise, ReduceThen};

type Made = Result<(BufferId, [usize; 2]), TtError>;

pub struct CudaEngine {
    raw: *mut sys::b200_engine,
}
// Driven by the device's one server thread (server.rs:2801-2820).
unsafe impl Send for CudaEngine {}

impl Drop for CudaEngine {
    fn drop(&mut self) {
        unsafe { sys::b200_engine_destroy(self.raw) }
    }
}

fn text(raw: *const sys::b200_engine) -> String {
    let mut buf = vec![0u8; 1024];
    let n = unsafe { sys::b200_last_error(raw, buf.as_mut_ptr() as *mut _, buf.len()) };
    String::from_utf8_lossy(&buf[..n.min(buf.len() - 1)]).into_owned()
}

impl CudaEngine {
    pub fn new(ordinal: i32) -> Result<Self, TtError> {
        let mut raw = std::ptr::null_mut();
        let cfg = sys::b200_config::default();
        let st = unsafe { sys::b200_engine_create(ordinal, &cfg, &mut raw) };
        if st != 0 {
            return Err(match st {
                7 => TtError::NoDriver,
                _ => TtError::Device(text(std::ptr::null())),
            });
        }
        Ok(CudaEngine { raw })
    }

    /// b200_status -> TtError (crates/burn-tt/src/error.rs:26-67).
    fn check(&self, st: i32) -> Result<(), TtError> {
        if st == 0 {
            return Ok(());
        }
        let what = text(self.raw);
        Err(match st {
            1 => {
                let mut o = [0u64; 3];
                unsafe { sys::b200_last_oom(self.raw, o.as_mut_ptr()) };
                TtError::OutOfMemory { slots: o[0], free: o[1], largest: o[2] }
            }
            2 => TtError::unsupported(what),
            4 => TtError::Timeout { detail: what },
            5 => TtError::StaleTensor { id: 0 },
            _ => TtError::Device(what), // 3 DEVICE, 6 DOMAIN, 7 NO_DEVICE
        })
    }

    fn made(&self, st: i32, id: u64, d: [u64; 2]) -> Made {
        self.check(st)?;
        Ok((id, [d[0] as usize, d[1] as usize]))
    }

    fn dims(&self, id: BufferId) -> Result<([usize; 2], i32), TtError> {
        let (mut d, mut e) = ([0u64; 2], 0i32);
        if unsafe { sys::b200_dims(self.raw, id, d.as_mut_ptr(), &mut e) } != 0 {
            return Err(TtError::StaleTensor { id });
        }
        Ok(([d[0] as usize, d[1] as usize], e))
    }
}

/// What the trait's `trace_footprint`, `trace_ops`, `profile_mode` and `profile_report` (server.rs:664-688) would
/// carry, in this engine's own terms: those methods return Tensix records (`UnitFootprint`, `OpRecord`,
/// `Profile`), so they keep the trait's defaults and the figures are offered beside the trait.
impl CudaEngine {
    /// Device bytes `trace` holds until it is released.
    pub fn trace_bytes(&self, trace: u64) -> Result<u64, TtError> {
        let mut n = 0u64;
        match unsafe { sys::b200_trace_footprint(self.raw, trace, &mut n) } {
            0 => Ok(n),
            _ => Err(TtError::Device(format!("no trace {trace}"))),
        }
    }
    /// The ops `trace` captured, in order: (label, kernels).
    pub fn trace_labels(&self, trace: u64) -> Result<Vec<(String, u64)>, TtError> {
        let mut n = 0u64;
        if unsafe { sys::b200_trace_ops(self.raw, trace, std::ptr::null_mut(), 0, &mut n) } != 0 {
            return Err(TtError::Device(format!("no trace {trace}")));
        }
        let mut rows = vec![unsafe { std::mem::zeroed::<sys::b200_op_stat>() }; n as usize];
        unsafe { sys::b200_trace_ops(self.raw, trace, rows.as_mut_ptr(), n, &mut n) };
        Ok(rows.iter().map(|r| (label_of(r), r.launches)).collect())
    }
    /// Per-op device time: on, then off with the table (label, calls, kernels, ms).
    pub fn profile_start(&mut self) -> Result<(), TtError> {
        let st = unsafe { sys::b200_profile_start(self.raw) };
        self.check(st)
    }
    pub fn profile_stop(&mut self) -> Result<Vec<(String, u64, u64, f64)>, TtError> {
        let st = unsafe { sys::b200_profile_stop(self.raw) };
        self.check(st)?;
        let mut n = 0u64;
        unsafe { sys::b200_profile_read(self.raw, std::ptr::null_mut(), 0, &mut n) };
        let mut rows = vec![unsafe { std::mem::zeroed::<sys::b200_op_stat>() }; n as usize];
        unsafe { sys::b200_profile_read(self.raw, rows.as_mut_ptr(), n, &mut n) };
        Ok(rows.iter().map(|r| (label_of(r), r.calls, r.launches, r.device_ms)).collect())
    }
}
fn label_of(r: &sys::b200_op_stat) -> String {
    let bytes: Vec<u8> = r.op.iter().take_while(|c| **c != 0).map(|c| *c as u8).collect();
    String::from_utf8_lossy(&bytes).into_owned()
}

fn elem_code(elem: Elem, bf16: bool) -> i32 {
    if bf16 {
        return 3;
    }
    match elem {
        Elem::F32 => 0,
        Elem::I32 => 1,
        Elem::Bool => 2,
        Elem::Packed(_) => 3,
    }
}
fn block(b: &Block) -> sys::b200_block {
    sys::b200_block { at: [b.at[0] as u64, b.at[1] as u64], transposed: b.transposed as i32, _pad: 0 }
}
fn arg(b: &BlockArg) -> sys::b200_block_arg {
    sys::b200_block_arg { id: b.id, at: [b.at[0] as u64, b.at[1] as u64], dims: [b.dims[0] as u64, b.dims[1] as u64] }
}
fn op(o: &Eltwise) -> sys::b200_eltwise_op {
    sys::b200_eltwise_op { kind: o.kind, scalar: o.scalar, scalar2: o.scalar2 }
}
fn reduce_code(o: ReduceOp) -> i32 {
    match o {
        ReduceOp::Sum => 0, ReduceOp::Max => 1, ReduceOp::Prod => 2, ReduceOp::All => 3, ReduceOp::Any => 4,
        ReduceOp::BitOr => 5, ReduceOp::SumI32 => 6, ReduceOp::ProdI32 => 7, ReduceOp::MinI32 => 8, ReduceOp::MaxI32 => 9,
    }
}

/// The factory `burn_tt::attach` runs on the server thread.
pub fn cuda_factory(ordinal: i32) -> impl FnOnce(Serve) -> Result<(), TtError> {
    move |serve| {
        let mut engine = CudaEngine::new(ordinal)?;
        serve.serve(&mut engine)
    }
}

macro_rules! produce {
    ($self:ident, $f:ident ( $($a:expr),* )) => {{
        let (mut id, mut d) = (0u64, [0u64; 2]);
        let st = unsafe { sys::$f($self.raw, $($a,)* &mut id, d.as_mut_ptr()) };
        $self.made(st, id, d)
    }};
}

impl Engine for CudaEngine {
    fn supports_dram(&self) -> bool { true }
    fn supports_batched_layout(&self) -> bool { true }
    fn supports_exact_matmul(&self) -> bool { false }

    fn matmul(&mut self, a: &[f32], b: &[f32], mkn: [usize; 3]) -> Result<Vec<f32>, TtError> {
        let mut out = vec![0f32; mkn[0] * mkn[2]];
        let d = [mkn[0] as u64, mkn[1] as u64, mkn[2] as u64];
        let st = unsafe { sys::b200_matmul_host(self.raw, a.as_ptr(), b.as_ptr(), d.as_ptr(), out.as_mut_ptr()) };
        self.check(st).map(|_| out)
    }
    fn upload(&mut self, v: &[f32], rows: usize, cols: usize) -> Result<BufferId, TtError> {
        let mut id = 0u64;
        let st = unsafe { sys::b200_upload_f32(self.raw, v.as_ptr(), rows as u64, cols as u64, &mut id) };
        self.check(st).map(|_| id)
    }
    fn upload_bf16(&mut self, v: &[u16], rows: usize, cols: usize) -> Result<BufferId, TtError> {
        let mut id = 0u64;
        let st = unsafe { sys::b200_upload_bf16(self.raw, v.as_ptr(), rows as u64, cols as u64, &mut id) };
        self.check(st).map(|_| id)
    }
    fn upload_bits(&mut self, v: &[u32], rows: usize, cols: usize, elem: Elem) -> Result<BufferId, TtError> {
        let mut id = 0u64;
        let st = unsafe { sys::b200_upload_bits(self.raw, v.as_ptr(), rows as u64, cols as u64, elem_code(elem, false), &mut id) };
        self.check(st).map(|_| id)
    }
    fn download(&mut self, id: BufferId) -> Result<Vec<f32>, TtError> {
        let (d, _) = self.dims(id)?;
        let mut out = vec![0f32; d[0] * d[1]];
        let st = unsafe { sys::b200_download_f32(self.raw, id, out.as_mut_ptr(), out.len() as u64) };
        self.check(st).map(|_| out)
    }
    fn download_bf16(&mut self, id: BufferId) -> Result<Vec<u16>, TtError> {
        let (d, _) = self.dims(id)?;
        let mut out = vec![0u16; d[0] * d[1]];
        let st = unsafe { sys::b200_download_bf16(self.raw, id, out.as_mut_ptr(), out.len() as u64) };
        self.check(st).map(|_| out)
    }
    fn download_bits(&mut self, id: BufferId) -> Result<Vec<u32>, TtError> {
        let (d, _) = self.dims(id)?;
        let mut out = vec![0u32; d[0] * d[1]];
        let st = unsafe { sys::b200_download_bits(self.raw, id, out.as_mut_ptr(), out.len() as u64) };
        self.check(st).map(|_| out)
    }
    fn free(&mut self, id: BufferId) { unsafe { sys::b200_free(self.raw, id) } }
    fn zeros_dram(&mut self, dims: [usize; 2], elem: Elem, bf16: bool) -> Made {
        produce!(self, b200_zeros(dims[0] as u64, dims[1] as u64, elem_code(elem, bf16)))
    }
    fn copy_into(&mut self, src: BufferId, dst: BufferId) -> Result<(), TtError> {
        let st = unsafe { sys::b200_copy_into(self.raw, src, dst) };
        self.check(st)
    }
    fn cast_float(&mut self, a: BufferId, bf16: bool) -> Made { produce!(self, b200_cast_float(a, bf16 as i32)) }

    fn matmul_dram(&mut self, a: BufferId, ta: bool, b: BufferId, tb: bool) -> Made {
        produce!(self, b200_matmul(a, ta as i32, b, tb as i32, 0))
    }
    fn matmul_dram_bf16(&mut self, a: BufferId, ta: bool, b: BufferId, tb: bool) -> Made {
        produce!(self, b200_matmul(a, ta as i32, b, tb as i32, 1))
    }
    // A fidelity names how many of the Tensix multiplier's passes a product takes (server.rs:203-226); this
    // engine's products are F32-accurate whatever is asked, which is the highest fidelity's result, and exact on
    // the integer slices `MatmulMode::Accurate` multiplies at the lowest one.
    fn matmul_dram_at(&mut self, a: BufferId, ta: bool, b: BufferId, tb: bool, _fidelity: tt_kernels::matmul::Fidelity) -> Made {
        self.matmul_dram(a, ta, b, tb)
    }
    fn matmul_dram_batched_at(&mut self, a: BufferId, b: BufferId, items: &[(Block, Block)], mkn: [usize; 3],
                              _fidelity: tt_kernels::matmul::Fidelity) -> Made {
        self.matmul_dram_batched(a, b, items, mkn)
    }
    fn matmul_dram_batched(&mut self, a: BufferId, b: BufferId, items: &[(Block, Block)], mkn: [usize; 3]) -> Made {
        self.matmul_dram_batched_layout(a, b, items, mkn, BatchedLayout::STACKED)
    }
    fn matmul_dram_batched_layout(&mut self, a: BufferId, b: BufferId, items: &[(Block, Block)], mkn: [usize; 3],
                                  layout: BatchedLayout) -> Made {
        let ab: Vec<_> = items.iter().map(|(x, _)| block(x)).collect();
        let bb: Vec<_> = items.iter().map(|(_, y)| block(y)).collect();
        let d = [mkn[0] as u64, mkn[1] as u64, mkn[2] as u64];
        let l = sys::b200_batched_layout { lhs_padded: layout.lhs_padded as i32, stacked: layout.stacked as i32 };
        // the result takes its operands' type: BF16 operands give a BF16 product (ops.rs:464-503)
        let bf16 = self.dims(a)?.1 == 3;
        produce!(self, b200_matmul_batched(a, b, ab.as_ptr(), bb.as_ptr(), items.len() as u64, d.as_ptr(), &l, bf16 as i32))
    }

    fn eltwise(&mut self, kind: u32, scalar: f32, a: BufferId, b: Option<BufferId>) -> Made {
        self.eltwise_op_as(Eltwise { kind, scalar, scalar2: 0.0 }, a, b, None, false)
    }
    fn eltwise_op(&mut self, o: Eltwise, a: BufferId, b: Option<BufferId>, c: Option<BufferId>) -> Made {
        self.eltwise_op_as(o, a, b, c, false)
    }
    fn eltwise_op_as(&mut self, o: Eltwise, a: BufferId, b: Option<BufferId>, c: Option<BufferId>, bf16: bool) -> Made {
        let o = op(&o);
        produce!(self, b200_eltwise(&o, a, b.unwrap_or(0), c.unwrap_or(0), bf16 as i32))
    }
    fn eltwise_blocks(&mut self, o: Eltwise, a: BlockArg, b: Option<BlockArg>, c: Option<BlockArg>) -> Made {
        self.eltwise_blocks_as(o, a, b, c, false)
    }
    fn eltwise_blocks_as(&mut self, o: Eltwise, a: BlockArg, b: Option<BlockArg>, c: Option<BlockArg>, bf16: bool) -> Made {
        let (o, a) = (op(&o), arg(&a));
        let (b, c) = (b.as_ref().map(arg), c.as_ref().map(arg));
        let pb = b.as_ref().map_or(std::ptr::null(), |x| x as *const _);
        let pc = c.as_ref().map_or(std::ptr::null(), |x| x as *const _);
        produce!(self, b200_eltwise_blocks(&o, &a, pb, pc, bf16 as i32))
    }
    fn rope_blocks(&mut self, x: BlockArg, cos: BlockArg, sin: BlockArg, head: usize, bf16: bool) -> Made {
        let (x, c, s) = (arg(&x), arg(&cos), arg(&sin));
        produce!(self, b200_rope_blocks(&x, &c, &s, head as u64, bf16 as i32))
    }

    fn reduce(&mut self, a: BufferId, o: ReduceOp, axis: Axis, then: ReduceThen) -> Made {
        let (k, bits) = then.unwrap_or((0, 0));
        produce!(self, b200_reduce(a, reduce_code(o), matches!(axis, Axis::Cols) as i32, k, bits))
    }
    fn sum_rows(&mut self, a: BufferId) -> Made { produce!(self, b200_sum_rows(a)) }
    fn full_reduce(&mut self, values: &[f32], dims: [usize; 2], mean: bool) -> Result<f32, TtError> {
        let (d, mut out) = ([dims[0] as u64, dims[1] as u64], 0f32);
        let st = unsafe { sys::b200_full_reduce(self.raw, values.as_ptr(), d.as_ptr(), mean as i32, &mut out) };
        self.check(st).map(|_| out)
    }
    fn softmax_rows(&mut self, x: BufferId, mask: BufferId, scale: f32) -> Made { produce!(self, b200_softmax_rows(x, mask, scale)) }
    fn rms(&mut self, a: BufferId, eps: f32) -> Made { produce!(self, b200_rms(a, eps)) }
    fn rms_norm(&mut self, a: BufferId, gamma: Option<BufferId>, eps: f32) -> Made {
        produce!(self, b200_rms_norm(a, gamma.unwrap_or(0), eps, 0))
    }
    fn rms_norm_as(&mut self, a: BufferId, gamma: Option<BufferId>, eps: f32, bf16: bool) -> Made {
        produce!(self, b200_rms_norm(a, gamma.unwrap_or(0), eps, bf16 as i32))
    }
    fn add_rms_norm(&mut self, a: BufferId, b: BufferId, gamma: Option<BufferId>, eps: f32)
        -> Result<[(BufferId, [usize; 2]); 2], TtError> {
        let (mut ids, mut d) = ([0u64; 2], [0u64; 2]);
        let st = unsafe { sys::b200_add_rms_norm(self.raw, a, b, gamma.unwrap_or(0), eps, ids.as_mut_ptr(), d.as_mut_ptr()) };
        self.check(st)?;
        let dims = [d[0] as usize, d[1] as usize];
        Ok([(ids[0], dims), (ids[1], dims)])
    }
    fn argmax_row(&mut self, a: BufferId) -> Made { produce!(self, b200_argmax_row(a)) }

    fn select_rows(&mut self, table: BufferId, idx: BufferId) -> Made { produce!(self, b200_select_rows(table, idx)) }
    fn pick_columns(&mut self, x: BufferId, idx: BufferId) -> Made { produce!(self, b200_pick_columns(x, idx)) }
    fn select_add_rows(&mut self, t: BufferId, idx: BufferId, v: BufferId) -> Made { produce!(self, b200_select_add_rows(t, idx, v)) }
    fn gather_indexed(&mut self, x: BufferId, idx: BufferId) -> Made { produce!(self, b200_gather_indexed(x, idx)) }
    fn scatter_rows(&mut self, t: BufferId, idx: BufferId, v: BufferId, column: bool) -> Made {
        produce!(self, b200_scatter_rows(t, idx, v, column as i32))
    }
    fn scatter_rows_into(&mut self, t: BufferId, idx: BufferId, v: BlockArg, column: bool) -> Result<(), TtError> {
        let b = sys::b200_block_arg { id: v.id, at: [v.at[0] as u64, v.at[1] as u64], dims: [v.dims[0] as u64, v.dims[1] as u64] };
        let st = unsafe { sys::b200_scatter_rows_into(self.raw, t, idx, &b, column as i32) };
        self.check(st)
    }
    fn rows_add(&mut self, t: BufferId, indices: &[usize], v: BufferId) -> Made {
        let i: Vec<u64> = indices.iter().map(|&x| x as u64).collect();
        produce!(self, b200_rows_add(t, i.as_ptr(), i.len() as u64, v))
    }
    fn assign_rows(&mut self, t: BufferId, v: BufferId, rows: &[(usize, usize)]) -> Made {
        let p: Vec<u64> = rows.iter().flat_map(|&(d, s)| [d as u64, s as u64]).collect();
        produce!(self, b200_assign_rows(t, v, p.as_ptr(), rows.len() as u64))
    }
    fn gather_rows(&mut self, sources: &[BufferId], rows: &[(usize, usize)], cols: usize) -> Made {
        let p: Vec<u64> = rows.iter().flat_map(|&(s, r)| [s as u64, r as u64]).collect();
        produce!(self, b200_gather_rows(sources.as_ptr(), sources.len() as u64, p.as_ptr(), rows.len() as u64, cols as u64))
    }
    fn slice_rows(&mut self, a: BufferId, first: usize, rows: usize) -> Made {
        produce!(self, b200_slice_rows(a, first as u64, rows as u64))
    }
    fn copy_blocks(&mut self, a: BufferId, moves: &[BlockMove], dims: [usize; 2]) -> Made {
        let m: Vec<_> = moves.iter().map(|m| sys::b200_block_move {
            from: [m.from[0] as u64, m.from[1] as u64], to: [m.to[0] as u64, m.to[1] as u64],
            extent: [m.extent[0] as u64, m.extent[1] as u64], transposed: m.transposed as i32, _pad: 0 }).collect();
        let d = [dims[0] as u64, dims[1] as u64];
        produce!(self, b200_copy_blocks(a, m.as_ptr(), m.len() as u64, d.as_ptr()))
    }
    fn attention_rows(&mut self, buffers: [BufferId; 4], items: &[tt_kernels::attention::Item], dims: [usize; 4], scale: f32) -> Made {
        let it: Vec<_> = items.iter().map(|i| sys::b200_attention_item {
            q: [i.q[0] as u64, i.q[1] as u64], k: [i.k[0] as u64, i.k[1] as u64], v: [i.v[0] as u64, i.v[1] as u64] }).collect();
        let d = [dims[0] as u64, dims[1] as u64, dims[2] as u64, dims[3] as u64];
        produce!(self, b200_attention_rows(buffers.as_ptr(), it.as_ptr(), it.len() as u64, d.as_ptr(), scale))
    }
    fn repack(&mut self, a: BufferId, sources: &[[usize; 2]], dims: [usize; 2]) -> Made {
        let p: Vec<u64> = sources.iter().flat_map(|s| [s[0] as u64, s[1] as u64]).collect();
        let d = [dims[0] as u64, dims[1] as u64];
        produce!(self, b200_repack(a, p.as_ptr(), d.as_ptr()))
    }

    fn repack_many(&mut self, inputs: &[BufferId], sources: &[(usize, [usize; 2])], dims: [usize; 2]) -> Made {
        let p: Vec<u64> = sources.iter().flat_map(|&(i, at)| [i as u64, at[0] as u64, at[1] as u64]).collect();
        let d = [dims[0] as u64, dims[1] as u64];
        produce!(self, b200_repack_many(inputs.as_ptr(), inputs.len() as u64, p.as_ptr(), sources.len() as u64, d.as_ptr()))
    }
    fn select_taps(&mut self, table: BufferId, idx: BufferId, zero_row: bool) -> Made {
        produce!(self, b200_select_taps(table, idx, zero_row as i32))
    }
    fn cast_block(&mut self, a: BlockArg, bf16: bool) -> Made {
        let b = sys::b200_block_arg { id: a.id, at: [a.at[0] as u64, a.at[1] as u64], dims: [a.dims[0] as u64, a.dims[1] as u64] };
        produce!(self, b200_cast_block(&b, bf16 as i32))
    }
    // A logical F32 buffer kept as BF16 (half the bytes, read by a product as its B) and back: the storage is
    // plain BF16 here, and `b200_matmul` takes one F32 and one BF16 operand (server.rs:150-158).
    fn cast_bf16_storage(&mut self, id: BufferId, store: bool) -> Made { produce!(self, b200_cast_float(id, store as i32)) }
    // Explicit block-float storage (server.rs:141): BFP8 is kept; BFP4 and BFP2 are refused by the engine (format codes
    // 4 and 2 are not ones it takes).  `None` widens to F32.
    fn cast_bfp(&mut self, id: BufferId, format: Option<tt_kernels::bfp::BfpFormat>) -> Made {
        use tt_kernels::bfp::BfpFormat::*;
        let code = match format { None => 0, Some(Bfp8) => 8, Some(Bfp4) => 4, Some(Bfp2) => 2 };
        produce!(self, b200_cast_bfp(id, code))
    }
    fn cast_f16(&mut self, id: BufferId, to_f16: bool) -> Made { produce!(self, b200_cast_f16(id, to_f16 as i32)) }
    fn pow(&mut self, x: BufferId, y: PowArg) -> Made {
        match y {
            PowArg::Tensor(t) => produce!(self, b200_pow(x, 0, t, 0.0)),
            PowArg::Scalar(s) => produce!(self, b200_pow(x, 1, 0, s)),
            PowArg::Int(t) => produce!(self, b200_pow(x, 2, t, 0.0)),
        }
    }
    fn scan(&mut self, a: BufferId, op: tt_kernels::sfpu::scan::ScanOp) -> Made {
        use tt_kernels::sfpu::scan::ScanOp::*;
        let code = match op { Sum => 0, Prod => 1, Min => 2, Max => 3, MinNan => 4, MaxNan => 5, ISum => 6, IProd => 7, IMin => 8, IMax => 9 };
        produce!(self, b200_scan(a, code))
    }
    fn sort_planes(&mut self, a: BufferId, spec: tt_kernels::sfpu::sort::Spec) -> Result<SortedBuffers, TtError> {
        let (mut keys, mut idx, mut d) = (0u64, 0u64, [0u64; 2]);
        let ip = if spec.indices { &mut idx as *mut u64 } else { std::ptr::null_mut() };
        let st = unsafe { sys::b200_sort_planes(self.raw, a, elem_code(spec.elem, false), spec.n as u64, spec.descending as i32, &mut keys, ip, d.as_mut_ptr()) };
        self.check(st)?;
        let dims = [d[0] as usize, d[1] as usize];
        Ok(SortedBuffers { keys: (keys, dims), indices: spec.indices.then_some((idx, dims)) })
    }
    fn random_dram(&mut self, dims: [usize; 2], draw: burn_tt::random::Draw, base: u64) -> Made {
        use burn_tt::random::Draw::*;
        let d = [dims[0] as u64, dims[1] as u64];
        let (code, a, b, lo, hi, int) = match draw {
            Unit => (0, 0.0, 0.0, 0, 0, false),
            Uniform(lo, hi) => (1, lo, hi, 0, 0, false),
            Bernoulli { p, int } => (2, p, 0.0, 0, 0, int),
            Normal { mean, std, int } => (3, mean, std, 0, 0, int),
            IntRange(lo, hi) => (4, 0.0, 0.0, lo, hi, false),
            IntWords => (5, 0.0, 0.0, 0, 0, false),
        };
        produce!(self, b200_random(d.as_ptr(), code, a, b, lo, hi, int as i32, base))
    }
    fn pool_bf16(&mut self, a: BufferId, windows: &[Vec<[usize; 2]>], divisors: &[usize], dims: [usize; 2]) -> Made {
        if divisors.len() != windows.len() { return Err(TtError::unsupported("invalid BF16 pool windows")); }
        let mut offsets = vec![0u64];
        for w in windows { offsets.push(offsets.last().unwrap() + w.len() as u64); }
        let coords: Vec<u64> = windows.iter().flatten().flat_map(|rc| [rc[0] as u64, rc[1] as u64]).collect();
        let div: Vec<u64> = divisors.iter().map(|&d| d as u64).collect();
        let d = [dims[0] as u64, dims[1] as u64];
        produce!(self, b200_pool_bf16(a, offsets.as_ptr(), coords.as_ptr(), div.as_ptr(), windows.len() as u64, d.as_ptr()))
    }
    fn metadata(&mut self, bits: &[u32], dims: [usize; 2], elem: Elem) -> Result<BufferId, TtError> {
        let (mut id, d) = (0u64, [dims[0] as u64, dims[1] as u64]);
        let st = unsafe { sys::b200_metadata(self.raw, bits.as_ptr(), d.as_ptr(), elem_code(elem, false), &mut id) };
        self.check(st).map(|_| id)
    }
    fn gddr_free_bytes(&mut self) -> Result<(u64, u64), TtError> {
        let mut out = [0u64; 2];
        let st = unsafe { sys::b200_free_bytes(self.raw, out.as_mut_ptr()) };
        self.check(st).map(|_| (out[0], out[1]))
    }

    // Traces are CUDA graphs (server.rs:591-660).
    fn begin_trace(&mut self) -> Result<(), TtError> { let st = unsafe { sys::b200_begin_trace(self.raw) }; self.check(st) }
    fn end_trace(&mut self) -> Result<u64, TtError> {
        let mut t = 0u64;
        let st = unsafe { sys::b200_end_trace(self.raw, &mut t) };
        self.check(st).map(|_| t)
    }
    // One round trip (server.rs:648-657, 1114-1143): wait for what was queued, write the input, replay to its
    // end, read the output; the three times are the write's, the replay's and the read's.
    fn run_trace(&mut self, trace: u64, input: BufferId, values: &[f32], output: BufferId) -> Result<TraceRun, TtError> {
        use std::time::Instant;
        let st = unsafe { sys::b200_sync(self.raw) }; self.check(st)?;
        let t0 = Instant::now();
        let st = unsafe { sys::b200_write_f32(self.raw, input, values.as_ptr(), values.len() as u64) }; self.check(st)?;
        let t1 = Instant::now();
        let st = unsafe { sys::b200_run_trace(self.raw, trace) }; self.check(st)?;
        let st = unsafe { sys::b200_sync(self.raw) }; self.check(st)?;
        let t2 = Instant::now();
        let output = self.download(output)?;
        Ok(TraceRun { output, write: t1 - t0, replay: t2 - t1, read: t2.elapsed() })
    }
    // Several inputs overwritten, the replay, several outputs read (server.rs:746-753, 1205-1238).  A 32-bit
    // payload of either kind is written as words: `b200_write_f32` copies four-byte elements whatever their type.
    fn run_generic_trace(&mut self, trace: u64, inputs: &[(BufferId, InputPayload)], outputs: &[(BufferId, OutputKind)])
                         -> Result<GenericTraceRun, TtError> {
        use std::time::Instant;
        let st = unsafe { sys::b200_sync(self.raw) }; self.check(st)?;
        let t0 = Instant::now();
        for (id, payload) in inputs {
            let (p, n) = match payload {
                InputPayload::F32(v) => (v.as_ptr(), v.len()),
                InputPayload::Bits(v) => (v.as_ptr() as *const f32, v.len()),
            };
            let st = unsafe { sys::b200_write_f32(self.raw, *id, p, n as u64) }; self.check(st)?;
        }
        let t1 = Instant::now();
        let st = unsafe { sys::b200_run_trace(self.raw, trace) }; self.check(st)?;
        let st = unsafe { sys::b200_sync(self.raw) }; self.check(st)?;
        let t2 = Instant::now();
        let mut read = Vec::with_capacity(outputs.len());
        for (id, kind) in outputs {
            read.push(match kind {
                OutputKind::F32 => OutputPayload::F32(self.download(*id)?),
                OutputKind::Bits => OutputPayload::Bits(self.download_bits(*id)?),
            });
        }
        Ok(GenericTraceRun { outputs: read, write: t1 - t0, replay: t2 - t1, read: t2.elapsed() })
    }
    fn release_trace(&mut self, trace: u64) { unsafe { sys::b200_release_trace(self.raw, trace) } }
    fn set_op_label(&mut self, label: &'static str) {
        let c = std::ffi::CString::new(label).unwrap();
        unsafe { sys::b200_set_op_label(self.raw, c.as_ptr()) }
    }
}
