"""Host-side mirror of the reference's `Engine` trait over the C ABI.

`CudaEngine` has the method names, argument meaning and failure behaviour of
`burn_tt::Engine` (crates/burn-tt/src/server.rs:42-786): tensors are opaque buffer ids,
every producing method returns `(id, [rows, cols])`, failures raise `TtError` with the
variant the reference would return (crates/burn-tt/src/error.rs:26-67).  It is a thin
ctypes binding of include/b200tt.h: no arithmetic happens here, and there is no
fallback -- without the built library, or without a B200, construction fails.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from pathlib import Path
from typing import Optional, Sequence, Tuple

import numpy as np

from . import kinds

_LIB_PATH = Path(__file__).resolve().parent / "libb200tt.so"
_lib = None

OK, OUT_OF_MEMORY, UNSUPPORTED, DEVICE, TIMEOUT, STALE, DOMAIN, NO_DEVICE = range(8)
F32, I32, BOOL, BF16, BFP8 = range(5)
SUM, MAX, PROD, ALL, ANY, BITOR, SUM_I32, PROD_I32, MIN_I32, MAX_I32 = range(10)
ROWS, COLS = 0, 1
# crates/tt-kernels/src/sfpu/scan.rs:19-41 `ScanOp`, in its order
(SCAN_SUM, SCAN_PROD, SCAN_MIN, SCAN_MAX, SCAN_MIN_NAN, SCAN_MAX_NAN, SCAN_ISUM, SCAN_IPROD, SCAN_IMIN,
 SCAN_IMAX) = range(10)

_STATUS_NAMES = {1: "OutOfMemory", 2: "Unsupported", 3: "Device", 4: "Timeout", 5: "StaleTensor",
                 6: "Device(DOMAIN)", 7: "NoDriver"}


class TtError(RuntimeError):
    """A failed engine call: `status` is the b200_status code, `variant` the reference's name."""

    def __init__(self, status: int, text: str):
        self.status = status
        self.variant = _STATUS_NAMES.get(status, str(status))
        super().__init__(f"{self.variant}: {text}")


class EltwiseOp(C.Structure):  # tt-kernels/src/tensor.rs:3785
    _fields_ = [("kind", C.c_uint32), ("scalar", C.c_float), ("scalar2", C.c_float)]


class Block(C.Structure):  # tt-kernels/src/tensor.rs:3479
    _fields_ = [("at", C.c_uint64 * 2), ("transposed", C.c_int32), ("_pad", C.c_int32)]


class BlockMove(C.Structure):  # tt-kernels/src/tensor.rs:6659
    _fields_ = [("from_", C.c_uint64 * 2), ("to", C.c_uint64 * 2), ("extent", C.c_uint64 * 2),
                ("transposed", C.c_int32), ("_pad", C.c_int32)]


class AttentionItem(C.Structure):  # tt-kernels/src/attention.rs:40
    _fields_ = [("q", C.c_uint64 * 2), ("k", C.c_uint64 * 2), ("v", C.c_uint64 * 2)]


class AttentionBlock(C.Structure):  # b200_attention_block
    _fields_ = [("q", C.c_uint64 * 2), ("k", C.c_uint64 * 2), ("v", C.c_uint64 * 2), ("o", C.c_uint64 * 2)]


class BlockArg(C.Structure):  # burn-tt/src/server.rs:3449
    _fields_ = [("id", C.c_uint64), ("at", C.c_uint64 * 2), ("dims", C.c_uint64 * 2)]


class BatchedLayout(C.Structure):  # tt-kernels/src/session.rs:802
    _fields_ = [("lhs_padded", C.c_int32), ("stacked", C.c_int32)]


class Traffic(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("bytes_h2d", "bytes_d2h", "h2d_calls", "d2h_calls", "launches",
                                          "pool_reserved", "pool_in_use", "pool_high_water")]


class Config(C.Structure):
    _fields_ = [("f32_matmul_mode", C.c_int32), ("bf16_matmul_mode", C.c_int32), ("pool_limit_bytes", C.c_uint64),
                ("fail_alloc_at", C.c_int32), ("_pad", C.c_int32), ("wait_limit_cycles", C.c_uint64)]


class DecodeShape(C.Structure):  # b200_decode_shape
    _fields_ = [(n, C.c_uint32) for n in ("layers", "hidden", "heads", "kv_heads", "head_dim", "ff", "max_len", "attend")] + \
               [("eps", C.c_float), ("scale", C.c_float)]


class OpStat(C.Structure):  # burn-tt/src/report.rs:27 `OpStat`, reduced (b200_op_stat)
    _fields_ = [("op", C.c_char * 48), ("calls", C.c_uint64), ("launches", C.c_uint64), ("device_ms", C.c_double)]


def library_path() -> Path:
    return _LIB_PATH


def _prepare(_lib: C.CDLL) -> C.CDLL:
    """Declare the return types ctypes would otherwise guess wrong."""
    if getattr(_lib, "_b200_prepared", False):
        return _lib
    _lib._b200_prepared = True
    if True:
        _lib.b200_last_error.restype = C.c_size_t
        _lib.b200_last_error.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t]
        _lib.b200_stream.restype = C.c_void_p
        _lib.b200_stream.argtypes = [C.c_void_p]
        _lib.b200_last_matmul_path.restype = C.c_char_p
        _lib.b200_last_matmul_path.argtypes = [C.c_void_p]
        _lib.b200_last_decode_form.restype = C.c_char_p
        _lib.b200_last_decode_form.argtypes = [C.c_void_p]
        _lib.b200_engine_destroy.restype = None
        _lib.b200_free.restype = None
        _lib.b200_set_op_label.restype = None
        _lib.b200_set_matmul_sm_limit.restype = None
        _lib.b200_traffic_get.restype = None
        _lib.b200_last_oom.restype = None
        _lib.b200_release_trace.restype = None
    return _lib


def load_library() -> C.CDLL:
    """dlopen the engine.  Raises if it was not built: there is no other implementation."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise ImportError(f"{_LIB_PATH} is missing: run `python -m metalium_rs_b200.build` "
                              "(the engine has no CPU or PyTorch fallback)")
        _lib = _prepare(C.CDLL(str(_LIB_PATH)))
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _block(b) -> "BlockArg":
    if isinstance(b, BlockArg):
        return b
    bid, at, dims = b
    return BlockArg(bid, (C.c_uint64 * 2)(*at), (C.c_uint64 * 2)(*dims))


Out = Tuple[int, Tuple[int, int]]


class CudaEngine:
    """One GPU's engine; the B200 counterpart of `KmdEngine` (server.rs:4071)."""

    def __init__(self, device: int = 0, *, f32_matmul_mode: int = 0, bf16_matmul_mode: int = 0,
                 pool_limit_bytes: int = 0, fail_alloc_at: int = 0, wait_limit_cycles: int = 0, lib=None):
        # `lib`: a library handle to use instead of libb200tt.so -- the test suite passes the
        # engine's host logic linked against a host-only stand-in for the CUDA runtime.
        self._lib = _prepare(lib) if lib is not None else load_library()
        self._e = C.c_void_p()
        cfg = Config(f32_matmul_mode, bf16_matmul_mode, pool_limit_bytes, fail_alloc_at, 0, wait_limit_cycles)
        st = self._lib.b200_engine_create(C.c_int32(device), C.byref(cfg), C.byref(self._e))
        if st:
            buf = C.create_string_buffer(1024)
            self._lib.b200_last_error(None, buf, 1024)
            self._e = None
            raise TtError(st, buf.value.decode())
        self.device = device
        self.profiling = False

    # -- plumbing ------------------------------------------------------------
    def close(self):
        if getattr(self, "_e", None):
            self._lib.b200_engine_destroy(self._e)
            self._e = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def _check(self, st: int):
        if st:
            buf = C.create_string_buffer(2048)
            self._lib.b200_last_error(self._e, buf, 2048)
            raise TtError(st, buf.value.decode())

    def _call(self, fn, *args) -> Out:
        out = C.c_uint64()
        dims = (C.c_uint64 * 2)()
        self._check(fn(self._e, *args, C.byref(out), dims))
        return out.value, (dims[0], dims[1])

    # -- capabilities (server.rs:53,75,240) --------------------------------------
    def supports_dram(self) -> bool:
        return bool(self._lib.b200_supports_dram(self._e))

    def supports_batched_layout(self) -> bool:
        return bool(self._lib.b200_supports_batched_layout(self._e))

    def supports_exact_matmul(self) -> bool:
        return bool(self._lib.b200_supports_exact_matmul(self._e))

    # -- storage (server.rs:91-174, 285) -----------------------------------------
    def upload(self, values, rows: int, cols: int) -> int:
        a = np.ascontiguousarray(values, dtype=np.float32)
        assert a.size == rows * cols
        out = C.c_uint64()
        self._check(self._lib.b200_upload_f32(self._e, _ptr(a), C.c_uint64(rows), C.c_uint64(cols), C.byref(out)))
        return out.value

    def upload_bf16(self, values, rows: int, cols: int) -> int:
        a = np.ascontiguousarray(values, dtype=np.uint16)
        assert a.size == rows * cols
        out = C.c_uint64()
        self._check(self._lib.b200_upload_bf16(self._e, _ptr(a), C.c_uint64(rows), C.c_uint64(cols), C.byref(out)))
        return out.value

    def upload_bits(self, bits, rows: int, cols: int, elem: int) -> int:
        a = np.ascontiguousarray(bits).view(np.uint32) if np.asarray(bits).dtype.itemsize == 4 \
            else np.ascontiguousarray(bits, dtype=np.uint32)
        assert a.size == rows * cols
        out = C.c_uint64()
        self._check(self._lib.b200_upload_bits(self._e, _ptr(a), C.c_uint64(rows), C.c_uint64(cols), C.c_int32(elem),
                                               C.byref(out)))
        return out.value

    def upload_ptr(self, host_ptr: int, rows: int, cols: int, elem: int = F32) -> int:
        """Upload from a raw host address (e.g. pinned memory another library owns)."""
        out = C.c_uint64()
        fn = {F32: self._lib.b200_upload_f32, BF16: self._lib.b200_upload_bf16}.get(elem)
        if fn is None:
            self._check(self._lib.b200_upload_bits(self._e, C.c_void_p(host_ptr), C.c_uint64(rows), C.c_uint64(cols),
                                                   C.c_int32(elem), C.byref(out)))
        else:
            self._check(fn(self._e, C.c_void_p(host_ptr), C.c_uint64(rows), C.c_uint64(cols), C.byref(out)))
        return out.value

    def dims_of(self, buf: int) -> Tuple[Tuple[int, int], int]:
        dims = (C.c_uint64 * 2)()
        elem = C.c_int32()
        st = self._lib.b200_dims(self._e, C.c_uint64(buf), dims, C.byref(elem))
        if st:
            raise TtError(st, f"buffer {buf} is not live on this engine")
        return (dims[0], dims[1]), elem.value

    def download(self, buf: int) -> np.ndarray:
        (r, c), _ = self.dims_of(buf)
        out = np.empty((r, c), dtype=np.float32)
        self._check(self._lib.b200_download_f32(self._e, C.c_uint64(buf), _ptr(out), C.c_uint64(out.size)))
        return out

    def download_bf16(self, buf: int) -> np.ndarray:
        (r, c), _ = self.dims_of(buf)
        out = np.empty((r, c), dtype=np.uint16)
        self._check(self._lib.b200_download_bf16(self._e, C.c_uint64(buf), _ptr(out), C.c_uint64(out.size)))
        return out

    def download_bits(self, buf: int) -> np.ndarray:
        (r, c), _ = self.dims_of(buf)
        out = np.empty((r, c), dtype=np.uint32)
        self._check(self._lib.b200_download_bits(self._e, C.c_uint64(buf), _ptr(out), C.c_uint64(out.size)))
        return out

    def download_into(self, buf: int, host_ptr: int, capacity_elems: int, elem_bytes: int = 4):
        fn = self._lib.b200_download_bits if elem_bytes == 4 else self._lib.b200_download_bf16
        self._check(fn(self._e, C.c_uint64(buf), C.c_void_p(host_ptr), C.c_uint64(capacity_elems)))

    def free(self, buf: int):
        self._lib.b200_free(self._e, C.c_uint64(buf))

    def zeros_dram(self, dims, elem: int = F32, bf16: bool = False) -> Out:
        return self._call(self._lib.b200_zeros, C.c_uint64(dims[0]), C.c_uint64(dims[1]),
                          C.c_int32(BF16 if bf16 else elem))

    def device_ptr(self, buf: int) -> Tuple[int, int]:
        p = C.c_void_p()
        n = C.c_uint64()
        st = self._lib.b200_device_ptr(self._e, C.c_uint64(buf), C.byref(p), C.byref(n))
        if st:
            raise TtError(st, f"buffer {buf} is not live on this engine")
        return p.value, n.value

    def adopt(self, device_ptr: int, rows: int, cols: int, elem: int) -> int:
        out = C.c_uint64()
        self._check(self._lib.b200_adopt(self._e, C.c_void_p(device_ptr), C.c_uint64(rows), C.c_uint64(cols),
                                         C.c_int32(elem), C.byref(out)))
        return out.value

    def copy_into(self, src: int, dst: int):
        self._check(self._lib.b200_copy_into(self._e, C.c_uint64(src), C.c_uint64(dst)))

    def write_ptr(self, buf: int, host_ptr: int, n: int, elem_bytes: int = 4):
        fn = self._lib.b200_write_f32 if elem_bytes == 4 else self._lib.b200_write_bf16
        self._check(fn(self._e, C.c_uint64(buf), C.c_void_p(host_ptr), C.c_uint64(n)))

    # -- products (server.rs:70,178,191,229,245) -----------------------------------
    def matmul(self, a, b, mkn) -> np.ndarray:
        a = np.ascontiguousarray(a, dtype=np.float32)
        b = np.ascontiguousarray(b, dtype=np.float32)
        out = np.empty((mkn[0], mkn[2]), dtype=np.float32)
        self._check(self._lib.b200_matmul_host(self._e, _ptr(a), _ptr(b), (C.c_uint64 * 3)(*mkn), _ptr(out)))
        return out

    def matmul_bf16(self, a_bits, b_bits, mkn) -> np.ndarray:
        """Host-staged BF16 product (bits in, bits out), copies overlapped with the product in row panels."""
        a = np.ascontiguousarray(a_bits, dtype=np.uint16)
        b = np.ascontiguousarray(b_bits, dtype=np.uint16)
        out = np.empty((mkn[0], mkn[2]), dtype=np.uint16)
        self.matmul_host_bf16_ptr(a.ctypes.data, b.ctypes.data, out.ctypes.data, mkn)
        return out

    def matmul_host_bf16_ptr(self, a_ptr: int, b_ptr: int, out_ptr: int, mkn):
        """The same from raw host addresses (pinned memory another library owns)."""
        self._check(self._lib.b200_matmul_host_bf16(self._e, C.c_void_p(a_ptr), C.c_void_p(b_ptr), (C.c_uint64 * 3)(*mkn),
                                                    C.c_void_p(out_ptr)))

    def matmul_silu_mul(self, a: int, b: int) -> Out:
        """silu(A Bg) * (A Bu) with B's gate and up columns interleaved in groups of 128 (see `interleave_gate_up`)."""
        return self._call(self._lib.b200_matmul_silu_mul, C.c_uint64(a), C.c_uint64(b))

    def matmul_rope(self, a: int, b: int, cos, sin, rope_cols: int) -> Out:
        """A B as BF16 with RoPE applied, in the product's epilogue, to the heads of 64 columns below `rope_cols`."""
        bc, bs = _block(cos), _block(sin)
        return self._call(self._lib.b200_matmul_rope, C.c_uint64(a), C.c_uint64(b), C.byref(bc), C.byref(bs), C.c_uint64(rope_cols))

    def matmul_add_rms_norm(self, a: int, b: int, resid: int, gains: int, eps: float):
        """(s, norm): s = resid + A B (F32), norm = RMSNorm(s) * gains as BF16, one kernel (see `b200_matmul_add_rms_norm`)."""
        out = (C.c_uint64 * 2)()
        dims = (C.c_uint64 * 2)()
        self._check(self._lib.b200_matmul_add_rms_norm(self._e, C.c_uint64(a), C.c_uint64(b), C.c_uint64(resid), C.c_uint64(gains),
                                                       C.c_float(eps), out, dims))
        d = (dims[0], dims[1])
        return [(out[0], d), (out[1], d)]

    def matmul_into(self, a: int, b: int, dst_ptrs, dst_dims, col_first: int, bf16: bool = True):
        """C = A B stored from the product's epilogue into columns [col_first, ...) of every matrix in
        `dst_ptrs` (device addresses: this GPU's or, opened with `ipc_open`, a peer's)."""
        arr = (C.c_void_p * len(dst_ptrs))(*dst_ptrs)
        self._check(self._lib.b200_matmul_into(self._e, C.c_uint64(a), C.c_uint64(b), arr, C.c_int32(len(dst_ptrs)),
                                               C.c_uint64(dst_dims[0]), C.c_uint64(dst_dims[1]), C.c_uint64(col_first),
                                               C.c_int32(1 if bf16 else 0)))

    def store_block_into(self, src, dst_ptrs, dst_dims, col_first: int):
        """A block (buffer, (row, col), (rows, cols)) stored into columns [col_first, ...) of every matrix in `dst_ptrs`."""
        sid, at, dims = src
        blk = BlockArg(sid, (C.c_uint64 * 2)(*at), (C.c_uint64 * 2)(*dims))
        arr = (C.c_void_p * len(dst_ptrs))(*dst_ptrs)
        self._check(self._lib.b200_store_block_into(self._e, C.byref(blk), arr, C.c_int32(len(dst_ptrs)), C.c_uint64(dst_dims[0]),
                                                    C.c_uint64(dst_dims[1]), C.c_uint64(col_first)))

    def matmul_into_multicast(self, a: int, b: int, multicast_ptr: int, dst_dims, col_first: int, bf16: bool = True):
        """`matmul_into` with the destination a multicast address that maps every rank's C: each piece is stored once
        and the NVSwitch delivers it to every GPU of the group."""
        self._check(self._lib.b200_matmul_into_multicast(self._e, C.c_uint64(a), C.c_uint64(b), C.c_void_p(multicast_ptr),
                                                         C.c_uint64(dst_dims[0]), C.c_uint64(dst_dims[1]), C.c_uint64(col_first),
                                                         C.c_int32(int(bf16))))

    def store_block_into_multicast(self, src, multicast_ptr: int, dst_dims, col_first: int):
        self._check(self._lib.b200_store_block_into_multicast(self._e, C.byref(_block(src)), C.c_void_p(multicast_ptr),
                                                              C.c_uint64(dst_dims[0]), C.c_uint64(dst_dims[1]), C.c_uint64(col_first)))

    def ipc_export(self, buf: int) -> bytes:
        h = (C.c_uint8 * 64)()
        self._check(self._lib.b200_ipc_export(self._e, C.c_uint64(buf), h))
        return bytes(h)

    def ipc_open(self, handle: bytes) -> int:
        h = (C.c_uint8 * 64)(*handle)
        p = C.c_void_p()
        self._check(self._lib.b200_ipc_open(self._e, h, C.byref(p)))
        return p.value

    def ipc_close(self, ptr: int):
        self._check(self._lib.b200_ipc_close(self._e, C.c_void_p(ptr)))

    def matmul_dram(self, a: int, a_transposed: bool, b: int, b_transposed: bool) -> Out:
        return self._call(self._lib.b200_matmul, C.c_uint64(a), C.c_int32(a_transposed), C.c_uint64(b),
                          C.c_int32(b_transposed), C.c_int32(0))

    def matmul_dram_bf16(self, a: int, a_transposed: bool, b: int, b_transposed: bool) -> Out:
        return self._call(self._lib.b200_matmul, C.c_uint64(a), C.c_int32(a_transposed), C.c_uint64(b),
                          C.c_int32(b_transposed), C.c_int32(1))

    def matmul_dram_batched_layout(self, a: int, b: int, items, mkn, layout: Optional[BatchedLayout] = None,
                                   bf16: bool = False) -> Out:
        n = len(items)
        ab = (Block * max(n, 1))()
        bb = (Block * max(n, 1))()
        for i, (x, y) in enumerate(items):
            ab[i] = Block((C.c_uint64 * 2)(*x[0]), int(x[1]), 0)
            bb[i] = Block((C.c_uint64 * 2)(*y[0]), int(y[1]), 0)
        lay = C.byref(layout) if layout is not None else None
        return self._call(self._lib.b200_matmul_batched, C.c_uint64(a), C.c_uint64(b), ab, bb, C.c_uint64(n),
                          (C.c_uint64 * 3)(*mkn), lay, C.c_int32(bf16))

    def matmul_dram_batched(self, a: int, b: int, items, mkn, bf16: bool = False) -> Out:
        return self.matmul_dram_batched_layout(a, b, items, mkn, None, bf16)

    def last_matmul_path(self) -> str:
        return self._lib.b200_last_matmul_path(self._e).decode()

    def last_decode_form(self) -> str:
        """ "cluster16x3" (and the like) / "cluster16" / "cluster8" / "grid": the form the last `decode_layers` took."""
        return self._lib.b200_last_decode_form(self._e).decode()

    # -- element-wise (server.rs:492-566) --------------------------------------------
    def eltwise_op_as(self, op, a: int, b: Optional[int] = None, c: Optional[int] = None, bf16: bool = False) -> Out:
        if not isinstance(op, EltwiseOp):
            op = EltwiseOp(*op)
        return self._call(self._lib.b200_eltwise, C.byref(op), C.c_uint64(a), C.c_uint64(b or 0), C.c_uint64(c or 0),
                          C.c_int32(bf16))

    def eltwise_op(self, op, a, b=None, c=None) -> Out:
        return self.eltwise_op_as(op, a, b, c, False)

    def eltwise(self, kind: int, scalar: float, a: int, b: Optional[int] = None) -> Out:
        return self.eltwise_op_as(EltwiseOp(kind, scalar, 0.0), a, b, None, False)

    def eltwise_blocks_as(self, op, a, b=None, c=None, bf16: bool = False) -> Out:
        if not isinstance(op, EltwiseOp):
            op = EltwiseOp(*op)
        ba = _block(a)
        bb = _block(b) if b is not None else None
        bc = _block(c) if c is not None else None
        return self._call(self._lib.b200_eltwise_blocks, C.byref(op), C.byref(ba),
                          C.byref(bb) if bb is not None else None, C.byref(bc) if bc is not None else None,
                          C.c_int32(bf16))

    def eltwise_blocks(self, op, a, b=None, c=None) -> Out:
        return self.eltwise_blocks_as(op, a, b, c, False)

    def cast_float(self, a: int, bf16: bool) -> Out:
        return self._call(self._lib.b200_cast_float, C.c_uint64(a), C.c_int32(bf16))

    def cast_bfp(self, a: int, format: Optional[int]) -> Out:
        """`cast_bfp(id, format)` (server.rs:141): format 8 stores an F32 or BF16 buffer as BFP8; None widens a BFP8
        buffer to F32 (the trait's `None`); "bf16" widens it to BF16."""
        code = {8: 8, None: 0, "bf16": -16}[format]
        return self._call(self._lib.b200_cast_bfp, C.c_uint64(a), C.c_int32(code))

    def download_bfp(self, buf: int):
        """(datums u8 [rows, cols], exponents u8 [rows, cols / 16]) of a BFP8 buffer, as stored."""
        (rows, cols), elem = self.dims_of(buf)
        d = np.empty((rows, cols), dtype=np.uint8)
        x = np.empty((rows, max(cols // 16, 1)), dtype=np.uint8)
        self._check(self._lib.b200_download_bfp(self._e, C.c_uint64(buf), _ptr(d), _ptr(x), C.c_uint64(d.size)))
        return d, x[:, :cols // 16]

    def rope_blocks(self, x, cos, sin, head: int, bf16: bool = False) -> Out:
        bx, bc, bs = _block(x), _block(cos), _block(sin)
        return self._call(self._lib.b200_rope_blocks, C.byref(bx), C.byref(bc), C.byref(bs), C.c_uint64(head),
                          C.c_int32(bf16))

    # -- reductions (server.rs:80,399-477) ---------------------------------------------
    def reduce(self, a: int, op: int, axis: int, then: Optional[Tuple[int, int]] = None) -> Out:
        tk, tb = then if then else (0, 0)
        return self._call(self._lib.b200_reduce, C.c_uint64(a), C.c_int32(op), C.c_int32(axis), C.c_uint32(tk),
                          C.c_uint32(tb))

    def sum_rows(self, a: int) -> Out:
        return self._call(self._lib.b200_sum_rows, C.c_uint64(a))

    def full_sum(self, a: int, mean: bool = False) -> Out:
        return self._call(self._lib.b200_full_sum, C.c_uint64(a), C.c_int32(mean))

    def full_reduce(self, values, dims, mean: bool) -> float:
        a = np.ascontiguousarray(values, dtype=np.float32)
        out = C.c_float()
        self._check(self._lib.b200_full_reduce(self._e, _ptr(a), (C.c_uint64 * 2)(*dims), C.c_int32(mean),
                                               C.byref(out)))
        return out.value

    def softmax_rows(self, x: int, mask: Optional[int], scale: float) -> Out:
        return self._call(self._lib.b200_softmax_rows, C.c_uint64(x), C.c_uint64(mask or 0), C.c_float(scale))

    def softmax_rows_as(self, x: int, mask: Optional[int], scale: float, bf16: bool) -> Out:
        return self._call(self._lib.b200_softmax_rows_as, C.c_uint64(x), C.c_uint64(mask or 0), C.c_float(scale),
                          C.c_int32(bf16))

    def log_softmax_rows(self, x: int) -> Out:
        return self._call(self._lib.b200_log_softmax_rows, C.c_uint64(x))

    def rms(self, a: int, eps: float) -> Out:
        return self._call(self._lib.b200_rms, C.c_uint64(a), C.c_float(eps))

    def rms_norm_as(self, a: int, gamma: Optional[int], eps: float, bf16: bool) -> Out:
        return self._call(self._lib.b200_rms_norm, C.c_uint64(a), C.c_uint64(gamma or 0), C.c_float(eps),
                          C.c_int32(bf16))

    def rms_norm(self, a: int, gamma: Optional[int], eps: float) -> Out:
        return self.rms_norm_as(a, gamma, eps, False)

    def add_rms_norm(self, a: int, b: int, gamma: Optional[int], eps: float):
        return self.add_rms_norm_as(a, b, gamma, eps, False)

    def add_rms_norm_as(self, a: int, b: int, gamma: Optional[int], eps: float, bf16: bool):
        """(s, norm): s = a + b, norm = RMSNorm(s) * gamma, the norm rounded once to BF16 where `bf16`."""
        out = (C.c_uint64 * 2)()
        dims = (C.c_uint64 * 2)()
        self._check(self._lib.b200_add_rms_norm_as(self._e, C.c_uint64(a), C.c_uint64(b), C.c_uint64(gamma or 0),
                                                   C.c_float(eps), C.c_int32(1 if bf16 else 0), out, dims))
        d = (dims[0], dims[1])
        return [(out[0], d), (out[1], d)]

    def argmax_row(self, a: int) -> Out:
        return self._call(self._lib.b200_argmax_row, C.c_uint64(a))

    # -- indexing (server.rs:269-379,482) -----------------------------------------------
    def select_rows(self, table: int, indices: int) -> Out:
        return self._call(self._lib.b200_select_rows, C.c_uint64(table), C.c_uint64(indices))

    def pick_columns(self, input: int, indices: int) -> Out:
        return self._call(self._lib.b200_pick_columns, C.c_uint64(input), C.c_uint64(indices))

    def scatter_add_columns(self, t: int, indices: int, value: int) -> Out:
        return self._call(self._lib.b200_scatter_add_columns, C.c_uint64(t), C.c_uint64(indices), C.c_uint64(value))

    def select_add_rows(self, t: int, indices: int, value: int) -> Out:
        return self._call(self._lib.b200_select_add_rows, C.c_uint64(t), C.c_uint64(indices), C.c_uint64(value))

    def rows_add(self, t: int, indices: Sequence[int], value: int) -> Out:
        idx = (C.c_uint64 * max(len(indices), 1))(*indices)
        return self._call(self._lib.b200_rows_add, C.c_uint64(t), idx, C.c_uint64(len(indices)), C.c_uint64(value))

    def assign_rows(self, t: int, value: int, rows: Sequence[Tuple[int, int]]) -> Out:
        flat = [x for p in rows for x in p]
        arr = (C.c_uint64 * max(len(flat), 1))(*flat)
        return self._call(self._lib.b200_assign_rows, C.c_uint64(t), C.c_uint64(value), arr, C.c_uint64(len(rows)))

    def scatter_rows(self, table: int, indices: int, values: int, column: bool) -> Out:
        return self._call(self._lib.b200_scatter_rows, C.c_uint64(table), C.c_uint64(indices), C.c_uint64(values),
                          C.c_int32(column))

    def scatter_rows_into(self, table: int, indices: int, values, column: bool = False):
        """`scatter_rows` into `table` itself (server.rs:389); values = (buffer, (row, col), (rows, cols))."""
        vid, at, dims = values
        blk = BlockArg(vid, (C.c_uint64 * 2)(*at), (C.c_uint64 * 2)(*dims))
        self._check(self._lib.b200_scatter_rows_into(self._e, C.c_uint64(table), C.c_uint64(indices), C.byref(blk),
                                                     C.c_int32(column)))

    def reshape(self, a: int, rows: int, cols: int) -> Out:
        """The same words as another [rows, cols]: a view (no copy)."""
        return self._call(self._lib.b200_reshape, C.c_uint64(a), C.c_uint64(rows), C.c_uint64(cols))

    def gather_indexed(self, input: int, indices: int) -> Out:
        return self._call(self._lib.b200_gather_indexed, C.c_uint64(input), C.c_uint64(indices))

    def gather_rows(self, sources: Sequence[int], rows: Sequence[Tuple[int, int]], cols: int) -> Out:
        src = (C.c_uint64 * max(len(sources), 1))(*sources)
        flat = [x for p in rows for x in p]
        arr = (C.c_uint64 * max(len(flat), 1))(*flat)
        return self._call(self._lib.b200_gather_rows, src, C.c_uint64(len(sources)), arr, C.c_uint64(len(rows)),
                          C.c_uint64(cols))

    def slice_rows(self, a: int, first: int, rows: int) -> Out:
        return self._call(self._lib.b200_slice_rows, C.c_uint64(a), C.c_uint64(first), C.c_uint64(rows))

    def copy_blocks(self, a: int, moves, dims) -> Out:
        n = len(moves)
        arr = (BlockMove * max(n, 1))()
        for i, m in enumerate(moves):
            frm, to, ext, tr = m
            arr[i] = BlockMove((C.c_uint64 * 2)(*frm), (C.c_uint64 * 2)(*to), (C.c_uint64 * 2)(*ext), int(tr), 0)
        return self._call(self._lib.b200_copy_blocks, C.c_uint64(a), arr, C.c_uint64(n), (C.c_uint64 * 2)(*dims))

    def repack(self, a: int, sources, dims) -> Out:
        src = np.ascontiguousarray(sources, dtype=np.uint64).reshape(-1)
        assert src.size == 2 * dims[0] * dims[1]
        return self._call(self._lib.b200_repack, C.c_uint64(a), _ptr(src), (C.c_uint64 * 2)(*dims))

    def repack_many(self, inputs: Sequence[int], sources, dims) -> Out:
        """`repack_many(inputs, [(input, [row, col])...], dims)` (server.rs:317): one source a result element."""
        src = np.ascontiguousarray([(i, r, c) for i, (r, c) in sources], dtype=np.uint64).reshape(-1)
        ids = (C.c_uint64 * max(len(inputs), 1))(*inputs)
        return self._call(self._lib.b200_repack_many, ids, C.c_uint64(len(inputs)), _ptr(src), C.c_uint64(len(sources)),
                          (C.c_uint64 * 2)(*dims))

    def select_taps(self, table: int, indices: int, zero_row: bool) -> Out:
        return self._call(self._lib.b200_select_taps, C.c_uint64(table), C.c_uint64(indices), C.c_int32(zero_row))

    def cast_block(self, a, bf16: bool) -> Out:
        blk = _block(a)
        return self._call(self._lib.b200_cast_block, C.byref(blk), C.c_int32(bf16))

    def cast_bf16_storage(self, a: int, store: bool) -> Out:
        """`cast_bf16_storage` (server.rs:150): an F32 buffer kept as BF16, which a product reads beside an F32
        operand, or such a buffer widened back."""
        return self.cast_float(a, store)

    def cast_f16(self, a: int, to_f16: bool) -> Out:
        return self._call(self._lib.b200_cast_f16, C.c_uint64(a), C.c_int32(to_f16))

    def pow(self, x: int, y) -> Out:
        """`pow(x, PowArg)` (server.rs:578): y = ("tensor", id), ("scalar", s) or ("int", id)."""
        kind, v = y
        code = {"tensor": 0, "scalar": 1, "int": 2}[kind]
        return self._call(self._lib.b200_pow, C.c_uint64(x), C.c_int32(code), C.c_uint64(0 if code == 1 else v),
                          C.c_float(v if code == 1 else 0.0))

    def scan(self, a: int, op: int) -> Out:
        return self._call(self._lib.b200_scan, C.c_uint64(a), C.c_int32(op))

    def sort_planes(self, a: int, elem: int, n: int, descending: bool, indices: bool):
        """`sort_planes(a, Spec{elem, n, descending, indices})` (server.rs:758): ((keys, dims), (indices, dims) | None)."""
        keys, idx = C.c_uint64(), C.c_uint64()
        dims = (C.c_uint64 * 2)()
        self._check(self._lib.b200_sort_planes(self._e, C.c_uint64(a), C.c_int32(elem), C.c_uint64(n), C.c_int32(descending),
                                               C.byref(keys), C.byref(idx) if indices else None, dims))
        d = (dims[0], dims[1])
        return (keys.value, d), ((idx.value, d) if indices else None)

    def random_dram(self, dims, draw, base: int) -> Out:
        """`random_dram(dims, Draw, base)` (server.rs:768).  draw: ("unit",), ("uniform", lo, hi),
        ("bernoulli", p, int), ("normal", mean, std, int), ("int_range", lo, hi), ("int_words",)."""
        name, args = draw[0], draw[1:]
        code = {"unit": 0, "uniform": 1, "bernoulli": 2, "normal": 3, "int_range": 4, "int_words": 5}[name]
        a = b = 0.0
        lo = hi = 0
        as_int = False
        if name == "uniform":
            a, b = args
        elif name == "bernoulli":
            a, as_int = args
        elif name == "normal":
            a, b, as_int = args
        elif name == "int_range":
            lo, hi = args
        return self._call(self._lib.b200_random, (C.c_uint64 * 2)(*dims), C.c_int32(code), C.c_float(a), C.c_float(b),
                          C.c_int32(lo), C.c_int32(hi), C.c_int32(as_int), C.c_uint64(base & (2**64 - 1)))

    def pool_bf16(self, a: int, windows, divisors, dims) -> Out:
        """`pool_bf16(a, windows, divisors, dims)` (server.rs:118): windows is a list of lists of [row, col]."""
        offsets = np.zeros(len(windows) + 1, dtype=np.uint64)
        offsets[1:] = np.cumsum([len(w) for w in windows])
        coords = np.ascontiguousarray([rc for w in windows for rc in w], dtype=np.uint64).reshape(-1)
        if coords.size == 0:
            coords = np.zeros(2, dtype=np.uint64)
        div = np.ascontiguousarray(divisors, dtype=np.uint64)
        assert div.size == len(windows)
        return self._call(self._lib.b200_pool_bf16, C.c_uint64(a), _ptr(offsets), _ptr(coords), _ptr(div if div.size else np.zeros(1, np.uint64)),
                          C.c_uint64(len(windows)), (C.c_uint64 * 2)(*dims))

    def metadata(self, bits, dims, elem: int) -> int:
        a = np.ascontiguousarray(bits).view(np.uint32) if np.asarray(bits).dtype.itemsize == 4 \
            else np.ascontiguousarray(bits, dtype=np.uint32)
        assert a.size == dims[0] * dims[1]
        out = C.c_uint64()
        self._check(self._lib.b200_metadata(self._e, _ptr(a), (C.c_uint64 * 2)(*dims), C.c_int32(elem), C.byref(out)))
        return out.value

    def gddr_free_bytes(self) -> Tuple[int, int]:
        out = (C.c_uint64 * 2)()
        self._check(self._lib.b200_free_bytes(self._e, out))
        return out[0], out[1]

    @staticmethod
    def attention_item_array(items):
        """The head list marshalled once, for a caller that issues the same list every step."""
        arr = (AttentionItem * max(len(items), 1))()
        for i, (q, k, v) in enumerate(items):
            arr[i] = AttentionItem((C.c_uint64 * 2)(*q), (C.c_uint64 * 2)(*k), (C.c_uint64 * 2)(*v))
        return arr

    def attention_rows(self, buffers, items, dims, scale: float) -> Out:
        """`attention_rows([q, k, v, mask], items, [m, d, l, dv], scale)` (server.rs:257): each item is
        the (row, col) of a head's query, key and value blocks; the result is the
        [1, len(items) * m * dv] row of the heads' rows."""
        return self.attention_rows_as(buffers, items, dims, scale, False)

    def attention_rows_as(self, buffers, items, dims, scale: float, bf16: bool) -> Out:
        """`attention_rows` with its result rounded once to BF16 where `bf16`."""
        arr = items if isinstance(items, C.Array) else self.attention_item_array(items)
        return self._call(self._lib.b200_attention_rows_as, (C.c_uint64 * 4)(*buffers), arr, C.c_uint64(len(items)),
                          (C.c_uint64 * 4)(*dims), C.c_float(scale), C.c_int32(1 if bf16 else 0))

    @staticmethod
    def attention_block_array(items):
        """The block list marshalled once, for a caller that issues the same list every step."""
        arr = (AttentionBlock * max(len(items), 1))()
        for i, (a, b, c, o) in enumerate(items):
            arr[i] = AttentionBlock((C.c_uint64 * 2)(*a), (C.c_uint64 * 2)(*b), (C.c_uint64 * 2)(*c), (C.c_uint64 * 2)(*o))
        return arr

    def attention_blocks(self, q: int, k: int, v: int, items, dims, scale: float, causal: bool, result_dims) -> Out:
        """Fused attention over whole sequences (what ops.rs:4825 `padded_attention` composes): items are
        ((q_row, q_col), (k_row, k_col), (v_row, v_col), (o_row, o_col)); dims [sq, d, sk, dv]; BF16 in and out."""
        arr = items if isinstance(items, C.Array) else self.attention_block_array(items)
        n = len(items)
        return self._call(self._lib.b200_attention_blocks, C.c_uint64(q), C.c_uint64(k), C.c_uint64(v), arr, C.c_uint64(n),
                          (C.c_uint64 * 4)(*dims), C.c_float(scale), C.c_int32(1 if causal else 0), (C.c_uint64 * 2)(*result_dims))

    def decode_layers(self, shape: "DecodeShape", x: int, layer_buffers: Sequence[int], final_norm: int, cos: int, sin: int,
                      position: int) -> Out:
        """One generation step through every layer as one launch (`b200_decode_layers`): 8 buffer ids a layer -- norm1, Wqkv,
        Wo, norm2, Wgate|up, Wdown, key cache, value cache.  Returns the final norm of the stream, BF16 [rows, hidden]."""
        ids = (C.c_uint64 * len(layer_buffers))(*layer_buffers)
        return self._call(self._lib.b200_decode_layers, C.byref(shape), C.c_uint64(x), ids, C.c_uint64(final_norm), C.c_uint64(cos),
                          C.c_uint64(sin), C.c_uint64(position))

    def set_matmul_sm_limit(self, sms: int):
        """Tensor-core products use at most `sms` SMs (0 = all): room for a collective beside them."""
        self._lib.b200_set_matmul_sm_limit(self._e, C.c_int32(sms))

    # -- traces (server.rs:591-660) ------------------------------------------------------------
    def begin_trace(self):
        self._check(self._lib.b200_begin_trace(self._e))

    def end_trace(self) -> int:
        t = C.c_uint64()
        self._check(self._lib.b200_end_trace(self._e, C.byref(t)))
        return t.value

    def run_trace(self, trace: int):
        self._check(self._lib.b200_run_trace(self._e, C.c_uint64(trace)))

    def run_trace_io(self, trace: int, input: int, values, output: int):
        """The trait's `run_trace(trace, input, values, output)` (server.rs:648-657): overwrite the input, replay,
        read the output back; returns (output, (write_s, replay_s, read_s))."""
        run = self.run_generic_trace(trace, [(input, values)], [(output, "f32")])
        return run[0][0], run[1]

    def run_generic_trace(self, trace: int, inputs, outputs):
        """`run_generic_trace` (server.rs:746-753, 1205-1238): inputs = [(buffer, array of 32-bit values)], outputs =
        [(buffer, "f32" | "bits")]; returns ([arrays], (write_s, replay_s, read_s))."""
        import time
        self.sync()
        t0 = time.perf_counter()
        for buf, values in inputs:
            a = np.ascontiguousarray(values)
            assert a.dtype.itemsize == 4
            self._check(self._lib.b200_write_f32(self._e, C.c_uint64(buf), _ptr(a), C.c_uint64(a.size)))
        t1 = time.perf_counter()
        self.run_trace(trace)
        self.sync()
        t2 = time.perf_counter()
        read = [self.download(buf) if kind == "f32" else self.download_bits(buf) for buf, kind in outputs]
        return read, (t1 - t0, t2 - t1, time.perf_counter() - t2)

    def release_trace(self, trace: int):
        self._lib.b200_release_trace(self._e, C.c_uint64(trace))

    def trace_footprint(self, trace: int) -> int:
        """`trace_footprint` (server.rs:688): the device bytes the trace holds until it is released."""
        n = C.c_uint64()
        st = self._lib.b200_trace_footprint(self._e, C.c_uint64(trace), C.byref(n))
        if st:
            raise TtError(st, f"no trace {trace}")
        return n.value

    def trace_ops(self, trace: int):
        """`trace_ops` (server.rs:664): [(label, kernels)] of the captured ops, in capture order."""
        n = C.c_uint64()
        st = self._lib.b200_trace_ops(self._e, C.c_uint64(trace), None, C.c_uint64(0), C.byref(n))
        if st:
            raise TtError(st, f"no trace {trace}")
        rows = (OpStat * max(1, n.value))()
        self._lib.b200_trace_ops(self._e, C.c_uint64(trace), rows, C.c_uint64(n.value), C.byref(n))
        return [(rows[i].op.decode(), int(rows[i].launches)) for i in range(n.value)]

    # -- the profile mode (server.rs:672 `profile_mode`, :683 `profile_report`) --------------
    def profile_mode(self, on: bool):
        """On: from here every `set_op_label` marks the stream.  Off: waits for the device and returns the table
        `profile_report` gives."""
        if on:
            self._check(self._lib.b200_profile_start(self._e))
            self.profiling = True
            return None
        self.profiling = False
        self._check(self._lib.b200_profile_stop(self._e))
        return self.profile_report()

    def profile_report(self):
        """[{op, calls, launches, device_ms}] by label, in order of first appearance."""
        n = C.c_uint64()
        self._check(self._lib.b200_profile_read(self._e, None, C.c_uint64(0), C.byref(n)))
        rows = (OpStat * max(1, n.value))()
        self._check(self._lib.b200_profile_read(self._e, rows, C.c_uint64(n.value), C.byref(n)))
        return [{"op": rows[i].op.decode(), "calls": int(rows[i].calls), "launches": int(rows[i].launches),
                 "device_ms": float(rows[i].device_ms)} for i in range(n.value)]

    def debug_stalled_wait(self):
        """Runs a bounded device wait that nothing ends (needs `wait_limit_cycles`): the next wait raises Timeout."""
        self._check(self._lib.b200_debug_stalled_wait(self._e))

    # -- waits and observability (lib.rs:218, server.rs:584,663) ---------------------------
    def sync(self):
        self._check(self._lib.b200_sync(self._e))

    def set_op_label(self, label: str):
        self._lib.b200_set_op_label(self._e, label.encode())

    def device_traffic(self) -> Traffic:
        t = Traffic()
        self._lib.b200_traffic_get(self._e, C.byref(t))
        return t

    def last_oom(self) -> Tuple[int, int, int]:
        o = (C.c_uint64 * 3)()
        self._lib.b200_last_oom(self._e, o)
        return o[0], o[1], o[2]

    def timer_start(self):
        self._check(self._lib.b200_timer_start(self._e))

    def timer_stop(self) -> float:
        ms = C.c_float()
        self._check(self._lib.b200_timer_stop(self._e, C.byref(ms)))
        return ms.value

    def stream(self) -> int:
        return self._lib.b200_stream(self._e)


__all__ = ["CudaEngine", "TtError", "EltwiseOp", "Block", "BlockMove", "BlockArg", "BatchedLayout", "Traffic", "OpStat",
           "load_library", "library_path", "kinds",
           "F32", "I32", "BOOL", "BF16", "BFP8", "SUM", "MAX", "PROD", "ALL", "ANY", "BITOR", "SUM_I32", "PROD_I32",
           "MIN_I32", "MAX_I32", "ROWS", "COLS"]
