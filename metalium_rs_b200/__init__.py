"""B200 engine for the hot path metalium-rs's `burn-tt` backend sends to `tt-kernels`.

The product is `libb200tt.so` (CUDA kernels for sm_100a behind the C ABI in
include/b200tt.h).  `CudaEngine` is the host-side mirror of the reference's `Engine`
trait over that ABI.
"""
from . import kinds
from .engine import (ALL, ANY, BF16, BFP8, BITOR, BOOL, COLS, F32, I32, MAX, MAX_I32, MIN_I32, PROD, PROD_I32, ROWS, SUM,
                     SUM_I32, UNSUPPORTED, AttentionItem, BatchedLayout, Block, BlockArg, BlockMove, CudaEngine, EltwiseOp, Traffic, TtError,
                     library_path, load_library)

__all__ = ["CudaEngine", "TtError", "EltwiseOp", "Block", "BlockMove", "BlockArg", "BatchedLayout", "Traffic",
           "AttentionItem", "UNSUPPORTED", "load_library", "library_path", "kinds", "F32", "I32", "BOOL", "BF16", "BFP8", "SUM", "MAX", "PROD", "ALL", "ANY",
           "BITOR", "SUM_I32", "PROD_I32", "MIN_I32", "MAX_I32", "ROWS", "COLS"]
