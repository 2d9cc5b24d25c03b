"""The C-ABI library loads and exports every symbol include/b200tt.h declares.
No compute call is made: this runs without a GPU."""
import ctypes
import re
from pathlib import Path

from metalium_rs_b200 import CudaEngine, TtError, engine

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "b200tt.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 55
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in b200tt.h but not exported: {missing}"


def test_library_needs_no_driver_to_load(lib):
    # The engine resolves the driver's tensor-map encoder at run time, so a machine
    # without libcuda can still load the library and be told there is no device.
    assert engine.library_path().exists()


def test_struct_layouts_match_the_header():
    assert ctypes.sizeof(engine.EltwiseOp) == 12
    assert ctypes.sizeof(engine.Block) == 24
    assert ctypes.sizeof(engine.BlockMove) == 56
    assert ctypes.sizeof(engine.BlockArg) == 40
    assert ctypes.sizeof(engine.BatchedLayout) == 8
    assert ctypes.sizeof(engine.Traffic) == 64
    assert ctypes.sizeof(engine.Config) == 32
    assert ctypes.sizeof(engine.OpStat) == 72


def test_create_without_a_device_is_refused_not_faked(lib):
    import torch
    if torch.cuda.is_available():
        return
    try:
        CudaEngine(0)
    except TtError as e:
        assert e.status == engine.NO_DEVICE
    else:
        raise AssertionError("an engine came up without a GPU: there must be no CPU fallback")


def test_kind_numbers_are_the_reference_s():
    from metalium_rs_b200 import kinds
    # crates/tt-kernels/src/kind.rs:12-26 and crates/tt-kernels/src/sfpu/ops.rs:24-251
    assert (kinds.ADD, kinds.SUB, kinds.MUL, kinds.MUL_SCALAR, kinds.RELU, kinds.RELU_BACKWARD, kinds.ADD_ROW,
            kinds.ADD_SCALAR) == (1, 2, 3, 4, 5, 6, 7, 11)
    assert (kinds.RECIP, kinds.DIV, kinds.EXP, kinds.LOG, kinds.SQRT, kinds.SIGMOID, kinds.GELU) == \
        (0x100, 0x101, 0x103, 0x104, 0x123, 0x12B, 0x12F)
    assert (kinds.ADD_RELU, kinds.SILU, kinds.SILU_MUL, kinds.SUB_EXP, kinds.MUL_ADD, kinds.SCALE_MASK_FILL) == \
        (0x1F0, 0x1F1, 0x1F2, 0x1F3, 0x1F4, 0x1F5)
    assert kinds.INT_ADD == 0x170 and kinds.INT_LE_S == 0x18D and kinds.ROUND == 0x190


def test_the_rust_shim_sources_follow_the_header_and_the_build():
    # The Rust crates are shipped as source (no cargo here): keep them from drifting.  Every function the
    # header declares is declared in b200-sys, and its build.rs compiles every CUDA source build.py does.
    import re
    from pathlib import Path
    from metalium_rs_b200 import build
    root = Path(__file__).resolve().parent.parent
    header = (root / "include" / "b200tt.h").read_text()
    declared = set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", header))
    ffi = (root / "metalium_rs_b200" / "rust" / "b200-sys" / "src" / "lib.rs").read_text()
    bound = set(re.findall(r"pub fn (b200_[a-z0-9_]+)\(", ffi))
    assert declared == bound, (sorted(declared - bound), sorted(bound - declared))
    build_rs = (root / "metalium_rs_b200" / "rust" / "b200-sys" / "build.rs").read_text()
    for src in build.SOURCES:
        assert f'"{src}"' in build_rs, src


def test_the_rust_shim_overrides_only_trait_methods_with_the_trait_s_signatures():
    # No Rust compiler here, so the shim's `impl Engine for CudaEngine` is held to the trait by text: every method
    # it defines is a method of `pub trait Engine` (crates/burn-tt/src/server.rs:42-786) with the same parameter
    # types and result type.  tests/golden/engine_trait.json is the trait's method list (made by
    # tests/golden/make_trait_signatures.py); where the reference tree is mounted the list is re-derived too.
    import json
    from tests.golden.make_trait_signatures import block_after, signatures, trait_signatures
    trait = json.loads((ROOT / "tests" / "golden" / "engine_trait.json").read_text())
    reference = Path(json.loads((ROOT / "BASELINE.json").read_text()).get("reference_path", ""))   # where the reference tree is mounted, if it is
    if (reference / "crates" / "burn-tt" / "src" / "server.rs").exists():
        assert trait_signatures(reference) == trait, "engine_trait.json is stale: run tests/golden/make_trait_signatures.py"
    shim = (ROOT / "metalium_rs_b200" / "rust" / "burn-tt-b200" / "src" / "lib.rs").read_text()
    impl = signatures(block_after(shim, r"impl Engine for CudaEngine"))
    alias = {"Made": "Result<(BufferId,[usize;2]),TtError>"}          # the shim's `type Made`
    assert len(impl) >= 60
    for name, sig in impl.items():
        assert name in trait, f"{name} is not a method of the trait"
        assert sig["params"] == trait[name]["params"], (name, sig["params"], trait[name]["params"])
        assert alias.get(sig["ret"], sig["ret"]) == trait[name]["ret"], (name, sig["ret"], trait[name]["ret"])
    # the required method and the capability probes are there (server.rs:53,70,75,240)
    for name in ("matmul", "supports_dram", "supports_batched_layout", "supports_exact_matmul"):
        assert name in impl
