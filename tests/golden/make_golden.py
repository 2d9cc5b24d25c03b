"""Writes tests/golden/hot_path.npz and more_ops.npz: outputs of the CPU oracle on small seeded inputs.

The reference's own golden file (crates/tt-tests/tests/golden/mnist_reduced.txt) pins Tensix
TF32 bits on MNIST and cannot be reproduced on a GPU, and the reference (Rust) cannot be
imported, so these vectors are the oracle's: committed so that a later change of the oracle,
or of the engine, shows up against fixed numbers.  Inputs are regenerated from their seeds by
the tests; only outputs are stored.

    python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import models as M  # noqa: E402
from oracle import oracle as orc  # noqa: E402

SEED = 0x601D
EXACT_KINDS = ["ADD", "SUB", "MUL", "DIV", "RECIP", "SQRT", "RELU", "RELU_BACKWARD", "NEG", "ABS", "ADD_RELU", "MUL_ADD",
               "CLAMP_MIN", "GT", "FLOOR", "ROUND", "LEAKY_RELU"]
APPROX_KINDS = ["EXP", "LOG", "SIGMOID", "SILU", "SILU_MUL", "TANH", "GELU", "GELU_TANH", "SUB_EXP"]


def inputs():
    a = orc.uniform(SEED, 1, (24, 40), -4, 4)
    b = orc.uniform(SEED, 2, (24, 40), 0.25, 4)
    c = orc.uniform(SEED, 3, (24, 40), -4, 4)
    return a, b, c


def build():
    a, b, c = inputs()
    out = {}
    for k in EXACT_KINDS + APPROX_KINDS:
        src = b if k in ("LOG", "SQRT", "RECIP") else a
        out["elt_" + k] = orc.eltwise(k, src, b, c, 0.5, 1.5)
    out["bf16"] = orc.to_bf16(a)
    out["sum_rows"] = orc.sum_rows_in_order(a).view(np.uint32)
    out["max_cols"] = orc.reduce(a, "MAX", 1)
    out["softmax"] = orc.softmax_rows(a)
    out["softmax_masked"] = orc.softmax_rows(a, (orc.integers(SEED, 4, (24, 40), 3) == 0).astype(np.uint32), 0.5)
    out["argmax"] = orc.argmax_rows(a)
    out["rms_norm"] = orc.rms_norm(a, b[0], 1e-5)
    cos, sin = orc.rope_tables(24, 8, 10000.0)
    out["rope"] = orc.rope(a, cos, sin, 8)
    rng = np.random.default_rng(SEED)
    ia, ib = rng.integers(-7, 8, (24, 40)).astype(np.float32), rng.integers(-7, 8, (40, 16)).astype(np.float32)
    out["gemm_int"] = orc.gemm_f32(ia, ib)
    out["gemm_bf16"] = orc.gemm_bf16(orc.to_bf16(a), orc.to_bf16(b.T.copy()))[0]
    idx = orc.integers(SEED, 5, (1, 10), 24)
    out["select_rows"] = orc.select_rows(a, idx).view(np.uint32)
    x = orc.normal(SEED, 6, (16, 784)); y = orc.integers(SEED, 7, (16, 1), 10)
    step = M.mlp_step(x, y, *M.mlp_init(seed=SEED))
    out["mlp_loss"] = np.array([step["loss"]], np.float32)
    out["mlp_logits"] = step["logits"]
    # attention for a few query rows a head (decode), its composition in F32
    q, k, v, mask, items, dims = attention_rows_case()
    out["attention_rows"] = orc.attention_rows(q, k, v, mask, items, dims, 0.25)
    # attention over whole sequences (prefill), F64
    xq, xk, xv = attention_blocks_case()
    o, s = orc.attention_blocks(orc.from_bf16(xq), orc.from_bf16(xk), orc.from_bf16(xv), 0.125, True)
    out["attention_blocks"] = o.astype(np.float32)
    out["attention_blocks_scale"] = s.astype(np.float32)
    # residual add + RMSNorm
    out["add_rms_norm"] = orc.rms_norm((a + c).astype(np.float32), b[0], 1e-5)
    return out


def attention_rows_case():
    m, d, l, dv = 2, 32, 64, 32
    q = orc.normal(SEED, 8, (2 * m, d))
    k = orc.normal(SEED, 9, (l, d))
    v = orc.normal(SEED, 10, (l, dv))
    mask = np.zeros(l, np.uint32)
    mask[50:] = 1
    items = [((0, 0), (0, 0), (0, 0)), ((m, 0), (0, 0), (0, 0))]      # two heads on one key/value head
    return q, k, v, mask, items, [m, d, l, dv]


def attention_blocks_case():
    return tuple(orc.to_bf16(orc.normal(SEED, t, (128, 64))) for t in (11, 12, 13))


# ---- the rest of the trait: scans, sort, binary16, taps, pooling windows, draws (tests/golden/more_ops.npz) ----
SPECIAL = np.array([0x00000000, 0x80000000, 0x7F800000, 0xFF800000, 0x7FC00000, 0xFFC00001, 0x3F800000, 0xBF800000,
                    0x00000001, 0x7F7FFFFF], dtype=np.uint32)


def more_inputs():
    x = np.round(orc.uniform(SEED, 21, (40, 24), -4, 4)).view(np.uint32).copy()
    sel = orc.integers(SEED, 22, (40, 24), 7) == 0
    x[sel] = SPECIAL[orc.integers(SEED, 23, (40, 24), len(SPECIAL))[sel]]
    xi = (orc.splitmix64(SEED, 24, 40 * 24) >> np.uint64(32)).astype(np.uint32).reshape(40, 24)
    sums = orc.uniform(SEED, 25, (40, 24), -4, 4).view(np.uint32)
    table = orc.normal(SEED, 26, (20, 24))
    taps = orc.integers(SEED, 27, (3, 11), 21).astype(np.int32)
    windows = [[[r, c], [r + 1, c], [r, c + 1], [r + 1, c + 1]] for r in range(0, 18, 3) for c in range(0, 20, 5)]
    windows[1] = [[i % 20, (7 * i) % 24] for i in range(37)]           # more than two blocks of sixteen
    return x, xi, sums, table, taps, windows


def build_more():
    x, xi, sums, table, taps, windows = more_inputs()
    out = {}
    for op in orc.SCAN_OPS:
        src = xi if op.startswith("i") else (sums if op in ("sum", "prod") else x)
        out["scan_" + op] = orc.scan(src, op)
    for desc in (False, True):
        k, i = orc.sort_rows(x[:, :20].T.copy(), False, desc)          # 20 problems of 40 positions
        out[f"sort_f32_{int(desc)}_keys"], out[f"sort_f32_{int(desc)}_idx"] = k, i
        k, i = orc.sort_rows(xi[:, :20].T.copy() & np.uint32(0x8000000F), True, desc)
        out[f"sort_i32_{int(desc)}_keys"], out[f"sort_i32_{int(desc)}_idx"] = k, i
    out["f16_narrow"] = orc.f16_bits_from_f32_bits(np.concatenate([x.ravel(), sums.ravel(), xi.ravel()]))
    out["f16_widen"] = orc.f32_bits_from_f16_bits((xi.ravel() >> np.uint32(16)).astype(np.uint16))
    out["select_taps"] = orc.select_taps(table.view(np.uint32), taps, True)
    out["pool_bf16"] = orc.pool_bf16(orc.to_bf16(table), windows, [len(w) for w in windows], (6, 4)).view(np.uint32)
    out["repack_many"] = orc.repack_many([x, sums], [(i % 2, ((5 * i) % 40, (3 * i) % 24)) for i in range(60)], (6, 10))
    for name, draw in (("unit", ("unit",)), ("uniform", ("uniform", -3.0, 5.5)), ("bernoulli", ("bernoulli", 0.3, True)),
                       ("int_range", ("int_range", -5, 12)), ("int_words", ("int_words",))):
        out["draw_" + name] = orc.random_draw((9, 31), draw, 0x5EED)
    return out


if __name__ == "__main__":
    np.savez_compressed(Path(__file__).with_name("hot_path.npz"), **build())
    print("wrote", Path(__file__).with_name("hot_path.npz"))
    np.savez_compressed(Path(__file__).with_name("more_ops.npz"), **build_more())
    print("wrote", Path(__file__).with_name("more_ops.npz"))
