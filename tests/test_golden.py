"""The committed golden vectors (tests/golden/hot_path.npz, made by tests/golden/make_golden.py):
the oracle must still reproduce them (no GPU), and the engine must match them through the C ABI."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest

from oracle import models as M
from oracle import oracle as orc

HERE = Path(__file__).resolve().parent
spec = importlib.util.spec_from_file_location("make_golden", HERE / "golden" / "make_golden.py")
G = importlib.util.module_from_spec(spec)
spec.loader.exec_module(G)
GOLD = np.load(HERE / "golden" / "hot_path.npz")


def test_oracle_reproduces_the_golden_vectors():
    now = G.build()
    assert sorted(now) == sorted(GOLD.files)
    for k in GOLD.files:
        a, b = np.asarray(now[k]), GOLD[k]
        assert a.shape == b.shape and a.dtype == b.dtype, k
        same = (a.view(np.uint8) == b.view(np.uint8)).all() if a.dtype.kind != "f" else \
            np.array_equal(a.view(np.uint32) if a.dtype == np.float32 else a, b.view(np.uint32) if b.dtype == np.float32 else b)
        assert same, f"{k}: the oracle no longer gives its committed vector"


@pytest.mark.gpu
def test_engine_matches_the_golden_vectors(eng):
    from metalium_rs_b200 import BOOL, COLS, I32, MAX, ROWS, SUM, EltwiseOp, kinds
    a, b, c = G.inputs()
    ia, ib, ic = (eng.upload(x, 24, 40) for x in (a, b, c))
    for k in G.EXACT_KINDS + G.APPROX_KINDS:
        src = ib if k in ("LOG", "SQRT", "RECIP") else ia
        ar = kinds.ARITY[getattr(kinds, k)]
        out, _ = eng.eltwise_op(EltwiseOp(getattr(kinds, k), 0.5, 1.5), src, ib if ar >= 2 else None, ic if ar == 3 else None)
        got = eng.download_bits(out)
        if k in G.EXACT_KINDS:
            assert np.array_equal(got, GOLD["elt_" + k]), k
        else:
            assert orc.ulp_error(got, GOLD["elt_" + k]) <= orc.ULP_BOUND[k] + 1, k
        eng.free(out)
    o, _ = eng.cast_float(ia, True)
    assert np.array_equal(eng.download_bf16(o), GOLD["bf16"]); eng.free(o)
    o, _ = eng.reduce(ia, SUM, ROWS)
    assert np.array_equal(eng.download_bits(o), GOLD["sum_rows"]); eng.free(o)
    o, _ = eng.reduce(ia, MAX, COLS)
    assert np.array_equal(eng.download_bits(o), GOLD["max_cols"]); eng.free(o)
    o, _ = eng.softmax_rows(ia, None, 1.0)
    assert np.max(np.abs(eng.download(o) - GOLD["softmax"]) / GOLD["softmax"]) <= orc.softmax_bound(40); eng.free(o)
    mask = (orc.integers(G.SEED, 4, (24, 40), 3) == 0).astype(np.uint32)
    im = eng.upload_bits(mask, 24, 40, BOOL)
    o, _ = eng.softmax_rows(ia, im, 0.5)
    got, want = eng.download(o), GOLD["softmax_masked"]
    assert np.array_equal(got == 0, want == 0)
    assert np.max(np.abs(got - want)[want > 0] / want[want > 0]) <= orc.softmax_bound(40); eng.free(o)
    o, _ = eng.argmax_row(ia)
    assert np.array_equal(eng.download_bits(o).view(np.int32), GOLD["argmax"]); eng.free(o)
    ig = eng.upload(b[0].reshape(1, -1), 1, 40)
    o, _ = eng.rms_norm(ia, ig, 1e-5)
    assert np.max(np.abs(eng.download(o) - GOLD["rms_norm"])) <= 1e-5 * np.abs(GOLD["rms_norm"]).max(); eng.free(o)
    cos, sin = orc.rope_tables(24, 8, 10000.0)
    ico, isi = eng.upload(cos, 24, 8), eng.upload(sin, 24, 8)
    o, _ = eng.rope_blocks((ia, (0, 0), (24, 40)), (ico, (0, 0), (24, 8)), (isi, (0, 0), (24, 8)), 8)
    assert np.array_equal(eng.download(o).view(np.uint32), GOLD["rope"].view(np.uint32)); eng.free(o)
    rng = np.random.default_rng(G.SEED)
    xa, xb = rng.integers(-7, 8, (24, 40)).astype(np.float32), rng.integers(-7, 8, (40, 16)).astype(np.float32)
    ja, jb = eng.upload(xa, 24, 40), eng.upload(xb, 40, 16)
    o, _ = eng.matmul_dram(ja, False, jb, False)
    assert np.array_equal(eng.download(o), GOLD["gemm_int"]); eng.free(o)
    ha, hb = eng.upload_bf16(orc.to_bf16(a), 24, 40), eng.upload_bf16(orc.to_bf16(b.T.copy()), 40, 24)
    o, _ = eng.matmul_dram_bf16(ha, False, hb, False)
    step = np.abs(eng.download_bf16(o).astype(np.int32) - GOLD["gemm_bf16"].astype(np.int32))
    assert (step <= 1).mean() > 0.99 and (step == 0).mean() > 0.9; eng.free(o)
    idx = orc.integers(G.SEED, 5, (1, 10), 24)
    ii = eng.upload_bits(idx.view(np.uint32), 1, 10, I32)
    o, _ = eng.select_rows(ia, ii)
    assert np.array_equal(eng.download_bits(o), GOLD["select_rows"]); eng.free(o)
    from metalium_rs_b200 import workloads as W
    x = orc.normal(G.SEED, 6, (16, 784)); y = orc.integers(G.SEED, 7, (16, 1), 10)
    mlp = W.MlpStep(eng, *M.mlp_init(seed=G.SEED))
    ix, iy = eng.upload(x, 16, 784), eng.upload_bits(y.view(np.uint32), 16, 1, I32)
    res = mlp.step(ix, iy, 16, keep=True)
    assert abs(float(eng.download(res["loss"])[0, 0]) - float(GOLD["mlp_loss"][0])) <= 1e-5 * float(GOLD["mlp_loss"][0])
    assert np.max(np.abs(eng.download(res["logits"]) - GOLD["mlp_logits"])) <= 1e-5
    q, k, v, amask, items, dims = G.attention_rows_case()
    iq, ik, iv = eng.upload(q, *q.shape), eng.upload(k, *k.shape), eng.upload(v, *v.shape)
    iam = eng.upload_bits(amask, 1, dims[2], BOOL)
    o, _ = eng.attention_rows([iq, ik, iv, iam], items, dims, 0.25)
    assert np.max(np.abs(eng.download(o) - GOLD["attention_rows"])) <= 1e-5 * np.abs(v).max(); eng.free(o)
    xq, xk, xv = G.attention_blocks_case()
    jq, jk, jv = (eng.upload_bf16(x, 128, 64) for x in (xq, xk, xv))
    o, _ = eng.attention_blocks(jq, jk, jv, [((0, 0), (0, 0), (0, 0), (0, 0))], [128, 64, 128, 64], 0.125, True, [128, 64])
    got = orc.from_bf16(eng.download_bf16(o)).astype(np.float64)
    want, scale = GOLD["attention_blocks"].astype(np.float64), GOLD["attention_blocks_scale"].astype(np.float64)
    assert np.all(np.abs(got - want) <= 2.0 ** -7 * scale + 2.0 ** -9 * np.abs(want) + 1e-6); eng.free(o)
    (s2, _), (n2, _) = eng.add_rms_norm(ia, ic, ig, 1e-5)
    assert np.max(np.abs(eng.download(n2) - GOLD["add_rms_norm"])) <= 1e-5 * np.abs(GOLD["add_rms_norm"]).max()
    for v in list(res.values()) + [ia, ib, ic, im, ig, ico, isi, ja, jb, ha, hb, ii, ix, iy, iq, ik, iv, iam, jq, jk, jv, s2, n2]:
        eng.free(v)


MORE = np.load(HERE / "golden" / "more_ops.npz")


def test_oracle_reproduces_the_vectors_of_the_rest_of_the_trait():
    now = G.build_more()
    assert sorted(now) == sorted(MORE.files)
    for k in MORE.files:
        a, b = np.asarray(now[k]), MORE[k]
        assert a.shape == b.shape and a.dtype == b.dtype, k
        assert (np.ascontiguousarray(a).view(np.uint8) == np.ascontiguousarray(b).view(np.uint8)).all(), k


@pytest.mark.gpu
def test_engine_matches_the_vectors_of_the_rest_of_the_trait(eng):
    from metalium_rs_b200 import F32, I32
    x, xi, sums, table, taps, windows = G.more_inputs()
    ix, ixi, isums = eng.upload_bits(x, 40, 24, F32), eng.upload_bits(xi, 40, 24, I32), eng.upload_bits(sums, 40, 24, F32)
    for code, op in enumerate(orc.SCAN_OPS):
        src = ixi if op.startswith("i") else (isums if op in ("sum", "prod") else ix)
        o, _ = eng.scan(src, code)
        got, want = eng.download_bits(o), MORE["scan_" + op]
        if op in ("sum", "prod"):      # an arithmetic NaN's payload is not compared
            g, w = got.view(np.float32), want.view(np.float32)
            assert np.all((got == want) | (np.isnan(g) & np.isnan(w))), op
        else:
            assert np.array_equal(got, want), op
        eng.free(o)
    for is_i32, name, src in ((False, "f32", x[:, :20].T.copy()), (True, "i32", xi[:, :20].T.copy() & np.uint32(0x8000000F))):
        planes = orc.to_planes(src)
        ip = eng.upload_bits(planes, *planes.shape, I32 if is_i32 else F32)
        for desc in (False, True):
            (k, dims), idx = eng.sort_planes(ip, I32 if is_i32 else F32, 40, desc, True)
            assert np.array_equal(orc.from_planes(eng.download_bits(k), 20, 40), MORE[f"sort_{name}_{int(desc)}_keys"])
            assert np.array_equal(orc.from_planes(eng.download_bits(idx[0]), 20, 40).view(np.int32), MORE[f"sort_{name}_{int(desc)}_idx"])
            eng.free(k); eng.free(idx[0])
        eng.free(ip)
    words = np.concatenate([x.ravel(), sums.ravel(), xi.ravel()]).reshape(-1, 24)
    iw = eng.upload_bits(words, *words.shape, F32)
    o, _ = eng.cast_f16(iw, True)
    assert np.array_equal(eng.download_bf16(o).ravel(), MORE["f16_narrow"]); eng.free(o); eng.free(iw)
    halves = (xi >> np.uint32(16)).astype(np.uint16)
    ih = eng.upload_bf16(halves, 40, 24)
    o, _ = eng.cast_f16(ih, False)
    assert np.array_equal(eng.download_bits(o).ravel(), MORE["f16_widen"]); eng.free(o); eng.free(ih)
    it, itap = eng.upload(table, 20, 24), eng.upload_bits(taps, 3, 11, I32)
    o, _ = eng.select_taps(it, itap, True)
    assert np.array_equal(eng.download_bits(o), MORE["select_taps"]); eng.free(o)
    ib = eng.upload_bf16(orc.to_bf16(table), 20, 24)
    o, _ = eng.pool_bf16(ib, windows, [len(w) for w in windows], (6, 4))
    assert np.array_equal(eng.download_bits(o), MORE["pool_bf16"]); eng.free(o)
    o, _ = eng.repack_many([ix, isums], [(i % 2, ((5 * i) % 40, (3 * i) % 24)) for i in range(60)], (6, 10))
    assert np.array_equal(eng.download_bits(o), MORE["repack_many"]); eng.free(o)
    for name, draw in (("unit", ("unit",)), ("uniform", ("uniform", -3.0, 5.5)), ("bernoulli", ("bernoulli", 0.3, True)),
                       ("int_range", ("int_range", -5, 12)), ("int_words", ("int_words",))):
        o, _ = eng.random_dram((9, 31), draw, 0x5EED)
        assert np.array_equal(eng.download_bits(o), np.ascontiguousarray(MORE["draw_" + name]).view(np.uint32)), name
        eng.free(o)
    for i in (ix, ixi, isums, it, itap, ib):
        eng.free(i)
