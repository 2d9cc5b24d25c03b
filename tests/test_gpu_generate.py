"""Generation with a fixed-shape key/value cache: `scatter_rows_into` (crates/burn-tt/src/server.rs:389), the
reshape view, and decode steps (`attention_rows` over the cache) against the prefill of the same tokens
and against the CPU restatement.  What a cached step must equal is what the reference holds its own to
(crates/tt-models/src/kv_cache.rs:16-19, `step185_fixed_decode`): the growing-cache arithmetic, a masked
position adding an exact zero.  Tolerance: the logits' 2e-2 of the prefill test (BF16 weights and
activations; the two paths round their probabilities differently)."""
import numpy as np
import pytest

from metalium_rs_b200 import BF16, F32, I32, TtError, workloads as W
from oracle import models as M
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _i32(eng, a, r, c):
    return eng.upload_bits(np.ascontiguousarray(a, dtype=np.int32).view(np.uint32), r, c, I32)


@pytest.mark.parametrize("bf16", [False, True])
def test_scatter_rows_into_writes_the_table_itself(eng, bf16):
    table = orc.normal(0x6E, 1, (40, 24))
    values = orc.normal(0x6E, 2, (6, 64))            # the rows written are columns 16..40 of rows 1..5
    idx = np.array([[3, 39, 0, 3]], np.int32)        # row 3 twice: the later one stays
    if bf16:
        tb, vb = orc.to_bf16(table), orc.to_bf16(values)
        it, iv = eng.upload_bf16(tb, 40, 24), eng.upload_bf16(vb, 6, 64)
        want = tb.copy()
        src = vb
    else:
        it, iv = eng.upload(table, 40, 24), eng.upload(values, 6, 64)
        want = table.copy()
        src = values
    ii = _i32(eng, idx, 1, 4)
    eng.scatter_rows_into(it, ii, (iv, (1, 16), (4, 24)))
    for n, r in enumerate(idx[0]):
        want[r] = src[1 + n, 16:40]
    got = eng.download_bf16(it) if bf16 else eng.download(it)
    assert np.array_equal(got, want)
    assert eng.dims_of(it) == ((40, 24), BF16 if bf16 else F32)
    with pytest.raises(TtError):
        eng.scatter_rows_into(it, ii, (iv, (1, 16), (3, 24)))      # three rows for four indices
    with pytest.raises(TtError):
        eng.scatter_rows_into(it, ii, (iv, (4, 16), (4, 24)))      # the block leaves its buffer
    for i in (it, iv, ii):
        eng.free(i)


def test_scatter_rows_into_rounds_f32_rows_into_a_bf16_table(eng):   # a BF16 cache fed F32 keys: one rounding
    table = orc.to_bf16(orc.normal(0x6E2, 1, (16, 24)))
    values = orc.normal(0x6E2, 2, (3, 40))
    values[0, 8] = np.float32(1.00390625)            # a tie at the 8th mantissa bit: rounds to even
    it, iv = eng.upload_bf16(table, 16, 24), eng.upload(values, 3, 40)
    ii = _i32(eng, [[5, 0, 15]], 1, 3)
    eng.scatter_rows_into(it, ii, (iv, (0, 8), (3, 24)))
    want = table.copy()
    for n, r in enumerate((5, 0, 15)):
        want[r] = orc.to_bf16(values[n, 8:32])
    assert np.array_equal(eng.download_bf16(it), want)
    for i in (it, iv, ii):
        eng.free(i)


def test_scatter_rows_into_reports_a_row_outside_the_table(fresh_eng):
    e = fresh_eng
    it, iv = e.upload(np.zeros((4, 8), np.float32), 4, 8), e.upload(np.ones((1, 8), np.float32), 1, 8)
    ii = _i32(e, [[4]], 1, 1)
    e.scatter_rows_into(it, ii, (iv, (0, 0), (1, 8)))
    with pytest.raises(TtError) as err:
        e.sync()
    assert err.value.status == 6                     # DOMAIN, at the next wait


def test_reshape_is_a_view_of_the_same_words(eng):
    a = np.arange(48, dtype=np.float32).reshape(4, 12)
    ia = eng.upload(a, 4, 12)
    v, dims = eng.reshape(ia, 6, 8)
    assert dims == (6, 8) and np.array_equal(eng.download(v), a.reshape(6, 8))
    eng.free(ia)                                     # the view keeps the words alive
    assert np.array_equal(eng.download(v), a.reshape(6, 8))
    with pytest.raises(TtError):
        eng.reshape(v, 5, 8)
    eng.free(v)


def small_llama():
    return W.LlamaConfig(layers=3, hidden=576, heads=9, kv_heads=3, head_dim=64, ff=1536, vocab=2048)


def test_cached_steps_equal_the_prefill_of_the_same_tokens(eng):
    cfg = small_llama()
    batch, t = 2, 32
    w = W.llama_weights(cfg, seed=11)
    ids = orc.integers(0x6E1, 9, (batch, t), cfg.vocab)
    pre = W.LlamaPrefill(eng, cfg, w, batch, t)
    assert not pre.fused                             # 32 tokens: the composed attention
    ii = _i32(eng, ids.reshape(1, -1), 1, batch * t)
    la, aa = pre.forward(ii, all_positions=True)
    want = eng.download(la).reshape(batch, t, cfg.vocab)
    dec = W.LlamaDecode(eng, cfg, pre.w, batch, max_len=64)
    dec.reset(ids[:, 0])
    worst, seen = 0.0, []
    for step in range(t):
        dec.set_ids(ids[:, step])
        lg, am = dec.step()
        got = eng.download(lg)
        worst = max(worst, float(np.max(np.abs(got - want[:, step]))))
        seen.append(eng.download_bits(am).view(np.int32).ravel().copy())
        assert np.array_equal(seen[-1], got.argmax(1))
        eng.free(lg); eng.free(am)
    assert worst <= 2e-2, worst
    assert np.array_equal(dec.generated(0, t), np.stack(seen))   # every step's choice was recorded at its position
    # and the CPU restatement at the last position
    wb = {k: orc.from_bf16(orc.to_bf16(v)) for k, v in w.items()}
    cpu = M.llama_prefill(cfg, wb, ids.reshape(1, -1), batch, t)
    assert np.max(np.abs(got - cpu)) <= 2e-2
    for i in (ii, la, aa):
        eng.free(i)


def test_a_traced_generation_is_the_eager_one(eng):
    cfg = small_llama()
    batch, n = 2, 24
    pre = W.LlamaPrefill(eng, cfg, W.llama_weights(cfg, seed=11), batch, 32)
    first = np.array([5, 1999], np.int32)
    eager = W.LlamaDecode(eng, cfg, pre.w, batch, max_len=64)
    eager.reset(first)
    toks = []
    for _ in range(n):
        lg, am = eager.step()
        toks.append(eng.download_bits(am).view(np.int32).ravel().copy())
        eng.free(lg); eng.free(am)
    toks = np.stack(toks)
    assert np.array_equal(eager.generated(0, n), toks)
    traced = W.LlamaDecode(eng, cfg, pre.w, batch, max_len=64)
    traced.reset(first)
    lg, am = traced.capture()
    traced.reset(first)                              # the capture's own eager step wrote position 0
    l0 = eng.device_traffic().launches
    for _ in range(n):
        traced.replay()                              # nothing is read back between steps
    assert eng.device_traffic().launches - l0 >= n * 10 * cfg.layers
    assert np.array_equal(traced.generated(0, n), toks)
    assert np.array_equal(eng.download_bits(am).view(np.int32).ravel(), toks[-1])
    eng.release_trace(traced.trace)
    eng.free(lg); eng.free(am)


@pytest.mark.parametrize("t", [32, 128])
def test_a_prompt_prefilled_into_the_cache_continues_as_the_stepped_one(eng, t):
    # crates/tt-models/src/kv_cache.rs:231-241 (the first chunk write).  The prefill and the steps reach the same
    # rows through different kernels (tensor-core tiles against the few-row product, two attention kernels), so the
    # rows agree to BF16 rounding and the continued logits to the tolerance the cached steps are held to (2e-2).
    cfg = small_llama()
    batch, more, max_len = 2, 8, 160
    w = W.llama_weights(cfg, seed=11)
    ids = orc.integers(0x6E2, 9, (batch, t), cfg.vocab)
    pre = W.LlamaPrefill(eng, cfg, w, batch, t)
    assert pre.fused == (t == 128)                   # both attention forms write the cache
    stepped = W.LlamaDecode(eng, cfg, pre.w, batch, max_len=max_len)
    stepped.reset(ids[:, 0])
    for step in range(t):                            # the prompt fed a token a step
        stepped.set_ids(ids[:, step])
        lg, am = stepped.step()
        last_logits, choice = eng.download(lg), eng.download_bits(am).view(np.int32).ravel().copy()
        eng.free(lg); eng.free(am)
    filled = W.LlamaDecode(eng, cfg, pre.w, batch, max_len=max_len)
    ii = _i32(eng, ids.reshape(1, -1), 1, batch * t)
    lg, am = pre.forward(ii, cache=filled)
    for l in range(cfg.layers):                      # the prompt's rows are written, the rest is still zero
        for mine, theirs in ((filled.kc[l], stepped.kc[l]), (filled.vc[l], stepped.vc[l])):
            a = orc.from_bf16(eng.download_bf16(mine)).reshape(batch, max_len, -1)
            b = orc.from_bf16(eng.download_bf16(theirs)).reshape(batch, max_len, -1)
            assert not a[:, t:].any() and a[:, :t].any()
            assert np.max(np.abs(a[:, :t] - b[:, :t])) <= 2.0 ** -6 * np.abs(b).max(), l
    assert np.max(np.abs(eng.download(lg) - last_logits)) <= 2e-2
    filled.continue_from(am, t)
    assert eng.download_bits(filled.pos)[0, 0] == t and np.array_equal(eng.download_bits(filled.ids), eng.download_bits(am))
    eng.free(lg); eng.free(am); eng.free(ii)
    worst = 0.0
    for _ in range(more):
        filled.set_ids(choice); stepped.set_ids(choice)      # the same input for both, whatever a near-tie chose
        la, aa = filled.step()
        lb, ab = stepped.step()
        worst = max(worst, float(np.max(np.abs(eng.download(la) - eng.download(lb)))))
        choice = eng.download_bits(ab).view(np.int32).ravel().copy()
        for i in (la, aa, lb, ab):
            eng.free(i)
    assert worst <= 2e-2, worst
    assert np.array_equal(filled.generated(t, more).shape, (more, batch))


def test_a_prompt_prefilled_in_chunks_is_the_prompt_prefilled_at_once(eng):
    # crates/tt-models/src/kv_cache.rs:231-296: a later chunk writes its rows and attends to the cache up to each
    # token's own position; the cache and the last logits are those of one prefill of the whole prompt (BF16 rounding:
    # the chunk's projections run on other tile shapes than the whole prompt's)
    cfg = small_llama()
    batch, chunk, max_len = 2, 128, 384
    w = W.llama_weights(cfg, seed=11)
    ids = orc.integers(0x6E3, 9, (batch, 2 * chunk), cfg.vocab)
    whole = W.LlamaPrefill(eng, cfg, w, batch, 2 * chunk)
    part = W.LlamaPrefill(eng, cfg, w, batch, chunk)
    a, b = (W.LlamaDecode(eng, cfg, whole.w, batch, max_len=max_len) for _ in range(2))
    iw = _i32(eng, ids.reshape(1, -1), 1, batch * 2 * chunk)
    lw, aw = whole.forward(iw, cache=a)
    outs = []
    for k in range(2):
        ic = _i32(eng, ids[:, k * chunk:(k + 1) * chunk].reshape(1, -1), 1, batch * chunk)
        outs.append(part.forward(ic, cache=b, start=k * chunk))
        eng.free(ic)
    lc, ac = outs[-1]
    assert np.max(np.abs(eng.download(lc) - eng.download(lw))) <= 2e-2
    for l in range(cfg.layers):
        for mine, theirs in ((b.kc[l], a.kc[l]), (b.vc[l], a.vc[l])):
            x = orc.from_bf16(eng.download_bf16(mine)).reshape(batch, max_len, -1)
            y = orc.from_bf16(eng.download_bf16(theirs)).reshape(batch, max_len, -1)
            assert not x[:, 2 * chunk:].any() and np.max(np.abs(x - y)) <= 2.0 ** -6 * np.abs(y).max(), l
    with pytest.raises(ValueError):
        part.forward(iw, cache=b, start=64)
    b.continue_from(ac, 2 * chunk)
    lg, am = b.step()                                  # the generation goes on from the chunked prompt
    assert np.isfinite(eng.download(lg)).all()
    for i in (lw, aw, lg, am, iw) + tuple(x for o in outs for x in o):
        eng.free(i)


@pytest.mark.parametrize("batch", [1, 2, 4])
@pytest.mark.parametrize("storage", ["bf16", "bfp8"])
@pytest.mark.parametrize("form", ["cluster", "one", "grid"])
def test_the_one_launch_step_is_the_composed_step(eng, batch, storage, form, monkeypatch):
    # `decode_layers` (one launch for every layer of a step: as several thread-block clusters that share the heads and ff,
    # as one cluster, or as a cooperative grid: the switch is read at every call) against the step composed of the trait's ops:
    # the same steps and roundings, sums in another fixed order, so the two agree as two correct BF16 evaluations do
    # (see the tolerance below), the cache rows to one BF16 step, and the choices wherever the composed step's margin is
    # clear.  Both are fed the same tokens.  With BFP8 weights both read the same compressed matrices.
    monkeypatch.setenv("B200TT_DECODE", form)
    cfg = small_llama()
    max_len, steps = 128, 70                           # past position 64: a second chunk of cache positions is attended
    pre = W.LlamaPrefill(eng, cfg, W.llama_weights(cfg, seed=11), batch, 32)
    composed = W.LlamaDecode(eng, cfg, pre.w, batch, max_len=max_len, weight_storage=storage)
    fused = W.LlamaDecode(eng, cfg, pre.w, batch, max_len=max_len, fused=True, weight_storage=storage)
    ids = orc.integers(0x6E5, 3, (steps, batch), cfg.vocab)
    composed.reset(ids[0]); fused.reset(ids[0])
    l0 = eng.device_traffic().launches
    worst, total, disagreements = 0.0, 0.0, 0
    for t in range(steps):
        composed.set_ids(ids[t]); fused.set_ids(ids[t])
        la, aa = composed.step()
        before = eng.device_traffic().launches
        lb, ab = fused.step()
        fused_launches = eng.device_traffic().launches - before
        a, b = eng.download(la), eng.download(lb)
        worst = max(worst, float(np.max(np.abs(a - b))))
        total += float(np.mean(np.abs(a - b)))
        top2 = np.sort(a, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 4e-2
        ca, cb = eng.download_bits(aa).view(np.int32).ravel(), eng.download_bits(ab).view(np.int32).ravel()
        assert np.array_equal(ca[clear], cb[clear]), t
        disagreements += int((ca != cb).sum())
        for i in (la, aa, lb, ab):
            eng.free(i)
    # Each step rounds its activations to BF16 some dozen times; where the two orders of summation land on either side of
    # a rounding boundary the activation moves by one BF16 step and the logits by up to several thousandths, so the worst
    # element is held to the 2e-2 the cached steps are held to, and the typical one to a fraction of it
    assert worst <= 2e-2 and total / steps <= 1.5e-3, (worst, total / steps)
    assert fused_launches <= 12                        # embedding, cast, the layers, head, argmax, bookkeeping
    # "cluster16x3" (three clusters of sixteen blocks: this shape's nine heads over three key/value heads) / "cluster16" /
    # "grid"; BFP8 matrices take the several-cluster form (which decodes a chunk before it multiplies) or the grid form
    took = eng.last_decode_form()
    if form == "grid" or (form == "one" and storage == "bfp8"):
        assert took == "grid"
    elif form == "one":
        assert took in ("cluster16", "cluster8")
    else:
        assert took in ("cluster16x3", "cluster8x3")
    for l in range(cfg.layers):
        for mine, theirs in ((fused.kc[l], composed.kc[l]), (fused.vc[l], composed.vc[l])):
            x = orc.from_bf16(eng.download_bf16(mine)).reshape(batch, max_len, -1)
            y = orc.from_bf16(eng.download_bf16(theirs)).reshape(batch, max_len, -1)
            assert not x[:, steps:].any() and x[:, :steps].any()
            assert np.max(np.abs(x - y)) <= 2.0 ** -6 * np.abs(y).max(), l      # BF16 rounding, as between the prefill's rows and the steps'
    assert np.array_equal(fused.generated(0, steps).shape, (steps, batch))


@pytest.mark.parametrize("heads,kv_heads,ff,tp,batch,max_len", [
    (8, 4, 1024, 0, 2, 128),      # four clusters: two query heads on one key/value head each
    (8, 4, 1024, 2, 1, 128),      # two clusters: four query heads on two key/value heads each
    (4, 4, 768, 0, 4, 128),       # four clusters, a query head a key/value head
    (6, 2, 1024, 0, 2, 128),      # two clusters (neither 4 nor 3 divides): three query heads a key/value head
    (9, 3, 1536, 0, 3, 128),      # three sequences in a four-row step
    (9, 3, 1536, 0, 4, 1024),     # sixteen chunks of positions a head: four attention items a block, most of them past the step
    (8, 4, 1024, 2, 2, 512),      # two key/value heads a cluster over eight chunks: two items a block
])
def test_the_several_cluster_step_over_other_cuts(eng, heads, kv_heads, ff, tp, batch, max_len, monkeypatch):
    # The several-cluster form cuts the heads, the key/value heads and ff by the number of clusters: the cuts the
    # SmolLM2-135M shape does not reach (more than one key/value head a cluster, one query head a key/value head, two and
    # four clusters), against the composed step as above.
    monkeypatch.delenv("B200TT_DECODE", raising=False)
    if tp:
        monkeypatch.setenv("B200TT_DECODE_TP", str(tp))
    cfg = W.LlamaConfig(layers=2, hidden=heads * 64, heads=heads, kv_heads=kv_heads, head_dim=64, ff=ff, vocab=1024)
    steps = 70
    pre = W.LlamaPrefill(eng, cfg, W.llama_weights(cfg, seed=5), batch, 32)
    composed = W.LlamaDecode(eng, cfg, pre.w, batch, max_len=max_len)
    fused = W.LlamaDecode(eng, cfg, pre.w, batch, max_len=max_len, fused=True)
    ids = orc.integers(0x6E9, 4, (steps, batch), cfg.vocab)
    composed.reset(ids[0]); fused.reset(ids[0])
    worst, total = 0.0, 0.0
    for t in range(steps):
        composed.set_ids(ids[t]); fused.set_ids(ids[t])
        la, aa = composed.step()
        lb, ab = fused.step()
        a, b = eng.download(la), eng.download(lb)
        worst = max(worst, float(np.max(np.abs(a - b))))
        total += float(np.mean(np.abs(a - b)))
        top2 = np.sort(a, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 4e-2
        ca, cb = eng.download_bits(aa).view(np.int32).ravel(), eng.download_bits(ab).view(np.int32).ravel()
        assert np.array_equal(ca[clear], cb[clear]), t
        for i in (la, aa, lb, ab):
            eng.free(i)
    assert worst <= 2e-2 and total / steps <= 1.5e-3, (worst, total / steps)
    want = tp if tp else next(g for g in (4, 3, 2) if heads % g == 0 and kv_heads % g == 0 and ff % (64 * g) == 0)
    assert eng.last_decode_form() in (f"cluster16x{want}", f"cluster8x{want}")
    for l in range(cfg.layers):
        for mine, theirs in ((fused.kc[l], composed.kc[l]), (fused.vc[l], composed.vc[l])):
            x = orc.from_bf16(eng.download_bf16(mine)).reshape(batch, max_len, -1)
            y = orc.from_bf16(eng.download_bf16(theirs)).reshape(batch, max_len, -1)
            assert not x[:, steps:].any() and x[:, :steps].any()
            assert np.max(np.abs(x - y)) <= 2.0 ** -6 * np.abs(y).max(), l


def test_a_block_that_never_reports_runs_the_other_blocks_polls_out(monkeypatch):
    # The several-cluster step's blocks wait for one another's words in global memory, every wait bounded by the engine's
    # limit.  A test's hook keeps one block from ever storing its end-of-layer word (a flag that nothing sets): the polls
    # for it run out after the limit (here 2e6 cycles, a millisecond), the step reports TIMEOUT at the next wait instead
    # of hanging, every block still leaves (no copy in flight into its shared memory), and the context stays usable:
    # a new engine's step is the composed step's.
    from metalium_rs_b200 import CudaEngine
    cfg = small_llama()
    ids = np.array([7], np.int32)
    monkeypatch.delenv("B200TT_DECODE", raising=False)
    with CudaEngine(0, wait_limit_cycles=2_000_000) as e:
        pre = W.LlamaPrefill(e, cfg, W.llama_weights(cfg, seed=11), 1, 32)
        dec = W.LlamaDecode(e, cfg, pre.w, 1, max_len=64, fused=True)
        dec.reset(ids)
        lg, am = dec.step()                            # a whole step first: the form is the several-cluster one and it works
        e.sync()
        assert e.last_decode_form() in ("cluster16x3", "cluster8x3") and np.isfinite(e.download(lg)).all()
        monkeypatch.setenv("B200TT_DEBUG_DECODE_SKIP_DONE", "5")
        dec.step()
        with pytest.raises(TtError) as ei:
            e.sync()
        assert ei.value.status == 4 and ei.value.variant == "Timeout"
    monkeypatch.delenv("B200TT_DEBUG_DECODE_SKIP_DONE")
    with CudaEngine(0) as e:
        pre = W.LlamaPrefill(e, cfg, W.llama_weights(cfg, seed=11), 1, 32)
        composed = W.LlamaDecode(e, cfg, pre.w, 1, max_len=64)
        fused = W.LlamaDecode(e, cfg, pre.w, 1, max_len=64, fused=True)
        composed.reset(ids); fused.reset(ids)
        for _ in range(3):
            la, _a = composed.step()
            lb, _b = fused.step()
        assert np.max(np.abs(e.download(la) - e.download(lb))) <= 2e-2


def test_a_traced_one_launch_generation_is_its_eager_one(eng):
    cfg = small_llama()
    batch, n = 2, 24
    pre = W.LlamaPrefill(eng, cfg, W.llama_weights(cfg, seed=11), batch, 32)
    first = np.array([5, 1999], np.int32)
    eager = W.LlamaDecode(eng, cfg, pre.w, batch, max_len=64, fused=True)
    eager.reset(first)
    toks = []
    for _ in range(n):
        lg, am = eager.step()
        toks.append(eng.download_bits(am).view(np.int32).ravel().copy())
        eng.free(lg); eng.free(am)
    toks = np.stack(toks)
    traced = W.LlamaDecode(eng, cfg, pre.w, batch, max_len=64, fused=True)
    traced.reset(first)
    lg, am = traced.capture()
    traced.reset(first)
    l0 = eng.device_traffic().launches
    for _ in range(n):
        traced.replay()
    assert eng.device_traffic().launches - l0 <= n * 12
    assert np.array_equal(traced.generated(0, n), toks)    # the same kernel, the same fixed order of sums: the same bits
    eng.release_trace(traced.trace)
    eng.free(lg); eng.free(am)


def test_one_launch_steps_equal_the_prefill_and_the_cpu_restatement(eng):
    cfg = small_llama()
    batch, t = 2, 32
    w = W.llama_weights(cfg, seed=11)
    ids = orc.integers(0x6E1, 9, (batch, t), cfg.vocab)
    pre = W.LlamaPrefill(eng, cfg, w, batch, t)
    dec = W.LlamaDecode(eng, cfg, pre.w, batch, max_len=64, fused=True)
    dec.reset(ids[:, 0])
    for step in range(t):
        dec.set_ids(ids[:, step])
        lg, am = dec.step()
        got = eng.download(lg)
        eng.free(lg); eng.free(am)
    wb = {k: orc.from_bf16(orc.to_bf16(v)) for k, v in w.items()}
    cpu = M.llama_prefill(cfg, wb, ids.reshape(1, -1), batch, t)
    assert np.max(np.abs(got - cpu)) <= 2e-2


def test_the_one_launch_step_refuses_what_it_was_not_written_for(eng):
    cfg = W.LlamaConfig(layers=1, hidden=128, heads=2, kv_heads=1, head_dim=32, ff=128, vocab=256)
    pre = W.LlamaPrefill(eng, cfg, W.llama_weights(cfg, seed=3), 1, 32)
    dec = W.LlamaDecode(eng, cfg, pre.w, 1, max_len=64, fused=True)      # heads of 32 columns
    dec.reset(np.array([1], np.int32))
    with pytest.raises(TtError) as ei:
        dec.step()
    assert ei.value.status == 2 and "64" in str(ei.value)
