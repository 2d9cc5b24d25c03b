"""The callers of the hot path -- the MLP training step, the Llama-architecture prefill and
the attention products -- driven through the C ABI and checked against the CPU oracle with
the contract's tolerances: F32 within 1e-5 relative, labels/argmax exact, model logits within
2e-2 max-abs (BASELINE north star)."""
import numpy as np
import pytest

from metalium_rs_b200 import BF16, I32, workloads as W
from oracle import models as M
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def rel(got, want):
    scale = np.maximum(np.abs(want), 1e-3 * np.abs(want).max())
    return float(np.max(np.abs(got.astype(np.float64) - want.astype(np.float64)) / scale))


@pytest.mark.parametrize("fused", [True, False])
def test_mlp_training_step_matches_the_oracle(eng, fused):
    # config 1: x [64,784] ~ N(0,1), Linear 784->128, ReLU, Linear 128->10, labels uniform 0..9, SGD lr 0.01
    x = orc.normal(0xC0F1, 0, (64, 784))
    labels = orc.integers(0xC0F1, 5, (64, 1), 10)
    w1, b1, w2, b2 = M.mlp_init()
    want = M.mlp_step(x, labels, w1, b1, w2, b2)
    mlp = W.MlpStep(eng, w1, b1, w2, b2, lr=0.01, fused_add_relu=fused)
    ix, il = eng.upload(x, 64, 784), eng.upload_bits(labels.view(np.uint32), 64, 1, I32)
    t0 = eng.device_traffic()
    out = mlp.step(ix, il, 64, keep=True)
    loss = float(eng.download(out["loss"])[0, 0])
    t1 = eng.device_traffic()
    assert abs(loss - float(want["loss"])) <= 1e-5 * abs(float(want["loss"]))
    h_ref = np.maximum((M.mm(x, w1) + b1).astype(np.float32), 0)
    s_logits = np.abs(h_ref).astype(np.float64) @ np.abs(w2).astype(np.float64) + np.abs(b2)
    assert np.max(np.abs(eng.download(out["logits"]).astype(np.float64) - want["logits"]) / s_logits) <= 1e-5
    # weight gradients are products x^T g: held, like every product, to 1e-5 of S = |x|^T |g|
    h = h_ref
    g2 = eng.download(out["dz"]); g1 = eng.download(out["dpre"])
    for name, left, right in (("dw1", x, g1), ("dw2", h, g2)):
        s_norm = np.abs(left).T.astype(np.float64) @ np.abs(right).astype(np.float64)
        err = np.abs(eng.download(out[name]).astype(np.float64) - want[name].astype(np.float64))
        assert np.max(err / np.maximum(s_norm, 1e-30)) <= 1e-5, name
    # bias gradients are column sums: held to 1e-5 of the sum of magnitudes
    for name, gmat in (("db1", g1), ("db2", g2)):
        err = np.abs(eng.download(out[name]).ravel().astype(np.float64) - want[name])
        assert np.max(err / np.abs(gmat).astype(np.float64).sum(0)) <= 1e-5, name
    for name in ("w1", "w2"):
        assert np.max(np.abs(eng.download(getattr(mlp, name)) - want[name])) <= 1e-5 * np.abs(want[name]).max(), name
    for name in ("b1", "b2"):
        assert np.max(np.abs(eng.download(getattr(mlp, name)).ravel() - want[name])) <= 1e-5 * np.abs(want[name]).max(), name
    # the predicted classes are the oracle's
    assert np.array_equal(eng.download(out["logits"]).argmax(1), want["logits"].argmax(1))
    # steady state: one scalar comes back, nothing else moves (step12_mnist.rs:287-301)
    assert t1.bytes_d2h - t0.bytes_d2h == 4 and t1.bytes_h2d == t0.bytes_h2d
    # a second step from the updated weights still agrees (the update really landed on the device)
    want2 = M.mlp_step(x, labels, want["w1"], want["b1"], want["w2"], want["b2"])
    out2 = mlp.step(ix, il, 64)
    assert abs(float(eng.download(out2["loss"])[0, 0]) - float(want2["loss"])) <= 2e-5 * abs(float(want2["loss"]))
    assert float(want2["loss"]) < float(want["loss"])
    for k, v in out.items():
        eng.free(v)
    eng.free(out2["loss"])
    for i in (ix, il, mlp.w1, mlp.b1, mlp.w2, mlp.b2):
        eng.free(i)


def small_llama():
    return W.LlamaConfig(layers=3, hidden=576, heads=9, kv_heads=3, head_dim=64, ff=1536, vocab=2048)


def test_llama_prefill_of_a_prompt_that_is_not_whole_tiles(eng):
    # 200 tokens a sequence: the fused attention kernel masks its second tile's tail by index, where the reference pads
    # (crates/burn-tt/src/ops.rs:4838-4842); both forms against the restatement, and against each other
    cfg = small_llama()
    batch, seq = 2, 200
    w = W.llama_weights(cfg, seed=7)
    wb = {k: orc.from_bf16(orc.to_bf16(v)) for k, v in w.items()}
    ids = orc.integers(0xC0F4, 11, (1, batch * seq), cfg.vocab)
    want = M.llama_prefill(cfg, wb, ids, batch, seq)
    ii = eng.upload_bits(ids.view(np.uint32), 1, batch * seq, I32)
    got = {}
    for fused in (True, False):
        model = W.LlamaPrefill(eng, cfg, w, batch, seq, fused_attention=fused)
        assert model.fused == fused
        logits, am = model.forward(ii)
        got[fused] = eng.download(logits)
        assert np.max(np.abs(got[fused] - want)) <= 2e-2, fused
        eng.free(logits); eng.free(am)
    assert W.LlamaPrefill(eng, cfg, w, batch, seq).fused      # and it is the default from a tile of tokens up
    assert np.max(np.abs(got[True] - got[False])) <= 2e-2
    eng.free(ii)


@pytest.mark.parametrize("fused", [False, True])   # the composed attention (ops.rs:4825) and the one-kernel form
def test_llama_prefill_logits_and_argmax(eng, fused):
    # the SmolLM2-135M layer shape, fewer layers and a smaller vocabulary so the oracle runs in seconds
    cfg = small_llama()
    batch, seq = 2, 128
    w = W.llama_weights(cfg, seed=7)
    wb = {k: orc.from_bf16(orc.to_bf16(v)) for k, v in w.items()}   # the oracle sees the BF16 weights
    ids = orc.integers(0xC0F4, 9, (1, batch * seq), cfg.vocab)
    model = W.LlamaPrefill(eng, cfg, w, batch, seq, fused_attention=fused)
    assert model.fused == fused
    ii = eng.upload_bits(ids.view(np.uint32), 1, batch * seq, I32)
    logits, am = model.forward(ii)
    got = eng.download(logits)
    want = M.llama_prefill(cfg, wb, ids, batch, seq)
    assert got.shape == (batch, cfg.vocab)
    assert np.max(np.abs(got - want)) <= 2e-2
    got_am = eng.download_bits(am).view(np.int32).ravel()
    assert np.array_equal(got_am, got.argmax(1))          # the device's argmax is its logits' argmax
    top2 = np.sort(want, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 4e-2                 # where the oracle's margin exceeds twice the tolerance
    assert np.array_equal(got_am[clear], want.argmax(1)[clear])
    eng.free(logits); eng.free(am)
    # all positions: causality -- the logits at position t do not depend on later tokens
    la, aa = model.forward(ii, all_positions=True)
    full = eng.download(la)
    assert np.max(np.abs(full[[seq - 1, 2 * seq - 1]] - got)) <= 1e-5  # the head's product takes another tile path
    ids2 = ids.copy()
    ids2[0, seq - 1] = (ids2[0, seq - 1] + 1) % cfg.vocab    # change sequence 0's last token
    i2 = eng.upload_bits(ids2.view(np.uint32), 1, batch * seq, I32)
    lb, ab = model.forward(i2, all_positions=True)
    full2 = eng.download(lb)
    assert np.array_equal(full2[:seq - 1], full[:seq - 1]) and np.array_equal(full2[seq:], full[seq:])
    assert not np.array_equal(full2[seq - 1], full[seq - 1])
    for i in (la, aa, lb, ab, ii, i2):
        eng.free(i)


def test_the_fused_gate_up_product_leaves_the_prefill_s_bits_alone(eng):
    cfg = small_llama()
    batch, seq = 2, 128
    w = W.llama_weights(cfg, seed=7)
    ids = orc.integers(0xC0F4, 9, (1, batch * seq), cfg.vocab)
    ii = eng.upload_bits(ids.view(np.uint32), 1, batch * seq, I32)
    outs = []
    for fused in (False, True):
        model = W.LlamaPrefill(eng, cfg, w, batch, seq, fused_mlp=fused)
        assert model.fused_mlp == fused
        lg, am = model.forward(ii)
        outs.append(eng.download_bits(lg))
        eng.free(lg); eng.free(am)
    assert np.array_equal(outs[0], outs[1])
    eng.free(ii)


def test_attention_products_on_rank4_views(eng):
    # config 5's shape scaled down: [2,4,256,128] BF16 ~ N(0,1)
    bh, t, d = 8, 256, 128
    q, k, v = (orc.to_bf16(orc.normal(0xC0F5, i, (bh * t, d))) for i in (1, 2, 3))
    iq, ik, iv = (eng.upload_bf16(x, bh * t, d) for x in (q, k, v))
    o = W.attention_products(eng, iq, ik, iv, bh, t, d)
    got = orc.from_bf16(eng.download_bf16(o)).astype(np.float64)
    assert eng.last_matmul_path() == "tcgen05"
    for i in range(bh):
        r = slice(i * t, (i + 1) * t)
        want = M.attention_item(orc.from_bf16(q[r]), orc.from_bf16(k[r]), orc.from_bf16(v[r]))
        # P is rounded to BF16 before P V and O is BF16: 1e-2 relative to the row's scale
        assert np.max(np.abs(got[r] - want)) <= 1e-2 * np.max(np.abs(want)), i
    # the one-kernel form of the same attention
    of = W.attention_fused(eng, iq, ik, iv, bh, t, d)
    gotf = orc.from_bf16(eng.download_bf16(of)).astype(np.float64)
    for i in range(bh):
        r = slice(i * t, (i + 1) * t)
        want = M.attention_item(orc.from_bf16(q[r]), orc.from_bf16(k[r]), orc.from_bf16(v[r]))
        assert np.max(np.abs(gotf[r] - want)) <= 1e-2 * np.max(np.abs(want)), i
    for x in (iq, ik, iv, o, of):
        eng.free(x)


def test_traced_prefill_replays_the_eager_bits(eng):  # server.rs:591-660; trace.rs: replay == eager
    cfg = small_llama()
    batch, seq = 2, 128
    model = W.LlamaPrefill(eng, cfg, W.llama_weights(cfg, seed=7), batch, seq)
    ids = orc.integers(0xC0F4, 9, (1, batch * seq), cfg.vocab)
    ids2 = orc.integers(0xC0F4, 10, (1, batch * seq), cfg.vocab)
    ii = eng.upload_bits(ids.view(np.uint32), 1, batch * seq, I32)
    i2 = eng.upload_bits(ids2.view(np.uint32), 1, batch * seq, I32)
    lg, am = model.forward(ii)
    eager1 = eng.download_bits(lg); eng.free(lg); eng.free(am)
    lg, am = model.forward(i2)
    eager2 = eng.download_bits(lg); eng.free(lg); eng.free(am)
    tl, ta = model.capture(ii)
    l0 = eng.device_traffic().launches
    model.replay()
    per = eng.device_traffic().launches - l0
    assert per >= 6 * cfg.layers                      # the replay is counted as the kernels it runs (six a layer)
    assert np.array_equal(eng.download_bits(tl), eager1)
    eng.copy_into(i2, ii)                              # new ids into the captured input buffer
    model.replay()
    assert np.array_equal(eng.download_bits(tl), eager2)
    assert np.array_equal(eng.download_bits(ta).view(np.int32).ravel(), eager2.view(np.float32).argmax(1))
    # other work between replays does not disturb the trace's buffers
    junk = [eng.upload(np.ones((256, 256), np.float32), 256, 256) for _ in range(8)]
    for j in junk:
        eng.free(j)
    eng.copy_into(i2, ii); model.replay()
    assert np.array_equal(eng.download_bits(tl), eager2)
    eng.begin_trace()
    with pytest.raises(Exception):
        eng.sync()                                     # a wait inside a capture is refused
    eng.release_trace(eng.end_trace())
    eng.release_trace(model.trace)
    for i in (tl, ta, ii, i2):
        eng.free(i)


def test_traced_mlp_training_matches_eager_training(eng):
    x = orc.normal(0xC0F1, 0, (64, 784)); labels = orc.integers(0xC0F1, 5, (64, 1), 10)
    w = M.mlp_init()
    ix, il = eng.upload(x, 64, 784), eng.upload_bits(labels.view(np.uint32), 64, 1, I32)
    eager = W.MlpStep(eng, *w, in_place=True)
    want = []
    for _ in range(6):
        o = eager.step(ix, il, 64); want.append(eng.download_bits(o["loss"])[0, 0]); eng.free(o["loss"])
    traced = W.MlpStep(eng, *w, in_place=True)
    loss = traced.capture(ix, il, 64)
    got = []
    # the capture pass does not execute, so after capture() one step has run
    for _ in range(5):
        traced.replay(); got.append(eng.download_bits(loss)[0, 0])
    assert got == want[1:6]
    assert want[5].view(np.float32) < want[0].view(np.float32)
    eng.release_trace(traced.trace)
    for i in (ix, il, loss):
        eng.free(i)
