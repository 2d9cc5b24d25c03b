"""Fused attention over whole sequences (`b200_attention_blocks`) against an F64 restatement of the
composition burn-tt runs (crates/burn-tt/src/ops.rs:4825-4960: batched Q K^T, scale and causal mask
fill, row softmax, batched P V).  Shapes: the SmolLM2-shaped prefill's heads (grouped-query, Q, K and V
side by side in one projection buffer) and the [2048, 128] heads of the attention-shaped workload.
Tolerance: BF16 steps -- the probabilities and the result are each rounded once to 8 bits -- so
|got - want| <= 2^-7 * sum_j p_j |v_j| + 2^-9 |want| + 1e-6."""
import numpy as np
import pytest

from metalium_rs_b200 import UNSUPPORTED, TtError
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


_want = orc.attention_blocks


def _check(got, want, bound_s):
    err = np.abs(got.astype(np.float64) - want)
    lim = 2.0 ** -7 * bound_s + 2.0 ** -9 * np.abs(want) + 1e-6
    assert np.all(err <= lim), (float(err.max()), float((err / lim).max()))


@pytest.mark.parametrize("batch,heads,kv_heads,s,d,causal", [
    (2, 9, 3, 512, 64, True),      # the prefill's attention: 9 query heads on 3 key/value heads
    (1, 2, 2, 256, 128, False),
    (1, 4, 1, 384, 128, True),
    (3, 1, 1, 128, 64, False),     # one tile
])
def test_heads_side_by_side_in_one_projection_buffer(eng, batch, heads, kv_heads, s, d, causal):
    width = (heads + 2 * kv_heads) * d
    x = orc.to_bf16(orc.normal(0xF1A, 1, (batch * s, width), 1.5))
    xf = orc.from_bf16(x)
    ix = eng.upload_bf16(x, batch * s, width)
    rep = heads // kv_heads
    items = []
    for b in range(batch):
        for h in range(heads):
            kvh = h // rep
            items.append(((b * s, h * d), (b * s, (heads + kvh) * d), (b * s, (heads + kv_heads + kvh) * d), (b * s, h * d)))
    scale = 1.0 / np.sqrt(d)
    out, dims = eng.attention_blocks(ix, ix, ix, items, [s, d, s, d], scale, causal, [batch * s, heads * d])
    assert dims == (batch * s, heads * d)
    got = orc.from_bf16(eng.download_bf16(out))
    for (qa, ka, va, oa) in items:
        want, bound = _want(xf[qa[0]:qa[0] + s, qa[1]:qa[1] + d], xf[ka[0]:ka[0] + s, ka[1]:ka[1] + d],
                            xf[va[0]:va[0] + s, va[1]:va[1] + d], scale, causal)
        _check(got[oa[0]:oa[0] + s, oa[1]:oa[1] + d], want, bound)
    eng.free(ix); eng.free(out)


def test_more_keys_than_queries_and_future_keys_are_not_seen(eng):
    sq, sk, d = 128, 384, 64
    q = orc.to_bf16(orc.normal(0xF1B, 1, (sq, d)))
    k = orc.to_bf16(orc.normal(0xF1B, 2, (sk, d)))
    v = orc.to_bf16(orc.normal(0xF1B, 3, (sk, d)))
    qf, kf, vf = orc.from_bf16(q), orc.from_bf16(k), orc.from_bf16(v)
    iq, ik, iv = eng.upload_bf16(q, sq, d), eng.upload_bf16(k, sk, d), eng.upload_bf16(v, sk, d)
    item = [((0, 0), (0, 0), (0, 0), (0, 0))]
    out, _ = eng.attention_blocks(iq, ik, iv, item, [sq, d, sk, d], 0.2, True, [sq, d])
    want, bound = _want(qf, kf, vf, 0.2, True)
    _check(orc.from_bf16(eng.download_bf16(out)), want, bound)
    eng.free(out)
    # the last key is seen by the last query alone: make it dominate and look at who moved
    k2 = kf.copy(); k2[-1] = 40.0 * np.sign(qf[-1])
    v2 = vf.copy(); v2[-1] = 100.0
    ik2, iv2 = eng.upload_bf16(orc.to_bf16(k2), sk, d), eng.upload_bf16(orc.to_bf16(v2), sk, d)
    out2, _ = eng.attention_blocks(iq, ik2, iv2, item, [sq, d, sk, d], 0.2, True, [sq, d])
    got2 = orc.from_bf16(eng.download_bf16(out2))
    want2, bound2 = _want(qf, orc.from_bf16(orc.to_bf16(k2)), orc.from_bf16(orc.to_bf16(v2)), 0.2, True)
    _check(got2, want2, bound2)
    assert np.all(np.abs(got2[:-1]) < 10.0) and np.all(got2[-1] > 90.0)
    for i in (iq, ik, iv, ik2, iv2, out2):
        eng.free(i)


@pytest.mark.parametrize("blocks,sq,sk,d,causal", [
    (3, 100, 100, 64, True),       # a prompt of 100 tokens: one partial tile
    (2, 500, 500, 64, True),       # the 500-token prompt of ops.rs:4838's padding: three whole tiles and a tail
    (2, 77, 333, 128, False),      # ragged on both sides
    (2, 129, 257, 64, True),       # one row and one key past a tile
    (1, 1, 1, 64, False), (1, 200, 129, 128, False),
])
def test_heads_whose_lengths_are_not_whole_tiles(eng, blocks, sq, sk, d, causal):
    # the blocks lie one after another in their buffers, so a tail tile reads the next block's rows (the last block's
    # tail reads past the buffer): none of that may reach a result, and rows past sq must not be written
    q = orc.to_bf16(orc.normal(0xF1D, 1, (blocks * sq, d), 1.5))
    k = orc.to_bf16(orc.normal(0xF1D, 2, (blocks * sk, d), 1.5))
    v = orc.to_bf16(orc.normal(0xF1D, 3, (blocks * sk, d), 1.5))
    qf, kf, vf = orc.from_bf16(q), orc.from_bf16(k), orc.from_bf16(v)
    iq, ik, iv = eng.upload_bf16(q, blocks * sq, d), eng.upload_bf16(k, blocks * sk, d), eng.upload_bf16(v, blocks * sk, d)
    pad = 64                                           # rows of the result no block covers: they stay zero
    items = [((b * sq, 0), (b * sk, 0), (b * sk, 0), (b * (sq + pad), 0)) for b in range(blocks)]
    scale = 1.0 / np.sqrt(d)
    out, dims = eng.attention_blocks(iq, ik, iv, items, [sq, d, sk, d], scale, causal, [blocks * (sq + pad), d])
    got = orc.from_bf16(eng.download_bf16(out))
    for b in range(blocks):
        want, bound = _want(qf[b * sq:(b + 1) * sq], kf[b * sk:(b + 1) * sk], vf[b * sk:(b + 1) * sk], scale, causal)
        r0 = b * (sq + pad)
        _check(got[r0:r0 + sq], want, bound)
        assert not got[r0 + sq:r0 + sq + pad].any(), b    # a partial query tile wrote nothing past its block
    for i in (iq, ik, iv, out):
        eng.free(i)


@pytest.mark.parametrize("d,causal", [(64, False), (128, False), (64, True)])
def test_scores_that_keep_growing_along_the_keys(eng, d, causal):
    # The kernel walks the keys once with a running reference that it moves -- rescaling the accumulated result and the
    # sum -- only when a tile's scores exceed it by 2^8.  Random scores move it in the first tiles only; here the scores
    # of a row grow steadily with the key's position (to ~170 in log2 units: some twenty moves, in every tile for the
    # steepest rows), and shrink again in the second block, where the reference must stay.
    sq, sk = 256, 1024
    rng = np.random.default_rng(0xF1E)
    e = np.full(d, 1.0 / np.sqrt(d))
    steep = rng.uniform(0.05, 1.5, (sq, 1))
    q = orc.to_bf16((np.sqrt(d) * steep * e + 0.05 * rng.standard_normal((sq, d))).astype(np.float32))
    ramp = np.linspace(0.0, 1.0, sk)[:, None]
    k_up = (80.0 * ramp * e + 0.05 * rng.standard_normal((sk, d))).astype(np.float32)
    k_down = (80.0 * (1.0 - ramp) * e + 0.05 * rng.standard_normal((sk, d))).astype(np.float32)
    k = orc.to_bf16(np.concatenate([k_up, k_down]))
    v = orc.to_bf16(orc.normal(0xF1E, 3, (2 * sk, d)))
    qf, kf, vf = orc.from_bf16(q), orc.from_bf16(k), orc.from_bf16(v)
    iq, ik, iv = eng.upload_bf16(q, sq, d), eng.upload_bf16(k, 2 * sk, d), eng.upload_bf16(v, 2 * sk, d)
    items = [((0, 0), (0, 0), (0, 0), (0, 0)), ((0, 0), (sk, 0), (sk, 0), (sq, 0))]
    scale = 1.0 / np.sqrt(d)
    out, _ = eng.attention_blocks(iq, ik, iv, items, [sq, d, sk, d], scale, causal, [2 * sq, d])
    got = orc.from_bf16(eng.download_bf16(out))
    for b in range(2):
        want, bound = _want(qf, kf[b * sk:(b + 1) * sk], vf[b * sk:(b + 1) * sk], scale, causal)
        _check(got[b * sq:(b + 1) * sq], want, bound)
    for i in (iq, ik, iv, out):
        eng.free(i)


def test_uncovered_result_elements_are_zero(eng):
    s, d = 128, 64
    x = orc.to_bf16(orc.normal(0xF1C, 1, (s, 3 * d)))
    ix = eng.upload_bf16(x, s, 3 * d)
    out, dims = eng.attention_blocks(ix, ix, ix, [((0, 0), (0, d), (0, 2 * d), (128, 64))], [s, d, s, d], 0.125, False, [384, 192])
    got = eng.download_bf16(out)
    assert dims == (384, 192)
    covered = np.zeros((384, 192), bool); covered[128:256, 64:128] = True
    assert np.all(got[~covered] == 0) and np.any(got[covered] != 0)
    eng.free(ix); eng.free(out)


@pytest.mark.parametrize("dims,scale,causal", [
    ([128, 32, 128, 32], 1.0, False), ([128, 64, 128, 128], 1.0, False), ([0, 64, 128, 64], 1.0, False),
    ([256, 64, 128, 64], 1.0, True), ([128, 64, 128, 64], 0.0, False),
])
def test_shapes_outside_the_kernel_are_refused(eng, dims, scale, causal):
    sq, d, sk, dv = dims
    iq = eng.upload_bf16(np.zeros((256, 128), np.uint16), 256, 128)
    with pytest.raises(TtError) as err:
        eng.attention_blocks(iq, iq, iq, [((0, 0), (0, 0), (0, 0), (0, 0))], dims, scale, causal, [256, 128])
    assert err.value.status == UNSUPPORTED
    eng.free(iq)
