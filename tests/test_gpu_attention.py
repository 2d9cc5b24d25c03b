"""`attention_rows` (a decode step's attention as one op) through the C ABI against the composition
it stands for.  Contract and shapes: crates/tt-kernels/src/attention.rs:360-372 (the result row, the
[1, l] mask, F32 or BF16 keys and values), :156-171 (what is refused), and its caller
crates/burn-tt/src/ops.rs:4683-4760 (items from the batched plan, grouped-query heads sharing keys).
Tolerance: 1e-5 of the largest |V| entry (F32 products and a softmax; the same figure the
reference's composed attention is held to in step59)."""
import numpy as np
import pytest

from metalium_rs_b200 import BOOL, UNSUPPORTED, TtError
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _case(eng, heads, kv_heads, m, d, l, dv, bf16, masked_tail, seed, q_row0=0):
    rep = heads // kv_heads
    q = orc.normal(seed, 1, (q_row0 + heads * m, d))
    k = orc.normal(seed, 2, (kv_heads * l, d))
    v = orc.normal(seed, 3, (kv_heads * l, dv))
    mask = np.zeros(l, dtype=np.uint32)
    if masked_tail:
        mask[l - masked_tail:] = 1
    if bf16:
        kb, vb = orc.to_bf16(k), orc.to_bf16(v)
        k, v = orc.from_bf16(kb), orc.from_bf16(vb)
        ik, iv = eng.upload_bf16(kb, *k.shape), eng.upload_bf16(vb, *v.shape)
    else:
        ik, iv = eng.upload(k, *k.shape), eng.upload(v, *v.shape)
    iq = eng.upload(q, *q.shape)
    im = eng.upload_bits(mask, 1, l, BOOL)
    items = [((q_row0 + h * m, 0), ((h // rep) * l, 0), ((h // rep) * l, 0)) for h in range(heads)]
    scale = 1.0 / np.sqrt(d)
    out, dims = eng.attention_rows([iq, ik, iv, im], items, [m, d, l, dv], scale)
    assert dims == (1, heads * m * dv)
    got = eng.download(out)
    want = orc.attention_rows(q, k, v, mask, items, [m, d, l, dv], scale)
    for i in (iq, ik, iv, im, out):
        eng.free(i)
    return got, want, np.abs(v).max()


@pytest.mark.parametrize("heads,kv_heads,m,d,l,dv,bf16,tail", [
    (9, 3, 1, 64, 512, 64, False, 0),        # SmolLM2-shaped decode step, grouped-query heads
    (9, 3, 1, 64, 512, 64, True, 100),       # a BF16 KV cache, the unwritten tail masked
    (2, 2, 1, 128, 8192, 128, True, 1000),   # few heads, long context: positions split over blocks
    (32, 8, 1, 128, 2048, 128, False, 48),
    (4, 4, 8, 64, 1024, 64, False, 0),       # several rows a head
    (3, 1, 32, 32, 320, 96, True, 7),        # a full tile of rows, odd tile counts
    (600, 600, 2, 32, 64, 32, False, 0),     # many heads: one block each
    (1, 1, 5, 160, 2048, 32, False, 1),      # d above 128: more than one pass of a key
])
def test_attention_rows_matches_the_composition(eng, heads, kv_heads, m, d, l, dv, bf16, tail):
    got, want, vmax = _case(eng, heads, kv_heads, m, d, l, dv, bf16, tail, 0xA77)
    assert got.shape == want.shape
    assert np.all(np.abs(got - want) <= 1e-5 * vmax + 1e-7), float(np.abs(got - want).max())


def test_attention_rows_as_rounds_the_result_once(eng):   # the trait's `_as` convention (server.rs:446-463)
    heads, m, d, l = 6, 2, 64, 1024
    q = orc.normal(0xA7C, 1, (heads * m, d))
    kb, vb = orc.to_bf16(orc.normal(0xA7C, 2, (2 * l, d))), orc.to_bf16(orc.normal(0xA7C, 3, (2 * l, d)))
    iq, ik, iv = eng.upload(q, *q.shape), eng.upload_bf16(kb, 2 * l, d), eng.upload_bf16(vb, 2 * l, d)
    im = eng.upload_bits(np.zeros(l, np.uint32), 1, l, BOOL)
    items = [((h * m, 0), ((h // 3) * l, 0), ((h // 3) * l, 0)) for h in range(heads)]
    full, _ = eng.attention_rows([iq, ik, iv, im], items, [m, d, l, d], 0.125)
    cast, _ = eng.cast_float(full, True)
    narrow, dims = eng.attention_rows_as([iq, ik, iv, im], items, [m, d, l, d], 0.125, True)
    assert dims == (1, heads * m * d)
    assert np.array_equal(eng.download_bf16(narrow), eng.download_bf16(cast))
    for i in (iq, ik, iv, im, full, cast, narrow):
        eng.free(i)


def test_query_rows_may_start_anywhere_in_their_buffer(eng):  # attention.rs:146-149 (`r0`)
    got, want, vmax = _case(eng, 4, 2, 3, 64, 256, 64, False, 0, 0xA78, q_row0=13)
    assert np.all(np.abs(got - want) <= 1e-5 * vmax + 1e-7)


def test_a_fully_masked_head_gives_zeros(eng):  # the clamps of sfpu/softmax.rs:37-43
    got, want, _ = _case(eng, 2, 2, 2, 32, 64, 32, False, 64, 0xA79)
    assert np.array_equal(got, np.zeros_like(got)) and np.array_equal(want, np.zeros_like(want))
    got, want, _ = _case(eng, 1, 1, 1, 64, 4096, 64, True, 4096, 0xA7A)   # split positions, every block masked
    assert np.array_equal(got, np.zeros_like(got))


def test_key_and_value_blocks_inside_wider_buffers(eng):
    m, d, l, dv = 2, 32, 96, 32
    q = orc.normal(0xA7B, 1, (m, d))
    kv = orc.normal(0xA7B, 2, (l, 3 * d + dv + 4))        # K at column 32, V at column 100
    mask = np.zeros(l, dtype=np.uint32)
    iq, ikv, im = eng.upload(q, m, d), eng.upload(kv, *kv.shape), eng.upload_bits(mask, 1, l, BOOL)
    items = [((0, 0), (0, 32), (0, 100))]
    out, _ = eng.attention_rows([iq, ikv, ikv, im], items, [m, d, l, dv], 0.25)
    got = eng.download(out)
    want = orc.attention_rows(q, kv, kv, mask, items, [m, d, l, dv], 0.25)
    assert np.all(np.abs(got - want) <= 1e-5 * np.abs(kv).max())
    for i in (iq, ikv, im, out):
        eng.free(i)


@pytest.mark.parametrize("dims,why", [
    ([33, 64, 64, 64], "more than a tile of rows"),
    ([0, 64, 64, 64], "no rows"),
    ([1, 48, 64, 64], "d is not whole tiles"),
    ([1, 64, 80, 64], "l is not whole tiles"),
    ([1, 64, 64, 16], "dv is not whole tiles"),
])
def test_shapes_the_reference_refuses_are_refused(eng, dims, why):  # attention.rs:156-171
    m, d, l, dv = dims
    iq = eng.upload(np.zeros((max(m, 1), d), np.float32), max(m, 1), d)
    ik = eng.upload(np.zeros((l, d), np.float32), l, d)
    iv = eng.upload(np.zeros((l, dv), np.float32), l, dv)
    im = eng.upload_bits(np.zeros(l, np.uint32), 1, l, BOOL)
    with pytest.raises(TtError) as err:
        eng.attention_rows([iq, ik, iv, im], [((0, 0), (0, 0), (0, 0))], dims, 1.0)
    assert err.value.status == UNSUPPORTED, why
    for i in (iq, ik, iv, im):
        eng.free(i)


def test_wrong_operands_are_refused(eng):  # attention.rs:386-415
    m, d, l, dv = 1, 32, 64, 32
    iq = eng.upload(np.zeros((m, d), np.float32), m, d)
    ik = eng.upload(np.zeros((l, d), np.float32), l, d)
    iv = eng.upload(np.zeros((l, dv), np.float32), l, dv)
    ivb = eng.upload_bf16(np.zeros((l, dv), np.uint16), l, dv)
    im = eng.upload_bits(np.zeros(l, np.uint32), 1, l, BOOL)
    im_short = eng.upload_bits(np.zeros(32, np.uint32), 1, 32, BOOL)
    one = [((0, 0), (0, 0), (0, 0))]
    for buffers, items in (([iq, ik, ivb, im], one),        # keys F32, values BF16
                           ([iq, ik, iv, im_short], one),   # a mask for other positions
                           ([iq, ik, iv, iq], one),         # the mask is not Bool
                           ([iq, ik, iv, im], []),          # no heads
                           ([iq, ik, iv, im], [((0, 0), (32, 0), (0, 0))])):   # keys past the buffer
        with pytest.raises(TtError) as err:
            eng.attention_rows(buffers, items, [m, d, l, dv], 1.0)
        assert err.value.status == UNSUPPORTED
    for i in (iq, ik, iv, ivb, im, im_short):
        eng.free(i)
