"""Indexing and copies move bits (crates/tt-tests/tests/step61_burn_gather.rs:111,128;
crates/burn-tt/src/server.rs:269-379,482)."""
import numpy as np
import pytest

from metalium_rs_b200 import BF16, F32, I32, TtError
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def special_table(rows, cols, seed):
    t = orc.normal(seed, 1, (rows, cols))
    bits = t.view(np.uint32)
    bits[0, 0] = 0x80000000      # -0.0 survives a gather (the GPU moves bits; burn-flex's answer)
    bits[1, min(1, cols - 1)] = 0x7FC0BEEF      # a NaN payload
    bits[2, min(2, cols - 1)] = 0x00000001      # a denormal
    return t


@pytest.mark.parametrize("cols", [576, 70, 1])
def test_select_rows_is_an_embedding_lookup_bit_for_bit(eng, cols):
    table = special_table(1000, cols, 0x61)
    idx = orc.integers(0x61, 2, (1, 257), 1000)
    idx[0, :3] = [0, 1, 2]
    it, ii = eng.upload(table, 1000, cols), eng.upload_bits(idx.view(np.uint32), 1, 257, I32)
    out, dims = eng.select_rows(it, ii)
    assert dims == (257, cols)
    assert np.array_equal(eng.download_bits(out), orc.select_rows(table, idx).view(np.uint32))
    for i in (it, ii, out):
        eng.free(i)


def test_select_rows_of_a_bf16_table(eng):
    table = orc.to_bf16(orc.normal(0x61, 3, (512, 576), 0.02))
    idx = orc.integers(0x61, 4, (1, 100), 512)
    it, ii = eng.upload_bf16(table, 512, 576), eng.upload_bits(idx.view(np.uint32), 1, 100, I32)
    out, dims = eng.select_rows(it, ii)
    assert np.array_equal(eng.download_bf16(out), table[idx.ravel()])
    for i in (it, ii, out):
        eng.free(i)


def test_an_index_outside_the_table_is_a_domain_error(fresh_eng):
    e = fresh_eng
    it = e.upload(np.zeros((10, 8), np.float32), 10, 8)
    ii = e.upload_bits(np.array([[1, 10]], dtype=np.int32).view(np.uint32), 1, 2, I32)
    out, _ = e.select_rows(it, ii)
    with pytest.raises(TtError) as ei:
        e.sync()
    assert "DOMAIN" in str(ei.value)


def test_pick_columns_and_its_backward(eng):  # burn-tt/src/ops.rs:1001,1043
    x = special_table(64, 10, 0x62)
    idx = orc.integers(0x62, 2, (64, 1), 10)
    idx[0, 0], idx[1, 0], idx[2, 0] = 0, 1, 2
    g = orc.normal(0x62, 3, (64, 1))
    ix, ii, ig = eng.upload(x, 64, 10), eng.upload_bits(idx.view(np.uint32), 64, 1, I32), eng.upload(g, 64, 1)
    out, dims = eng.pick_columns(ix, ii)
    assert dims == (64, 1)
    assert np.array_equal(eng.download_bits(out), orc.pick_columns(x, idx).view(np.uint32))
    z, _ = eng.zeros_dram((64, 10))
    sc, _ = eng.scatter_add_columns(z, ii, ig)
    assert np.array_equal(eng.download_bits(sc), orc.scatter_add_columns(np.zeros((64, 10), np.float32), idx, g).view(np.uint32))
    sc2, _ = eng.scatter_add_columns(ix, ii, ig)
    got2, want2 = eng.download_bits(sc2), orc.scatter_add_columns(x, idx, g).view(np.uint32)
    both_nan = np.isnan(got2.view(np.float32)) & np.isnan(want2.view(np.float32))  # NaN + g: the payload is the adder's
    assert np.array_equal(got2[~both_nan], want2[~both_nan])
    gi, _ = eng.gather_indexed(ix, ii)
    assert np.array_equal(eng.download_bits(gi), eng.download_bits(out))
    for i in (ix, ii, ig, out, z, sc, sc2, gi):
        eng.free(i)


def test_select_add_rows_adds_duplicates_in_index_order(eng):  # server.rs:358; step61_burn_gather.rs
    t = orc.normal(0x63, 1, (50, 96))
    idx = np.array([[3, 7, 3, 3, 49, 0, 7]], dtype=np.int32)
    v = orc.uniform(0x63, 2, (7, 96), -1e3, 1e3)
    it, ii, iv = eng.upload(t, 50, 96), eng.upload_bits(idx.view(np.uint32), 1, 7, I32), eng.upload(v, 7, 96)
    out, dims = eng.select_add_rows(it, ii, iv)
    want = orc.select_add_rows(t, idx, v)
    assert np.array_equal(eng.download_bits(out), want.view(np.uint32))
    o2, _ = eng.rows_add(it, [3, 7, 3, 3, 49, 0, 7], iv)
    assert np.array_equal(eng.download_bits(o2), want.view(np.uint32))
    assert np.array_equal(eng.download(it), t)  # the input is untouched
    for i in (it, ii, iv, out, o2):
        eng.free(i)


def test_scatter_assign_gather_and_slice_rows(eng):
    t = orc.normal(0x64, 1, (40, 33))
    v = orc.normal(0x64, 2, (5, 33))
    idx = np.array([[4, 9, 4, 0, 39]], dtype=np.int32)
    it, iv, ii = eng.upload(t, 40, 33), eng.upload(v, 5, 33), eng.upload_bits(idx.view(np.uint32), 1, 5, I32)
    out, _ = eng.scatter_rows(it, ii, iv, False)
    assert np.array_equal(eng.download(out), orc.scatter_rows(t, idx, v))
    ic = eng.upload_bits(idx.reshape(5, 1).view(np.uint32), 5, 1, I32)
    o2, _ = eng.scatter_rows(it, ic, iv, True)
    assert np.array_equal(eng.download(o2), orc.scatter_rows(t, idx, v))
    a, _ = eng.assign_rows(it, iv, [(1, 0), (2, 4), (1, 3)])
    want = t.copy(); want[1] = v[0]; want[2] = v[4]; want[1] = v[3]
    assert np.array_equal(eng.download(a), want)
    g, dims = eng.gather_rows([it, iv], [(0, 5), (1, 2), (0, 39), (1, 0)], 33)
    assert dims == (4, 33)
    assert np.array_equal(eng.download(g), np.stack([t[5], v[2], t[39], v[0]]))
    s, dims = eng.slice_rows(it, 8, 16)
    assert dims == (16, 33) and np.array_equal(eng.download(s), t[8:24])
    # the parent may be freed first: the view keeps it alive (server.rs:480-481)
    eng.free(it)
    assert np.array_equal(eng.download(s), t[8:24])
    with pytest.raises(TtError):
        eng.download(it)
    for i in (iv, ii, ic, out, o2, a, g, s):
        eng.free(i)


def test_copy_blocks_splits_and_merges_heads(eng):  # tensor.rs:6659-6680: a head's columns into its own rows
    t, heads, hd = 64, 3, 32
    x = orc.normal(0x65, 1, (t, heads * hd))
    ix = eng.upload(x, t, heads * hd)
    moves = [((0, h * hd), (h * t, 0), (t, hd), False) for h in range(heads)]
    out, dims = eng.copy_blocks(ix, moves, (heads * t, hd))
    assert dims == (heads * t, hd)
    want = x.reshape(t, heads, hd).transpose(1, 0, 2).reshape(heads * t, hd)
    assert np.array_equal(eng.download(out), want)
    # transposed blocks: K^T per head
    mt = [((h * t, 0), (h * hd, 0), (hd, t), True) for h in range(heads)]
    tr, dims = eng.copy_blocks(out, mt, (heads * hd, t))
    assert np.array_equal(eng.download(tr), want.reshape(heads, t, hd).transpose(0, 2, 1).reshape(heads * hd, t))
    with pytest.raises(TtError):
        eng.copy_blocks(ix, moves[:2], (heads * t, hd))  # does not cover the output
    xb = orc.to_bf16(x)
    ib = eng.upload_bf16(xb, t, heads * hd)
    ob, _ = eng.copy_blocks(ib, moves, (heads * t, hd))
    assert np.array_equal(eng.download_bf16(ob), xb.reshape(t, heads, hd).transpose(1, 0, 2).reshape(heads * t, hd))
    for i in (ix, out, tr, ib, ob):
        eng.free(i)


def test_repack_takes_one_source_per_output_element(eng):  # tensor.rs:654-658
    x = orc.normal(0x66, 1, (17, 23))
    ix = eng.upload(x, 17, 23)
    rr, cc = np.meshgrid(np.arange(23), np.arange(17), indexing="ij")  # the transpose
    src = np.stack([cc.ravel(), rr.ravel()], axis=1)
    out, dims = eng.repack(ix, src, (23, 17))
    assert dims == (23, 17) and np.array_equal(eng.download(out), x.T)
    eng.free(ix); eng.free(out)
