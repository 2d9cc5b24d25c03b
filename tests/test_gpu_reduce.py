"""Reductions, full sums, softmax, RMS norm and argmax through the C ABI against the oracle.
Shapes and claims follow crates/tt-tests/tests/step31_reduce.rs:85, step63_burn_full_reduce.rs:126,
step32_burn_softmax.rs:47, step230_softmax_rows.rs:123 and step211_argmax_row.rs:78."""
import numpy as np
import pytest

from metalium_rs_b200 import (ALL, ANY, BF16, BITOR, BOOL, COLS, F32, I32, MAX, MAX_I32, MIN_I32, PROD, PROD_I32, ROWS, SUM,
                              SUM_I32, TtError, kinds)
from oracle import oracle as orc
from tests import helpers as H

pytestmark = pytest.mark.gpu

SHAPES = [(1, 1), (1, 70), (37, 70), (64, 10), (64, 128), (33, 2048), (5, 4100), (300, 1), (8193, 3)]


@pytest.mark.parametrize("shape", SHAPES)
def test_sum_over_rows_is_the_left_fold_bit_for_bit(eng, shape):  # sfpu/reduce.rs:1162-1193
    a = orc.normal(0x5E, 1, shape)
    if shape[1] > 5:
        a[:, 5] = -0.0
    ia = eng.upload(a, *shape)
    out, dims = eng.reduce(ia, SUM, ROWS)
    assert dims == (1, shape[1])
    assert np.array_equal(eng.download_bits(out), orc.sum_rows_in_order(a).view(np.uint32))
    o2, _ = eng.sum_rows(ia)
    assert np.array_equal(eng.download_bits(o2), eng.download_bits(out))
    for i in (ia, out, o2):
        eng.free(i)


@pytest.mark.parametrize("shape", SHAPES)
def test_sum_over_columns_within_the_reference_bound(eng, shape):  # step31_reduce.rs header: 2(n-1)u sum|x|
    a = orc.normal(0x5E, 2, shape)
    ia = eng.upload(a, *shape)
    out, dims = eng.reduce(ia, SUM, COLS)
    assert dims == (shape[0], 1)
    got = eng.download(out).astype(np.float64)
    truth = a.astype(np.float64).sum(1, keepdims=True)
    assert np.all(np.abs(got - truth) <= orc.sum_bound(a, axis=1))
    # the same call twice gives the same bits: the tree is fixed
    o2, _ = eng.reduce(ia, SUM, COLS)
    assert np.array_equal(eng.download_bits(o2), eng.download_bits(out))
    for i in (ia, out, o2):
        eng.free(i)


@pytest.mark.parametrize("axis", [ROWS, COLS])
@pytest.mark.parametrize("shape", [(37, 70), (64, 128), (5, 4100)])
def test_exact_folds(eng, shape, axis):
    a = orc.normal(0x5E, 3, shape)
    a[1, 3] = np.nan if shape[1] > 3 else a[1, 0]
    ia = eng.upload(a, *shape)
    out, _ = eng.reduce(ia, MAX, axis)
    assert np.array_equal(eng.download_bits(out), orc.reduce(a, "MAX", axis))
    eng.free(out)
    ints = (orc.splitmix64(0x5E, 4, a.size) >> np.uint64(40)).astype(np.int64).astype(np.int32).reshape(shape) - (1 << 22)
    ii = eng.upload_bits(ints.view(np.uint32), *shape, I32)
    for op, name in ((SUM_I32, "SUM_I32"), (PROD_I32, "PROD_I32"), (MIN_I32, "MIN_I32"), (MAX_I32, "MAX_I32"), (BITOR, "BITOR")):
        out, _ = eng.reduce(ii, op, axis)
        assert np.array_equal(eng.download_bits(out), orc.reduce(ints, name, axis)), name
        eng.free(out)
    bools = (ints & 1).astype(np.uint32)
    ib = eng.upload_bits(bools, *shape, BOOL)
    for op, name in ((ALL, "ALL"), (ANY, "ANY")):
        out, _ = eng.reduce(ib, op, axis)
        assert np.array_equal(eng.download_bits(out), orc.reduce(bools, name, axis)), name
        eng.free(out)
    small = orc.uniform(0x5E, 5, shape, 0.9, 1.1)
    ip = eng.upload(small, *shape)
    out, _ = eng.reduce(ip, PROD, axis)
    want = small.astype(np.float64).prod(axis=axis, keepdims=True)
    assert np.all(np.abs(eng.download(out) - want) <= 1e-5 * np.abs(want))
    for i in (ia, ii, ib, ip, out):
        eng.free(i)


def test_reduce_then_applies_an_exact_kind(eng):  # tensor.rs:6038: a softmax's clamped maximum
    a = np.full((4, 64), -np.inf, dtype=np.float32)
    a[0, 3] = 2.0
    ia = eng.upload(a, 4, 64)
    fmax = np.array([-np.finfo(np.float32).max], dtype=np.float32).view(np.uint32)[0]
    out, _ = eng.reduce(ia, MAX, COLS, (kinds.CLAMP_MIN, int(fmax)))
    got = eng.download(out).ravel()
    assert got[0] == 2.0 and np.all(got[1:] == -np.finfo(np.float32).max)
    with pytest.raises(TtError):
        eng.reduce(ia, MAX, COLS, (kinds.EXP, 0))  # not an exact unary kind
    eng.free(ia); eng.free(out)


@pytest.mark.parametrize("shape", [(1, 1), (1, 70), (37, 70), (64, 10), (15, 70), (20, 7), (37, 8193), (8193, 1)])
def test_full_sum_and_mean_shapes(eng, shape):  # step63_burn_full_reduce.rs:16-20,126-138
    v = H.full_sum_values(shape[0] * shape[1]).reshape(shape)
    ia = eng.upload(v, *shape)
    for mean in (False, True):
        out, dims = eng.full_sum(ia, mean)
        assert dims == (1, 1)
        got = float(eng.download(out)[0, 0])
        truth, bound = orc.full_sum(v, mean)
        exact = v.astype(np.float64).mean() if mean else v.astype(np.float64).sum()
        assert abs(got - exact) <= bound, (shape, mean, got, exact, bound)
        eng.free(out)
    assert abs(eng.full_reduce(v, shape, False) - v.astype(np.float64).sum()) <= orc.full_sum(v)[1]
    eng.free(ia)


@pytest.mark.parametrize("value", [-0.0, np.finfo(np.float32).tiny / 2, np.inf, -np.inf, np.nan])
def test_full_sum_special_values(eng, value):  # step63_burn_full_reduce.rs:142-165
    v = np.full((37, 70), value, dtype=np.float32)
    ia = eng.upload(v, 37, 70)
    out, _ = eng.full_sum(ia, False)
    got = float(eng.download(out)[0, 0])
    want = float(np.float32(np.float64(value) * 37 * 70))
    assert (np.isnan(got) and np.isnan(want)) or got == want or abs(got - want) <= 1e-6 * abs(want)
    eng.free(ia); eng.free(out)


def test_full_sum_is_the_same_bits_twice(eng):
    v = orc.uniform(0x5F, 1, (2048, 4096), -4, 4)
    ia = eng.upload(v, 2048, 4096)
    a, _ = eng.full_sum(ia)
    b, _ = eng.full_sum(ia)
    assert np.array_equal(eng.download_bits(a), eng.download_bits(b))
    truth, bound = orc.full_sum(v)
    assert abs(float(eng.download(a)[0, 0]) - v.astype(np.float64).sum()) <= bound
    for i in (ia, a, b):
        eng.free(i)


@pytest.mark.parametrize("shape", [(256, 10), (70, 120), (40, 400), (64, 10), (5, 7), (16, 2048), (8, 4096), (3, 32768), (2, 40000), (9, 1000), (6, 8196), (4, 65536), (2, 70000), (5, 12288), (3, 131072), (2, 140000)])
def test_softmax_rows_within_the_reference_bound(eng, shape):  # step32_burn_softmax.rs:51,94-95
    x = orc.uniform(0x50, 1, shape, -4, 4)
    ix = eng.upload(x, *shape)
    out, dims = eng.softmax_rows(ix, None, 1.0)
    assert dims == shape
    got = eng.download(out).astype(np.float64)
    x64 = x.astype(np.float64)
    e = np.exp(x64 - x64.max(1, keepdims=True))
    want = e / e.sum(1, keepdims=True)
    assert np.max(np.abs(got - want) / want) <= orc.softmax_bound(shape[1])
    assert np.max(np.abs(got - orc.softmax_rows(x)) / want) <= orc.softmax_bound(shape[1])
    lo, _ = eng.log_softmax_rows(ix)
    assert np.max(np.abs(eng.download(lo) - np.log(want))) <= 2e-6 * np.log(shape[1]) + 1e-5
    for i in (ix, out, lo):
        eng.free(i)


def test_softmax_scale_mask_and_a_fully_masked_row(eng):  # step230_softmax_rows.rs header
    shape = (64, 256)
    x = orc.uniform(0x50, 2, shape, -4, 4)
    mask = np.zeros((32, 256), dtype=np.uint32)  # read for rows r % 32 (server.rs:428)
    mask[1, :] = 1
    mask[2, ::2] = 1
    mask[5, 200:] = 1
    ix, im = eng.upload(x, *shape), eng.upload_bits(mask, 32, 256, BOOL)
    out, _ = eng.softmax_rows(ix, im, 0.125)
    got = eng.download(out)
    want = orc.softmax_rows(x, mask, 0.125)
    assert np.all(got[1] == 0) and np.all(got[33] == 0)
    live = want > 0
    assert np.array_equal(got == 0, ~live)
    assert np.max(np.abs(got[live] - want[live]) / want[live]) <= orc.softmax_bound(256)
    for i in (ix, im, out):
        eng.free(i)


def test_softmax_propagates_nan_rows_only(eng):
    x = orc.uniform(0x50, 3, (4, 512), -4, 4)
    x[2, 100] = np.nan
    ix = eng.upload(x, 4, 512)
    out, _ = eng.softmax_rows(ix, None, 1.0)
    got = eng.download(out)
    assert np.isnan(got[2]).all() and not np.isnan(got[[0, 1, 3]]).any()
    eng.free(ix); eng.free(out)


@pytest.mark.parametrize("shape", [(1, 576), (33, 576), (4096, 576), (7, 70), (2, 4097)])
def test_rms_and_rms_norm(eng, shape):  # sfpu/norm.rs:1-25
    x = orc.normal(0x52, 1, shape)
    gamma = orc.uniform(0x52, 2, (1, shape[1]), 0.5, 1.5)
    ix, ig = eng.upload(x, *shape), eng.upload(gamma, 1, shape[1])
    st, dims = eng.rms(ix, 1e-5)
    assert dims == (shape[0], 1)
    want = orc.rms(x, 1e-5)
    assert np.max(np.abs(eng.download(st) - want) / want) <= 1e-6
    n, _ = eng.rms_norm(ix, ig, 1e-5)
    wn = orc.rms_norm(x, gamma, 1e-5)
    assert np.max(np.abs(eng.download(n) - wn)) <= 1e-5 * np.max(np.abs(wn))
    nb, _ = eng.rms_norm_as(ix, ig, 1e-5, True)
    got_b = orc.from_bf16(eng.download_bf16(nb))
    assert np.max(np.abs(got_b - wn)) <= 2 ** -8 * np.max(np.abs(wn))
    # bit for bit the F32 norm narrowed (session.rs:8692-8695)
    assert np.array_equal(eng.download_bf16(nb), orc.to_bf16(eng.download(n)))
    for i in (ix, ig, st, n, nb):
        eng.free(i)


def test_add_rms_norm_returns_the_sum_and_its_norm(eng):  # server.rs:466
    a, b = orc.normal(0x52, 3, (65, 576)), orc.normal(0x52, 4, (65, 576))
    gamma = orc.uniform(0x52, 5, (1, 576), 0.5, 1.5)
    ia, ib, ig = eng.upload(a, 65, 576), eng.upload(b, 65, 576), eng.upload(gamma, 1, 576)
    (s, d1), (n, d2) = eng.add_rms_norm(ia, ib, ig, 1e-5)
    assert d1 == d2 == (65, 576)
    ssum = (a + b).astype(np.float32)
    assert np.array_equal(eng.download(s), ssum)
    wn = orc.rms_norm(ssum, gamma, 1e-5)
    assert np.max(np.abs(eng.download(n) - wn)) <= 1e-5 * np.max(np.abs(wn))
    for i in (ia, ib, ig, s, n):
        eng.free(i)


@pytest.mark.parametrize("shape", [(65, 576), (7, 70), (33, 2052)])   # the register kernel, ragged columns, wide rows
def test_add_rms_norm_as_is_the_composition_bit_for_bit(eng, shape):  # server.rs:446-463: norm, then cast_float
    a, b = orc.normal(0x54, 3, shape), orc.normal(0x54, 4, shape)
    gamma = orc.uniform(0x54, 5, (1, shape[1]), 0.5, 1.5)
    ia, ib, ig = eng.upload(a, *shape), eng.upload(b, *shape), eng.upload(gamma, 1, shape[1])
    (s0, _), (n0, _) = eng.add_rms_norm(ia, ib, ig, 1e-5)
    (s1, _), (n1, d1) = eng.add_rms_norm_as(ia, ib, ig, 1e-5, True)
    assert d1 == shape and eng.dims_of(n1) == (shape, BF16) and eng.dims_of(s1) == (shape, F32)
    assert np.array_equal(eng.download_bits(s1), eng.download_bits(s0))
    assert np.array_equal(eng.download(s1), (a + b).astype(np.float32))
    cast, _ = eng.cast_float(n0, True)
    assert np.array_equal(eng.download_bf16(n1), eng.download_bf16(cast))
    # and the two-op form: ADD, then rms_norm_as
    for i in (ia, ib, ig, s0, n0, s1, n1, cast):
        eng.free(i)


@pytest.mark.parametrize("n", [32, 33, 100, 1024, 3000, 4096, 49152, 65601])
def test_argmax_row_cases(eng, n):  # step211_argmax_row.rs:42-110
    for what, v in H.argmax_cases(n):
        for vec in (v, -v):
            ia = eng.upload(vec.reshape(1, n), 1, n)
            out, dims = eng.argmax_row(ia)
            assert dims == (1, 1)
            assert int(eng.download_bits(out).view(np.int32)[0, 0]) == H.host_argmax(vec), (n, what)
            eng.free(ia); eng.free(out)


def test_argmax_many_rows_and_the_moved_maximum(eng):  # step211_argmax_row.rs:112-124
    a = orc.normal(0x53, 1, (8, 49152))
    ia = eng.upload(a, 8, 49152)
    out, dims = eng.argmax_row(ia)
    assert dims == (8, 1)
    assert np.array_equal(eng.download_bits(out).view(np.int32), orc.argmax_rows(a))
    v = H.lcg_row(13, 4096)
    first = H.host_argmax(v)
    v[first] -= 100.0
    iv = eng.upload(v.reshape(1, -1), 1, 4096)
    o2, _ = eng.argmax_row(iv)
    assert int(eng.download_bits(o2)[0, 0]) == H.host_argmax(v) != first
    for i in (ia, out, iv, o2):
        eng.free(i)


def test_softmax_rows_as_bf16_is_the_f32_result_narrowed(eng):  # the `_as` pattern: one rounding, no F32 written
    for shape in [(64, 512), (16, 2048), (4, 8192), (3, 12288), (5, 100)]:
        x = orc.uniform(0x50, 7, shape, -4, 4)
        mask = (orc.integers(0x50, 8, (shape[0], shape[1]), 4) == 0).astype(np.uint32)
        ix, im = eng.upload(x, *shape), eng.upload_bits(mask, *shape, BOOL)
        f, _ = eng.softmax_rows(ix, im, 0.5)
        b, dims = eng.softmax_rows_as(ix, im, 0.5, True)
        assert dims == shape
        assert np.array_equal(eng.download_bf16(b), orc.to_bf16(eng.download(f))), shape
        for i in (ix, im, f, b):
            eng.free(i)
