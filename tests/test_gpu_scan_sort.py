"""`scan` and `sort_planes` through the C ABI against the oracle's restatement of the reference's scalar
models: crates/tt-kernels/src/sfpu/scan.rs:196-231 (every column from its first row, from the op's
identity; test inputs follow scan.rs's own tests: signed zeros, NaNs of both signs, infinities, ties) and
crates/tt-kernels/src/sfpu/sort.rs:1-66 (the stable order on (key, index), planes layout :198).  Bit for bit,
except that an arithmetic NaN's payload is not compared (the reference's NaN canonicalisation is its
mover's, crates/tt-kernels/src/sfpu/ops.rs:3910-3915)."""
import numpy as np
import pytest

from metalium_rs_b200 import F32, I32, UNSUPPORTED, TtError
from metalium_rs_b200 import engine as E
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

SCAN_CODE = {name: i for i, name in enumerate(orc.SCAN_OPS)}
SPECIAL = np.array([0x00000000, 0x80000000, 0x7F800000, 0xFF800000, 0x7FC00000, 0xFFC00001, 0x7F800001, 0x3F800000,
                    0xBF800000, 0x00000001, 0x80000001, 0x7F7FFFFF], dtype=np.uint32)


def _same(got, want, arithmetic):
    if not arithmetic:
        return np.array_equal(got, want)
    g, w = got.view(np.float32), want.view(np.float32)
    return bool(np.all((got == want) | (np.isnan(g) & np.isnan(w))))


def _scan_input(op, rows, cols, seed):
    if op.startswith("i"):
        if op == "iprod":
            x = orc.integers(seed, 1, (rows, cols), 7).astype(np.int64) - 3
            return x.astype(np.int32).view(np.uint32)
        return (orc.splitmix64(seed, 1, rows * cols) >> np.uint64(32)).astype(np.uint32).reshape(rows, cols)
    if op == "prod":
        x = orc.uniform(seed, 1, (rows, cols), 0.7, 1.4)
        x[orc.integers(seed, 2, (rows, cols), 5) == 0] *= -1
        return x.view(np.uint32)
    x = orc.uniform(seed, 1, (rows, cols), -4.0, 4.0).view(np.uint32).copy()
    if op != "sum":
        x = np.round(x.view(np.float32)).view(np.uint32).copy()      # ties, and both zeros after rounding
    sel = orc.integers(seed, 3, (rows, cols), 9) == 0
    x[sel] = SPECIAL[orc.integers(seed, 4, (rows, cols), len(SPECIAL))[sel]]
    return x


@pytest.mark.parametrize("op", orc.SCAN_OPS)
@pytest.mark.parametrize("rows,cols", [(1, 1), (33, 70), (257, 1000), (5000, 3), (2048, 40000), (70000, 40)])
def test_scan_matches_the_row_order_model(eng, op, rows, cols):
    if rows * cols > 3_000_000 and op not in ("sum", "min_nan", "isum"):
        pytest.skip("the large shapes run for one op of each family")
    x = _scan_input(op, rows, cols, 0x5CA0 + rows)
    elem = I32 if op.startswith("i") else F32
    a = eng.upload_bits(x, rows, cols, elem)
    out, dims = eng.scan(a, SCAN_CODE[op])
    assert dims == (rows, cols)
    got = eng.download_bits(out)
    want = orc.scan(x, op)
    assert _same(got.reshape(rows, cols), want, op in ("sum", "prod"))
    eng.free(a); eng.free(out)


def test_a_sum_scan_starts_from_plus_zero(eng):   # scan.rs:196: the fold starts at +0.0, so a leading -0 becomes +0
    x = np.array([[0x80000000, 0x80000000], [0x80000000, 0x3F800000]], dtype=np.uint32)
    a = eng.upload_bits(x, 2, 2, F32)
    out, _ = eng.scan(a, E.SCAN_SUM)
    assert np.array_equal(eng.download_bits(out).reshape(2, 2), np.array([[0, 0], [0, 0x3F800000]], dtype=np.uint32))
    p, _ = eng.scan(a, E.SCAN_PROD)                # 1.0 * -0 = -0; -0 * -0 = +0
    assert np.array_equal(eng.download_bits(p).reshape(2, 2), np.array([[0x80000000, 0x80000000], [0, 0x80000000]], dtype=np.uint32))
    for i in (a, out, p):
        eng.free(i)


def test_scan_refuses_the_wrong_element_type(eng):   # scan.rs:44-49
    a = eng.upload(np.zeros((4, 4), np.float32), 4, 4)
    with pytest.raises(TtError) as err:
        eng.scan(a, E.SCAN_ISUM)
    assert err.value.status == UNSUPPORTED
    with pytest.raises(TtError):
        eng.scan(a, 10)
    eng.free(a)


def _sort_case(eng, problems, n, is_i32, descending, indices, seed):
    if is_i32:
        v = (orc.splitmix64(seed, 1, problems * n) >> np.uint64(32)).astype(np.uint32).reshape(problems, n)
        v[:, ::3] &= np.uint32(7)                                          # many ties
    else:
        v = np.round(orc.uniform(seed, 1, (problems, n), -6.0, 6.0)).view(np.uint32).copy()
        sel = orc.integers(seed, 2, (problems, n), 6) == 0
        v[sel] = SPECIAL[orc.integers(seed, 3, (problems, n), len(SPECIAL))[sel]]
    planes = orc.to_planes(v, fill=0x12345678)
    elem = I32 if is_i32 else F32
    a = eng.upload_bits(planes, *planes.shape, elem)
    (keys, dims), idx = eng.sort_planes(a, elem, n, descending, indices)
    assert dims == planes.shape
    want_k, want_i = orc.sort_rows(v, is_i32, descending)
    got_k = orc.from_planes(eng.download_bits(keys).reshape(dims), problems, n)
    assert np.array_equal(got_k, want_k)
    eng.free(keys)
    if indices:
        got_i = orc.from_planes(eng.download_bits(idx[0]).reshape(dims), problems, n)
        assert np.array_equal(got_i.view(np.int32), want_i)
        eng.free(idx[0])
    eng.free(a)


@pytest.mark.parametrize("n", [1, 2, 31, 32, 33, 100, 512, 1000, 1024])
@pytest.mark.parametrize("is_i32,descending", [(False, False), (False, True), (True, False), (True, True)])
def test_sort_planes_is_the_stable_order(eng, n, is_i32, descending):
    _sort_case(eng, 37 if n > 64 else 70, n, is_i32, descending, True, 0x50 + n)


def test_sort_without_indices_and_many_problems(eng):
    _sort_case(eng, 600, 96, False, False, False, 0x51)


def test_an_element_equal_to_the_sentinel_is_still_returned(eng):   # sort.rs:47-52
    v = np.full((3, 40), 0x7FFFFFFF, dtype=np.uint32)
    v[:, ::2] = 0x3F800000
    planes = orc.to_planes(v, fill=0)
    a = eng.upload_bits(planes, *planes.shape, F32)
    (keys, dims), idx = eng.sort_planes(a, F32, 40, False, True)
    got_i = orc.from_planes(eng.download_bits(idx[0]).reshape(dims), 3, 40).view(np.int32)
    assert np.array_equal(got_i, orc.sort_rows(v, False, False)[1]) and got_i.max() == 39
    for i in (a, keys, idx[0]):
        eng.free(i)


@pytest.mark.parametrize("rows,cols,elem,n", [(32, 32, F32, 0), (64, 32, F32, 1025), (32, 32, F32, 33), (64, 40, F32, 40),
                                              (32, 32, I32, 8)])
def test_what_a_sort_refuses(eng, rows, cols, elem, n):   # sort.rs:132-146, 705-713
    a = eng.upload(np.zeros((rows, cols), np.float32), rows, cols)
    with pytest.raises(TtError) as err:
        eng.sort_planes(a, elem, n, False, False)
    assert err.value.status == UNSUPPORTED
    eng.free(a)
