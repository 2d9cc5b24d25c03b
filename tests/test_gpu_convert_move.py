"""`cast_block`, `cast_f16`, `repack_many`, `select_taps`, `pow`, `metadata` and `gddr_free_bytes` through the
C ABI.  Every one but `pow` moves or converts bits, so the comparisons are exact: the casts against the
oracle's restatement of crates/tt-kernels/src/fp16.rs:172-176, 271-275 (itself checked against IEEE binary16
on the CPU side) and of the BF16 rule; the movers against plain indexing (crates/tt-kernels/src/tensor.rs:6791,
crates/tt-kernels/src/index.rs:136-160)."""
import numpy as np
import pytest

from metalium_rs_b200 import F32, I32, UNSUPPORTED, TtError, kinds
from oracle import oracle as orc

DOMAIN_STATUS = 6

pytestmark = pytest.mark.gpu


def test_cast_f16_on_every_binary16_pattern_and_back(eng):
    h = np.arange(65536, dtype=np.uint32).astype(np.uint16).reshape(256, 256)
    a = eng.upload_bf16(h, 256, 256)                       # FP16 lives in two-byte storage (server.rs:2189-2200)
    wide, dims = eng.cast_f16(a, False)
    assert dims == (256, 256)
    w = eng.download_bits(wide)
    assert np.array_equal(w, orc.f32_bits_from_f16_bits(h))
    back, _ = eng.cast_f16(wide, True)
    b = eng.download_bf16(back)
    quiet = np.where((h & 0x7FFF) > 0x7C00, h | 0x0200, h)   # a signalling NaN comes back quiet
    assert np.array_equal(b.reshape(256, 256), quiet)
    for i in (a, wide, back):
        eng.free(i)


def test_cast_f16_rounds_ties_to_even_everywhere(eng):
    edge = np.array([0, 0x80000000, 0x33000000, 0x33000001, 0x337FFFFF, 0x33800000, 0x387FE000, 0x387FDFFF, 0x387FFFFF,
                     0x38800000, 0x38801000, 0x38803000, 0x477FEFFF, 0x477FF000, 0x47800000, 0x7F800000, 0xFF800000,
                     0x7F800001, 0xFFC12345, 0x7FFFFFFF, 0x00000001, 0x807FFFFF], dtype=np.uint32)
    rnd = (orc.splitmix64(0xF16, 1, 1 << 20) >> np.uint64(32)).astype(np.uint32)
    near = (orc.uniform(0xF16, 2, (1 << 18,), -70000.0, 70000.0)).view(np.uint32)
    tiny = (orc.uniform(0xF16, 3, (1 << 18,), -1.3e-4, 1.3e-4)).view(np.uint32)
    x = np.concatenate([edge, rnd, near, tiny])
    x = np.resize(x, (x.size + 7) // 8 * 8).reshape(-1, 8)
    a = eng.upload_bits(x, *x.shape, F32)
    out, _ = eng.cast_f16(a, True)
    got = eng.download_bf16(out).reshape(x.shape)
    assert np.array_equal(got, orc.f16_bits_from_f32_bits(x))
    eng.free(a); eng.free(out)


def test_cast_f16_refuses_the_wrong_storage(eng):
    a = eng.upload(np.zeros((2, 2), np.float32), 2, 2)
    with pytest.raises(TtError) as err:
        eng.cast_f16(a, False)
    assert err.value.status == UNSUPPORTED
    eng.free(a)


@pytest.mark.parametrize("at,dims", [((0, 0), (70, 100)), ((32, 64), (33, 31)), ((5, 3), (1, 1)), ((0, 96), (70, 4))])
def test_cast_block_is_the_cast_of_those_elements(eng, at, dims):   # session.rs:3727-3731
    x = orc.normal(0xCB, 1, (70, 100))
    x.view(np.uint32)[3, 5] = 0x7F800001
    a = eng.upload(x, 70, 100)
    out, od = eng.cast_block((a, at, dims), True)
    assert od == dims
    blk = x[at[0]:at[0] + dims[0], at[1]:at[1] + dims[1]]
    assert np.array_equal(eng.download_bf16(out).reshape(dims), orc.to_bf16(blk))
    whole, _ = eng.cast_float(a, True)
    back, bd = eng.cast_block((whole, at, dims), False)
    assert bd == dims and np.array_equal(eng.download_bits(back).reshape(dims), orc.to_bf16(blk).astype(np.uint32) << 16)
    with pytest.raises(TtError) as err:
        eng.cast_block((a, (60, 0), (11, 4)), True)
    assert err.value.status == UNSUPPORTED
    for i in (a, out, whole, back):
        eng.free(i)


@pytest.mark.parametrize("bf16", [False, True])
def test_repack_many_gathers_from_several_buffers(eng, bf16):
    shapes = [(37, 70), (1, 5), (64, 64)]
    if bf16:
        mats = [orc.to_bf16(orc.normal(0xAE, i, s)) for i, s in enumerate(shapes)]
        ids = [eng.upload_bf16(m, *m.shape) for m in mats]
    else:
        mats = [orc.normal(0xAE, i, s).view(np.uint32) for i, s in enumerate(shapes)]
        ids = [eng.upload_bits(m, *m.shape, F32) for m in mats]
    dims = (45, 33)
    n = dims[0] * dims[1]
    which = orc.integers(0xAE, 9, (n,), 3)
    sources = [(int(s), (int(orc.integers(0xAE, 10 + i, (1,), shapes[s][0])[0]), int(orc.integers(0xAE, 5000 + i, (1,), shapes[s][1])[0])))
               for i, s in enumerate(which)]
    out, od = eng.repack_many(ids, sources, dims)
    assert od == dims
    got = (eng.download_bf16(out) if bf16 else eng.download_bits(out)).reshape(dims)
    assert np.array_equal(got, orc.repack_many(mats, sources, dims))
    with pytest.raises(TtError) as err:
        eng.repack_many(ids, [(1, (1, 0))], (1, 1))
    assert err.value.status == DOMAIN_STATUS
    with pytest.raises(TtError) as err:
        eng.repack_many(ids, [(0, (0, 0))] * 3, (1, 2))      # tensor.rs:6803 the count must be the result's
    assert err.value.status == UNSUPPORTED
    for i in ids + [out]:
        eng.free(i)


@pytest.mark.parametrize("rows,cols,taps,n,zero_row,bf16", [(50, 24, 9, 200, True, False), (64, 32, 3, 77, True, True),
                                                           (10, 70, 1, 5, False, False), (33, 5, 4, 1000, False, True),
                                                           (4096, 64, 9, 4096, True, True)])
def test_select_taps_is_an_im2col(eng, rows, cols, taps, n, zero_row, bf16):
    table = orc.normal(0x7A, 1, (rows, cols))
    idx = orc.integers(0x7A, 2, (taps, n), rows + (1 if zero_row else 0)).astype(np.int32)
    if bf16:
        tb = orc.to_bf16(table)
        t = eng.upload_bf16(tb, rows, cols)
    else:
        tb = table.view(np.uint32)
        t = eng.upload(table, rows, cols)
    i = eng.upload_bits(idx, taps, n, I32)
    out, dims = eng.select_taps(t, i, zero_row)
    want = orc.select_taps(tb, idx, zero_row)
    assert dims == want.shape
    got = (eng.download_bf16(out) if bf16 else eng.download_bits(out)).reshape(dims)
    assert np.array_equal(got, want)
    for b in (t, i, out):
        eng.free(b)


def test_select_taps_past_the_table_is_a_domain_error(fresh_eng):
    eng = fresh_eng
    t = eng.upload(np.ones((8, 8), np.float32), 8, 8)
    i = eng.upload_bits(np.array([[0, 8]], np.int32), 1, 2, I32)
    out, _ = eng.select_taps(t, i, False)          # 8 is the zero row only when asked for
    with pytest.raises(TtError) as err:
        eng.sync()
    assert err.value.status == DOMAIN_STATUS


def test_pow_is_the_three_eltwise_kinds(eng):   # session.rs:7734-7755
    x = orc.uniform(0xB0, 1, (33, 70), 0.1, 3.0)
    y = orc.uniform(0xB0, 2, (33, 70), -2.0, 2.0)
    yi = (orc.integers(0xB0, 3, (33, 70), 7).astype(np.int32) - 3)
    ix, iy, ii = eng.upload(x, 33, 70), eng.upload(y, 33, 70), eng.upload_bits(yi, 33, 70, I32)
    for arg, kind_name, b, s in ((("tensor", iy), "POW", iy, 0.0), (("scalar", 1.5), "POW_S", 0, 1.5), (("int", ii), "POW_I", ii, 0.0)):
        got, dims = eng.pow(ix, arg)
        ref, _ = eng.eltwise_op((getattr(kinds, kind_name), s, 0.0), ix, b or None)
        assert dims == (33, 70) and np.array_equal(eng.download_bits(got), eng.download_bits(ref))
        eng.free(got); eng.free(ref)
    small = eng.upload(y[:3], 3, 70)
    with pytest.raises(TtError) as err:
        eng.pow(ix, ("tensor", small))
    assert err.value.status == UNSUPPORTED
    with pytest.raises(TtError):
        eng.pow(ix, ("int", iy))
    for i in (ix, iy, ii, small):
        eng.free(i)


def test_metadata_is_resident_words_and_free_bytes_follow_the_pool(eng):
    words = np.arange(24, dtype=np.uint32).reshape(3, 8)
    m = eng.metadata(words, (3, 8), I32)
    assert np.array_equal(eng.download_bits(m), words)
    largest, total = eng.gddr_free_bytes()
    assert 0 < largest <= total
    big = eng.upload(np.zeros((4096, 4096), np.float32), 4096, 4096)
    _, after = eng.gddr_free_bytes()
    assert after <= total - 4096 * 4096 * 4 + (64 << 20)
    eng.free(big)
    _, again = eng.gddr_free_bytes()
    assert again >= after + 4096 * 4096 * 4 - (1 << 20)
    eng.free(m)


@pytest.mark.parametrize("h,w,k,stride", [(8, 8, 2, 2), (30, 41, 3, 1), (64, 64, 5, 3), (12, 12, 7, 1)])
def test_pool_bf16_is_a_window_mean(eng, h, w, k, stride):   # crates/tt-kernels/src/fpu.rs:39-132
    x = orc.to_bf16(orc.normal(0xB001, 1, (h, w)))
    oh, ow = (h - k) // stride + 1, (w - k) // stride + 1
    windows = [[[i * stride + di, j * stride + dj] for di in range(k) for dj in range(k)] for i in range(oh) for j in range(ow)]
    windows[0] = windows[0][:1]                                   # a one-tap window and its own divisor
    divisors = [len(t) for t in windows]
    divisors[-1] = k * k + 3                                      # a count that includes padding taps
    a = eng.upload_bf16(x, h, w)
    out, dims = eng.pool_bf16(a, windows, divisors, (oh, ow))
    assert dims == (oh, ow)
    assert np.array_equal(eng.download_bits(out), orc.pool_bf16(x, windows, divisors, (oh, ow)).view(np.uint32))
    for bad, status in (((windows[:3], divisors[:3], (2, 2)), UNSUPPORTED), (([[]], [1], (1, 1)), UNSUPPORTED),
                        (([[[0, 0]]], [0], (1, 1)), UNSUPPORTED), (([[[0, 0]]], [(1 << 24) + 1], (1, 1)), UNSUPPORTED),
                        (([[[h, 0]]], [1], (1, 1)), DOMAIN_STATUS)):
        with pytest.raises(TtError) as err:
            eng.pool_bf16(a, *bad)
        assert err.value.status == status
    f = eng.upload(np.zeros((2, 2), np.float32), 2, 2)
    with pytest.raises(TtError):
        eng.pool_bf16(f, [[[0, 0]]], [1], (1, 1))               # server.rs:968 "no BF16 buffer"
    for i in (a, out, f):
        eng.free(i)
