"""Pins the CPU oracle to the closed-form known-answer cases the reference's own tests hold
for this path.  None needs a GPU.  Each case names the reference test it restates."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests import helpers as H

F = np.float32


# --- products: small integers are exact in any order (step11_burn.rs:131-168) -------------
@pytest.mark.parametrize("sa,sb", [((32, 32), (32, 32)), ((13, 47), (47, 29)), ((1, 64), (64, 96))])
def test_small_integer_products_are_the_integer_product(sa, sb):
    rng = np.random.default_rng(0xB11)
    a, b = H.small_ints(rng, sa), H.small_ints(rng, sb)
    want = a.astype(np.int64) @ b.astype(np.int64)
    got = orc.gemm_f32(a, b)
    assert np.array_equal(got.astype(np.int64), want)
    truth, s = orc.gemm_truth(a, b)
    assert np.array_equal(truth, want.astype(np.float64))
    assert orc.gemm_rel_error(got, truth, s) == (0.0, 0.0)


def test_a_transposed_right_operand(  # step11_burn.rs:157-166 "A @ B^T"
):
    rng = np.random.default_rng(7)
    a, b = H.small_ints(rng, (24, 40)), H.small_ints(rng, (30, 40))
    got = orc.gemm_f32(a, b, b_t=True)
    assert np.array_equal(got, (a.astype(np.int64) @ b.astype(np.int64).T).astype(np.float32))
    got_t = orc.gemm_f32(np.ascontiguousarray(a.T), b, a_t=True, b_t=True)
    assert np.array_equal(got, got_t)


def test_the_tile_reference_is_the_integer_product():
    # crates/tt-isa/src/numerics.rs:338-354: a 32x32 tile of small integers
    a = (np.arange(1024).reshape(32, 32) % 7 - 3).astype(np.float32)
    b = (np.arange(1024).reshape(32, 32) % 5 - 2).astype(np.float32)
    assert np.array_equal(orc.gemm_f32(a, b), (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32))


# --- in-order row sum (sfpu/reduce.rs:1162-1193) -------------------------------------------
def test_sum_over_rows_is_a_left_fold_with_a_negative_zero_column():
    rng = np.random.default_rng(3)
    a = rng.standard_normal((37, 70)).astype(np.float32)
    a[:, 5] = -0.0
    got = orc.sum_rows_in_order(a)
    acc = [F(0.0)] * 70
    for r in range(37):
        for c in range(70):
            acc[c] = F(acc[c] + a[r, c])
    assert np.array_equal(got.view(np.uint32).ravel(), np.array(acc, dtype=np.float32).view(np.uint32))
    # from +0.0: a column of -0.0 sums to +0.0 (reduce.rs:31-38)
    assert got.view(np.uint32)[0, 5] == 0
    import ctypes as C
    out = np.empty(70, dtype=np.float32)
    orc.clib().orc_sum_rows_in_order(a.ctypes.data_as(C.c_void_p), C.c_uint64(37), C.c_uint64(70), out.ctypes.data_as(C.c_void_p))
    assert np.array_equal(out.view(np.uint32), got.view(np.uint32).ravel())


def test_integer_valued_reductions_are_exact():
    # sfpu/reduce.rs:1156-1230: integer-valued inputs, any order
    a = (np.arange(64 * 96).reshape(64, 96) % 13 - 6).astype(np.float32)
    assert np.array_equal(orc.reduce(a, "SUM", 1).view(np.float32).ravel(), a.astype(np.int64).sum(1).astype(np.float32))
    assert np.array_equal(orc.reduce(a, "SUM", 0).view(np.float32).ravel(), a.astype(np.int64).sum(0).astype(np.float32))
    assert np.array_equal(orc.reduce(a, "MAX", 1).view(np.float32).ravel(), a.max(1))
    ai = a.astype(np.int32)
    assert np.array_equal(orc.reduce(ai, "SUM_I32", 0).view(np.int32).ravel(), ai.sum(0))
    assert np.array_equal(orc.reduce(ai, "MIN_I32", 1).view(np.int32).ravel(), ai.min(1))


def test_max_propagates_a_positive_nan():  # sfpu/reduce.rs:24-26
    a = np.array([[1.0, np.nan, 3.0], [-np.inf, -1.0, -0.0]], dtype=np.float32)
    got = orc.reduce(a, "MAX", 1).view(np.float32).ravel()
    assert np.isnan(got[0]) and got[1] == 0.0


# --- full sums (step63_burn_full_reduce.rs:16-20,126-138) -----------------------------------
@pytest.mark.parametrize("shape", [(1,), (70,), (37, 70), (64, 10), (3, 5, 70), (2, 2, 5, 7), (37, 8193), (8193, 1)])
def test_full_sum_shapes_within_the_reference_bound(shape):
    n = int(np.prod(shape))
    v = H.full_sum_values(n)
    stored = v.reshape(-1, shape[-1])  # [prod(leading), last] (burn-tt/src/tensor.rs:905)
    truth, bound = orc.full_sum(stored)
    in_order = orc.full_sum_reference_order(stored)
    assert abs(float(in_order) - float(stored.astype(np.float64).sum())) <= bound
    assert abs(float(truth) - float(in_order)) <= bound
    m, mb = orc.full_sum(stored, mean=True)
    assert abs(float(m) - float(stored.astype(np.float64).mean())) <= mb


@pytest.mark.parametrize("value", [-0.0, np.finfo(np.float32).tiny / 2, np.inf, -np.inf, np.nan])
def test_full_sum_special_values(value):  # step63_burn_full_reduce.rs:142-165
    v = np.full((37, 70), value, dtype=np.float32)
    s = orc.full_sum_reference_order(v)
    want = np.float64(value) * 37 * 70
    if np.isnan(want):
        assert np.isnan(s)
    elif value == 0:
        assert s == 0.0
    else:
        assert np.isclose(float(s), float(F(want)), rtol=1e-6) or float(s) == float(F(want))


# --- argmax (step211_argmax_row.rs:43-67,78-110) ---------------------------------------------
@pytest.mark.parametrize("n", [32, 33, 100, 1024, 3000])
def test_argmax_is_the_host_s_rule(n):
    for what, v in H.argmax_cases(n):
        assert orc.argmax_rows(v.reshape(1, -1))[0, 0] == H.host_argmax(v), what
        neg = -v
        assert orc.argmax_rows(neg.reshape(1, -1))[0, 0] == H.host_argmax(neg), what + " (argmin)"


def test_the_maximum_moved_is_the_other_index():  # step211_argmax_row.rs:112-124
    v = H.lcg_row(13, 4096)
    first = H.host_argmax(v)
    v[first] -= 100.0
    assert orc.argmax_rows(v.reshape(1, -1))[0, 0] == H.host_argmax(v) != first


# --- bf16 narrowing over every pattern (step270_native_bf16.rs:116,244-255; step76_burn_bf16.rs:152-169) ---
def _round_f64_grid(bits: np.ndarray) -> np.ndarray:
    """The independent F64-grid model of crates/tt-tests/tests/step76_burn_bf16.rs:152-169."""
    out = np.empty(bits.shape, dtype=np.uint32)
    for i, b in enumerate(bits.tolist()):
        sign = b & 0x80000000
        mag = b & 0x7FFFFFFF
        if mag > 0x7F800000:
            out[i] = (b | 0x00400000) & 0xFFFF0000
            continue
        if mag == 0x7F800000:
            out[i] = b
            continue
        exponent = ((b >> 23) & 255) - 127
        quantum = 2.0 ** (max(exponent, -126) - 7)
        value = float(np.uint32(mag).view(np.float32))
        q = value / quantum
        r = np.rint(q) * quantum  # ties to even
        if r < 2.0 ** -126:
            out[i] = sign
        else:
            out[i] = sign | int(np.float32(r).view(np.uint32))
    return out


def test_bf16_narrowing_matches_the_independent_model_on_every_high_half():
    # every BF16 pattern as the high half, with low halves that land below, on and above the tie
    highs = np.arange(65536, dtype=np.uint32) << 16
    for low in (0x0000, 0x7FFF, 0x8000, 0x8001, 0xFFFF):
        bits = highs | np.uint32(low)
        got = orc.bf16_round_bits(bits).astype(np.uint32) << 16
        want = _round_f64_grid(bits)
        assert np.array_equal(got, want), hex(low)
    import ctypes as C
    bits = highs | np.uint32(0x8000)
    out = np.empty(bits.shape, dtype=np.uint16)
    orc.clib().orc_bf16_round_n(bits.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), C.c_uint64(bits.size))
    assert np.array_equal(out, orc.bf16_round_bits(bits))


def test_bf16_widening_is_exact():
    h = np.arange(65536, dtype=np.uint16)
    f = orc.from_bf16(h)
    back = orc.to_bf16(f)
    sub = ((h & 0x7F80) == 0) & ((h & 0x7F) != 0)  # BF16 subnormals flush on the way back
    nan = ((h & 0x7F80) == 0x7F80) & ((h & 0x7F) != 0)
    keep = ~sub & ~nan
    assert np.array_equal(back[keep], h[keep])
    assert np.array_equal(back[sub], h[sub] & 0x8000)
    assert np.array_equal(back[nan], h[nan] | 0x0040)


# --- element-wise special values (sfpu/ops.rs:3877-3915, 4055-4110; Appendix of IEEE cases) -------
def _w(x):
    return np.array(x, dtype=np.float32).reshape(1, -1)


def test_relu_family_on_special_values():
    a = _w([np.nan, -0.0, 0.0, -1.0, 2.5, np.inf, -np.inf])
    r = orc.eltwise("RELU", a).view(np.float32).ravel()
    assert np.array_equal(r.view(np.uint32), _w([0, 0, 0, 0, 2.5, np.inf, 0]).view(np.uint32).ravel())
    g = _w([1, 2, 3, 4, 5, 6, 7])
    rb = orc.eltwise("RELU_BACKWARD", a, g).view(np.float32).ravel()
    assert np.array_equal(rb, _w([0, 0, 0, 0, 5, 6, 0]).ravel())


def test_recip_div_sqrt_ieee_cases():
    a = _w([0.0, -0.0, np.inf, -np.inf, 1.0, 3.0])
    r = orc.eltwise("RECIP", a).view(np.float32).ravel()
    assert np.array_equal(r.view(np.uint32), _w([np.inf, -np.inf, 0.0, -0.0, 1.0, F(1) / F(3)]).view(np.uint32).ravel())
    s = orc.eltwise("SQRT", _w([0.0, -0.0, np.inf, 4.0, -1.0])).view(np.float32).ravel()
    assert np.array_equal(s[:4].view(np.uint32), _w([0.0, -0.0, np.inf, 2.0]).view(np.uint32).ravel()) and np.isnan(s[4])
    d = orc.eltwise("DIV", _w([1.0, -1.0, 0.0, 6.0]), _w([0.0, 0.0, 0.0, 3.0])).view(np.float32).ravel()
    assert d[0] == np.inf and d[1] == -np.inf and np.isnan(d[2]) and d[3] == 2.0


def test_clamp_min_nan_rule_and_comparisons():  # sfpu/ops.rs:56-60,65-72
    a = _w([np.nan, 1.0, -0.0, 5.0])
    assert np.array_equal(orc.eltwise("CLAMP_MIN", a, s1=0.0).view(np.float32).ravel(), _w([0.0, 1.0, 0.0, 5.0]).ravel())
    x, y = _w([-0.0, np.nan, 1.0]), _w([0.0, np.nan, 2.0])
    assert orc.eltwise("EQ", x, y).ravel().tolist() == [1, 0, 0]
    assert orc.eltwise("NE", x, y).ravel().tolist() == [0, 1, 1]
    assert orc.eltwise("LT", x, y).ravel().tolist() == [0, 0, 1]


def test_sigmoid_two_branches_and_gelu_at_infinity():  # sfpu/ops.rs:772-799, 2036-2055
    s = orc.eltwise("SIGMOID", _w([np.inf, -np.inf, -0.0, -100.0])).view(np.float32).ravel()
    assert s[0] == 1.0 and s[1] == 0.0 and s[2] == 0.5 and s[3] >= 0.0 and s[3] < 1e-40
    g = orc.eltwise("GELU", _w([-np.inf, np.inf, 0.0])).view(np.float32).ravel()
    assert np.isnan(g[0]) and g[1] == np.inf and g[2] == 0.0


def test_int_ops_wrap_and_shift_mod_32():  # crates/burn-tt/README.md:194-199
    a = np.array([[0x7FFFFFFF, -8, 5]], dtype=np.int32)
    b = np.array([[1, 33, 35]], dtype=np.int32)
    assert orc.eltwise("INT_ADD", a, b).view(np.int32).ravel().tolist() == [-2147483648, 25, 40]
    assert orc.eltwise("INT_SHR", a, b).view(np.int32).ravel().tolist() == [0x3FFFFFFF, -4, 0]
    assert orc.eltwise("INT_SHL", a, b).view(np.int32).ravel().tolist() == [-2, -16, 40]
    f = orc.eltwise("F32_TO_I32", _w([1e20, -1e20, np.nan, -2.7])).view(np.int32).ravel().tolist()
    assert f == [2147483647, -2147483648, 0, -2]


# --- softmax (step32_burn_softmax.rs:51; step230_softmax_rows.rs header) -------------------------
@pytest.mark.parametrize("shape", [(256, 10), (70, 120), (40, 400), (64, 10), (5, 7)])
def test_softmax_rows_sum_to_one_and_match_f64(shape):
    x = orc.uniform(0x51, 1, shape, -4, 4)
    p = orc.softmax_rows(x)
    x64 = x.astype(np.float64)
    e = np.exp(x64 - x64.max(1, keepdims=True))
    want = e / e.sum(1, keepdims=True)
    assert np.max(np.abs(p - want) / want) <= orc.softmax_bound(shape[1])
    lp = orc.softmax_rows(x, log_form=True)
    assert np.max(np.abs(lp - np.log(want))) <= 1e-5


def test_a_fully_masked_row_is_zeros():
    x = orc.uniform(0x51, 2, (4, 64), -4, 4)
    mask = np.zeros((4, 64), dtype=np.uint32)
    mask[1, :] = 1
    mask[2, ::2] = 1
    p = orc.softmax_rows(x, mask, scale=0.5)
    assert np.all(p[1] == 0.0)
    assert np.all(p[2, ::2] == 0.0) and abs(p[2].sum() - 1) < 1e-6


# --- rms norm / rope --------------------------------------------------------------------------------
def test_rms_statistic_is_the_five_ops():  # sfpu/norm.rs:1-5
    x = orc.normal(0x52, 1, (33, 576))
    st = orc.rms(x, 1e-5)
    want = np.sqrt((x.astype(np.float64) ** 2).mean(1, keepdims=True) + 1e-5)
    assert np.max(np.abs(st - want) / want) < 1e-6
    nx = orc.rms_norm(x, np.ones(576, dtype=np.float32), 1e-5)
    assert np.allclose((nx.astype(np.float64) ** 2).mean(1), 1.0, atol=1e-4)


def test_rope_is_the_rotate_half_composition():  # tt-models/src/rope.rs:151-161
    head, heads, t = 64, 3, 16
    cos, sin = orc.rope_tables(t, head, 10000.0)
    x = orc.normal(0x53, 1, (t, heads * head))
    y = orc.rope(x, cos, sin, head)
    xs = x.reshape(t, heads, head)
    x1, x2 = xs[..., :32], xs[..., 32:]
    c, s = cos[:, None, :32].astype(np.float64), -sin[:, None, :32].astype(np.float64)
    want = np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s], axis=-1).reshape(t, -1)
    assert np.max(np.abs(y - want)) < 1e-6
    # position 0 is the identity
    assert np.array_equal(y[0], x[0])


# --- the seeded generator is stable (its first draws are written down) ------------------------------
def test_seeded_generator_first_draws():
    z = orc.splitmix64(0xC0F2, 0, 3)
    assert [int(v) for v in z] == [int(v) for v in orc.splitmix64(0xC0F2, 0, 5)[:3]]
    u = orc.uniform(0xC0F2, 0, (4,), -1, 1)
    assert np.all((u >= -1) & (u < 1))
    assert orc.integers(0xC0F1, 5, (64,), 10).max() <= 9
    g = orc.normal(0xC0F4, 1, (10000,), 0.02)
    assert abs(g.std() - 0.02) < 1e-3


def test_binary16_conversions_are_ieee():   # crates/tt-kernels/src/fp16.rs:172-176, 271-275 against numpy's binary16
    x = (orc.splitmix64(0xF16, 1, 200000) >> np.uint64(32)).astype(np.uint32)
    edge = np.array([0, 0x80000000, 0x33000000, 0x33000001, 0x387FE000, 0x387FFFFF, 0x38800000, 0x477FEFFF, 0x477FF000,
                     0x7F800000, 0xFF800000, 0x33800000, 1], dtype=np.uint32)
    x = np.concatenate([x, edge])
    f = x.view(np.float32)
    ok = ~np.isnan(f)
    with np.errstate(all="ignore"):
        want = f[ok].astype(np.float16).view(np.uint16)
    assert np.array_equal(orc.f16_bits_from_f32_bits(x[ok]), want)
    h = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    w = orc.f32_bits_from_f16_bits(h)
    fin = ~np.isnan(h.view(np.float16))
    assert np.array_equal(w[fin], h.view(np.float16)[fin].astype(np.float32).view(np.uint32))
    assert np.array_equal(orc.f16_bits_from_f32_bits(w[fin]), h[fin])              # widening then narrowing is the identity
    # a NaN keeps its sign and top payload bits and is made quiet
    assert orc.f16_bits_from_f32_bits(np.array([0xFFC12345, 0x7F800001], np.uint32)).tolist() == [0xFE09, 0x7E00]
    assert orc.f32_bits_from_f16_bits(np.array([0xFC01, 0x7E00], np.uint16)).tolist() == [0xFFC02000, 0x7FC00000]


def test_scans_follow_row_order_from_the_identity():   # crates/tt-kernels/src/sfpu/scan.rs:196-231
    x = np.array([[1.0, -0.0], [2.0, -0.0], [3.0, 5.0]], dtype=np.float32)
    assert np.array_equal(orc.scan(x.view(np.uint32), "sum").view(np.float32), [[1, 0], [3, 0], [6, 5]])
    assert orc.scan(x.view(np.uint32), "sum")[0, 1] == 0                               # +0.0 + -0.0 = +0.0
    assert orc.scan(x.view(np.uint32), "prod")[1, 1] == 0                              # 1 * -0 * -0 = +0
    nan, nnan = np.uint32(0x7FC00001), np.uint32(0xFFC00002)
    col = np.array([[0x40000000], [0x80000000], [0x00000000], [nan], [0x3F800000], [nnan]], dtype=np.uint32)
    # Flex's cummin: the earlier zero wins a tie; a NaN replaces the accumulator and is only replaced by a NaN
    assert orc.scan(col, "min_nan").ravel().tolist() == [0x40000000, 0x80000000, 0x80000000, nan, nan, nnan]
    # raw total order: -NaN < ... < -0 < +0 < ... < +NaN
    assert orc.scan(col, "min").ravel().tolist() == [0x40000000, 0x80000000, 0x80000000, 0x80000000, 0x80000000, nnan]
    assert orc.scan(col, "max").ravel().tolist() == [0x40000000, 0x40000000, 0x40000000, nan, nan, nan]
    i = np.array([[0x7FFFFFFF], [1], [0x80000000]], dtype=np.uint32)
    assert orc.scan(i, "isum").ravel().tolist() == [0x7FFFFFFF, 0x80000000, 0]        # wrapping
    assert orc.scan(i, "imin").ravel().tolist() == [0x7FFFFFFF, 1, 0x80000000]
    assert orc.scan(np.array([[3], [0x80000001], [2]], np.uint32), "iprod").ravel().tolist() == [3, 0x80000003, 6]


def test_sort_order_and_the_planes_layout():   # crates/tt-kernels/src/sfpu/sort.rs:5-13, 198-228
    v = np.array([[0x7FC00000, 0x80000000, 0x00000000, 0xFFC00000, 0x3F800000, 0x3F800000, 0xFF800000]], dtype=np.uint32)
    k, i = orc.sort_rows(v, False, False)
    assert k.ravel().tolist() == [0xFFC00000, 0xFF800000, 0x80000000, 0, 0x3F800000, 0x3F800000, 0x7FC00000]
    assert i.ravel().tolist() == [3, 6, 1, 2, 4, 5, 0]
    k, i = orc.sort_rows(v, False, True)
    assert i.ravel().tolist() == [0, 4, 5, 2, 1, 6, 3]                                 # ties still in ascending index
    k, i = orc.sort_rows(np.array([[5, 0xFFFFFFFF, 5, 0x80000000]], np.uint32), True, False)
    assert i.ravel().tolist() == [3, 1, 0, 2]
    assert orc.plane_dims(33, 100) == (128, 64) and orc.plane_dims(1, 1) == (32, 32)
    seen = {orc.plane_coord(q, e) for q in range(32) for e in range(32)}
    assert len(seen) == 1024 and max(r for r, _ in seen) == 31 and max(c for _, c in seen) == 31   # a tile: 32 problems x 32 positions
    assert orc.plane_coord(0, 0) == (0, 0) and orc.plane_coord(1, 0) == (0, 2) and orc.plane_coord(0, 1) == (0, 1)
    assert orc.plane_coord(8, 0) == (1, 0) and orc.plane_coord(0, 2) == (4, 0) and orc.plane_coord(0, 8) == (0, 16)
    assert orc.plane_coord(0, 16) == (16, 0) and orc.plane_coord(32, 32) == (32, 32)


def test_device_draws_are_the_reference_arithmetic_on_unit_uniforms():   # crates/tt-kernels/src/prng.rs:41-42, 449-595
    u = orc.random_draw((300, 300), ("unit",), 5)
    assert u.min() >= 0 and u.max() < 1 and np.array_equal(u * 2.0**23, np.round(u * 2.0**23)) and abs(u.mean() - 0.5) < 5e-3
    v = orc.random_draw((300, 300), ("uniform", 1.0, 1.0000002), 5)
    assert v.max() < np.float32(1.0000002) and v.min() >= 1.0
    r = orc.random_draw((300, 300), ("int_range", -5, 12), 5)
    assert r.min() == -5 and r.max() == 11 and r.dtype == np.int32
    z = orc.random_draw((400, 400), ("normal", 2.0, 3.0, False), 5)
    assert abs(z.mean() - 2.0) < 0.03 and abs(z.std() - 3.0) < 0.03
    b = orc.random_draw((400, 400), ("bernoulli", 0.3, True), 5)
    assert abs(b.mean() - 0.3) < 5e-3 and set(np.unique(b)) == {0, 1}
    assert orc.select_taps(np.arange(6, dtype=np.uint32).reshape(2, 3), np.array([[1, 2], [0, 1]]), True).tolist() == \
        [[3, 4, 5] + [0] * 29 + [0, 1, 2], [0] * 32 + [3, 4, 5]]


def test_convolution_and_pooling_restatements_agree_with_torch_cpu():   # a second, independent check (never the only one)
    import torch
    x = orc.normal(1, 1, (2, 5, 9, 8)); w = orc.uniform(1, 2, (4, 5, 3, 2), -1, 1); b = orc.uniform(1, 3, (4,), -1, 1)
    truth, s = orc.conv2d(x, w, b, (2, 1), (1, 2), (1, 2))
    ref = torch.nn.functional.conv2d(torch.from_numpy(x).double(), torch.from_numpy(w).double(), torch.from_numpy(b).double(),
                                     stride=(2, 1), padding=(1, 2), dilation=(1, 2)).numpy()
    assert truth.shape == ref.shape and np.abs(truth - ref).max() <= 1e-12 and np.all(s >= np.abs(truth) - 1e-12)
    xb = np.round(orc.uniform(2, 1, (1, 3, 8, 9), -3, 3))
    m = orc.max_pool2d(xb.view(np.uint32), (3, 2), (2, 1), (1, 0), (1, 2)).view(np.float32)
    assert np.array_equal(m, torch.nn.functional.max_pool2d(torch.from_numpy(xb), (3, 2), (2, 1), (1, 0), (1, 2)).numpy())
    nan = np.array([[[[1.0, np.nan], [5.0, np.nan]]]], np.float32)
    nan.view(np.uint32)[0, 0, 1, 1] = 0xFFC00005
    assert orc.max_pool2d(nan.view(np.uint32), (2, 2), (1, 1), (0, 0), (1, 1))[0, 0, 0, 0] == 0x7FC00000   # the first NaN


def test_the_c_twins_of_the_draws_and_of_the_ulp_measure_agree_with_numpy():
    # Large tensors are drawn and compared by C loops (oracle.c) instead of NumPy passes; on a size both forms take,
    # the same numbers come out.
    n = (1 << 20) + 7
    for tag, lo, hi in ((1, -4.0, 4.0), (2, 0.01, 4.0)):
        c_form = orc.uniform(0xC0F3, tag, (n,), lo, hi)
        u = (orc.splitmix64(0xC0F3, tag, n) >> np.uint64(40)).astype(np.float32) / np.float32(16777216.0)
        numpy_form = (np.float32(lo) + (np.float32(hi) - np.float32(lo)) * u).astype(np.float32)
        assert np.array_equal(c_form, numpy_form)
    want = orc.eltwise("EXP", c_form)
    got = want.copy()
    got[5] += 3
    got[9] = np.float32(np.nan).view(np.uint32)
    small = orc.ulp_error(got[:1000], want[:1000])                  # the NumPy form
    assert small == np.inf and orc.ulp_error(got, want) == np.inf   # a NaN against a number: infinite in both
    got[9] = want[9]
    assert abs(orc.ulp_error(got, want) - orc.ulp_error(got[:1000], want[:1000])) < 1e-9
    assert orc.ulp_error(want, want) == 0.0
