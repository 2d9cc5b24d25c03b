"""Element-wise parity through the C ABI against the CPU oracle, kind by kind, in the
shape of crates/tt-tests/tests/step19_eltwise.rs:121 and step27_burn_eltwise.rs:51:
exact kinds bit for bit, transcendental kinds within the reference's derived bound."""
import numpy as np
import pytest

from metalium_rs_b200 import BF16, BOOL, F32, I32, EltwiseOp, TtError, kinds
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

SPECIALS = np.array([0.0, -0.0, 1.0, -1.0, np.inf, -np.inf, np.nan, 1e-40, -1e-40, 3.4e38, -3.4e38, 1.17549435e-38,
                     88.0, -88.0, 89.0, -104.0, 0.5, 2.0, 1e-8, 123456.789], dtype=np.float32)


def inputs(kind_name, shape, seed):
    lo, hi = -4.0, 4.0
    if kind_name in ("LOG", "SQRT", "RSQRT", "RECIP", "LOG1P", "ACOSH", "POW", "POW_S"):
        lo, hi = 0.01, 4.0
    if kind_name in ("ASIN", "ACOS", "ATANH"):
        lo, hi = -0.99, 0.99
    if kind_name == "ACOSH":
        lo, hi = 1.01, 4.0
    a = orc.uniform(seed, 1, shape, lo, hi)
    b = orc.uniform(seed, 2, shape, lo, hi)
    c = orc.uniform(seed, 3, shape, lo, hi)
    return a, b, c


FLOAT_KINDS = ["ADD", "SUB", "MUL", "MUL_SCALAR", "ADD_SCALAR", "RELU", "RELU_BACKWARD", "RECIP", "DIV", "DIV_SCALAR", "EXP",
               "LOG", "NEG", "ABS", "SIGN", "CLAMP", "CLAMP_MIN", "CLAMP_MAX", "LEAKY_RELU", "HARD_SIGMOID", "PRELU", "FILL",
               "SQRT", "RSQRT", "LOG1P", "POW", "POW_S", "EXPM1", "SIGMOID", "SIGMOID_BACKWARD", "TANH", "ERF", "GELU",
               "GELU_TANH", "GELU_BACKWARD", "SINH", "COSH", "ASINH", "ACOSH", "ATANH", "LOG_SIGMOID", "LOG_SIGMOID_BACKWARD",
               "SIN", "COS", "TAN", "ATAN", "ATAN2", "ASIN", "ACOS", "REM", "REM_S", "ROUND", "FLOOR", "CEIL", "TRUNC",
               "POW2_FLOOR", "POW2_FLOOR_INV", "ADD_RELU", "SILU", "SILU_MUL", "SUB_EXP", "MUL_ADD",
               "EQ", "NE", "GT", "GE", "LT", "LE", "EQ_S", "NE_S", "GT_S", "GE_S", "LT_S", "LE_S", "IS_NAN", "IS_INF",
               "F32_TO_I32"]


def run(eng, name, a, b=None, c=None, s1=0.0, s2=0.0, elem=F32, bf16=False):
    k = getattr(kinds, name)
    r, cc = a.shape
    ia = eng.upload_bits(a.view(np.uint32), r, cc, elem)
    ib = eng.upload_bits(b.view(np.uint32), b.shape[0], b.shape[1], elem if name not in MASKED else BOOL) if b is not None else None
    ic = eng.upload_bits(c.view(np.uint32), r, cc, elem) if c is not None else None
    out, dims = eng.eltwise_op_as(EltwiseOp(k, s1, s2), ia, ib, ic, bf16)
    got = eng.download_bf16(out) if bf16 else eng.download_bits(out)
    for i in (ia, ib, ic, out):
        if i:
            eng.free(i)
    return got, dims


MASKED = {"MASK_FILL", "MASK_WHERE", "INT_MASK_FILL", "INT_MASK_WHERE", "BOOL_MASK_FILL", "BOOL_MASK_WHERE", "SCALE_MASK_FILL"}


@pytest.mark.parametrize("name", FLOAT_KINDS)
@pytest.mark.parametrize("shape", [(64, 128), (37, 70)])
def test_float_kind_against_oracle(eng, name, shape):
    a, b, c = inputs(name, shape, 0xE17)
    # specials in the first row
    a.ravel()[:SPECIALS.size] = SPECIALS
    b.ravel()[:SPECIALS.size] = SPECIALS[::-1]
    ar = kinds.ARITY[getattr(kinds, name)]
    s1, s2 = (0.75, 1.5) if name != "CLAMP" else (-1.0, 2.0)
    if name == "HARD_SIGMOID":
        s1, s2 = 0.2, 0.5
    got, dims = run(eng, name, a, b if ar >= 2 else None, c if ar == 3 else None, s1, s2)
    want = orc.eltwise(name, a, b if ar >= 2 else None, c if ar == 3 else None, s1, s2)
    assert dims == shape
    bound = orc.ULP_BOUND.get(name)
    if bound is None or bound == 0.0:
        nan_both = (np.isnan(got.view(np.float32)) & np.isnan(want.view(np.float32))) if name not in ("NEG", "ABS") else np.zeros(got.shape, bool)
        bad = (got != want) & ~nan_both
        assert not bad.any(), f"{name}: {int(bad.sum())} words differ, first at {np.argwhere(bad)[0]}: " \
                              f"{got[bad][0]:#x} vs {want[bad][0]:#x} (a={a[bad][0]!r})"
    else:
        # the contract: 1e-5 relative (north star); the tighter derived bound is asserted too
        if name == "GELU_BACKWARD":  # has a root near x = -0.75: the bound is absolute there
            d = np.abs(got.view(np.float32).astype(np.float64) - want.view(np.float32).astype(np.float64))
            ok = np.isnan(d) | (d <= 1e-5 * np.abs(want.view(np.float32)) + 4e-6 * np.abs(b))
            assert ok.all()
            return
        e = orc.ulp_error(got, want)
        assert e <= bound + 1.0, f"{name}: {e:.2f} u exceeds the reference's bound {bound} u (+1 u for the oracle's own rounding)"


@pytest.mark.parametrize("name", ["ADD", "SUB", "MUL", "DIV", "ADD_RELU", "SUB_EXP", "GT", "PRELU"])
def test_broadcast_forms(eng, name):
    # b as one row, one column, and whole rows repeated (tt-kernels/src/tensor.rs:3799-3859)
    a = orc.uniform(0xB0, 1, (96, 64), -4, 4)
    for bshape in [(1, 64), (96, 1), (32, 64), (96, 64)]:
        b = orc.uniform(0xB0, 2, bshape, 0.5, 4)
        got, dims = run(eng, name, a, b)
        want = orc.eltwise(name, a, b)
        assert dims == (96, 64)
        if orc.ULP_BOUND.get(name):
            assert orc.ulp_error(got, want) <= orc.ULP_BOUND[name] + 1
        else:
            assert np.array_equal(got, want), (name, bshape)


def test_add_and_mul_take_the_broadcast_operand_on_the_left(eng):  # burn-tt/src/ops.rs:1850
    a = orc.uniform(0xB1, 1, (1, 64), -4, 4)
    b = orc.uniform(0xB1, 2, (48, 64), -4, 4)
    for name in ("ADD", "MUL"):
        got, dims = run(eng, name, a, b)
        assert dims == (48, 64) and np.array_equal(got, orc.eltwise(name, b, a))


def test_add_row_is_add_with_a_row(eng):  # kind.rs:24
    a = orc.uniform(0xB2, 1, (64, 128), -4, 4)
    b = orc.uniform(0xB2, 2, (1, 128), -4, 4)
    got, _ = run(eng, "ADD_ROW", a, b)
    assert np.array_equal(got, orc.eltwise("ADD", a, b))


@pytest.mark.parametrize("name", ["MASK_FILL", "MASK_WHERE", "SCALE_MASK_FILL"])
def test_mask_kinds(eng, name):
    a = orc.uniform(0xB3, 1, (40, 72), -4, 4)
    c = orc.uniform(0xB3, 3, (40, 72), -4, 4)
    mask = (orc.integers(0xB3, 2, (40, 72), 2)).astype(np.uint32)
    ar = kinds.ARITY[getattr(kinds, name)]
    got, _ = run(eng, name, a, mask.view(np.float32), c if ar == 3 else None, 0.125, -np.inf)
    want = orc.eltwise(name, a, mask, c if ar == 3 else None, 0.125, -np.inf)
    assert np.array_equal(got, want)


INT_KINDS = ["INT_ADD", "INT_SUB", "INT_MUL", "INT_AND", "INT_OR", "INT_XOR", "INT_SHL", "INT_SHR", "INT_EQ", "INT_NE",
             "INT_GT", "INT_GE", "INT_LT", "INT_LE", "INT_NOT", "INT_ABS", "INT_ADD_S", "INT_SUB_S", "INT_MUL_S", "INT_AND_S",
             "INT_SHL_S", "INT_SHR_S", "INT_EQ_S", "INT_LT_S", "INT_DIV", "INT_REM", "INT_DIV_S", "INT_REM_S", "I32_TO_F32"]


@pytest.mark.parametrize("name", INT_KINDS)
def test_int_kinds_bit_exact(eng, name):
    a = (orc.splitmix64(0x1A7, 1, 50 * 40) >> np.uint64(32)).astype(np.uint32).view(np.int32).reshape(50, 40).copy()
    b = (orc.splitmix64(0x1A7, 2, 50 * 40) >> np.uint64(32)).astype(np.uint32).view(np.int32).reshape(50, 40).copy()
    a.ravel()[:4] = [np.iinfo(np.int32).min, np.iinfo(np.int32).max, -1, 0]
    if name in ("INT_DIV", "INT_REM"):
        b[b == 0] = 3
        b.ravel()[:4] = [-1, -1, 7, 5]
    ar = kinds.ARITY[getattr(kinds, name)]
    s_bits = np.array([12345 if "SH" not in name else 35], dtype=np.int32).view(np.float32)[0]
    got, _ = run(eng, name, a.view(np.float32), b.view(np.float32) if ar == 2 else None, None, float(s_bits), 0.0, elem=I32)
    want = orc.eltwise(name, a, b if ar == 2 else None, None, s_bits)
    assert np.array_equal(got, want), name


def test_int_division_by_zero_is_a_domain_error_at_the_next_wait(fresh_eng):
    e = fresh_eng
    a = np.arange(64, dtype=np.int32).reshape(8, 8)
    b = np.ones((8, 8), dtype=np.int32)
    b[3, 3] = 0
    ia = e.upload_bits(a.view(np.uint32), 8, 8, I32)
    ib = e.upload_bits(b.view(np.uint32), 8, 8, I32)
    out, _ = e.eltwise_op_as(EltwiseOp(kinds.INT_DIV, 0, 0), ia, ib)  # returns: the failure is asynchronous
    with pytest.raises(TtError) as ei:
        e.download_bits(out)
    assert "DOMAIN" in str(ei.value)
    with pytest.raises(TtError):  # every later wait reports the first failure (server.rs:2392-2405)
        e.sync()


@pytest.mark.parametrize("name", ["ADD", "MUL", "SILU_MUL", "RELU", "EXP"])
def test_bf16_operands_and_results_round_once(eng, name):
    # step270_native_bf16.rs: op(x.cast(F32)).cast(BF16), bit for bit for exact kinds
    a = orc.to_bf16(orc.uniform(0xBF, 1, (33, 96), -4, 4))
    b = orc.to_bf16(orc.uniform(0xBF, 2, (33, 96), -4, 4))
    ia, ib = eng.upload_bf16(a, 33, 96), eng.upload_bf16(b, 33, 96)
    ar = kinds.ARITY[getattr(kinds, name)]
    out, dims = eng.eltwise_op_as(EltwiseOp(getattr(kinds, name), 0, 0), ia, ib if ar == 2 else None, None, True)
    got = eng.download_bf16(out)
    want32 = orc.eltwise(name, orc.from_bf16(a), orc.from_bf16(b) if ar == 2 else None)
    want = orc.bf16_round_bits(want32)
    if orc.ULP_BOUND.get(name):
        diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
        assert diff.max() <= 1  # one BF16 step where the F32 values straddle a tie
    else:
        assert np.array_equal(got, want)
    for i in (ia, ib, out):
        eng.free(i)


def test_eltwise_blocks_reads_blocks_where_they_lie(eng):  # server.rs:536-566
    a = orc.uniform(0xB7, 1, (128, 192), -4, 4)
    b = orc.uniform(0xB7, 2, (64, 256), -4, 4)
    ia, ib = eng.upload(a, 128, 192), eng.upload(b, 64, 256)
    out, dims = eng.eltwise_blocks(EltwiseOp(kinds.MUL, 0, 0), (ia, (32, 64), (64, 96)), (ib, (0, 128), (64, 96)))
    assert dims == (64, 96)
    got = eng.download(out)
    assert np.array_equal(got, a[32:96, 64:160] * b[:, 128:224])
    for i in (ia, ib, out):
        eng.free(i)


def test_cast_float_every_pattern(eng):  # step270_native_bf16.rs:116
    highs = (np.arange(65536, dtype=np.uint32) << 16)
    for low in (0x0000, 0x7FFF, 0x8000, 0x8001):
        bits = (highs | np.uint32(low)).reshape(256, 256)
        ia = eng.upload_bits(bits, 256, 256, F32)
        out, _ = eng.cast_float(ia, True)
        got = eng.download_bf16(out)
        assert np.array_equal(got.ravel(), orc.bf16_round_bits(bits.ravel())), hex(low)
        back, _ = eng.cast_float(out, False)
        assert np.array_equal(eng.download_bits(back).ravel(), got.ravel().astype(np.uint32) << 16)
        for i in (ia, out, back):
            eng.free(i)


def test_rope_blocks(eng):  # tt-kernels/src/tensor.rs:5545-5552
    head, heads, t = 64, 9, 96
    cos, sin = orc.rope_tables(t, head, 10000.0)
    x = orc.normal(0xB8, 1, (t, heads * head))
    ix, ic, isn = eng.upload(x, t, heads * head), eng.upload(cos, t, head), eng.upload(sin, t, head)
    out, dims = eng.rope_blocks((ix, (0, 0), (t, heads * head)), (ic, (0, 0), (t, head)), (isn, (0, 0), (t, head)), head)
    assert np.array_equal(eng.download(out).view(np.uint32), orc.rope(x, cos, sin, head).view(np.uint32))
    ob, _ = eng.rope_blocks((ix, (0, 0), (t, heads * head)), (ic, (0, 0), (t, head)), (isn, (0, 0), (t, head)), head, True)
    assert np.array_equal(eng.download_bf16(ob), orc.to_bf16(orc.rope(x, cos, sin, head)))
    for i in (ix, ic, isn, out, ob):
        eng.free(i)


def test_unknown_kind_and_bad_shapes_are_refused(eng):
    a = eng.upload(np.zeros((4, 4), np.float32), 4, 4)
    b = eng.upload(np.zeros((3, 4), np.float32), 3, 4)
    with pytest.raises(TtError) as ei:
        eng.eltwise_op(EltwiseOp(0x1b0, 0, 0), a)  # HARDWARE_ROUND: a Tensix rounding mode
    assert ei.value.status == 2
    with pytest.raises(TtError):
        eng.eltwise_op(EltwiseOp(kinds.ADD, 0, 0), a, b)
    with pytest.raises(TtError):
        eng.eltwise_op(EltwiseOp(kinds.EXP, 0, 0), a, b)  # a unary kind with two operands
    with pytest.raises(TtError):
        eng.eltwise_op(EltwiseOp(kinds.CLAMP, 2.0, 1.0), a)  # crossed bounds, as f32::clamp panics
    eng.free(a); eng.free(b)


def test_large_unary_and_row_broadcast_fast_path(eng):
    # the 128-bit fast path at a size past L2, against the oracle
    a = orc.uniform(0xC0F3, 1, (4096, 8192), -4, 4)
    row = orc.uniform(0xC0F3, 2, (1, 8192), -4, 4)
    ia, ir = eng.upload(a, 4096, 8192), eng.upload(row, 1, 8192)
    for name, bb in (("RELU", None), ("MUL", ir), ("ADD", ir)):
        out, _ = eng.eltwise_op(EltwiseOp(getattr(kinds, name), 0, 0), ia, bb)
        got = eng.download_bits(out)
        want = orc.eltwise(name, a, row if bb else None)
        assert np.array_equal(got, want), name
        eng.free(out)
    eng.free(ia); eng.free(ir)


@pytest.mark.parametrize("name", ["ADD", "MUL", "SILU_MUL", "SUB", "ADD_RELU", "MUL_ADD"])
@pytest.mark.parametrize("mix", ["f32", "bf16", "mixed"])
def test_block_operands_of_either_type(eng, name, mix):
    # blocks of wider buffers, F32 or BF16 on either side, F32 or BF16 out: the 8-wide path and
    # the element path must give the same bits as the oracle on the widened values
    a = orc.uniform(0xB9, 1, (96, 256), -4, 4)
    b = orc.uniform(0xB9, 2, (64, 384), -4, 4)
    c = orc.uniform(0xB9, 3, (64, 128), -4, 4)
    abf, bbf = mix == "bf16", mix in ("bf16", "mixed")
    ah, bh = orc.to_bf16(a), orc.to_bf16(b)
    av = orc.from_bf16(ah) if abf else a
    bv = orc.from_bf16(bh) if bbf else b
    ia = eng.upload_bf16(ah, 96, 256) if abf else eng.upload(a, 96, 256)
    ib = eng.upload_bf16(bh, 64, 384) if bbf else eng.upload(b, 64, 384)
    ic = eng.upload(c, 64, 128)
    ar = kinds.ARITY[getattr(kinds, name)]
    for (ac, bc, w) in ((64, 128, 128), (8, 16, 40), (3, 5, 37)):   # aligned, aligned-narrow, ragged
        blk_a = (ia, (32, ac), (64, w))
        blk_b = (ib, (0, bc), (64, w))
        blk_c = (ic, (0, 0), (64, w)) if ar == 3 else None
        want = orc.eltwise(name, av[32:96, ac:ac + w], bv[:, bc:bc + w], c[:, :w] if ar == 3 else None)
        for out_bf in (False, True):
            out, dims = eng.eltwise_blocks_as(EltwiseOp(getattr(kinds, name), 0, 0), blk_a, blk_b, blk_c, out_bf)
            assert dims == (64, w)
            if out_bf:
                got, ref = eng.download_bf16(out), orc.bf16_round_bits(want)
            else:
                got, ref = eng.download_bits(out), want
            if orc.ULP_BOUND.get(name):
                if out_bf:
                    assert np.abs(got.astype(np.int32) - ref.astype(np.int32)).max() <= 1
                else:
                    assert orc.ulp_error(got, ref) <= orc.ULP_BOUND[name] + 1
            else:
                assert np.array_equal(got, ref), (name, mix, w, out_bf)
            eng.free(out)
    for i in (ia, ib, ic):
        eng.free(i)


def test_rope_blocks_of_a_wider_bf16_buffer(eng):
    # q and k as column blocks of one [t, q+k+v] BF16 buffer, tables shorter than the rows (r % t)
    head, t, batch = 64, 32, 3
    cos, sin = orc.rope_tables(t, head, 10000.0)
    x = orc.to_bf16(orc.normal(0xBA, 1, (batch * t, 15 * head)))
    ix, ic, isn = eng.upload_bf16(x, batch * t, 15 * head), eng.upload(cos, t, head), eng.upload(sin, t, head)
    xv = orc.from_bf16(x)
    for c0, heads in ((0, 9), (9 * head, 3)):
        out, dims = eng.rope_blocks((ix, (0, c0), (batch * t, heads * head)), (ic, (0, 0), (t, head)),
                                    (isn, (0, 0), (t, head)), head, True)
        want = orc.rope(xv[:, c0:c0 + heads * head], cos, sin, head)
        assert np.array_equal(eng.download_bf16(out), orc.to_bf16(want))
        eng.free(out)
    for i in (ix, ic, isn):
        eng.free(i)
