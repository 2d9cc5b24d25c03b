"""`random_dram` through the C ABI (crates/burn-tt/src/server.rs:768).  The engine's word stream is its own
(the reference's differs between its simulator and its silicon, crates/tt-kernels/src/prng.rs:49-50), so the
check is in two parts: the draws equal the oracle's restatement of the same stream and of the reference's
arithmetic on unit uniforms (prng.rs:449-595) -- exactly where that arithmetic is exact, within 4 ulp of the
radius and angle functions for the normal draw -- and the statistics the reference's own gate holds a draw to
(mean, variance, range, the half-open interval)."""
import numpy as np
import pytest

from metalium_rs_b200 import UNSUPPORTED, TtError
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
DIMS = (517, 1030)


def _draw(eng, draw, base, dims=DIMS, integer=False):
    out, od = eng.random_dram(dims, draw, base)
    assert od == dims
    bits = eng.download_bits(out)
    eng.free(out)
    return bits.view(np.int32) if integer else bits.view(np.float32)


@pytest.mark.parametrize("draw,integer", [(("unit",), False), (("uniform", -3.0, 5.5), False), (("uniform", 1.0, 1.0000002), False),
                                          (("bernoulli", 0.3, False), False), (("bernoulli", 0.75, True), True),
                                          (("int_range", -5, 12), True), (("int_range", 0, 1 << 23), True), (("int_words",), True)])
def test_exact_draws_equal_the_restated_stream(eng, draw, integer):
    got = _draw(eng, draw, 0xBA5E, integer=integer)
    want = orc.random_draw(DIMS, draw, 0xBA5E)
    assert got.dtype == want.dtype and np.array_equal(got, want)


def test_unit_draws_are_multiples_of_two_to_the_minus_23_below_one(eng):   # prng.rs:41-42
    u = _draw(eng, ("unit",), 1)
    assert u.min() >= 0.0 and u.max() < 1.0 and np.array_equal(u * 2.0**23, np.round(u * 2.0**23))
    assert abs(u.mean() - 0.5) < 2e-3 and abs(u.var() - 1 / 12) < 2e-3


def test_a_uniform_draw_never_reaches_its_upper_end(eng):   # prng.rs:449-452: clamped to the float below hi
    v = _draw(eng, ("uniform", 1.0, 1.0000002), 3)
    assert v.min() >= 1.0 and v.max() < np.float32(1.0000002)


@pytest.mark.parametrize("as_int", [False, True])
def test_normal_draws(eng, as_int):
    got = _draw(eng, ("normal", 2.0, 3.0, as_int), 0x4042, integer=as_int)
    want = orc.random_draw(DIMS, ("normal", 2.0, 3.0, as_int), 0x4042)
    if as_int:
        assert np.mean(got != want) < 1e-4 and np.abs(got.astype(np.int64) - want).max() <= 1    # a truncation may fall either side
    else:
        assert np.abs(got - want).max() <= 3.0 * 6 * 2.0**-22      # std x the radius's largest value x 4 ulp of a unit value
        assert abs(got.mean() - 2.0) < 0.02 and abs(got.std() - 3.0) < 0.02
        assert np.abs(got - 2.0).max() <= 3.0 * 5.65                # the tail is cut at sqrt(-2 ln 2^-23) sigma (prng.rs:506-507)


def test_a_draw_depends_on_base_role_and_position_only(eng):   # prng.rs:34-36
    a = _draw(eng, ("unit",), 77, dims=(64, 100))
    b = _draw(eng, ("unit",), 77, dims=(100, 64))
    assert np.array_equal(a.ravel(), b.ravel())
    c = _draw(eng, ("unit",), 78, dims=(64, 100))
    assert np.mean(a == c) < 1e-3
    d = _draw(eng, ("uniform", 0.0, 1.0), 77, dims=(64, 100))   # another role: another stream
    assert np.mean(a == d) < 1e-3


@pytest.mark.parametrize("draw", [("uniform", 1.0, 1.0), ("uniform", 0.0, float("inf")), ("bernoulli", 1.5, False),
                                  ("normal", 0.0, -1.0, False), ("int_range", 5, 5), ("int_range", 0, (1 << 23) + 1)])
def test_draws_the_reference_refuses(eng, draw):   # prng.rs:462-466, 487-491, 517-521, 574-578
    with pytest.raises(TtError) as err:
        eng.random_dram((4, 4), draw, 0)
    assert err.value.status == UNSUPPORTED
