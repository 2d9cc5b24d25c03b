"""The block-float (BFP8) rules the engine's `cast_bfp` is held to, pinned on the CPU: the decoder is the reference's
`bfp8_to_bf16` (crates/tt-isa/src/tile.rs:619-634), whose own test proves it over all 65,536 inputs against the
documented routine (tile.rs:1118-1146) and records the -infinity trap (tile.rs:1148-1160); the encoder is the engine's
(the reference's is its packer hardware) and is checked through that decoder."""
import numpy as np

from oracle import oracle as orc


def documented_routine(datum: int, exp: int) -> int:
    """The specification's C as the reference's test transliterates it (tile.rs:1121-1135), one datum at a time and
    sharing no code with `orc.bfp8_decode_bits`."""
    sign = datum >> 7
    mag = (datum << 1) & 0xFF
    if mag == 0:
        return 0xFF80 if sign else 0
    lz = 8 - mag.bit_length()
    mag = (mag << lz) & 0xFF
    return (sign << 15) | (((exp - lz) & 0xFF) << 7) | (mag & 0x7E)


def test_the_decoder_is_the_documented_routine_over_its_whole_domain():      # tile.rs:1118-1146
    d, e = np.meshgrid(np.arange(256, dtype=np.uint8), np.arange(256, dtype=np.uint8), indexing="ij")
    want = np.array([[documented_routine(int(x), int(y)) for y in range(256)] for x in range(256)], dtype=np.uint16)
    assert np.array_equal(orc.bfp8_decode_bits(d, e), want)


def test_a_negative_zero_magnitude_datum_is_not_negative_zero():             # tile.rs:1148-1160
    assert orc.bfp8_decode_bits(np.uint8(0x00), np.uint8(0x7F)) == 0x0000
    assert orc.bfp8_decode_bits(np.uint8(0x80), np.uint8(0x7F)) == 0xFF80


def test_decoded_values_are_magnitude_times_a_power_of_two():
    # away from the wrap: value = +-mag7 * 2^(E - 133), every one a BF16 value
    d, e = np.meshgrid(np.arange(1, 128, dtype=np.uint8), np.arange(8, 255, dtype=np.uint8), indexing="ij")
    got = orc.from_bf16(orc.bfp8_decode_bits(d, e)).astype(np.float64)
    assert np.array_equal(got, np.ldexp(d.astype(np.float64), e.astype(np.int32) - 133))
    neg = orc.from_bf16(orc.bfp8_decode_bits(d | np.uint8(0x80), e)).astype(np.float64)
    assert np.array_equal(neg, -got)


def test_the_encoder_rounds_to_nearest_within_half_a_step_of_the_group():
    rng = np.random.default_rng(0xBF8)
    x = (rng.standard_normal((96, 256)) * np.exp(3 * rng.standard_normal((96, 256)))).astype(np.float32)
    x[0, :16] = 0.0
    x[1, 3] = -0.0
    x[5, :16] = np.float32(1.9999999)              # every magnitude rounds up to 128: the exponent moves up by one
    x[6, :16] = np.float32(-3.0e38)
    x[7, 16:32] = np.float32(1e-40)                # below 2^-119: stored as zeros
    d, e = orc.bfp8_encode(x)
    assert d.shape == x.shape and e.shape == (96, 16) and d.dtype == e.dtype == np.uint8
    dec = orc.bfp8_decode(d, e).astype(np.float64)
    ee = np.repeat(e, 16, axis=1).astype(np.int32)
    live = ee > 0
    step = np.ldexp(1.0, ee - 133)
    assert np.all(np.abs(dec - x.astype(np.float64))[live] <= step[live] / 2)
    assert not np.any(d == 0x80)                   # the -infinity pattern is never written for a finite value
    assert np.all(dec[0, :16] == 0) and dec[1, 3] == 0 and np.all(dec[5, :16] == 2.0) and np.all(dec[7, 16:32] == 0)
    # every group uses its range: the largest magnitude of a live group has its top bit set
    top = (d & 0x7F).reshape(96, 16, 16).max(axis=2)
    assert np.all(top[e > 0] >= 64)
    # what was decoded encodes to itself
    d2, e2 = orc.bfp8_encode(dec.astype(np.float32))
    assert np.array_equal(orc.bfp8_decode(d2, e2), dec.astype(np.float32))


def test_infinities_and_nans_survive_and_flush_their_group():
    x = np.ones((1, 32), np.float32)
    x[0, 2], x[0, 5], x[0, 9] = np.inf, -np.inf, np.nan
    d, e = orc.bfp8_encode(x)
    dec = orc.bfp8_decode(d, e)
    assert e[0, 0] == 255 and dec[0, 2] == np.inf and dec[0, 5] == -np.inf and np.isnan(dec[0, 9])
    assert np.all(dec[0, [0, 1, 3, 4]] == 0) and np.all(dec[0, 16:] == 1.0)
