"""Block-float weight storage through the C ABI: `cast_bfp` (crates/burn-tt/src/server.rs:141) against the oracle's
encoder and the reference's decoder (crates/tt-isa/src/tile.rs:619-634), and a product that reads a BFP8 weight as its B
(crates/burn-tt/src/storage.rs:117-123) against the product with the weight widened."""
import numpy as np
import pytest

from metalium_rs_b200 import BF16, BFP8, F32, EltwiseOp, TtError, kinds
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def weights(shape, seed):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal(shape) * np.exp(2 * rng.standard_normal(shape))).astype(np.float32)


@pytest.mark.parametrize("shape", [(1, 16), (37, 48), (576, 960), (1536, 576)])
@pytest.mark.parametrize("from_bf16", [False, True])
def test_cast_bfp_stores_the_oracle_s_bytes_and_widens_through_the_reference_s_decoder(eng, shape, from_bf16):
    x = weights(shape, 0xBF0 + shape[1])
    x.ravel()[:6] = [0.0, -0.0, 1.9999999, -3.0e38, 1e-40, 5e-39]
    if from_bf16:
        x = orc.from_bf16(orc.to_bf16(x))
        src = eng.upload_bf16(orc.to_bf16(x), *shape)
    else:
        src = eng.upload(x, *shape)
    packed, dims = eng.cast_bfp(src, 8)
    assert dims == shape and eng.dims_of(packed) == (shape, BFP8)
    d, e = eng.download_bfp(packed)
    want_d, want_e = orc.bfp8_encode(x)
    assert np.array_equal(d, want_d) and np.array_equal(e, want_e)
    wide, wdims = eng.cast_bfp(packed, None)                     # the trait's `None`: back to F32
    assert wdims == shape and eng.dims_of(wide)[1] == F32
    dec = eng.download(wide)
    assert np.array_equal(dec.view(np.uint32), orc.bfp8_decode(d, e).view(np.uint32))
    ee = np.repeat(e, 16, axis=1).astype(np.int32)
    live = ee > 0
    assert np.all(np.abs(dec.astype(np.float64) - x.astype(np.float64))[live] <= np.ldexp(1.0, ee - 133)[live] / 2)
    half, _ = eng.cast_bfp(packed, "bf16")                       # every decoded value is a BF16 value
    assert eng.dims_of(half)[1] == BF16 and np.array_equal(orc.from_bf16(eng.download_bf16(half)), dec)
    for i in (src, packed, wide, half):
        eng.free(i)


def test_non_finite_values_and_refusals(eng):
    x = np.ones((2, 32), np.float32)
    x[0, 2], x[0, 5], x[1, 20] = np.inf, -np.inf, np.nan
    src = eng.upload(x, 2, 32)
    packed, _ = eng.cast_bfp(src, 8)
    wide, _ = eng.cast_bfp(packed, None)
    got = eng.download(wide)
    assert np.array_equal(got.view(np.uint32), orc.bfp8_decode(*orc.bfp8_encode(x)).view(np.uint32))
    assert got[0, 2] == np.inf and got[0, 5] == -np.inf and np.isnan(got[1, 20]) and got[0, 0] == 0 and got[0, 16] == 1
    for bad in (lambda: eng.cast_bfp(src, None),                                   # not packed
                lambda: eng.cast_bfp(packed, 8),                                   # already packed
                lambda: eng.cast_bfp(eng.upload(np.ones((2, 24), np.float32), 2, 24), 8),   # not whole groups of sixteen
                lambda: eng.download(packed),                                      # packed storage is not F32
                lambda: eng.eltwise_op(EltwiseOp(kinds.RELU, 0, 0), packed),       # no op but a product and cast_bfp reads it
                lambda: eng.matmul_dram(packed, False, src, False)):               # and a product only as its B
        with pytest.raises(TtError) as ei:
            bad()
        assert ei.value.status == 2
    for i in (src, packed, wide):
        eng.free(i)


@pytest.mark.parametrize("m", [1, 2, 4])
@pytest.mark.parametrize("kn", [(576, 960), (576, 3072), (1536, 576), (576, 576)])
@pytest.mark.parametrize("out_bf16", [False, True])
def test_a_few_row_product_reads_a_bfp8_weight_where_it_lies(eng, m, kn, out_bf16):
    # a decode step's projections with the weights kept compressed: bit for bit the product with the weight widened
    k, n = kn
    a = orc.to_bf16(orc.uniform(0xBF1, 1, (m, k), -1, 1))
    w = weights((k, n), 0xBF2) * np.float32(0.02)
    ia, iw = eng.upload_bf16(a, m, k), eng.upload(w, k, n)
    packed, _ = eng.cast_bfp(iw, 8)
    wide, _ = eng.cast_bfp(packed, "bf16")
    mm = eng.matmul_dram_bf16 if out_bf16 else eng.matmul_dram
    got, dims = mm(ia, False, packed, False)
    assert dims == (m, n) and eng.last_matmul_path() == "skinny-bfp8"
    want, _ = mm(ia, False, wide, False)
    assert eng.last_matmul_path() == "skinny"
    dl = eng.download_bf16 if out_bf16 else eng.download_bits
    assert np.array_equal(dl(got), dl(want))
    # and against the F64 product of the decoded weight
    dec = orc.bfp8_decode(*eng.download_bfp(packed))
    truth, s = orc.gemm_truth(orc.from_bf16(a), dec)
    if not out_bf16:
        assert orc.gemm_rel_error(eng.download(got), truth, s)[0] <= 1e-6
    for i in (ia, iw, packed, wide, got, want):
        eng.free(i)


@pytest.mark.parametrize("a_f32", [False, True])
def test_a_taller_product_multiplies_by_the_weight_widened_for_the_call(eng, a_f32):
    m, k, n = 256, 192, 320
    a = orc.uniform(0xBF3, 1, (m, k), -1, 1)
    w = weights((k, n), 0xBF4)
    ia = eng.upload(a, m, k) if a_f32 else eng.upload_bf16(orc.to_bf16(a), m, k)
    iw = eng.upload(w, k, n)
    packed, _ = eng.cast_bfp(iw, 8)
    wide, _ = eng.cast_bfp(packed, None if a_f32 else "bf16")
    in_use = eng.device_traffic().pool_in_use
    got, dims = eng.matmul_dram(ia, False, packed, False)
    want, _ = eng.matmul_dram(ia, False, wide, False)
    assert dims == (m, n) and np.array_equal(eng.download_bits(got), eng.download_bits(want))
    eng.free(got); eng.free(want)
    assert eng.device_traffic().pool_in_use == in_use          # the widened copy lived for the call only
    for i in (ia, iw, packed, wide):
        eng.free(i)
