"""Products through the C ABI against the oracle, in the shape of
crates/tt-tests/tests/step11_burn.rs (exact on small integers :131-168, a bound on random
floats :101-111, a negative control :197-220) and step270_native_bf16.rs:462 (a BF16 product
is the F32 product rounded once)."""
import numpy as np
import pytest

from metalium_rs_b200 import BatchedLayout, CudaEngine, TtError
from oracle import oracle as orc
from tests import helpers as H

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5   # north star: F32 ops within 1e-5 relative (normalised by S = |A||B|)
BF16_TOL = 1e-2  # north star: BF16 GEMM within 1e-2 relative, FP32 accumulate


def up(eng, x, bf16=False):
    return eng.upload_bf16(orc.to_bf16(x), *x.shape) if bf16 else eng.upload(x, *x.shape)


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("sa,sb", [((32, 32), (32, 32)), ((13, 47), (47, 29)), ((1, 64), (64, 96)), ((128, 256), (256, 384)),
                                   ((200, 136), (136, 328))])
def test_small_integer_products_are_bit_exact(eng, sa, sb, bf16):
    rng = np.random.default_rng(0xB11)
    a, b = H.small_ints(rng, sa), H.small_ints(rng, sb)
    ia, ib = up(eng, a, bf16), up(eng, b, bf16)
    out, dims = (eng.matmul_dram_bf16 if bf16 else eng.matmul_dram)(ia, False, ib, False)
    assert dims == (sa[0], sb[1])
    want = (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32)
    got = orc.from_bf16(eng.download_bf16(out)) if bf16 else eng.download(out)
    if bf16:
        want = orc.from_bf16(orc.to_bf16(want))
    assert np.array_equal(got, want)
    for i in (ia, ib, out):
        eng.free(i)


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("mkn", [(64, 784, 128), (64, 128, 10), (784, 64, 128), (300, 200, 100), (512, 512, 512)])
def test_f32_products_hold_f32_accuracy(eng, mkn, ta, tb):
    m, k, n = mkn
    a = orc.uniform(0xC0F2, 1, (k, m) if ta else (m, k), -1, 1)
    b = orc.uniform(0xC0F2, 2, (n, k) if tb else (k, n), -1, 1)
    ia, ib = up(eng, a), up(eng, b)
    out, dims = eng.matmul_dram(ia, ta, ib, tb)
    assert dims == (m, n)
    got = eng.download(out)
    truth, s = orc.gemm_truth(a, b, ta, tb)
    e_s, e_t = orc.gemm_rel_error(got, truth, s)
    cpu = orc.gemm_f32(a, b, ta, tb)
    c_s, _ = orc.gemm_rel_error(cpu, truth, s)
    assert e_s <= F32_TOL, (e_s, c_s)
    assert e_s <= 4 * c_s + 2 ** -20  # never far from the CPU restatement's own rounding (the split path drops a_lo b_lo)
    for i in (ia, ib, out):
        eng.free(i)


def test_f32_negative_control(eng):  # step11_burn.rs:197-220: a BF16-grade product must fail the F32 bound
    a = orc.uniform(0xC0F2, 3, (256, 256), -1, 1)
    b = orc.uniform(0xC0F2, 4, (256, 256), -1, 1)
    truth, s = orc.gemm_truth(a, b)
    lo = orc.from_bf16(orc.to_bf16(a)).astype(np.float64) @ orc.from_bf16(orc.to_bf16(b)).astype(np.float64)
    e_s, _ = orc.gemm_rel_error(lo, truth, s)
    assert e_s > F32_TOL


TC_SHAPES = [(128, 64, 128), (256, 512, 384), (384, 192, 640), (200, 136, 328), (1024, 1024, 1024), (64, 64, 64), (4096, 576, 576),
             (130, 72, 1536)]


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("mkn", TC_SHAPES)
def test_bf16_products_take_the_tensor_cores_and_round_once(eng, mkn, ta, tb):
    m, k, n = mkn
    a = orc.to_bf16(orc.uniform(0xC0F2, 5, (k, m) if ta else (m, k), -1, 1))
    b = orc.to_bf16(orc.uniform(0xC0F2, 6, (n, k) if tb else (k, n), -1, 1))
    ia = eng.upload_bf16(a, *a.shape)
    ib = eng.upload_bf16(b, *b.shape)
    out, dims = eng.matmul_dram_bf16(ia, ta, ib, tb)
    assert dims == (m, n)
    aligned = (a.shape[1] % 8 == 0) and (b.shape[1] % 8 == 0)
    assert eng.last_matmul_path() == ("tcgen05" if aligned else "simt")
    got_bits = eng.download_bf16(out)
    want_bits, truth, s = orc.gemm_bf16(a, b, ta, tb)
    got = orc.from_bf16(got_bits)
    e_s, e_t = orc.gemm_rel_error(got, truth, s)
    assert e_s <= BF16_TOL and e_t <= BF16_TOL, (e_s, e_t)
    # the F32 product rounded once: within one BF16 step of the truth plus the F32 sum's own
    # rounding (which matters only where the sum cancels), and the same bits almost everywhere
    step = np.abs(got_bits.astype(np.int32) - want_bits.astype(np.int32))
    assert np.all(np.abs(got.astype(np.float64) - truth) <= 2.0 ** -8 * np.abs(truth) + 1e-6 * s)
    assert (step == 0).mean() > 0.95 and (step <= 1).mean() > 0.999
    # F32 result of BF16 operands
    o32, _ = eng.matmul_dram(ia, ta, ib, tb)
    e32, _ = orc.gemm_rel_error(eng.download(o32), truth, s)
    assert e32 <= 1e-5
    for i in (ia, ib, out, o32):
        eng.free(i)


def test_tensor_core_and_simt_paths_agree(lib):
    a = orc.to_bf16(orc.normal(0xC0F5, 1, (512, 256)))
    b = orc.to_bf16(orc.normal(0xC0F5, 2, (256, 320)))
    res = []
    for mode in (1, 2):
        with CudaEngine(0, bf16_matmul_mode=mode) as e:
            ia, ib = e.upload_bf16(a, 512, 256), e.upload_bf16(b, 256, 320)
            out, _ = e.matmul_dram(ia, False, ib, False)
            res.append(e.download(out))
            assert e.last_matmul_path() == ("simt" if mode == 1 else "tcgen05")
    truth, s = orc.gemm_truth(orc.from_bf16(a), orc.from_bf16(b))
    for r in res:
        assert orc.gemm_rel_error(r, truth, s)[0] <= 1e-6


def test_the_tensor_core_only_mode_refuses_what_it_cannot_take(lib):
    with CudaEngine(0, bf16_matmul_mode=2) as e:
        a = e.upload_bf16(np.zeros((13, 47), np.uint16), 13, 47)
        b = e.upload_bf16(np.zeros((47, 29), np.uint16), 47, 29)
        with pytest.raises(TtError) as ei:
            e.matmul_dram_bf16(a, False, b, False)
        assert ei.value.status == 2


def test_mismatched_inner_dimensions_are_refused(eng):
    a, b = eng.upload(np.zeros((4, 5), np.float32), 4, 5), eng.upload(np.zeros((6, 4), np.float32), 6, 4)
    with pytest.raises(TtError):
        eng.matmul_dram(a, False, b, False)
    out, dims = eng.matmul_dram(a, True, b, True)  # [5,4] x [4,6]
    assert dims == (5, 6)
    for i in (a, b, out):
        eng.free(i)


def test_host_staged_matmul(eng):  # server.rs:70
    a, b = orc.uniform(1, 1, (33, 65), -1, 1), orc.uniform(1, 2, (65, 17), -1, 1)
    got = eng.matmul(a, b, (33, 65, 17))
    truth, s = orc.gemm_truth(a, b)
    assert orc.gemm_rel_error(got, truth, s)[0] <= F32_TOL


@pytest.mark.parametrize("bf16", [False, True])
def test_batched_products_read_blocks_where_they_lie(eng, bf16):
    # heads side by side in one buffer: Q [t, heads*hd] blocks at column h*hd; K^T read as a
    # transposed block (server.rs:229; ops.rs:3008-3081)
    t, heads, hd = 128, 4, 64
    q = orc.normal(0xC0F5, 3, (t, heads * hd))
    kx = orc.normal(0xC0F5, 4, (t, heads * hd))
    if bf16:
        q, kx = orc.from_bf16(orc.to_bf16(q)), orc.from_bf16(orc.to_bf16(kx))
    iq, ik = up(eng, q, bf16), up(eng, kx, bf16)
    items = [(((0, h * hd), False), ((0, h * hd), True)) for h in range(heads)]
    out, dims = eng.matmul_dram_batched(iq, ik, items, (t, hd, t), bf16=False)
    assert dims == (heads * t, t)
    got = eng.download(out)
    for h in range(heads):
        truth, s = orc.gemm_truth(q[:, h * hd:(h + 1) * hd], kx[:, h * hd:(h + 1) * hd], False, True)
        assert orc.gemm_rel_error(got[h * t:(h + 1) * t], truth, s)[0] <= F32_TOL, h
    if bf16:
        assert eng.last_matmul_path() == "tcgen05"
    # P.V: [t,t] blocks stacked in rows x V blocks by column
    p = eng.download(out)
    if bf16:
        p = orc.from_bf16(orc.to_bf16(p))
    ip = up(eng, p, bf16)
    items2 = [(((h * t, 0), False), ((0, h * hd), False)) for h in range(heads)]
    o2, dims2 = eng.matmul_dram_batched(ip, ik, items2, (t, t, hd), bf16=False)
    assert dims2 == (heads * t, hd)
    g2 = eng.download(o2)
    for h in range(heads):
        truth, s = orc.gemm_truth(p[h * t:(h + 1) * t], kx[:, h * hd:(h + 1) * hd])
        assert orc.gemm_rel_error(g2[h * t:(h + 1) * t], truth, s)[0] <= F32_TOL, h
    for i in (iq, ik, out, ip, o2):
        eng.free(i)


def test_unstacked_layout_places_each_product_on_a_tile_row(eng):  # server.rs:3749-3754
    m, k, n, items_n = 20, 40, 33, 3
    a = orc.uniform(2, 1, (items_n * 32, k), -1, 1)
    b = orc.uniform(2, 2, (k, items_n * n), -1, 1)
    ia, ib = up(eng, a), up(eng, b)
    items = [(((i * 32, 0), False), ((0, i * n), False)) for i in range(items_n)]
    out, dims = eng.matmul_dram_batched_layout(ia, ib, items, (m, k, n), BatchedLayout(1, 0))
    assert dims == (items_n * 32, n)
    got = eng.download(out)
    for i in range(items_n):
        truth, s = orc.gemm_truth(a[i * 32:i * 32 + m], b[:, i * n:(i + 1) * n])
        assert orc.gemm_rel_error(got[i * 32:i * 32 + m], truth, s)[0] <= F32_TOL
    st, dims = eng.matmul_dram_batched(ia, ib, items, (m, k, n))
    assert dims == (items_n * m, n)
    assert np.array_equal(eng.download(st), np.concatenate([got[i * 32:i * 32 + m] for i in range(items_n)]))
    for i in (ia, ib, out, st):
        eng.free(i)


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("mkn", [(2048, 2048, 2048), (4096, 1024, 2304), (2304, 4096, 2048)])
def test_the_pair_kernel_with_every_operand_order(eng, mkn, ta, tb):
    # From 64 tiles of 256 x 256 one product takes the CTA-pair kernel, whose four instantiations differ in the TMA
    # boxes and the shared-memory descriptors of an MN-major operand (A^T B and A B^T: weight gradients, a tied head;
    # crates/tt-tests/tests/step11_burn.rs:157-166 gates A B^T).  Too large for the whole F64 product in seconds: the
    # row-sum identity C 1 = op(A) (op(B) 1) on every row, and 256 sampled elements against F64 dot products.
    m, k, n = mkn
    a = orc.to_bf16(orc.uniform(0xC0F2, 21, (k, m) if ta else (m, k), -1, 1))
    b = orc.to_bf16(orc.uniform(0xC0F2, 22, (n, k) if tb else (k, n), -1, 1))
    ia, ib = eng.upload_bf16(a, *a.shape), eng.upload_bf16(b, *b.shape)
    out, dims = eng.matmul_dram(ia, ta, ib, tb)              # F32 result keeps the identity tight
    assert dims == (m, n) and eng.last_matmul_path() == "tcgen05-pair"
    c = eng.download(out).astype(np.float64)
    af, bf = orc.from_bf16(a).astype(np.float64), orc.from_bf16(b).astype(np.float64)
    la, lb = (af.T if ta else af), (bf.T if tb else bf)      # the logical operands
    rows = la @ lb.sum(1)
    s_rows = np.abs(la) @ np.abs(lb).sum(1)
    assert np.max(np.abs(c.sum(1) - rows) / s_rows) <= 1e-6
    cols = la.sum(0) @ lb                                     # and 1^T C = (1^T op(A)) op(B): every column
    s_cols = np.abs(la).sum(0) @ np.abs(lb)
    assert np.max(np.abs(c.sum(0) - cols) / s_cols) <= 1e-6
    rng = np.random.default_rng(11)
    for i, j in zip(rng.integers(0, m, 256), rng.integers(0, n, 256)):
        t = la[i] @ lb[:, j]
        s_ = np.abs(la[i]) @ np.abs(lb[:, j])
        assert abs(c[i, j] - t) <= 1e-6 * s_, (i, j)
    ob, _ = eng.matmul_dram_bf16(ia, ta, ib, tb)             # the BF16 result is that accumulator rounded once
    assert eng.last_matmul_path() == "tcgen05-pair"
    assert np.array_equal(eng.download_bf16(ob), orc.to_bf16(c.astype(np.float32)))
    for i in (ia, ib, out, ob):
        eng.free(i)


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("mkn,a_at,a_t,b_at,b_t", [
    ((128, 64, 128), (0, 0), False, (0, 0), True),            # one head's Q K^T: item ((0,0),False), ((0,0),True)
    ((256, 320, 384), (64, 128), False, (32, 256), False),    # blocks at a non-zero row and column
    ((256, 256, 256), (128, 64), True, (64, 0), True),        # both stored transposed
    ((2048, 256, 2048), (0, 256), False, (256, 0), True),     # large enough for the pair kernel (BF16)
    ((96, 72, 80), (8, 16), False, (24, 40), False),          # k not a multiple of 64
])
def test_a_batched_call_of_one_item_is_that_item_s_product(eng, bf16, mkn, a_at, a_t, b_at, b_t):
    # One (Block, Block) pair (server.rs:229): the block offsets and transposed flags of the single item decide
    # what is multiplied, on every kernel path.
    m, k, n = mkn
    ar, ac = (k, m) if a_t else (m, k)
    br, bc = (n, k) if b_t else (k, n)
    big_a = orc.uniform(0xC0FA, 1, (a_at[0] + ar + 32, a_at[1] + ac + 64), -1, 1)
    big_b = orc.uniform(0xC0FA, 2, (b_at[0] + br + 32, b_at[1] + bc + 64), -1, 1)
    if bf16:
        big_a, big_b = orc.from_bf16(orc.to_bf16(big_a)), orc.from_bf16(orc.to_bf16(big_b))
    ia, ib = up(eng, big_a, bf16), up(eng, big_b, bf16)
    out, dims = eng.matmul_dram_batched(ia, ib, [((a_at, a_t), (b_at, b_t))], mkn, bf16=False)
    assert dims == (m, n)
    got = eng.download(out)
    sa = big_a[a_at[0]:a_at[0] + ar, a_at[1]:a_at[1] + ac]
    sb = big_b[b_at[0]:b_at[0] + br, b_at[1]:b_at[1] + bc]
    truth, s_ = orc.gemm_truth(np.ascontiguousarray(sa), np.ascontiguousarray(sb), a_t, b_t)
    assert orc.gemm_rel_error(got, truth, s_)[0] <= (1e-6 if bf16 else F32_TOL)
    if bf16 and k % 64 == 0:
        assert eng.last_matmul_path().startswith("tcgen05")
    if not bf16 and min(m, k, n) >= 256:
        assert eng.last_matmul_path() == "tcgen05-tf32x3"
    for i in (ia, ib, out):
        eng.free(i)


def test_bf16_product_at_4096_by_properties(eng):
    # Too large for the F64 oracle in seconds: check the row-sum identity C 1 = A (B 1) and
    # 64 sampled elements against F64 dot products.
    n = 4096
    a = orc.to_bf16(orc.uniform(0xC0F2, 7, (n, n), -1, 1))
    b = orc.to_bf16(orc.uniform(0xC0F2, 8, (n, n), -1, 1))
    ia, ib = eng.upload_bf16(a, n, n), eng.upload_bf16(b, n, n)
    out, _ = eng.matmul_dram(ia, False, ib, False)  # F32 result keeps the identity tight
    assert eng.last_matmul_path() == "tcgen05-pair"  # 256 tiles of 256 x 256: the CTA-pair kernel
    c = eng.download(out).astype(np.float64)
    af, bf = orc.from_bf16(a).astype(np.float64), orc.from_bf16(b).astype(np.float64)
    rows = af @ bf.sum(1)
    s_rows = np.abs(af) @ np.abs(bf).sum(1)
    assert np.max(np.abs(c.sum(1) - rows) / s_rows) <= 1e-6
    rng = np.random.default_rng(5)
    for i, j in zip(rng.integers(0, n, 64), rng.integers(0, n, 64)):
        t = af[i] @ bf[:, j]
        s = np.abs(af[i]) @ np.abs(bf[:, j])
        assert abs(c[i, j] - t) <= 1e-6 * s
    ob, _ = eng.matmul_dram_bf16(ia, False, ib, False)
    assert np.array_equal(eng.download_bf16(ob), orc.to_bf16(c.astype(np.float32)))
    for i in (ia, ib, out, ob):
        eng.free(i)


@pytest.mark.parametrize("m", [3, 8, 33])
def test_short_m_products_take_the_tensor_cores(eng, m):
    # a prefill's head: a few rows against a [vocab, hidden] table read transposed
    a = orc.to_bf16(orc.uniform(0xC0F4, 20, (m, 576), -1, 1))
    table = orc.to_bf16(orc.normal(0xC0F4, 21, (4096, 576), 0.02))
    ia, it = eng.upload_bf16(a, m, 576), eng.upload_bf16(table, 4096, 576)
    out, dims = eng.matmul_dram(ia, False, it, True)
    assert dims == (m, 4096) and eng.last_matmul_path() == "tcgen05"
    truth, s = orc.gemm_truth(orc.from_bf16(a), orc.from_bf16(table), False, True)
    assert orc.gemm_rel_error(eng.download(out), truth, s)[0] <= 1e-6
    for i in (ia, it, out):
        eng.free(i)


@pytest.mark.parametrize("mkn", [(2048, 512, 768), (1500, 640, 520), (3000, 256, 256), (64, 64, 64), (5, 576, 960)])
def test_the_host_staged_bf16_product_is_the_resident_one(eng, mkn):  # server.rs:70 `matmul`, for BF16 operands
    m, k, n = mkn
    a = orc.to_bf16(orc.uniform(0xC0F7, 1, (m, k), -1, 1))
    b = orc.to_bf16(orc.uniform(0xC0F7, 2, (k, n), -1, 1))
    got = eng.matmul_bf16(a, b, mkn)                      # uploaded, multiplied and downloaded in row panels
    ia, ib = eng.upload_bf16(a, m, k), eng.upload_bf16(b, k, n)
    out, _ = eng.matmul_dram_bf16(ia, False, ib, False)
    assert np.array_equal(got, eng.download_bf16(out))    # K is whole in every panel: the same sums, the same bits
    _, truth, s = orc.gemm_bf16(a, b, False, False)
    assert np.all(np.abs(orc.from_bf16(got).astype(np.float64) - truth) <= 2.0 ** -8 * np.abs(truth) + 1e-6 * s)
    for i in (ia, ib, out):
        eng.free(i)


@pytest.mark.parametrize("mkn,first,width", [((512, 256, 384), 128, 640), ((300, 192, 200), 64, 328), ((256, 128, 256), 8, 272)])
def test_a_product_stored_into_several_matrices_at_a_column(eng, mkn, first, width):
    # the sharded product's fused step (crates/tt-kernels/src/shard.rs:348-458) with both "ranks" on one GPU:
    # the slice lands at its columns of every destination, the same bits as the product on its own
    m, k, n = mkn
    a = orc.to_bf16(orc.uniform(0xC0F8, 1, (m, k), -1, 1))
    b = orc.to_bf16(orc.uniform(0xC0F8, 2, (k, n), -1, 1))
    ia, ib = eng.upload_bf16(a, m, k), eng.upload_bf16(b, k, n)
    alone, _ = eng.matmul_dram_bf16(ia, False, ib, False)
    want = eng.download_bf16(alone)
    fill = np.full((m, width), 0x7fc0, np.uint16)
    c0, c1 = eng.upload_bf16(fill, m, width), eng.upload_bf16(fill, m, width)
    ptrs = [eng.device_ptr(c0)[0], eng.device_ptr(c1)[0]]
    eng.matmul_into(ia, ib, ptrs, (m, width), first)
    for c in (c0, c1):
        got = eng.download_bf16(c)
        assert np.array_equal(got[:, first:first + n], want)
        assert np.all(got[:, :first] == 0x7fc0) and np.all(got[:, first + n:] == 0x7fc0)   # nothing else is touched
    # a block of a buffer stored the same way (an activation's slice of an all-gather)
    eng.store_block_into((alone, (0, 0), (m, n)), ptrs[:1], (m, width), width - n)
    got = eng.download_bf16(c0)
    assert np.array_equal(got[:, width - n:], want)
    with pytest.raises(TtError):
        eng.matmul_into(ia, ib, ptrs, (m, width), width - n + 8)      # the slice would end past the last column
    for i in (ia, ib, alone, c0, c1):
        eng.free(i)


@pytest.mark.parametrize("mkf", [(4096, 576, 1536), (256, 128, 256), (300, 64, 128), (130, 192, 640)])
def test_the_gated_product_is_the_product_then_silu_mul_bit_for_bit(eng, mkf):   # tt-models/src/llama.rs:498
    from metalium_rs_b200 import EltwiseOp, kinds, workloads as W
    m, k, ff = mkf
    a = orc.to_bf16(orc.normal(0xC0F9, 1, (m, k), 1.0))
    w = orc.to_bf16(orc.normal(0xC0F9, 2, (k, 2 * ff), 0.2))              # gate | up side by side
    ia, iw = eng.upload_bf16(a, m, k), eng.upload_bf16(w, k, 2 * ff)
    iwi = eng.upload_bf16(W.interleave_gate_up(w), k, 2 * ff)
    gu, _ = eng.matmul_dram_bf16(ia, False, iw, False)
    want, _ = eng.eltwise_blocks_as(EltwiseOp(kinds.SILU_MUL, 0.0, 0.0), (gu, (0, 0), (m, ff)), (gu, (0, ff), (m, ff)), None, True)
    got, dims = eng.matmul_silu_mul(ia, iwi)
    assert dims == (m, ff) and eng.last_matmul_path() == ("tcgen05-pair" if m >= 4096 else "tcgen05")
    assert np.array_equal(eng.download_bf16(got), eng.download_bf16(want))
    with pytest.raises(TtError):
        eng.matmul_silu_mul(ia, eng.upload_bf16(w[:, :2 * ff - 8], k, 2 * ff - 8))   # not whole groups of 256 columns
    for i in (ia, iw, iwi, gu, want, got):
        eng.free(i)


@pytest.mark.parametrize("mknr", [(4096, 576, 960, 768, 512),    # the prefill's fused QKV projection: the CTA-pair kernel
                                  (256, 576, 960, 768, 128),     # the single-CTA kernel, tiles that end inside the key heads
                                  (384, 128, 192, 192, 384),     # every column rotated, a table row a product row
                                  (130, 64, 320, 64, 65)])       # one head rotated, rows that are not whole tiles
def test_the_projection_with_rope_is_the_product_then_rope_blocks_bit_for_bit(eng, mknr):   # tt-models/src/llama.rs:404-433
    from metalium_rs_b200 import workloads as W
    m, k, n, rope_cols, r = mknr
    a = orc.to_bf16(orc.normal(0xC0FA, 1, (m, k), 1.0))
    w = orc.to_bf16(orc.normal(0xC0FA, 2, (k, n), 0.2))
    cos, sin = W.rope_tables(r, 64, 10000.0)
    ia, iw = eng.upload_bf16(a, m, k), eng.upload_bf16(w, k, n)
    ic, isn = eng.upload(cos, r, 64), eng.upload(sin, r, 64)
    plain, _ = eng.matmul_dram_bf16(ia, False, iw, False)
    rot, _ = eng.rope_blocks((plain, (0, 0), (m, rope_cols)), (ic, (0, 0), (r, 64)), (isn, (0, 0), (r, 64)), 64, True)
    got, dims = eng.matmul_rope(ia, iw, (ic, (0, 0), (r, 64)), (isn, (0, 0), (r, 64)), rope_cols)
    assert dims == (m, n) and eng.last_matmul_path() == ("tcgen05-pair" if m >= 4096 else "tcgen05")
    g = eng.download_bf16(got)
    assert np.array_equal(g[:, :rope_cols], eng.download_bf16(rot))              # the rotated heads
    assert np.array_equal(g[:, rope_cols:], eng.download_bf16(plain)[:, rope_cols:])   # the rest as the product leaves them
    for bad in (rope_cols + 8, n + 64):
        with pytest.raises(TtError):
            eng.matmul_rope(ia, iw, (ic, (0, 0), (r, 64)), (isn, (0, 0), (r, 64)), bad)
    with pytest.raises(TtError):                                                  # a table whose rows do not divide the product's
        eng.matmul_rope(ia, iw, (ic, (0, 0), (r - 1, 64)), (isn, (0, 0), (r - 1, 64)), rope_cols)
    for i in (ia, iw, ic, isn, plain, rot, got):
        eng.free(i)


@pytest.mark.parametrize("mkn", [(4096, 576, 576),      # the prefill's output projection: three CTAs a row panel
                                 (4096, 1536, 576),     # its down projection
                                 (200, 576, 576),       # rows that are not whole tiles
                                 (256, 512, 768),       # four CTAs a panel
                                 (128, 64, 192),        # one CTA a panel, one k-block
                                 (300, 320, 1536)])     # eight CTAs a panel
def test_the_projection_into_the_residual_and_its_norm(eng, mkn):   # tt-models/src/llama.rs:371-507
    # `matmul_add_rms_norm` against the composition it replaces: `matmul_dram` (F32 product of BF16 operands), then
    # `add_rms_norm_as(resid, product, gains, eps, bf16)`.  The sum is that composition's bit for bit (the same product,
    # one F32 addition).  The norm's statistic is summed in another fixed order, so a quotient may round the other way:
    # held to one BF16 step, with nearly every element equal.
    m, k, n = mkn
    a = orc.to_bf16(orc.normal(0xADD0, 1, (m, k), 1.0))
    w = orc.to_bf16(orc.normal(0xADD0, 2, (k, n), 0.05))
    resid = orc.normal(0xADD0, 3, (m, n), 1.0).astype(np.float32)
    gains = orc.to_bf16(1.0 + orc.normal(0xADD0, 4, (1, n), 0.1))
    ia, iw, ir, ig = eng.upload_bf16(a, m, k), eng.upload_bf16(w, k, n), eng.upload(resid, m, n), eng.upload_bf16(gains, 1, n)
    prod, _ = eng.matmul_dram(ia, False, iw, False)
    (s_want, _), (n_want, _) = eng.add_rms_norm_as(ir, prod, ig, 1e-5, True)
    (s_got, d0), (n_got, d1) = eng.matmul_add_rms_norm(ia, iw, ir, ig, 1e-5)
    assert d0 == d1 == (m, n) and eng.last_matmul_path() == "tcgen05-addnorm"
    assert np.array_equal(eng.download(s_got).view(np.uint32), eng.download(s_want).view(np.uint32))
    got, want = eng.download_bf16(n_got).astype(np.int32), eng.download_bf16(n_want).astype(np.int32)
    step = np.abs(got - want)
    assert step.max() <= 1 and (step == 0).mean() > 0.99, (int(step.max()), float((step == 0).mean()))
    # against F64: the norm of the F32 sum, to BF16's half step and the F32 statistic's rounding
    s64 = eng.download(s_got).astype(np.float64)
    ref = s64 / np.sqrt((s64 * s64).mean(axis=1, keepdims=True) + 1e-5) * orc.from_bf16(gains).astype(np.float64)
    assert np.all(np.abs(orc.from_bf16(eng.download_bf16(n_got)).astype(np.float64) - ref) <= 2.0 ** -8 * np.abs(ref) + 1e-6)
    for bad in (lambda: eng.matmul_add_rms_norm(ia, iw, ir, iw, 1e-5),          # gains of the wrong length
                lambda: eng.matmul_add_rms_norm(ia, iw, prod, ia, 1e-5),
                lambda: eng.matmul_add_rms_norm(iw, ia, ir, ig, 1e-5)):         # shapes that do not meet
        with pytest.raises(TtError):
            bad()
    for i in (ia, iw, ir, ig, prod, s_want, n_want, s_got, n_got):
        eng.free(i)


@pytest.mark.parametrize("m", [1, 2, 3, 4])
@pytest.mark.parametrize("kn", [(576, 960), (576, 576), (576, 3072), (1536, 576), (100, 72), (5000, 8)])
def test_a_handful_of_rows_streams_the_weights_once(eng, m, kn):
    # a decode step's projections: [m, k] x [k, n], both as stored.  Same claims as the tensor-core path.
    k, n = kn
    a = orc.to_bf16(orc.uniform(0xC0F6, 1, (m, k), -1, 1))
    b = orc.to_bf16(orc.uniform(0xC0F6, 2, (k, n), -1, 1))
    ia, ib = eng.upload_bf16(a, m, k), eng.upload_bf16(b, k, n)
    out, dims = eng.matmul_dram_bf16(ia, False, ib, False)
    assert dims == (m, n) and eng.last_matmul_path() == "skinny"
    want_bits, truth, s = orc.gemm_bf16(a, b, False, False)
    got_bits = eng.download_bf16(out)
    got = orc.from_bf16(got_bits)
    assert np.all(np.abs(got.astype(np.float64) - truth) <= 2.0 ** -8 * np.abs(truth) + 1e-6 * s)
    step = np.abs(got_bits.astype(np.int32) - want_bits.astype(np.int32))
    assert (step <= 1).mean() > 0.999
    o32, _ = eng.matmul_dram(ia, False, ib, False)
    assert eng.last_matmul_path() == "skinny"
    assert orc.gemm_rel_error(eng.download(o32), truth, s)[0] <= 1e-6
    for i in (ia, ib, out, o32):
        eng.free(i)


@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("kn", [(576, 49152), (576, 2048), (64, 1024), (1536, 4100)])
def test_one_or_two_rows_against_a_table_stored_by_rows(eng, m, kn):   # tt-models/src/llama.rs:1090: the tied head
    # logits = x table^T: [m, k] x ([n, k])^T with B as stored.  The same claims as above; past two rows, or a short
    # table, the tensor-core tile takes it.
    k, n = kn
    a = orc.to_bf16(orc.uniform(0xC0F8, 1, (m, k), -1, 1))
    b = orc.to_bf16(orc.uniform(0xC0F8, 2, (n, k), -1, 1))
    ia, ib = eng.upload_bf16(a, m, k), eng.upload_bf16(b, n, k)
    o32, dims = eng.matmul_dram(ia, False, ib, True)
    assert dims == (m, n) and eng.last_matmul_path() == "skinny"
    af, bf = orc.from_bf16(a).astype(np.float64), orc.from_bf16(b).astype(np.float64)
    truth = af @ bf.T
    s = np.abs(af) @ np.abs(bf).T
    assert np.all(np.abs(eng.download(o32).astype(np.float64) - truth) <= 1e-6 * s)
    out, _ = eng.matmul_dram_bf16(ia, False, ib, True)
    assert eng.last_matmul_path() == "skinny"
    got = orc.from_bf16(eng.download_bf16(out)).astype(np.float64)
    assert np.all(np.abs(got - truth) <= 2.0 ** -8 * np.abs(truth) + 1e-6 * s)
    for i in (ia, ib, out, o32):
        eng.free(i)


def test_a_tensor_only_engine_never_takes_the_skinny_kernel(lib):
    a = orc.to_bf16(orc.uniform(0xC0F6, 3, (4, 576), -1, 1))
    b = orc.to_bf16(orc.uniform(0xC0F6, 4, (576, 576), -1, 1))
    with CudaEngine(0, bf16_matmul_mode=2) as e:
        ia, ib = e.upload_bf16(a, 4, 576), e.upload_bf16(b, 576, 576)
        out, _ = e.matmul_dram_bf16(ia, False, ib, False)
        assert e.last_matmul_path() == "tcgen05"
        tc = e.download_bf16(out)
    with CudaEngine(0) as e:
        ia, ib = e.upload_bf16(a, 4, 576), e.upload_bf16(b, 576, 576)
        out, _ = e.matmul_dram_bf16(ia, False, ib, False)
        assert e.last_matmul_path() == "skinny"
        sk = e.download_bf16(out)
    step = np.abs(tc.astype(np.int32) - sk.astype(np.int32))
    assert (step <= 1).all() and (step == 0).mean() > 0.98


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("mkn", [(256, 256, 256), (384, 160, 512), (1024, 1024, 1024), (200, 132, 328)])
def test_f32_products_on_the_split_tf32_tensor_path(lib, mkn, ta, tb):
    # a = a_hi + a_lo in TF32, three products, FP32 accumulation: F32-grade, not TF32-grade
    m, k, n = mkn
    a = orc.uniform(0xC0F2, 11, (k, m) if ta else (m, k), -1, 1)
    b = orc.uniform(0xC0F2, 12, (n, k) if tb else (k, n), -1, 1)
    with CudaEngine(0, f32_matmul_mode=2) as e:
        ia, ib = e.upload(a, *a.shape), e.upload(b, *b.shape)
        out, dims = e.matmul_dram(ia, ta, ib, tb)
        assert dims == (m, n) and e.last_matmul_path() == "tcgen05-tf32x3"
        got = e.download(out)
    truth, s = orc.gemm_truth(a, b, ta, tb)
    e_s, _ = orc.gemm_rel_error(got, truth, s)
    assert e_s <= 2e-6, e_s                        # far inside the contract's 1e-5
    tf32 = lambda x: (x.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)
    lo, _ = orc.gemm_rel_error(orc.gemm_truth(tf32(a), tf32(b), ta, tb)[0], truth, s)
    assert lo > 10 * e_s                           # negative control: one TF32 product is far worse (step11_burn.rs:197-220)


def test_split_tf32_path_is_exact_on_small_integers_and_chosen_automatically(eng):
    rng = np.random.default_rng(3)
    a, b = H.small_ints(rng, (512, 320)), H.small_ints(rng, (320, 640))
    ia, ib = eng.upload(a, 512, 320), eng.upload(b, 320, 640)
    out, _ = eng.matmul_dram(ia, False, ib, False)
    assert eng.last_matmul_path() == "tcgen05-tf32x3"
    assert np.array_equal(eng.download(out), (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32))
    small, _ = eng.matmul_dram(ia, True, ia, False)   # [320,512]x[512,320]: still large enough
    for i in (ia, ib, out, small):
        eng.free(i)


@pytest.mark.parametrize("mkn,stored_b,tb", [((64, 784, 128), True, False), ((33, 70, 50), True, True), ((512, 576, 1536), True, False),
                                              ((48, 96, 40), False, False)])
def test_a_weight_kept_in_bf16_storage_multiplies_as_its_widened_self(eng, mkn, stored_b, tb):
    # crates/burn-tt/src/server.rs:150-158, crates/tt-kernels/src/session.rs:3751-3756: bit for bit the F32 product
    m, k, n = mkn
    a = orc.uniform(0xB16, 1, (m, k), -1.0, 1.0)
    b = orc.uniform(0xB16, 2, (n, k) if tb else (k, n), -1.0, 1.0)
    ia, ib = eng.upload(a, *a.shape), eng.upload(b, *b.shape)
    which = ib if stored_b else ia
    stored, sd = eng.cast_bf16_storage(which, True)
    wide, wd = eng.cast_bf16_storage(stored, False)
    assert sd == wd
    if stored_b:
        mixed, dims = eng.matmul_dram(ia, False, stored, tb)
        plain, _ = eng.matmul_dram(ia, False, wide, tb)
    else:
        mixed, dims = eng.matmul_dram(stored, False, ib, tb)
        plain, _ = eng.matmul_dram(wide, False, ib, tb)
    assert dims == (m, n) and np.array_equal(eng.download_bits(mixed), eng.download_bits(plain))
    for i in (ia, ib, stored, wide, mixed, plain):
        eng.free(i)
