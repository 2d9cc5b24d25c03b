"""The engine's host logic without a GPU: engine.cu compiled with g++ against a host-only
stand-in for the CUDA runtime (tests/fake_cuda), every kernel launch a no-op.  Checked here:
result dims of every op (burn-tt fails an op whose dims differ from its own prediction,
crates/burn-tt/src/server.rs:2963-2972), refusals, buffer-id safety
(crates/burn-tt/tests/stale_buffer.rs), views, the pool, out-of-memory reports, the path
choice of products and the trace state machine -- with failures injected on the host only."""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np
import pytest

from metalium_rs_b200 import (BF16, BOOL, COLS, F32, I32, MAX, ROWS, SUM, BatchedLayout, CudaEngine, EltwiseOp, TtError,
                              kinds)

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def fake():
    out = ROOT / "tests" / "_build" / "libb200tt_fake.so"
    out.parent.mkdir(exist_ok=True)
    srcs = [ROOT / "metalium_rs_b200" / "csrc" / "engine.cu", ROOT / "tests" / "fake_cuda" / "fake_kernels.cpp"]
    subprocess.run(["g++", "-std=c++17", "-O1", "-fPIC", "-shared", "-x", "c++", "-I", str(ROOT / "tests" / "fake_cuda"),
                    "-I", str(ROOT / "metalium_rs_b200" / "csrc"), *map(str, srcs), "-o", str(out)], check=True)
    return C.CDLL(str(out))


@pytest.fixture()
def e(fake):
    C.c_uint64.in_dll(fake, "fake_cuda_memory_limit").value = 0
    C.c_int.in_dll(fake, "fake_tc_supported").value = 1
    eng = CudaEngine(0, lib=fake)
    yield eng
    eng.close()


def f32(e, r, c):
    return e.upload(np.arange(r * c, dtype=np.float32).reshape(r, c), r, c)


def test_storage_round_trips_and_ids(e):
    x = np.arange(12, dtype=np.float32).reshape(3, 4)
    i = e.upload(x, 3, 4)
    assert np.array_equal(e.download(i), x) and e.dims_of(i) == ((3, 4), F32)
    j = e.upload(x, 3, 4)
    assert j != i                                   # ids are unique within an engine
    e.free(i); e.free(i); e.free(987654)            # unknown ids: no-ops (server.rs:174)
    with pytest.raises(TtError) as err:
        e.download(i)
    assert err.value.status == 5                    # StaleTensor
    h = e.upload_bf16(np.arange(6, dtype=np.uint16).reshape(2, 3), 2, 3)
    assert e.dims_of(h) == ((2, 3), BF16)
    with pytest.raises(TtError):
        e.download(h)                               # not F32
    with pytest.raises(TtError):
        e.upload_bits(np.zeros((1, 1), np.uint32), 1, 1, BF16)


def test_result_dims_of_every_op(e):
    a, b = f32(e, 64, 96), f32(e, 96, 32)
    assert e.matmul_dram(a, False, b, False)[1] == (64, 32)
    assert e.matmul_dram(a, True, a, False)[1] == (96, 96)
    assert e.matmul_dram(b, True, a, True)[1] == (32, 64)
    with pytest.raises(TtError):
        e.matmul_dram(a, False, a, False)
    row, col, blk = f32(e, 1, 96), f32(e, 64, 1), f32(e, 32, 96)
    for other in (a, row, col, blk):
        assert e.eltwise_op(EltwiseOp(kinds.ADD, 0, 0), a, other)[1] == (64, 96)
    assert e.eltwise_op(EltwiseOp(kinds.MUL, 0, 0), row, a)[1] == (64, 96)      # broadcast operand on the left
    with pytest.raises(TtError):
        e.eltwise_op(EltwiseOp(kinds.SILU_MUL, 0, 0), a, row)                    # a kind that takes no broadcast
    assert e.eltwise_op(EltwiseOp(kinds.GT, 0, 0), a, a)[0] and e.dims_of(e.eltwise_op(EltwiseOp(kinds.GT, 0, 0), a, a)[0])[1] == BOOL
    assert e.dims_of(e.eltwise_op_as(EltwiseOp(kinds.EXP, 0, 0), a, None, None, True)[0])[1] == BF16
    with pytest.raises(TtError):
        e.eltwise_op_as(EltwiseOp(kinds.GT, 0, 0), a, a, None, True)             # no BF16 result of a Bool kind
    assert e.reduce(a, SUM, ROWS)[1] == (1, 96) and e.reduce(a, MAX, COLS)[1] == (64, 1)
    assert e.sum_rows(a)[1] == (1, 96) and e.full_sum(a)[1] == (1, 1)
    assert e.softmax_rows(a, None, 1.0)[1] == (64, 96) and e.log_softmax_rows(a)[1] == (64, 96)
    assert e.rms(a, 1e-5)[1] == (64, 1) and e.rms_norm(a, row, 1e-5)[1] == (64, 96)
    (s, d1), (n, d2) = e.add_rms_norm(a, a, row, 1e-5)
    assert d1 == d2 == (64, 96)
    assert e.argmax_row(a)[1] == (64, 1)
    idx = e.upload_bits(np.zeros((1, 7), np.uint32), 1, 7, I32)
    assert e.select_rows(a, idx)[1] == (7, 96)
    ridx = e.upload_bits(np.zeros((64, 1), np.uint32), 64, 1, I32)
    assert e.pick_columns(a, ridx)[1] == (64, 1)
    assert e.scatter_add_columns(a, ridx, col)[1] == (64, 96)
    v = f32(e, 7, 96)
    assert e.select_add_rows(a, idx, v)[1] == (64, 96) and e.rows_add(a, [0] * 7, v)[1] == (64, 96)
    assert e.scatter_rows(a, idx, v, False)[1] == (64, 96)
    assert e.assign_rows(a, v, [(1, 0), (2, 6)])[1] == (64, 96)
    with pytest.raises(TtError) as err:
        e.assign_rows(a, v, [(64, 0)])
    assert err.value.status == 6                                                # DOMAIN, found on the host
    assert e.gather_rows([a, v], [(0, 3), (1, 6)], 96)[1] == (2, 96)
    assert e.slice_rows(a, 32, 16)[1] == (16, 96)
    with pytest.raises(TtError):
        e.slice_rows(a, 60, 16)
    assert e.copy_blocks(a, [((0, 0), (0, 0), (64, 32), False), ((0, 32), (64, 0), (64, 32), False),
                             ((0, 64), (128, 0), (64, 32), False)], (192, 32))[1] == (192, 32)
    assert e.copy_blocks(a, [((0, 0), (0, 0), (96, 64), True)], (96, 64))[1] == (96, 64)
    with pytest.raises(TtError):
        e.copy_blocks(a, [((0, 0), (0, 0), (64, 32), False)], (192, 32))       # does not cover the output
    assert e.repack(a, np.zeros((6, 2), np.uint64), (2, 3))[1] == (2, 3)
    assert e.cast_float(a, True)[1] == (64, 96)
    x = f32(e, 128, 192)
    assert e.rope_blocks((x, (0, 0), (128, 128)), (x, (0, 0), (32, 64)), (x, (0, 0), (32, 64)), 64)[1] == (128, 128)
    with pytest.raises(TtError):
        e.rope_blocks((x, (0, 0), (128, 100)), (x, (0, 0), (32, 64)), (x, (0, 0), (32, 64)), 64)
    assert e.eltwise_blocks(EltwiseOp(kinds.MUL, 0, 0), (x, (32, 64), (64, 96)), (x, (0, 0), (64, 96)))[1] == (64, 96)
    with pytest.raises(TtError):
        e.eltwise_blocks(EltwiseOp(kinds.MUL, 0, 0), (x, (100, 0), (64, 96)), (x, (0, 0), (64, 96)))


def test_batched_product_layouts(e):                                            # server.rs:3749-3754
    a, b = f32(e, 96, 40), f32(e, 40, 99)
    items = [(((i * 32, 0), False), ((0, i * 33), False)) for i in range(3)]
    assert e.matmul_dram_batched(a, b, items, (20, 40, 33))[1] == (60, 33)       # stacked
    assert e.matmul_dram_batched_layout(a, b, items, (20, 40, 33), BatchedLayout(1, 0))[1] == (96, 33)  # a tile row each
    with pytest.raises(TtError):
        e.matmul_dram_batched(a, b, [(((90, 0), False), ((0, 0), False))], (20, 40, 33))   # block outside its buffer


def test_product_path_choice(fake, e):
    a, b = e.upload_bf16(np.zeros((256, 128), np.uint16), 256, 128), e.upload_bf16(np.zeros((128, 256), np.uint16), 128, 256)
    e.matmul_dram_bf16(a, False, b, False)
    assert e.last_matmul_path() == "tcgen05"
    f = f32(e, 256, 256)
    e.matmul_dram(f, False, f, False)
    assert e.last_matmul_path() == "tcgen05-tf32x3"
    s = f32(e, 64, 64)
    e.matmul_dram(s, False, s, False)
    assert e.last_matmul_path() == "simt"
    with pytest.raises(TtError):
        e.matmul_dram(a, False, f, False)                                       # mixed operand types
    C.c_int.in_dll(fake, "fake_tc_supported").value = 0
    e.matmul_dram_bf16(a, False, b, False)
    assert e.last_matmul_path() == "simt"                                       # automatic mode falls back
    strict = CudaEngine(0, bf16_matmul_mode=2, lib=fake)
    x, y = strict.upload_bf16(np.zeros((64, 64), np.uint16), 64, 64), strict.upload_bf16(np.zeros((64, 64), np.uint16), 64, 64)
    with pytest.raises(TtError) as err:
        strict.matmul_dram_bf16(x, False, y, False)                             # tensor cores only: refused, never slower silently
    assert err.value.status == 2
    strict.close()


def test_attention_rows_dims_and_refusals(e):                                      # tt-kernels/src/attention.rs:156-171, 386-415
    q, k, v = f32(e, 4, 64), f32(e, 512, 64), f32(e, 512, 32)
    mask = e.upload_bits(np.zeros((1, 512), np.uint32), 1, 512, BOOL)
    heads = [((0, 0), (0, 0), (0, 0)), ((2, 0), (0, 0), (0, 0))]
    before = e.device_traffic().launches
    out, dims = e.attention_rows([q, k, v, mask], heads, [2, 64, 512, 32], 0.125)
    assert dims == (1, 2 * 2 * 32) and e.dims_of(out) == ((1, 128), F32)
    assert e.device_traffic().launches - before == 2          # positions split over blocks, then joined
    assert C.c_int.in_dll(e._lib, "fake_last_attention_jobs").value == 1   # both heads share K and V: one job of 4 rows
    short, _ = e.attention_rows([q, k, v, mask], heads, [2, 64, 512, 32][:1] + [64, 512, 32], 0.125)
    e.free(short)
    for dims4 in ([33, 64, 512, 32], [2, 48, 512, 32], [2, 64, 500, 32], [2, 64, 512, 16], [0, 64, 512, 32]):
        with pytest.raises(TtError) as err:
            e.attention_rows([q, k, v, mask], heads, dims4, 1.0)
        assert err.value.status == 2
    for buffers, items in (([q, k, v, q], heads), ([q, k, v, mask], []), ([q, k, v, mask], [((3, 0), (0, 0), (0, 0))]),
                           ([q, k, v, mask], [((0, 0), (0, 2), (0, 0))])):
        with pytest.raises(TtError) as err:
            e.attention_rows(buffers, items, [2, 64, 512, 32], 1.0)
        assert err.value.status == 2
    with pytest.raises(TtError) as err:
        e.attention_rows([q, 424242, v, mask], heads, [2, 64, 512, 32], 1.0)
    assert err.value.status == 5


def test_matmul_into_and_ipc_handles(e):          # the sharded product's fused step (tt-kernels/src/shard.rs:348-458)
    a = e.upload_bf16(np.zeros((256, 128), np.uint16), 256, 128)
    b = e.upload_bf16(np.zeros((128, 64), np.uint16), 128, 64)
    c, _ = e.zeros_dram((256, 192), bf16=True)
    mine, _ = e.device_ptr(c)
    handle = e.ipc_export(c)
    assert len(handle) == 64
    peer = e.ipc_open(handle)                     # the stand-in runtime hands the same address back
    assert peer == mine
    before = e.device_traffic().launches
    e.matmul_into(a, b, [mine, peer], (256, 192), 64)
    assert e.device_traffic().launches - before == 1 and e.last_matmul_path() == "tcgen05"
    e.ipc_close(peer)
    for args in (([mine], (256, 192), 160),       # the slice would end past the last column
                 ([mine], (128, 192), 0),         # C has other rows than the product
                 ([], (256, 192), 0), ([mine] * 9, (256, 192), 0), ([mine, 0], (256, 192), 0)):
        with pytest.raises(TtError) as err:
            e.matmul_into(a, b, *args)
        assert err.value.status == 2
    f = f32(e, 256, 128)
    with pytest.raises(TtError):
        e.matmul_into(f, b, [mine], (256, 192), 0)          # F32 operands
    v, _ = e.slice_rows(c, 0, 128)
    with pytest.raises(TtError):
        e.ipc_export(v)                                       # a view has no allocation of its own


def test_gated_product_dims_and_refusals(e):       # tt-models/src/llama.rs:498 as one product
    a = e.upload_bf16(np.zeros((64, 128), np.uint16), 64, 128)
    w = e.upload_bf16(np.zeros((128, 512), np.uint16), 128, 512)
    out, dims = e.matmul_silu_mul(a, w)
    assert dims == (64, 256) and e.dims_of(out) == ((64, 256), BF16)
    for bad in (e.upload_bf16(np.zeros((128, 384), np.uint16), 128, 384),      # not whole groups of 256 columns
                e.upload_bf16(np.zeros((64, 512), np.uint16), 64, 512),        # inner dimensions differ
                f32(e, 128, 512)):                                             # F32 weights
        with pytest.raises(TtError) as err:
            e.matmul_silu_mul(a, bad)
        assert err.value.status == 2


def test_projection_with_rope_dims_and_refusals(e):   # tt-models/src/llama.rs:404-433 as one product
    a = e.upload_bf16(np.zeros((128, 64), np.uint16), 128, 64)
    w = e.upload_bf16(np.zeros((64, 320), np.uint16), 64, 320)
    cos, sin = f32(e, 64, 64), f32(e, 64, 64)
    tab = lambda t, r=64: (t, (0, 0), (r, 64))
    launches = e.device_traffic().launches
    out, dims = e.matmul_rope(a, w, tab(cos), tab(sin), 192)
    assert dims == (128, 320) and e.dims_of(out) == ((128, 320), BF16) and e.device_traffic().launches - launches == 1
    for bad_cols in (0, 100, 384):                                              # none, not whole heads of 64, past the product
        with pytest.raises(TtError) as err:
            e.matmul_rope(a, w, tab(cos), tab(sin), bad_cols)
        assert err.value.status == 2
    with pytest.raises(TtError):                                                # 48 table rows do not divide 128 product rows
        e.matmul_rope(a, w, tab(cos, 48), tab(sin, 48), 192)
    with pytest.raises(TtError):                                                # F32 weights
        e.matmul_rope(a, f32(e, 64, 320), tab(cos), tab(sin), 192)
    wide = f32(e, 64, 96)
    with pytest.raises(TtError):                                                # a table block 32 columns wide
        e.matmul_rope(a, w, (wide, (0, 0), (64, 32)), tab(sin), 192)


def test_projection_into_the_residual_and_its_norm_dims_and_refusals(e):   # tt-models/src/llama.rs:371-507 as one product
    a = e.upload_bf16(np.zeros((128, 64), np.uint16), 128, 64)
    w = e.upload_bf16(np.zeros((64, 576), np.uint16), 64, 576)
    resid = f32(e, 128, 576)
    gains = e.upload_bf16(np.zeros((1, 576), np.uint16), 1, 576)
    launches = e.device_traffic().launches
    (s, d0), (n, d1) = e.matmul_add_rms_norm(a, w, resid, gains, 1e-5)
    assert d0 == d1 == (128, 576) and e.dims_of(s) == ((128, 576), F32) and e.dims_of(n) == ((128, 576), BF16)
    assert e.device_traffic().launches - launches == 1 and e.last_matmul_path() == "tcgen05-addnorm"
    for bad in (lambda: e.matmul_add_rms_norm(a, w, f32(e, 128, 512), gains, 1e-5),                     # a residual of another shape
                lambda: e.matmul_add_rms_norm(a, w, resid, e.upload_bf16(np.zeros((1, 64), np.uint16), 1, 64), 1e-5),   # too few gains
                lambda: e.matmul_add_rms_norm(a, w, resid, f32(e, 1, 576), 1e-5),                       # F32 gains
                lambda: e.matmul_add_rms_norm(a, f32(e, 64, 576), resid, gains, 1e-5),                  # F32 weights
                lambda: e.matmul_add_rms_norm(a, e.upload_bf16(np.zeros((64, 320), np.uint16), 64, 320), f32(e, 128, 320),
                                              e.upload_bf16(np.zeros((1, 320), np.uint16), 1, 320), 1e-5)):   # 320 columns: not tiles of 192
        with pytest.raises(TtError) as err:
            bad()
        assert err.value.status == 2


def test_views_keep_their_parent_alive(e):                                      # server.rs:480-481
    t0 = e.device_traffic().pool_in_use
    a = f32(e, 64, 8)
    v = e.slice_rows(a, 8, 16)[0]
    e.free(a)
    with pytest.raises(TtError):
        e.download(a)                                                           # the id is gone
    assert np.array_equal(e.download(v), np.arange(64, 192, dtype=np.float32).reshape(16, 8))
    assert e.device_traffic().pool_in_use > t0                                  # ... but its memory is not
    e.free(v)
    assert e.device_traffic().pool_in_use == t0


def test_pool_reuse_and_out_of_memory(fake, e):
    a = f32(e, 256, 256)
    r0 = e.device_traffic().pool_reserved
    for _ in range(10):
        o, _ = e.eltwise_op(EltwiseOp(kinds.RELU, 0, 0), a)
        e.free(o)
    assert e.device_traffic().pool_reserved == r0 + 256 * 256 * 4               # one block, reused nine times
    C.c_uint64.in_dll(fake, "fake_cuda_memory_limit").value = C.c_uint64.in_dll(fake, "fake_cuda_memory_in_use").value + (1 << 20)
    with pytest.raises(TtError) as err:
        f32(e, 1024, 1024)                                                      # the driver has no room: reported, not fatal
    assert err.value.status == 1 and e.last_oom()[0] == 4 << 20
    C.c_uint64.in_dll(fake, "fake_cuda_memory_limit").value = 0
    assert f32(e, 1024, 1024)
    lim = CudaEngine(0, pool_limit_bytes=1 << 20, lib=fake)
    lim.upload(np.zeros((256, 256), np.float32), 256, 256)
    with pytest.raises(TtError) as err:
        lim.upload(np.zeros((512, 512), np.float32), 512, 512)
    assert err.value.status == 1 and lim.last_oom() == (1 << 20, 768 << 10, 768 << 10)
    lim.close()
    nth = CudaEngine(0, fail_alloc_at=2, lib=fake)
    x = nth.upload(np.zeros((4, 4), np.float32), 4, 4)
    with pytest.raises(TtError):
        nth.eltwise_op(EltwiseOp(kinds.RELU, 0, 0), x)                          # the second allocation is told to fail
    assert nth.eltwise_op(EltwiseOp(kinds.RELU, 0, 0), x)[1] == (4, 4)          # and the engine carries on
    nth.close()


def test_trace_state_machine(fake, e):                                          # server.rs:591-660
    a = f32(e, 64, 64)
    with pytest.raises(TtError):
        e.end_trace()                                                           # nothing open
    e.begin_trace()
    with pytest.raises(TtError):
        e.begin_trace()                                                         # one at a time
    for call in (lambda: e.sync(), lambda: e.download(a), lambda: f32(e, 2, 2)):
        with pytest.raises(TtError) as err:
            call()                                                              # no wait, download or upload inside
        assert err.value.status == 2
    o1, _ = e.eltwise_op(EltwiseOp(kinds.RELU, 0, 0), a)
    t1, _ = e.eltwise_op(EltwiseOp(kinds.EXP, 0, 0), o1)
    e.free(o1)
    o2, _ = e.eltwise_op(EltwiseOp(kinds.NEG, 0, 0), t1)                        # may reuse o1's block inside the capture
    trace = e.end_trace()
    in_use = e.device_traffic().pool_in_use
    l0 = e.device_traffic().launches
    e.run_trace(trace)
    assert e.device_traffic().launches - l0 == 3                                # a replay counts the kernels it runs
    junk = [f32(e, 64, 64) for _ in range(4)]                                   # the pool must not hand out the trace's blocks
    ptrs = {e.device_ptr(j)[0] for j in junk}
    assert e.device_ptr(o2)[0] not in ptrs and e.device_ptr(t1)[0] not in ptrs
    e.free(t1)                                                                  # an output freed by the caller stays the trace's
    more = {e.device_ptr(f32(e, 64, 64))[0] for _ in range(4)}
    with pytest.raises(TtError):
        e.run_trace(trace + 7)
    e.release_trace(trace)
    e.release_trace(trace)                                                      # twice: a no-op
    with pytest.raises(TtError):
        e.run_trace(trace)
    assert e.download(o2).shape == (64, 64)                                     # a live output outlives its trace


def test_errors_carry_the_op_label_and_shapes(e):                               # server.rs:663, 2974-2980
    e.set_op_label("float_matmul")
    a = f32(e, 2, 3)
    with pytest.raises(TtError) as err:
        e.matmul_dram(a, False, a, False)
    assert "float_matmul" in str(err.value) and "[2,3] x [2,3]" in str(err.value)


def test_no_device_is_reported(fake):
    C.c_int.in_dll(fake, "fake_cuda_device_count").value = 0
    try:
        with pytest.raises(TtError) as err:
            CudaEngine(0, lib=fake)
        assert err.value.status == 7
    finally:
        C.c_int.in_dll(fake, "fake_cuda_device_count").value = 1
    with pytest.raises(TtError):
        CudaEngine(3, lib=fake)                                                 # no such card


def test_movers_casts_scan_sort_and_draws_dims_and_refusals(e):     # server.rs:137,309,317,414,578,758,768,779
    from metalium_rs_b200 import engine as E
    a, h = f32(e, 70, 100), e.upload_bf16(np.zeros((70, 100), np.uint16), 70, 100)
    assert e.cast_block((a, (32, 64), (33, 31)), True)[1] == (33, 31)
    assert e.cast_block((h, (0, 0), (70, 100)), False)[1] == (70, 100)
    assert e.cast_f16(a, True)[1] == (70, 100) and e.cast_f16(h, False)[1] == (70, 100)
    for bad in (lambda: e.cast_block((h, (0, 0), (1, 1)), True), lambda: e.cast_block((a, (69, 0), (2, 1)), True),
                lambda: e.cast_f16(h, True), lambda: e.cast_f16(a, False)):
        with pytest.raises(TtError) as err:
            bad()
        assert err.value.status == 2
    b = f32(e, 3, 5)
    assert e.repack_many([a, b], [(0, (69, 99)), (1, (2, 4))] * 3, (2, 3))[1] == (2, 3)
    with pytest.raises(TtError) as err:
        e.repack_many([a, b], [(1, (3, 0))], (1, 1))
    assert err.value.status == 6                                                   # DOMAIN, found on the host
    for bad in (lambda: e.repack_many([a, h], [(0, (0, 0))], (1, 1)), lambda: e.repack_many([a], [(0, (0, 0))], (1, 2)),
                lambda: e.repack_many([], [], (0, 0))):
        with pytest.raises(TtError) as err:
            bad()
        assert err.value.status == 2
    idx = e.upload_bits(np.zeros((9, 40), np.int32), 9, 40, I32)
    assert e.select_taps(a, idx, True)[1] == (40, 8 * 128 + 100)                 # index.rs:139-141
    assert e.select_taps(b, idx, False)[1] == (40, 8 * 32 + 5)
    with pytest.raises(TtError):
        e.select_taps(a, a, False)                                                 # indices must be I32
    i32 = e.upload_bits(np.zeros((70, 100), np.int32), 70, 100, I32)
    assert e.scan(a, E.SCAN_SUM)[1] == (70, 100) and e.scan(i32, E.SCAN_IMAX)[1] == (70, 100)
    big = e.upload_bits(np.zeros((600, 4), np.int32), 600, 4, I32)
    t0 = e.device_traffic().launches
    e.scan(big, E.SCAN_ISUM)
    assert e.device_traffic().launches - t0 == 2                                   # row chunks: fold, then scan from the prefix
    for bad in (lambda: e.scan(a, E.SCAN_ISUM), lambda: e.scan(i32, E.SCAN_MIN_NAN), lambda: e.scan(a, 10)):
        with pytest.raises(TtError) as err:
            bad()
        assert err.value.status == 2
    planes = f32(e, 64, 96)
    (k, kd), idx_out = e.sort_planes(planes, F32, 40, True, True)
    assert kd == (64, 96) and idx_out[1] == (64, 96) and e.dims_of(idx_out[0]) == ((64, 96), I32)
    assert e.sort_planes(planes, F32, 64, False, False)[1] is None
    for n, elem in ((0, F32), (1025, F32), (32, F32), (65, F32), (40, I32)):
        with pytest.raises(TtError) as err:
            e.sort_planes(planes, elem, n, False, False)
        assert err.value.status == 2
    assert e.pow(a, ("scalar", 2.0))[1] == (70, 100) and e.pow(a, ("int", i32))[1] == (70, 100)
    with pytest.raises(TtError):
        e.pow(a, ("tensor", b))
    for draw, elem in ((("unit",), F32), (("uniform", -1.0, 1.0), F32), (("bernoulli", 0.5, True), I32), (("normal", 0.0, 1.0, False), F32),
                       (("normal", 0.0, 1.0, True), I32), (("int_range", -3, 9), I32), (("int_words",), I32)):
        out, dims = e.random_dram((5, 7), draw, 42)
        assert dims == (5, 7) and e.dims_of(out) == ((5, 7), elem)
    for draw in (("uniform", 1.0, 1.0), ("bernoulli", -0.1, False), ("normal", 0.0, float("nan"), False), ("int_range", 0, 0),
                 ("int_range", -(1 << 23), 1)):
        with pytest.raises(TtError) as err:
            e.random_dram((2, 2), draw, 0)
        assert err.value.status == 2
    assert e.pool_bf16(h, [[[0, 0], [1, 1]], [[69, 99]]] * 3, [2, 1] * 3, (2, 3))[1] == (2, 3)
    assert e.dims_of(e.pool_bf16(h, [[[0, 0]]], [1], (1, 1))[0]) == ((1, 1), F32)
    for bad, status in ((([[[0, 0]]] * 2, [1, 1], (1, 1)), 2), (([[]], [1], (1, 1)), 2), (([[[0, 0]]], [0], (1, 1)), 2),
                        (([[[70, 0]]], [1], (1, 1)), 6)):
        with pytest.raises(TtError) as err:
            e.pool_bf16(h, *bad)
        assert err.value.status == status
    with pytest.raises(TtError):
        e.pool_bf16(a, [[[0, 0]]], [1], (1, 1))
    w = e.cast_bf16_storage(f32(e, 100, 40), True)[0]                              # server.rs:150
    assert e.dims_of(w) == ((100, 40), BF16) and e.matmul_dram(a, False, w, False)[1] == (70, 40)
    assert e.matmul_dram(w, True, a, True)[1] == (40, 70)
    m = e.metadata(np.arange(6, dtype=np.uint32), (2, 3), I32)
    assert np.array_equal(e.download_bits(m).ravel(), np.arange(6)) and e.dims_of(m) == ((2, 3), I32)
    largest, total = e.gddr_free_bytes()
    assert largest <= total


def test_metadata_inside_a_trace_is_replayed(fake, e):              # server.rs:95 "replayable mover immediates"
    a = f32(e, 4, 4)
    e.begin_trace()
    m = e.metadata(np.arange(16, dtype=np.uint32), (4, 4), I32)
    e.eltwise(kinds.RELU, 0.0, a)
    t = e.end_trace()
    e.run_trace(t)
    assert e.dims_of(m) == ((4, 4), I32)
    e.release_trace(t)


def test_convolution_and_pooling_callers_issue_the_reference_sequence(e):   # burn-tt/src/ops/nhwc.rs:226-292, 296-418
    from metalium_rs_b200 import workloads as W
    t = f32(e, 2 * 6 * 6, 3)
    l0 = e.device_traffic().launches
    out, (oh, ow) = W.conv2d_nhwc(e, t, (2, 3, 6, 6), np.ones((8, 3, 3, 3), np.float32), np.zeros(8, np.float32), (1, 1), (1, 1))
    assert (oh, ow) == (6, 6) and e.dims_of(out) == ((72, 8), F32)
    assert e.device_traffic().launches - l0 == 4             # select_taps, repack_many, product, bias add (zeros is a memset)
    p = f32(e, 1 * 8 * 8, 32)
    best, (oh, ow) = W.max_pool2d_nhwc(e, p, (1, 32, 8, 8), (2, 2), (2, 2))
    assert (oh, ow) == (4, 4) and e.dims_of(best) == ((16, 32), F32)


def test_prompt_chunks_and_the_generation_after_them_issue_consistent_ops(e):   # tt-models/src/kv_cache.rs:231-296
    from metalium_rs_b200 import workloads as W
    cfg = W.LlamaConfig(layers=2, hidden=64, heads=2, kv_heads=1, head_dim=64, ff=128, vocab=256)
    batch, chunk, max_len = 2, 128, 384
    pre = W.LlamaPrefill(e, cfg, W.llama_weights(cfg, seed=3), batch, chunk)
    assert pre.fused
    dec = W.LlamaDecode(e, cfg, pre.w, batch, max_len=max_len)
    ids = e.upload_bits(np.zeros((1, batch * chunk), np.int32), 1, batch * chunk, I32)
    for k in range(2):                                   # every op of a chunk passes the engine's bounds and dims checks
        lg, am = pre.forward(ids, cache=dec, start=k * chunk)
        assert e.dims_of(lg) == ((batch, cfg.vocab), F32) and e.dims_of(am) == ((batch, 1), I32)
        if k == 0:
            e.free(lg); e.free(am)
    with pytest.raises(ValueError):
        pre.forward(ids, cache=dec, start=64)            # not whole 128-position tiles
    with pytest.raises(ValueError):
        pre.forward(ids, start=128)                      # a later chunk has no cache to attend to
    with pytest.raises(AssertionError):
        pre.forward(ids, cache=dec, start=384)           # past the cache
    dec.continue_from(am, 2 * chunk)
    lg2, am2 = dec.step()
    assert e.dims_of(lg2) == ((batch, cfg.vocab), F32)


def test_launch_set_up_is_done_on_every_device_an_engine_lives_on(fake):
    # A kernel's opt-in to large shared memory is an attribute of the function on ONE device: an engine on a second
    # ordinal of the same process must set it again, once.
    C.c_int.in_dll(fake, "fake_cuda_device_count").value = 2
    calls = (C.c_int * 8).in_dll(fake, "fake_smem_attr_calls")
    try:
        before = [calls[0], calls[1]]
        e0, e1 = CudaEngine(0, lib=fake), CudaEngine(1, lib=fake)
        for eng in (e0, e1, e0, e1):
            a = eng.upload_bf16(np.zeros((256, 128), np.uint16), 256, 128)
            b = eng.upload_bf16(np.zeros((128, 256), np.uint16), 128, 256)
            eng.matmul_dram_bf16(a, False, b, False)
        assert calls[0] - before[0] <= 1 and calls[1] - before[1] == 1      # device 0 may have been set by an earlier test
        assert calls[0] >= 1
        e0.close(); e1.close()
    finally:
        C.c_int.in_dll(fake, "fake_cuda_device_count").value = 1
        C.c_int.in_dll(fake, "fake_cuda_current_device").value = 0


def test_a_batched_call_of_one_item_takes_the_plain_product_s_route(fake, e):
    # One (Block, Block) pair is folded into a plain product on the blocks (offsets into the bases, the item's flags):
    # an F32 item of 256 and up reaches the split-TF32 path, which refuses batches.
    f = f32(e, 512, 512)
    out, dims = e.matmul_dram_batched(f, f, [(((128, 64), False), ((0, 256), True))], (256, 256, 256))
    assert dims == (256, 256) and e.last_matmul_path() == "tcgen05-tf32x3"
    out, dims = e.matmul_dram_batched(f, f, [(((0, 0), False), ((0, 0), False)), (((256, 0), False), ((0, 0), False))], (256, 256, 256))
    assert dims == (512, 256) and e.last_matmul_path() == "simt"                # two F32 items: the batched SIMT kernel


def test_out_of_memory_inside_a_capture_does_not_touch_the_stream(fake, e):
    # the retry path synchronises the stream, which would invalidate an open capture: inside one the failure is immediate
    a = f32(e, 64, 64)
    e.begin_trace()
    syncs = C.c_int.in_dll(fake, "fake_sync_in_capture").value
    C.c_uint64.in_dll(fake, "fake_cuda_memory_limit").value = C.c_uint64.in_dll(fake, "fake_cuda_memory_in_use").value + 1024
    with pytest.raises(TtError) as err:
        e.zeros_dram((2048, 2048))                                              # 16 MB asked with 1 KB of room
    assert err.value.status == 1
    assert C.c_int.in_dll(fake, "fake_sync_in_capture").value == syncs          # no synchronise-and-retry
    C.c_uint64.in_dll(fake, "fake_cuda_memory_limit").value = 0
    o, _ = e.eltwise_op(EltwiseOp(kinds.RELU, 0, 0), a)                         # the capture is still open and usable
    t = e.end_trace()
    e.run_trace(t)
    e.release_trace(t)


def test_rows_add_trace_ops_and_footprint(fake, e):
    t0, v = f32(e, 16, 32), f32(e, 3, 32)
    e.begin_trace()
    e.set_op_label("embedding_backward")
    out, dims = e.rows_add(t0, [5, 2, 5], v)                                    # an index list inside a capture: a copy node, not an upload
    assert dims == (16, 32)
    e.set_op_label("relu")
    r, _ = e.eltwise_op(EltwiseOp(kinds.RELU, 0, 0), out)
    tr = e.end_trace()
    assert e.trace_ops(tr) == [("embedding_backward", 1), ("relu", 1)]
    assert e.trace_footprint(tr) >= 2 * 16 * 32 * 4
    e.release_trace(tr)
    with pytest.raises(TtError):
        e.trace_ops(tr)
    with pytest.raises(TtError):
        e.rows_add(t0, [1, 2], v)                                               # two indices, three value rows


def test_profile_mode_state_machine(fake, e):
    a = f32(e, 8, 8)
    with pytest.raises(TtError):
        e.profile_mode(False)                                                   # not on
    e.profile_mode(True)
    for label in ("relu", "exp", "relu"):
        e.set_op_label(label)
        e.eltwise_op(EltwiseOp(kinds.RELU if label == "relu" else kinds.EXP, 0, 0), a)
    table = e.profile_mode(False)
    assert [(r["op"], r["calls"], r["launches"]) for r in table] == [("relu", 2, 2), ("exp", 1, 1)]
    assert e.profile_report() == table
    e.set_op_label("after")                                                     # off: labels cost nothing and record nothing
    assert e.profile_report() == table


def test_bfp8_storage_dims_bytes_and_refusals(e):                  # server.rs:141 `cast_bfp`
    from metalium_rs_b200 import BFP8
    w = f32(e, 64, 96)
    in_use = e.device_traffic().pool_in_use
    packed, dims = e.cast_bfp(w, 8)
    assert dims == (64, 96) and e.dims_of(packed) == ((64, 96), BFP8)
    assert e.device_traffic().pool_in_use - in_use == 8192         # 64 * 96 * 17 / 16 = 6,528 bytes, in a pool block of 8,192
    assert e.cast_bfp(packed, None)[1] == (64, 96) and e.dims_of(e.cast_bfp(packed, "bf16")[0])[1] == BF16
    a = e.upload_bf16(np.zeros((2, 64), np.uint16), 2, 64)
    assert e.matmul_dram_bf16(a, False, packed, False)[1] == (2, 96) and e.last_matmul_path() == "skinny-bfp8"
    tall = e.upload_bf16(np.zeros((128, 64), np.uint16), 128, 64)
    assert e.matmul_dram_bf16(tall, False, packed, False)[1] == (128, 96) and e.last_matmul_path() == "tcgen05"   # widened for the call
    for bad in (lambda: e.cast_bfp(w, None), lambda: e.cast_bfp(packed, 8), lambda: e.cast_bfp(f32(e, 4, 24), 8),
                lambda: e.download(packed), lambda: e.eltwise_op(EltwiseOp(kinds.EXP, 0, 0), packed),
                lambda: e.reduce(packed, SUM, ROWS), lambda: e.matmul_dram(packed, False, w, False),
                lambda: e.slice_rows(packed, 0, 32)):
        with pytest.raises(TtError) as err:
            bad()
        assert err.value.status == 2


def test_the_one_launch_decode_step_checks_its_operands(e):
    from metalium_rs_b200 import workloads as W
    cfg = W.LlamaConfig(layers=2, hidden=128, heads=2, kv_heads=1, head_dim=64, ff=256, vocab=256)
    pre = W.LlamaPrefill(e, cfg, W.llama_weights(cfg, seed=3), 2, 128)
    dec = W.LlamaDecode(e, cfg, pre.w, 2, max_len=128, fused=True, weight_storage="bfp8")
    dec.reset(np.array([1, 2], np.int32))
    l0 = e.device_traffic().launches
    lg, am = dec.step()
    assert e.dims_of(lg) == ((2, cfg.vocab), F32) and e.device_traffic().launches - l0 <= 12
    assert e.last_decode_form() == "grid"                             # BFP8 weights: no descriptors are built, the grid form runs
    plain = W.LlamaDecode(e, cfg, pre.w, 2, max_len=128, fused=True)
    plain.reset(np.array([1, 2], np.int32))
    h0 = e.device_traffic().bytes_h2d
    plain.step()
    assert e.last_decode_form() == "cluster16"                        # BF16 weights: the descriptors go up beside the layer records
    assert e.device_traffic().bytes_h2d - h0 >= cfg.layers * 4 * 128
    bad = list(dec.layer_ids)
    bad[1], bad[2] = bad[2], bad[1]                                   # Wqkv and Wo exchanged: the shapes do not meet
    with pytest.raises(TtError) as err:
        e.decode_layers(dec.shape, e.upload(np.zeros((2, 128), np.float32), 2, 128), bad, dec.w["final_norm"], dec.cos, dec.sin, dec.pos)
    assert err.value.status == 2 and "layer 0 operand 1" in str(err.value)
    with pytest.raises(TtError):                                       # five sequences a step
        e.decode_layers(dec.shape, e.upload(np.zeros((5, 128), np.float32), 5, 128), dec.layer_ids, dec.w["final_norm"], dec.cos, dec.sin, dec.pos)
