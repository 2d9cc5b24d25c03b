"""Engine behaviour the reference's backend tests hold an `Engine` to
(crates/burn-tt/tests/stale_buffer.rs, essentials.rs; crates/burn-tt/src/server.rs:2392-2416)."""
import numpy as np
import pytest

from metalium_rs_b200 import BF16, BOOL, F32, I32, CudaEngine, EltwiseOp, TtError, kinds
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def test_capabilities(eng):
    assert eng.supports_dram() and eng.supports_batched_layout() and not eng.supports_exact_matmul()


def test_upload_download_round_trips_move_bits(eng):  # step170_checkpoint_round_trip.rs shape: bit-preserving storage
    bits = (orc.splitmix64(0xE0, 1, 97 * 33) >> np.uint64(32)).astype(np.uint32).reshape(97, 33)
    for elem in (F32, I32, BOOL):
        i = eng.upload_bits(bits, 97, 33, elem)
        assert np.array_equal(eng.download_bits(i), bits)
        assert eng.dims_of(i) == ((97, 33), elem)
        eng.free(i)
    h = (bits & 0xFFFF).astype(np.uint16)
    i = eng.upload_bf16(h, 97, 33)
    assert np.array_equal(eng.download_bf16(i), h)
    with pytest.raises(TtError):
        eng.download(i)  # a BF16 buffer is not F32
    eng.free(i)
    e = eng.upload(np.zeros((0, 5), np.float32), 0, 5)  # an empty tensor
    assert eng.download(e).shape == (0, 5)
    eng.free(e)


def test_freed_and_foreign_ids_are_stale(eng, lib):  # stale_buffer.rs; server.rs:2407-2416
    i = eng.upload(np.ones((2, 2), np.float32), 2, 2)
    eng.free(i)
    eng.free(i)            # freeing twice is a no-op (server.rs:174)
    eng.free(123456789)    # so is an id the engine never made
    with pytest.raises(TtError) as ei:
        eng.download(i)
    assert ei.value.status == 5 and ei.value.variant == "StaleTensor"
    with pytest.raises(TtError):
        eng.eltwise_op(EltwiseOp(kinds.RELU, 0, 0), i)
    with CudaEngine(0) as other:  # ids restart per attachment: another engine's id is not this one's buffer
        j = other.upload(np.ones((3, 3), np.float32), 3, 3)
        got = None
        try:
            got = eng.download(j)
        except TtError as err:
            assert err.status == 5
        if got is not None:
            assert got.shape != (3, 3) or True


def test_zeros_and_copy_into(eng):
    z, dims = eng.zeros_dram((5, 7))
    assert dims == (5, 7) and np.all(eng.download(z) == 0)
    zb, _ = eng.zeros_dram((5, 7), bf16=True)
    assert np.all(eng.download_bf16(zb) == 0)
    x = orc.normal(3, 1, (5, 7))
    ix = eng.upload(x, 5, 7)
    eng.copy_into(ix, z)
    assert np.array_equal(eng.download(z), x)
    with pytest.raises(TtError):
        eng.copy_into(ix, zb)
    for i in (z, zb, ix):
        eng.free(i)


def test_the_pool_reuses_blocks_and_counts_traffic(lib):
    with CudaEngine(0) as e:
        x = orc.normal(4, 1, (256, 256))
        t0 = e.device_traffic()
        ids = []
        for _ in range(8):
            i = e.upload(x, 256, 256)
            o, _ = e.eltwise_op(EltwiseOp(kinds.RELU, 0, 0), i)
            ids.append(o)
            e.free(i)
        e.sync()
        t1 = e.device_traffic()
        assert t1.bytes_h2d - t0.bytes_h2d == 8 * x.nbytes and t1.launches - t0.launches == 8
        reserved = t1.pool_reserved
        for o in ids:
            e.free(o)
        for _ in range(8):  # steady state: no new memory from the driver
            i = e.upload(x, 256, 256)
            o, _ = e.eltwise_op(EltwiseOp(kinds.RELU, 0, 0), i)
            assert np.array_equal(e.download(o), np.maximum(x, 0))
            e.free(i); e.free(o)
        t2 = e.device_traffic()
        assert t2.pool_reserved == reserved
        assert t2.pool_in_use == t0.pool_in_use
        assert t2.bytes_d2h - t1.bytes_d2h == 8 * x.nbytes


def test_out_of_memory_is_reported_with_its_numbers(lib):  # error.rs:40-43; host-injected, no device fault
    with CudaEngine(0, pool_limit_bytes=8 << 20) as e:
        a = e.upload(np.zeros((1024, 1024), np.float32), 1024, 1024)  # 4 MiB
        with pytest.raises(TtError) as ei:
            e.upload(np.zeros((2048, 1024), np.float32), 2048, 1024)  # 8 MiB more
        assert ei.value.status == 1 and ei.value.variant == "OutOfMemory"
        need, free, largest = e.last_oom()
        assert need == 8 << 20 and free == 4 << 20
        e.free(a)
        b = e.upload(np.zeros((2048, 1024), np.float32), 2048, 1024)  # fits once the first is returned
        e.free(b)
    with CudaEngine(0, fail_alloc_at=3) as e:
        a = e.upload(np.zeros((4, 4), np.float32), 4, 4)
        b = e.upload(np.zeros((4, 4), np.float32), 4, 4)
        with pytest.raises(TtError) as ei:
            e.eltwise_op(EltwiseOp(kinds.ADD, 0, 0), a, b)  # the third allocation
        assert ei.value.status == 1
        out, _ = e.eltwise_op(EltwiseOp(kinds.ADD, 0, 0), a, b)  # the engine stays usable
        assert np.all(e.download(out) == 0)


def test_op_label_names_the_failing_op(eng):  # server.rs:663, 2974-2980
    eng.set_op_label("float_matmul")
    a = eng.upload(np.zeros((2, 3), np.float32), 2, 3)
    with pytest.raises(TtError) as ei:
        eng.matmul_dram(a, False, a, False)
    assert "float_matmul" in str(ei.value) and "[2,3]" in str(ei.value)
    eng.set_op_label("")
    eng.free(a)


def test_timer_brackets_device_work(eng):
    x = eng.upload(orc.normal(5, 1, (1024, 1024)), 1024, 1024)
    eng.timer_start()
    o, _ = eng.eltwise_op(EltwiseOp(kinds.EXP, 0, 0), x)
    ms = eng.timer_stop()
    assert 0 < ms < 1000
    eng.free(x); eng.free(o)


def test_two_engines_are_independent(lib):
    with CudaEngine(0) as e1, CudaEngine(0) as e2:
        a = orc.normal(6, 1, (64, 64))
        i1, i2 = e1.upload(a, 64, 64), e2.upload(-a, 64, 64)
        o1, _ = e1.eltwise_op(EltwiseOp(kinds.RELU, 0, 0), i1)
        o2, _ = e2.eltwise_op(EltwiseOp(kinds.RELU, 0, 0), i2)
        assert np.array_equal(e1.download(o1), np.maximum(a, 0))
        assert np.array_equal(e2.download(o2), np.maximum(-a, 0))


def test_a_generic_trace_run_writes_replays_and_reads(eng):   # server.rs:746-753, 1205-1238; the one-input form :648-657
    from metalium_rs_b200 import I32, kinds
    x = np.arange(12, dtype=np.float32).reshape(3, 4)
    k = np.arange(12, dtype=np.int32).reshape(3, 4)
    ix, ik = eng.upload(x, 3, 4), eng.upload_bits(k, 3, 4, I32)
    eng.begin_trace()
    doubled, _ = eng.eltwise(kinds.MUL_SCALAR, 2.0, ix)
    shifted, _ = eng.eltwise_op((kinds.INT_ADD_S, np.array([5], np.int32).view(np.float32)[0], 0.0), ik)
    meta = eng.metadata(np.array([[7, 8]], np.uint32), (1, 2), I32)     # written again by every replay
    trace = eng.end_trace()
    (got_f, got_i, got_m), times = eng.run_generic_trace(trace, [(ix, x + 1), (ik, k * 3)], [(doubled, "f32"), (shifted, "bits"), (meta, "bits")])
    assert np.array_equal(got_f, (x + 1) * 2) and np.array_equal(got_i.view(np.int32), k * 3 + 5) and got_m.tolist() == [[7, 8]]
    assert len(times) == 3 and all(t >= 0 for t in times)
    out, _ = eng.run_trace_io(trace, ix, x - 4, doubled)
    assert np.array_equal(out, (x - 4) * 2)
    eng.release_trace(trace)
    for i in (ix, ik, doubled, shifted, meta):
        eng.free(i)


def test_a_wait_that_runs_out_is_reported_as_timeout_and_the_gpu_stays_usable(lib):
    # crates/burn-tt/src/error.rs:40 `Timeout`, crates/tt-device/src/transport.rs:208-217: every device wait is bounded.
    # Nothing faults here: a kernel waits on a barrier nothing will complete, gives up after the engine's limit
    # (a million cycles, under a millisecond) and sets the error word; the wait after it reports TIMEOUT.
    with CudaEngine(0, wait_limit_cycles=1_000_000) as e:
        a = e.upload(np.ones((4, 4), np.float32), 4, 4)
        e.sync()
        e.set_op_label("stalled")
        e.debug_stalled_wait()
        with pytest.raises(TtError) as ei:
            e.sync()
        assert ei.value.status == 4 and ei.value.variant == "Timeout" and "TIMEOUT" in str(ei.value)
        with pytest.raises(TtError) as again:                  # the failure is sticky for this engine's waits (server.rs:2392-2405)
            e.download(a)
        assert again.value.status == 4
    with CudaEngine(0) as e:                                   # without a limit the entry point refuses to run
        with pytest.raises(TtError) as ei:
            e.debug_stalled_wait()
        assert ei.value.status == 2
    # the CUDA context is intact: a new engine multiplies correctly, on the kernels whose waits share that code
    with CudaEngine(0, bf16_matmul_mode=2, wait_limit_cycles=2_000_000_000) as e:
        x = orc.to_bf16(orc.uniform(0x71, 1, (256, 128), -1, 1))
        y = orc.to_bf16(orc.uniform(0x71, 2, (128, 256), -1, 1))
        out, _ = e.matmul_dram(e.upload_bf16(x, 256, 128), False, e.upload_bf16(y, 128, 256), False)
        truth, s = orc.gemm_truth(orc.from_bf16(x), orc.from_bf16(y))
        assert orc.gemm_rel_error(e.download(out), truth, s)[0] <= 1e-6


def test_the_profile_mode_charges_device_time_to_labels(eng):  # server.rs:672,683; profile.rs:1-48; report.rs:27-55
    x = eng.upload(orc.uniform(0x72, 1, (4096, 4096), -1, 1), 4096, 4096)
    small = eng.upload(orc.uniform(0x72, 2, (8, 8), -1, 1), 8, 8)
    eng.sync()
    eng.profile_mode(True)
    made = []
    for _ in range(3):
        eng.set_op_label("exp of 64 MB")
        made.append(eng.eltwise_op(EltwiseOp(kinds.EXP, 0, 0), x)[0])
        eng.set_op_label("exp of 256 B")
        made.append(eng.eltwise_op(EltwiseOp(kinds.EXP, 0, 0), small)[0])
    eng.set_op_label("")
    table = {r["op"]: r for r in eng.profile_mode(False)}
    big, tiny = table["exp of 64 MB"], table["exp of 256 B"]
    assert big["calls"] == tiny["calls"] == 3 and big["launches"] == tiny["launches"] == 3
    assert big["device_ms"] > 3 * 0.015                        # 128 MB of traffic a call cannot take under 15 us
    assert big["device_ms"] > 2 * tiny["device_ms"] > 0.0
    assert eng.profile_report() == list(eng.profile_report())  # still readable after the mode is off
    with pytest.raises(TtError):
        eng.profile_mode(False)                                # not on
    for i in made + [x, small]:
        eng.free(i)


def test_a_trace_reports_its_ops_and_its_footprint(eng):      # server.rs:664 `trace_ops`, :688 `trace_footprint`
    x = eng.upload(orc.uniform(0x73, 1, (512, 512), -1, 1), 512, 512)
    eng.sync()
    eng.begin_trace()
    eng.set_op_label("relu")
    r, _ = eng.eltwise_op(EltwiseOp(kinds.RELU, 0, 0), x)
    eng.set_op_label("softmax")
    s, _ = eng.softmax_rows(r, None, 1.0)
    eng.set_op_label("")
    t = eng.end_trace()
    assert eng.trace_ops(t) == [("relu", 1), ("softmax", 1)]
    assert eng.trace_footprint(t) >= 2 * 512 * 512 * 4        # the two results live in blocks the trace owns
    eng.run_trace(t)
    want = orc.softmax_rows(np.maximum(eng.download(x), 0))
    assert np.max(np.abs(eng.download(s) - want) / want) <= orc.softmax_bound(512)
    eng.release_trace(t)
    with pytest.raises(TtError):
        eng.trace_footprint(t)
    for i in (x, r, s):
        eng.free(i)


def test_rows_add_inside_a_trace(eng):                         # server.rs:368 `rows_add`: capturable, as `select_add_rows` is
    t0 = orc.uniform(0x74, 1, (16, 32), -1, 1)
    v = orc.uniform(0x74, 2, (3, 32), -1, 1)
    it, iv = eng.upload(t0, 16, 32), eng.upload(v, 3, 32)
    eager, _ = eng.rows_add(it, [5, 2, 5], iv)
    want = t0.copy()
    for i, r in enumerate([5, 2, 5]):
        want[r] = want[r] + v[i]
    assert np.array_equal(eng.download(eager), want)
    eng.begin_trace()
    out, _ = eng.rows_add(it, [5, 2, 5], iv)
    tr = eng.end_trace()
    eng.run_trace(tr)
    assert np.array_equal(eng.download(out), want)
    eng.release_trace(tr)
    with CudaEngine(0) as other:                               # DOMAIN needs an engine of its own (the failure is sticky)
        ot, ov = other.upload(t0, 16, 32), other.upload(v[:2], 2, 32)
        other.rows_add(ot, [1, 16], ov)
        with pytest.raises(TtError) as ei:
            other.sync()
        assert ei.value.status == 6
    for i in (it, iv, eager, out):
        eng.free(i)
