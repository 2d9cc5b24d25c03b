"""The full sum for callers that cannot allocate device memory (a host whose GPU memory is
handed out by another runtime in fixed arenas, or a code path where a cudaMalloc would
stall the device): `b200_full_sum_noalloc` keeps its per-block partials in an array inside
the library image.  Checked through the C ABI against `b200_full_sum`, which keeps them in
a buffer the engine allocates -- on two calls in a row, because the array is shared and
keeps the last call's contents.  Collected last, so a run that stops at the first failure
has already run everything else."""
import ctypes as C

import numpy as np
import pytest

from metalium_rs_b200 import F32
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _noalloc(lib, eng, buf_in, n, mean, buf_out):
    lib.b200_full_sum_noalloc.restype = C.c_int32
    lib.b200_full_sum_noalloc.argtypes = [C.c_void_p, C.c_uint64, C.c_int32, C.c_void_p, C.c_void_p]
    src, _ = eng.device_ptr(buf_in)
    dst, _ = eng.device_ptr(buf_out)
    return lib.b200_full_sum_noalloc(src, n, int(mean), dst, eng.stream())


def test_no_alloc_full_sum_matches_the_allocating_entry_point_twice_in_a_row(lib, eng):
    shapes = [(2048, 4096), (37, 8193)]  # two calls in a row, different sizes: the array is reused
    for call, shape in enumerate(shapes):
        v = orc.uniform(0x2A, call + 1, shape, -4, 4)
        n = v.size
        ia = eng.upload(v, *shape)
        for mean in (False, True):
            want_id, _ = eng.full_sum(ia, mean)
            want = eng.download(want_id)
            out_id, _ = eng.zeros_dram((1, 1))
            reserved = eng.device_traffic().pool_reserved
            assert _noalloc(lib, eng, ia, n, mean, out_id) == 0
            got = eng.download(out_id)  # waits on the engine's stream, which the call used
            assert eng.device_traffic().pool_reserved == reserved  # nothing came from the pool either
            truth, bound = orc.full_sum(v, mean)
            exact = v.astype(np.float64).mean() if mean else v.astype(np.float64).sum()
            assert abs(float(got[0, 0]) - exact) <= bound      # the tolerance the other full-sum tests use
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32))  # and the same bits
            eng.free(want_id); eng.free(out_id)
        eng.free(ia)


def test_no_alloc_full_sum_refuses_what_is_beyond_its_limit(lib, eng):
    ia = eng.upload(np.ones((4, 4), np.float32), 4, 4)
    out_id, _ = eng.zeros_dram((1, 1))
    assert _noalloc(lib, eng, ia, (1 << 31) + 1, False, out_id) == 2  # B200_UNSUPPORTED, nothing launched
    buf = C.create_string_buffer(256)
    lib.b200_last_error(None, buf, 256)
    assert b"exceed the limit" in buf.value
    assert float(eng.download(out_id)[0, 0]) == 0.0
    assert _noalloc(lib, eng, ia, 16, False, out_id) == 0
    assert float(eng.download(out_id)[0, 0]) == 16.0
    eng.free(ia); eng.free(out_id)


def test_no_alloc_full_sum_of_nothing(lib, eng):
    ia = eng.upload(np.ones((4, 4), np.float32), 4, 4)
    out_id = eng.upload(np.full((1, 1), 7.0, np.float32), 1, 1)
    assert _noalloc(lib, eng, ia, 0, False, out_id) == 0           # the sum of no elements is +0.0
    assert eng.download_bits(out_id)[0, 0] == 0
    assert _noalloc(lib, eng, ia, 0, True, out_id) == 2            # their mean is 0 / 0: refused, not a silent NaN
    buf = C.create_string_buffer(256)
    lib.b200_last_error(None, buf, 256)
    assert b"mean of no elements" in buf.value
    assert _noalloc(lib, eng, ia, 16, True, out_id) == 0            # and the entry point still works after a refusal
    assert float(eng.download(out_id)[0, 0]) == 1.0
    eng.free(ia); eng.free(out_id)
