"""A 2-D convolution and a max pooling through the ops the reference sends for them
(crates/burn-tt/src/ops/nhwc.rs:226-292, 296-418): `select_taps` for the patch matrix, `repack_many` for the weights'
relay, one product; `select_taps`, `copy_blocks` and exact compares and selects for the pooling.  The convolution
is held to the F32 product's bound (1e-5 of S, the sum of the products' magnitudes, as the products are in
tests/test_gpu_matmul.py); the pooling is bit for bit, NaNs and signed zeros included."""
import numpy as np
import pytest

from metalium_rs_b200 import workloads as W
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _nhwc(x):
    n, c, h, w = x.shape
    return np.ascontiguousarray(x.transpose(0, 2, 3, 1)).reshape(n * h * w, c)


@pytest.mark.parametrize("shape,wshape,stride,padding,dilation,bias", [
    ((2, 3, 12, 12), (8, 3, 3, 3), (1, 1), (1, 1), (1, 1), True),       # a first layer: 3 channels, padded
    ((1, 32, 9, 11), (16, 32, 3, 3), (2, 2), (0, 0), (1, 1), False),    # whole-tile channels, strided, no padding
    ((2, 40, 8, 8), (10, 40, 2, 3), (1, 2), (1, 0), (2, 1), True),      # ragged channels, a dilated ragged kernel
    ((1, 5, 7, 7), (4, 5, 1, 1), (1, 1), (0, 0), (1, 1), False),        # one tap: the patch matrix is the table
])
def test_conv2d_through_select_taps_and_one_product(eng, shape, wshape, stride, padding, dilation, bias):
    x = orc.normal(0xC0, 1, shape)
    wt = orc.uniform(0xC0, 2, wshape, -0.5, 0.5)
    b = orc.uniform(0xC0, 3, (wshape[0],), -1.0, 1.0) if bias else None
    t = eng.upload(_nhwc(x), shape[0] * shape[2] * shape[3], shape[1])
    out, (oh, ow) = W.conv2d_nhwc(eng, t, shape, wt, b, stride, padding, dilation)
    truth, s = orc.conv2d(x, wt, b, stride, padding, dilation)
    assert truth.shape[2:] == (oh, ow)
    got = eng.download(out).reshape(shape[0], oh, ow, wshape[0]).transpose(0, 3, 1, 2)
    assert np.max(np.abs(got - truth) / s) <= 1e-5
    eng.free(t); eng.free(out)


@pytest.mark.parametrize("shape,kernel,stride,padding,dilation", [((2, 32, 10, 10), (2, 2), (2, 2), (0, 0), (1, 1)),
                                                                  ((1, 64, 9, 7), (3, 3), (2, 1), (1, 1), (1, 1)),
                                                                  ((1, 32, 8, 8), (2, 3), (1, 1), (0, 1), (2, 1))])
def test_max_pool2d_is_the_first_nan_else_the_first_maximum(eng, shape, kernel, stride, padding, dilation):
    x = np.round(orc.uniform(0xC1, 1, shape, -3.0, 3.0)).view(np.uint32).copy()       # ties and both zeros
    special = np.array([0x7FC00000, 0xFFC00001, 0x7F800000, 0xFF800000, 0x80000000], np.uint32)
    sel = orc.integers(0xC1, 2, shape, 11) == 0
    x[sel] = special[orc.integers(0xC1, 3, shape, len(special))[sel]]
    t = eng.upload_bits(_nhwc(x), shape[0] * shape[2] * shape[3], shape[1], 0)
    out, (oh, ow) = W.max_pool2d_nhwc(eng, t, shape, kernel, stride, padding, dilation)
    want = orc.max_pool2d(x, kernel, stride, padding, dilation)
    got = eng.download_bits(out).reshape(shape[0], oh, ow, shape[1]).transpose(0, 3, 1, 2)
    assert np.array_equal(got, want)
    eng.free(t); eng.free(out)


@pytest.mark.parametrize("shape,kernel,stride,padding,include", [((2, 3, 8, 8), (2, 2), (2, 2), (0, 0), True),
                                                                 ((1, 4, 9, 7), (3, 3), (2, 1), (1, 1), False),
                                                                 ((1, 2, 12, 12), (5, 5), (3, 3), (2, 2), True)])
def test_avg_pool2d_of_a_bf16_tensor(eng, shape, kernel, stride, padding, include):   # burn-tt/src/ops/pool.rs:254-275
    import torch
    x = orc.to_bf16(orc.normal(0xC2, 1, shape))
    n, c, h, w = shape
    buf = eng.upload_bf16(x.reshape(n * c * h, w), n * c * h, w)
    out = W.avg_pool2d_bf16(eng, buf, shape, kernel, stride, padding, include)
    windows, divisors, dims = W.avg_pool2d_windows(shape, kernel, stride, padding, include)
    want = orc.to_bf16(orc.pool_bf16(x.reshape(n * c * h, w), windows, divisors, dims))
    got = eng.download_bf16(out).reshape(dims)
    assert np.array_equal(got, want)
    ref = torch.nn.functional.avg_pool2d(torch.from_numpy(orc.from_bf16(x)), kernel, stride, padding, count_include_pad=include).numpy()
    assert np.max(np.abs(orc.from_bf16(got).reshape(ref.shape) - ref)) <= 2.0 ** -8 * np.abs(ref).max() + 1e-6    # one BF16 rounding
    eng.free(buf); eng.free(out)
