"""Shared helpers of the parity tests: the generators the reference's own tests use
for their inputs, restated, and upload shorthands."""
import numpy as np


def lcg_row(seed: int, n: int) -> np.ndarray:
    """crates/tt-tests/tests/step211_argmax_row.rs:31-41: n values in [-20, 20)."""
    s = (seed | 1) & 0xFFFFFFFFFFFFFFFF
    out = np.empty(n, dtype=np.float32)
    for i in range(n):
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        out[i] = np.float32(np.float32(s >> 40) / np.float32(1 << 24)) * np.float32(40.0) - np.float32(20.0)
    return out


def full_sum_values(n: int) -> np.ndarray:
    """crates/tt-tests/tests/step63_burn_full_reduce.rs:16-20."""
    i = np.arange(n, dtype=np.int64)
    return (((i * 73 % 257).astype(np.float32) - np.float32(128.0)) / np.float32(37.0)).astype(np.float32)


def small_ints(rng: np.random.Generator, shape, span: int = 7) -> np.ndarray:
    """Small-integer operands, so every order of summation is exact
    (crates/tt-tests/tests/step11_burn.rs:128-130)."""
    return rng.integers(-span, span + 1, size=shape).astype(np.float32)


def argmax_cases(n: int):
    """crates/tt-tests/tests/step211_argmax_row.rs:43-67."""
    out = [("random", lcg_row(n, n))]
    tie = lcg_row(7, n)
    for i in (n // 3, n // 2, n - 1):
        tie[i] = 25.0
    out.append(("three equal maxima", tie))
    nan = lcg_row(9, n)
    nan[n // 4] = np.inf
    nan[n // 2] = np.float32(np.uint32(0xFFC00000).view(np.float32))
    nan[n - 1] = np.nan
    out.append(("NaN beside infinity, two NaNs", nan))
    z = np.full(n, -1.0, dtype=np.float32)
    z[n // 3] = -0.0
    z[n // 2] = 0.0
    out.append(("signed zeros", z))
    out.append(("all equal", np.full(n, -3.5, dtype=np.float32)))
    small = np.full(n, -np.finfo(np.float32).max, dtype=np.float32)
    small[n // 5] = np.uint32(1).view(np.float32)
    small[n // 7] = np.uint32(0x80000001).view(np.float32)
    out.append(("a subnormal maximum", small))
    return out


def host_argmax(v: np.ndarray) -> int:
    """The host's rule, written independently of the oracle: the first NaN if any, else the
    first maximum (`select::host`, named at crates/tt-tests/tests/step211_argmax_row.rs:8)."""
    best = None
    for i, x in enumerate(v.tolist()):
        if x != x:
            return i
        if best is None or x > v[best]:
            best = i
    return best
