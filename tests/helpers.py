"""Helpers shared by the parity tests: tolerances in the reference's convention and comparison."""
import math

import numpy as np

# Per-element tolerances of the reference's tests (test/test_add.py:23-24, test/test_loss.py:130-131).
RTOL = {"float32": 1.3e-6, "bfloat16": 1.6e-2, "float16": 1e-3, "float64": 1e-12}
ATOL = {"float32": 1e-5, "bfloat16": 1e-5, "float16": 1e-5, "float64": 1e-12}


def accumulation_tol(n, dtype="float32"):
    """Tolerance of a reduction over n terms, the rule of test/test_loss.py:134-146:
    k = 4 (log2 n - 4) for n > 32, rtol = k * 1.3e-6, atol = k * 1e-5; 16-bit types use fixed values."""
    if dtype in ("bfloat16", "float16"):
        return 1.6e-2, 1e-3
    k = 4.0 * (math.log2(n) - 4.0) if n > 32 else 1.0
    return k * 1.3e-6, k * 1e-5


def assert_close(actual, expected, rtol, atol, what=""):
    a = np.asarray(actual, dtype=np.float64)
    e = np.asarray(expected, dtype=np.float64)
    assert a.shape == e.shape, f"{what}: shape {a.shape} vs {e.shape}"
    nan_a, nan_e = np.isnan(a), np.isnan(e)
    assert np.array_equal(nan_a, nan_e), f"{what}: NaN pattern differs"
    inf_mask = np.isinf(e)
    assert np.array_equal(a[inf_mask], e[inf_mask]), f"{what}: infinities differ"
    ok = ~(nan_e | inf_mask)
    diff = np.abs(a[ok] - e[ok])
    bound = atol + rtol * np.abs(e[ok])
    if not np.all(diff <= bound):
        worst = np.argmax(diff - bound)
        raise AssertionError(
            f"{what}: {np.count_nonzero(diff > bound)} of {diff.size} elements out of tolerance "
            f"(rtol={rtol}, atol={atol}); worst |diff|={diff[worst]:.3e} at expected={e[ok][worst]:.6e} "
            f"actual={a[ok][worst]:.6e}")


def rel_err(actual, expected):
    a, e = float(actual), float(expected)
    return abs(a - e) / max(abs(e), 1e-30)
