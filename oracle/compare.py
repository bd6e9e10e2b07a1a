"""The reference's tolerance rule for kernel-vs-reference comparisons (test infrastructure).

Follows `compare` in src/autokernel/api.py:320-364: exact for integers; rtol 1e-4 for f32; for 16-bit results, or
f32 results computed from 16-bit inputs, rtol 2e-2 and atol = 2e-2 * max|want| (at least 2e-2); NaN equals NaN.
"""

from __future__ import annotations

import numpy as np


def _is_float(dtype) -> bool:
    return np.dtype(dtype).kind == "f" or "float" in np.dtype(dtype).name


def compare(what, got, want, rtol=None, atol=None, input_dtypes=()) -> float:
    """Largest absolute difference; AssertionError beyond the tolerances (api.py:329-363)."""
    dtype = np.dtype(want.dtype)
    narrow = any(_is_float(d) and np.dtype(d).itemsize <= 2 for d in input_dtypes)
    if not _is_float(dtype):
        default = 0.0
    elif dtype.itemsize <= 2 or narrow:
        default = 2e-2
    else:
        default = 1e-4
    rtol = default if rtol is None else rtol
    g = np.asarray(got).reshape(-1).astype(np.float64)
    w = np.asarray(want).reshape(-1).astype(np.float64)
    if atol is None:
        scale = 1.0
        if default >= 2e-2 and w.size:
            finite = np.abs(w[np.isfinite(w)])
            scale = max(scale, float(finite.max(initial=0.0)))
        atol = default * scale
    same = (g == w) | (np.isnan(g) & np.isnan(w))
    with np.errstate(invalid="ignore"):
        error = float(np.max(np.abs(np.where(same, 0.0, g - w)), initial=0.0))
    differ = int(np.sum(~np.isclose(g, w, rtol=rtol, atol=atol, equal_nan=True)))
    if differ:
        raise AssertionError(
            f"{what}: the kernel and its reference differ in {differ} of {w.size} elements "
            f"(largest difference {error:.3g}; rtol={rtol}, atol={atol:.3g})"
        )
    return error
