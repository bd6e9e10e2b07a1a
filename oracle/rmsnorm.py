"""CPU restatement of `rmsnorm_matmul` (examples/rmsnorm_matmul.py:31-47). Test infrastructure only."""

from __future__ import annotations

import numpy as np

from .matmul import _f32


def rmsnorm_matmul_ref(x, gamma, w, tm: int, tn: int, tk: int, eps: float = 1e-6, out_dtype=None) -> np.ndarray:
    """Tile by tile, as the loop nest: per k block the row's squares are summed in f32 and
    `(xk * gamma_k)` — rounded to the input dtype, examples/rmsnorm_matmul.py:44 — is multiplied with w's block,
    accumulating in f32 (src/autokernel/mxu.py:21-35); the tile is scaled by rsqrt(sum_sq / D + eps) and cast once."""
    M, D = x.shape
    N = w.shape[1]
    tm, tn, tk = min(tm, M), min(tn, N), min(tk, D)
    out_dtype = x.dtype if out_dtype is None else out_dtype
    out = np.zeros((M, N), out_dtype)
    xf, gf, wf = _f32(x), _f32(gamma), _f32(w)
    for i in range(0, M, tm):
        for j in range(0, N, tn):
            acc = np.zeros((tm, tn), np.float32)
            sum_sq = np.zeros((tm, 1), np.float32)
            for k in range(0, D, tk):
                xk = xf[i : i + tm, k : k + tk]
                sum_sq += np.sum(xk * xk, axis=1, keepdims=True, dtype=np.float32)
                scaled = (xk * gf[0:1, k : k + tk]).astype(x.dtype).astype(np.float32)
                acc += scaled @ wf[k : k + tk, j : j + tn]
            scale = (1.0 / np.sqrt(sum_sq / np.float32(D) + np.float32(eps))).astype(np.float32)
            out[i : i + tm, j : j + tn] = (acc * scale).astype(out_dtype)
    return out


def rmsnorm_matmul_f64(x, gamma, w, eps: float = 1e-6) -> np.ndarray:
    """Independent check in float64: rmsnorm(x) @ w with nothing rounded in between."""
    xf, gf, wf = (np.asarray(a).astype(np.float64) for a in (x, gamma, w))
    normed = xf / np.sqrt(np.mean(xf * xf, axis=1, keepdims=True) + eps) * gf
    return normed @ wf
