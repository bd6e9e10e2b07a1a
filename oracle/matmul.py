"""Oracle for `matmul`, `causal_matmul` and `all_gather_matmul` (test infrastructure; see oracle/__init__.py).

The numeric rule is the reference's `@` (src/autokernel/mxu.py:21-35): bf16 operands, products accumulated in
f32, one f32 partial per reduction block added to the carried accumulator in block order, one cast at the end.
"""

from __future__ import annotations

import numpy as np


def _f32(a) -> np.ndarray:
    return np.asarray(a).astype(np.float32)


def matmul_ref(x, y, tm: int, tn: int, tk: int, out_dtype=None, causal: bool = False) -> np.ndarray:
    """examples/matmul.py:22-35 (and causal_matmul.py:23-40 with `causal`): tile by tile, acc f32 zeros,
    `acc += x[i:i+tm, k:k+tk] @ y[k:k+tk, j:j+tn]` per block, skipped tiles keep the zeros fill, diagonal tiles
    masked with `where(cols <= rows, acc, 0)`, then cast to the output dtype."""
    M, K = x.shape
    N = y.shape[1]
    tm, tn, tk = min(tm, M), min(tn, N), min(tk, K)
    out_dtype = x.dtype if out_dtype is None else out_dtype
    xf, yf = _f32(x), _f32(y)
    out = np.zeros((M, N), out_dtype)
    for i in range(0, M, tm):
        for j in range(0, N, tn):
            if causal and j > i + tm - 1:
                continue
            acc = np.zeros((tm, tn), np.float32)
            for k in range(0, K, tk):
                acc += xf[i : i + tm, k : k + tk] @ yf[k : k + tk, j : j + tn]
            if causal:
                rows = i + np.arange(tm)[:, None]
                cols = j + np.arange(tn)[None, :]
                acc = np.where(cols <= rows, acc, np.float32(0.0))
            out[i : i + tm, j : j + tn] = acc.astype(out_dtype)
    return out


def causal_matmul_ref(x, y, tm: int, tn: int, tk: int, out_dtype=None) -> np.ndarray:
    return matmul_ref(x, y, tm, tn, tk, out_dtype, causal=True)


def collective_row_order(me: int, chips: int, shard_blocks: int) -> np.ndarray:
    """The order a chip walks the row blocks of the gathered xs: a shard at a time, its own first, ring step r
    reading chip (me - r) mod chips (src/autokernel/plan.py:225-238, src/autokernel/codegen.py:958-962;
    the formula tests/test_collective.py:98-124 pins for 8 chips with 2 blocks per shard)."""
    order = []
    for i_blk in range(chips * shard_blocks):
        r, within = divmod(i_blk, shard_blocks)
        order.append(((me + chips - r) % chips) * shard_blocks + within)
    return np.array(order, np.int32)
