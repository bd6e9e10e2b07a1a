"""Oracle for `causal_attention` (test infrastructure; see oracle/__init__.py)."""

from __future__ import annotations

import numpy as np

MASK_VALUE = np.float32(-1e30)  # examples/causal_attention.py:26


def causal_attention_ref(q, k, v, block_q: int, block_kv: int) -> np.ndarray:
    """examples/causal_attention.py:37-63, blockwise and in the same order: per (b, h, query block) a running
    row max, row sum and f32 accumulator over the key blocks not wholly in the future; scores in f32 from bf16
    operands, masked elementwise with MASK_VALUE, P rounded to the input dtype before P @ v (:60), one division
    at the end. (The reference keeps the row statistics lane-replicated; that is layout, not arithmetic.)"""
    B, H, S, D = q.shape
    bq, bk = min(block_q, S), min(block_kv, S)
    dtype = q.dtype
    qf, kf, vf = (np.asarray(a).astype(np.float32) for a in (q, k, v))
    out = np.zeros((B, H, S, D), dtype)
    for b in range(B):
        for h in range(H):
            for i in range(0, S, bq):
                row_max = np.full((bq, 1), MASK_VALUE, np.float32)
                row_sum = np.zeros((bq, 1), np.float32)
                acc = np.zeros((bq, D), np.float32)
                for j in range(0, S, bk):
                    if j > i + bq - 1:
                        continue
                    s = qf[b, h, i : i + bq] @ kf[b, h, j : j + bk].T
                    rows = i + np.arange(bq)[:, None]
                    cols = j + np.arange(bk)[None, :]
                    s = np.where(cols <= rows, s, MASK_VALUE)
                    max_new = np.maximum(row_max, s.max(axis=1, keepdims=True))
                    p = np.exp(s - max_new)
                    alpha = np.exp(row_max - max_new)
                    row_sum = alpha * row_sum + p.sum(axis=1, keepdims=True, dtype=np.float32)
                    acc = alpha * acc + p.astype(dtype).astype(np.float32) @ vf[b, h, j : j + bk]
                    row_max = max_new
                out[b, h, i : i + bq] = (acc / row_sum).astype(dtype)
    return out


def causal_attention_f64(q, k, v) -> np.ndarray:
    """Independent check, as tests/test_examples.py:71-77 does it: dense softmax in float64."""
    qf, kf, vf = (np.asarray(a).astype(np.float64) for a in (q, k, v))
    S = q.shape[2]
    s = np.einsum("bhqd,bhkd->bhqk", qf, kf)
    s = np.where(np.tril(np.ones((S, S), bool)), s, -np.inf)
    p = np.exp(s - s.max(axis=-1, keepdims=True))
    p /= p.sum(axis=-1, keepdims=True)
    return np.einsum("bhqk,bhkd->bhqd", p, vf)
