"""Oracle for `attention_block` (test infrastructure; see oracle/__init__.py)."""

from __future__ import annotations

import numpy as np

from .attention import MASK_VALUE, causal_attention_f64

EPS = 1e-6  # examples/attention_block.py:26


def gelu_tanh(x: np.ndarray) -> np.ndarray:
    """jax.nn.gelu's default (approximate=True), in x's precision."""
    c = x.dtype.type(np.sqrt(2.0 / np.pi))
    return x.dtype.type(0.5) * x * (x.dtype.type(1) + np.tanh(c * (x + x.dtype.type(0.044715) * x * x * x)))


def attention_block_ref(q, k, v, gamma, w_up, w_down, block_q: int, block_kv: int, block_f: int, eps: float = EPS):
    """examples/attention_block.py:49-85, tile by tile and in the same order. Phase 1, per (b, query block): the
    online softmax of every head over the key blocks not wholly in the future (scores in f32 from bf16 operands,
    src/autokernel/mxu.py:21-43; P rounded to the input dtype before P @ v, :71); `heads = acc / row_sum` in f32,
    the heads side by side (:75-76). Then `normed` rounded to the input dtype (:77), and phase 2 over blocks of
    hidden units: gelu of the f32 product, rounded, times w_down's block, added in f32 (:79-82); one rounding of the
    tile at the end (:83)."""
    B, H, S, Dh = q.shape
    D, F = H * Dh, w_up.shape[1]
    bq, bk, bf = min(block_q, S), min(block_kv, S), min(block_f, F)
    dtype = q.dtype
    qf, kf, vf, gf, uf, df = (np.asarray(a).astype(np.float32) for a in (q, k, v, gamma, w_up, w_down))
    out = np.zeros((B, S, D), dtype)
    for b in range(B):
        for i in range(0, S, bq):
            row_max = np.full((H, bq, 1), MASK_VALUE, np.float32)
            row_sum = np.zeros((H, bq, 1), np.float32)
            acc = np.zeros((H, bq, Dh), np.float32)
            for j in range(0, S, bk):
                if j > i + bq - 1:
                    continue
                rows = i + np.arange(bq)[:, None]
                cols = j + np.arange(bk)[None, :]
                s = np.stack([np.where(cols <= rows, qf[b, h, i : i + bq] @ kf[b, h, j : j + bk].T, MASK_VALUE)
                              for h in range(H)]).astype(np.float32)
                max_new = np.maximum(row_max, s.max(axis=2, keepdims=True))
                p = np.exp(s - max_new)
                alpha = np.exp(row_max - max_new)
                row_sum = alpha * row_sum + p.sum(axis=2, keepdims=True, dtype=np.float32)
                pv = np.stack([p[h].astype(dtype).astype(np.float32) @ vf[b, h, j : j + bk] for h in range(H)])
                acc = alpha * acc + pv
                row_max = max_new
            heads = acc / row_sum
            a = np.concatenate([heads[h] for h in range(H)], axis=1)
            scale = (1.0 / np.sqrt(np.mean(a * a, axis=1, keepdims=True, dtype=np.float32) + np.float32(eps))).astype(np.float32)
            normed = (a * scale * gf[0:1, :]).astype(dtype).astype(np.float32)
            y = np.zeros((bq, D), np.float32)
            for f in range(0, F, bf):
                hidden = gelu_tanh((normed @ uf[:, f : f + bf]).astype(np.float32))
                y += hidden.astype(dtype).astype(np.float32) @ df[f : f + bf, :]
            out[b, i : i + bq, :] = y.astype(dtype)
    return out


def attention_block_f64(q, k, v, gamma, w_up, w_down, eps: float = EPS) -> np.ndarray:
    """Independent check, as tests/test_examples.py:168-176 does it: everything in float64, nothing rounded."""
    a = causal_attention_f64(q, k, v)
    B, H, S, Dh = a.shape
    a = a.transpose(0, 2, 1, 3).reshape(B, S, H * Dh)
    g, up, down = (np.asarray(x).astype(np.float64) for x in (gamma, w_up, w_down))
    normed = a / np.sqrt(np.mean(a * a, axis=-1, keepdims=True) + eps) * g
    return gelu_tanh(normed @ up) @ down
