"""Seeded synthetic inputs with the shapes and value distributions of the reference's benchmarks
(benchmarks/matmul.py:28-29, benchmarks/attention.py:32-34, benchmarks/decode.py:66-99): N(0, 1) entries rounded
to bf16, queries pre-scaled by 1/sqrt(head_dim), uniform ragged lengths, random page tables.

The reference draws with JAX's threefry PRNG, which is not reproducible without JAX; these use NumPy's PCG64
with the same seeds, so the distributions match and the streams do not.
"""

from __future__ import annotations

import numpy as np


def bf16_dtype():
    import ml_dtypes

    return ml_dtypes.bfloat16


def normal_bf16(shape, seed: int, scale: float = 1.0) -> np.ndarray:
    """N(0, 1) * scale as bf16 (NumPy array of ml_dtypes.bfloat16)."""
    x = np.random.default_rng(seed).standard_normal(shape, dtype=np.float32)
    if scale != 1.0:
        x *= np.float32(scale)
    return x.astype(bf16_dtype())


def matmul_inputs(M: int, K: int, N: int):
    return normal_bf16((M, K), 0), normal_bf16((K, N), 1)


def attention_inputs(B: int, H: int, S: int, D: int):
    q, k, v = (normal_bf16((B, H, S, D), seed) for seed in (0, 1, 2))
    q = (q.astype(np.float32) * np.float32(D**-0.5)).astype(bf16_dtype())
    return q, k, v


def decode_inputs(B: int, H: int, Hkv: int, D: int, page_size: int, pages_per_seq: int, num_pages: int,
                  distinct_pages: bool = False, seed: int = 0):
    """q [B,1,H,D], k_pages / v_pages [num_pages, page_size, Hkv*D], block_tables [B, pages_per_seq], lengths [B]
    uniform in [1, page_size * pages_per_seq]. With `distinct_pages` every (sequence, page) slot gets its own
    page (a permutation, as examples/kv_cache.py:54-60); otherwise pages are drawn with replacement."""
    rng = np.random.default_rng(seed)
    lengths = rng.integers(1, page_size * pages_per_seq + 1, B).astype(np.int32)
    if distinct_pages:
        assert B * pages_per_seq <= num_pages
        block_tables = rng.permutation(num_pages)[: B * pages_per_seq].reshape(B, pages_per_seq).astype(np.int32)
    else:
        block_tables = rng.integers(0, num_pages, (B, pages_per_seq)).astype(np.int32)
    k_pages = normal_bf16((num_pages, page_size, Hkv * D), 1)
    v_pages = normal_bf16((num_pages, page_size, Hkv * D), 2)
    q = normal_bf16((B, 1, H, D), 3, scale=D**-0.5)
    return q, k_pages, v_pages, block_tables, lengths
