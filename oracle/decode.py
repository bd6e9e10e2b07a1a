"""Oracle for `paged_gqa_decode`, one new token per sequence (test infrastructure; see oracle/__init__.py)."""

from __future__ import annotations

import numpy as np

MASK_VALUE = np.float32(-1e30)  # examples/decode.py:84


def to_pages(cache, block_tables, num_pages=None):
    """A contiguous cache (B, S, W) laid out in pages (num_pages, P, W) by block_tables (B, S / P)
    (examples/kv_cache.py:63-70)."""
    b, s, w = cache.shape
    per_seq = block_tables.shape[1]
    page = s // per_seq
    num_pages = b * per_seq if num_pages is None else num_pages
    pages = np.zeros((num_pages, page, w), cache.dtype)
    pages[np.asarray(block_tables).reshape(-1)] = np.asarray(cache).reshape(b * per_seq, page, w)
    return pages


def paged_gqa_decode_ref(q, k_pages, v_pages, block_tables, lengths) -> np.ndarray:
    """examples/decode.py:199-223 with T = 1, page by page in order. Query head h attends with KV head
    h // (H / Hkv) (`row_index`, :118-124; the block-diagonal layout of :127-142 only places each head's query
    against its own KV head's columns, zeros elsewhere add nothing). Per page: skip if p * P >= lengths[b]
    (:214-215); page index clamped into the pool (src/autokernel/codegen.py:1045-1048); scores f32, positions
    >= lengths[b] masked (`visible`, :145-152); `online_softmax` (:155-165) with P rounded to the cache dtype;
    `finish` (:168-172): acc * 1 / max(row_sum, 1e-30), so an empty sequence gives zeros."""
    B, T, H, Dh = q.shape
    assert T == 1
    num_pages, P, W = k_pages.shape
    Hkv = W // Dh
    G = H // Hkv
    pages = block_tables.shape[1]
    dtype = q.dtype
    qf = np.asarray(q).astype(np.float32)
    out = np.zeros((B, T, H, Dh), dtype)
    bt = np.asarray(block_tables)
    for b in range(B):
        n = int(lengths[b])
        qt = qf[b, 0].reshape(Hkv, G, Dh)
        row_max = np.full((Hkv, G, 1), MASK_VALUE, np.float32)
        row_sum = np.zeros((Hkv, G, 1), np.float32)
        acc = np.zeros((Hkv, G, Dh), np.float32)
        for p in range(pages):
            if p * P >= n:
                continue
            page = int(np.clip(bt[b, p], 0, num_pages - 1))
            kt = np.asarray(k_pages[page]).astype(np.float32).reshape(P, Hkv, Dh).transpose(1, 0, 2)
            vt = np.asarray(v_pages[page]).reshape(P, Hkv, Dh).transpose(1, 0, 2)
            s = qt @ kt.transpose(0, 2, 1)  # (Hkv, G, P)
            ok = (p * P + np.arange(P)) < n
            s = np.where(ok[None, None, :], s, MASK_VALUE)
            max_new = np.maximum(row_max, s.max(axis=2, keepdims=True))
            pr = np.exp(s - max_new)
            alpha = np.exp(row_max - max_new)
            row_sum = alpha * row_sum + pr.sum(axis=2, keepdims=True, dtype=np.float32)
            acc = alpha * acc + pr.astype(dtype).astype(np.float32) @ vt.astype(np.float32)
            row_max = max_new
        res = acc * (np.float32(1.0) / np.maximum(row_sum, np.float32(1e-30)))
        out[b, 0] = res.reshape(H, Dh).astype(dtype)
    return out


def gqa_decode_ref(q, k_cache, v_cache, lengths, block_kv: int = 512) -> np.ndarray:
    """examples/decode.py:176-196 with T = 1: the contiguous cache (B, S, Hkv * Dh) walked in blocks of
    min(block_kv, S) positions, a block skipped when its first position is >= lengths[b] (:190-191), the same
    `visible` mask, `online_softmax` and `finish` as the paged nest. Written out on its own (not through the paged
    restatement) so that the two can be checked against each other."""
    B, T, H, Dh = q.shape
    assert T == 1
    S, W = k_cache.shape[1], k_cache.shape[2]
    Hkv = W // Dh
    G = H // Hkv
    bk = min(block_kv, S)
    dtype = q.dtype
    qf = np.asarray(q).astype(np.float32)
    out = np.zeros((B, T, H, Dh), dtype)
    for b in range(B):
        n = int(lengths[b])
        qt = qf[b, 0].reshape(Hkv, G, Dh)
        row_max = np.full((Hkv, G, 1), MASK_VALUE, np.float32)
        row_sum = np.zeros((Hkv, G, 1), np.float32)
        acc = np.zeros((Hkv, G, Dh), np.float32)
        for j in range(0, S, bk):
            if j >= n:
                continue
            kt = np.asarray(k_cache[b, j : j + bk]).astype(np.float32).reshape(bk, Hkv, Dh).transpose(1, 0, 2)
            vt = np.asarray(v_cache[b, j : j + bk]).astype(np.float32).reshape(bk, Hkv, Dh).transpose(1, 0, 2)
            s = qt @ kt.transpose(0, 2, 1)
            ok = (j + np.arange(bk)) < n
            s = np.where(ok[None, None, :], s, MASK_VALUE)
            max_new = np.maximum(row_max, s.max(axis=2, keepdims=True))
            pr = np.exp(s - max_new)
            alpha = np.exp(row_max - max_new)
            row_sum = alpha * row_sum + pr.sum(axis=2, keepdims=True, dtype=np.float32)
            acc = alpha * acc + pr.astype(dtype).astype(np.float32) @ vt
            row_max = max_new
        res = acc * (np.float32(1.0) / np.maximum(row_sum, np.float32(1e-30)))
        out[b, 0] = res.reshape(H, Dh).astype(dtype)
    return out


def paged_gqa_decode_f64(q, k_pages, v_pages, block_tables, lengths) -> np.ndarray:
    """Independent check in float64 (the shape of tests/test_decode.py:62-76): gather each sequence's valid
    positions, dense softmax; zeros for an empty sequence."""
    B, T, H, Dh = q.shape
    num_pages, P, W = k_pages.shape
    Hkv = W // Dh
    G = H // Hkv
    out = np.zeros((B, T, H, Dh))
    bt = np.clip(np.asarray(block_tables), 0, num_pages - 1)
    for b in range(B):
        n = int(lengths[b])
        if n == 0:
            continue
        used = bt[b, : -(-n // P)]
        kk = np.asarray(k_pages[used]).astype(np.float64).reshape(-1, Hkv, Dh)[:n]
        vv = np.asarray(v_pages[used]).astype(np.float64).reshape(-1, Hkv, Dh)[:n]
        qq = np.asarray(q[b, 0]).astype(np.float64).reshape(Hkv, G, Dh)
        s = np.einsum("kgd,nkd->kgn", qq, kk)
        p = np.exp(s - s.max(axis=-1, keepdims=True))
        p /= p.sum(axis=-1, keepdims=True)
        out[b, 0] = np.einsum("kgn,nkd->kgd", p, vv).reshape(H, Dh)
    return out
