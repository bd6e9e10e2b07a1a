"""Oracle for `gqa_decode` and `paged_gqa_decode`, T new tokens per sequence (test infrastructure; see
oracle/__init__.py)."""

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


def _rows_by_kv_head(qb, kv_heads):
    """A sequence's queries (T, H, Dh) as (Hkv, T * G, Dh) in f32: KV head k's rows are (token t, its query head g),
    t-major — the rows `row_index` assigns to group k (examples/decode.py:118-124)."""
    T, H, Dh = qb.shape
    G = H // kv_heads
    return np.asarray(qb).astype(np.float32).reshape(T, kv_heads, G, Dh).transpose(1, 0, 2, 3).reshape(kv_heads, T * G, Dh)


def _visible(first, count, length, T, G):
    """(1, T * G, count): may row (t, g) attend to position first + c? `visible` (examples/decode.py:145-152): new
    token t sits at position length - T + t and sees the positions up to its own; for T = 1 that is c < length."""
    cols = first + np.arange(count)
    tok = np.repeat(np.arange(T), G)
    return (cols[None, :] <= (length - T + tok)[:, None])[None]


def _rows_to_output(res, T, H, kv_heads, dtype):
    """(Hkv, T * G, Dh) back to (T, H, Dh)."""
    G = H // kv_heads
    return res.reshape(kv_heads, T, G, -1).transpose(1, 0, 2, 3).reshape(T, H, -1).astype(dtype)


def paged_gqa_decode_ref(q, k_pages, v_pages, block_tables, lengths) -> np.ndarray:
    """examples/decode.py:199-223 with T = 1, page by page in order. Query head h attends with KV head
    h // (H / Hkv) (`row_index`, :118-124; the block-diagonal layout of :127-142 only places each head's query
    against its own KV head's columns, zeros elsewhere add nothing). Per page: skip if p * P >= lengths[b]
    (:214-215); page index clamped into the pool (src/autokernel/codegen.py:1045-1048); scores f32, positions
    >= lengths[b] masked (`visible`, :145-152); `online_softmax` (:155-165) with P rounded to the cache dtype;
    `finish` (:168-172): acc * 1 / max(row_sum, 1e-30), so an empty sequence gives zeros."""
    B, T, H, Dh = q.shape
    num_pages, P, W = k_pages.shape
    Hkv = W // Dh
    G = H // Hkv
    pages = block_tables.shape[1]
    dtype = q.dtype
    out = np.zeros((B, T, H, Dh), dtype)
    bt = np.asarray(block_tables)
    for b in range(B):
        n = int(lengths[b])
        qt = _rows_by_kv_head(q[b], Hkv)
        row_max = np.full((Hkv, T * G, 1), MASK_VALUE, np.float32)
        row_sum = np.zeros((Hkv, T * G, 1), np.float32)
        acc = np.zeros((Hkv, T * G, Dh), np.float32)
        for p in range(pages):
            if p * P >= n:
                continue
            page = int(np.clip(bt[b, p], 0, num_pages - 1))
            kt = np.asarray(k_pages[page]).astype(np.float32).reshape(P, Hkv, Dh).transpose(1, 0, 2)
            vt = np.asarray(v_pages[page]).reshape(P, Hkv, Dh).transpose(1, 0, 2)
            s = qt @ kt.transpose(0, 2, 1)  # (Hkv, T * G, P)
            s = np.where(_visible(p * P, P, n, T, G), s, MASK_VALUE)
            max_new = np.maximum(row_max, s.max(axis=2, keepdims=True))
            pr = np.exp(s - max_new)
            alpha = np.exp(row_max - max_new)
            row_sum = alpha * row_sum + pr.sum(axis=2, keepdims=True, dtype=np.float32)
            acc = alpha * acc + pr.astype(dtype).astype(np.float32) @ vt.astype(np.float32)
            row_max = max_new
        res = acc * (np.float32(1.0) / np.maximum(row_sum, np.float32(1e-30)))
        out[b] = _rows_to_output(res, T, H, Hkv, dtype)
    return out


def gqa_decode_ref(q, k_cache, v_cache, lengths, block_kv: int = 512) -> np.ndarray:
    """examples/decode.py:176-196 with T = 1: the contiguous cache (B, S, Hkv * Dh) walked in blocks of
    min(block_kv, S) positions, a block skipped when its first position is >= lengths[b] (:190-191), the same
    `visible` mask, `online_softmax` and `finish` as the paged nest. Written out on its own (not through the paged
    restatement) so that the two can be checked against each other."""
    B, T, H, Dh = q.shape
    S, W = k_cache.shape[1], k_cache.shape[2]
    Hkv = W // Dh
    G = H // Hkv
    bk = min(block_kv, S)
    dtype = q.dtype
    out = np.zeros((B, T, H, Dh), dtype)
    for b in range(B):
        n = int(lengths[b])
        qt = _rows_by_kv_head(q[b], Hkv)
        row_max = np.full((Hkv, T * G, 1), MASK_VALUE, np.float32)
        row_sum = np.zeros((Hkv, T * G, 1), np.float32)
        acc = np.zeros((Hkv, T * G, Dh), np.float32)
        for j in range(0, S, bk):
            if j >= n:
                continue
            kt = np.asarray(k_cache[b, j : j + bk]).astype(np.float32).reshape(bk, Hkv, Dh).transpose(1, 0, 2)
            vt = np.asarray(v_cache[b, j : j + bk]).astype(np.float32).reshape(bk, Hkv, Dh).transpose(1, 0, 2)
            s = qt @ kt.transpose(0, 2, 1)
            s = np.where(_visible(j, bk, n, T, G), s, MASK_VALUE)
            max_new = np.maximum(row_max, s.max(axis=2, keepdims=True))
            pr = np.exp(s - max_new)
            alpha = np.exp(row_max - max_new)
            row_sum = alpha * row_sum + pr.sum(axis=2, keepdims=True, dtype=np.float32)
            acc = alpha * acc + pr.astype(dtype).astype(np.float32) @ vt
            row_max = max_new
        res = acc * (np.float32(1.0) / np.maximum(row_sum, np.float32(1e-30)))
        out[b] = _rows_to_output(res, T, H, Hkv, dtype)
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
        kk = np.asarray(k_pages[used]).astype(np.float64).reshape(-1, Hkv, Dh)
        vv = np.asarray(v_pages[used]).astype(np.float64).reshape(-1, Hkv, Dh)
        for t in range(T):
            seen = n - T + t + 1  # new token t sits at position n - T + t and sees the positions up to its own
            if seen <= 0:
                continue
            qq = np.asarray(q[b, t]).astype(np.float64).reshape(Hkv, G, Dh)
            s = np.einsum("kgd,nkd->kgn", qq, kk[:seen])
            p = np.exp(s - s.max(axis=-1, keepdims=True))
            p /= p.sum(axis=-1, keepdims=True)
            out[b, t] = np.einsum("kgn,nkd->kgd", p, vv[:seen]).reshape(H, Dh)
    return out


def mla_decode_ref(q_c, q_r, c_kv, k_rope, lengths, block_kv: int = 512) -> np.ndarray:
    """examples/decode.py:226-250: a sequence's rows are its (new token, head) pairs, token-major (`query_rows`,
    :104-107); scores `qc @ ct.T + qr @ k_rope.T` in f32 from the cache dtype's operands (:246), blocks of
    min(block_kv, S) positions skipped when their first position is >= lengths[b] (:243-244), `visible` (new token t
    sees the positions up to lengths[b] - T + t, :145-152) and `online_softmax` against the latents themselves
    (:247-248), `finish` (:249)."""
    B, T, H, C = q_c.shape
    S = c_kv.shape[1]
    bk = min(block_kv, S)
    dtype = q_c.dtype
    out = np.zeros((B, T, H, C), dtype)
    token = (np.arange(T * H) // H)[:, None]
    for b in range(B):
        n = int(lengths[b])
        qc = np.asarray(q_c[b]).reshape(T * H, C).astype(np.float32)
        qr = np.asarray(q_r[b]).reshape(T * H, -1).astype(np.float32)
        row_max = np.full((T * H, 1), MASK_VALUE, np.float32)
        row_sum = np.zeros((T * H, 1), np.float32)
        acc = np.zeros((T * H, C), np.float32)
        for j in range(0, S, bk):
            if j >= n:
                continue
            ct = np.asarray(c_kv[b, j : j + bk]).astype(np.float32)
            s = qc @ ct.T + qr @ np.asarray(k_rope[b, j : j + bk]).astype(np.float32).T
            s = np.where((j + np.arange(bk))[None, :] <= n - T + token, s, MASK_VALUE)
            max_new = np.maximum(row_max, s.max(axis=1, keepdims=True))
            pr = np.exp(s - max_new)
            alpha = np.exp(row_max - max_new)
            row_sum = alpha * row_sum + pr.sum(axis=1, keepdims=True, dtype=np.float32)
            acc = alpha * acc + pr.astype(dtype).astype(np.float32) @ ct
            row_max = max_new
        out[b] = (acc * (np.float32(1.0) / np.maximum(row_sum, np.float32(1e-30)))).astype(dtype).reshape(T, H, C)
    return out


def mla_decode_f64(q_c, q_r, c_kv, k_rope, lengths) -> np.ndarray:
    """Independent check in float64 (`xla_mla_decode`, examples/decode.py:305-310): dense softmax over the valid
    positions; zeros for an empty sequence."""
    B, T, H, C = q_c.shape
    out = np.zeros((B, T, H, C))
    for b in range(B):
        n = int(lengths[b])
        for t in range(T):
            seen = n - T + t + 1  # new token t sees the positions before this one
            if seen <= 0:
                continue
            c = np.asarray(c_kv[b, :seen]).astype(np.float64)
            s = np.asarray(q_c[b, t]).astype(np.float64) @ c.T
            s += np.asarray(q_r[b, t]).astype(np.float64) @ np.asarray(k_rope[b, :seen]).astype(np.float64).T
            p = np.exp(s - s.max(axis=1, keepdims=True))
            p /= p.sum(axis=1, keepdims=True)
            out[b, t] = p @ c
    return out
