"""Oracle for ragged paged attention's cache write and decode case (test infrastructure; see oracle/__init__.py)."""

from __future__ import annotations

import numpy as np

from .attention import MASK_VALUE


def rpa_inputs(q_lens, kv_lens, *, heads=32, kv_heads=8, head_dim=128, page_size=128, max_len=1024, max_tokens=None,
               max_seqs=None, seed=0, dtype=None):
    """One step's inputs in the ABI of examples/ragged_paged_attention.py:1-10 (what its `make_inputs`, :293-345,
    describes): sequences with these new-token counts and cache lengths (new tokens included), decode sequences
    (one new token) first; every sequence's pages are distinct pages of the pool, page 0 unused, entries past a
    sequence's pages arbitrary; tokens and sequences padded to `max_tokens` / `max_seqs`. The cache already holds the
    OLD positions; the new tokens' keys and values come separately."""
    import ml_dtypes

    dtype = ml_dtypes.bfloat16 if dtype is None else dtype
    rng = np.random.default_rng(seed)
    S, T = len(q_lens), int(sum(q_lens))
    assert all(q >= 1 for q in q_lens) and all(k >= q for q, k in zip(q_lens, kv_lens, strict=True))
    decodes = sum(1 for q in q_lens if q == 1)
    assert all(q == 1 for q in q_lens[:decodes]), "decode sequences first"
    max_tokens = T if max_tokens is None else max_tokens
    max_seqs = S if max_seqs is None else max_seqs
    pps = max_len // page_size
    used = [-(-k // page_size) for k in kv_lens]
    pages = sum(used) + 1
    pool = 1 + rng.permutation(pages - 1)
    table = rng.integers(0, pages, (max_seqs, pps)).astype(np.int32)
    at = 0
    for s, n in enumerate(used):
        table[s, :n] = pool[at : at + n]
        at += n
    cache = rng.standard_normal((pages, page_size, kv_heads, 2, head_dim), np.float32).astype(dtype)
    q = np.zeros((max_tokens, heads, head_dim), dtype)
    k = np.zeros((max_tokens, kv_heads, head_dim), dtype)
    v = np.zeros((max_tokens, kv_heads, head_dim), dtype)
    q[:T] = rng.standard_normal((T, heads, head_dim), np.float32).astype(dtype)
    k[:T] = rng.standard_normal((T, kv_heads, head_dim), np.float32).astype(dtype)
    v[:T] = rng.standard_normal((T, kv_heads, head_dim), np.float32).astype(dtype)
    lens = np.zeros(max_seqs, np.int32)
    lens[:S] = kv_lens
    cu = np.full(max_seqs + 1, T, np.int32)
    cu[: S + 1] = np.concatenate([[0], np.cumsum(q_lens)])
    return dict(q=q, keys=k, values=v, kv_cache=cache, kv_lens=lens, page_indices=table.reshape(-1),
                cu_q_lens=cu, distribution=np.array([decodes, decodes, S], np.int32))


def rpa_write_runs(kv_lens, page_indices, cu_q_lens, distribution, page_size: int, max_tokens: int) -> dict:
    """`writes` (examples/ragged_paged_attention.py:49-71) in NumPy: sequence s's new tokens, at positions
    [kv_len - q_len, kv_len), cut at page boundaries; int32 arrays of the run count's bound, cdiv(T, page_size) + S,
    in the order of `rpa_write`'s parameters, n_writes of shape (1,)."""
    S = kv_lens.shape[0]
    pps = page_indices.shape[0] // S
    seqs = np.arange(S)
    q_len = np.where(seqs < distribution[2], cu_q_lens[1:] - cu_q_lens[:-1], 0)
    first = kv_lens - q_len
    n_runs = np.where(q_len > 0, (kv_lens - 1) // page_size - first // page_size + 1, 0)
    ends = np.cumsum(n_runs)
    w = np.arange(-(-max_tokens // page_size) + S)
    seq = np.minimum((ends[None, :] <= w[:, None]).sum(axis=1), S - 1)
    page = first[seq] // page_size + w - (ends[seq] - n_runs[seq])
    start = np.maximum(first[seq], page * page_size)
    i32 = lambda a: np.asarray(a, np.int32)  # noqa: E731
    return dict(write_page=i32(seq * pps + page), write_rows=i32(cu_q_lens[seq] + start - first[seq]),
                write_first=i32(start - page * page_size),
                write_stop=i32(np.minimum(kv_lens[seq], (page + 1) * page_size) - page * page_size),
                n_writes=i32(ends[-1:]))


def rpa_write_ref(kv_cache, keys, values, kv_lens, page_indices, cu_q_lens, distribution) -> np.ndarray:
    """examples/ragged_paged_attention.py:33-79 token by token: sequence s < distribution[2] has q_len =
    cu_q_lens[s + 1] - cu_q_lens[s] new tokens at positions [kv_len - q_len, kv_len) (:56-58); position p lives in page
    page_indices[s * pps + p // page_size] at row p % page_size (:63-71), key in [..., 0, :] and value in [..., 1, :]
    (`key_value_words` / `unpairs`, :101-105 and src/autokernel/packing.py:28-31). The runs of `writes` only batch
    these per page."""
    out = np.array(kv_cache, copy=True)
    ps = out.shape[1]
    S = kv_lens.shape[0]
    pps = page_indices.shape[0] // S
    for s in range(min(S, int(distribution[2]))):
        first, q_len = int(cu_q_lens[s]), int(cu_q_lens[s + 1] - cu_q_lens[s])
        for i in range(q_len):
            p = int(kv_lens[s]) - q_len + i
            page = int(page_indices[s * pps + p // ps])
            out[page, p % ps, :, 0, :] = keys[first + i]
            out[page, p % ps, :, 1, :] = values[first + i]
    return out


def rpa_decode_ref(q, kv_cache, kv_lens, page_indices, distribution, sm_scale: float) -> np.ndarray:
    """examples/ragged_paged_attention.py:121-149, page by page and in the same order: for sequence s < min(S, T) the
    query rows (H, D) score every KV head's keys of a page, `(qs @ k.T) * sm_scale` in f32 (:140), masked to the
    row's own KV head and to positions before kv_lens[s] (`own_heads`, :84-93); `online_softmax` (:96-107) with P
    rounded to the cache dtype before P @ v; `acc / max(row_sum, 1e-30)`; rows of sequences from distribution[0] on
    keep the query (:147)."""
    T, H, D = q.shape
    ps, Hkv = kv_cache.shape[1], kv_cache.shape[2]
    G = H // Hkv
    S = kv_lens.shape[0]
    pps = page_indices.shape[0] // S
    dtype = q.dtype
    out = np.array(q, copy=True)
    scale = np.float32(sm_scale)
    for s in range(min(S, T)):
        if s >= int(distribution[0]):
            continue
        qs = np.asarray(q[s]).astype(np.float32)
        n = int(kv_lens[s])
        row_max = np.full((H, 1), MASK_VALUE, np.float32)
        row_sum = np.zeros((H, 1), np.float32)
        acc = np.zeros((H, D), np.float32)
        for p in range((n + ps - 1) // ps):
            page = np.asarray(kv_cache[int(page_indices[s * pps + p])]).astype(np.float32)  # (ps, Hkv, 2, D)
            sc = np.full((H, ps), MASK_VALUE, np.float32)
            pv_in = np.zeros((H, ps, D), np.float32)
            ok = (p * ps + np.arange(ps)) < n
            for h in range(H):
                g = h // G
                sc[h] = np.where(ok, (qs[h] @ page[:, g, 0, :].T) * scale, MASK_VALUE)
                pv_in[h] = page[:, g, 1, :]
            max_new = np.maximum(row_max, sc.max(axis=1, keepdims=True))
            pr = np.exp(sc - max_new)
            alpha = np.exp(row_max - max_new)
            row_sum = alpha * row_sum + pr.sum(axis=1, keepdims=True, dtype=np.float32)
            prb = pr.astype(dtype).astype(np.float32)
            acc = alpha * acc + np.einsum("hp,hpd->hd", prb, pv_in).astype(np.float32)
            row_max = max_new
        out[s] = (acc * (np.float32(1.0) / np.maximum(row_sum, np.float32(1e-30)))).astype(dtype)
    return out


def rpa_decode_f64(q, kv_cache, kv_lens, page_indices, distribution, sm_scale: float) -> np.ndarray:
    """Independent check in float64: dense softmax over each decode sequence's cached positions."""
    T, H, D = q.shape
    ps, Hkv = kv_cache.shape[1], kv_cache.shape[2]
    G = H // Hkv
    S = kv_lens.shape[0]
    pps = page_indices.shape[0] // S
    out = np.asarray(q).astype(np.float64)
    for s in range(min(S, T, int(distribution[0]))):
        n = int(kv_lens[s])
        if n == 0:
            out[s] = 0
            continue
        pages = [int(page_indices[s * pps + p]) for p in range((n + ps - 1) // ps)]
        kv = np.concatenate([np.asarray(kv_cache[pg]).astype(np.float64) for pg in pages])[:n]  # (n, Hkv, 2, D)
        for h in range(H):
            sc = kv[:, h // G, 0, :] @ np.asarray(q[s, h]).astype(np.float64) * sm_scale
            w = np.exp(sc - sc.max())
            out[s, h] = (w / w.sum()) @ kv[:, h // G, 1, :]
    return out


BLOCK_Q = 256  # examples/ragged_paged_attention.py:154


def rpa_prefill_tiles(kv_lens, page_indices, cu_q_lens, distribution, max_tokens: int, block_q: int = BLOCK_Q) -> dict:
    """`prefill_tiles` (examples/ragged_paged_attention.py:252-275) in NumPy: a tile per block of block_q queries of
    each sequence in [distribution[0], distribution[2]); int32 arrays of the tile count's bound, cdiv(T, block_q) + S
    (tile_rows one longer), in the order of `rpa_prefill`'s parameters, n_tiles of shape (1,)."""
    S = kv_lens.shape[0]
    pps = page_indices.shape[0] // S
    seqs = np.arange(S)
    q_len = cu_q_lens[1:] - cu_q_lens[:-1]
    mixed = (seqs >= distribution[0]) & (seqs < distribution[2])
    blocks = np.where(mixed, (q_len + block_q - 1) // block_q, 0)
    ends = np.cumsum(blocks)
    k = np.arange(-(-max_tokens // block_q) + S)
    seq = np.minimum((ends[None, :] <= k[:, None]).sum(axis=1), S - 1)
    b = k - (ends[seq] - blocks[seq])
    rows = cu_q_lens[seq] + b * block_q
    stop = np.minimum(rows + block_q, cu_q_lens[seq + 1])
    pos = kv_lens[seq] - q_len[seq] + b * block_q
    i32 = lambda a: np.asarray(a, np.int32)  # noqa: E731
    return dict(tile_page=i32(seq * pps), tile_rows=i32(np.concatenate([rows[:1], stop])), tile_pos=i32(pos),
                tile_stop=i32(pos + (stop - rows)), n_tiles=i32(ends[-1:]))


def rpa_prefill_ref(q, kv_cache, kv_lens, page_indices, cu_q_lens, distribution, sm_scale: float, pages_per_step: int = 4):
    """examples/ragged_paged_attention.py:196-275, tile by tile and step by step: a tile is a block of up to 256 new
    tokens of a sequence in [distribution[0], distribution[2]) (`prefill_tiles`, :252-275), its first token at cache
    position kv_len - q_len + 256 b; a step is `pages_per_step` pages (:219); scores `s * sm_scale` in f32 (:232),
    a query at position p sees the positions up to p (`visible`, :172-181); `online_softmax_heads` (:184-193) with P
    rounded to the cache dtype before P @ v; rows not in a tile keep q."""
    T, H, D = q.shape
    ps, Hkv = kv_cache.shape[1], kv_cache.shape[2]
    G = H // Hkv
    S = kv_lens.shape[0]
    pps = page_indices.shape[0] // S
    dtype = q.dtype
    out = np.array(q, copy=True)
    scale = np.float32(sm_scale)
    for s in range(int(distribution[0]), min(S, int(distribution[2]))):
        first, q_len = int(cu_q_lens[s]), int(cu_q_lens[s + 1] - cu_q_lens[s])
        for b0 in range(0, q_len, BLOCK_Q):
            rows = min(BLOCK_Q, q_len - b0)
            pos0 = int(kv_lens[s]) - q_len + b0
            stop = pos0 + rows
            qt = np.asarray(q[first + b0 : first + b0 + rows]).astype(np.float32)  # (rows, H, D)
            row_max = np.full((H, rows, 1), MASK_VALUE, np.float32)
            row_sum = np.zeros((H, rows, 1), np.float32)
            acc = np.zeros((H, rows, D), np.float32)
            pos = pos0 + np.arange(rows)[:, None]
            for j in range(0, stop, pages_per_step * ps):
                pages = [int(page_indices[s * pps + min(j // ps + x, pps - 1)]) for x in range(pages_per_step)]
                kv = np.concatenate([np.asarray(kv_cache[pg]).astype(np.float32) for pg in pages])  # (NP * ps, Hkv, 2, D)
                col = j + np.arange(kv.shape[0])[None, :]
                ok = (col <= pos) & (col < stop)
                sc = np.stack([np.where(ok, (qt[:, h, :] @ kv[:, h // G, 0, :].T) * scale, MASK_VALUE) for h in range(H)])
                max_new = np.maximum(row_max, sc.max(axis=2, keepdims=True))
                pr = np.exp(sc - max_new)
                alpha = np.exp(row_max - max_new)
                row_sum = alpha * row_sum + pr.sum(axis=2, keepdims=True, dtype=np.float32)
                prb = pr.astype(dtype).astype(np.float32)
                acc = alpha * acc + np.stack([prb[h] @ kv[:, h // G, 1, :] for h in range(H)])
                row_max = max_new
            o = acc * (np.float32(1.0) / np.maximum(row_sum, np.float32(1e-30)))
            out[first + b0 : first + b0 + rows] = o.transpose(1, 0, 2).astype(dtype)
    return out


def rpa_prefill_f64(q, kv_cache, kv_lens, page_indices, cu_q_lens, distribution, sm_scale: float) -> np.ndarray:
    """Independent check in float64: dense causal softmax of every new token of the prefill / mixed sequences over
    its sequence's cached positions up to its own."""
    T, H, D = q.shape
    ps, Hkv = kv_cache.shape[1], kv_cache.shape[2]
    G = H // Hkv
    S = kv_lens.shape[0]
    pps = page_indices.shape[0] // S
    out = np.asarray(q).astype(np.float64)
    for s in range(int(distribution[0]), min(S, int(distribution[2]))):
        first, q_len, n = int(cu_q_lens[s]), int(cu_q_lens[s + 1] - cu_q_lens[s]), int(kv_lens[s])
        if q_len == 0:
            continue
        pages = [int(page_indices[s * pps + x]) for x in range((n + ps - 1) // ps)]
        kv = np.concatenate([np.asarray(kv_cache[pg]).astype(np.float64) for pg in pages])[:n]
        for i in range(q_len):
            seen = n - q_len + i + 1
            for h in range(H):
                sc = kv[:seen, h // G, 0, :] @ np.asarray(q[first + i, h]).astype(np.float64) * sm_scale
                w = np.exp(sc - sc.max())
                out[first + i, h] = (w / w.sum()) @ kv[:seen, h // G, 1, :]
    return out
