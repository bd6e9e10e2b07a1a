"""The hot-path loop nests, written against this package: the workloads the sm_100a kernels run.

Each is the plain loop nest over tiles whose meaning the kernel must reproduce — `kernel.fn` runs it as written on
the CPU — with the same structure as the reference's examples (examples/matmul.py, causal_matmul.py,
causal_attention.py, rmsnorm_matmul.py, decode.py `gqa_decode`, `mla_decode` and `paged_gqa_decode`,
ragged_paged_attention.py `rpa_write`, `rpa_decode`, `rpa_prefill` and the step `autokernel_rpa`,
collective_matmul.py). Row statistics are kept as (rows, 1)
columns here: the reference's lane-replicated (rows, 128) layout is a TPU register trick, not arithmetic.
"""

from __future__ import annotations

import tilejax_b200.autokernel as autokernel
from tilejax_b200.autokernel import jaxlike as jax

jnp = jax.numpy
MASK_VALUE = -1e30  # finite, so exp(old max - new max) never computes -inf + inf


@autokernel.tunable
class MatmulTiles:
    """(tm, tn) output tiles, each summing tk-deep products."""

    tm: int = autokernel.choice(128, 256, 512, 1024, 2048, default=512)
    tn: int = autokernel.choice(128, 256, 512, 1024, 2048, default=512)
    tk: int = autokernel.choice(128, 256, 512, 1024, 2048, default=512)


@autokernel.tunable
class AttentionBlocks:
    """Queries and keys per block."""

    block_q: int = autokernel.choice(128, 256, 512, 1024, default=512)
    block_kv: int = autokernel.choice(128, 256, 512, 1024, default=512)


@autokernel.tunable
class CollectiveTiles:
    """(tm, tn) output tiles summing tk-deep products; tm rows at a time of one rank's shard of x."""

    tm: int = autokernel.choice(128, 256, 512, 1024, default=256)
    tn: int = autokernel.choice(128, 256, 512, 1024, 2048, default=512)
    tk: int = autokernel.choice(128, 256, 512, 1024, 2048, default=512)


@autokernel.tunable
class DecodeTiles:
    """Cache positions per step."""

    block_kv: int = autokernel.choice(128, 256, 512, 1024, 2048, default=512)


@autokernel.kernel
def matmul(x, y, tiles=MatmulTiles()):
    M, K = x.shape
    N = y.shape[1]
    tm, tn, tk = min(tiles.tm, M), min(tiles.tn, N), min(tiles.tk, K)
    dtype = x.dtype
    out = jnp.zeros((M, N), dtype)
    for i in range(0, M, tm):
        for j in range(0, N, tn):
            acc = jnp.zeros((tm, tn), jnp.float32)
            for k in range(0, K, tk):
                acc += x[i : i + tm, k : k + tk] @ y[k : k + tk, j : j + tn]
            out = out.at[i : i + tm, j : j + tn].set(acc.astype(dtype))
    return out


@autokernel.kernel
def causal_matmul(x, y, tiles=MatmulTiles()):
    M, K = x.shape
    N = y.shape[1]
    tm, tn, tk = min(tiles.tm, M), min(tiles.tn, N), min(tiles.tk, K)
    dtype = x.dtype
    out = jnp.zeros((M, N), dtype)
    for i in range(0, M, tm):
        for j in range(0, N, tn):
            if j > i + tm - 1:  # the whole tile is above the diagonal
                continue
            acc = jnp.zeros((tm, tn), jnp.float32)
            for k in range(0, K, tk):
                acc += x[i : i + tm, k : k + tk] @ y[k : k + tk, j : j + tn]
            rows = i + jax.lax.broadcasted_iota(jnp.int32, (tm, tn), 0)
            cols = j + jax.lax.broadcasted_iota(jnp.int32, (tm, tn), 1)
            out = out.at[i : i + tm, j : j + tn].set(jnp.where(cols <= rows, acc, 0.0).astype(dtype))
    return out


EPS = 1e-6


@autokernel.tunable
class NormMatmulTiles:
    """(tm, tn) output tiles, each summing tk-deep products (and tm rows' squares) over the model dim."""

    tm: int = autokernel.choice(128, 256, 512, 1024, 2048, default=512)
    tn: int = autokernel.choice(128, 256, 512, 1024, 2048, default=512)
    tk: int = autokernel.choice(128, 256, 512, 1024, 2048, default=512)


@autokernel.kernel
def rmsnorm_matmul(x, gamma, w, tiles=NormMatmulTiles()):
    """rmsnorm(x) @ w in one pass over x: the row scale commutes with the matmul, so one reduction accumulates
    (x * gamma) @ w and each row's sum of squares, and the tile is scaled once at the end."""
    M, D = x.shape
    N = w.shape[1]
    tm, tn, tk = min(tiles.tm, M), min(tiles.tn, N), min(tiles.tk, D)
    dtype = x.dtype
    out = jnp.zeros((M, N), dtype)
    for i in range(0, M, tm):
        for j in range(0, N, tn):
            acc = jnp.zeros((tm, tn), jnp.float32)  # (x * gamma) @ w
            sum_sq = jnp.zeros((tm, 1), jnp.float32)  # each row's sum of squares
            for k in range(0, D, tk):
                xk = x[i : i + tm, k : k + tk].astype(jnp.float32)
                sum_sq += jnp.sum(xk * xk, axis=1, keepdims=True)
                acc += (xk * gamma[0:1, k : k + tk].astype(jnp.float32)).astype(dtype) @ w[k : k + tk, j : j + tn]
            scale = jax.lax.rsqrt(sum_sq / D + EPS)
            out = out.at[i : i + tm, j : j + tn].set((acc * scale).astype(dtype))
    return out


@autokernel.kernel
def causal_attention(q, k, v, blocks=AttentionBlocks()):
    B, H, S, D = q.shape
    bq, bk = min(blocks.block_q, S), min(blocks.block_kv, S)
    dtype = q.dtype
    out = jnp.zeros((B, H, S, D), dtype)
    for b in range(B):
        for h in range(H):
            for i in range(0, S, bq):
                row_max = jnp.full((bq, 1), MASK_VALUE, jnp.float32)
                row_sum = jnp.zeros((bq, 1), jnp.float32)  # of exp(s - row_max)
                acc = jnp.zeros((bq, D), jnp.float32)  # sum of exp(s - row_max) @ v
                for j in range(0, S, bk):
                    if j > i + bq - 1:  # every key is in the future of every query
                        continue
                    s = q[b, h, i : i + bq, :] @ k[b, h, j : j + bk, :].T
                    rows = i + jax.lax.broadcasted_iota(jnp.int32, (bq, bk), 0)
                    cols = j + jax.lax.broadcasted_iota(jnp.int32, (bq, bk), 1)
                    s = jnp.where(cols <= rows, s, MASK_VALUE)
                    max_new = jnp.maximum(row_max, jnp.max(s, axis=1, keepdims=True))
                    p = jnp.exp(s - max_new)
                    alpha = jnp.exp(row_max - max_new)
                    row_sum = alpha * row_sum + jnp.sum(p, axis=1, keepdims=True)
                    acc = alpha * acc + p.astype(dtype) @ v[b, h, j : j + bk, :]
                    row_max = max_new
                out = out.at[b, h, i : i + bq, :].set((acc / row_sum).astype(dtype))
    return out


@autokernel.tunable
class BlockTiles:
    """Queries per output tile, keys per attention step, and hidden units per feed-forward step (one block of all
    of them makes the feed-forward phase a single step)."""

    block_q: int = autokernel.choice(128, 256, 512, 1024, default=256)
    block_kv: int = autokernel.choice(128, 256, 512, 1024, default=256)
    block_f: int = autokernel.choice(256, 512, 1024, 2048, 4096, 8192, 16384, default=1024)


@autokernel.kernel
def attention_block(q, k, v, gamma, w_up, w_down, tiles=BlockTiles()):
    """Causal multi-head attention, the RMSNorm after it and the feed-forward layer: per (batch, query block) two
    reduction loops, one after the other — the key blocks (an online softmax for every head), then, with the heads
    side by side and normalised together, the blocks of hidden units. q arrives pre-scaled."""
    B, H, S, Dh = q.shape
    D, F = H * Dh, w_up.shape[1]
    bq, bk, bf = min(tiles.block_q, S), min(tiles.block_kv, S), min(tiles.block_f, F)
    dtype = q.dtype
    out = jnp.zeros((B, S, D), dtype)
    for b in range(B):
        for i in range(0, S, bq):
            row_max = jnp.full((H, bq, 1), MASK_VALUE, jnp.float32)
            row_sum = jnp.zeros((H, bq, 1), jnp.float32)  # of exp(s - row_max)
            acc = jnp.zeros((H, bq, Dh), jnp.float32)  # sum of exp(s - row_max) @ v
            for j in range(0, S, bk):  # phase 1: causal attention, every head
                if j > i + bq - 1:  # every key is in the future of every query
                    continue
                qt, kt, vt = q[b, :, i : i + bq, :], k[b, :, j : j + bk, :], v[b, :, j : j + bk, :]
                rows = i + jax.lax.broadcasted_iota(jnp.int32, (bq, bk), 0)
                cols = j + jax.lax.broadcasted_iota(jnp.int32, (bq, bk), 1)
                s = jnp.stack([jnp.where(cols <= rows, qt[h] @ kt[h].T, MASK_VALUE) for h in range(H)])
                max_new = jnp.maximum(row_max, jnp.max(s, axis=2, keepdims=True))
                p = jnp.exp(s - max_new)
                alpha = jnp.exp(row_max - max_new)
                row_sum = alpha * row_sum + jnp.sum(p, axis=2, keepdims=True)
                pv = jnp.stack([p[h].astype(dtype) @ vt[h] for h in range(H)])
                acc = alpha * acc + pv
                row_max = max_new
            heads = acc / row_sum
            a = jnp.concatenate([heads[h] for h in range(H)], axis=1)  # (bq, D): the heads side by side
            normed = (a * jax.lax.rsqrt(jnp.mean(a * a, axis=1, keepdims=True) + EPS) * gamma[0:1, :]).astype(dtype)
            y = jnp.zeros((bq, D), jnp.float32)
            for f in range(0, F, bf):  # phase 2: the feed-forward layer, bf hidden units at a time
                hidden = jax.nn.gelu(normed @ w_up[:, f : f + bf])
                y += hidden.astype(dtype) @ w_down[f : f + bf, :]
            out = out.at[b, i : i + bq, :].set(y.astype(dtype))
    return out


def queries_by_kv_head(qt, kv_heads):
    """A sequence's queries (T, H, Dh) as (Hkv, T * G, Dh): head h attends with KV head h // G, and a KV head's
    rows are its (new token, query head) pairs, token-major."""
    t, h, d = qt.shape
    return qt.reshape(t, kv_heads, h // kv_heads, d).transpose(1, 0, 2, 3).reshape(kv_heads, t * (h // kv_heads), d)


def page_by_kv_head(page, kv_heads):
    """A page (P, Hkv * Dh) as (Hkv, P, Dh)."""
    p, w = page.shape
    return page.reshape(p, kv_heads, w // kv_heads).transpose(1, 0, 2)


def visible(page_size, first, length, new_tokens, group):
    """Which (query row, position) pairs of a page starting at `first` attend: (1, T * G, P). New token t sits at
    position length - T + t and sees the positions up to its own; for one new token that is `cols < length`."""
    rows = new_tokens * group
    cols = first + jax.lax.broadcasted_iota(jnp.int32, (1, rows, page_size), 2)
    token = jax.lax.broadcasted_iota(jnp.int32, (1, rows, page_size), 1) // group
    return cols <= length - new_tokens + token


def online_softmax(s, v, ok, row_max, row_sum, acc):
    """One online-softmax step over scores s (Hkv, G, P) against values v (Hkv, P, Dh)."""
    s = jnp.where(ok, s, MASK_VALUE)
    max_new = jnp.maximum(row_max, jnp.max(s, axis=2, keepdims=True))
    p = jnp.exp(s - max_new)
    alpha = jnp.exp(row_max - max_new)
    row_sum = alpha * row_sum + jnp.sum(p, axis=2, keepdims=True)
    acc = alpha * acc + jnp.dot(p.astype(v.dtype), v, preferred_element_type=jnp.float32)
    return max_new, row_sum, acc


def finish(acc, row_sum, shape, dtype):
    """The normalised output (Hkv, T * G, Dh) as `shape` (T, H, Dh); rows that saw no key (an empty sequence)
    are 0."""
    t, h, d = shape
    out = acc * (1.0 / jnp.maximum(row_sum, 1e-30))
    kv_heads = out.shape[0]
    return out.reshape(kv_heads, t, h // kv_heads, d).transpose(1, 0, 2, 3).reshape(shape).astype(dtype)


@autokernel.kernel
def gqa_decode(q, k_cache, v_cache, lengths, tiles=DecodeTiles()):
    """GQA decode attention over a contiguous cache: q (B, T, H, Dh), caches (B, S_max, Hkv * Dh), sequence b's
    valid positions lengths[b], its T new tokens included."""
    B, T, H, Dh = q.shape
    S, W = k_cache.shape[1], k_cache.shape[2]
    Hkv = W // Dh
    bk, dtype = min(tiles.block_kv, S), q.dtype
    out = jnp.zeros((B, T, H, Dh), dtype)
    for b in range(B):
        qt = queries_by_kv_head(q[b, :, :, :], Hkv)
        row_max = jnp.full((Hkv, T * (H // Hkv), 1), MASK_VALUE, jnp.float32)
        row_sum = jnp.zeros((Hkv, T * (H // Hkv), 1), jnp.float32)
        acc = jnp.zeros((Hkv, T * (H // Hkv), Dh), jnp.float32)
        for j in range(0, S, bk):
            if j >= lengths[b]:  # past the sequence's end: decided on the device, before the kernel runs
                continue
            kt = page_by_kv_head(k_cache[b, j : j + bk, :], Hkv)
            s = jnp.dot(qt, kt.transpose(0, 2, 1), preferred_element_type=jnp.float32)
            ok = visible(bk, j, lengths[b], T, H // Hkv)
            vt = page_by_kv_head(v_cache[b, j : j + bk, :], Hkv)
            row_max, row_sum, acc = online_softmax(s, vt, ok, row_max, row_sum, acc)
        out = out.at[b, :, :, :].set(finish(acc, row_sum, (T, H, Dh), dtype))
    return out


def mla_softmax_step(s, ct, ok, row_max, row_sum, acc):
    """One online-softmax step of MLA decode: scores s (H, bk) against the latents ct (bk, C) themselves."""
    s = jnp.where(ok, s, MASK_VALUE)
    max_new = jnp.maximum(row_max, jnp.max(s, axis=1, keepdims=True))
    p = jnp.exp(s - max_new)
    alpha = jnp.exp(row_max - max_new)
    row_sum = alpha * row_sum + jnp.sum(p, axis=1, keepdims=True)
    acc = alpha * acc + jnp.dot(p.astype(ct.dtype), ct, preferred_element_type=jnp.float32)
    return max_new, row_sum, acc


def rows_see(new_tokens, heads, block, first, length):
    """Which (query row, position) pairs of a block starting at `first` attend: (T * H, block). Row t * H + h is new
    token t, at position length - T + t, and sees the positions up to its own; for one new token that is
    `cols < length`."""
    rows = new_tokens * heads
    cols = first + jax.lax.broadcasted_iota(jnp.int32, (rows, block), 1)
    token = jax.lax.broadcasted_iota(jnp.int32, (rows, block), 0) // heads
    return cols <= length - new_tokens + token


@autokernel.kernel
def mla_decode(q_c, q_r, c_kv, k_rope, lengths, tiles=DecodeTiles()):
    """Absorbed MLA decode attention: q_c (B, T, H, C), q_r (B, T, H, 128), the latent cache (B, S_max, C) and the
    RoPE key cache (B, S_max, 128); out (B, T, H, C), each head's softmax-weighted latents. A sequence's rows are
    its (new token, head) pairs, token-major."""
    B, T, H, C = q_c.shape
    S = c_kv.shape[1]
    bk, dtype = min(tiles.block_kv, S), q_c.dtype
    out = jnp.zeros((B, T, H, C), dtype)
    for b in range(B):
        qc = q_c[b, :, :, :].reshape(T * H, C)
        qr = q_r[b, :, :, :].reshape(T * H, 128)
        row_max = jnp.full((T * H, 1), MASK_VALUE, jnp.float32)
        row_sum = jnp.zeros((T * H, 1), jnp.float32)
        acc = jnp.zeros((T * H, C), jnp.float32)
        for j in range(0, S, bk):
            if j >= lengths[b]:  # past the sequence's end: decided on the device, before the kernel runs
                continue
            ct = c_kv[b, j : j + bk, :]
            s = jnp.dot(qc, ct.T, preferred_element_type=jnp.float32)
            s = s + jnp.dot(qr, k_rope[b, j : j + bk, :].T, preferred_element_type=jnp.float32)
            ok = rows_see(T, H, bk, j, lengths[b])
            row_max, row_sum, acc = mla_softmax_step(s, ct, ok, row_max, row_sum, acc)
        res = acc * (1.0 / jnp.maximum(row_sum, 1e-30))
        out = out.at[b, :, :, :].set(res.reshape(T, H, C).astype(dtype))
    return out


@autokernel.kernel
def paged_gqa_decode(q, k_pages, v_pages, block_tables, lengths):
    """GQA decode attention over a paged cache: q (B, T, H, Dh), pages (num_pages, page_size, Hkv * Dh), sequence
    b's pages listed in block_tables[b, :], its valid positions lengths[b], its T new tokens included."""
    B, T, H, Dh = q.shape
    P, W = k_pages.shape[1], k_pages.shape[2]
    pages = block_tables.shape[1]
    Hkv = W // Dh
    dtype = q.dtype
    out = jnp.zeros((B, T, H, Dh), dtype)
    for b in range(B):
        qt = queries_by_kv_head(q[b, :, :, :], Hkv)
        row_max = jnp.full((Hkv, T * (H // Hkv), 1), MASK_VALUE, jnp.float32)
        row_sum = jnp.zeros((Hkv, T * (H // Hkv), 1), jnp.float32)
        acc = jnp.zeros((Hkv, T * (H // Hkv), Dh), jnp.float32)
        for p in range(pages):
            if p * P >= lengths[b]:  # past the sequence's end: decided on the device, before the kernel runs
                continue
            kt = page_by_kv_head(k_pages[block_tables[b, p], :, :], Hkv)
            s = jnp.dot(qt, kt.transpose(0, 2, 1), preferred_element_type=jnp.float32)
            ok = visible(P, p * P, lengths[b], T, H // Hkv)
            vt = page_by_kv_head(v_pages[block_tables[b, p], :, :], Hkv)
            row_max, row_sum, acc = online_softmax(s, vt, ok, row_max, row_sum, acc)
        out = out.at[b, :, :, :].set(finish(acc, row_sum, (T, H, Dh), dtype))
    return out


@autokernel.kernel
def rpa_write(kv_cache, keys, values, page_indices, write_page, write_rows, write_first, write_stop, n_writes):
    """Ragged paged attention's cache write (examples/ragged_paged_attention.py:33-47): the cache (pages, page_size,
    Hkv, 2, Dh) with the step's new keys and values (T, Hkv, Dh) in it. Run w < n_writes[0] is a stretch of one
    sequence's new tokens that lands in one page: the tokens from write_rows[w] on go to rows write_first[w] ..
    write_stop[w] - 1 of page page_indices[write_page[w]]. How many runs there are is read as the kernel runs."""
    P = kv_cache.shape[1]
    out = kv_cache
    for w in range(n_writes[0]):
        tokens = autokernel.rows(write_rows[w], write_rows[w] + write_stop[w] - write_first[w], P)
        side_by_side = jnp.stack([keys[tokens, :, :], values[tokens, :, :]], axis=2)
        out = out.at[page_indices[write_page[w]], autokernel.rows(write_first[w], write_stop[w], P), :, :, :].set(side_by_side)
    return out


def cache_page_by_kv_head(page):
    """A page of a cache that holds each head's key and value side by side, (P, Hkv, 2, Dh), as keys and values
    (Hkv, P, Dh)."""
    return page[:, :, 0, :].transpose(1, 0, 2), page[:, :, 1, :].transpose(1, 0, 2)


def make_rpa_decode(sm_scale: float) -> autokernel.Kernel:
    """Ragged paged attention's decode case for one softmax scale (examples/ragged_paged_attention.py:110-149): q
    (T, H, Dh) holds every sequence's new tokens and sequence s < distribution[0] is token s; the cache (pages,
    page_size, Hkv, 2, Dh) already holds the new tokens; kv_lens (S,) counts them in; sequence s's pages are
    page_indices[s * pages_per_seq :]. The result is q with the decode tokens' rows replaced by their attention
    outputs. How many pages a sequence walks is read from kv_lens as the kernel runs."""

    @autokernel.kernel
    def rpa_decode(q, kv_cache, kv_lens, page_indices, distribution):
        T, H, Dh = q.shape
        P, Hkv = kv_cache.shape[1], kv_cache.shape[2]
        S = kv_lens.shape[0]
        per_seq = page_indices.shape[0] // S
        dtype = q.dtype
        out = q
        for s in range(min(S, T)):
            qt = queries_by_kv_head(q[s : s + 1, :, :], Hkv)
            row_max = jnp.full((Hkv, H // Hkv, 1), MASK_VALUE, jnp.float32)
            row_sum = jnp.zeros((Hkv, H // Hkv, 1), jnp.float32)
            acc = jnp.zeros((Hkv, H // Hkv, Dh), jnp.float32)
            for p in range((kv_lens[s] + P - 1) // P if s < distribution[0] else 0):
                kt, vt = cache_page_by_kv_head(kv_cache[page_indices[s * per_seq + p], :, :, :, :])
                scores = jnp.dot(qt, kt.transpose(0, 2, 1), preferred_element_type=jnp.float32) * sm_scale
                ok = visible(P, p * P, kv_lens[s], 1, H // Hkv)
                row_max, row_sum, acc = online_softmax(scores, vt, ok, row_max, row_sum, acc)
            attended = finish(acc, row_sum, (1, H, Dh), dtype)
            out = out.at[s, :, :].set(jnp.where(s < distribution[0], attended[0, :, :], q[s, :, :]))
        return out

    return rpa_decode


PREFILL_QUERIES = 256  # query rows per prefill tile (examples/ragged_paged_attention.py:154)


def make_rpa_prefill(sm_scale: float) -> autokernel.Kernel:
    """Ragged paged attention's prefill / mixed case for one softmax scale (examples/ragged_paged_attention.py:196-243):
    tile k < n_tiles[0] is the rows tile_rows[k] .. tile_rows[k + 1] - 1 of q (at most 256), the new tokens of a
    sequence whose pages start at page_indices[tile_page[k]]; the first sits at cache position tile_pos[k], and a row
    at position p attends to the positions up to p, all before tile_stop[k]. The result is q with those rows replaced.
    How many tiles there are, and how many pages a tile walks, is read as the kernel runs."""

    @autokernel.kernel
    def rpa_prefill(q, kv_cache, page_indices, tile_page, tile_rows, tile_pos, tile_stop, n_tiles):
        _, H, Dh = q.shape
        P, Hkv = kv_cache.shape[1], kv_cache.shape[2]
        rows = PREFILL_QUERIES * (H // Hkv)
        dtype = q.dtype
        out = q
        for k in range(n_tiles[0]):
            tokens = autokernel.rows(tile_rows[k], tile_rows[k + 1], PREFILL_QUERIES)
            qt = queries_by_kv_head(q[tokens, :, :], Hkv)
            row_max = jnp.full((Hkv, rows, 1), MASK_VALUE, jnp.float32)
            row_sum = jnp.zeros((Hkv, rows, 1), jnp.float32)
            acc = jnp.zeros((Hkv, rows, Dh), jnp.float32)
            for j in range(0, tile_stop[k], P):
                kt, vt = cache_page_by_kv_head(kv_cache[page_indices[tile_page[k] + j // P], :, :, :, :])
                scores = jnp.dot(qt, kt.transpose(0, 2, 1), preferred_element_type=jnp.float32) * sm_scale
                ok = visible(P, j, tile_pos[k] + PREFILL_QUERIES, PREFILL_QUERIES, H // Hkv)
                row_max, row_sum, acc = online_softmax(scores, vt, ok, row_max, row_sum, acc)
            out = out.at[tokens, :, :].set(finish(acc, row_sum, (PREFILL_QUERIES, H, Dh), dtype))
        return out

    return rpa_prefill


def autokernel_rpa(queries, keys, values, kv_cache, kv_lens, page_indices, cu_q_lens, distribution, *, sm_scale=1.0):
    """RPA v3's `ragged_paged_attention` as the reference composes it (examples/ragged_paged_attention.py:279-290: the
    new tokens written into the cache, the decode sequences' attention, then the others'): (out (T, H, D), the
    updated cache) for CUDA tensors. The reference runs three kernels with plain-JAX index arithmetic between them
    and donates the queries and the cache; here the whole step, index arithmetic included, is one call into the
    library (tilejax_b200.ops.ragged_paged_attention), the cache updated in place and the queries left alone."""
    from tilejax_b200 import ops

    return ops.ragged_paged_attention(queries, keys, values, kv_cache, kv_lens, page_indices, cu_q_lens, distribution,
                                      float(sm_scale))


@autokernel.kernel
def all_gather_matmul(x, w, tiles=CollectiveTiles()):
    """x: this rank's rows (m, K); w: (K, n). Every rank's rows times these columns."""
    xs = autokernel.all_gather(x, "x")
    M, K = xs.shape
    N = w.shape[1]
    tm, tn, tk = min(tiles.tm, x.shape[0]), min(tiles.tn, N), min(tiles.tk, K)
    dtype = x.dtype
    out = jnp.zeros((M, N), dtype)
    for i in range(0, M, tm):
        for j in range(0, N, tn):
            acc = jnp.zeros((tm, tn), jnp.float32)
            for k in range(0, K, tk):
                acc += xs[i : i + tm, k : k + tk] @ w[k : k + tk, j : j + tn]
            out = out.at[i : i + tm, j : j + tn].set(acc.astype(dtype))
    return out
