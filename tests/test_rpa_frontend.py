"""Ragged paged attention's cache write, decode case and prefill case through the front end (`@autokernel.kernel` on the
loop nests of examples/ragged_paged_attention.py:33-47, :121-149 and :204-243): trip counts read from inputs as the kernel runs, outputs
that are inputs updated, rows chosen as the kernel runs (`rows`), a cache read and written as paired words. On the CPU: what the nest means (`kernel.reference`) against the
oracle bit for bit, what it lowers to, what is refused. The reference's own example is used unmodified when its tree
is at hand."""

import os

import numpy as np
import pytest

import oracle
import tilejax_b200.autokernel as autokernel
from tilejax_b200.autokernel import KernelError, fingerprint, jaxlike
from tilejax_b200.autokernel import kernels as K
from tilejax_b200.autokernel.recognised import RECOGNISED

jax = jaxlike
jnp = jaxlike.numpy
MASK_VALUE = K.MASK_VALUE

EXAMPLES = os.environ.get("AUTOKERNEL_EXAMPLES") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference", "examples")
needs_reference = pytest.mark.skipif(not os.path.isdir(EXAMPLES), reason="the reference's tree is not on this machine")
SCALE = 128**-0.5


def step_inputs(**sizes):
    """Three decode sequences (one token, one page and a bit, four full pages), a prefill sequence, padding."""
    sizes = dict(dict(heads=8, kv_heads=2, head_dim=128, page_size=64, max_len=256, max_tokens=12, max_seqs=6, seed=3), **sizes)
    inp = oracle.rpa_inputs([1, 1, 1, 5], [1, 130, 256, 200], **sizes)
    cache = oracle.rpa_write_ref(inp["kv_cache"], inp["keys"], inp["values"], inp["kv_lens"], inp["page_indices"],
                                 inp["cu_q_lens"], inp["distribution"])
    return inp["q"], cache, inp["kv_lens"], inp["page_indices"], inp["distribution"]


def test_the_nest_means_what_the_oracle_says_and_is_parsed_as_runtime_and_in_place():
    kernel = K.make_rpa_decode(SCALE)
    assert kernel.nest.inplace == {"out": "q"} and kernel.nest.runtime_ranges and not kernel.nest.runtime_masks
    assert kernel.nest.range_reads == {"kv_lens", "distribution"}
    args = step_inputs()
    want = oracle.rpa_decode_ref(*args, SCALE)
    got = kernel.reference(*args)
    np.testing.assert_array_equal(got.view(np.uint16), want.view(np.uint16))
    np.testing.assert_array_equal(got[3:].view(np.uint16), args[0][3:].view(np.uint16))  # non-decode rows: the query
    assert fingerprint.fingerprint(kernel) in RECOGNISED["rpa_decode"]
    assert fingerprint.fingerprint(K.make_rpa_decode(0.5)) == fingerprint.fingerprint(kernel)  # the scale is an argument


def test_it_lowers_to_the_rpa_decode_entry_with_its_scale():
    args = step_inputs()
    lowered = K.make_rpa_decode(0.25).lower(*args)
    p = lowered.plan.params
    assert lowered.plan.family == "decode" and p["rpa"] and p["sm_scale"] == 0.25
    assert (p["B"], p["H"], p["Hkv"], p["D"], p["page"], p["pages"]) == (6, 8, 2, 128, 64, 4)
    assert lowered.tiles == 6 and lowered.steps == 24  # at most: a sequence walks cdiv(kv_lens[s], page_size) pages
    assert "tjx_rpa_decode_bf16" in lowered.source and "softmax scale 0.25" in lowered.source


def test_what_is_not_that_nest_is_refused():
    args = step_inputs()

    def other_mask_value(sm_scale):
        @autokernel.kernel
        def rpa_decode(q, kv_cache, kv_lens, page_indices, distribution):
            T, H, Dh = q.shape
            P, Hkv = kv_cache.shape[1], kv_cache.shape[2]
            S = kv_lens.shape[0]
            per_seq = page_indices.shape[0] // S
            dtype = q.dtype
            out = q
            for s in range(min(S, T)):
                qt = K.queries_by_kv_head(q[s : s + 1, :, :], Hkv)
                row_max = jnp.full((Hkv, H // Hkv, 1), -1e9, jnp.float32)
                row_sum = jnp.zeros((Hkv, H // Hkv, 1), jnp.float32)
                acc = jnp.zeros((Hkv, H // Hkv, Dh), jnp.float32)
                for p in range((kv_lens[s] + P - 1) // P if s < distribution[0] else 0):
                    kt, vt = K.cache_page_by_kv_head(kv_cache[page_indices[s * per_seq + p], :, :, :, :])
                    scores = jnp.dot(qt, kt.transpose(0, 2, 1), preferred_element_type=jnp.float32) * sm_scale
                    ok = K.visible(P, p * P, kv_lens[s], 1, H // Hkv)
                    row_max, row_sum, acc = K.online_softmax(scores, vt, ok, row_max, row_sum, acc)
                attended = K.finish(acc, row_sum, (1, H, Dh), dtype)
                out = out.at[s, :, :].set(jnp.where(s < distribution[0], attended[0, :, :], q[s, :, :]))
            return out

        return rpa_decode

    with pytest.raises(KernelError, match="not a form of it"):
        other_mask_value(SCALE).lower(*args)

    def every_sequence_decodes(sm_scale):
        @autokernel.kernel
        def rpa_decode(q, kv_cache, kv_lens, page_indices, distribution):
            T, H, Dh = q.shape
            P, Hkv = kv_cache.shape[1], kv_cache.shape[2]
            S = kv_lens.shape[0]
            per_seq = page_indices.shape[0] // S
            dtype = q.dtype
            out = q
            for s in range(min(S, T)):
                qt = K.queries_by_kv_head(q[s : s + 1, :, :], Hkv)
                row_max = jnp.full((Hkv, H // Hkv, 1), MASK_VALUE, jnp.float32)
                row_sum = jnp.zeros((Hkv, H // Hkv, 1), jnp.float32)
                acc = jnp.zeros((Hkv, H // Hkv, Dh), jnp.float32)
                for p in range((kv_lens[s] + P - 1) // P):  # no distribution: not the decode case
                    kt, vt = K.cache_page_by_kv_head(kv_cache[page_indices[s * per_seq + p], :, :, :, :])
                    scores = jnp.dot(qt, kt.transpose(0, 2, 1), preferred_element_type=jnp.float32) * sm_scale
                    ok = K.visible(P, p * P, kv_lens[s], 1, H // Hkv)
                    row_max, row_sum, acc = K.online_softmax(scores, vt, ok, row_max, row_sum, acc)
                out = out.at[s, :, :].set(K.finish(acc, row_sum, (1, H, Dh), dtype)[0, :, :])
            return out

        return rpa_decode

    with pytest.raises(KernelError, match="read from kv_lens and distribution"):
        every_sequence_decodes(SCALE).lower(*args)

    # The kernel's shape rules are reported the same way: a head dimension the decode kernel does not take.
    small = step_inputs(head_dim=64)
    with pytest.raises(KernelError, match="head_dim 128"):
        K.make_rpa_decode(SCALE).lower(*small)


@needs_reference
def test_the_references_own_decode_kernel_is_recognised_unmodified():
    stand_ins = {"jax": jaxlike, "jnp": jaxlike.numpy, "autokernel": autokernel, "__name__": "example"}
    ns = fingerprint.load_example(os.path.join(EXAMPLES, "ragged_paged_attention.py"), stand_ins)
    kernel = ns["make_decode"](SCALE)  # paired words, shifts and bitcasts, lane-wide row statistics
    assert fingerprint.fingerprint(kernel) in RECOGNISED["rpa_decode"]
    # Its scores and P @ v are one matmul over every KV head's positions (the other heads' masked to zero weight):
    # the same sums as the oracle's per-head ones in another order, so equal to f32 rounding, not bit for bit.
    args = step_inputs()
    got, want = kernel.reference(*args), oracle.rpa_decode_ref(*args, SCALE)
    assert np.abs(got.astype(np.float64) - want.astype(np.float64)).max() <= 2e-2
    np.testing.assert_array_equal(got[3:].view(np.uint16), args[0][3:].view(np.uint16))
    lowered = kernel.lower(*args)
    assert "tjx_rpa_decode_bf16" in lowered.source and lowered.plan.params["sm_scale"] == SCALE
    # Llama-3-8B heads and pages of 128, as the example's own inputs (examples/ragged_paged_attention.py:22-24).
    big = step_inputs(heads=32, kv_heads=8, page_size=128, max_len=512)
    got, want = kernel.reference(*big), oracle.rpa_decode_ref(*big, SCALE)
    assert np.abs(got.astype(np.float64) - want.astype(np.float64)).max() <= 2e-2
    assert np.abs(got.astype(np.float64) - oracle.rpa_decode_f64(*big, SCALE)).max() <= 2e-2


# ----------------------------------------------------------------------------- the cache write


def write_inputs():
    inp = oracle.rpa_inputs([1, 1, 1, 300, 7, 130], [513, 1, 128, 300, 135, 400], max_len=1024, max_tokens=448,
                            max_seqs=8, seed=3)
    runs = oracle.rpa_write_runs(inp["kv_lens"], inp["page_indices"], inp["cu_q_lens"], inp["distribution"], 128, 448)
    want = oracle.rpa_write_ref(inp["kv_cache"], inp["keys"], inp["values"], inp["kv_lens"], inp["page_indices"],
                                inp["cu_q_lens"], inp["distribution"])
    return (inp["kv_cache"], inp["keys"], inp["values"], inp["page_indices"], *runs.values()), want


def test_the_write_nest_means_the_token_by_token_write_and_lowers_to_the_run_kernel():
    args, want = write_inputs()
    kernel = K.rpa_write
    assert kernel.nest.inplace == {"out": "kv_cache"} and kernel.nest.range_reads == {"n_writes"}
    assert len(kernel.nest.parallel) == 1 and not kernel.nest.reductions
    np.testing.assert_array_equal(kernel.reference(*args).view(np.uint16), want.view(np.uint16))
    assert fingerprint.fingerprint(kernel) in RECOGNISED["rpa_write"]
    lowered = kernel.lower(*args)
    assert lowered.plan.family == "rpa_write" and "tjx_rpa_write_runs_bf16" in lowered.source
    assert lowered.tiles == args[4].shape[0]  # at most: the run count is read on the device
    # Another store is another kernel: keys where the values go.
    @autokernel.kernel
    def swapped(kv_cache, keys, values, page_indices, write_page, write_rows, write_first, write_stop, n_writes):
        P = kv_cache.shape[1]
        out = kv_cache
        for w in range(n_writes[0]):
            tokens = autokernel.rows(write_rows[w], write_rows[w] + write_stop[w] - write_first[w], P)
            side_by_side = jnp.stack([values[tokens, :, :], keys[tokens, :, :]], axis=2)
            out = out.at[page_indices[write_page[w]], autokernel.rows(write_first[w], write_stop[w], P), :, :, :].set(side_by_side)
        return out

    with pytest.raises(KernelError, match="not a form of it"):
        swapped.lower(*args)


def test_rows_reads_clamp_and_stores_past_the_stop_are_dropped():
    # `rows(start, stop, n)` (src/autokernel/ragged.py:23-28): n indices from start, those at or past stop out of range.
    index = jaxlike.to_numpy(autokernel.rows(3, 5, 4))
    assert index[:2].tolist() == [3, 4] and (index[2:] > 10**9).all()
    x = jaxlike.Array(np.arange(12, dtype=np.float32).reshape(6, 2))
    read = jaxlike.to_numpy(x[autokernel.rows(4, 6, 4), :])
    assert read.tolist() == [[8, 9], [10, 11], [10, 11], [10, 11]]        # a read out of range clamps
    stored = jaxlike.to_numpy(x.at[autokernel.rows(1, 3, 4), :].set(jnp.full((4, 2), -1.0)))
    assert stored[:, 0].tolist() == [0, -1, -1, 6, 8, 10]                  # a store out of range is dropped


@needs_reference
def test_the_references_own_write_kernel_is_recognised_unmodified():
    stand_ins = {"jax": jaxlike, "jnp": jaxlike.numpy, "autokernel": autokernel, "__name__": "example"}
    ns = fingerprint.load_example(os.path.join(EXAMPLES, "ragged_paged_attention.py"), stand_ins)
    kernel = ns["rpa_write"]  # keys and values packed into words, stored with `unpairs`
    assert fingerprint.fingerprint(kernel) in RECOGNISED["rpa_write"]
    args, want = write_inputs()
    np.testing.assert_array_equal(kernel.reference(*args).view(np.uint16), want.view(np.uint16))
    assert "tjx_rpa_write_runs_bf16" in kernel.lower(*args).source


# ----------------------------------------------------------------------------- the prefill / mixed case


def prefill_inputs(**sizes):
    """Two decode sequences, then three with 300, 7 and 130 new tokens on prefixes of 0, 128 and 270 positions."""
    sizes = dict(dict(heads=8, kv_heads=2, max_len=1024, max_tokens=448, max_seqs=8, seed=3), **sizes)
    inp = oracle.rpa_inputs([1, 1, 300, 7, 130], [513, 1, 300, 135, 400], **sizes)
    cache = oracle.rpa_write_ref(inp["kv_cache"], inp["keys"], inp["values"], inp["kv_lens"], inp["page_indices"],
                                 inp["cu_q_lens"], inp["distribution"])
    tiles = oracle.rpa_prefill_tiles(inp["kv_lens"], inp["page_indices"], inp["cu_q_lens"], inp["distribution"], 448)
    return inp, cache, (inp["q"], cache, inp["page_indices"], *tiles.values())


def test_the_prefill_nest_means_what_the_oracle_says_and_lowers_to_the_tile_kernel():
    inp, cache, args = prefill_inputs()
    kernel = K.make_rpa_prefill(SCALE)
    assert kernel.nest.inplace == {"out": "q"} and kernel.nest.range_reads == {"n_tiles", "tile_stop"}
    want = oracle.rpa_prefill_ref(inp["q"], cache, inp["kv_lens"], inp["page_indices"], inp["cu_q_lens"],
                                  inp["distribution"], SCALE, pages_per_step=1)
    got = kernel.reference(*args)
    np.testing.assert_array_equal(got.view(np.uint16), want.view(np.uint16))
    np.testing.assert_array_equal(got[:2].view(np.uint16), inp["q"][:2].view(np.uint16))  # the decode tokens' rows stay
    exact = oracle.rpa_prefill_f64(inp["q"], cache, inp["kv_lens"], inp["page_indices"], inp["cu_q_lens"],
                                   inp["distribution"], SCALE)
    assert np.abs(got.astype(np.float64) - exact).max() <= 2e-2
    assert fingerprint.fingerprint(kernel) in RECOGNISED["rpa_prefill"]
    lowered = kernel.lower(*args)
    p = lowered.plan.params
    assert lowered.plan.family == "rpa_prefill" and p["sm_scale"] == SCALE and p["max_tiles"] == args[3].shape[0]
    assert "tjx_rpa_prefill_tiles_bf16" in lowered.source
    # The kernel's own limits are KernelErrors before anything runs: pages of 64, an odd group of query heads.
    _, _, small_pages = prefill_inputs(page_size=64)
    with pytest.raises(KernelError, match="pages of 128"):
        kernel.lower(*small_pages)
    _, _, odd = prefill_inputs(heads=6, kv_heads=2)
    with pytest.raises(KernelError, match="even number of query heads"):
        kernel.lower(*odd)


@needs_reference
def test_the_references_own_prefill_kernel_is_recognised_unmodified():
    stand_ins = {"jax": jaxlike, "jnp": jaxlike.numpy, "autokernel": autokernel, "__name__": "example"}
    ns = fingerprint.load_example(os.path.join(EXAMPLES, "ragged_paged_attention.py"), stand_ins)
    kernel = ns["make_prefill"](SCALE)  # head_rows / token_heads, dot_general over every KV head, four pages a step
    assert fingerprint.fingerprint(kernel) in RECOGNISED["rpa_prefill"]
    inp, cache, args = prefill_inputs()
    tiles = ns["PrefillTiles"](pages=2)
    want = oracle.rpa_prefill_ref(inp["q"], cache, inp["kv_lens"], inp["page_indices"], inp["cu_q_lens"],
                                  inp["distribution"], SCALE, pages_per_step=2)
    got = kernel.reference(*args, tiles)
    assert np.abs(got.astype(np.float64) - want.astype(np.float64)).max() <= 2e-2  # the same sums in another order
    lowered = kernel.lower(*args, tiles)
    assert "tjx_rpa_prefill_tiles_bf16" in lowered.source and lowered.plan.params["sm_scale"] == SCALE
    assert kernel.lower(*args, ns["PrefillTiles"](pages=8)).entry is not None  # pages per step: not the kernel's business
