"""Ragged paged attention's cache write and decode case on the CPU side (examples/ragged_paged_attention.py): the
oracle's token-by-token write against the reference's run arithmetic (`writes`, :49-71; `oracle.rpa_write_runs`), and its decode
against float64."""

import numpy as np

import oracle


def test_the_token_by_token_write_is_the_references_run_by_run_write():
    inp = oracle.rpa_inputs([1, 1, 1, 300, 7, 130], [513, 1, 128, 300, 135, 400], max_len=1024, max_tokens=448,
                            max_seqs=8, seed=3)
    got = oracle.rpa_write_ref(inp["kv_cache"], inp["keys"], inp["values"], inp["kv_lens"], inp["page_indices"],
                               inp["cu_q_lens"], inp["distribution"])
    r = oracle.rpa_write_runs(inp["kv_lens"], inp["page_indices"], inp["cu_q_lens"], inp["distribution"], 128, 448)
    want = inp["kv_cache"].copy()
    for w in range(int(r["n_writes"][0])):  # rpa_write (:33-46): a run lands in one page
        page = inp["page_indices"][r["write_page"][w]]
        n = r["write_stop"][w] - r["write_first"][w]
        rows = slice(r["write_rows"][w], r["write_rows"][w] + n)
        want[page, r["write_first"][w] : r["write_stop"][w], :, 0, :] = inp["keys"][rows]
        want[page, r["write_first"][w] : r["write_stop"][w], :, 1, :] = inp["values"][rows]
    np.testing.assert_array_equal(got.view(np.uint16), want.view(np.uint16))
    changed = (got.view(np.uint16) != inp["kv_cache"].view(np.uint16)).any(axis=(2, 3, 4)).sum()
    assert changed == 1 + 1 + 1 + 300 + 7 + 130  # one cache row per new token, nothing else


def test_decode_oracle_against_float64():
    inp = oracle.rpa_inputs([1, 1, 1, 1, 9], [1, 128, 129, 700, 64], heads=8, kv_heads=2, max_len=1024, max_seqs=8, seed=1)
    cache = oracle.rpa_write_ref(inp["kv_cache"], inp["keys"], inp["values"], inp["kv_lens"], inp["page_indices"],
                                 inp["cu_q_lens"], inp["distribution"])
    scale = 128**-0.5
    got = oracle.rpa_decode_ref(inp["q"], cache, inp["kv_lens"], inp["page_indices"], inp["distribution"], scale)
    want = oracle.rpa_decode_f64(inp["q"], cache, inp["kv_lens"], inp["page_indices"], inp["distribution"], scale)
    assert np.abs(got.astype(np.float64) - want).max() <= 2e-2
    # Rows that are not decode tokens keep the query, bit for bit.
    np.testing.assert_array_equal(got[4:].view(np.uint16), inp["q"][4:].view(np.uint16))
    # A sequence of one position attends to that position only: its output is that position's values.
    page = inp["page_indices"][0]
    for h in range(8):
        np.testing.assert_array_equal(got[0, h].view(np.uint16), cache[page, 0, h // 4, 1].view(np.uint16))


def test_prefill_oracle_against_float64():
    inp = oracle.rpa_inputs([1, 1, 300, 7, 130], [513, 1, 300, 135, 400], heads=4, kv_heads=2, max_len=1024,
                            max_tokens=448, max_seqs=8, seed=3)
    cache = oracle.rpa_write_ref(inp["kv_cache"], inp["keys"], inp["values"], inp["kv_lens"], inp["page_indices"],
                                 inp["cu_q_lens"], inp["distribution"])
    scale = 128**-0.5
    args = (inp["q"], cache, inp["kv_lens"], inp["page_indices"], inp["cu_q_lens"], inp["distribution"], scale)
    got = oracle.rpa_prefill_ref(*args)
    want = oracle.rpa_prefill_f64(*args)
    assert np.abs(got.astype(np.float64) - want).max() <= 2e-2
    # Steps of one page or of four: the same attention.
    one = oracle.rpa_prefill_ref(*args, pages_per_step=1)
    assert np.abs(one.astype(np.float64) - got.astype(np.float64)).max() <= 2e-2
    # The decode tokens and the padding rows keep the query.
    np.testing.assert_array_equal(got[:2].view(np.uint16), inp["q"][:2].view(np.uint16))
    np.testing.assert_array_equal(got[439:].view(np.uint16), inp["q"][439:].view(np.uint16))
