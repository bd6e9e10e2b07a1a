"""Ragged paged GQA decode through the C ABI against the oracle (`paged_gqa_decode`, examples/decode.py:199-223).

Tolerance: atol 2e-2 * max|want| (tests/test_decode.py:168-169); the step tables the call built are bit-exact.
"""

import numpy as np
import pytest
from helpers import f64, rand_bf16, to_device, to_host

import oracle
from tilejax_b200 import ops, synthetic
from tilejax_b200._lib import NativeError

pytestmark = pytest.mark.gpu


def run_decode(q, kp, vp, bt, lengths):
    out = ops.paged_gqa_decode(*map(to_device, (q, kp, vp, bt, lengths)))
    assert ops.device_status() == 0
    bufs = ops.paged_gqa_decode.last_buffers
    P, pages = kp.shape[1], bt.shape[1]
    tile, code, count = oracle.device_step_tables(oracle.lengths_runs(lengths, pages, 0, P))
    np.testing.assert_array_equal(to_host(bufs.step_tile), tile)
    np.testing.assert_array_equal(to_host(bufs.step_code), code)
    assert int(bufs.step_count[0]) == int(count[0])
    return to_host(out)


def close(got, want, tol=2e-2):
    assert np.abs(f64(got) - f64(want)).max() <= tol * max(np.abs(f64(want)).max(), 1e-6)


@pytest.mark.parametrize(("heads", "kv_heads", "page"), [(8, 2, 16), (8, 2, 128), (4, 4, 64), (16, 8, 16), (8, 1, 32)])
def test_ragged_lengths_match_the_oracle(heads, kv_heads, page):
    # The reference's ragged case (tests/test_decode.py:163-165): empty, one token, a partial block, full.
    pages = 512 // page
    q, kp, vp, bt, lengths = synthetic.decode_inputs(4, heads, kv_heads, 128, page, pages, 4 * pages,
                                                     distinct_pages=True)
    lengths[:] = [0, 1, 300, 512]
    got = run_decode(q, kp, vp, bt, lengths)
    close(got, oracle.paged_gqa_decode_ref(q, kp, vp, bt, lengths))
    close(got, oracle.paged_gqa_decode_f64(q, kp, vp, bt, lengths))
    assert not f64(got[0]).any()  # the empty sequence


def test_benchmark_configuration_matches_the_oracle():
    # BASELINE config 4: batch 64, 32 / 8 heads, D 128, 16-token pages, 8192 pages, lengths in [1, 4096].
    q, kp, vp, bt, lengths = synthetic.decode_inputs(64, 32, 8, 128, 16, 256, 8192)
    got = run_decode(q, kp, vp, bt, lengths)
    close(got, oracle.paged_gqa_decode_ref(q, kp, vp, bt, lengths))


def test_out_of_range_pages_are_clamped():
    q, kp, vp, bt, lengths = synthetic.decode_inputs(3, 8, 2, 128, 16, 8, 24)
    lengths[:] = [128, 17, 64]
    bad = bt.copy()
    bad[0, 1], bad[1, 0] = 9999, -5
    fixed = bt.copy()
    fixed[0, 1], fixed[1, 0] = 23, 0
    np.testing.assert_array_equal(f64(run_decode(q, kp, vp, bad, lengths)), f64(run_decode(q, kp, vp, fixed, lengths)))


def test_paged_equals_the_same_cache_laid_out_in_order():
    # tests/test_decode.py:209: paging is only a layout; the result is bit-equal.
    B, S, P = 3, 256, 16
    k, v = rand_bf16((B, S, 256), 1), rand_bf16((B, S, 256), 2)
    q = rand_bf16((B, 1, 8, 128), 3, 128**-0.5)
    lengths = np.array([5, 100, 256], np.int32)
    order = np.random.default_rng(1).permutation(B * S // P).reshape(B, S // P).astype(np.int32)
    ident = np.arange(B * S // P, dtype=np.int32).reshape(B, S // P)
    a = run_decode(q, oracle.to_pages(k, order), oracle.to_pages(v, order), order, lengths)
    b = run_decode(q, oracle.to_pages(k, ident), oracle.to_pages(v, ident), ident, lengths)
    np.testing.assert_array_equal(f64(a), f64(b))


@pytest.mark.parametrize("block", [128, 512])
def test_contiguous_cache_is_the_identity_block_table(block):
    # `gqa_decode` (examples/decode.py:176-196): against its own oracle, and bit-equal to the paged call over the
    # same cache cut into pages in order.
    B, S = 4, 1024
    k, v = rand_bf16((B, S, 512), 1), rand_bf16((B, S, 512), 2)
    q = rand_bf16((B, 1, 16, 128), 3, 128**-0.5)
    lengths = np.array([0, 1, 700, 1024], np.int32)
    got = to_host(ops.gqa_decode(to_device(q), to_device(k), to_device(v), to_device(lengths), block))
    assert ops.device_status() == 0
    want = oracle.gqa_decode_ref(q, k, v, lengths, block)
    assert np.abs(f64(got) - f64(want)).max() <= 2e-2 * np.abs(f64(want)).max()
    assert not f64(got[0]).any()
    ident = np.arange(B * S // block, dtype=np.int32).reshape(B, S // block)
    paged = run_decode(q, oracle.to_pages(k, ident), oracle.to_pages(v, ident), ident, lengths)
    np.testing.assert_array_equal(f64(got), f64(paged))


@pytest.mark.parametrize(("heads", "kv_heads", "new_tokens", "page"), [(8, 2, 2, 64), (8, 2, 4, 16), (4, 4, 3, 32),
                                                                       (16, 2, 2, 16), (8, 8, 16, 128)])
def test_several_new_tokens_per_sequence(heads, kv_heads, new_tokens, page):
    # tests/test_decode.py:215-220 (64-token pages, T = 2) and wider: new token t sits at position length - T + t
    # and sees the positions up to its own. Up to 8 query rows per KV head use half of the MMA's rows, up to 16 all.
    B, S, T = 4, 512, new_tokens
    k, v = rand_bf16((B, S, kv_heads * 128), 1), rand_bf16((B, S, kv_heads * 128), 2)
    q = rand_bf16((B, T, heads, 128), 3, 128**-0.5)
    lengths = np.array([0, T, 300, 512], np.int32)
    order = np.random.default_rng(1).permutation(B * S // page).reshape(B, S // page).astype(np.int32)
    kp, vp = oracle.to_pages(k, order), oracle.to_pages(v, order)
    got = run_decode(q, kp, vp, order, lengths)
    want = oracle.paged_gqa_decode_ref(q, kp, vp, order, lengths)
    assert np.abs(f64(got) - f64(want)).max() <= 2e-2 * np.abs(f64(want)).max()
    exact = oracle.paged_gqa_decode_f64(q, kp, vp, order, lengths)
    assert np.abs(f64(got) - exact).max() <= 2e-2 * np.abs(exact).max()
    assert not f64(got[0]).any()
    # Each new token alone, as a one-token call on the prefix it sees, agrees to rounding.
    for t in range(T):
        alone = run_decode(np.ascontiguousarray(q[:, t : t + 1]), kp, vp, order, np.maximum(lengths - (T - 1 - t), 0))
        assert np.abs(f64(got[1:, t]) - f64(alone[1:, 0])).max() <= 2e-2 * np.abs(exact).max()


def test_too_many_query_rows_per_kv_head_is_an_error():
    q, kp, vp, bt, lengths = synthetic.decode_inputs(2, 8, 2, 128, 16, 4, 8)
    q5 = np.repeat(q, 5, axis=1)
    with pytest.raises(NativeError, match="must not exceed 16"):
        run_decode(q5, kp, vp, bt, lengths)


def test_long_sequences_merge_more_than_32_partials():
    # 512 pages per sequence = 43 chunks of 12 steps: the merge walks its partials 32 at a time.
    B, S, page = 2, 8192, 16
    k, v = rand_bf16((B, S, 128), 1), rand_bf16((B, S, 128), 2)
    q = rand_bf16((B, 1, 2, 128), 3, 128**-0.5)
    lengths = np.array([8192, 7000], np.int32)
    ident = np.arange(B * S // page, dtype=np.int32).reshape(B, S // page)
    kp, vp = oracle.to_pages(k, ident), oracle.to_pages(v, ident)
    got = run_decode(q, kp, vp, ident, lengths)
    want = oracle.paged_gqa_decode_f64(q, kp, vp, ident, lengths)
    assert np.abs(f64(got) - want).max() <= 2e-2 * np.abs(want).max()


def test_all_sequences_empty():
    q, kp, vp, bt, lengths = synthetic.decode_inputs(5, 8, 2, 128, 16, 4, 20)
    lengths[:] = 0
    assert not f64(run_decode(q, kp, vp, bt, lengths)).any()


def test_unsupported_shapes_are_errors():
    q, kp, vp, bt, lengths = synthetic.decode_inputs(2, 8, 2, 128, 8, 4, 8)
    with pytest.raises(NativeError, match="multiple of 16"):
        ops.paged_gqa_decode(*map(to_device, (q, kp, vp, bt, lengths)))
    q, kp, vp, bt, lengths = synthetic.decode_inputs(2, 6, 2, 128, 16, 4, 8)
    with pytest.raises(NativeError, match="1, 2, 4 or 8"):
        ops.paged_gqa_decode(*map(to_device, (q, kp, vp, bt, lengths)))
