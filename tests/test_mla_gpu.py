"""Absorbed MLA decode through the C ABI against the oracle (`mla_decode`, examples/decode.py:226-250).

Tolerance: atol 2e-2 against float64, as tests/test_decode.py:235; the step tables the call built are bit-exact."""

import numpy as np
import pytest
from helpers import f64, rand_bf16, to_device, to_host

import oracle
from tilejax_b200 import ops
from tilejax_b200._lib import NativeError

pytestmark = pytest.mark.gpu


def mla_inputs(B, H, S, seed=0, T=1):
    q_c = rand_bf16((B, T, H, 512), seed, 192**-0.5 * 0.1)
    q_r, k_rope = rand_bf16((B, T, H, 128), seed + 1, 192**-0.5), rand_bf16((B, S, 128), seed + 3)
    q_r[..., 64:] = 0
    k_rope[..., 64:] = 0
    return q_c, q_r, rand_bf16((B, S, 512), seed + 2), k_rope


def run(q_c, q_r, c_kv, k_rope, lengths, block):
    out = ops.mla_decode(*map(to_device, (q_c, q_r, c_kv, k_rope, lengths)), block)
    assert ops.device_status() == 0
    bufs = ops.mla_decode.last_buffers
    blocks = c_kv.shape[1] // min(block, c_kv.shape[1])
    tile, code, count = oracle.device_step_tables(oracle.lengths_runs(lengths, blocks, 0, min(block, c_kv.shape[1])))
    np.testing.assert_array_equal(to_host(bufs.step_tile), tile)
    np.testing.assert_array_equal(to_host(bufs.step_code), code)
    assert int(bufs.step_count[0]) == int(count[0])
    return to_host(out)


@pytest.mark.parametrize(("heads", "block"), [(16, 128), (16, 512), (32, 64), (128, 256), (16, 16)])
def test_matches_the_oracle_on_ragged_lengths(heads, block):
    # tests/test_decode.py:224-235: 16 heads at blocks 128 / 256, lengths (0, 1, 300, S); wider head counts as the
    # reference's benchmark (H 16-128).
    q_c, q_r, c_kv, k_rope = mla_inputs(4, heads, 512)
    lengths = np.array([0, 1, 300, 512], np.int32)
    got = run(q_c, q_r, c_kv, k_rope, lengths, block)
    want = oracle.mla_decode_ref(q_c, q_r, c_kv, k_rope, lengths, block)
    assert np.abs(f64(got) - f64(want)).max() <= 2e-2
    assert np.abs(f64(got) - oracle.mla_decode_f64(q_c, q_r, c_kv, k_rope, lengths)).max() <= 2e-2
    assert not f64(got[0]).any()


@pytest.mark.parametrize(("tokens", "heads", "block"), [(2, 16, 128), (4, 32, 64), (3, 16, 512)])
def test_several_new_tokens_each_see_the_positions_up_to_their_own(tokens, heads, block):
    # tests/test_decode.py:163-220 runs the decode kernels with T new tokens; `visible` (examples/decode.py:145-152):
    # token t of T sits at lengths[b] - T + t. Lengths (the new tokens included, so never below T): exactly T, one
    # more, a partial block, the whole cache.
    q_c, q_r, c_kv, k_rope = mla_inputs(4, heads, 512, seed=11, T=tokens)
    lengths = np.array([tokens, tokens + 1, 300, 512], np.int32)
    got = run(q_c, q_r, c_kv, k_rope, lengths, block)
    want = oracle.mla_decode_ref(q_c, q_r, c_kv, k_rope, lengths, block)
    assert np.abs(f64(got) - f64(want)).max() <= 2e-2
    assert np.abs(f64(got) - oracle.mla_decode_f64(q_c, q_r, c_kv, k_rope, lengths)).max() <= 2e-2
    # The last new token sees everything the single-token call sees.
    single = run(q_c[:, -1:].copy(), q_r[:, -1:].copy(), c_kv, k_rope, lengths, block)
    assert np.abs(f64(got[:, -1:]) - f64(single)).max() <= 2e-2


@pytest.mark.parametrize(("batch", "heads", "longest", "seed"), [(200, 16, 96, 0), (333, 64, 40, 1), (150, 32, 700, 2)])
def test_many_short_and_empty_sequences_share_the_ctas(batch, heads, longest, seed):
    # More sequences than CTAs, a third of them empty, many of a single 32-position unit: a CTA's range then crosses
    # several sequences, ends inside the margin the split counts in front of a sequence, or holds whole sequences
    # that are written without a merge. Every row against float64; empty sequences are zeros.
    rng = np.random.default_rng(seed)
    S = 1024
    lengths = rng.integers(1, longest + 1, batch).astype(np.int32)
    lengths[rng.random(batch) < 0.33] = 0
    lengths[-1] = S
    q_c, q_r, c_kv, k_rope = mla_inputs(batch, heads, S, seed=20 + seed)
    got = run(q_c, q_r, c_kv, k_rope, lengths, 256)
    want = oracle.mla_decode_f64(q_c, q_r, c_kv, k_rope, lengths)
    assert np.abs(f64(got) - want).max() <= 2e-2
    assert not f64(got[lengths == 0]).any()
    np.testing.assert_array_equal(f64(got), f64(run(q_c, q_r, c_kv, k_rope, lengths, 256)))


def test_block_size_is_only_a_schedule():
    # The same cache walked in blocks of 64 or 512 positions agrees to rounding; two calls in a row agree exactly.
    q_c, q_r, c_kv, k_rope = mla_inputs(8, 16, 2048, seed=5)
    lengths = np.random.default_rng(0).integers(1, 2049, 8).astype(np.int32)
    a = run(q_c, q_r, c_kv, k_rope, lengths, 64)
    b = run(q_c, q_r, c_kv, k_rope, lengths, 512)
    assert np.abs(f64(a) - f64(b)).max() <= 2e-2
    np.testing.assert_array_equal(f64(a), f64(run(q_c, q_r, c_kv, k_rope, lengths, 64)))
    assert np.abs(f64(b) - oracle.mla_decode_f64(q_c, q_r, c_kv, k_rope, lengths)).max() <= 2e-2


def test_unsupported_shapes_are_errors():
    q_c, q_r, c_kv, k_rope = mla_inputs(2, 8, 128)
    lengths = np.array([5, 128], np.int32)
    with pytest.raises(NativeError, match="multiple of 16"):
        run(q_c, q_r, c_kv, k_rope, lengths, 128)
    q_c, q_r, c_kv, k_rope = mla_inputs(2, 16, 128)
    with pytest.raises(NativeError, match="multiple of 16 positions"):
        run(q_c, q_r, c_kv, k_rope, lengths, 8)


def test_the_kernel_shares_units_out_as_the_host_side_statement_says():
    # The counters every CTA of the tcgen05 kernel leaves (units and pieces it ran) against schedule.mla_unit_ranges.
    import ctypes

    import torch

    from tilejax_b200 import schedule
    from tilejax_b200._lib import check, library

    rng = np.random.default_rng(3)
    batch, heads, S = 40, 64, 2048
    lengths = rng.integers(0, S + 1, batch).astype(np.int32)
    lengths[::7] = 0
    q_c, q_r, c_kv, k_rope = mla_inputs(batch, heads, S, seed=30)
    dev = [to_device(a) for a in (q_c, q_r, c_kv, k_rope, lengths)]
    ctas = min(256, torch.cuda.get_device_properties(0).multi_processor_count)
    buf = torch.zeros(ctas * 16, dtype=torch.int64, device="cuda")
    check(library().tjx_set_profile_buffer(ctypes.c_void_p(buf.data_ptr()), buf.numel() * 8))
    try:
        got = to_host(ops.mla_decode(*dev, 512))
        torch.cuda.synchronize()
    finally:
        check(library().tjx_set_profile_buffer(None, 0))
    assert ops.device_status() == 0
    records = buf.cpu().numpy().reshape(ctas, 16)
    want = schedule.mla_unit_ranges(lengths, ctas)
    np.testing.assert_array_equal(records[:, 6], [sum(n for _, _, n in pieces) for pieces in want])
    np.testing.assert_array_equal(records[:, 11], [len(pieces) for pieces in want])
    assert np.abs(f64(got) - oracle.mla_decode_f64(q_c, q_r, c_kv, k_rope, lengths)).max() <= 2e-2
