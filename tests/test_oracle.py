"""The oracle against the known answers the reference's own tests hold for the hot path, and against
independent float64 formulas (the way the reference's tests check its kernels). CPU only."""

import numpy as np
import pytest
from helpers import BF16, f64, rand_bf16

import oracle
from tilejax_b200 import schedule


# ----------------------------------------------------------------------------- integer tables (pinned)


def test_device_tables_for_the_reference_ragged_lengths():
    # tests/test_index_arrays.py:57-72 and tests/test_decode.py:195-199: lengths (0, 1, 300, 512), S 512,
    # blocks of 128: 1 + 1 + 3 + 4 steps run (the empty sequence takes one empty step) of at most 16.
    tile, code, count = oracle.device_step_tables(oracle.lengths_runs([0, 1, 300, 512], 4, 0, 128))
    assert int(count[0]) == 1 + 1 + 3 + 4 and tile.size == 16
    # Every entry, from src/autokernel/codegen.py:392-431: kept steps first, the rest in their order, flags 0.
    assert tile.tolist() == [0, 1, 2, 2, 2, 3, 3, 3, 3, 0, 0, 0, 1, 1, 1, 2]
    assert code.tolist() == [7, 3, 2, 8, 17, 2, 8, 16, 25, 8, 16, 24, 8, 16, 24, 24]
    assert tile.dtype == np.int32 and code.dtype == np.int32 and count.dtype == np.int32


def test_device_tables_walk_exactly_the_steps_the_loop_nest_runs():
    rng = np.random.default_rng(5)
    lengths = rng.integers(0, 700, 9)
    lengths[[2, 5]] = 0
    tile, code, count = oracle.device_step_tables(oracle.lengths_runs(lengths, 10, 0, 64))
    n = int(count[0])
    steps, _ = oracle.walk_nest([range(9)], range(0, 640, 64), step_mask=lambda b, j: j >= lengths[b])
    assert n == len(steps)
    for s, ((b,), kb) in enumerate(steps):
        assert tile[s] == b
        assert (code[s] >> 3) == (0 if kb is None else kb) and bool(code[s] & 4) == (kb is None)
    firsts = [s for s in range(n) if code[s] & 2]
    lasts = [s for s in range(n) if code[s] & 1]
    assert len(firsts) == len(lasts) == 9  # every tile has exactly one first and one last step
    assert not (code[n:] & 7).any()  # the tail carries no flags


def test_causal_matmul_tables_match_the_reference_counts():
    # tests/test_examples.py:56-63: 512x256 @ 256x512 at 128^3: 10 of 16 tiles, 20 steps.
    sch = schedule.causal_matmul_schedule(512, 512, 256, 128, 128, 128)
    assert (sch.tiles, sch.total_tiles, sch.steps) == (10, 16, 20)
    tables = oracle.causal_tile_tables(512, 512, 128, 128)
    for name in ("tile_i", "tile_j", "fill_i", "fill_j"):
        np.testing.assert_array_equal(sch.tables[name], tables[name])
    steps, fills = oracle.walk_nest([range(0, 512, 128), range(0, 512, 128)], range(0, 256, 128),
                                    tile_mask=lambda i, j: j > i + 128 - 1)
    ran = list(dict.fromkeys(t for t, _ in steps))
    assert ran == list(zip(tables["tile_i"].tolist(), tables["tile_j"].tolist(), strict=True))
    assert fills == list(zip(tables["fill_i"].tolist(), tables["fill_j"].tolist(), strict=True))
    # A one-tile causal matmul has no tables (tests/test_schedule.py:189-198).
    assert oracle.causal_tile_tables(128, 128, 128, 128) == {}
    assert schedule.causal_matmul_schedule(128, 128, 128, 128, 128, 128).tables == {}


@pytest.mark.parametrize(("tiles", "want"), [((512, 512, 512), (136, 256, 2176, 120)),
                                             ((1024, 2048, 1024), (20, 32, 160, 12))])
def test_causal_matmul_schedule_at_the_benchmark_shape(tiles, want):
    sch = schedule.causal_matmul_schedule(8192, 8192, 8192, *tiles)
    assert (sch.tiles, sch.total_tiles, sch.steps, sch.fills) == want
    tables = oracle.causal_tile_tables(8192, 8192, tiles[0], tiles[1])
    for name, values in tables.items():
        np.testing.assert_array_equal(sch.tables[name], values)


def test_attention_tables_match_the_reference_counts():
    # tests/test_examples.py:91-95: (2, 4, 512, 128) at 128^2: steps 2*4*(1+2+3+4), 8 repeats, 10 table entries.
    sch = schedule.causal_attention_schedule(2, 4, 512, 128, 128)
    assert sch.steps == 2 * 4 * (1 + 2 + 3 + 4) and sch.repeats == 8 and len(sch.tables["step_tile"]) == 10
    tile, code = oracle.attention_step_tables(512, 128, 128)
    np.testing.assert_array_equal(sch.tables["step_tile"], tile)
    np.testing.assert_array_equal(sch.tables["step_code"], code)
    # The benchmark shape at 512^2: one (b, h) pattern of 4 tiles and 10 steps.
    sch = schedule.causal_attention_schedule(4, 16, 2048, 512, 512)
    assert (sch.tiles, sch.steps, sch.pattern_tiles, sch.pattern_steps) == (256, 640, 4, 10)
    assert sch.tables["step_tile"].tolist() == [0, 1, 1, 2, 2, 2, 3, 3, 3, 3]
    assert sch.tables["step_code"].tolist() == [3, 2, 9, 2, 8, 17, 2, 8, 16, 25]
    steps, _ = oracle.walk_nest([range(0, 2048, 512)], range(0, 2048, 512), step_mask=lambda i, j: j > i + 511)
    assert [(t, c >> 3) for t, c in zip(*oracle.attention_step_tables(2048, 512, 512), strict=True)] == [
        (t[0], kb) for t, kb in steps]
    for bq, n in ((256, 36), (1024, 3)):
        assert schedule.causal_attention_schedule(1, 1, 2048, bq, bq).pattern_steps == n
    assert schedule.causal_attention_schedule(1, 16, 4096, 512, 512).pattern_steps == 36


def test_matmul_schedule_matches_the_reference_counts():
    # tests/test_api.py:20-30: 256x384 @ 384x256 at 128^3 -> (steps, tiles, total_tiles) == (12, 4, 4).
    sch = schedule.matmul_schedule(256, 256, 384, 128, 128, 128)
    assert (sch.steps, sch.tiles, sch.total_tiles) == (12, 4, 4)
    assert schedule.matmul_schedule(4096, 4096, 4096, 512, 512, 512).steps == 512


def test_collective_row_order_is_the_reference_ring_formula():
    # tests/test_collective.py:98-124: i_blk = rem(me + 8 - (i_blk >> 1), 8) * 2 + (i_blk & 1).
    for me in range(8):
        want = [((me + 8 - (i >> 1)) % 8) * 2 + (i & 1) for i in range(16)]
        assert oracle.collective_row_order(me, 8, 2).tolist() == want
        assert schedule.collective_row_blocks(me, 8, 2).tolist() == want
    assert schedule.collective_row_blocks(0, 1, 4).tolist() == [0, 1, 2, 3]


# ----------------------------------------------------------------------------- floating point (tolerance)


def test_matmul_oracle_against_float64():
    x, y = rand_bf16((256, 384), 0), rand_bf16((384, 256), 1)
    out = oracle.matmul_ref(x, y, 128, 128, 128)
    assert out.dtype == BF16
    np.testing.assert_allclose(f64(out), f64(x) @ f64(y), rtol=2e-2, atol=0.2)  # tests/test_examples.py:31
    acc = oracle.matmul_ref(x, y, 128, 128, 128, out_dtype=np.float32)
    assert np.abs(f64(acc) - f64(x) @ f64(y)).max() <= 1e-5 * np.abs(f64(x) @ f64(y)).max()


def test_causal_matmul_oracle_is_tril():
    x, y = rand_bf16((512, 256), 0), rand_bf16((256, 512), 1)
    out = oracle.causal_matmul_ref(x, y, 128, 128, 128)
    np.testing.assert_allclose(f64(out), np.tril(f64(x) @ f64(y)), rtol=2e-2, atol=0.5)  # test_examples.py:60
    assert not f64(out)[np.triu_indices(512, 1)].any()


def test_attention_oracle_against_float64():
    q, k, v = (rand_bf16((1, 2, 512, 128), s) for s in (0, 1, 2))
    q = (q.astype(np.float32) * np.float32(128**-0.5)).astype(BF16)
    want = oracle.causal_attention_f64(q, k, v)
    for blocks in ((128, 128), (256, 128), (512, 512)):
        out = oracle.causal_attention_ref(q, k, v, *blocks)
        np.testing.assert_allclose(f64(out), want, atol=2e-2)  # tests/test_examples.py:86-87


def test_decode_oracle_against_float64_and_empty_sequence_is_zero():
    from tilejax_b200 import synthetic

    q, kp, vp, bt, lengths = synthetic.decode_inputs(4, 8, 2, 128, 16, 32, 64)
    lengths[:] = [0, 1, 300, 512]  # tests/test_decode.py:163-165
    out = oracle.paged_gqa_decode_ref(q, kp, vp, bt, lengths)
    want = oracle.paged_gqa_decode_f64(q, kp, vp, bt, lengths)
    assert np.abs(f64(out) - want).max() <= 2e-2 * np.abs(want).max()  # tests/test_decode.py:168-169
    assert not f64(out[0]).any()
    bt2 = bt.copy()
    bt2[1, 0] = bt[1, 0] + 64 * 100  # an out-of-range page index is clamped into the pool
    clamped = oracle.paged_gqa_decode_ref(q, kp, vp, bt2, lengths)
    bt3 = bt.copy()
    bt3[1, 0] = 63
    np.testing.assert_array_equal(f64(clamped), f64(oracle.paged_gqa_decode_ref(q, kp, vp, bt3, lengths)))


def test_paged_oracle_equals_contiguous_layout():
    # tests/test_decode.py:209: the paged result is bit-equal to the same cache laid out contiguously.
    B, S, P = 3, 256, 16
    k, v = rand_bf16((B, S, 256), 1), rand_bf16((B, S, 256), 2)
    q = rand_bf16((B, 1, 8, 128), 3, 128**-0.5)
    lengths = np.array([5, 100, 256], np.int32)
    order = np.random.default_rng(1).permutation(B * S // P).reshape(B, S // P).astype(np.int32)
    ident = np.arange(B * S // P, dtype=np.int32).reshape(B, S // P)
    a = oracle.paged_gqa_decode_ref(q, oracle.to_pages(k, order), oracle.to_pages(v, order), order, lengths)
    b = oracle.paged_gqa_decode_ref(q, oracle.to_pages(k, ident), oracle.to_pages(v, ident), ident, lengths)
    np.testing.assert_array_equal(f64(a), f64(b))
    # And the contiguous nest written out on its own (examples/decode.py:176-196) gives the same bits at the
    # same block size, and stays within the decode tolerance of float64 at the default one.
    np.testing.assert_array_equal(f64(oracle.gqa_decode_ref(q, k, v, lengths, P)), f64(b))
    want = oracle.paged_gqa_decode_f64(q, oracle.to_pages(k, ident), oracle.to_pages(v, ident), ident, lengths)
    assert np.abs(f64(oracle.gqa_decode_ref(q, k, v, lengths)) - want).max() <= 2e-2 * np.abs(want).max()


def test_several_new_tokens_see_only_positions_up_to_their_own():
    # tests/test_decode.py:215-220 (64-token pages, T = 2) and `visible` (examples/decode.py:145-152): new token t
    # sits at position length - T + t. Against float64, and row by row against the single-token call on the
    # prefix that row sees.
    B, S, P, T = 3, 256, 64, 2
    k, v = rand_bf16((B, S, 256), 1), rand_bf16((B, S, 256), 2)
    q = rand_bf16((B, T, 8, 128), 3, 128**-0.5)
    lengths = np.array([2, 100, 256], np.int32)
    ident = np.arange(B * S // P, dtype=np.int32).reshape(B, S // P)
    kp, vp = oracle.to_pages(k, ident), oracle.to_pages(v, ident)
    got = oracle.paged_gqa_decode_ref(q, kp, vp, ident, lengths)
    want = oracle.paged_gqa_decode_f64(q, kp, vp, ident, lengths)
    assert np.abs(f64(got) - want).max() <= 2e-2 * np.abs(want).max()
    np.testing.assert_array_equal(f64(oracle.gqa_decode_ref(q, k, v, lengths, P)), f64(got))
    for t in range(T):
        alone = oracle.paged_gqa_decode_ref(q[:, t : t + 1], kp, vp, ident, lengths - (T - 1 - t))
        np.testing.assert_array_equal(f64(got[:, t]), f64(alone[:, 0]))


def mla_inputs(B, H, S, seed=0):
    # tests/test_decode.py:152-160 in shape: latents 512 wide, RoPE keys 64 wide padded with zeros to 128.
    q_c = rand_bf16((B, 1, H, 512), seed, 192**-0.5 * 0.1)
    q_r, k_rope = rand_bf16((B, 1, H, 128), seed + 1, 192**-0.5), rand_bf16((B, S, 128), seed + 3)
    q_r[..., 64:] = 0
    k_rope[..., 64:] = 0
    return q_c, q_r, rand_bf16((B, S, 512), seed + 2), k_rope


def test_mla_decode_oracle_against_float64():
    # tests/test_decode.py:224-235 (16 heads, block 128) with the ragged lengths of :163-165.
    q_c, q_r, c_kv, k_rope = mla_inputs(4, 16, 512)
    lengths = np.array([0, 1, 300, 512], np.int32)
    want = oracle.mla_decode_f64(q_c, q_r, c_kv, k_rope, lengths)
    for block in (128, 512):
        got = oracle.mla_decode_ref(q_c, q_r, c_kv, k_rope, lengths, block)
        assert np.abs(f64(got) - want).max() <= 2e-2  # atol of tests/test_decode.py:235
        assert not f64(got[0]).any()


def test_mla_decode_oracle_with_several_new_tokens():
    # `visible` (examples/decode.py:145-152): new token t of T sees the positions up to lengths[b] - T + t.
    B, T, H, S = 3, 2, 16, 256
    q_c, q_r = rand_bf16((B, T, H, 512), 20, 192**-0.5 * 0.1), rand_bf16((B, T, H, 128), 21, 192**-0.5)
    c_kv, k_rope = rand_bf16((B, S, 512), 22), rand_bf16((B, S, 128), 23)
    lengths = np.array([2, 130, 256], np.int32)
    want = oracle.mla_decode_f64(q_c, q_r, c_kv, k_rope, lengths)
    for block in (128, 256):
        got = oracle.mla_decode_ref(q_c, q_r, c_kv, k_rope, lengths, block)
        assert np.abs(f64(got) - want).max() <= 2e-2
    # Token 0 of a 2-token step is the single-token step one position earlier.
    one = oracle.mla_decode_ref(q_c[:, :1], q_r[:, :1], c_kv, k_rope, lengths - 1, 128)
    two = oracle.mla_decode_ref(q_c, q_r, c_kv, k_rope, lengths, 128)
    np.testing.assert_array_equal(f64(two[:, :1]), f64(one))
    # And this package's nest means the same.
    from tilejax_b200.autokernel import kernels as K
    np.testing.assert_array_equal(f64(K.mla_decode.reference(q_c, q_r, c_kv, k_rope, lengths, K.DecodeTiles(block_kv=128))),
                                  f64(two))


def test_compare_rule():
    # src/autokernel/api.py:320-364 and tests/test_api.py:87-108: NaN equals NaN; 16-bit tolerance scales with
    # the largest value; integers are exact.
    want = np.array([1.0, np.nan, 100.0], np.float32).astype(BF16)
    assert oracle.compare("x", want.copy(), want) == 0.0
    got = np.array([1.0, np.nan, 101.0], np.float32).astype(BF16)
    assert oracle.compare("x", got, want) > 0
    with pytest.raises(AssertionError, match="differ in 1 of 3"):
        oracle.compare("x", np.array([4.0, np.nan, 100.0], np.float32).astype(BF16), want)
    with pytest.raises(AssertionError):
        oracle.compare("i", np.array([1, 2]), np.array([1, 3]))


def test_committed_known_answers():
    # tests/golden/known_answers.json (written by tests/golden/make_golden.py from the reference's tests and
    # sources): the oracle and the host schedules reproduce every integer in it.
    import json
    from pathlib import Path

    from tilejax_b200 import schedule

    known = json.loads((Path(__file__).resolve().parent / "golden" / "known_answers.json").read_text())
    d = known["device_step_tables_lengths_0_1_300_512_block_128"]
    tile, code, count = oracle.device_step_tables(oracle.lengths_runs(d["lengths"], d["blocks"], 0, d["block_size"]))
    assert (tile.tolist(), code.tolist(), int(count[0])) == (d["step_tile"], d["step_code"], d["step_count"])
    a = known["causal_attention_S2048_blocks_512"]
    sch = schedule.causal_attention_schedule(4, 16, a["S"], a["block_q"], a["block_kv"])
    assert sch.tables["step_tile"].tolist() == a["step_tile"] and sch.tables["step_code"].tolist() == a["step_code"]
    assert (sch.tiles, sch.steps) == (a["tiles"], a["steps"])
    tile, code = oracle.attention_step_tables(a["S"], a["block_q"], a["block_kv"])
    assert (tile.tolist(), code.tolist()) == (a["step_tile"], a["step_code"])
    b = known["causal_attention_2_4_512_128_blocks_128"]
    sch = schedule.causal_attention_schedule(2, 4, 512, 128, 128)
    assert (sch.steps, sch.repeats, len(sch.tables["step_tile"])) == (b["steps"], b["repeats"], b["pattern_steps"])
    m = known["matmul_256x384x256_tiles_128"]
    sch = schedule.matmul_schedule(256, 256, 384, 128, 128, 128)
    assert (sch.steps, sch.tiles, sch.total_tiles) == (m["steps"], m["tiles"], m["total_tiles"])
    for key, args in (("causal_matmul_512x256x512_tiles_128", (512, 512, 256, 128, 128, 128)),
                      ("causal_matmul_8192_tiles_512", (8192, 8192, 8192, 512, 512, 512)),
                      ("causal_matmul_8192_tiles_1024x2048x1024", (8192, 8192, 8192, 1024, 2048, 1024))):
        c = known[key]
        sch = schedule.causal_matmul_schedule(*args)
        assert (sch.tiles, sch.steps) == (c["tiles"], c["steps"])
        if "fills" in c:
            assert sch.fills == c["fills"]
        if "total_tiles" in c:
            assert sch.total_tiles == c["total_tiles"]
    r = known["collective_ring_order_8_chips_2_blocks"]
    for me in range(r["chips"]):
        i_blk = np.arange(r["chips"] * r["shard_blocks"])
        want = ((me + 8 - (i_blk >> 1)) % 8) * 2 + (i_blk & 1)
        np.testing.assert_array_equal(schedule.collective_row_blocks(me, r["chips"], r["shard_blocks"]), want)
