"""Step order and tables of ANY loop nest with static masks — the reference's known answers for `make_schedule`,
`Schedule.step_at` / `blocks_at` and the code radices (tests/test_schedule.py, tests/test_codegen.py:29-61), on
nests no kernel here runs: a schedule exists for every parsed nest, recognised family or not."""

import itertools

import numpy as np
import pytest
from helpers import make_kernel, spec

from tilejax_b200 import schedule
from tilejax_b200.autokernel import KernelError

F32 = np.float32


def schedule_of(source: str, *inputs, **names):
    return make_kernel(source, **names).schedule_of(*inputs)


BANDED = """
def f(x):
    out = jnp.zeros((B, 512, 512))
    for b in range(B):
        for i in range(0, 512, 128):
            for j in range(0, 512, 128):
                if j > i:
                    continue
                acc = jnp.zeros((128, 128))
                for k in range(0, 512, 128):
                    if k < i - 128:
                        continue
                    acc += x[b, i : i + 128, k : k + 128]
                out = out.at[b, i : i + 128, j : j + 128].set(acc)
    return out
"""


def test_tables_walk_exactly_the_nests_steps():
    # tests/test_schedule.py:17-51
    sch = schedule_of(BANDED, spec(3, 512, 512, dtype=F32), B=3)
    want = [((b, i, j), k) for b, i, j in itertools.product(range(3), range(4), range(4)) if j <= i
            for k in range(4) if k >= i - 1]
    got = []
    for step in range(sch.steps):
        tile, phase, k = sch.step_at(step)
        assert phase == 0
        got.append((sch.blocks_at(tile), k))
    assert got == want
    assert sch.tiles == 30 and sch.total_tiles == 48 and sch.fills == 18 and sch.repeats == 3
    assert [r.var for r in sch.outer] == ["b"] and [r.var for r in sch.inner] == ["i", "j"]
    # first / last flags bracket each tile's steps, in order.
    firsts = [s for s in range(sch.steps) if sch.first_at(s)]
    lasts = [s for s in range(sch.steps) if sch.last_at(s)]
    assert len(firsts) == len(lasts) == 30 and all(f <= l for f, l in zip(firsts, lasts))


def test_without_masks_steps_are_arithmetic():
    # tests/test_schedule.py:54-73
    sch = schedule_of(BANDED.replace("if j > i:", "if False:").replace("if k < i - 128:", "if False:"),
                      spec(2, 512, 512, dtype=F32), B=2)
    assert sch.tables == {} and sch.steps_per_tile == 4  # masks that skip nothing make no tables
    sch = schedule_of(
        """
        def f(x):
            out = jnp.zeros((256, 256))
            for i in range(0, 256, 128):
                for j in range(0, 256, 128):
                    out = out.at[i : i + 128, j : j + 128].set(x[i : i + 128, j : j + 128])
            return out
        """, spec(256, 256, dtype=F32))
    assert (sch.steps, sch.steps_per_tile, sch.tables) == (4, 1, {})
    assert [sch.blocks_at(t) for t in range(4)] == [(0, 0), (0, 1), (1, 0), (1, 1)]


@pytest.mark.parametrize(("tile_mask", "step_mask", "message"), [
    ("True", "False", "the masks skip every output tile"),
    ("False", "undefined", "can't evaluate `undefined`"),
    ("False", "jnp.ones(2) > 0", "masks are Python conditions on loop variables"),
])
def test_mask_errors(tile_mask, step_mask, message):
    # tests/test_schedule.py:76-100
    source = f"""
        def f(x):
            out = jnp.zeros((256, 128))
            for i in range(0, 256, 128):
                if {tile_mask}:
                    continue
                acc = jnp.zeros((128, 128))
                for k in range(0, 256, 128):
                    if {step_mask}:
                        continue
                    acc += x[i : i + 128, k : k + 128]
                out = out.at[i : i + 128, :].set(acc)
            return out
        """
    with pytest.raises(KernelError, match=message):
        schedule_of(source, spec(256, 256, dtype=F32))


@pytest.mark.parametrize("skip", ["True", "i == 0", "i == 128 and k == 0"])
def test_a_phase_whose_mask_skips_all_of_a_tiles_blocks_takes_one_empty_step(skip):
    # tests/test_schedule.py:103-128 (the schedule half)
    sch = schedule_of(f"""
        def f(x):
            out = jnp.zeros((256, 128))
            for i in range(0, 256, 128):
                acc = jnp.full((128, 128), 2.0)
                for k in range(0, 256, 128):
                    if {skip}:
                        continue
                    acc += x[i : i + 128, k : k + 128]
                out = out.at[i : i + 128, :].set(acc + 1)
            return out
        """, spec(256, 256, dtype=F32))
    runs = {(i, k) for i in (0, 128) for k in (0, 128) if not eval(skip, {"i": i, "k": k})}
    assert sch.empty == (len({i for i, _ in runs}) < 2)
    steps = [(sch.step_at(s), sch.empty_at(s)) for s in range(sch.steps)]
    for i in (0, 128):
        mine = [k for (tile, _, k), empty in steps if tile == i // 128 and not empty]
        assert mine == [k // 128 for ii, k in sorted(runs) if ii == i]
    # An empty step's code is block 0 | empty | first | last = 7 (src/autokernel/schedule.py:339-342).
    if sch.empty:
        assert 7 in sch.tables["step_code"].tolist()


MASKED = """
def f(x, y):
    out = jnp.full((4, 512, 256), -jnp.inf)
    other = jnp.zeros((4, 512, 256), jnp.bfloat16)
    for b in range(4):
        for i in range(0, 512, 128):
            for j in range(0, 256, 128):
                if j > i:
                    continue
                acc = jnp.zeros((128, 128))
                for k in range(0, 384, 128):
                    if k > i + 128 or k < i - 128:
                        continue
                    acc += x[b, i : i + 128, k : k + 128] @ y[k : k + 128, j : j + 128]
                out = out.at[b, i : i + 128, j : j + 128].set(acc)
                other = other.at[b, i : i + 128, j : j + 128].set((acc * 2).astype(jnp.bfloat16))
    return out, other
"""


def test_tile_and_step_masks_with_an_outer_loop_and_two_outputs():
    # tests/test_codegen.py:49-61 (the schedule half)
    sch = schedule_of(MASKED, spec(4, 512, 384, dtype=F32), spec(384, 256, dtype=F32))
    assert sch.repeats == 4 and sch.pattern_tiles == 7 and sch.pattern_fills == 1 and sch.fills == 4
    assert sch.steps == 4 * sum(min(3, i // 128 + 2) - max(0, i // 128 - 1)
                                for i in range(0, 512, 128) for j in range(0, 256, 128) if j <= i)
    assert sch.tables["fill_i"].tolist() == [0] and sch.tables["fill_j"].tolist() == [1]


TWO_PASS = """
def f(x, w):
    M, D = x.shape
    out = jnp.zeros((M, 256))
    for i in range(0, M, 128):
        sum_sq = jnp.zeros((128, 128))
        for k in range(0, D, 128):
            xk = x[i : i + 128, k : k + 128]
            sum_sq += xk * xk
        scale = jax.lax.rsqrt(jnp.sum(sum_sq, axis=1, keepdims=True) / D + 1e-6)
        acc = jnp.zeros((128, 256))
        for k2 in range(0, D, 128):
            acc += (x[i : i + 128, k2 : k2 + 128] * scale) @ w[k2 : k2 + 128, :]
        out = out.at[i : i + 128, :].set(acc)
    return out
"""


def test_phases_decode_arithmetically():
    # tests/test_schedule.py:200-207
    sch = schedule_of(TWO_PASS, spec(256, 384, dtype=F32), spec(384, 256, dtype=F32))
    assert not sch.step_tables and sch.phase_counts == (3, 3) and sch.phase_steps == (6, 6)
    want = [(tile, phase, k) for tile in range(2) for phase in range(2) for k in range(3)]
    assert [sch.step_at(s) for s in range(sch.steps)] == want


def test_masked_phases_pack_the_phase_into_the_code():
    # Two phases, the first masked: the codes hold (block * 2 + phase) << 3 | flags (phase radix 2).
    sch = schedule_of("""
        def f(x, w):
            out = jnp.zeros((256, 128))
            for i in range(0, 256, 128):
                a = jnp.zeros((128, 128))
                for k in range(0, 384, 128):
                    if k > i:
                        continue
                    a += x[i : i + 128, k : k + 128]
                acc = jnp.zeros((128, 128))
                for k2 in range(0, 256, 128):
                    acc += a @ w[k2 : k2 + 128, :]
                out = out.at[i : i + 128, :].set(acc)
            return out
        """, spec(256, 384, dtype=F32), spec(256, 128, dtype=F32))
    assert sch.step_tables and sch.phase_radix == 2 and sch.phase_counts == (3, 2)
    want = [(0, 0, 0), (0, 1, 0), (0, 1, 1), (1, 0, 0), (1, 0, 1), (1, 1, 0), (1, 1, 1)]
    assert [sch.step_at(s) for s in range(sch.steps)] == want and sch.phase_steps == (3, 4)


def test_step_codes_take_power_of_two_radices_while_they_fit():
    # tests/test_schedule.py:210-221
    assert schedule.radices(3, 5, 100) == (4, 8)        # decoded with shifts and masks
    assert schedule.radices(3, 5, 2**26) == (3, 5)      # 2**26 * 4 * 8 << 3 overflows int32: exact radices


def test_step_arithmetic_stays_in_int32():
    # tests/test_schedule.py:174-186
    source = """
        def f(x):
            out = jnp.zeros((2**20, 256, 128))
            for b in range(2**20):
                for i in range(0, 256, 128):
                    if i:
                        continue
                    out = out.at[b, i : i + 128, :].set(1.0)
            return out
        """
    with pytest.raises(KernelError, match="int32 step arithmetic"):
        schedule_of(source, spec(8, 128, dtype=F32))


def test_the_hot_path_nests_get_the_same_tables_from_the_general_builder():
    import oracle

    sch = schedule.causal_matmul_schedule(8192, 8192, 8192, 512, 512, 512)
    assert (sch.tiles, sch.total_tiles, sch.fills, sch.steps) == (136, 256, 120, 2176)
    for name, values in oracle.causal_tile_tables(8192, 8192, 512, 512).items():
        np.testing.assert_array_equal(sch.tables[name], values)
    sch = schedule.causal_attention_schedule(4, 16, 2048, 512, 512)
    tile, code = oracle.attention_step_tables(2048, 512, 512)
    np.testing.assert_array_equal(sch.tables["step_tile"], tile)
    np.testing.assert_array_equal(sch.tables["step_code"], code)
    assert sch.tables["step_code"].tolist() == [3, 2, 9, 2, 8, 17, 2, 8, 16, 25] and sch.repeats == 64
    assert [r.var for r in sch.outer] == ["b", "h"] and (sch.tiles, sch.steps) == (256, 640)
    one = schedule.causal_matmul_schedule(256, 256, 256, 256, 256, 128)  # tests/test_schedule.py:189-198
    assert one.tables == {}
    decode = schedule.paged_decode_schedule(64, 256)
    assert decode.runtime and decode.empty and decode.steps == 64 * 256 and decode.tiles == 64
