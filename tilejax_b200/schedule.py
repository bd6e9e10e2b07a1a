"""Static schedules of the hot-path kernels: which tiles and steps run, and the int32 tables that say so.

Masks that read only loop variables are evaluated here, on the host, once per kernel build; the kernels walk
the resulting tables. The table names, packing and skip rules are the reference's
(src/autokernel/schedule.py:46-55, :138-220, :339-358), so the tables are bit-identical to its own:

  tile tables  "tile_<var>" / "fill_<var>": block index of each parallel loop for the tiles that run / that a
               tile mask skips (those are written with the output's fill value)
  step tables  "step_tile" / "step_code": for every step of one pattern, its tile and
               block << 3 | empty << 2 | first << 1 | last

Tables cover only the loops the masks read: causal attention's masks read neither batch nor head, so its tables
hold one (b, h) pattern, repeated `repeats` times (schedule.py:14-16).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

CODE_SHIFT = 3


@dataclass(frozen=True)
class Schedule:
    """Counts and tables of a kernel's steps. Field meanings as the reference's Schedule (schedule.py:58-92)."""

    tiles: int
    total_tiles: int
    steps: int
    step_tables: bool
    tile_tables: bool
    pattern_tiles: int
    pattern_steps: int
    pattern_fills: int
    repeats: int = 1
    tables: dict[str, np.ndarray] = field(default_factory=dict)
    empty: bool = False
    runtime: bool = False  # step tables made on the device; `steps` is the most there can be

    @property
    def fills(self) -> int:
        return self.pattern_fills * self.repeats


def step_code(block: int, empty: bool, first: bool, last: bool) -> int:
    return block << CODE_SHIFT | int(empty) << 2 | int(first) << 1 | int(last)


def matmul_schedule(M: int, N: int, K: int, tm: int, tn: int, tk: int) -> Schedule:
    """Dense matmul: every tile runs every block, no tables (schedule.py:379-396)."""
    tiles = (M // tm) * (N // tn)
    per_tile = K // tk
    return Schedule(tiles, tiles, tiles * per_tile, False, False, tiles, tiles * per_tile, 0)


def causal_matmul_schedule(M: int, N: int, K: int, tm: int, tn: int, tk: int) -> Schedule:
    """Tile mask `j > i + tm - 1` (examples/causal_matmul.py:32): tile tables when it skips anything; the steps
    inside a tile stay arithmetic (schedule.py:172-193)."""
    bi, bj = np.meshgrid(np.arange(M // tm), np.arange(N // tn), indexing="ij")
    skip = (bj * tn > bi * tm + tm - 1).reshape(-1)
    bi, bj = bi.reshape(-1).astype(np.int32), bj.reshape(-1).astype(np.int32)
    per_tile = K // tk
    active = int((~skip).sum())
    tables = {}
    if skip.any():
        tables = {"tile_i": bi[~skip], "tile_j": bj[~skip], "fill_i": bi[skip], "fill_j": bj[skip]}
    return Schedule(active, skip.size, active * per_tile, False, bool(skip.any()), active, active * per_tile,
                    int(skip.sum()), 1, tables)


def causal_attention_schedule(B: int, H: int, S: int, bq: int, bk: int) -> Schedule:
    """Step mask `j > i + bq - 1` (examples/causal_attention.py:49): step tables for one (b, h) pattern,
    repeated B * H times; no tile is skipped, so no tile tables and no fills."""
    nq, nk = S // bq, S // bk
    j = np.arange(nk) * bk
    tile_of, codes = [], []
    for t in range(nq):
        runs = np.flatnonzero(~(j > t * bq + bq - 1))
        for n, kb in enumerate(runs):
            tile_of.append(t)
            codes.append(step_code(int(kb), False, n == 0, n == len(runs) - 1))
    skipped = len(codes) != nq * nk
    tables = {}
    if skipped:
        tables = {"step_tile": np.array(tile_of, np.int32), "step_code": np.array(codes, np.int32)}
    repeats = B * H
    return Schedule(repeats * nq, repeats * nq, repeats * len(codes), skipped, False, nq, len(codes), 0, repeats, tables)


def paged_decode_schedule(B: int, pages_per_seq: int) -> Schedule:
    """Runtime mask `p * P >= lengths[b]`: the step tables are made on the device; every (sequence, page) step
    could run, and a sequence with none takes one empty step (schedule.py:241-298)."""
    capacity = B * pages_per_seq
    return Schedule(B, B, capacity, True, False, B, capacity, 0, 1, {}, True, True)


def collective_row_blocks(me: int, chips: int, shard_blocks: int) -> np.ndarray:
    """Row blocks of the gathered operand in the order chip `me` walks them: a shard at a time, its own first,
    then the shard of chip (me - r) mod chips at ring step r (src/autokernel/plan.py:225-238,
    src/autokernel/codegen.py:958-962)."""
    i_blk = np.arange(chips * shard_blocks)
    r, within = np.divmod(i_blk, shard_blocks)
    return (((me + chips - r) % chips) * shard_blocks + within).astype(np.int32)
