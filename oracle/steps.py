"""Oracle for the integer half of the hot path: which tiles and steps run, and the tables that say so.

Test infrastructure only (see oracle/__init__.py). Three restatements:

  walk_nest             the loop nest itself, with its `continue` masks, as the ground truth for every table
                        (how tests/test_schedule.py:35-51 checks the reference's schedules)
  causal_tile_tables    static tile / fill tables for a tile mask (src/autokernel/schedule.py:159-193, :349-358)
  attention_step_tables static step tables for a step mask (schedule.py:196-211, code packing :339-342)
  device_step_tables    the tables the generated `<kernel>_steps` makes on the device for runtime masks
                        (src/autokernel/codegen.py:386-431)
"""

from __future__ import annotations

import numpy as np

CODE_SHIFT = 3  # schedule.py:55


def pack_code(block: int, empty: bool, first: bool, last: bool, phase: int = 0, phases: int = 1,
              iteration: int = 0, iterations: int = 1) -> int:
    """A step's code (schedule.py:339-342): ((block * phases + phase) * iterations + iteration) << 3 | flags."""
    return ((block * phases + phase) * iterations + iteration) << CODE_SHIFT | int(empty) << 2 | int(first) << 1 | int(last)


def walk_nest(tile_ranges, block_range, tile_mask=None, step_mask=None):
    """Run a loop nest of parallel loops `tile_ranges` (each a Python range) around one reduction loop
    `block_range`, honouring `if tile_mask(*tile_values): continue` on the innermost parallel loop and
    `if step_mask(*tile_values, block_value): continue` on the reduction loop.

    Returns (steps, fills): steps = [(tile_blocks, block_index or None)] in execution order, where a tile
    whose every block is masked takes one empty step (block None), as the reference's kernels do
    (schedule.py:17-20); fills = [tile_blocks] of the tiles the tile mask skips."""
    steps, fills = [], []

    def rec(depth, values, blocks):
        if depth == len(tile_ranges):
            if tile_mask is not None and tile_mask(*values):
                fills.append(tuple(blocks))
                return
            ran = False
            for kb, kv in enumerate(block_range):
                if step_mask is not None and step_mask(*values, kv):
                    continue
                steps.append((tuple(blocks), kb))
                ran = True
            if not ran:
                steps.append((tuple(blocks), None))
            return
        for b, v in enumerate(tile_ranges[depth]):
            rec(depth + 1, [*values, v], [*blocks, b])

    rec(0, [], [])
    return steps, fills


def causal_tile_tables(M: int, N: int, tm: int, tn: int):
    """Tables of `causal_matmul` (examples/causal_matmul.py:29-33): the tile mask `j > i + tm - 1` evaluated per
    (i, j) in row-major order; tiles that run go to tile_i / tile_j, skipped ones to fill_i / fill_j
    (schedule.py:159-166, :349-358). Returns a dict of int32 arrays; empty when nothing is skipped (:189-190)."""
    active, skipped = [], []
    for bi, i in enumerate(range(0, M, tm)):
        for bj, j in enumerate(range(0, N, tn)):
            (skipped if j > i + tm - 1 else active).append((bi, bj))
    if not skipped:
        return {}
    as_table = lambda pairs, d: np.array([p[d] for p in pairs], np.int32)  # noqa: E731
    return {"tile_i": as_table(active, 0), "tile_j": as_table(active, 1),
            "fill_i": as_table(skipped, 0), "fill_j": as_table(skipped, 1)}


def attention_step_tables(S: int, bq: int, bk: int):
    """Step tables of `causal_attention` (examples/causal_attention.py:45-50) for one (b, h): the step mask
    `j > i + bq - 1` per query block i and key block j (schedule.py:167-176, :196-211). Returns
    (step_tile, step_code) int32, or None when the mask skips nothing (a single block: schedule.py:189-190)."""
    tile_of, codes, skipped_any = [], [], False
    for t, i in enumerate(range(0, S, bq)):
        runs = [kb for kb, j in enumerate(range(0, S, bk)) if not j > i + bq - 1]
        skipped_any |= len(runs) != len(range(0, S, bk))
        runs_or_empty = runs or [0]
        for n, kb in enumerate(runs_or_empty):
            tile_of.append(t)
            codes.append(pack_code(kb, not runs, n == 0, n == len(runs_or_empty) - 1))
    if not skipped_any:
        return None
    return np.array(tile_of, np.int32), np.array(codes, np.int32)


def lengths_runs(lengths, blocks: int, value0: int, value_step: int, tile_values=None) -> np.ndarray:
    """run[t, k] for the runtime mask `value0 + k * value_step >= lengths[tile_values[t]]: continue`
    (examples/decode.py:188 and :214; vectorised as codegen.py:440-443 does)."""
    lengths = np.asarray(lengths, np.int64)
    tv = np.arange(len(lengths)) if tile_values is None else np.asarray(tile_values)
    values = value0 + np.arange(blocks, dtype=np.int64) * value_step
    return np.logical_not(values[None, :] >= lengths[tv][:, None])


def device_step_tables(run: np.ndarray):
    """(step_tile, step_code, step_count) from run[tiles, blocks], one phase, no repeat loop
    (codegen.py:392-403 for the codes, :425-431 for the compaction)."""
    run = np.asarray(run, bool)
    tiles, blocks = run.shape
    k = np.arange(blocks)
    empty = ~run.any(axis=1, keepdims=True) & (k == 0)
    keep = run | empty
    first = k == np.argmax(keep, axis=1)[:, None]
    last = k == blocks - 1 - np.argmax(keep[:, ::-1], axis=1)[:, None]
    code = (k << CODE_SHIFT) | (empty.astype(np.int64) << 2) | (first.astype(np.int64) << 1) | last.astype(np.int64)
    code = np.broadcast_to(code, run.shape).reshape(-1).astype(np.int32)
    tile = np.repeat(np.arange(tiles, dtype=np.int32), blocks)
    keep = keep.reshape(-1)
    order = np.argsort(~keep, kind="stable")
    return tile[order], code[order], np.array([keep.sum()], np.int32)
