"""The order a kernel runs its steps in, and the int32 tables that say which tiles and steps run.

A kernel is one loop over steps. Tiles run in the parallel loops' order (row-major, outermost slowest); a tile's
steps are its phases' steps back to back — a phase is one reduction loop of the tile. Masks that read only loop
variables are evaluated here, on the host, once per kernel build, and the kernels walk the resulting tables. The
table names, the packing of a step's code and the skip rules are the reference's (src/autokernel/schedule.py:46-55,
:138-220, :339-358), so the tables are bit-identical to its own:

  tile tables  "tile_<var>" / "fill_<var>": block index of each covered parallel loop for the tiles that run / that
               a tile mask skips (those are written with the output's fill value)
  step tables  "step_tile" / "step_code": for every step of one pattern, its tile and
               ((block * phases + phase) * iterations + iteration) << 3 | empty << 2 | first << 1 | last

Tables cover only the loops the masks read — the innermost parallel loops from the first one any mask reads:
causal attention's masks read neither batch nor head, so its tables hold one (b, h) pattern, repeated
(schedule.py:14-16). Without masks (or with masks that skip nothing) a step's tile, phase and block are arithmetic
on the step index and there are no tables. A tile whose mask skips every block of a phase still takes one step of
it, an empty one. Masks that read index arrays can only be evaluated on the device: such a schedule describes every
step that could run (`runtime`), and the tables are built by tjx_build_steps just before the kernel.
"""

from __future__ import annotations

import itertools
import math
from collections.abc import Callable, Mapping, Sequence
from dataclasses import dataclass, field

import numpy as np

CODE_SHIFT = 3
STEP_TILE, STEP_CODE = "step_tile", "step_code"


class ScheduleError(ValueError):
    """A schedule that cannot be built (the masks leave nothing to run)."""


@dataclass(frozen=True)
class Range:
    """One `for var in range(start, stop, step)` loop."""

    var: str
    start: int
    stop: int
    step: int

    @property
    def count(self) -> int:
        return max(0, -(-(self.stop - self.start) // self.step))

    def value(self, block: int) -> int:
        return self.start + block * self.step


@dataclass(frozen=True)
class Mask:
    """`if holds(values): continue` at the top of loop `on`'s body; `reads` are the loop variables it looks at."""

    on: str
    reads: frozenset[str]
    holds: Callable[[Mapping[str, int]], bool]


@dataclass(frozen=True)
class Schedule:
    """Which tiles and steps a kernel runs, in order, and the tables that find them. Field meanings as the
    reference's Schedule (src/autokernel/schedule.py:58-92)."""

    tiles: int                       # output tiles that run
    total_tiles: int                 # output tiles, skipped ones included
    steps: int
    step_tables: bool                # are steps found through tables (a mask skips steps), or arithmetic
    tile_tables: bool                # are tiles found through tables (a tile mask skips tiles), or arithmetic
    pattern_tiles: int               # tiles that run per combination of the outer loops
    pattern_steps: int               # steps per combination of the outer loops
    pattern_fills: int               # tiles skipped per combination of the outer loops
    tables: dict[str, np.ndarray] = field(default_factory=dict)
    empty: bool = False              # may a step be empty
    runtime: bool = False            # step tables made on the device; `steps` is the most there can be
    phase_counts: tuple[int, ...] = ()   # each phase's reduction blocks
    phase_steps: tuple[int, ...] = ()    # each phase's steps over the whole run
    outer: tuple[Range, ...] = ()    # parallel loops no mask reads: arithmetic on the step or tile index
    inner: tuple[Range, ...] = ()    # the parallel loops the tables cover
    iterations: int = 1              # radix of the repeat-loop iteration in a step's code (no repeat loops here: 1)
    phase_radix: int = 1             # radix of the phase in a step's code

    @property
    def steps_per_tile(self) -> int:
        """A tile's steps when nothing is masked: every phase's blocks (one step if there are no phases)."""
        return sum(self.phase_counts) or 1

    @property
    def repeats(self) -> int:
        """How many times the tables' pattern repeats: once per combination of the outer loops."""
        return math.prod(r.count for r in self.outer)

    @property
    def fills(self) -> int:
        return self.pattern_fills * self.repeats

    def step_at(self, step: int) -> tuple[int, int, int]:
        """(the tile, the phase, the reduction block) of a step (src/autokernel/schedule.py:109-122)."""
        if not self.step_tables:
            tile, within = divmod(step, self.steps_per_tile)
            phase = 0
            for count in self.phase_counts[:-1]:
                if within < count:
                    break
                within -= count
                phase += 1
            return tile, phase, within
        repeat, at = divmod(step, self.pattern_steps)
        packed = (int(self.tables[STEP_CODE][at]) >> CODE_SHIFT) // self.iterations
        return repeat * self.pattern_tiles + int(self.tables[STEP_TILE][at]), packed % self.phase_radix, packed // self.phase_radix

    def first_at(self, step: int) -> bool:
        return bool(int(self.tables[STEP_CODE][step % self.pattern_steps]) & 2)

    def last_at(self, step: int) -> bool:
        return bool(int(self.tables[STEP_CODE][step % self.pattern_steps]) & 1)

    def empty_at(self, step: int) -> bool:
        return self.empty and self.step_tables and bool(int(self.tables[STEP_CODE][step % self.pattern_steps]) & 4)

    def blocks_at(self, tile: int) -> tuple[int, ...]:
        """The parallel loops' blocks of the `tile`-th tile that runs (src/autokernel/schedule.py:138-144)."""
        if not self.tile_tables:
            return _mixed_radix(tile, self.outer + self.inner)
        repeat, at = divmod(tile, self.pattern_tiles)
        covered = tuple(int(self.tables[f"tile_{r.var}"][at]) for r in self.inner)
        return _mixed_radix(repeat, self.outer) + covered


def _mixed_radix(index: int, ranges: Sequence[Range]) -> tuple[int, ...]:
    """The block of each loop at row-major position `index` (outermost first)."""
    digits = []
    for r in reversed(ranges):
        index, digit = divmod(index, r.count)
        digits.append(digit)
    return tuple(reversed(digits))


def step_code(block: int, empty: bool, first: bool, last: bool, phase: int = 0, phase_radix: int = 1,
              iteration: int = 0, iterations: int = 1) -> int:
    return ((block * phase_radix + phase) * iterations + iteration) << CODE_SHIFT | int(empty) << 2 | int(first) << 1 | int(last)


def radices(phases: int, iterations: int, blocks: int) -> tuple[int, int]:
    """The radices of the phase and of the iteration in a step's code: powers of two while every code still fits in
    31 bits (so a step decodes with shifts and masks), else the exact counts (src/autokernel/schedule.py:222-232)."""
    rounded = tuple(1 << max(n - 1, 0).bit_length() for n in (phases, iterations))
    if (blocks * rounded[0] * rounded[1]) << CODE_SHIFT < 2**31:
        return rounded
    return phases, iterations


def make_schedule(parallel: Sequence[Range], phases: Sequence[Range], masks: Sequence[Mask] = ()) -> Schedule:
    """The schedule of a loop nest whose masks read loop variables only. Raises ScheduleError if the masks leave no
    tile to run. Tables are made only for what the masks actually skip."""
    parallel, phases = tuple(parallel), tuple(phases)
    counts = tuple(r.count for r in phases)
    parallel_vars = {r.var for r in parallel}
    tile_masks = [m for m in masks if m.on in parallel_vars]
    step_masks = {m.on: m for m in masks if m.on not in parallel_vars}
    if not masks:
        return _arithmetic(parallel, counts)
    read = set().union(*(m.reads for m in masks))
    split = next((n for n, r in enumerate(parallel) if r.var in read), len(parallel))
    outer, inner = parallel[:split], parallel[split:]
    phase_radix, iterations = radices(len(phases), 1, max(counts, default=1))

    active: list[tuple[int, ...]] = []
    skipped: list[tuple[int, ...]] = []
    runs: list[list[list[int]]] = []  # per active tile, per phase, the blocks that run
    for blocks in itertools.product(*(range(r.count) for r in inner)):
        values = {r.var: r.value(b) for r, b in zip(inner, blocks, strict=True)}
        if any(m.holds(values) for m in tile_masks):
            skipped.append(blocks)
            continue
        active.append(blocks)
        per_phase = []
        for r in phases:
            m = step_masks.get(r.var)
            per_phase.append([kb for kb in range(r.count) if m is None or not m.holds({**values, r.var: r.value(kb)})])
        runs.append(per_phase)
    if not active:
        raise ScheduleError("the masks skip every output tile")
    stepwise = any(ks != list(range(r.count)) for tile in runs for ks, r in zip(tile, phases, strict=True))
    if not skipped and not stepwise:
        return _arithmetic(parallel, counts)  # the masks skip nothing

    tables: dict[str, np.ndarray] = {}
    if skipped:
        for n, r in enumerate(inner):
            tables[f"tile_{r.var}"] = np.array([b[n] for b in active], np.int32)
            tables[f"fill_{r.var}"] = np.array([b[n] for b in skipped], np.int32)
    any_empty = False
    if stepwise:
        tile_of: list[int] = []
        codes: list[int] = []
        for t, tile in enumerate(runs):
            for phase, ks in enumerate(tile):
                taken = ks or [0]  # a phase none of whose blocks run takes one empty step
                any_empty |= not ks
                tile_of += [t] * len(taken)
                codes += [step_code(kb, not ks, n == 0, n == len(taken) - 1, phase, phase_radix, 0, iterations)
                          for n, kb in enumerate(taken)]
        tables[STEP_TILE] = np.array(tile_of, np.int32)
        tables[STEP_CODE] = np.array(codes, np.int32)
    per_phase_steps = [sum(max(len(tile[p]), 1) for tile in runs) for p in range(len(phases))]
    pattern_steps = sum(per_phase_steps) or len(active)
    repeats = math.prod(r.count for r in outer)
    if repeats * len(active) * max(repeats * len(skipped), 1) >= 2**31:  # src/autokernel/schedule.py:372-376
        raise ScheduleError("too many output tiles for the kernel's int32 step arithmetic")
    return Schedule(
        tiles=repeats * len(active), total_tiles=math.prod(r.count for r in parallel), steps=repeats * pattern_steps,
        step_tables=stepwise, tile_tables=bool(skipped), pattern_tiles=len(active), pattern_steps=pattern_steps,
        pattern_fills=len(skipped), tables=tables, empty=any_empty, phase_counts=counts,
        phase_steps=tuple(repeats * n for n in per_phase_steps), outer=outer, inner=inner, iterations=iterations,
        phase_radix=phase_radix)


def _arithmetic(parallel: tuple[Range, ...], counts: tuple[int, ...]) -> Schedule:
    """Every tile runs every step: no tables (src/autokernel/schedule.py:379-396)."""
    tiles = math.prod(r.count for r in parallel)
    per_tile = sum(counts) or 1
    return Schedule(tiles=tiles, total_tiles=tiles, steps=tiles * per_tile, step_tables=False, tile_tables=False,
                    pattern_tiles=tiles, pattern_steps=tiles * per_tile, pattern_fills=0, phase_counts=counts,
                    phase_steps=tuple(tiles * c for c in counts), outer=parallel, inner=())


def runtime_schedule(parallel: Sequence[Range], phases: Sequence[Range]) -> Schedule:
    """A schedule whose step tables are made on the device (a mask reads an index array): every (tile, block) step
    could run, a tile with none takes one empty step, and `steps` is the most there can be
    (src/autokernel/schedule.py:241-298)."""
    parallel, phases = tuple(parallel), tuple(phases)
    counts = tuple(r.count for r in phases)
    tiles = math.prod(r.count for r in parallel)
    capacity = tiles * sum(counts)
    phase_radix, iterations = radices(len(phases), 1, max(counts, default=1))
    return Schedule(tiles=tiles, total_tiles=tiles, steps=capacity, step_tables=True, tile_tables=False,
                    pattern_tiles=tiles, pattern_steps=capacity, pattern_fills=0, empty=True, runtime=True,
                    phase_counts=counts, phase_steps=tuple(tiles * c for c in counts), outer=(), inner=parallel,
                    iterations=iterations, phase_radix=phase_radix)


# ------------------------------------------------------------------------------------------ the hot-path nests


def matmul_schedule(M: int, N: int, K: int, tm: int, tn: int, tk: int) -> Schedule:
    """Dense matmul (examples/matmul.py:22-35): every tile runs every block, no tables."""
    return make_schedule([Range("i", 0, M, tm), Range("j", 0, N, tn)], [Range("k", 0, K, tk)])


def causal_matmul_schedule(M: int, N: int, K: int, tm: int, tn: int, tk: int) -> Schedule:
    """Tile mask `j > i + tm - 1` (examples/causal_matmul.py:32): tile tables when it skips anything; the steps inside
    a tile stay arithmetic."""
    above = Mask("j", frozenset({"i", "j"}), lambda v: v["j"] > v["i"] + tm - 1)
    return make_schedule([Range("i", 0, M, tm), Range("j", 0, N, tn)], [Range("k", 0, K, tk)], [above])


def causal_attention_schedule(B: int, H: int, S: int, bq: int, bk: int) -> Schedule:
    """Step mask `j > i + bq - 1` (examples/causal_attention.py:49): step tables for one (b, h) pattern, repeated
    B * H times; no tile is skipped, so no tile tables and no fills."""
    future = Mask("j", frozenset({"i", "j"}), lambda v: v["j"] > v["i"] + bq - 1)
    return make_schedule([Range("b", 0, B, 1), Range("h", 0, H, 1), Range("i", 0, S, bq)], [Range("j", 0, S, bk)],
                         [future])


def paged_decode_schedule(B: int, pages_per_seq: int) -> Schedule:
    """Runtime mask `p * P >= lengths[b]`: the step tables are made on the device."""
    return runtime_schedule([Range("b", 0, B, 1)], [Range("p", 0, pages_per_seq, 1)])


def collective_row_blocks(me: int, chips: int, shard_blocks: int) -> np.ndarray:
    """Row blocks of the gathered operand in the order chip `me` walks them: a shard at a time, its own first,
    then the shard of chip (me - r) mod chips at ring step r (src/autokernel/plan.py:225-238,
    src/autokernel/codegen.py:958-962)."""
    i_blk = np.arange(chips * shard_blocks)
    r, within = np.divmod(i_blk, shard_blocks)
    return (((me + chips - r) % chips) * shard_blocks + within).astype(np.int32)


MLA_UNIT = 32        # positions per unit of the tcgen05 MLA decode kernel's work
MLA_PIECE_COST = 3   # what starting on a sequence costs a CTA, in units
MLA_MIN_SHARE = 2    # units a CTA takes at least


def mla_unit_ranges(lengths: Sequence[int], ctas: int) -> list[list[tuple[int, int, int]]]:
    """How the tcgen05 MLA decode kernel shares a launch's work out, as the kernel itself derives it from `lengths`
    (every CTA runs the same arithmetic; there is no table): per CTA the list of its pieces (sequence, first unit,
    units). A sequence's cache is cut into units of 32 positions; the units of all sequences lie on one line with
    MLA_PIECE_COST more positions in front of every sequence that has any, and CTA c takes the positions
    [c * share, (c + 1) * share) of that line, share = max(MLA_MIN_SHARE + MLA_PIECE_COST, ceil(line / ctas)): a CTA
    whose range crosses into another sequence gets fewer units, by about what starting a piece costs it. The pieces of
    a sequence come from consecutive CTAs, first = (start of its units) // share, so its partials sit at consecutive
    workspace indices (CTA + sequence) and the merge kernel finds them with the same arithmetic."""
    units = [(max(int(n), 0) + MLA_UNIT - 1) // MLA_UNIT for n in lengths]
    before = [0]
    for n in units:
        before.append(before[-1] + (n + MLA_PIECE_COST if n else 0))
    line = before[-1]
    share = max(MLA_MIN_SHARE + MLA_PIECE_COST, -(-line // max(ctas, 1)))
    out: list[list[tuple[int, int, int]]] = []
    for c in range(ctas):
        begin = min(c * share, line)
        end = min(begin + share, line)
        pieces = []
        u = begin
        while u < end:
            b = max(i for i in range(len(units)) if before[i] <= u)
            first_unit = before[b] + MLA_PIECE_COST
            start, stop = max(u, first_unit), min(end, before[b + 1])
            if stop > start:
                pieces.append((b, start - first_unit, stop - start))
            u = min(end, before[b + 1])
        out.append(pieces)
    return out


def mla_pieces_of(lengths: Sequence[int], ctas: int, b: int) -> tuple[int, int]:
    """(first CTA, number of pieces) of sequence `b` under `mla_unit_ranges`, by the merge kernel's closed form."""
    units = [(max(int(n), 0) + MLA_UNIT - 1) // MLA_UNIT for n in lengths]
    before = [0]
    for n in units:
        before.append(before[-1] + (n + MLA_PIECE_COST if n else 0))
    if before[b + 1] == before[b]:
        return 0, 0
    share = max(MLA_MIN_SHARE + MLA_PIECE_COST, -(-before[-1] // max(ctas, 1)))
    first = (before[b] + MLA_PIECE_COST) // share
    return first, (before[b + 1] - 1) // share - first + 1
