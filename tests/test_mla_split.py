"""How the tcgen05 MLA decode kernel shares units of 32 positions out over its CTAs (`schedule.mla_unit_ranges`, the
host-side statement of the arithmetic every CTA of `mla_tc_kernel` runs on `lengths`): every unit exactly once, a
sequence's pieces on consecutive CTAs where the merge kernel's closed form says, fewer units for a CTA that starts on
more sequences."""

import numpy as np

from tilejax_b200 import schedule


def check(lengths, ctas):
    ranges = schedule.mla_unit_ranges(lengths, ctas)
    assert len(ranges) == ctas
    units = [(max(int(n), 0) + 31) // 32 for n in lengths]
    seen = [np.zeros(n, int) for n in units]
    owners = [[] for _ in units]
    for c, pieces in enumerate(ranges):
        assert [b for b, _, _ in pieces] == sorted({b for b, _, _ in pieces})  # one piece per sequence, in order
        for b, first, n in pieces:
            assert n > 0
            seen[b][first : first + n] += 1
            owners[b].append(c)
    for b, n in enumerate(units):
        assert (seen[b] == 1).all()
        first, count = schedule.mla_pieces_of(lengths, ctas, b)
        assert owners[b] == list(range(first, first + count))
    return ranges


def test_every_unit_once_and_pieces_where_the_merge_looks_for_them():
    rng = np.random.default_rng(0)
    for _ in range(200):
        batch = int(rng.integers(1, 300))
        lengths = rng.integers(0, int(rng.integers(2, 3000)), batch)
        lengths[rng.random(batch) < 0.3] = 0
        check(lengths, int(rng.integers(1, 257)))
    check([0, 0, 0], 148)
    check([1], 148)
    check([4096] * 32, 148)


def test_a_cta_that_crosses_into_another_sequence_gets_fewer_units():
    lengths = np.random.default_rng(0).integers(1024, 3073, 32)  # the benchmark's shape
    ranges = check(lengths, 148)
    by_pieces = {}
    for pieces in ranges:
        if pieces:
            by_pieces.setdefault(len(pieces), []).append(sum(n for _, _, n in pieces))
    assert set(by_pieces) == {1, 2}
    full = [n for n in by_pieces[1] if n == max(by_pieces[1])]
    assert len(full) > len(by_pieces[1]) // 2                      # most one-piece CTAs take a whole share
    assert max(by_pieces[2]) <= max(by_pieces[1]) - schedule.MLA_PIECE_COST  # a second piece costs its margin
