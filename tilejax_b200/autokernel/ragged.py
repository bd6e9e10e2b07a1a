"""`pairs`, `unpairs` and `rows`: the reference's helpers for paged caches and ragged batches
(src/autokernel/packing.py:22-31, src/autokernel/ragged.py:23-28), on the CPU stand-in for jax.numpy.

They are what a loop nest MEANS when `kernel.fn` / `kernel.reference` run it on the CPU. The sm_100a kernels read a
cache page's keys and values where they lie (two tensor maps over the one buffer) and write only the rows that are
valid; nothing is packed into words on the GPU.
"""

from __future__ import annotations

import numpy as np

from . import jaxlike

PAST = 2**31 - 1  # an index out of every array: a store there is dropped, a read clamps


def pairs(x):
    """The tile `x` (..., 2, d) of a 16-bit dtype as uint32 words (..., d): x[..., 0, i] in each word's low 16 bits,
    x[..., 1, i] in its high 16 bits."""
    return jaxlike.lax.bitcast_convert_type(jaxlike.numpy.swapaxes(x, -1, -2), np.uint32)


def unpairs(words, dtype):
    """`pairs` undone: uint32 words (..., d) as a tile (..., 2, d) of the 16-bit `dtype`."""
    return jaxlike.numpy.swapaxes(jaxlike.lax.bitcast_convert_type(words, dtype), -1, -2)


def rows(start, stop, size: int):
    """The row indices start, ..., start + size - 1, those at or past `stop` out of bounds."""
    index = int(jaxlike.to_numpy(start)) + np.arange(size, dtype=np.int32)
    return jaxlike.Array(np.where(index < int(jaxlike.to_numpy(stop)), index, PAST).astype(np.int32))
