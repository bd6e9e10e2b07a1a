"""`autokernel.all_gather`: an input gathered across the GPUs of a process group, as kernel code reads it.

In a kernel's prologue `xs = autokernel.all_gather(x, "x")` is every rank's `x` stacked along its first dimension in
rank order (the reference's meaning: `jax.lax.all_gather(x, axis, axis=0, tiled=True)`,
src/autokernel/collective.py:21-29). Run as plain code — `kernel.fn` / `kernel.reference` — it gathers through
`torch.distributed` if a process group is up, and is the identity on one process.
"""

from __future__ import annotations

from typing import Any

import numpy as np

from .errors import KernelError


def axis_size(axis_name: str = "x") -> int:
    """How many ranks the gather spans: the world size of the default process group (1 without one)."""
    try:
        import torch.distributed as dist

        return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    except Exception:
        return 1


def all_gather(x: Any, axis_name: str) -> Any:
    from . import jaxlike
    from .plan import Spec

    if isinstance(x, Spec):
        raise KernelError("autokernel.all_gather is a prologue statement of its own, `xs = autokernel.all_gather(x, "
                          "axis)`, on an input of the kernel")
    if axis_size(axis_name) == 1:
        return x
    import torch
    import torch.distributed as dist

    host = np.ascontiguousarray(jaxlike.to_numpy(x))
    raw = torch.from_numpy(host.view(np.uint8).reshape(host.shape[0], -1))  # bytes: every backend moves those
    parts = [torch.empty_like(raw) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, raw)
    out = torch.cat(parts, dim=0).numpy().view(host.dtype)
    return jaxlike.Array(out.reshape(-1, *host.shape[1:]))
