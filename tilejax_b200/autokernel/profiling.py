"""Where a kernel's time goes on the GPU: `autokernel.profile(kernel, args)`.

The reference reads TPU trace regions its generated kernels carry — input waits, output-slot waits, the tile code
(src/autokernel/profiling.py:1-20) — and its tuner steers by them. Here the kernels carry cycle counters instead
(include/tilejax_b200.h, tjx_set_profile_buffer): every CTA records how long its issuing thread (the one that
feeds the tensor cores; in decode, a warp's leader) waited for inputs to arrive in its ring, how long for room for
its results, and when it started and finished its work items. Averaged over the CTAs that had work and scaled to
the call's device time (CUDA events) they give the same quantities under the same names:

  wait_s      waiting for inputs (TMA loads not hidden behind compute); fill_s of it is the first wait, the ring
              filling, which no amount of buffering removes
  out_wait_s  waiting for room for results (an accumulator the epilogue is still draining)
  compute_s   the issuing thread busy: the tensor pipe (or the warp's arithmetic) has work
  other_s     the rest of the call: set-up before the first work item, draining after the last, launches and, for
              decode, the step-table kernel

`bottleneck` applies the reference's thresholds (src/autokernel/profiling.py:53-55, :128-140).
"""

from __future__ import annotations

import ctypes
from collections.abc import Sequence
from dataclasses import dataclass, field
from typing import Any

DMA_BOUND_SHARE = 0.2       # exposed input + output waits above this share of the device time: "dma"
OVERHEAD_BOUND_SHARE = 0.3  # time outside waits and compute above this share: "overhead"
RECORD_WORDS = 16           # int64 words per CTA in the profile buffer
MAX_CTAS = 8192


@dataclass
class KernelProfile:
    """A kernel's time per call on the device, averaged over the calls profiled (seconds). Field order and names
    are the reference's (src/autokernel/profiling.py:96-113)."""

    name: str
    config: Any
    calls: int
    device_s: float
    regions: bool = False  # did the kernel's counters report (else only `device_s` is known)
    steps: float = 0.0
    wait_s: float = 0.0
    fill_s: float = 0.0
    out_wait_s: float = 0.0
    compute_s: float = 0.0
    scopes: dict[str, float] = field(default_factory=dict)
    logdir: str = ""  # kept for the reference's signature: there is no trace directory here

    @property
    def exposed_wait_s(self) -> float:
        """Input waits the ring did not hide, its filling left out."""
        return max(self.wait_s - self.fill_s, 0.0)

    @property
    def other_s(self) -> float:
        """Whatever is neither waiting nor computing: set-up, draining, launches."""
        return max(self.device_s - (self.wait_s + self.out_wait_s + self.compute_s), 0.0)

    @property
    def bottleneck(self) -> str | None:
        """"dma", "overhead" or "compute"; None when the counters did not report."""
        if not self.regions:
            return None
        if self.exposed_wait_s + self.out_wait_s > DMA_BOUND_SHARE * self.device_s:
            return "dma"
        return "overhead" if self.other_s > OVERHEAD_BOUND_SHARE * self.device_s else "compute"

    def __str__(self) -> str:
        def us(seconds: float) -> str:
            return f"{seconds * 1e6:10.1f} us"

        head = f"{self.name} ({self.config}): {us(self.device_s).strip()} per call over {self.calls} calls"
        if not self.regions:
            return head + "\n  no counters: this kernel does not report where its time goes"
        each = self.device_s / self.steps * 1e6 if self.steps else 0.0
        rows = [
            f"  steps          {self.steps:10.0f}     ({each:.2f} us each)",
            f"  compute        {us(self.compute_s)}",
            f"  input waits    {us(self.exposed_wait_s)}  (+{us(self.fill_s).strip()} filling the pipeline)",
            f"  output waits   {us(self.out_wait_s)}",
            f"  other          {us(self.other_s)}  (set-up, draining, launches)",
        ]
        rows += [f"  scope {name!r:9}{us(seconds)}" for name, seconds in self.scopes.items()]
        rows.append(f"  bottleneck: {self.bottleneck}")
        return "\n".join([head, *rows])


def shares(records) -> dict[str, float] | None:
    """Per-CTA counter records [n, 16] (int64) -> the mean share of a CTA's lifetime its issuing thread spent
    waiting for inputs, filling, waiting for room, computing, and outside its work items. None if no CTA with work
    reported."""
    import numpy as np

    r = np.asarray(records, dtype=np.int64).reshape(-1, RECORD_WORDS)
    life = (r[:, 7] - r[:, 0]).astype(np.float64)
    busy = r[(r[:, 6] > 0) & (life > 0)]
    if busy.shape[0] == 0:
        return None
    life = (busy[:, 7] - busy[:, 0]).astype(np.float64)
    # (The two threads that read the clock sit in different quarters of the SM, whose counters are some cycles apart:
    # the issuing thread's span is held within the CTA's lifetime.)
    span = np.minimum((busy[:, 2] - busy[:, 1]).astype(np.float64), life)
    out = {
        "wait": float(np.mean(busy[:, 3] / life)),
        "fill": float(np.mean(busy[:, 4] / life)),
        "out_wait": float(np.mean(busy[:, 5] / life)),
        "compute": float(np.mean(np.maximum(span - busy[:, 3] - busy[:, 5], 0.0) / life)),
        "outside": float(np.mean(np.maximum(life - span, 0.0) / life)),
        "ctas": int(busy.shape[0]),
    }
    if busy[:, 8].any():  # attention: of the issuing thread's busy time, what it spent waiting for the softmax warps
        out["scopes"] = {"softmax": float(np.mean(busy[:, 8] / life))}
    return out


def measure(lowered, inputs: Sequence[Any], runs: int = 5) -> KernelProfile:
    """Run a built kernel `runs` times (after a warm-up call) between CUDA events, then once more with the
    counters on, and put the two together."""
    import torch

    from .. import ops
    from .._lib import check, library
    from . import api

    name = lowered.plan.nest.name
    dev = [api.to_device(x) for x in inputs]
    lowered.entry(*dev)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(runs):
        lowered.entry(*dev)
    end.record()
    end.synchronize()
    device_s = start.elapsed_time(end) / runs / 1e3

    buffer = torch.zeros(MAX_CTAS * RECORD_WORDS, dtype=torch.int64, device=dev[0].device)
    check(library().tjx_set_profile_buffer(ctypes.c_void_p(buffer.data_ptr()), buffer.numel() * 8))
    try:
        lowered.entry(*dev)
        torch.cuda.synchronize()
    finally:
        check(library().tjx_set_profile_buffer(None, 0))
    ops.device_status()
    found = shares(buffer.cpu().numpy())
    if found is None:
        return KernelProfile(name, lowered.config, runs, device_s, False, float(lowered.steps))
    scopes = {k: v * device_s for k, v in found.get("scopes", {}).items()}
    return KernelProfile(name, lowered.config, runs, device_s, True, float(lowered.steps), found["wait"] * device_s,
                         found["fill"] * device_s, found["out_wait"] * device_s, found["compute"] * device_s, scopes)


def profile(kernel, args: Sequence[Any], runs: int = 5) -> KernelProfile:
    """Where `kernel`'s time goes on the GPU for these inputs (and tunable, if given; else the schedule the kernel
    uses for them) — the reference's `autokernel.profile` (src/autokernel/profiling.py:267-274)."""
    from .errors import KernelError
    from .tune import can_time

    if not can_time():
        raise KernelError("profiling needs an sm_100 GPU: it reads the kernels' own counters")
    arrays, _ = kernel._split(tuple(args))
    config = kernel.lower(*args).config
    lowered = kernel.lowered(kernel.signature(*arrays), config)
    return measure(lowered, arrays, runs)
