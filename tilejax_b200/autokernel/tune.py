"""The autotuner: a hill climb over a kernel's tunable and its buffering, timed on the device.

Same shape as the reference's (src/autokernel/tune.py:108-131, :167-206): start from the defaults; every candidate
must first agree with the reference; move to the first proposal that is more than 1% faster; at most 12 trials; a
candidate that fails to build or run counts as infinitely slow. What differs is what a candidate maps to and how it
is timed: a tunable's tile sizes choose the user tile the persistent kernels walk, `Pipeline.input_buffers` chooses
the depth of the TMA ring (3 or 4 slots of 128x64 + 64xBN; 6 for 128-wide CTA tiles), and time comes from CUDA
events around repeated launches instead of TPU trace regions.
"""

from __future__ import annotations

import dataclasses
import math
from collections.abc import Callable, Sequence
from dataclasses import dataclass, field
from typing import Any

from .errors import KernelError
from .tunable import choices, neighbours

BUDGET = 12       # candidates run per tuning, the defaults included
RUNS = 5          # timed calls per candidate
MIN_GAIN = 0.01   # a schedule must be this much faster to replace the best so far
MAX_INPUT_BUFFERS = 4
MAX_OUTPUT_BUFFERS = 3


@dataclass(frozen=True, order=True)
class Pipeline:
    """How deeply a kernel buffers: `input_buffers` ring slots per streamed input tile, `output_buffers` staging
    slots per output tile (the reference's Pipeline, src/autokernel/pipeline.py:42-88, without bursts)."""

    input_buffers: int = 3
    output_buffers: int = 2

    def __post_init__(self) -> None:
        if not (1 <= self.input_buffers <= MAX_INPUT_BUFFERS and 1 <= self.output_buffers <= MAX_OUTPUT_BUFFERS):
            raise KernelError(
                f"a pipeline has 1 to {MAX_INPUT_BUFFERS} input buffers and 1 to {MAX_OUTPUT_BUFFERS} output "
                f"buffers, not {self.input_buffers} and {self.output_buffers}"
            )

    def __str__(self) -> str:
        return f"{self.input_buffers} input / {self.output_buffers} output buffers"


@dataclass(frozen=True)
class Config:
    """A schedule: the kernel's tunable (None if it has none) and its buffering."""

    tunable: Any
    pipeline: Pipeline = Pipeline()
    cursor: bool = False  # kept for the reference's signature; this backend always builds step tables

    def __str__(self) -> str:
        if self.tunable is None:
            return str(self.pipeline)
        fields = ", ".join(f"{k}={getattr(self.tunable, k)!r}" for k in choices(self.tunable))
        return f"{type(self.tunable).__name__}({fields}), {self.pipeline}"


@dataclass(frozen=True)
class KernelProfile:
    """What timing a candidate found: seconds per call on the device and what bounds it."""

    device_s: float
    tensor_fraction: float   # achieved / peak on the tensor pipe (0 for kernels that use none)
    hbm_fraction: float      # achieved / peak HBM bandwidth for the bytes the math needs
    steps: int

    @property
    def bottleneck(self) -> str:
        """`dma` if memory-bound, `overhead` if neither pipe is busy (tiles too small), else `compute`."""
        if max(self.tensor_fraction, self.hbm_fraction) < 0.15:
            return "overhead"
        return "dma" if self.hbm_fraction > self.tensor_fraction else "compute"

    def __str__(self) -> str:
        return (f"{self.device_s * 1e6:.1f} us per call, {self.steps} steps; tensor pipe {self.tensor_fraction:.0%}, "
                f"HBM {self.hbm_fraction:.0%}: {self.bottleneck}")


@dataclass
class Trial:
    config: Config
    profile: KernelProfile | None = None
    error: str | None = None

    @property
    def seconds(self) -> float:
        return self.profile.device_s if self.profile else math.inf


@dataclass
class Tuning:
    best: Trial
    trials: list[Trial] = field(default_factory=list)

    @property
    def config(self) -> Config:
        return self.best.config

    def __str__(self) -> str:
        lines = [f"chose {self.config}" + ("" if self.trials else " (the defaults: tuning needs an sm_100 GPU)")]
        for t in self.trials:
            mark = "*" if t is self.best else " "
            result = f"{t.seconds * 1e6:10.1f} us  {t.profile.bottleneck}" if t.profile else f"  {t.error}"
            lines.append(f" {mark} {t.config!s:72} {result}")
        return "\n".join(lines)


def search(start: Any, measure: Callable[[Any], Trial], propose: Callable[[Trial], Sequence[Any]], budget: int) -> Tuning:
    """Climb from `start`: measure what the best trial proposes, in order, moving to the first proposal that is
    faster; stop when none is, or after `budget` trials."""
    best = measure(start)
    trials = {start: best}
    improved = True
    while improved:
        improved = False
        for config in propose(best):
            if config in trials:
                continue
            if len(trials) >= budget:
                return Tuning(best, list(trials.values()))
            trial = trials[config] = measure(config)
            if trial.seconds < best.seconds * (1 - MIN_GAIN):
                best, improved = trial, True
                break
    if best.profile is None:
        errors = "; ".join(f"{t.config}: {t.error}" for t in trials.values())
        raise KernelError(f"no schedule tried ran: {errors}")
    return Tuning(best, list(trials.values()))


def proposals(kernel, signature, trial: Trial) -> list[Config]:
    """The schedules to try after `trial`: more ring slots when memory-bound, then the neighbouring tunables —
    fewer steps first when overhead-bound, else in order — skipping neighbours that build the same kernel (the
    code clamps a tile to the array) or do not build."""
    config, profile = trial.config, trial.profile
    moves: list[Config] = []
    pipe = config.pipeline
    if profile is None:
        if pipe != Pipeline(2, 2):
            moves.append(Config(config.tunable, Pipeline(2, 2)))
    elif profile.bottleneck == "dma" and pipe.input_buffers < MAX_INPUT_BUFFERS:
        moves.append(Config(config.tunable, dataclasses.replace(pipe, input_buffers=pipe.input_buffers + 1)))
    try:
        here = kernel.build(signature, config.tunable)
        loops = tuple((r.var, r.step, r.count) for r in here[0].loops)
    except KernelError:
        loops = None
    near = []
    for tunable in neighbours(config.tunable) if config.tunable is not None else ():
        try:
            plan, schedule = kernel.build(signature, tunable)
        except KernelError:
            continue
        if tuple((r.var, r.step, r.count) for r in plan.loops) == loops:
            continue
        near.append((schedule.steps, Config(tunable, pipe)))
    if profile is not None and profile.bottleneck == "overhead":
        near = [n for n in near if loops is None or n[0] < here[1].steps]
    near.sort(key=lambda n: n[0])
    return moves + [c for _, c in near]


def can_time() -> bool:
    """Tuning times candidates on the GPU: is there one?"""
    try:
        import torch

        return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] == 10
    except Exception:
        return False


def measure(kernel, signature, config: Config, inputs, want) -> Trial:
    """Build and run a candidate, check it against the reference's result, then time it."""
    from . import api

    try:
        lowered = kernel.lowered(signature, config)
        got = lowered.run(*inputs)
        outs = got if isinstance(got, tuple) else (got,)
        wants = want if isinstance(want, tuple) else (want,)
        for name, g, w in zip(kernel.nest.outputs, outs, wants, strict=True):
            api.compare(f"{kernel.nest.name} output {name!r}", api.to_host(g), w, None, None,
                        tuple(dtype for _, dtype in signature))
        return Trial(config, lowered.profile(*inputs, runs=RUNS))
    except Exception as e:  # a candidate that fails is infinitely slow
        return Trial(config, error=f"{type(e).__name__}: {str(e).splitlines()[0][:120]}")


def tune(kernel, signature, arrays) -> Tuning:
    """Tune `kernel` for this signature on the GPU; without one (or for kernels that gather across GPUs, whose
    timing needs every rank) return the defaults untimed, as the reference does off a TPU (tune.py:345-348)."""
    start = kernel.default_config(signature)
    if not can_time() or kernel.nest.all_gathers:
        return Tuning(Trial(start))
    from . import api

    inputs = api.device_inputs(kernel, signature, arrays)
    reference_tunable = start.tunable
    want = kernel.reference(*[api.to_host(x) for x in inputs], *((reference_tunable,) if kernel.nest.tunable else ()))
    want = tuple(api.to_host(w) for w in want) if isinstance(want, tuple) else api.to_host(want)
    return search(start, lambda c: measure(kernel, signature, c, inputs, want),
                  lambda t: proposals(kernel, signature, t), BUDGET)
