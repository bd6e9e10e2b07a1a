"""The autotuner: a hill climb over a kernel's tunable and its buffering, timed and profiled on the device.

The method is the reference's (src/autokernel/tune.py:1-27): start from the tunable's defaults; a candidate must
first compute what the loop nest run as plain code computes; each candidate is timed and its counters say what
limits it; the next candidates follow from that — more ring slots when input copies are exposed, schedules that
move fewer bytes when the kernel is copy-bound, fewer and bigger steps when per-step overhead dominates, every
neighbour otherwise; the climb moves to the first candidate more than 1 % faster and stops when none is, or after
12 candidates. A candidate that fails to build or run counts as infinitely slow.

What is particular to this backend: a candidate is what the C ABI launches, and several schedules launch the same
thing (the matmul kernels walk K in their own blocks of 64, so `tk` changes nothing; the attention kernel visits
the same keys whatever the block sizes; only the matmul's single-CTA ring has a depth to choose). Such candidates
are recognised by their launch key and never timed twice.
"""

from __future__ import annotations

import dataclasses
import math
from collections.abc import Callable, Sequence
from dataclasses import dataclass, field
from typing import Any

from .errors import KernelError
from .profiling import KernelProfile
from .tunable import choices, neighbours

BUDGET = 12            # candidates run per tuning, the defaults included
RUNS = 5               # timed calls per candidate
EXPOSED_SHARE = 0.03   # waits above this share of the device time are worth more buffering
MIN_GAIN = 0.01        # a schedule must be this much faster to replace the best so far
MAX_INPUT_BUFFERS = 4
MAX_OUTPUT_BUFFERS = 3


@dataclass(frozen=True, order=True)
class Pipeline:
    """How deeply a kernel buffers: `input_buffers` ring slots per streamed input tile, `output_buffers` staging
    slots per output tile (the reference's Pipeline, src/autokernel/pipeline.py:42-88, without bursts)."""

    input_buffers: int = 3
    output_buffers: int = 2

    def __post_init__(self) -> None:
        inside = 1 <= self.input_buffers <= MAX_INPUT_BUFFERS and 1 <= self.output_buffers <= MAX_OUTPUT_BUFFERS
        if not inside:
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
        parts = [str(self.pipeline)]
        if self.tunable is not None:
            values = [f"{name}={getattr(self.tunable, name)!r}" for name in choices(self.tunable)]
            parts.insert(0, f"{type(self.tunable).__name__}({', '.join(values)})")
        return ", ".join(parts)


@dataclass
class Trial:
    """One candidate run on the GPU: its profile, or why it was ruled out."""

    config: Any
    profile: KernelProfile | None = None
    error: str | None = None

    @property
    def seconds(self) -> float:
        return math.inf if self.profile is None else self.profile.device_s


@dataclass
class Tuning:
    """What tuning found: the fastest trial and every trial in the order they ran."""

    best: Trial
    trials: list[Trial] = field(default_factory=list)

    @property
    def config(self) -> Any:
        return self.best.config

    def _row(self, trial: Trial) -> str:
        star = "*" if trial is self.best else " "
        if trial.profile is None:
            outcome = f"  {trial.error}"
        else:
            outcome = f"{trial.seconds * 1e6:10.1f} us  {trial.profile.bottleneck}"
        return f" {star} {trial.config!s:72} {outcome}"

    def __str__(self) -> str:
        untimed = "" if self.trials else " (the defaults: tuning needs an sm_100 GPU)"
        return "\n".join([f"chose {self.config}{untimed}", *map(self._row, self.trials)])


def search(start: Any, measure: Callable[[Any], Trial], propose: Callable[[Trial], Sequence[Any]], budget: int) -> Tuning:
    """Climb from `start`. Each round measures what the current leader proposes, in order, skipping what has been
    measured; the first candidate faster than the leader by more than MIN_GAIN becomes the leader and a new round
    begins. The climb ends when a round finds no such candidate, or when `budget` candidates have run. A failed
    trial is infinitely slow, so a failing start yields to the first proposal that runs."""
    ran: dict[Any, Trial] = {}

    def run(config: Any) -> Trial:
        ran[config] = measure(config)
        return ran[config]

    leader = run(start)
    out_of_budget = False
    while not out_of_budget:
        successor = None
        for candidate in propose(leader):
            if candidate in ran:
                continue
            if len(ran) >= budget:
                out_of_budget = True
                break
            trial = run(candidate)
            if trial.seconds < leader.seconds * (1.0 - MIN_GAIN):
                successor = trial
                break
        if successor is None:
            break
        leader = successor
    if not out_of_budget and leader.profile is None:
        raise KernelError("no schedule tried ran: " + "; ".join(f"{t.config}: {t.error}" for t in ran.values()))
    return Tuning(leader, list(ran.values()))


def _traffic(plan, schedule) -> int:
    """Bytes a schedule's copies move between HBM and the SMs, from its tiles and steps (what the reference's
    `_stats` counts, src/autokernel/tune.py:141-155)."""
    p = plan.params
    if plan.family in ("gemm", "rmsnorm_gemm"):
        per_step = (p["tm"] * p["tk"] + p["tk"] * p["tn"]) * 2
        per_tile = p["tm"] * p["tn"] * (4 if str(p["out_dtype"]) == "float32" else 2)
        return schedule.steps * per_step + (schedule.tiles + schedule.fills) * per_tile
    if plan.family == "attention":
        return schedule.tiles * 2 * p["block_q"] * p["D"] * 2 + schedule.steps * 2 * p["block_kv"] * p["D"] * 2
    if plan.family == "attention_block":  # q and the output per tile, a K/V block of every head per step (an upper
        width = p["H"] * p["D"]           # bound once the weights stream: their steps move weights, not K/V)
        return schedule.tiles * 2 * p["block_q"] * width * 2 + schedule.steps * 2 * p["block_kv"] * width * 2
    width = (p["C"] + p["R"]) if p.get("mla") else 2 * p["Hkv"] * p["D"]
    return schedule.steps * p["page"] * width * 2


def proposals(kernel, signature, trial: Trial) -> list[Config]:
    """The schedules to try after `trial`, most promising first, as its profile's bottleneck says. Candidates that
    do not build, or that launch exactly what `trial` launched, are not proposed."""
    from . import api

    config, profile = trial.config, trial.profile
    pipe = config.pipeline
    if profile is None:  # it did not run: shallower buffering first, then the neighbours with the fewest steps
        fallback = [Config(config.tunable, Pipeline(2, 2))] if pipe != Pipeline(2, 2) else []
        try:
            plan, schedule = kernel.build(signature, config.tunable)
        except KernelError:
            plan = schedule = None
    else:
        fallback = []
        plan, schedule = kernel.build(signature, config.tunable)
    here_key = api.launch_key(plan, config) if plan is not None else None
    here_cost = (_traffic(plan, schedule), schedule.steps) if plan is not None else None

    moves: list[Config] = list(fallback)
    if profile is not None and profile.regions and plan is not None:
        exposed = EXPOSED_SHARE * profile.device_s
        deeper = []
        if profile.exposed_wait_s > exposed and pipe.input_buffers < MAX_INPUT_BUFFERS:
            deeper.append(dataclasses.replace(pipe, input_buffers=pipe.input_buffers + 1))
        if profile.out_wait_s > exposed and pipe.output_buffers < MAX_OUTPUT_BUFFERS:
            deeper.append(dataclasses.replace(pipe, output_buffers=pipe.output_buffers + 1))
        for candidate in deeper:
            other = Config(config.tunable, candidate)
            if api.launch_key(plan, other) != here_key:
                moves.append(other)

    near: list[tuple[tuple[int, int], Config]] = []
    for tunable in neighbours(config.tunable) if config.tunable is not None else ():
        try:
            near_plan, near_schedule = kernel.build(signature, tunable)
        except KernelError:
            continue  # breaks a shape rule of the kernel, does not divide a loop, ...
        other = Config(tunable, pipe)
        if here_key is not None and api.launch_key(near_plan, other) == here_key:
            continue  # the same launch: a tile clamped to the array, or a field the kernel does not depend on
        near.append(((_traffic(near_plan, near_schedule), near_schedule.steps), other))
    bottleneck = profile.bottleneck if profile is not None else None
    if bottleneck == "dma" and here_cost is not None:  # fewer bytes; or as many in fewer steps
        near = [n for n in near if n[0] < here_cost]
        near.sort(key=lambda n: n[0])
    elif bottleneck == "overhead" and here_cost is not None:
        near = [n for n in near if n[0][1] < here_cost[1]]
        near.sort(key=lambda n: n[0][1])
    else:
        near.sort(key=lambda n: n[0][1])
    return moves + [c for _, c in near]


def can_time() -> bool:
    """Tuning times candidates on the GPU: is there one?"""
    try:
        import torch

        return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] == 10
    except Exception:
        return False


def measure(kernel, signature, config: Config, inputs, want) -> Trial:
    """Build and run a candidate, check it against the reference's result, then time and profile it."""
    from . import api, profiling

    try:
        lowered = kernel.lowered(signature, config)
        got = lowered.run(*inputs)
        outs = got if isinstance(got, tuple) else (got,)
        wants = want if isinstance(want, tuple) else (want,)
        for name, g, w in zip(kernel.nest.outputs, outs, wants, strict=True):
            api.compare(f"{kernel.nest.name} output {name!r}", api.to_host(g), w, None, None,
                        tuple(dtype for _, dtype in signature))
        return Trial(config, profiling.measure(lowered, inputs, RUNS))
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
