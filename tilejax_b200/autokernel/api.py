"""`@autokernel.kernel`: a Python loop nest over tiles, run by a hand-written sm_100a kernel.

The public surface is the reference's (src/autokernel/api.py:85-284, README "API"): `kernel`, `Kernel.fn` (the
function as written), `.reference` (the same with `@` accumulating in f32), `.lower` / `.lowered` / `.source` /
`.build` / `.signature` / `.default_config`, `.verify` (kernel against reference under the `compare` tolerances) and
`.tuning`. What replaces the generated Pallas source is a launch of one of this backend's kernels through the C
ABI; `Lowered.source` is a readable description of that launch.

Arrays: a kernel call takes CUDA tensors (torch, bf16 / int32) and returns CUDA tensors; host arrays (NumPy with
ml_dtypes.bfloat16, or the jaxlike Array) are copied to the GPU and the result comes back as NumPy. `.fn` and
`.reference` always run on the CPU through `jaxlike`. There is no CPU execution of a *kernel*.
"""

from __future__ import annotations

import functools
from collections.abc import Callable
from dataclasses import dataclass, field
from typing import Any

import numpy as np

from . import collective, jaxlike
from .errors import KernelError
from .parse import Nest, parse
from .plan import Plan, Spec, make_plan
from .tunable import is_tunable, neighbours
from .profiling import KernelProfile
from .tune import Config, Pipeline, Tuning, tune

Signature = tuple[tuple[tuple[int, ...], np.dtype], ...]

COMPARE_CHUNK = 1 << 22  # elements `compare` checks at a time


def _bf16():
    import ml_dtypes

    return np.dtype(ml_dtypes.bfloat16)


def _is_torch(x) -> bool:
    return type(x).__module__.startswith("torch")


def _np_dtype(x) -> np.dtype:
    if _is_torch(x):
        import torch

        return {torch.bfloat16: _bf16(), torch.float32: np.dtype(np.float32), torch.int32: np.dtype(np.int32),
                torch.float16: np.dtype(np.float16), torch.int64: np.dtype(np.int64)}[x.dtype]
    return np.dtype(x.dtype)


def to_host(x) -> np.ndarray:
    """Any array this package handles -> NumPy (bf16 as ml_dtypes.bfloat16)."""
    if _is_torch(x):
        import torch

        t = x.detach().cpu().contiguous()
        return t.view(torch.uint16).numpy().view(_bf16()) if t.dtype == torch.bfloat16 else t.numpy()
    return jaxlike.to_numpy(x)


def to_device(x):
    """Any array this package handles -> a contiguous CUDA tensor on the current device."""
    import torch

    if _is_torch(x):
        return x.cuda().contiguous() if not x.is_cuda else x.contiguous()
    a = np.ascontiguousarray(jaxlike.to_numpy(x))
    if a.dtype == _bf16():
        return torch.from_numpy(a.view(np.uint16)).view(torch.bfloat16).cuda()
    return torch.from_numpy(a).cuda()


def device_inputs(kernel: Kernel, signature: Signature, arrays) -> list:
    """The caller's arrays on the GPU if they are concrete, else seeded random ones of the signature's shapes
    (N(0, 1) floats, zeros for index arrays), as the reference's tuner makes (src/autokernel/tune.py:248-268)."""
    out = []
    for n, ((shape, dtype), x) in enumerate(zip(signature, list(arrays) + [None] * len(signature))):
        if n >= len(kernel.nest.inputs):
            break
        if x is not None and not isinstance(x, Spec):
            out.append(to_device(x))
            continue
        rng = np.random.default_rng(n)
        host = rng.standard_normal(shape, dtype=np.float32).astype(dtype) if np.dtype(dtype).kind not in "iu" \
            else np.zeros(shape, dtype)
        out.append(to_device(host))
    return out


@dataclass(frozen=True)
class Lowered:
    """A kernel built for one input signature and schedule."""

    plan: Plan
    schedule: Any
    config: Config
    source: str
    entry: Callable[..., Any] = field(repr=False)  # entry(*device tensors) -> device tensor(s)

    @property
    def pipeline(self) -> Pipeline:
        return self.config.pipeline

    @property
    def steps(self) -> int:
        return self.schedule.steps

    @property
    def tiles(self) -> int:
        return self.schedule.tiles

    @property
    def total_tiles(self) -> int:
        return self.schedule.total_tiles

    def run(self, *inputs):
        host = not all(_is_torch(x) and x.is_cuda for x in inputs)
        out = self.entry(*[to_device(x) for x in inputs])
        if not host:
            return out
        return tuple(to_host(o) for o in out) if isinstance(out, tuple) else to_host(out)

    def profile(self, *inputs, runs: int = 5) -> KernelProfile:
        """Seconds per call from CUDA events around `runs` launches, and where they go from the kernel's counters."""
        from . import profiling

        return profiling.measure(self, inputs, runs)


class Kernel:
    """A loop nest run by an sm_100a kernel. Call it like the function it was made from: with its tunable
    (`matmul(x, y, MatmulTiles(tm=256))`) it uses it; without, it is tuned for the inputs' shapes when first called
    with them, and remembers the result."""

    def __init__(self, fn: Callable[..., Any]) -> None:
        functools.update_wrapper(self, fn)
        self.fn = fn
        self.nest: Nest = parse(fn)
        self.default_tunable = None
        if self.nest.tunable is not None:
            self.default_tunable = (fn.__defaults__ or (None,))[-1]
            if not is_tunable(self.default_tunable):
                raise self.nest.error(
                    f"`{self.nest.tunable}`'s default must be an @autokernel.tunable, not {self.default_tunable!r}",
                    self.nest.function.args)
        # What has been planned, bound to a launch and tuned so far, each keyed by the inputs' signature.
        self._builds: dict = {}
        self._lowered: dict = {}
        self._tunings: dict = {}

    def __repr__(self) -> str:
        return f"<autokernel.Kernel {self.nest.name}>"

    def __call__(self, *args: Any) -> Any:
        return self.lower(*args).run(*self._split(args)[0])

    def lower(self, *args: Any) -> Lowered:
        """The kernel for inputs like these (arrays or `Spec`s), and the tunable if given."""
        arrays, tunable = self._split(args)
        signature = self.signature(*arrays)
        if tunable is not None:
            self.build(signature, tunable)  # a KernelError here names the user's line
            config = Config(tunable, Pipeline())
        else:
            config = self.tuning(*arrays).config
        return self.lowered(signature, config)

    def source(self, *args: Any) -> str:
        return self.lower(*args).source

    def reference(self, *args: Any) -> Any:
        """What the kernel computes: the loop nest run as written on the CPU, with `@` accumulating in f32."""
        arrays, tunable = self._split(args)
        call = [jaxlike.Array(to_host(x)) for x in arrays]
        if self.nest.tunable is not None:
            call.append(tunable if tunable is not None else self.lower(*arrays).config.tunable)
        with jaxlike.mxu_semantics():
            result = self.fn(*call)
        return tuple(map(to_host, result)) if isinstance(result, tuple) else to_host(result)

    def verify(self, *args: Any, rtol: float | None = None, atol: float | None = None) -> float:
        """Run the kernel and its reference; AssertionError unless they agree within the tolerances for the dtypes
        (or `rtol` / `atol`). Returns the largest absolute difference."""
        arrays, tunable = self._split(args)
        call = tuple(arrays)
        if self.nest.tunable is not None:
            call += (tunable if tunable is not None else self.lower(*arrays).config.tunable,)
        got, want = self(*call), self.reference(*call)
        if not isinstance(got, tuple):
            got, want = (got,), (want,)
        dtypes = tuple(dtype for _, dtype in self.signature(*arrays)[: len(self.nest.inputs)])
        worst = 0.0
        for name, g, w in zip(self.nest.outputs, got, want, strict=True):
            worst = max(worst, compare(f"{self.nest.name} output {name!r}", to_host(g), w, rtol, atol, dtypes))
        return worst

    def tuning(self, *arrays: Any) -> Tuning:
        """The schedule for inputs like these: tuned on the GPU when first asked, the defaults elsewhere."""
        signature = self.signature(*arrays)
        found = self._tunings.get(signature)
        if found is None:
            found = self._tunings[signature] = tune(self, signature, arrays)
        return found

    # ------------------------------------------------------------------ building (used by tune.py too)

    def signature(self, *arrays: Any) -> Signature:
        """What the kernel is built for: each input's (shape, dtype), then each gathered array's (its input's rows
        times the ranks it is gathered over)."""
        names = self.nest.inputs
        if len(arrays) != len(names):
            raise KernelError(f"{self.nest.name} takes {len(names)} input arrays ({', '.join(names)}); got {len(arrays)}")
        entries: list[tuple[tuple[int, ...], np.dtype]] = []
        for name, x in zip(names, arrays):
            shape = tuple(int(d) for d in getattr(x, "shape", ()))
            if not shape or not hasattr(x, "dtype"):
                raise KernelError(f"{self.nest.name}: input `{name}` must be an array, got {type(x).__name__}")
            entries.append((shape, _np_dtype(x)))
        for gather in self.nest.all_gathers:
            shape, dtype = entries[names.index(gather.source)]
            entries.append(((shape[0] * collective.axis_size(gather.axis), *shape[1:]), dtype))
        return tuple(entries)

    def default_config(self, signature: Signature) -> Config:
        """The schedule to start from: the tunable's defaults or, if they do not build for these inputs, the
        tunable the fewest single-field steps away that does (ties in the order `neighbours` lists them)."""
        first_error = None
        for tunable in _outwards(self.default_tunable):
            try:
                self.build(signature, tunable)
            except KernelError as e:
                first_error = first_error or e
                continue
            return Config(tunable, Pipeline())
        raise first_error

    def build(self, signature: Signature, tunable: Any, cursor: bool = False):
        """(plan, schedule) for this signature and tunable; KernelError if the nest is not a recognised schedule or
        the shapes break a rule of the kernel that would run it."""
        key = (signature, tunable)
        if key not in self._builds:
            n = len(self.nest.inputs)
            specs = [Spec(shape, dtype) for shape, dtype in signature[:n]]
            chips = collective.axis_size() if self.nest.all_gathers else 1
            plan = make_plan(self.nest, self.fn, specs, tunable, chips)
            _check_kernel_rules(plan)
            self._builds[key] = (plan, plan.params["schedule"])
        return self._builds[key]

    def schedule_of(self, *arrays: Any, tunable: Any = None):
        """The schedule (tiles, steps, tables) of this loop nest for inputs like these, whether or not a kernel here
        can run it: what `make_schedule` makes of its loops and masks (src/autokernel/schedule.py:147-220)."""
        from . import plan as _plan

        signature = self.signature(*arrays)
        specs = [Spec(shape, dtype) for shape, dtype in signature[: len(self.nest.inputs)]]
        tunable = tunable if tunable is not None else self.default_tunable
        return _plan.schedule_only(self.nest, self.fn, specs, tunable)

    def lowered(self, signature: Signature, config: Config, trace: bool = False) -> Lowered:
        key = (signature, config)
        if key not in self._lowered:
            plan, schedule = self.build(signature, config.tunable)
            source, entry = _lower(plan, config)
            self._lowered[key] = Lowered(plan, schedule, config, source, entry)
        return self._lowered[key]

    def _split(self, args: tuple[Any, ...]) -> tuple[tuple[Any, ...], Any]:
        """(the input arrays, the tunable or None) of a call's arguments."""
        inputs, name = self.nest.inputs, self.nest.tunable
        with_tunable = name is not None and len(args) == len(inputs) + 1
        if len(args) != len(inputs) and not with_tunable:
            optional = f", then optionally `{name}`" if name is not None else ""
            raise KernelError(
                f"{self.nest.name} takes {len(inputs)} input arrays ({', '.join(inputs)}){optional}; got {len(args)}")
        if not with_tunable:
            return tuple(args), None
        *arrays, tunable = args
        wanted = type(self.default_tunable)
        if type(tunable) is not wanted:
            raise KernelError(
                f"{self.nest.name}: `{name}` must be a {wanted.__name__}, not {type(tunable).__name__}")
        return tuple(arrays), tunable


def _outwards(tunable: Any):
    """`tunable`, then every tunable reachable from it by single-field steps, nearest first (None yields itself)."""
    yield tunable
    if tunable is None:
        return
    reached = {tunable}
    ring = [tunable]
    while ring:
        next_ring = []
        for centre in ring:
            for other in neighbours(centre):
                if other not in reached:
                    reached.add(other)
                    next_ring.append(other)
                    yield other
        ring = next_ring


def kernel(fn: Callable[..., Any]) -> Kernel:
    """Run a Python loop nest over tiles with a hand-written sm_100a kernel. Raises KernelError, naming the line, for
    code that is not one of the schedules this backend has a kernel for."""
    return Kernel(fn)


# ------------------------------------------------------------------------------------------ lowering


def _check_kernel_rules(plan: Plan) -> None:
    """The shape rules of the CUDA kernels, reported as KernelErrors before anything runs (the reference reports
    its TPU layout rules the same way, tests/test_plan.py:150-170)."""
    p, nest = plan.params, plan.nest
    bf16 = _bf16()
    if plan.family in ("gemm", "rmsnorm_gemm"):
        if any(np.dtype(s.dtype) != bf16 for s in plan.specs[: 2 if plan.family == "gemm" else 3]):
            raise nest.error("the matmul kernel takes bfloat16 operands")
        if np.dtype(p["out_dtype"]) not in (bf16, np.dtype(np.float32)):
            raise nest.error("the matmul kernel writes bfloat16 or float32")
        if p["K"] % 8 or p["N"] % 8:
            raise nest.error("K and N must be multiples of 8: rows of 16 bytes for the TMA descriptors")
        if not (p["tm"] % 128 == 0 or p["tm"] == p["M"]) or not (p["tn"] % 128 == 0 or p["tn"] == p["N"]):
            raise nest.error(f"tiles of {p['tm']} x {p['tn']}: output tiles must be multiples of 128 (the tensor core's "
                             "tile) or span the matrix")
    elif plan.family == "attention_block":
        if p["D"] != 128 or p["S"] % 128 or p["block_q"] % 128 or p["block_kv"] % 128 or p["F"] % 128:
            raise nest.error("the attention block's kernels take head_dim 128, blocks that are multiples of 128 and a "
                             "hidden width that is a multiple of 128")
        if any(np.dtype(s.dtype) != bf16 for s in plan.specs[:6]):
            raise nest.error("the attention block's kernels take bfloat16 inputs")
    elif plan.family == "attention":
        if p["D"] != 128 or p["S"] % 128 or p["block_q"] % 128 or p["block_kv"] % 128:
            raise nest.error("the attention kernel takes head_dim 128 and blocks that are multiples of 128")
        if any(np.dtype(s.dtype) != bf16 for s in plan.specs[:3]):
            raise nest.error("the attention kernel takes bfloat16 q, k, v")
    elif plan.family == "rpa_prefill":
        if p["D"] != 128 or p["page"] != 128 or p["H"] % p["Hkv"] or (p["H"] // p["Hkv"]) % 2 \
                or any(np.dtype(s.dtype) != bf16 for s in plan.specs[:2]):
            raise nest.error("the paged prefill kernel takes bfloat16 q and cache, head_dim 128, pages of 128 positions and "
                             "an even number of query heads per KV head")
    elif plan.family == "rpa_write":
        if p["D"] != 128 or any(np.dtype(s.dtype) != bf16 for s in plan.specs[:3]):
            raise nest.error("the cache write kernel takes a bfloat16 cache, keys and values of head_dim 128")
    elif p.get("mla"):
        if p["C"] != 512 or p["R"] != 128 or p["H"] % 16 or p["page"] % 16:
            raise nest.error("the MLA decode kernel takes 512 latent and 128 RoPE columns, heads in multiples of 16 and "
                             "blocks of a multiple of 16 positions")
    else:
        if p["D"] != 128 or p["page"] % 16 or p["H"] % p["Hkv"] or p["H"] // p["Hkv"] not in (1, 2, 4, 8):
            raise nest.error("the decode kernel takes head_dim 128, pages of a multiple of 16 positions and 1, 2, 4 "
                             "or 8 query heads per KV head")
        if p["T"] * (p["H"] // p["Hkv"]) > 16:
            raise nest.error(f"{p['T']} new tokens x {p['H'] // p['Hkv']} query heads per KV head: the decode kernel "
                             "holds at most 16 query rows per KV head (the rows of one warp-level MMA)")


def _stages(pipeline: Pipeline, tn: int) -> int:
    """The GEMM's `stages` argument for a Pipeline. The default depth (3 input buffers) leaves the choice to the
    library (0): one MMA per pair of SMs with its own ring when the tiles are multiples of 256, else 4 slots.
    Shallower or deeper pipelines ask for the single-CTA ring explicitly: 3 or 4 slots for 256-wide CTA tiles, 4 or
    6 for 128-wide."""
    wide = tn % 256 == 0
    if pipeline.input_buffers <= 2:
        return 3 if wide else 4
    if pipeline.input_buffers == 3:
        return 0
    return 4 if wide else 6


def launch_key(plan: Plan, config: Config) -> tuple:
    """What a schedule makes the C ABI launch, as a hashable key: schedules with equal keys run the same kernel on the
    same tiles and differ in nothing that can be timed. The matmul kernels walk K in their own blocks of 64 (`tk` is
    not part of the key) and only their single-CTA ring has a depth (`output_buffers` never is); the attention
    kernel works in 128 x 128 blocks cut at each tile's diagonal whatever the user's blocks; paged decode reads the
    pages as they are; contiguous decode walks blocks of the chosen size; the MLA decode kernel shares the cache out in
    its own units of 32 positions, whatever the block (which only shapes the caller's step tables)."""
    p = plan.params
    if plan.family == "gemm":
        return ("gemm", p["tm"], p["tn"], _stages(config.pipeline, p["tn"]), p["causal"], p["transposed"])
    if plan.family == "rmsnorm_gemm":
        return ("rmsnorm_gemm", p["tm"], p["tn"])
    if plan.family == "attention":
        return ("attention",)
    if plan.family == "attention_block":
        return ("attention_block",)
    if plan.family == "rpa_write":
        return ("rpa_write",)
    if plan.family == "rpa_prefill":
        return ("rpa_prefill",)
    if p.get("mla"):
        return ("mla_decode",)
    if p.get("rpa"):
        return ("rpa_decode",)
    if p.get("contiguous"):
        return ("decode", p["page"])
    return ("decode",)


def _lower(plan: Plan, config: Config) -> tuple[str, Callable[..., Any]]:
    from .. import ops

    p, name = plan.params, plan.nest.name
    sch = p["schedule"]
    header = f"# {name}: {str(config).rsplit(', ', 1)[0] if config.tunable is not None else ''}; {config.pipeline}\n"
    if plan.family == "gemm":
        import torch

        stages = _stages(config.pipeline, p["tn"])
        out_dtype = torch.float32 if np.dtype(p["out_dtype"]) == np.float32 else torch.bfloat16
        names = list(plan.nest.inputs)
        ia, ib = (names.index(p["a"]) if p["a"] in names else None), names.index(p["b"])
        vi, vj = p["loop_vars"]
        bn = 256 if p["tn"] % 256 == 0 else 128
        text = header + (
            f"kernel      tjx_gemm_bf16 (persistent TMA + tcgen05, f32 accumulators in TMEM)\n"
            f"problem     out[{p['M']}, {p['N']}] = {p['a']}[{p['M']}, {p['K']}] @ {p['b']}"
            f"{'.T' if p['transposed'] else ''}, {'causal (tril), ' if p['causal'] else ''}output {np.dtype(p['out_dtype']).name}\n"
            f"user tile   {p['tm']} x {p['tn']} x {p['tk']}: {sch.tiles} of {sch.total_tiles} tiles run, {sch.steps} steps, "
            f"{sch.fills} filled with zeros\n"
            + (f"CTA pair    256 x 256 x 64 pieces, one MMA per pair of SMs (cta_group::2), ring of 3 slots x 2 K blocks, "
               f"2 TMEM accumulators per SM, TMA-store epilogue\n"
               if stages == 0 and p["tm"] % 256 == 0 and p["tn"] % 256 == 0 else
               f"CTA tile    128 x {bn} x 64, ring of {stages or 4} slots, 2 TMEM accumulators, TMA-store epilogue\n") +
            f"tables      {', '.join(f'{k}[{len(v)}]' for k, v in sch.tables.items()) or 'none (arithmetic tile order)'}\n")
        if p["gathered"]:
            from ..collective import AllGatherMatmul

            text += f"gather      {p['gathered']} = all_gather({plan.nest.all_gathers[0].source}) over {p['chips']} rank(s): " \
                    f"peer shards pulled over NVLink while the own shard's tiles run (collective.AllGatherMatmul), own shard first\n"
            op_holder: dict = {}

            def entry(*inputs):
                x, w = inputs[names.index(plan.nest.all_gathers[0].source)], inputs[ib]
                if "op" not in op_holder:
                    op_holder["op"] = AllGatherMatmul(x.shape[0], p["K"], p["N"], p["tm"], p["tn"], p["tk"])
                return op_holder["op"](x, w)

            return text, entry

        def entry(*inputs):
            tables = {}
            for key, values in sch.tables.items():
                short = key.replace(f"_{vi}", "_i").replace(f"_{vj}", "_j")
                tables[short] = ops.device_table((name, p["M"], p["N"], p["tm"], p["tn"], key), values, inputs[0].device)
            return ops.gemm(inputs[ia], inputs[ib], p["tm"], p["tn"], p["tk"], causal=p["causal"], out_dtype=out_dtype,
                            y_transposed=p["transposed"], stages=stages, **tables)

        return text, entry
    if plan.family == "rmsnorm_gemm":
        import torch

        out_dtype = torch.float32 if np.dtype(p["out_dtype"]) == np.float32 else torch.bfloat16
        text = header + (
            f"kernel      tjx_rmsnorm_gemm_bf16 (one pass over x for the gamma-scaled operand and the row scales, then the "
            f"persistent TMA + tcgen05 matmul with the row scale in its epilogue)\n"
            f"problem     out[{p['M']}, {p['N']}] = rsqrt(mean(x^2) + {p['eps']:g}) * ((x * gamma)[{p['M']}, {p['K']}] @ w), "
            f"output {np.dtype(p['out_dtype']).name}\n"
            f"user tile   {p['tm']} x {p['tn']} x {p['tk']}: {sch.tiles} tiles, {sch.steps} steps\n")
        return text, lambda x, gamma, w: ops.rmsnorm_matmul(x, gamma, w, p["tm"], p["tn"], p["tk"], p["eps"], out_dtype)
    if plan.family == "attention":
        text = header + (
            f"kernel      tjx_causal_attention_bf16 (TMA rings, tcgen05 with S, P and O in TMEM, online softmax)\n"
            f"problem     q, k, v, out [{p['B']}, {p['H']}, {p['S']}, {p['D']}] bfloat16, causal\n"
            f"user blocks {p['block_q']} x {p['block_kv']}: {sch.tiles} tiles, {sch.steps} steps "
            f"({sch.pattern_steps} per (b, h), repeated {sch.repeats} times)\n"
            f"CTA         two 128-row query tiles sharing each 128-key K/V block; future blocks skipped\n"
            f"tables      {', '.join(f'{k}[{len(v)}]' for k, v in sch.tables.items()) or 'none'}\n")
        return text, lambda q, k, v: ops.causal_attention(q, k, v, p["block_q"], p["block_kv"])
    if plan.family == "attention_block":
        D = p["H"] * p["D"]
        text = header + (
            f"kernel      tjx_attention_block_bf16 (four launches on one stream: tcgen05 attention writing the heads side "
            f"by side in f32, a row-wise RMSNorm, the matmul step loop with tanh GELU in its epilogue, the matmul step loop)\n"
            f"problem     q, k, v [{p['B']}, {p['H']}, {p['S']}, {p['D']}], gamma [1, {D}], w_up [{D}, {p['F']}], "
            f"w_down [{p['F']}, {D}] bfloat16 -> out [{p['B']}, {p['S']}, {D}]\n"
            f"user blocks {p['block_q']} x {p['block_kv']}, {p['block_f']} hidden units: {sch.tiles} tiles, {sch.steps} steps, "
            f"phases {', '.join(p['phases']) or 'none'}\n"
            f"on chip     the reference keeps a tile's attention output and hidden activations in VMEM; here they pass "
            f"through a workspace that stays in L2 at these sizes\n")
        return text, lambda q, k, v, gamma, w_up, w_down: ops.attention_block(
            q, k, v, gamma, w_up, w_down, p["block_q"], p["block_kv"], p["block_f"], p["eps"])
    if p.get("mla"):
        text = header + (
            f"kernel      tjx_mla_decode_bf16 (tcgen05: 64 (token, head) rows per CTA, scores and output in TMEM, the "
            f"cache shared out in units of 32 positions over persistent CTAs; partials merged by a second kernel; the "
            f"device step tables are built beside it)\n"
            f"problem     {p['B']} sequences, {p['T']} new token(s), {p['H']} heads, {p['C']} latent + {p['R']} RoPE columns, blocks of "
            f"{p['page']} of {p['S']} cache positions\n"
            f"steps       at most {sch.steps}: step_tile / step_code / step_count are built on the device from lengths "
            f"before the kernel\n")
        return text, lambda q_c, q_r, c_kv, k_rope, lengths: ops.mla_decode(q_c, q_r, c_kv, k_rope, lengths, p["page"])
    if plan.family == "rpa_write":
        text = header + (
            f"kernel      tjx_rpa_write_runs_bf16 (a CTA per (row of a page, run): the run's tokens' keys and values copied "
            f"side by side into their page, 16 bytes per thread)\n"
            f"problem     {p['T']} new tokens, {p['Hkv']} KV heads of {p['D']}, pages of {p['page']}, pool of "
            f"{p['num_pages']}, at most {p['max_runs']} runs: how many there are is read from n_writes on the device\n"
            f"in place    the reference donates the cache and updates it; this entry copies it first (ops.rpa_write_runs "
            f"and the C entry point write in place)\n")

        def write(cache, keys, values, page_indices, write_page, write_rows, write_first, write_stop, n_writes):
            return ops.rpa_write_runs(cache.clone(), keys, values, page_indices, write_page, write_rows, write_first,
                                      write_stop, n_writes)

        return text, write
    if plan.family == "rpa_prefill":
        text = header + (
            f"kernel      tjx_rpa_prefill_tiles_bf16 (the causal attention kernel's paged instantiation: a small kernel cuts "
            f"the tiles into 128 queries; a unit = (tile, KV head, two of its query heads), a block = one page through "
            f"page_indices by 3-D TMA; outputs replace the queries' rows)\n"
            f"problem     {p['T']} token rows, {p['H']} / {p['Hkv']} heads, head_dim {p['D']}, pages of {p['page']}, pool of "
            f"{p['num_pages']}, at most {p['max_tiles']} tiles of up to 256 queries, softmax scale {p['sm_scale']:.6g}\n"
            f"steps       how many tiles there are and how many pages each walks is read from n_tiles and tile_pos / "
            f"tile_rows on the device; a tunable's pages per step only shapes the reference's own steps\n"
            f"in place    the reference donates q and updates it; this entry returns a new array holding q's other rows\n")

        def prefill(q, cache, page_indices, tile_page, tile_rows, tile_pos, tile_stop, n_tiles):
            return ops.rpa_prefill_tiles(q, cache, page_indices, tile_page, tile_rows, tile_pos, n_tiles, p["sm_scale"])

        return text, prefill
    if p.get("rpa"):
        text = header + (
            f"kernel      tjx_rpa_decode_bf16 (the paged decode kernel on the cache's own layout: two tensor maps over the "
            f"one buffer, keys and values of a head side by side; lengths of the sequences outside [0, distribution[0]) "
            f"set to zero on the device; only the decode tokens' rows are written)\n"
            f"problem     {p['tokens']} token rows, {p['sequences']} sequences (sequence s is token s), {p['H']} / {p['Hkv']} "
            f"heads, head_dim {p['D']}, pages of {p['page']}, {p['pages']} pages per sequence, pool of {p['num_pages']}, "
            f"softmax scale {p['sm_scale']:.6g}\n"
            f"steps       at most {sch.steps}: how many pages a sequence walks is read from kv_lens on the device "
            f"(the reference's `for p in range(cdiv(kv_lens[s], page_size))`)\n"
            f"in place    the reference donates q and updates it; this entry returns a new array holding q's other rows\n")
        return text, lambda q, cache, kv_lens, page_indices, distribution: ops.rpa_decode(
            q, cache, kv_lens, page_indices, distribution, p["sm_scale"])
    text = header + (
        f"kernel      tjx_paged_gqa_decode_bf16 (device step tables, per-warp TMA rings, warp-level MMA, partials "
        f"merged by the last warp to arrive)\n"
        f"problem     {p['B']} sequences, {p['T']} new token(s), {p['H']} / {p['Hkv']} heads, head_dim {p['D']}, pages of {p['page']}, "
        f"{p['pages']} pages per sequence, pool of {p['num_pages']}"
        f"{' (a contiguous cache: the identity block table)' if p.get('contiguous') else ''}\n"
        f"steps       at most {sch.steps}: step_tile / step_code / step_count are built on the device from lengths "
        f"before the kernel\n")
    if p.get("contiguous"):
        return text, lambda q, kc, vc, lengths: ops.gqa_decode(q, kc, vc, lengths, p["page"])
    return text, lambda q, kp, vp, bt, lengths: ops.paged_gqa_decode(q, kp, vp, bt, lengths)


# ------------------------------------------------------------------------------------------ comparing


def compare(what: str, got: Any, want: Any, rtol: float | None = None, atol: float | None = None,
            inputs: tuple[Any, ...] = ()) -> float:
    """The largest absolute difference between `got` and `want`; AssertionError beyond `rtol` and `atol`. Defaults:
    exact for integers; 1e-4 for f32; for 16-bit results, and f32 results computed from 16-bit `inputs`, 2e-2
    relative and 2e-2 of the largest finite |want| absolute. NaN equals NaN. The arrays are walked in pieces of
    COMPARE_CHUNK elements so that float64 copies of a multi-GB output never exist at once. The reference's rule
    (src/autokernel/api.py:320-364), message included."""
    got, want = to_host(got), to_host(want)

    def is_float(d) -> bool:
        d = np.dtype(d)
        return d.kind == "f" or d == _bf16()

    if not is_float(want.dtype):
        loose, default = False, 0.0
    else:
        loose = np.dtype(want.dtype).itemsize <= 2 or any(is_float(d) and np.dtype(d).itemsize <= 2 for d in inputs)
        default = 2e-2 if loose else 1e-4
    rtol = default if rtol is None else rtol
    flat_got, flat_want = got.reshape(-1), want.reshape(-1)

    def pieces():
        for lo in range(0, flat_want.size, COMPARE_CHUNK):
            yield (flat_got[lo : lo + COMPARE_CHUNK].astype(np.float64), flat_want[lo : lo + COMPARE_CHUNK].astype(np.float64))

    if atol is None:
        largest = 1.0
        if loose:  # 16-bit results round at every step: the error grows with the output's magnitude
            for _, w in pieces():
                finite = np.abs(w[np.isfinite(w)])
                if finite.size:
                    largest = max(largest, float(finite.max()))
        atol = default * largest
    worst, mismatched = 0.0, 0
    for g, w in pieces():
        both_nan = np.isnan(g) & np.isnan(w)
        equal = (g == w) | both_nan
        with np.errstate(invalid="ignore"):
            gap = np.abs(g - w)
            within = equal | (np.isfinite(w) & (gap <= atol + rtol * np.abs(w)))
        gap[equal] = 0.0
        if gap.size:
            worst = max(worst, float(np.nanmax(gap)) if not np.all(np.isnan(gap)) else 0.0)
        mismatched += int(np.count_nonzero(~within))
    if mismatched:
        raise AssertionError(
            f"{what}: the kernel and its reference differ in {mismatched} of {flat_want.size} elements "
            f"(largest difference {worst:.3g}; rtol={rtol}, atol={atol:.3g})")
    return worst
