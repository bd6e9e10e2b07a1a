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
from .tune import Config, KernelProfile, Pipeline, Tuning, tune

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
        """Seconds per call from CUDA events around `runs` launches, and the roofline fractions they imply."""
        import torch

        from ..ops import device_status

        dev = [to_device(x) for x in inputs]
        self.entry(*dev)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(runs):
            self.entry(*dev)
        end.record()
        end.synchronize()
        device_status()
        seconds = start.elapsed_time(end) / runs / 1e3
        flops, nbytes = _work(self.plan, dev)
        return KernelProfile(seconds, flops / seconds / 1.65e15, nbytes / seconds / 6.5e12, self.steps)


def _work(plan: Plan, dev) -> tuple[float, float]:
    """Algorithmic flops on the tensor pipe and bytes the math needs from HBM, for the roofline fractions."""
    p = plan.params
    if plan.family == "gemm":
        flops = 2.0 * p["M"] * p["N"] * p["K"] * p["schedule"].tiles / max(p["schedule"].total_tiles, 1)
        return flops, 2.0 * (p["M"] * p["K"] + p["K"] * p["N"] + p["M"] * p["N"])
    if plan.family == "attention":
        sch = p["schedule"]
        per_step = 4.0 * p["block_q"] * p["block_kv"] * p["D"]
        return per_step * sch.steps, 2.0 * 4 * p["B"] * p["H"] * p["S"] * p["D"]
    lengths = dev[4]
    return 0.0, float(lengths.sum().item()) * p["Hkv"] * p["D"] * 2 * 2


class Kernel:
    """A loop nest run by an sm_100a kernel. Call it like the function it was made from: with its tunable
    (`matmul(x, y, MatmulTiles(tm=256))`) it uses it; without, it is tuned for the inputs' shapes when first called
    with them, and remembers the result."""

    def __init__(self, fn: Callable[..., Any]) -> None:
        self.fn = fn
        self.nest: Nest = parse(fn)
        functools.update_wrapper(self, fn)
        self.default_tunable = fn.__defaults__[-1] if self.nest.tunable else None
        if self.nest.tunable and not is_tunable(self.default_tunable):
            raise self.nest.error(
                f"`{self.nest.tunable}`'s default must be an @autokernel.tunable, not {self.default_tunable!r}",
                self.nest.function.args)
        self._builds: dict = {}
        self._lowered: dict = {}
        self._tunings: dict = {}

    def __repr__(self) -> str:
        return f"<autokernel.Kernel {self.nest.name}>"

    def __call__(self, *args: Any) -> Any:
        arrays, _ = self._split(args)
        return self.lower(*args).run(*arrays)

    def lower(self, *args: Any) -> Lowered:
        arrays, tunable = self._split(args)
        signature = self.signature(*arrays)
        if tunable is None:
            return self.lowered(signature, self.tuning(*arrays).config)
        self.build(signature, tunable)
        return self.lowered(signature, Config(tunable, Pipeline()))

    def source(self, *args: Any) -> str:
        return self.lower(*args).source

    def reference(self, *args: Any) -> Any:
        """What the kernel computes: the loop nest run as written on the CPU, with `@` accumulating in f32."""
        arrays, tunable = self._split(args)
        if self.nest.tunable and tunable is None:
            tunable = self.lower(*arrays).config.tunable
        host = [jaxlike.Array(to_host(x)) for x in arrays]
        with jaxlike.mxu_semantics():
            out = self.fn(*host, tunable) if self.nest.tunable else self.fn(*host)
        return tuple(to_host(o) for o in out) if isinstance(out, tuple) else to_host(out)

    def verify(self, *args: Any, rtol: float | None = None, atol: float | None = None) -> float:
        """Run the kernel and its reference; AssertionError unless they agree within the tolerances for the dtypes
        (or `rtol` / `atol`). Returns the largest absolute difference."""
        arrays, tunable = self._split(args)
        if self.nest.tunable:
            tunable = tunable if tunable is not None else self.lower(*arrays).config.tunable
            full = (*arrays, tunable)
        else:
            full = arrays
        got, want = self(*full), self.reference(*full)
        dtypes = tuple(dtype for _, dtype in self.signature(*arrays)[: len(self.nest.inputs)])
        got, want = (got, want) if isinstance(got, tuple) else ((got,), (want,))
        return max(compare(f"{self.nest.name} output {name!r}", to_host(g), w, rtol, atol, dtypes)
                   for name, g, w in zip(self.nest.outputs, got, want, strict=True))

    def tuning(self, *arrays: Any) -> Tuning:
        signature = self.signature(*arrays)
        if signature not in self._tunings:
            self._tunings[signature] = tune(self, signature, arrays)
        return self._tunings[signature]

    # ------------------------------------------------------------------ building (used by tune.py too)

    def signature(self, *arrays: Any) -> Signature:
        signature = []
        for name, x in zip(self.nest.inputs, arrays, strict=True):
            if not (hasattr(x, "shape") and hasattr(x, "dtype")) or not tuple(x.shape):
                raise KernelError(f"{self.nest.name}: input `{name}` must be an array, got {type(x).__name__}")
            signature.append((tuple(int(s) for s in x.shape), _np_dtype(x)))
        for gather in self.nest.all_gathers:
            (rows, *rest), dtype = signature[self.nest.inputs.index(gather.source)]
            signature.append(((rows * collective.axis_size(gather.axis), *rest), dtype))
        return tuple(signature)

    def default_config(self, signature: Signature) -> Config:
        """The schedule to start from: the tunable's defaults, or the nearest tunable that builds."""
        tunable = self.default_tunable
        try:
            self.build(signature, tunable)
            return Config(tunable, Pipeline())
        except KernelError:
            if tunable is None:
                raise
            seen, frontier = {tunable}, [tunable]
            while frontier:
                later = []
                for t in frontier:
                    for n in neighbours(t):
                        if n in seen:
                            continue
                        seen.add(n)
                        try:
                            self.build(signature, n)
                            return Config(n, Pipeline())
                        except KernelError:
                            later.append(n)
                frontier = later
            raise

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

    def lowered(self, signature: Signature, config: Config, trace: bool = False) -> Lowered:
        key = (signature, config)
        if key not in self._lowered:
            plan, schedule = self.build(signature, config.tunable)
            source, entry = _lower(plan, config)
            self._lowered[key] = Lowered(plan, schedule, config, source, entry)
        return self._lowered[key]

    def _split(self, args: tuple[Any, ...]) -> tuple[tuple[Any, ...], Any]:
        n = len(self.nest.inputs)
        if self.nest.tunable and len(args) == n + 1:
            tunable = args[-1]
            if type(tunable) is not type(self.default_tunable):
                raise KernelError(
                    f"{self.nest.name}: `{self.nest.tunable}` must be a {type(self.default_tunable).__name__}, "
                    f"not {type(tunable).__name__}")
            return args[:-1], tunable
        if len(args) != n:
            more = f", then optionally `{self.nest.tunable}`" if self.nest.tunable else ""
            raise KernelError(
                f"{self.nest.name} takes {n} input arrays ({', '.join(self.nest.inputs)}){more}; got {len(args)}")
        return args, None


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
    if plan.family == "gemm":
        if any(np.dtype(s.dtype) != bf16 for s in plan.specs[:2]):
            raise nest.error("the matmul kernel takes bfloat16 operands")
        if np.dtype(p["out_dtype"]) not in (bf16, np.dtype(np.float32)):
            raise nest.error("the matmul kernel writes bfloat16 or float32")
        if p["K"] % 8 or p["N"] % 8:
            raise nest.error("K and N must be multiples of 8: rows of 16 bytes for the TMA descriptors")
        if not (p["tm"] % 128 == 0 or p["tm"] == p["M"]) or not (p["tn"] % 128 == 0 or p["tn"] == p["N"]):
            raise nest.error(f"tiles of {p['tm']} x {p['tn']}: output tiles must be multiples of 128 (the tensor core's "
                             "tile) or span the matrix")
    elif plan.family == "attention":
        if p["D"] != 128 or p["S"] % 128 or p["block_q"] % 128 or p["block_kv"] % 128:
            raise nest.error("the attention kernel takes head_dim 128 and blocks that are multiples of 128")
        if any(np.dtype(s.dtype) != bf16 for s in plan.specs[:3]):
            raise nest.error("the attention kernel takes bfloat16 q, k, v")
    elif p.get("mla"):
        if p["C"] != 512 or p["R"] != 128 or p["H"] % 16 or p["page"] % 16 or p["T"] != 1:
            raise nest.error("the MLA decode kernel takes one new token, 512 latent and 128 RoPE columns, heads in "
                             "multiples of 16 and blocks of a multiple of 16 positions")
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
    if plan.family == "attention":
        text = header + (
            f"kernel      tjx_causal_attention_bf16 (TMA rings, tcgen05 with S, P and O in TMEM, online softmax)\n"
            f"problem     q, k, v, out [{p['B']}, {p['H']}, {p['S']}, {p['D']}] bfloat16, causal\n"
            f"user blocks {p['block_q']} x {p['block_kv']}: {sch.tiles} tiles, {sch.steps} steps "
            f"({sch.pattern_steps} per (b, h), repeated {sch.repeats} times)\n"
            f"CTA         two 128-row query tiles sharing each 128-key K/V block; future blocks skipped\n"
            f"tables      {', '.join(f'{k}[{len(v)}]' for k, v in sch.tables.items()) or 'none'}\n")
        return text, lambda q, k, v: ops.causal_attention(q, k, v, p["block_q"], p["block_kv"])
    if p.get("mla"):
        text = header + (
            f"kernel      tjx_mla_decode_bf16 (device step tables, CTA-wide TMA ring, warp-level MMA over 16 heads, "
            f"partials merged by the last CTA to arrive)\n"
            f"problem     {p['B']} sequences, {p['H']} heads, {p['C']} latent + {p['R']} RoPE columns, blocks of "
            f"{p['page']} of {p['S']} cache positions\n"
            f"steps       at most {sch.steps}: step_tile / step_code / step_count are built on the device from lengths "
            f"before the kernel\n")
        return text, lambda q_c, q_r, c_kv, k_rope, lengths: ops.mla_decode(q_c, q_r, c_kv, k_rope, lengths, p["page"])
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
    """The largest absolute difference between `got` and `want`; AssertionError beyond `rtol` and `atol` (default:
    exact for integers, 1e-4 for f32, 2e-2 of the largest value for 16-bit results and for f32 results computed
    from 16-bit inputs). NaN equals NaN. The reference's rule, src/autokernel/api.py:320-364."""
    got, want = to_host(got), to_host(want)
    dtype = np.dtype(want.dtype)

    def floating(d) -> bool:
        d = np.dtype(d)
        return d.kind == "f" or d == _bf16()

    narrow = any(floating(d) and np.dtype(d).itemsize <= 2 for d in inputs)
    default = 0.0 if not floating(dtype) else (2e-2 if dtype.itemsize <= 2 or narrow else 1e-4)
    rtol = default if rtol is None else rtol
    got_all, want_all = got.reshape(-1), want.reshape(-1)
    chunks = range(0, want_all.size, COMPARE_CHUNK)
    if atol is None:
        scale = 1.0
        if default >= 2e-2:
            for start in chunks:
                w = want_all[start : start + COMPARE_CHUNK].astype(np.float64)
                scale = max(scale, float(np.max(np.abs(w), where=np.isfinite(w), initial=0.0)))
        atol = default * scale
    error, differ = 0.0, 0
    for start in chunks:
        g = got_all[start : start + COMPARE_CHUNK].astype(np.float64)
        w = want_all[start : start + COMPARE_CHUNK].astype(np.float64)
        same = (g == w) | (np.isnan(g) & np.isnan(w))
        with np.errstate(invalid="ignore"):
            error = max(error, float(np.max(np.abs(np.where(same, 0.0, g - w)), initial=0.0)))
        differ += int(np.sum(~np.isclose(g, w, rtol=rtol, atol=atol, equal_nan=True)))
    if differ:
        raise AssertionError(
            f"{what}: the kernel and its reference differ in {differ} of {want_all.size} elements "
            f"(largest difference {error:.3g}; rtol={rtol}, atol={atol:.3g})")
    return error
