"""A parsed nest + input shapes + a tunable -> the numbers a kernel is built from, and which sm_100a kernel family
runs it.

The prologue is executed on shapes only (allocations are not performed), loop ranges become integers, static
masks are evaluated per tile and per step into the reference's tables (src/autokernel/schedule.py:138-220), and the
nest is matched against the schedules this backend has kernels for:

  gemm        two parallel loops, one reduction loop, `acc += a[i:i+tm, k:k+tk] @ b[k:k+tk, j:j+tn]`, an optional tile
              mask and an optional `where(cols <= rows, acc, 0)` on the stored tile; `a` may be an all-gathered input
  attention   three parallel loops (b, h, i), a reduction loop over key blocks with the causal step mask, an online
              softmax, `q @ k.T` and `p @ v`
  decode      one parallel loop over sequences, a reduction loop over pages masked by an index array, pages chosen
              through a block table
  attention_block  two parallel loops (b, i) and two reduction loops per tile: the key blocks of causal attention
              over all heads, then the hidden units of the feed-forward layer after an RMSNorm
  rmsnorm_gemm     RMSNorm fused with the projection after it
Anything else is a KernelError ("not a recognised schedule"): there is no generic code generator and no fallback.
"""

from __future__ import annotations

import ast
import itertools
from dataclasses import dataclass, field
from typing import Any

import numpy as np

from .. import schedule as _schedule
from .errors import KernelError
from .parse import Nest


@dataclass(frozen=True)
class Spec:
    """An array's shape and dtype, standing in for it while planning."""

    shape: tuple[int, ...]
    dtype: Any

    @property
    def ndim(self) -> int:
        return len(self.shape)


Range = _schedule.Range  # one `for var in range(start, stop, step)` loop


@dataclass(frozen=True)
class Plan:
    nest: Nest
    family: str                      # "gemm" | "attention" | "decode"
    specs: tuple[Spec, ...]          # inputs, then gathered arrays
    outputs: tuple[Spec, ...]
    parallel: tuple[Range, ...]
    reductions: tuple[Range, ...]
    params: dict[str, Any] = field(default_factory=dict)   # what the kernel launch needs (tile sizes, flags)
    runtime: bool = False

    @property
    def loops(self) -> tuple[Range, ...]:
        return self.parallel + self.reductions


class _AllocStub:
    """Stands in for the array module while the prologue runs on shapes: zeros/full give Specs."""

    def __init__(self, real):
        self._real = real

    def zeros(self, shape, dtype=None):
        return Spec(tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,))), np.dtype(dtype or np.float32))

    def full(self, shape, value, dtype=None):
        return self.zeros(shape, dtype)

    def __getattr__(self, name):
        return getattr(self._real, name)


def _namespace(fn) -> dict[str, Any]:
    ns = dict(fn.__globals__)
    if fn.__closure__:
        ns.update({n: c.cell_contents for n, c in zip(fn.__code__.co_freevars, fn.__closure__, strict=True)})
    return ns


def schedule_only(nest: Nest, fn, specs: list[Spec], tunable: Any, chips: int = 1) -> _schedule.Schedule:
    """The nest's schedule without asking whether a kernel can run it."""
    ns, _, _, parallel, reductions = _run_prologue(nest, fn, specs, tunable, chips, need_outputs=False)
    return nest_schedule(nest, ns, parallel, reductions)


def make_plan(nest: Nest, fn, specs: list[Spec], tunable: Any, chips: int = 1) -> Plan:
    ns, all_specs, outputs, parallel, reductions = _run_prologue(nest, fn, specs, tunable, chips)
    return _recognise(nest, fn, ns, all_specs, outputs, parallel, reductions, chips)


def _run_prologue(nest: Nest, fn, specs: list[Spec], tunable: Any, chips: int = 1, need_outputs: bool = True):
    """Run the code before the loops on shapes alone and turn the loops' ranges into integers: (namespace, specs of
    inputs and gathered arrays, output specs, parallel ranges, reduction ranges)."""
    ns = _namespace(fn)
    for name, spec in zip(nest.inputs, specs, strict=True):
        ns[name] = spec
    if nest.tunable:
        ns[nest.tunable] = tunable
    gathered = {}
    for s in nest.prologue:
        if isinstance(s, ast.Assign) and any(g.node is s for g in nest.all_gathers):
            g = next(g for g in nest.all_gathers if g.node is s)
            src = ns[g.source]
            ns[g.name] = gathered[g.name] = Spec((src.shape[0] * chips, *src.shape[1:]), src.dtype)
            continue
        if isinstance(s, ast.Assign) and isinstance(s.value, ast.Call) and isinstance(s.value.func, ast.Attribute) \
                and s.value.func.attr in ("zeros", "full") and isinstance(s.value.func.value, ast.Name):
            module = s.value.func.value.id
            local = dict(ns)
            local[module] = _AllocStub(ns.get(module))
            _exec(nest, s, local)
            ns[s.targets[0].id] = local[s.targets[0].id]
            continue
        _exec(nest, s, ns)
    outputs = []
    for name in nest.outputs:
        if not isinstance(ns.get(name), Spec):
            if not need_outputs:
                continue
            raise nest.error(f"output `{name}` must be allocated with jnp.zeros or jnp.full", nest.allocations[name])
        outputs.append(ns[name])

    def ranges(loops):
        out = []
        for loop in loops:
            if any(isinstance(n, ast.Subscript) and isinstance(n.value, ast.Name) and n.value.id in nest.range_reads
                   for a in loop.args for n in ast.walk(a)):
                # A trip count read from an input as the kernel runs: no integer here; the recogniser of the family
                # knows its bound (the pages a sequence may have).
                out.append(Range(loop.var, 0, 0, 1))
                continue
            try:
                args = [int(eval(compile(ast.Expression(a), nest.filename, "eval"), ns)) for a in loop.args]
            except Exception as e:
                raise nest.error(f"the bounds of `{loop.var}`'s range must be integers known from the shapes ({e})",
                                 loop.node) from e
            start, stop, step = (0, args[0], 1) if len(args) == 1 else (args[0], args[1], 1) if len(args) == 2 else tuple(args)
            if step <= 0:
                raise nest.error("loops count up", loop.node)
            if (stop - start) % step:
                raise nest.error(f"`{loop.var}` doesn't take a whole number of steps of {step} from {start} to {stop}",
                                 loop.node)
            out.append(Range(loop.var, start, stop, step))
        return tuple(out)

    parallel, reductions = ranges(nest.parallel), ranges(nest.reductions)
    return ns, tuple(specs) + tuple(gathered.values()), tuple(outputs), parallel, reductions


def _exec(nest: Nest, stmt: ast.stmt, ns: dict) -> None:
    try:
        exec(compile(ast.Module([stmt], []), nest.filename, "exec"), ns)
    except KernelError:
        raise
    except Exception as e:
        raise nest.error(f"the code before the loops must run on the inputs' shapes alone: {type(e).__name__}: {e}",
                         stmt) from e


# ------------------------------------------------------------------------------------------ recognition


def _unsupported(nest: Nest, why: str, node=None) -> KernelError:
    return nest.error(f"not a recognised schedule: {why}. This backend runs matmul, causal matmul, causal "
                      "attention, paged GQA decode and all-gather matmul loop nests on sm_100a and has no "
                      "fallback for others", node or nest.function)


def _window(node: ast.expr):
    """`v : v + size` -> (v, size expr); `:` -> (None, None); a bare name -> (name, 'index')."""
    if isinstance(node, ast.Slice):
        if node.lower is None and node.upper is None:
            return None, None
        if isinstance(node.lower, ast.Name) and isinstance(node.upper, ast.BinOp) and isinstance(node.upper.op, ast.Add) \
                and isinstance(node.upper.left, ast.Name) and node.upper.left.id == node.lower.id:
            return node.lower.id, node.upper.right
        return "?", None
    if isinstance(node, ast.Name):
        return node.id, "index"
    return "?", None


def _subscripts(node: ast.Subscript):
    idx = node.slice
    return list(idx.elts) if isinstance(idx, ast.Tuple) else [idx]


def _eval(nest, ns, node) -> int:
    return int(eval(compile(ast.Expression(node), nest.filename, "eval"), ns))


def _mask_fn(nest, ns, mask: ast.expr, names: list[str]):
    code = compile(ast.Expression(mask), nest.filename, "eval")

    def holds(*values) -> bool:
        return bool(eval(code, ns, dict(zip(names, values, strict=True))))

    return holds


def _loop_names_read(mask: ast.expr, loop_vars: set[str]) -> frozenset[str]:
    return frozenset(n.id for n in ast.walk(mask) if isinstance(n, ast.Name) and n.id in loop_vars)


def nest_schedule(nest: Nest, ns, parallel, reductions) -> _schedule.Schedule:
    """The schedule of any parsed nest — recognised family or not — from its loops and masks: static masks are
    evaluated here through `schedule.make_schedule` (src/autokernel/schedule.py:147-220); a mask that reads an index
    array makes it a runtime schedule, whose tables the device builds."""
    if nest.runtime_masks:
        return _schedule.runtime_schedule(parallel, reductions)
    loop_vars = {r.var for r in (*parallel, *reductions)}
    masks = []
    for loop in (*nest.parallel, *nest.reductions):
        if loop.mask is None:
            continue
        code = compile(ast.Expression(loop.mask), nest.filename, "eval")

        def holds(values, code=code, node=loop.mask) -> bool:
            try:
                result = eval(code, ns, dict(values))
            except NameError as e:
                raise nest.error(f"can't evaluate `{e.name}` in a mask: masks read loop variables and constants", node) from e
            try:
                return bool(result)
            except Exception as e:
                raise nest.error("masks are Python conditions on loop variables and constants, evaluated when "
                                 f"planning; this one gave {type(result).__name__}", node) from e

        masks.append(_schedule.Mask(loop.var, _loop_names_read(loop.mask, loop_vars), holds))
    try:
        return _schedule.make_schedule(parallel, reductions, masks)
    except _schedule.ScheduleError as e:
        raise nest.error(str(e), nest.parallel[0].node) from e


def _require_known_form(nest: Nest, fn, family: str) -> None:
    """The nest's code (and its helpers') must be one of the forms the family's kernel computes: see fingerprint.py."""
    from .fingerprint import fingerprint
    from .recognised import RECOGNISED

    try:
        digest = fingerprint(fn)
    except (OSError, TypeError) as e:
        raise _unsupported(nest, f"its source cannot be read to identify it ({e})") from e
    if digest not in RECOGNISED[family]:
        what = {"rmsnorm": "RMSNorm fused with the projection after it, `rsqrt(mean(x^2) + eps) * ((x * gamma) @ w)`",
                "attention": "causal attention's online softmax over `q @ k.T` and `p @ v`",
                "attention_block": "an attention block: causal attention over all heads, RMSNorm of the heads side by "
                                   "side, then `gelu(n @ w_up) @ w_down`",
                "decode": "GQA decode's online softmax over the cache blocks",
                "rpa_write": "ragged paged attention's cache write: runs of new tokens copied into their pages",
                "rpa_prefill": "ragged paged attention's prefill case: causal attention of a tile of a sequence's new tokens "
                               "over its pages",
                "rpa_decode": "ragged paged attention's decode case: the online softmax over a sequence's pages of a cache "
                              "that holds keys and values side by side",
                "mla": "absorbed MLA decode's online softmax over the latent cache"}[family]
        raise _unsupported(nest, f"the loops and masks are those of {what}, but the tile code is not a form of it this "
                                 f"backend's kernel is known to compute (fingerprint {digest[:12]})")


def _recognise(nest, fn, ns, specs, outputs, parallel, reductions, chips) -> Plan:
    n_par, n_red = len(parallel), len(reductions)
    if n_red == 2 and n_par == 2 and len(nest.inputs) == 6 and not nest.runtime_masks and not nest.all_gathers:
        plan = _recognise_attention_block(nest, ns, specs, outputs, parallel, reductions)
        _require_known_form(nest, fn, "attention_block")
        return plan
    if n_red == 0 and nest.runtime_ranges:
        plan = _recognise_rpa_write(nest, ns, specs, outputs, parallel)
        _require_known_form(nest, fn, "rpa_write")
        return plan
    if n_red != 1:
        raise _unsupported(nest, f"{n_red} reduction loops (one is supported, or the two phases of an attention block)")
    if nest.runtime_ranges and len(nest.inputs) == 8:
        plan = _recognise_rpa_prefill(nest, fn, ns, specs, outputs, parallel, reductions)
        _require_known_form(nest, fn, "rpa_prefill")
        return plan
    if nest.runtime_ranges:
        plan = _recognise_rpa_decode(nest, fn, ns, specs, outputs, parallel, reductions)
        _require_known_form(nest, fn, "rpa_decode")
        return plan
    if nest.runtime_masks:
        plan = _recognise_decode(nest, ns, specs, outputs, parallel, reductions)
        _require_known_form(nest, fn, "mla" if plan.params.get("mla") else "decode")
        return plan
    if n_par == 2 and len(nest.inputs) == 3 and not nest.all_gathers and len(nest.bodies[0]) == 3:
        plan = _recognise_rmsnorm(nest, ns, specs, outputs, parallel, reductions)
        _require_known_form(nest, fn, "rmsnorm")
        return plan
    if n_par == 2:
        return _recognise_gemm(nest, ns, specs, outputs, parallel, reductions, chips)
    if n_par == 3:
        plan = _recognise_attention(nest, ns, specs, outputs, parallel, reductions)
        _require_known_form(nest, fn, "attention")
        return plan
    raise _unsupported(nest, f"{n_par} parallel loops")


def _call_of(node, attr: str):
    """The call's arguments if `node` is `<anything>.attr(...)` (or a bare `attr(...)`), else None."""
    if not isinstance(node, ast.Call) or node.keywords and attr != "zeros" and attr != "full":
        return None
    f = node.func
    name = f.attr if isinstance(f, ast.Attribute) else f.id if isinstance(f, ast.Name) else None
    return node.args if name == attr else None


def _is_name(node, name: str) -> bool:
    return isinstance(node, ast.Name) and node.id == name


def _is_zero(node) -> bool:
    return isinstance(node, ast.Constant) and isinstance(node.value, (int, float)) and not isinstance(node.value, bool) \
        and node.value == 0


def _iota_plus(nest, ns, value, loop_var: str, shape: tuple[int, int], dimension: int) -> bool:
    """Is `value` the expression `loop_var + broadcasted_iota(int32, shape, dimension)` (either order)?"""
    if not (isinstance(value, ast.BinOp) and isinstance(value.op, ast.Add)):
        return False
    for var, iota in ((value.left, value.right), (value.right, value.left)):
        args = _call_of(iota, "broadcasted_iota")
        if not _is_name(var, loop_var) or args is None or len(args) != 3:
            continue
        try:
            dtype, shp, dim = (eval(compile(ast.Expression(a), nest.filename, "eval"), ns) for a in args)
            if np.dtype(dtype) == np.int32 and tuple(int(v) for v in shp) == shape and int(dim) == dimension:
                return True
        except Exception:
            return False
    return False


def _match_gemm_tile_code(nest, ns, acc: str, i, j, tm: int, tn: int, out: Spec) -> bool:
    """The tile code around the reduction loop must be exactly a matmul's or a causal matmul's; returns whether it
    is the causal one. Before the loop: `acc = zeros((tm, tn), float32)`. After it: the store of `acc.astype(dtype)`
    (or `acc` itself), or of `where(cols <= rows, acc, 0).astype(dtype)` with `rows = i + iota(dim 0)` and
    `cols = j + iota(dim 1)` assigned just before. The output must be allocated with zeros: the skipped tiles and
    the masked entries are written as zeros. Anything else (a scale, a bias, another fill) would be computed
    wrongly by the fixed kernel, so it is refused here."""
    before, after = ([s for s in seg if not isinstance(s, ast.Pass)] for seg in (nest.segments[0], nest.segments[-1]))
    args = _call_of(before[0].value, "zeros") if len(before) == 1 and isinstance(before[0], ast.Assign) else None
    ok = args is not None and len(before[0].targets) == 1 and _is_name(before[0].targets[0], acc) and len(args) >= 1
    if ok:
        try:
            shape = tuple(int(v) for v in eval(compile(ast.Expression(args[0]), nest.filename, "eval"), ns))
            kw = {k.arg: k.value for k in before[0].value.keywords}
            dtype_node = args[1] if len(args) > 1 else kw.get("dtype")
            dtype = np.float32 if dtype_node is None else eval(compile(ast.Expression(dtype_node), nest.filename, "eval"), ns)
            ok = shape == (tm, tn) and np.dtype(dtype) == np.float32
        except Exception:
            ok = False
    if not ok:
        raise _unsupported(nest, f"before the reduction loop the tile code must be `{acc} = jnp.zeros((tm, tn), "
                                 "jnp.float32)` and nothing else", before[0] if before else nest.reductions[0].node)
    alloc = nest.allocations[nest.outputs[0]].value
    fill_args = _call_of(alloc, "full")
    if _call_of(alloc, "zeros") is None and not (fill_args is not None and len(fill_args) >= 2 and _is_zero(fill_args[1])):
        raise _unsupported(nest, "the output must be allocated with zeros: skipped tiles are written as zeros",
                           nest.allocations[nest.outputs[0]])
    store = nest.stores[nest.outputs[0]]
    if not after or after[-1] is not store.node:
        raise _unsupported(nest, "the tile's store must be the last statement after the reduction loop", store.node)
    idx = store.index.elts if isinstance(store.index, ast.Tuple) else [store.index]
    if len(idx) != 2 or _window(idx[0])[0] != i.var or _window(idx[1])[0] != j.var:
        raise _unsupported(nest, "the tile is stored at `[i : i + tm, j : j + tn]`", store.node)
    value = store.value
    cast = _call_of(value, "astype")
    if cast is not None and isinstance(value.func, ast.Attribute) and len(cast) == 1:
        try:
            to = np.dtype(eval(compile(ast.Expression(cast[0]), nest.filename, "eval"), ns))
        except Exception as e:
            raise _unsupported(nest, f"the stored tile's dtype is not known from the shapes ({e})", store.node) from e
        if to != np.dtype(out.dtype):
            raise _unsupported(nest, "the stored tile must be cast to the output's dtype", store.node)
        value = value.func.value
    elif np.dtype(out.dtype) != np.float32:
        raise _unsupported(nest, "the stored tile must be `acc.astype(dtype)`", store.node)
    if _is_name(value, acc):
        if len(after) != 1:
            raise _unsupported(nest, "code after the reduction loop other than the store (a fused epilogue)", after[0])
        return False
    where = _call_of(value, "where")
    cond_ok = False
    if where is not None and len(where) == 3 and _is_name(where[1], acc) and _is_zero(where[2]):
        cond = where[0]
        if isinstance(cond, ast.Compare) and len(cond.ops) == 1 and len(cond.comparators) == 1 \
                and isinstance(cond.left, ast.Name) and isinstance(cond.comparators[0], ast.Name):
            left, right = cond.left.id, cond.comparators[0].id
            cols, rows = (left, right) if isinstance(cond.ops[0], ast.LtE) else (right, left) \
                if isinstance(cond.ops[0], ast.GtE) else (None, None)
            defs = {s.targets[0].id: s.value for s in after[:-1]
                    if isinstance(s, ast.Assign) and len(s.targets) == 1 and isinstance(s.targets[0], ast.Name)}
            cond_ok = (cols is not None and len(after) == 3 and set(defs) == {rows, cols} and rows != cols
                       and _iota_plus(nest, ns, defs[rows], i.var, (tm, tn), 0)
                       and _iota_plus(nest, ns, defs[cols], j.var, (tm, tn), 1))
    if not cond_ok:
        raise _unsupported(nest, "the stored tile must be the accumulator, `acc.astype(dtype)`, or its causal form "
                                 "`jnp.where(cols <= rows, acc, 0.0).astype(dtype)` with `rows = i + iota(.., 0)` and "
                                 "`cols = j + iota(.., 1)`; other epilogues are not built", store.node)
    return True


def _recognise_rmsnorm(nest, ns, specs, outputs, parallel, reductions) -> Plan:
    """`rmsnorm_matmul` (examples/rmsnorm_matmul.py:31-47): (x, gamma, w) with x (M, D), gamma (1, D), w (D, N); loops
    (i, j) over the output's tiles and k over the model dimension, no masks. What the tile code computes is pinned
    by its fingerprint (the caller checks it); here the shapes and the loops."""
    (i, j), (k,) = parallel, reductions
    x, gamma, w = specs[:3]
    if x.ndim != 2 or gamma.ndim != 2 or w.ndim != 2 or len(outputs) != 1 or outputs[0].ndim != 2:
        raise _unsupported(nest, "RMSNorm + matmul takes x (M, D), gamma (1, D) and w (D, N)")
    (M, D), N = x.shape, w.shape[1]
    if gamma.shape != (1, D) or w.shape[0] != D or outputs[0].shape != (M, N):
        raise _unsupported(nest, "RMSNorm + matmul takes x (M, D), gamma (1, D) and w (D, N) and stores (M, N)")
    if any(l.mask is not None for l in (*nest.parallel, *nest.reductions)):
        raise _unsupported(nest, "a mask on this loop")
    if (i.start, i.stop, j.start, j.stop, k.start, k.stop) != (0, M, 0, N, 0, D):
        raise _unsupported(nest, "the loops must cover the operands exactly")
    sch = nest_schedule(nest, ns, parallel, reductions)
    params = dict(M=M, N=N, K=D, tm=i.step, tn=j.step, tk=k.step, eps=float(ns.get("EPS", 1e-6)),
                  out_dtype=outputs[0].dtype, schedule=sch, causal=False, transposed=False)
    return Plan(nest, "rmsnorm_gemm", specs, outputs, parallel, reductions, params)


def _recognise_gemm(nest, ns, specs, outputs, parallel, reductions, chips) -> Plan:
    (i, j), (k,) = parallel, reductions
    body = nest.bodies[0]
    if len(body) != 1 or not (isinstance(body[0], ast.AugAssign) and isinstance(body[0].op, ast.Add)
                              and isinstance(body[0].value, ast.BinOp) and isinstance(body[0].value.op, ast.MatMult)):
        raise _unsupported(nest, "the reduction loop's body must be `acc += a[...] @ b[...]`", nest.reductions[0].node)
    acc = body[0].target.id
    left, right = body[0].value.left, body[0].value.right
    transposed = isinstance(right, ast.Attribute) and right.attr == "T"
    right = right.value if transposed else right
    if not (isinstance(left, ast.Subscript) and isinstance(right, ast.Subscript)
            and isinstance(left.value, ast.Name) and isinstance(right.value, ast.Name)):
        raise _unsupported(nest, "the matmul's operands must be tiles of inputs", body[0])
    names = list(nest.inputs) + [g.name for g in nest.all_gathers]
    a_name, b_name = left.value.id, right.value.id
    if a_name not in names or b_name not in names:
        raise _unsupported(nest, "the matmul's operands must be tiles of inputs", body[0])
    la, lb = _subscripts(left), _subscripts(right)
    if len(la) != 2 or len(lb) != 2:
        raise _unsupported(nest, "the matmul's operands must be 2-D tiles", body[0])
    (a0, tm_e), (a1, tk_e) = _window(la[0]), _window(la[1])
    b_rows, b_cols = (_window(lb[1]), _window(lb[0])) if transposed else (_window(lb[0]), _window(lb[1]))
    if (a0, a1, b_rows[0], b_cols[0]) != (i.var, k.var, k.var, j.var):
        raise _unsupported(nest, "expected `a[i:i+tm, k:k+tk] @ b[k:k+tk, j:j+tn]` over loops (i, j, k)", body[0])
    tm, tk, tn = _eval(nest, ns, tm_e), _eval(nest, ns, tk_e), _eval(nest, ns, b_cols[1])
    if (tm, tn, tk) != (i.step, j.step, k.step):
        raise _unsupported(nest, "tile sizes must equal the loops' steps", body[0])
    a_spec, b_spec = specs[names.index(a_name)], specs[names.index(b_name)]
    out = outputs[0]
    if len(outputs) != 1 or out.ndim != 2:
        raise _unsupported(nest, "one 2-D output")
    M, K = a_spec.shape
    N = b_spec.shape[0] if transposed else b_spec.shape[1]
    if (i.start, i.stop, j.start, j.stop, k.start, k.stop) != (0, M, 0, N, 0, K) or out.shape != (M, N):
        raise _unsupported(nest, "the loops must cover the operands exactly")
    causal = _match_gemm_tile_code(nest, ns, acc, i, j, tm, tn, out)
    store = nest.stores[nest.outputs[0]]
    tile_mask = nest.parallel[1].mask
    if nest.parallel[0].mask is not None or nest.reductions[0].mask is not None:
        raise _unsupported(nest, "a mask on this loop")
    gathered = nest.all_gathers[0] if nest.all_gathers else None
    if gathered is not None and (tile_mask is not None or a_name != gathered.name):
        raise _unsupported(nest, "a gathered input is the left operand of an unmasked matmul")
    sch = nest_schedule(nest, ns, parallel, reductions)
    if causal and not _is_tril_mask(nest, ns, tile_mask, i, j):
        raise _unsupported(nest, "an elementwise `where` on the tile other than the causal `cols <= rows` with "
                                 "its tile mask `j > i + tm - 1`", store.node)
    params = dict(M=M, N=N, K=K, tm=tm, tn=tn, tk=tk, causal=causal, transposed=transposed, a=a_name, b=b_name,
                  out_dtype=out.dtype, schedule=sch, gathered=gathered.name if gathered else None,
                  loop_vars=(i.var, j.var), chips=chips)
    return Plan(nest, "gemm", specs, outputs, parallel, reductions, params)


def _is_tril_mask(nest, ns, tile_mask, i, j) -> bool:
    """Does the tile mask skip exactly the tiles wholly above the diagonal (`j > i + tm - 1`)?"""
    if tile_mask is None:
        return i.count == 1 or j.count == 1 and j.step >= i.stop  # one tile per row band: nothing to skip
    holds = _mask_fn(nest, ns, tile_mask, [i.var, j.var])
    return all(holds(i.value(bi), j.value(bj)) == (j.value(bj) > i.value(bi) + i.step - 1)
               for bi in range(i.count) for bj in range(j.count))


def _recognise_attention(nest, ns, specs, outputs, parallel, reductions) -> Plan:
    (b, h, i), (j,) = parallel, reductions
    if len(nest.inputs) != 3 or any(s.ndim != 4 for s in specs[:3]) or len(outputs) != 1:
        raise _unsupported(nest, "causal attention takes q, k, v of shape (B, H, S, D)")
    B, H, S, D = specs[0].shape
    if any(s.shape != (B, H, S, D) for s in specs[:3]) or outputs[0].shape != (B, H, S, D):
        raise _unsupported(nest, "q, k, v and the output must share one shape (B, H, S, D)")
    mask = nest.reductions[0].mask
    if mask is None or any(l.mask is not None for l in nest.parallel):
        raise _unsupported(nest, "causal attention masks its key loop with `j > i + block_q - 1`")
    holds = _mask_fn(nest, ns, mask, [i.var, j.var])
    causal = all(holds(i.value(bi), j.value(bj)) == (j.value(bj) > i.value(bi) + i.step - 1)
                 for bi in range(i.count) for bj in range(j.count))
    if not causal or (b.count, h.count, i.stop, j.stop) != (B, H, S, S):
        raise _unsupported(nest, "the step mask must be the causal one, `j > i + block_q - 1`, over whole sequences",
                           nest.reductions[0].node)
    sch = nest_schedule(nest, ns, parallel, reductions)
    params = dict(B=B, H=H, S=S, D=D, block_q=i.step, block_kv=j.step, schedule=sch)
    return Plan(nest, "attention", specs, outputs, parallel, reductions, params)


def phases_of(nest: Nest, reductions) -> tuple[Range, ...]:
    """The reduction loops that take steps of their own: one of a single iteration and no mask runs inline, in the
    code around it (src/autokernel/plan.py:8-11)."""
    return tuple(r for r, loop in zip(reductions, nest.reductions, strict=True) if r.count > 1 or loop.mask is not None)


def _recognise_attention_block(nest, ns, specs, outputs, parallel, reductions) -> Plan:
    """`attention_block` (examples/attention_block.py:49-85): (q, k, v, gamma, w_up, w_down) with q, k, v
    (B, H, S, Dh), gamma (1, D), w_up (D, F), w_down (F, D), D = H * Dh; loops (b, i) over the query blocks, then two
    phases per tile: j over the key blocks with the causal step mask, f over the hidden units. What the tile code
    computes is pinned by its fingerprint (the caller checks it); here the shapes, the loops and the mask."""
    (b, i), (j, f) = parallel, reductions
    q, k, v, gamma, w_up, w_down = specs[:6]
    if q.ndim != 4 or k.shape != q.shape or v.shape != q.shape or len(outputs) != 1:
        raise _unsupported(nest, "an attention block takes q, k, v of one shape (B, H, S, Dh)")
    B, H, S, Dh = q.shape
    D = H * Dh
    if gamma.shape != (1, D) or w_up.ndim != 2 or w_up.shape[0] != D or w_down.shape != (w_up.shape[1], D) \
            or outputs[0].shape != (B, S, D):
        raise _unsupported(nest, f"an attention block takes gamma (1, {D}), w_up ({D}, F) and w_down (F, {D}) and "
                                 f"stores ({B}, {S}, {D})")
    F = w_up.shape[1]
    mask = nest.reductions[0].mask
    if mask is None or nest.reductions[1].mask is not None or any(l.mask is not None for l in nest.parallel):
        raise _unsupported(nest, "an attention block masks its key loop with `j > i + block_q - 1`, and nothing else")
    holds = _mask_fn(nest, ns, mask, [i.var, j.var])
    causal = all(holds(i.value(bi), j.value(bj)) == (j.value(bj) > i.value(bi) + i.step - 1)
                 for bi in range(i.count) for bj in range(j.count))
    if not causal or (b.start, b.stop, b.step, i.start, i.stop, j.start, j.stop, f.start, f.stop) != (0, B, 1, 0, S, 0, S, 0, F):
        raise _unsupported(nest, "the step mask must be the causal one, `j > i + block_q - 1`, and the loops must "
                                 "cover the batch, the sequence and the hidden units", nest.reductions[0].node)
    phases = phases_of(nest, reductions)
    sch = nest_schedule(nest, ns, parallel, phases)
    params = dict(B=B, H=H, S=S, D=Dh, F=F, block_q=i.step, block_kv=j.step, block_f=f.step,
                  eps=float(ns.get("EPS", 1e-6)), schedule=sch, phases=tuple(r.var for r in phases))
    return Plan(nest, "attention_block", specs, outputs, parallel, reductions, params)


def _recognise_contiguous_decode(nest, ns, specs, outputs, parallel, reductions) -> Plan:
    """`gqa_decode`: (q, k_cache, v_cache, lengths), blocks of the cache skipped with `j >= lengths[b]`. It runs as
    paged decode over the identity block table (block j of sequence b is page b * blocks + j)."""
    (b,), (j,) = parallel, reductions
    q, kc, vc, lengths = specs[:4]
    mask = nest.reductions[0].mask
    reads = {n.value.id for n in ast.walk(mask) if isinstance(n, ast.Subscript) and isinstance(n.value, ast.Name)}
    if reads != {nest.inputs[3]} or np.dtype(lengths.dtype) != np.int32:
        raise _unsupported(nest, "the block loop's mask must compare the block's first position with lengths[b]",
                           nest.reductions[0].node)
    if q.ndim != 4 or kc.ndim != 3 or kc.shape != vc.shape or lengths.ndim != 1:
        raise _unsupported(nest, "decode takes q (B, T, H, D), caches (B, S, Hkv * D) and lengths (B,)")
    B, T, H, D = q.shape
    _, S, W = kc.shape
    code = compile(ast.Expression(mask), nest.filename, "eval")

    def skipped(jv: int, length: int) -> bool:
        return bool(eval(code, dict(ns), {j.var: jv, b.var: 0, nest.inputs[3]: [length]}))

    block = j.step
    ok = all(skipped(jv, n) == (jv >= n) for jv in (0, block, (j.count - 1) * block) for n in (0, 1, block, block + 1, S))
    if not ok or (b.count, kc.shape[0]) != (B, B) or j.start != 0 or j.stop != S or S % block:
        raise _unsupported(nest, "the block loop must cover the cache and skip blocks with `j >= lengths[b]`",
                           nest.reductions[0].node)
    sch = _schedule.paged_decode_schedule(B, j.count)
    params = dict(B=B, T=T, H=H, Hkv=W // D, D=D, page=block, pages=j.count, num_pages=B * j.count, schedule=sch,
                  contiguous=True)
    return Plan(nest, "decode", specs, outputs, parallel, reductions, params, runtime=True)


def _recognise_mla_decode(nest, ns, specs, outputs, parallel, reductions) -> Plan:
    """`mla_decode`: (q_c, q_r, c_kv, k_rope, lengths), blocks of the latent cache skipped with `j >= lengths[b]`."""
    (b,), (j,) = parallel, reductions
    q_c, q_r, c_kv, k_rope, lengths = specs[:5]
    mask = nest.reductions[0].mask
    reads = {n.value.id for n in ast.walk(mask) if isinstance(n, ast.Subscript) and isinstance(n.value, ast.Name)}
    if reads != {nest.inputs[4]} or np.dtype(lengths.dtype) != np.int32:
        raise _unsupported(nest, "the block loop's mask must compare the block's first position with lengths[b]",
                           nest.reductions[0].node)
    if q_c.ndim != 4 or q_r.ndim != 4 or k_rope.ndim != 3 or lengths.ndim != 1 or q_c.shape[:3] != q_r.shape[:3] \
            or c_kv.shape[:2] != k_rope.shape[:2] or c_kv.shape[2] != q_c.shape[3] or k_rope.shape[2] != q_r.shape[3]:
        raise _unsupported(nest, "MLA decode takes q_c (B, T, H, C), q_r (B, T, H, R), c_kv (B, S, C), k_rope (B, S, R) "
                                 "and lengths (B,)")
    B, T, H, C = q_c.shape
    S, R = c_kv.shape[1], k_rope.shape[2]
    code = compile(ast.Expression(mask), nest.filename, "eval")

    def skipped(jv: int, length: int) -> bool:
        return bool(eval(code, dict(ns), {j.var: jv, b.var: 0, nest.inputs[4]: [length]}))

    block = j.step
    ok = all(skipped(jv, n) == (jv >= n) for jv in (0, block, (j.count - 1) * block) for n in (0, 1, block, block + 1, S))
    if not ok or b.count != B or j.start != 0 or j.stop != S or S % block:
        raise _unsupported(nest, "the block loop must cover the cache and skip blocks with `j >= lengths[b]`",
                           nest.reductions[0].node)
    sch = _schedule.paged_decode_schedule(B, j.count)
    params = dict(B=B, T=T, H=H, C=C, R=R, S=S, page=block, pages=j.count, schedule=sch, mla=True)
    return Plan(nest, "decode", specs, outputs, parallel, reductions, params, runtime=True)


def _recognise_rpa_write(nest, ns, specs, outputs, parallel) -> Plan:
    """`rpa_write` (examples/ragged_paged_attention.py:33-47): (kv_cache, keys, values, page_indices, write_page,
    write_rows, write_first, write_stop, n_writes), a tile per run, the run count read as the kernel runs, the output
    the cache updated. What a tile stores is pinned by the fingerprint (the caller checks it); here the shapes."""
    if len(parallel) != 1 or len(nest.inputs) != 9 or len(nest.outputs) != 1 \
            or nest.inplace != {nest.outputs[0]: nest.inputs[0]} or nest.range_reads != {nest.inputs[8]}:
        raise _unsupported(nest, "a run count read from an input other than ragged paged attention's cache write: "
                                 "(kv_cache, keys, values, page_indices, write_page, write_rows, write_first, write_stop, "
                                 "n_writes) with the cache updated in place")
    cache, keys, values, page_indices, *tables, n_writes = specs[:9]
    int32 = np.dtype(np.int32)
    if cache.ndim != 5 or cache.shape[3] != 2 or keys.shape != values.shape or keys.ndim != 3 \
            or keys.shape[1:] != (cache.shape[2], cache.shape[4]) or page_indices.ndim != 1 \
            or any(t.ndim != 1 or t.shape != tables[0].shape for t in tables) or n_writes.shape != (1,) \
            or any(np.dtype(x.dtype) != int32 for x in (page_indices, *tables, n_writes)) \
            or len({np.dtype(x.dtype) for x in (cache, keys, values)}) != 1:
        raise _unsupported(nest, "the cache write takes a cache (pages, page_size, Hkv, 2, D), keys and values (T, Hkv, D) "
                                 "of its dtype, page_indices, four run tables of one length and n_writes (1,), int32")
    max_runs = tables[0].shape[0]
    sch = _schedule.runtime_schedule([Range(parallel[0].var, 0, max_runs, 1)], [Range("row", 0, 1, 1)])
    params = dict(rpa_write=True, T=keys.shape[0], Hkv=cache.shape[2], D=cache.shape[4], page=cache.shape[1],
                  num_pages=cache.shape[0], max_runs=max_runs, schedule=sch)
    return Plan(nest, "rpa_write", specs, outputs, (Range(parallel[0].var, 0, max_runs, 1),), (), params, runtime=True)


def _closed_scale(nest, fn) -> float:
    """The softmax scale of a kernel made by `make_...(sm_scale)`: the one float the function closes over."""
    closed = [c.cell_contents for c in (fn.__closure__ or ()) if isinstance(c.cell_contents, float)]
    if len(closed) != 1:
        raise _unsupported(nest, "the kernel must close over its softmax scale, one float (`make_decode(sm_scale)`)")
    return float(closed[0])


def _recognise_rpa_prefill(nest, fn, ns, specs, outputs, parallel, reductions) -> Plan:
    """`rpa_prefill` (examples/ragged_paged_attention.py:204-243): (q, kv_cache, page_indices, tile_page, tile_rows,
    tile_pos, tile_stop, n_tiles), a tile per block of a sequence's new tokens, the tile count and each tile's pages
    read as the kernel runs, the output q updated. What the tile code computes is pinned by its fingerprint (the
    caller checks it); here the shapes and the loops."""
    if len(parallel) != 1 or len(nest.outputs) != 1 or nest.inplace != {nest.outputs[0]: nest.inputs[0]} \
            or nest.range_reads != {nest.inputs[6], nest.inputs[7]}:
        raise _unsupported(nest, "trip counts read from inputs other than ragged paged attention's prefill case: (q, "
                                 "kv_cache, page_indices, tile_page, tile_rows, tile_pos, tile_stop, n_tiles) with q "
                                 "updated in place, tiles counted by n_tiles and their pages by tile_stop")
    q, cache, page_indices, tile_page, tile_rows, tile_pos, tile_stop, n_tiles = specs[:8]
    int32 = np.dtype(np.int32)
    tiles = tile_page.shape[0] if tile_page.ndim == 1 else -1
    if q.ndim != 3 or cache.ndim != 5 or cache.shape[3] != 2 or cache.shape[4] != q.shape[2] or page_indices.ndim != 1 \
            or any(t.shape != (tiles,) for t in (tile_pos, tile_stop)) or tile_rows.shape != (tiles + 1,) \
            or n_tiles.shape != (1,) or np.dtype(q.dtype) != np.dtype(cache.dtype) \
            or any(np.dtype(x.dtype) != int32 for x in (page_indices, tile_page, tile_rows, tile_pos, tile_stop, n_tiles)):
        raise _unsupported(nest, "ragged paged prefill takes q (T, H, D), a cache (pages, page_size, Hkv, 2, D) of q's "
                                 "dtype, page_indices, tile tables (tile_rows one longer) and n_tiles (1,), int32")
    T, H, D = q.shape
    num_pages, page, Hkv = cache.shape[0], cache.shape[1], cache.shape[2]
    max_pages = page_indices.shape[0]  # a tile walks at most every listed page
    sch = _schedule.runtime_schedule([Range(parallel[0].var, 0, tiles, 1)], [Range(reductions[0].var, 0, max_pages, 1)])
    params = dict(rpa_prefill=True, T=T, H=H, Hkv=Hkv, D=D, page=page, num_pages=num_pages, max_tiles=tiles,
                  sm_scale=_closed_scale(nest, fn), schedule=sch)
    return Plan(nest, "rpa_prefill", specs, outputs, (Range(parallel[0].var, 0, tiles, 1),),
                (Range(reductions[0].var, 0, max_pages, 1),), params, runtime=True)


def _recognise_rpa_decode(nest, fn, ns, specs, outputs, parallel, reductions) -> Plan:
    """`rpa_decode` (examples/ragged_paged_attention.py:121-149): (q, kv_cache, kv_lens, page_indices, distribution), a
    tile per sequence, its pages counted from kv_lens as the kernel runs, the output q updated. What the tile code
    computes is pinned by its fingerprint (the caller checks it); here the shapes, the loops and the scale."""
    if len(parallel) != 1 or len(nest.inputs) != 5 or nest.inplace != {nest.outputs[0]: nest.inputs[0]} or len(nest.outputs) != 1:
        raise _unsupported(nest, "a trip count read from an input other than ragged paged attention's decode case: "
                                 "(q, kv_cache, kv_lens, page_indices, distribution) with q updated in place")
    q, cache, kv_lens, page_indices, distribution = specs[:5]
    int32 = np.dtype(np.int32)
    if q.ndim != 3 or cache.ndim != 5 or cache.shape[3] != 2 or cache.shape[4] != q.shape[2] or kv_lens.ndim != 1 \
            or page_indices.ndim != 1 or distribution.shape != (3,) or page_indices.shape[0] % kv_lens.shape[0] \
            or any(np.dtype(x.dtype) != int32 for x in (kv_lens, page_indices, distribution)) \
            or np.dtype(q.dtype) != np.dtype(cache.dtype):
        raise _unsupported(nest, "ragged paged decode takes q (T, H, D), a cache (pages, page_size, Hkv, 2, D) of q's "
                                 "dtype, kv_lens (S,), page_indices (S * pages_per_seq,) and distribution (3,), int32")
    if nest.range_reads != {nest.inputs[2], nest.inputs[4]}:
        raise _unsupported(nest, "the page loop's trip count must be read from kv_lens and distribution",
                           nest.reductions[0].node)
    T, H, D = q.shape
    num_pages, page, Hkv = cache.shape[0], cache.shape[1], cache.shape[2]
    S = kv_lens.shape[0]
    pages = page_indices.shape[0] // S
    (s_loop,) = parallel
    if (s_loop.start, s_loop.stop, s_loop.step) != (0, min(S, T), 1):
        raise _unsupported(nest, "the sequence loop must run over min(sequences, tokens): sequence s is token s",
                           nest.parallel[0].node)
    n = min(S, T)
    sch = _schedule.paged_decode_schedule(n, pages)
    params = dict(B=n, T=1, H=H, Hkv=Hkv, D=D, page=page, pages=pages, num_pages=num_pages, schedule=sch, rpa=True,
                  tokens=T, sequences=S, sm_scale=_closed_scale(nest, fn))
    reductions = (Range(reductions[0].var, 0, pages, 1),)
    return Plan(nest, "decode", specs, outputs, parallel, reductions, params, runtime=True)


def _recognise_decode(nest, ns, specs, outputs, parallel, reductions) -> Plan:
    if len(parallel) == 1 and len(nest.inputs) == 4:
        return _recognise_contiguous_decode(nest, ns, specs, outputs, parallel, reductions)
    if len(parallel) == 1 and len(nest.inputs) == 5 and specs[3].ndim == 3:
        return _recognise_mla_decode(nest, ns, specs, outputs, parallel, reductions)
    if len(parallel) != 1 or len(nest.inputs) != 5:
        raise _unsupported(nest, "a runtime mask other than decode's: (q, k_cache, v_cache, lengths) or "
                                 "(q, k_pages, v_pages, block_tables, lengths)")
    (b,), (p,) = parallel, reductions
    q, kp, vp, bt, lengths = specs[:5]
    mask = nest.reductions[0].mask
    reads = {n.value.id for n in ast.walk(mask) if isinstance(n, ast.Subscript) and isinstance(n.value, ast.Name)}
    if reads != {nest.inputs[4]} or np.dtype(lengths.dtype) != np.int32 or np.dtype(bt.dtype) != np.int32:
        raise _unsupported(nest, "the page loop's mask must compare the page's first position with lengths[b]",
                           nest.reductions[0].node)
    if q.ndim != 4 or kp.ndim != 3 or kp.shape != vp.shape or bt.ndim != 2 or lengths.ndim != 1:
        raise _unsupported(nest, "paged decode takes q (B, T, H, D), pages (num_pages, page, Hkv * D), block tables "
                                 "(B, pages) and lengths (B,)")
    B, T, H, D = q.shape
    num_pages, page, W = kp.shape
    # The mask must be `p * page >= lengths[b]`: check it on the extremes with a stand-in for lengths.
    probe_ns = dict(ns)
    code = compile(ast.Expression(mask), nest.filename, "eval")

    def skipped(pv: int, length: int) -> bool:
        return bool(eval(code, probe_ns, {p.var: pv, b.var: 0, nest.inputs[4]: [length]}))

    ok = all(skipped(pv, n) == (pv * page >= n) for pv in (0, 1, p.count - 1) for n in (0, 1, page, page + 1, page * p.count))
    if not ok or (b.count, p.count) != (B, bt.shape[1]) or p.step != 1 or p.start != 0:
        raise _unsupported(nest, "the page loop must skip pages with `p * page_size >= lengths[b]`", nest.reductions[0].node)
    sch = _schedule.paged_decode_schedule(B, p.count)
    params = dict(B=B, T=T, H=H, Hkv=W // D, D=D, page=page, pages=p.count, num_pages=num_pages, schedule=sch)
    return Plan(nest, "decode", specs, outputs, parallel, reductions, params, runtime=True)
