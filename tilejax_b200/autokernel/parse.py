"""A kernel function's source -> its loop nest, as written (syntax only).

The accepted shape is the reference's (src/autokernel/parse.py:187-228, README "The loop nest"): positional input
arrays then at most one defaulted tunable; a prologue of assignments and asserts (shapes, tile sizes, output
allocations, at most one `xs = autokernel.all_gather(x, axis)`); ONE loop nest of `for v in range(...)` loops — the
outer ones are the parallel loops (one output tile per combination), the innermost level may hold per-tile code
around reduction loops; a loop body may start with `if mask: continue`; a tile is stored once with
`out = out.at[idx].set(value)`; then `return` of the output names. Anything else is a KernelError naming the line.
"""

from __future__ import annotations

import ast
import inspect
import textwrap
from dataclasses import dataclass, field

from .errors import KernelError


@dataclass(frozen=True)
class Loop:
    var: str
    args: tuple[ast.expr, ...]       # the arguments of range(...)
    mask: ast.expr | None            # `if mask: continue` at the top of the body
    node: ast.For


@dataclass(frozen=True)
class Store:
    output: str
    index: ast.expr
    value: ast.expr
    node: ast.Assign


@dataclass(frozen=True)
class AllGather:
    name: str
    source: str
    axis: str
    node: ast.Assign


@dataclass(frozen=True)
class Nest:
    name: str
    filename: str
    function: ast.FunctionDef
    inputs: tuple[str, ...]
    tunable: str | None
    prologue: tuple[ast.stmt, ...]
    allocations: dict[str, ast.Assign]
    outputs: tuple[str, ...]
    parallel: tuple[Loop, ...]
    reductions: tuple[Loop, ...]
    bodies: tuple[tuple[ast.stmt, ...], ...]
    segments: tuple[tuple[ast.stmt, ...], ...]   # per-tile code before, between and after the reduction loops
    stores: dict[str, Store]
    all_gathers: tuple[AllGather, ...] = ()
    index_reads: frozenset[str] = field(default_factory=frozenset)  # inputs read element-wise in masks
    range_reads: frozenset[str] = field(default_factory=frozenset)  # inputs read element-wise in a loop's range
    inplace: dict[str, str] = field(default_factory=dict)           # output -> the input it starts as (`out = q`)

    @property
    def runtime_masks(self) -> bool:
        return bool(self.index_reads)

    @property
    def runtime_ranges(self) -> bool:
        """A loop runs a number of times read from an input as the kernel runs (`for w in range(n_writes[0])`,
        `for p in range(cdiv(kv_lens[s], page_size))`: examples/ragged_paged_attention.py:39, :138)."""
        return bool(self.range_reads)

    def error(self, message: str, node: ast.AST | None = None) -> KernelError:
        return KernelError(f"{self.name}: {message}", filename=self.filename, node=node)


def parse(fn) -> Nest:
    name = getattr(fn, "__name__", repr(fn))
    try:
        source = textwrap.dedent(inspect.getsource(fn))
        filename = inspect.getsourcefile(fn) or "<unknown>"
        first_line = inspect.getsourcelines(fn)[1]
    except (OSError, TypeError) as e:
        raise KernelError(f"{name}: can't read its source ({e}): a kernel is a Python function in a file") from e
    tree = ast.parse(source)
    if not tree.body or not isinstance(tree.body[0], ast.FunctionDef):
        raise KernelError(f"{name}: a kernel is a function defined with `def`")
    function = tree.body[0]
    ast.increment_lineno(function, first_line - 1)
    return _Parser(name, filename, function, fn).parse()


class _Parser:
    def __init__(self, name, filename, function, fn):
        self.name, self.filename, self.function, self.fn = name, filename, function, fn

    def error(self, message, node=None):
        return KernelError(f"{self.name}: {message}", filename=self.filename, node=node)

    def parse(self) -> Nest:
        f = self.function
        a = f.args
        n_defaults = len(a.defaults)
        if a.vararg or a.kwarg or a.kwonlyargs or a.posonlyargs or n_defaults > 1:
            raise self.error("its parameters are its input arrays, then optionally a tunable with a default", a)
        params = [p.arg for p in a.args]
        tunable = params.pop() if n_defaults else None
        if not params:
            raise self.error("a kernel takes at least one input array", a)

        body = [s for s in f.body if not _is_docstring(s)]
        loops = [i for i, s in enumerate(body) if isinstance(s, ast.For)]
        if not loops:
            raise self.error("there is no `for` loop: a kernel is a loop nest over output tiles", f)
        at = loops[0]
        prologue, nest_stmt, rest = body[:at], body[at], body[at + 1 :]
        for s in prologue:
            if not isinstance(s, (ast.Assign, ast.Assert, ast.Pass, ast.AnnAssign)):
                raise self.error("before the loops come assignments and asserts only (shapes, tile sizes, outputs)", s)
        if len(rest) != 1 or not isinstance(rest[0], ast.Return):
            raise self.error("the loop nest must be followed by `return` of the outputs, and nothing else",
                             rest[0] if rest else nest_stmt)
        outputs = self._returned(rest[0])
        all_gathers = self._all_gathers(prologue, params)
        allocations, inplace = self._allocations(prologue, outputs, params)

        parallel, tile_body = self._parallel(nest_stmt)
        reductions, bodies, segments = self._tile(tile_body)
        stores = self._stores(segments, bodies, outputs)
        index_reads = self._index_reads(reductions, params)
        range_reads = self._range_reads([*parallel, *reductions], params)
        return Nest(self.name, self.filename, f, tuple(params), tunable, tuple(prologue), allocations, outputs,
                    tuple(parallel), tuple(reductions), tuple(bodies), tuple(segments), stores, all_gathers,
                    frozenset(index_reads), frozenset(range_reads), inplace)

    def _returned(self, ret: ast.Return) -> tuple[str, ...]:
        value = ret.value
        names = value.elts if isinstance(value, ast.Tuple) else [value]
        if value is None or not all(isinstance(n, ast.Name) for n in names):
            raise self.error("return the outputs by name (`return out` or `return a, b`)", ret)
        out = tuple(n.id for n in names)
        if len(set(out)) != len(out):
            raise self.error("each output is returned once", ret)
        return out

    def _all_gathers(self, prologue, params):
        found = []
        for s in prologue:
            if not (isinstance(s, ast.Assign) and isinstance(s.value, ast.Call)):
                continue
            func = s.value.func
            if not (isinstance(func, ast.Attribute) and func.attr == "all_gather") and not (
                isinstance(func, ast.Name) and func.id == "all_gather"):
                continue
            ok = (len(s.targets) == 1 and isinstance(s.targets[0], ast.Name) and len(s.value.args) == 2
                  and isinstance(s.value.args[0], ast.Name) and s.value.args[0].id in params
                  and isinstance(s.value.args[1], ast.Constant) and isinstance(s.value.args[1].value, str))
            if not ok:
                raise self.error("an all-gather is a statement of its own, `xs = autokernel.all_gather(x, \"axis\")`, "
                                 "on an input of the kernel", s)
            found.append(AllGather(s.targets[0].id, s.value.args[0].id, s.value.args[1].value, s))
        if len(found) > 1:
            raise self.error("a kernel gathers one input across chips", found[1].node)
        return tuple(found)

    def _allocations(self, prologue, outputs, params):
        allocations, inplace = {}, {}
        for s in prologue:
            targets = s.targets if isinstance(s, ast.Assign) else []
            for t in targets:
                names = [n.id for n in ast.walk(t) if isinstance(n, ast.Name)]
                for name in names:
                    if name in outputs:
                        if name in allocations or not isinstance(t, ast.Name):
                            raise self.error(f"allocate output `{name}` once, with jnp.zeros or jnp.full", s)
                        allocations[name] = s
        for name in outputs:
            if name not in allocations:
                raise self.error(f"output `{name}` must be allocated before the loops (jnp.zeros or jnp.full)",
                                 self.function)
            call = allocations[name].value
            if isinstance(call, ast.Name) and call.id in params:
                inplace[name] = call.id  # `out = q`: the output is the input updated (examples/ragged_paged_attention.py:131)
                continue
            ok = isinstance(call, ast.Call) and isinstance(call.func, ast.Attribute) and call.func.attr in ("zeros", "full")
            if not ok:
                raise self.error(f"allocate output `{name}` once, with jnp.zeros or jnp.full", allocations[name])
        return allocations, inplace

    def _loop(self, node: ast.For):
        if node.orelse:
            raise self.error("loops take no `else`", node)
        it = node.iter
        ok = (isinstance(node.target, ast.Name) and isinstance(it, ast.Call) and isinstance(it.func, ast.Name)
              and it.func.id == "range" and 1 <= len(it.args) <= 3 and not it.keywords)
        if not ok:
            raise self.error("loops are `for v in range(...)` over one variable", node)
        body = list(node.body)
        mask = None
        first = body[0]
        if isinstance(first, ast.If):
            if not (len(first.body) == 1 and isinstance(first.body[0], ast.Continue) and not first.orelse):
                raise self.error("the only `if` is a mask at the top of a loop's body: `if condition: continue`", first)
            mask, body = first.test, body[1:]
        if not body:
            raise self.error("the loop's body is empty", node)
        return Loop(node.target.id, tuple(it.args), mask, node), body

    def _parallel(self, node: ast.For):
        parallel = []
        while True:
            loop, body = self._loop(node)
            parallel.append(loop)
            if len(body) == 1 and isinstance(body[0], ast.For):
                node = body[0]
                continue
            return parallel, body

    def _tile(self, body):
        reductions, bodies, segments, current = [], [], [], []
        for s in body:
            if isinstance(s, ast.For):
                loop, inner = self._loop(s)
                for t in inner:
                    self._check_tile_stmt(t)
                reductions.append(loop)
                bodies.append(tuple(inner))
                segments.append(tuple(current))
                current = []
            else:
                self._check_tile_stmt(s)
                current.append(s)
        segments.append(tuple(current))
        return reductions, bodies, segments

    def _check_tile_stmt(self, s):
        if isinstance(s, ast.For):
            raise self.error("reduction loops don't nest", s)
        if isinstance(s, ast.If):
            raise self.error("the only `if` is a mask at the top of a loop's body: `if condition: continue`", s)
        if not isinstance(s, (ast.Assign, ast.AugAssign, ast.Pass, ast.With)):
            raise self.error("tile code is assignments (and `with jax.named_scope(...)` blocks) only", s)
        for n in ast.walk(s):
            if isinstance(n, ast.NamedExpr):
                raise self.error("tile code is assignments only (no `:=`)", s)

    def _stores(self, segments, bodies, outputs):
        stores = {}
        for group in (*segments, *bodies):
            for s in group:
                if not _is_store(s):
                    continue
                target = s.targets[0].id
                call = s.value
                base = call.func.value.value.value.id
                if base != target or target not in outputs:
                    raise self.error("an output is stored with `out = out.at[index].set(value)`", s)
                if target in stores:
                    raise self.error(f"output `{target}` is stored once per tile", s)
                stores[target] = Store(target, call.func.value.slice, call.args[0], s)
        for name in outputs:
            if name not in stores:
                raise self.error(f"output `{name}` is never stored: `{name} = {name}.at[index].set(value)`", self.function)
        return stores

    def _range_reads(self, reductions, params):
        reads = set()
        for loop in reductions:
            for arg in loop.args:
                for n in ast.walk(arg):
                    if isinstance(n, ast.Subscript) and isinstance(n.value, ast.Name) and n.value.id in params:
                        reads.add(n.value.id)
        return reads

    def _index_reads(self, reductions, params):
        reads = set()
        for loop in reductions:
            if loop.mask is None:
                continue
            for n in ast.walk(loop.mask):
                if isinstance(n, ast.Subscript) and isinstance(n.value, ast.Name) and n.value.id in params:
                    reads.add(n.value.id)
        return reads


def _is_docstring(s) -> bool:
    return isinstance(s, ast.Expr) and isinstance(s.value, ast.Constant) and isinstance(s.value.value, str)


def _is_store(s) -> bool:
    """`name = name.at[index].set(value)`"""
    if not (isinstance(s, ast.Assign) and len(s.targets) == 1 and isinstance(s.targets[0], ast.Name)):
        return False
    call = s.value
    return (isinstance(call, ast.Call) and isinstance(call.func, ast.Attribute) and call.func.attr == "set"
            and len(call.args) == 1 and isinstance(call.func.value, ast.Subscript)
            and isinstance(call.func.value.value, ast.Attribute) and call.func.value.value.attr == "at"
            and isinstance(call.func.value.value.value, ast.Name))
