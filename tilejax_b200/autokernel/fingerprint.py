"""Structural identity of a loop nest's code: what lets the recogniser be strict about attention and decode.

The matmul family is matched statement by statement (plan._match_gemm_tile_code). The attention and decode families
have bodies of a dozen statements and helper functions; they are accepted only if their code — the kernel function
and every helper it calls — is, modulo the names of local variables and of the array modules, one of the forms this
backend's kernels were written and tested against (recognised.py). A different mask value, an extra scale, a
softmax without the bf16 rounding of P, a helper that does something else: each changes the fingerprint and is
refused with a KernelError instead of being sent to a fixed kernel that computes something else.

Canonical form of a function: its body without the docstring, with
  * local names (parameters, assigned names, loop variables) numbered in order of first appearance;
  * global names that hold numbers or strings replaced by their values (LANES -> 128, MASK_VALUE -> -1e30); a
    float the function closes over (the softmax scale of `make_decode(sm_scale)`) stays a name: it is an argument;
  * array modules and namespaces (`jnp`, `jax`, `jax.lax`, `autokernel`) collapsed, so that `jnp.where`,
    `jax.numpy.where` and `np.where` read alike;
  * helper functions replaced by a marker, their own canonical forms appended in order of first call.
The fingerprint is the SHA-256 of that text.

    python -m tilejax_b200.autokernel.fingerprint [reference/examples]   # rewrites recognised.py
"""

from __future__ import annotations

import ast
import builtins
import hashlib
import inspect
import textwrap
import types
from collections.abc import Callable
from typing import Any

_MODULE = "M"


def _source_tree(fn: Callable) -> ast.FunctionDef:
    tree = ast.parse(textwrap.dedent(inspect.getsource(fn)))
    node = tree.body[0]
    if not isinstance(node, ast.FunctionDef):
        raise TypeError(f"{fn!r} is not defined with `def`")
    return node


def _namespace(fn: Callable) -> dict[str, Any]:
    ns = dict(getattr(fn, "__globals__", {}))
    if getattr(fn, "__closure__", None):
        ns.update({n: c.cell_contents for n, c in zip(fn.__code__.co_freevars, fn.__closure__, strict=True)})
    return ns


def _is_namespace(value: Any) -> bool:
    return isinstance(value, (types.ModuleType, types.SimpleNamespace))


class _Canonical(ast.NodeTransformer):
    def __init__(self, fn: Callable, function: ast.FunctionDef):
        self.ns = _namespace(fn)
        # A float the function closes over is a parameter of the kernel (`make_decode(sm_scale)`,
        # examples/ragged_paged_attention.py:110-149), not part of its form: every scale is the same code.
        self.closed_floats = {n for n, c in zip(getattr(fn, "__code__", None).co_freevars if hasattr(fn, "__code__") else (),
                                                getattr(fn, "__closure__", None) or ())
                              if isinstance(c.cell_contents, float)}
        self.locals: dict[str, str] = {}
        self.helpers: list[Callable] = []
        assigned = {a.arg for a in function.args.args}
        for node in ast.walk(function):
            if isinstance(node, ast.Name) and isinstance(node.ctx, ast.Store):
                assigned.add(node.id)
        self.assigned = assigned

    def _local(self, name: str) -> str:
        return self.locals.setdefault(name, f"v{len(self.locals)}")

    def _resolve(self, node: ast.expr) -> tuple[bool, Any]:
        """(resolved?, object) for a Name / Attribute chain rooted at a global."""
        if isinstance(node, ast.Name):
            if node.id in self.assigned:
                return False, None
            if node.id in self.ns:
                return True, self.ns[node.id]
            if hasattr(builtins, node.id):
                return True, getattr(builtins, node.id)
            return False, None
        if isinstance(node, ast.Attribute):
            ok, base = self._resolve(node.value)
            if ok and _is_namespace(base) and hasattr(base, node.attr):
                return True, getattr(base, node.attr)
        return False, None

    def visit_Name(self, node: ast.Name) -> ast.AST:
        if node.id in self.assigned:
            return ast.Name(self._local(node.id), ast.Load())
        if node.id in self.closed_floats:
            return ast.Name("closed_float", ast.Load())
        ok, value = self._resolve(node)
        if not ok:
            return ast.Name(f"?{node.id}", ast.Load())
        if isinstance(value, (bool, int, float, str)) or value is None:
            return ast.Constant(value)
        if _is_namespace(value):
            return ast.Name(_MODULE, ast.Load())
        if isinstance(value, types.FunctionType) and getattr(value, "__module__", "") != "builtins":
            if value not in self.helpers:
                self.helpers.append(value)
            return ast.Name(f"helper{self.helpers.index(value)}", ast.Load())
        if isinstance(value, type) or callable(value):
            return ast.Name(getattr(value, "__name__", node.id), ast.Load())
        return ast.Name(f"?{node.id}", ast.Load())

    def visit_Attribute(self, node: ast.Attribute) -> ast.AST:
        ok, value = self._resolve(node)
        if ok:
            if _is_namespace(value):
                return ast.Name(_MODULE, ast.Load())
            if isinstance(value, (bool, int, float, str)):
                return ast.Constant(value)
        return ast.Attribute(self.visit(node.value), node.attr, ast.Load())

    def visit_arg(self, node: ast.arg) -> ast.AST:
        return ast.arg(self._local(node.arg), None)

    def visit_Constant(self, node: ast.Constant) -> ast.AST:
        return ast.Constant(node.value)


def canonical(fn: Callable) -> tuple[str, list[Callable]]:
    """(canonical text of `fn`'s parameters and body, the helper functions it calls in order of first call)."""
    function = _source_tree(fn)
    body = list(function.body)
    if body and isinstance(body[0], ast.Expr) and isinstance(body[0].value, ast.Constant) and isinstance(body[0].value.value, str):
        body = body[1:]
    walker = _Canonical(fn, function)
    params = [walker._local(a.arg) for a in function.args.args]
    text = [f"def({', '.join(params)})"]
    for stmt in body:
        text.append(ast.dump(walker.visit(stmt), annotate_fields=False))
    return "\n".join(text), walker.helpers


def fingerprint(fn: Callable) -> str:
    """SHA-256 (hex) of `fn`'s canonical form and of every helper's, helpers of helpers included."""
    fn = inspect.unwrap(getattr(fn, "fn", fn))
    seen: list[Callable] = []
    queue = [fn]
    parts: list[str] = []
    while queue:
        current = queue.pop(0)
        if current in seen:
            continue
        seen.append(current)
        text, helpers = canonical(current)
        parts.append(text)
        queue.extend(h for h in helpers if h not in seen)
    return hashlib.sha256("\n--\n".join(parts).encode()).hexdigest()


# ------------------------------------------------------------------------------------------ maintaining recognised.py


def load_example(path: str, names: dict[str, Any]) -> dict[str, Any]:
    """Execute the top-level constants, classes and functions of an example file (not its imports, not its `main`)
    with `names` as its globals; definitions that need something else are skipped. The code objects keep the
    file's name and line numbers, so `inspect` reads the functions' source from the file itself."""
    tree = ast.parse(open(path).read(), path)
    ns = dict(names)
    for node in tree.body:
        if not isinstance(node, (ast.Assign, ast.AnnAssign, ast.ClassDef, ast.FunctionDef)):
            continue
        try:
            exec(compile(ast.Module([node], []), path, "exec", dont_inherit=True), ns)
        except Exception:
            continue
    return ns


def _write(path: str, found: dict[str, dict[str, str]]) -> None:
    lines = ['"""Fingerprints (fingerprint.py) of the loop nests the attention and decode kernels accept, by family.',
             "",
             "Written by `python -m tilejax_b200.autokernel.fingerprint [reference/examples]`: the forms in this package's",
             "kernels.py and, when the reference's example files are at hand, the forms in examples/causal_attention.py,",
             'examples/decode.py, examples/rmsnorm_matmul.py, examples/attention_block.py and',
             'examples/ragged_paged_attention.py (lane-replicated row statistics, block-diagonal queries, paired words).',
             'Do not edit by hand."""',
             "", "RECOGNISED: dict[str, dict[str, str]] = {"]
    for family in sorted(found):
        lines.append(f'    "{family}": {{')
        for digest, label in sorted(found[family].items(), key=lambda kv: kv[1]):
            lines.append(f'        "{digest}": "{label}",')
        lines.append("    },")
    lines.append("}")
    open(path, "w").write("\n".join(lines) + "\n")


def main(argv: list[str]) -> None:
    import os

    import tilejax_b200.autokernel as autokernel
    from tilejax_b200.autokernel import jaxlike, kernels

    families = {"attention": ["causal_attention"], "decode": ["paged_gqa_decode", "gqa_decode"], "mla": ["mla_decode"],
                "rmsnorm": ["rmsnorm_matmul"], "attention_block": ["attention_block"], "rpa_write": ["rpa_write"]}
    # Kernels made by a function of the softmax scale: (family, the maker's name here, the maker's name there, file).
    makers = [("rpa_decode", "make_rpa_decode", "make_decode", "ragged_paged_attention.py"),
              ("rpa_prefill", "make_rpa_prefill", "make_prefill", "ragged_paged_attention.py")]
    found: dict[str, dict[str, str]] = {f: {} for f in [*families, *(m[0] for m in makers)]}
    for family, names in families.items():
        for name in names:
            found[family][fingerprint(getattr(kernels, name))] = f"tilejax_b200/autokernel/kernels.py {name}"
    for family, here, _, _ in makers:
        found[family][fingerprint(getattr(kernels, here)(1.0))] = f"tilejax_b200/autokernel/kernels.py {here}"
    if len(argv) > 1:
        stand_ins = {"jax": jaxlike, "jnp": jaxlike.numpy, "autokernel": autokernel, "__name__": "example"}
        for file in ("causal_attention.py", "decode.py", "rmsnorm_matmul.py", "attention_block.py",
                     "ragged_paged_attention.py"):
            ns = load_example(os.path.join(argv[1], file), stand_ins)
            for family, names in families.items():
                for name in names:
                    if name in ns:
                        found[family][fingerprint(ns[name])] = f"examples/{file} {name}"
        for family, _, there, file in makers:
            ns = load_example(os.path.join(argv[1], file), stand_ins)
            if there in ns:
                found[family][fingerprint(ns[there](1.0))] = f"examples/{file} {there}"
    _write(os.path.join(os.path.dirname(__file__), "recognised.py"), found)
    for family, entries in found.items():
        for digest, label in entries.items():
            print(family, digest[:16], label)


if __name__ == "__main__":
    import sys

    main(sys.argv)
