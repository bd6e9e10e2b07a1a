"""A small NumPy-backed stand-in for the parts of `jax.numpy` / `jax.lax` the hot-path loop nests use, so that
`kernel.fn` and `kernel.reference` run on the CPU where JAX is not installed.

This is the CPU meaning of a loop nest (what the kernel must compute), never a path the kernels take: the
sm_100a kernels have no CPU fallback. Semantics follow JAX where the loop nests depend on them:

  * arrays are immutable; `out.at[idx].set(v)` returns a new array;
  * `a @ b` on bf16 operands rounds the result to bf16, as plain JAX does; inside `mxu_semantics()` it
    accumulates in f32 and returns f32 (i32 for integers), as `@` means in kernel code
    (src/autokernel/mxu.py:21-43) — that is how `kernel.reference` differs from `kernel.fn`;
  * Python scalars are weakly typed (`where(c, acc_f32, 0.0)` stays f32);
  * an index taken from an array clamps into range, as JAX's gathers do.

Use it as `from tilejax_b200.autokernel import jaxlike as jax` and `jnp = jax.numpy`.
"""

from __future__ import annotations

import contextlib
import threading
import types

import ml_dtypes
import numpy as np

_state = threading.local()


@contextlib.contextmanager
def mxu_semantics():
    """Within this block `@` accumulates in f32 (i32 for integers) and returns that type."""
    previous = getattr(_state, "mxu", False)
    _state.mxu = True
    try:
        yield
    finally:
        _state.mxu = previous


def _raw(x):
    return x.value if isinstance(x, Array) else x


def _wrap(x):
    return Array(x) if isinstance(x, np.ndarray) or isinstance(x, np.generic) else x


def _matmul(a, b):
    a, b = np.asarray(_raw(a)), np.asarray(_raw(b))
    if a.dtype != b.dtype:
        common = np.promote_types(a.dtype, b.dtype)
        a, b = a.astype(common), b.astype(common)
    integer = np.issubdtype(a.dtype, np.integer)
    acc = np.int32 if integer else np.float32
    out = np.matmul(a.astype(acc), b.astype(acc))
    if getattr(_state, "mxu", False):
        return Array(out)
    return Array(out.astype(a.dtype))


class _At:
    def __init__(self, array):
        self.array = array

    def __getitem__(self, idx):
        return _Setter(self.array, idx)


class _Setter:
    def __init__(self, array, idx):
        self.array, self.idx = array, idx

    def set(self, value):
        out = self.array.value.copy()
        value = np.asarray(_raw(value))
        items = self.idx if isinstance(self.idx, tuple) else (self.idx,)
        vectors = [n for n, item in enumerate(items) if _is_index_vector(item)]
        if vectors:
            # A vector of row indices (`autokernel.rows`): a store at an index out of range is dropped, as JAX drops
            # it. The vector's entries run along the value's axis that its place in the index selects.
            if len(vectors) != 1:
                raise NotImplementedError("one vector of indices per store")
            at = vectors[0]
            rows = np.asarray(_raw(items[at])).astype(np.int64)
            keep = (rows >= 0) & (rows < out.shape[at])
            axis = sum(1 for item in items[:at] if isinstance(item, slice))
            value = np.broadcast_to(value, _stored_shape(items, out.shape, rows.shape[0]))
            value = np.compress(keep, value, axis=axis)
            items = (*items[:at], rows[keep], *items[at + 1:])
        out[_index(tuple(items), out.shape)] = value.astype(out.dtype)
        return Array(out)


def _is_index_vector(item) -> bool:
    return isinstance(item, (Array, np.ndarray)) and np.asarray(_raw(item)).ndim == 1


def _stored_shape(items, shape, n):
    """The shape a store's value takes: slices keep their dimension, scalars drop it, the index vector gives n."""
    dims = []
    for dim, item in enumerate(items):
        if isinstance(item, slice):
            dims.append(len(range(*item.indices(shape[dim]))))
        elif _is_index_vector(item):
            dims.append(n)
    return tuple(dims) + tuple(shape[len(items):])


def _index(idx, shape):
    """Indices with array scalars turned into clamped ints, and index vectors clamped into range (JAX clamps
    gathers into range)."""
    items = idx if isinstance(idx, tuple) else (idx,)
    out = []
    for dim, item in enumerate(items):
        if isinstance(item, (Array, np.generic)) or (isinstance(item, np.ndarray) and item.ndim == 0):
            if np.asarray(_raw(item)).ndim == 1:
                out.append(np.clip(np.asarray(_raw(item)).astype(np.int64), 0, shape[dim] - 1))
                continue
            value = int(np.asarray(_raw(item)))
            out.append(int(np.clip(value, 0, shape[dim] - 1)))
        elif isinstance(item, np.ndarray) and item.ndim == 1:
            out.append(np.clip(item.astype(np.int64), 0, shape[dim] - 1))
        else:
            out.append(item)
    return tuple(out)


class Array:
    """An immutable n-d array (a NumPy array underneath) with the JAX methods the loop nests use."""

    __array_priority__ = 100

    def __init__(self, value):
        self.value = np.asarray(_raw(value))

    shape = property(lambda self: self.value.shape)
    dtype = property(lambda self: self.value.dtype)
    ndim = property(lambda self: self.value.ndim)
    size = property(lambda self: self.value.size)
    T = property(lambda self: Array(self.value.T))
    at = property(lambda self: _At(self))

    def __array__(self, dtype=None, copy=None):
        return self.value if dtype is None else self.value.astype(dtype)

    def astype(self, dtype):
        return Array(self.value.astype(dtype))

    def reshape(self, *shape):
        return Array(self.value.reshape(*shape))

    def transpose(self, *axes):
        return Array(self.value.transpose(*axes))

    def __getitem__(self, idx):
        return Array(self.value[_index(idx, self.value.shape)])

    def __matmul__(self, other):
        return _matmul(self, other)

    def __rmatmul__(self, other):
        return _matmul(other, self)

    def __bool__(self):
        return bool(self.value)

    def __int__(self):
        return int(self.value)

    def __float__(self):
        return float(self.value)

    def __index__(self):
        return int(self.value)

    def __len__(self):
        return len(self.value)

    def __repr__(self):
        return f"Array({self.value!r})"


def _binary(name, op):
    def forward(self, other):
        return Array(op(self.value, _weak(other, self.value.dtype)))

    def reverse(self, other):
        return Array(op(_weak(other, self.value.dtype), self.value))

    setattr(Array, f"__{name}__", forward)
    setattr(Array, f"__r{name}__", reverse)


def _weak(x, dtype):
    """A Python scalar takes the array's dtype (floats keep integer arrays integer only if integral)."""
    x = _raw(x)
    if isinstance(x, (bool, int, float)) and not isinstance(x, np.generic):
        if isinstance(x, float) and not np.issubdtype(dtype, np.floating) and dtype != ml_dtypes.bfloat16:
            return np.float32(x)
        return np.asarray(x).astype(dtype)
    return x


for _name, _op in (("add", np.add), ("sub", np.subtract), ("mul", np.multiply), ("truediv", np.divide),
                   ("floordiv", np.floor_divide), ("mod", np.mod), ("and", np.bitwise_and), ("or", np.bitwise_or),
                   ("lshift", np.left_shift), ("rshift", np.right_shift)):
    _binary(_name, _op)
for _name, _op in (("lt", np.less), ("le", np.less_equal), ("gt", np.greater), ("ge", np.greater_equal),
                   ("eq", np.equal), ("ne", np.not_equal)):
    setattr(Array, f"__{_name}__", (lambda op: lambda self, other: Array(op(self.value, _weak(other, self.value.dtype))))(_op))
Array.__neg__ = lambda self: Array(-self.value)
Array.__hash__ = None


def _lift(fn):
    def call(*args, **kwargs):
        args = [_raw(a) for a in args]
        kwargs = {k: _raw(v) for k, v in kwargs.items()}
        return _wrap(fn(*args, **kwargs))

    return call


def _where(cond, a, b):
    a, b = _raw(a), _raw(b)
    ref = a if isinstance(a, np.ndarray) else b
    if isinstance(ref, np.ndarray):
        a, b = _weak(a, ref.dtype), _weak(b, ref.dtype)
    return Array(np.where(_raw(cond), a, b))


def _dot(a, b, preferred_element_type=None, precision=None):
    a, b = np.asarray(_raw(a)), np.asarray(_raw(b))
    acc = np.dtype(preferred_element_type) if preferred_element_type is not None else None
    if acc is None:
        return _matmul(a, b)
    return Array(np.matmul(a.astype(acc), b.astype(acc)))


def _dot_general(a, b, dimension_numbers, preferred_element_type=None, precision=None):
    """jax.lax.dot_general: contract and batch the listed dimensions; the result is (batch..., a's free..., b's
    free...), accumulated in `preferred_element_type` (else as `@` would)."""
    (ca, cb), (ba, bb) = dimension_numbers
    a, b = np.asarray(_raw(a)), np.asarray(_raw(b))
    acc = np.dtype(preferred_element_type) if preferred_element_type is not None else None
    letters = iter("abcdefghijklmnopqrstuvwxyz")
    ia, ib = [None] * a.ndim, [None] * b.ndim
    for x, y in zip(ba, bb):
        ia[x] = ib[y] = next(letters)
    for x, y in zip(ca, cb):
        ia[x] = ib[y] = next(letters)
    for names in (ia, ib):
        for n, name in enumerate(names):
            if name is None:
                names[n] = next(letters)
    free_a = [ia[n] for n in range(a.ndim) if n not in ba and n not in ca]
    free_b = [ib[n] for n in range(b.ndim) if n not in bb and n not in cb]
    spec = f"{''.join(ia)},{''.join(ib)}->{''.join(ia[x] for x in ba)}{''.join(free_a)}{''.join(free_b)}"
    if acc is None:
        integer = np.issubdtype(a.dtype, np.integer)
        wide = np.int32 if integer else np.float32
        out = np.einsum(spec, a.astype(wide), b.astype(wide))
        return Array(out if getattr(_state, "mxu", False) else out.astype(np.promote_types(a.dtype, b.dtype)))
    return Array(np.einsum(spec, a.astype(acc), b.astype(acc)))


def _concatenate(arrays, axis=0):
    return Array(np.concatenate([np.asarray(_raw(a)) for a in arrays], axis=axis))


def _stack(arrays, axis=0):
    return Array(np.stack([np.asarray(_raw(a)) for a in arrays], axis=axis))


def _gelu(x, approximate=True):
    """jax.nn.gelu: the tanh form by default, in x's own precision."""
    x = np.asarray(_raw(x))
    if not approximate:
        raise NotImplementedError("the exact (erf) GELU is not used by the hot-path loop nests")
    one, half = x.dtype.type(1), x.dtype.type(0.5)
    cubic = x + x.dtype.type(0.044715) * x * x * x
    return Array((half * x * (one + np.tanh(x.dtype.type(np.sqrt(2.0 / np.pi)) * cubic))).astype(x.dtype))


def _full(shape, value, dtype=None):
    return Array(np.full(shape, _raw(value), dtype or np.float32))


def _bitcast_convert_type(x, dtype):
    """jax.lax.bitcast_convert_type: the same bits as another type. Equal widths keep the shape; to a type twice as
    wide the last dimension (of two) goes away, first element in the low half; to one half as wide a last dimension
    of two appears."""
    x, dtype = np.ascontiguousarray(_raw(x)), np.dtype(dtype)
    if x.dtype.itemsize == dtype.itemsize:
        return Array(x.view(dtype))
    if x.dtype.itemsize * 2 == dtype.itemsize:
        if x.shape[-1] != 2:
            raise ValueError("bitcast to a type twice as wide needs a last dimension of 2")
        return Array(x.view(dtype)[..., 0])
    if x.dtype.itemsize == dtype.itemsize * 2:
        return Array(x[..., None].view(dtype))
    raise ValueError(f"bitcast from {x.dtype} to {dtype}")


def _broadcasted_iota(dtype, shape, dimension):
    index = np.arange(shape[dimension], dtype=dtype)
    view = [1] * len(shape)
    view[dimension] = shape[dimension]
    return Array(np.broadcast_to(index.reshape(view), shape).copy())


numpy = types.SimpleNamespace(
    float32=np.float32, float64=np.float64, int32=np.int32, int8=np.int8, uint32=np.uint32, bool_=np.bool_,
    bfloat16=ml_dtypes.bfloat16, float16=np.float16, ndarray=Array, inf=np.inf, nan=np.nan, pi=np.pi,
    asarray=lambda x, dtype=None: Array(np.asarray(_raw(x), dtype)),
    array=lambda x, dtype=None: Array(np.asarray(_raw(x), dtype)),
    zeros=lambda shape, dtype=None: Array(np.zeros(shape, dtype or np.float32)),
    ones=lambda shape, dtype=None: Array(np.ones(shape, dtype or np.float32)),
    full=_full,
    where=_where, exp=_lift(np.exp), maximum=_lift(np.maximum), minimum=_lift(np.minimum),
    max=_lift(np.max), sum=_lift(np.sum), tile=_lift(np.tile), concatenate=_concatenate,
    arange=_lift(np.arange), clip=_lift(np.clip), dot=_dot, matmul=_matmul, tril=_lift(np.tril),
    abs=_lift(np.abs), logical_not=_lift(np.logical_not), sqrt=_lift(np.sqrt), mean=_lift(np.mean),
    square=_lift(np.square), transpose=_lift(np.transpose), reshape=_lift(np.reshape), stack=_stack,
    tanh=_lift(np.tanh), swapaxes=_lift(np.swapaxes), uint16=np.uint16,
)
nn = types.SimpleNamespace(gelu=_gelu)
lax = types.SimpleNamespace(broadcasted_iota=_broadcasted_iota, bitcast_convert_type=_bitcast_convert_type,
                            dot_general=_dot_general,
                            rsqrt=_lift(lambda x: (1.0 / np.sqrt(np.asarray(x))).astype(np.asarray(x).dtype)))


def to_numpy(x) -> np.ndarray:
    return np.asarray(_raw(x))
