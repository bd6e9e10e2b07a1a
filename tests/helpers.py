"""Conversions between NumPy (ml_dtypes bfloat16) and CUDA tensors, and the tolerance rule, for the tests."""

import numpy as np
import torch

from tilejax_b200.synthetic import bf16_dtype

BF16 = bf16_dtype()


def to_device(a: np.ndarray) -> torch.Tensor:
    a = np.ascontiguousarray(a)
    if a.dtype == BF16:
        return torch.from_numpy(a.view(np.uint16)).view(torch.bfloat16).cuda()
    return torch.from_numpy(a).cuda()


def to_host(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy().view(BF16)
    return t.numpy()


def f64(a) -> np.ndarray:
    return np.asarray(a).astype(np.float64)


def rand_bf16(shape, seed, scale=1.0) -> np.ndarray:
    x = np.random.default_rng(seed).standard_normal(shape, dtype=np.float32) * np.float32(scale)
    return x.astype(BF16)


def make_function(source: str, name: str = "f", **names):
    """The function `name` of `source` (dedented), compiled under a file name `inspect` can read back, with the
    NumPy-backed `jax` / `jnp` stand-ins and `autokernel` in scope — as the reference's tests build their kernels
    from source strings (tests/helpers.py `make_kernel`)."""
    import linecache
    import textwrap

    import tilejax_b200.autokernel as autokernel
    from tilejax_b200.autokernel import jaxlike

    source = textwrap.dedent(source).lstrip("\n")
    filename = f"<test kernel {abs(hash(source))}>"
    linecache.cache[filename] = (len(source), None, source.splitlines(keepends=True), filename)
    ns = {"jnp": jaxlike.numpy, "jax": jaxlike, "autokernel": autokernel, **names}
    exec(compile(source, filename, "exec"), ns)
    return ns[name]


def make_kernel(source: str, name: str = "f", **names):
    import tilejax_b200.autokernel as autokernel

    return autokernel.kernel(make_function(source, name, **names))


def spec(*shape, dtype=None):
    from tilejax_b200.autokernel.plan import Spec

    return Spec(tuple(shape), np.dtype(BF16 if dtype is None else dtype))
