"""Tunables: the one object a kernel hands over to be optimised (the reference's src/autokernel/tunable.py).

    @autokernel.tunable
    class MatmulTiles:
        tm: int = autokernel.choice(128, 256, 512, default=512)

A tunable is a frozen dataclass whose every field lists its candidate values; `neighbours` are the tunables one
step away (one field moved to the next or previous of its choices). Where JAX is importable the class is also
registered as a pytree without leaves, so it stays static under `jax.jit`, as in the reference.
"""

from __future__ import annotations

import dataclasses
from collections.abc import Iterator
from typing import Any

_CHOICES = "autokernel.choices"


def choice(*values: Any, default: Any = None) -> Any:
    """A tunable field's candidate values, in order; its default is `default`, else the first value."""
    if not values:
        raise ValueError("a tunable field needs at least one value to choose from")
    default = values[0] if default is None else default
    if default not in values:
        raise ValueError(f"the default {default!r} isn't one of the choices {values}")
    return dataclasses.field(default=default, metadata={_CHOICES: tuple(values)})


def tunable(cls: type) -> type:
    """Make `cls` a tunable: a frozen dataclass whose fields are all declared with `choice(...)`."""
    cls = dataclasses.dataclass(frozen=True)(cls)
    fields = dataclasses.fields(cls)
    for f in fields:
        if _CHOICES not in f.metadata:
            raise TypeError(f"{cls.__name__}.{f.name}: declare tunable fields with autokernel.choice(...)")
    cls.__autokernel_tunable__ = True
    try:  # static under jax.jit where JAX exists
        import jax

        jax.tree_util.register_dataclass(cls, data_fields=[], meta_fields=[f.name for f in fields])
    except Exception:
        pass
    return cls


def is_tunable(value: Any) -> bool:
    return getattr(type(value), "__autokernel_tunable__", False) and not isinstance(value, type)


def choices(value: Any) -> dict[str, tuple[Any, ...]]:
    return {f.name: f.metadata[_CHOICES] for f in dataclasses.fields(value)}


def neighbours(value: Any) -> Iterator[Any]:
    for name, options in choices(value).items():
        current = getattr(value, name)
        at = options.index(current) if current in options else None
        for step in (1, -1):
            if at is not None and 0 <= at + step < len(options):
                yield dataclasses.replace(value, **{name: options[at + step]})
