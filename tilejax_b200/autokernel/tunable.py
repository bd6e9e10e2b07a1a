"""Tunables: the one object a kernel hands over to be optimised (the role of the reference's
src/autokernel/tunable.py; same names, same behaviour, its own mechanism).

    @autokernel.tunable
    class MatmulTiles:
        tm: int = autokernel.choice(128, 256, 512, default=512)

`choice(...)` leaves a `Choice` marker in the class body; `tunable` turns the class into a frozen dataclass whose
field defaults are the markers' defaults and keeps every field's candidate values in one table on the class. The
tunables "one step away" from a value — what the tuner's hill climb walks — move one field to the next or the
previous entry of its candidates. Where JAX is importable the class is also registered as a pytree without leaves,
so it stays static under `jax.jit`, as in the reference.
"""

from __future__ import annotations

import dataclasses
from collections.abc import Iterator
from typing import Any

_TABLE = "__autokernel_choices__"  # class attribute: {field name: its candidate values, in order}


@dataclasses.dataclass(frozen=True)
class Choice:
    """What `choice(...)` leaves in a class body until `tunable` picks it up."""

    values: tuple[Any, ...]
    default: Any


def choice(*values: Any, default: Any = None) -> Any:
    """A tunable field's candidate values, in order; its default is `default`, else the first value."""
    if len(values) == 0:
        raise ValueError("a tunable field needs at least one value to choose from")
    picked = default if default is not None else values[0]
    if picked not in values:
        raise ValueError(f"the default {picked!r} isn't one of the choices {values}")
    return Choice(tuple(values), picked)


def tunable(cls: type) -> type:
    """Make `cls` a tunable: a frozen dataclass whose fields are all declared with `choice(...)`."""
    table: dict[str, tuple[Any, ...]] = {}
    for name in getattr(cls, "__annotations__", {}):
        marker = cls.__dict__.get(name)
        if not isinstance(marker, Choice):
            raise TypeError(f"{cls.__name__}.{name}: declare tunable fields with autokernel.choice(...)")
        table[name] = marker.values
        setattr(cls, name, marker.default)  # what the dataclass machinery sees: a plain default
    made = dataclasses.dataclass(frozen=True)(cls)
    setattr(made, _TABLE, table)
    try:  # static under jax.jit where JAX exists: no leaves, every field part of the tree's structure
        import jax

        jax.tree_util.register_dataclass(made, data_fields=[], meta_fields=list(table))
    except Exception:
        pass
    return made


def is_tunable(value: Any) -> bool:
    """Is `value` an instance (not the class itself) of an `@autokernel.tunable` class?"""
    return not isinstance(value, type) and hasattr(type(value), _TABLE)


def choices(value: Any) -> dict[str, tuple[Any, ...]]:
    """Each field of a tunable and the values it may take."""
    return dict(getattr(type(value), _TABLE))


def neighbours(value: Any) -> Iterator[Any]:
    """The tunables one step away from `value`, field by field: the next candidate, then the previous one. A field
    whose current value is not among its candidates stays where it is."""
    for name, candidates in choices(value).items():
        here = getattr(value, name)
        if here not in candidates:
            continue
        position = candidates.index(here)
        for moved in (position + 1, position - 1):
            if moved in range(len(candidates)):
                yield dataclasses.replace(value, **{name: candidates[moved]})
