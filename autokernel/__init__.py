"""`import autokernel`: the reference package's import name (src/autokernel/__init__.py) on the sm_100a backend.

Everything lives in `tilejax_b200.autokernel`; this package re-exports its public names and makes its modules
importable under the reference's paths (`autokernel.tune`, `autokernel.tunable`, `autokernel.schedule`,
`autokernel.profiling`, `autokernel.errors`, `autokernel.api`, `autokernel.plan`, `autokernel.parse`), so code
written against the reference — `@autokernel.kernel`, `autokernel.choice`, `from autokernel.tune import search` —
imports unchanged. Where JAX is not installed, `autokernel.jaxlike` is the NumPy-backed stand-in for the few
`jax` / `jax.numpy` calls the loop nests make.
"""

import sys as _sys

import tilejax_b200.autokernel as _impl
from tilejax_b200 import schedule as _schedule
from tilejax_b200.autokernel import (  # noqa: F401
    Config,
    Kernel,
    KernelError,
    KernelProfile,
    Lowered,
    Pipeline,
    Trial,
    Tuning,
    all_gather,
    api,
    choice,
    collective,
    compare,
    errors,
    jaxlike,
    kernel,
    parse,
    plan,
    profile,
    profiling,
    tunable,
    tune,
)

__all__ = list(_impl.__all__)

for _name, _module in (("api", api), ("collective", collective), ("errors", errors), ("jaxlike", jaxlike),
                       ("parse", parse), ("plan", plan), ("profiling", profiling), ("schedule", _schedule),
                       ("tune", tune), ("tunable", _sys.modules["tilejax_b200.autokernel.tunable"])):
    _sys.modules[f"{__name__}.{_name}"] = _module
schedule = _schedule
del _name, _module
