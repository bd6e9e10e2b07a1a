"""The `autokernel` front end on the sm_100a backend: Python loop nests over tiles, run by hand-written CUDA.

    import tilejax_b200.autokernel as autokernel
    from tilejax_b200.autokernel import jaxlike as jax     # where JAX itself is not installed
    jnp = jax.numpy

Same names as the reference package (src/autokernel/__init__.py:32-50): `kernel`, `Kernel`, `Lowered`, `tunable`,
`choice`, `Config`, `Pipeline`, `Trial`, `Tuning`, `KernelProfile`, `profile`, `KernelError`, `all_gather`, `pairs`,
`unpairs`, `rows`.
"""

from .api import Kernel, Lowered, compare, kernel
from .collective import all_gather
from .errors import KernelError
from .profiling import KernelProfile, profile
from .ragged import pairs, rows, unpairs
from .tunable import choice, tunable
from .tune import Config, Pipeline, Trial, Tuning

__all__ = ["Config", "Kernel", "KernelError", "KernelProfile", "Lowered", "Pipeline", "Trial", "Tuning", "all_gather",
           "choice", "compare", "kernel", "pairs", "profile", "rows", "tunable", "unpairs"]
