"""CPU oracle for the step-loop hot path: a NumPy restatement of the reference's semantics (RKKatakam/tilejax,
package `autokernel`), function by function, each citing the reference lines it follows.

THIS IS TEST INFRASTRUCTURE, NOT A PRODUCT PATH. Only the tests, the smoke check and the benchmark's
CPU-baseline leg may import it; nothing under `tilejax_b200/` does, and the CUDA kernels never route through it.

Parity status. The reference is pure Python on JAX 0.11.2 / jaxlib 0.11.2 (third-party, pinned in its uv.lock),
which cannot be imported where this was written, so the oracle could not be run against the reference itself.
  * Integer work (static tile / step tables, device step tables, schedule counts) is PINNED: `tests/` checks it
    against every known answer the reference's own tests hold for this path (tests/test_api.py:20-30,
    tests/test_examples.py:56-63 and :91-95, tests/test_schedule.py:17-51 and :189-221, tests/test_index_arrays.py:57-72,
    tests/test_decode.py:195-199, tests/test_collective.py:98-124).
  * Floating-point element values are PARITY UNPINNED at the JAX boundary: the reference's tests hold no stored
    tensors, only tolerances against float64 NumPy (tests/test_examples.py:27-101, tests/test_decode.py:62-76,
    :163-220). The oracle restates the arithmetic rule (bf16 operands, f32 accumulation per block in order, P
    rounded to bf16 before P @ v) and is itself checked against independent float64 formulas, as those tests do.
"""

from .attention import causal_attention_f64, causal_attention_ref
from .compare import compare
from .decode import (
    gqa_decode_ref,
    mla_decode_f64,
    mla_decode_ref,
    paged_gqa_decode_f64,
    paged_gqa_decode_ref,
    to_pages,
)
from .matmul import causal_matmul_ref, collective_row_order, matmul_ref
from .rmsnorm import rmsnorm_matmul_f64, rmsnorm_matmul_ref
from .rpa import (rpa_decode_f64, rpa_decode_ref, rpa_inputs, rpa_prefill_f64, rpa_prefill_ref, rpa_prefill_tiles,
                  rpa_write_ref, rpa_write_runs)
from .steps import (
    attention_step_tables,
    causal_tile_tables,
    device_step_tables,
    lengths_runs,
    walk_nest,
)

__all__ = [
    "attention_step_tables",
    "causal_attention_f64",
    "causal_attention_ref",
    "causal_matmul_ref",
    "causal_tile_tables",
    "collective_row_order",
    "compare",
    "device_step_tables",
    "gqa_decode_ref",
    "lengths_runs",
    "matmul_ref",
    "mla_decode_f64",
    "mla_decode_ref",
    "paged_gqa_decode_f64",
    "paged_gqa_decode_ref",
    "rmsnorm_matmul_f64",
    "rmsnorm_matmul_ref",
    "rpa_decode_f64",
    "rpa_decode_ref",
    "rpa_inputs",
    "rpa_prefill_f64",
    "rpa_prefill_ref",
    "rpa_prefill_tiles",
    "rpa_write_ref",
    "rpa_write_runs",
    "to_pages",
    "walk_nest",
]
