"""The jax.ffi binding of the C ABI: the seam the reference's front end needs to run these kernels from jitted JAX
code — `Kernel.lowered(...).entry(*inputs)` (src/autokernel/api.py:258-266) becomes a `jax.ffi.ffi_call`.

Needs JAX with a CUDA backend, and libtilejax_b200_ffi.so (tilejax_b200/csrc/tjx_xla_ffi.cc, built by
`python -m tilejax_b200.csrc.build --ffi` where `jax.ffi.include_dir()` exists). Where either is missing `available()`
is False and everything else raises; the ctypes path (tilejax_b200.ops) is the one that is always there and always
tested. Nothing here computes anything: each function only describes a custom call.
"""

from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

from . import schedule as _schedule
from ._lib import LIBRARY

FFI_LIBRARY = Path(__file__).resolve().parent / "libtilejax_b200_ffi.so"
TARGETS = {"tjx_build_steps": "TjxBuildSteps", "tjx_gemm": "TjxGemm", "tjx_causal_attention": "TjxCausalAttention",
           "tjx_paged_gqa_decode": "TjxPagedGqaDecode", "tjx_rmsnorm_gemm": "TjxRmsnormGemm",
           "tjx_attention_block": "TjxAttentionBlock", "tjx_mla_decode": "TjxMlaDecode",
           "tjx_ragged_paged_attention": "TjxRaggedPagedAttention"}
_registered = False


def available() -> bool:
    """Is JAX importable and has the handler library been built?"""
    try:
        import jax  # noqa: F401
    except Exception:
        return False
    return FFI_LIBRARY.exists()


def register() -> None:
    """Load the handler library and register its targets with XLA for the CUDA platform (once per process)."""
    global _registered
    if _registered:
        return
    if not available():
        raise RuntimeError("the XLA FFI binding needs JAX and libtilejax_b200_ffi.so "
                           "(python -m tilejax_b200.csrc.build --ffi); use tilejax_b200.ops otherwise")
    import jax

    ctypes.CDLL(str(LIBRARY), mode=ctypes.RTLD_GLOBAL)  # the C ABI the handlers call into
    handlers = ctypes.CDLL(str(FFI_LIBRARY))
    for target, symbol in TARGETS.items():
        jax.ffi.register_ffi_target(target, jax.ffi.pycapsule(getattr(handlers, symbol)), platform="CUDA")
    _registered = True


def _i32(values):
    import jax.numpy as jnp

    return jnp.asarray(np.asarray(values, np.int32))


def gemm(x, y, tm: int, tn: int, tk: int, *, causal: bool = False, out_dtype=None, y_transposed: bool = False,
         stages: int = 0, tables: dict | None = None):
    """out = x @ y through `tjx_gemm`; `tables` holds the schedule's tile_i / tile_j / fill_i / fill_j (NumPy)."""
    import jax
    import jax.numpy as jnp

    register()
    tables = tables or {}
    M, N = x.shape[0], (y.shape[0] if y_transposed else y.shape[1])
    empty = np.zeros(0, np.int32)
    args = [_i32(tables.get(name, empty)) for name in ("tile_i", "tile_j", "fill_i", "fill_j")]
    call = jax.ffi.ffi_call("tjx_gemm", jax.ShapeDtypeStruct((M, N), out_dtype or jnp.bfloat16))
    return call(x, y, *args, tm=np.int32(tm), tn=np.int32(tn), tk=np.int32(tk), stages=np.int32(stages),
                causal=np.int32(causal), y_transposed=np.int32(y_transposed))


def causal_matmul(x, y, tm: int = 512, tn: int = 512, tk: int = 512):
    M, K = x.shape
    N = y.shape[1]
    tm, tn, tk = min(tm, M), min(tn, N), min(tk, K)
    return gemm(x, y, tm, tn, tk, causal=True, tables=_schedule.causal_matmul_schedule(M, N, K, tm, tn, tk).tables)


def causal_attention(q, k, v, block_q: int = 512, block_kv: int = 512):
    import jax

    register()
    B, H, S, D = q.shape
    bq, bk = min(block_q, S), min(block_kv, S)
    sch = _schedule.causal_attention_schedule(B, H, S, bq, bk)
    if sch.step_tables:
        tile, code = sch.tables["step_tile"], sch.tables["step_code"]
    else:
        nq, nk = S // bq, S // bk
        tile, block = np.repeat(np.arange(nq, dtype=np.int32), nk), np.tile(np.arange(nk, dtype=np.int32), nq)
        code = (block << _schedule.CODE_SHIFT) | ((block == 0) << 1) | (block == nk - 1)
    call = jax.ffi.ffi_call("tjx_causal_attention", jax.ShapeDtypeStruct(q.shape, q.dtype))
    return call(q, k, v, _i32(tile), _i32(code), block_q=np.int32(bq), block_kv=np.int32(bk),
                pattern_tiles=np.int32(S // bq))


def paged_gqa_decode(q, k_pages, v_pages, block_tables, lengths):
    """Returns (out, step_tile, step_code, step_count): the tables the call built on the device ride along as extra
    results, the scratch as a last one that is dropped here."""
    import jax
    import jax.numpy as jnp

    register()
    B, T, H, D = q.shape
    pages = block_tables.shape[1]
    lib = ctypes.CDLL(str(LIBRARY))
    lib.tjx_paged_gqa_decode_workspace_bytes.restype = ctypes.c_size_t
    scratch = int(lib.tjx_paged_gqa_decode_workspace_bytes(B, T, H, D, pages)) + 256
    results = (jax.ShapeDtypeStruct(q.shape, q.dtype), jax.ShapeDtypeStruct((B * pages,), jnp.int32),
               jax.ShapeDtypeStruct((B * pages,), jnp.int32), jax.ShapeDtypeStruct((1,), jnp.int32),
               jax.ShapeDtypeStruct((B + 1,), jnp.int32), jax.ShapeDtypeStruct((scratch,), jnp.uint8))
    out, tile, code, count, _, _ = jax.ffi.ffi_call("tjx_paged_gqa_decode", results)(q, k_pages, v_pages, block_tables, lengths)
    return out, tile, code, count


def _scratch(symbol: str, *sizes: int) -> int:
    lib = ctypes.CDLL(str(LIBRARY))
    fn = getattr(lib, symbol)
    fn.restype = ctypes.c_size_t
    return int(fn(*sizes)) + 256


def rmsnorm_matmul(x, gamma, w, tm: int = 512, tn: int = 512, tk: int = 512, eps: float = 1e-6):
    """rmsnorm(x) @ w through `tjx_rmsnorm_gemm` (examples/rmsnorm_matmul.py:31-47)."""
    import jax
    import jax.numpy as jnp

    register()
    (M, D), N = x.shape, w.shape[1]
    results = (jax.ShapeDtypeStruct((M, N), x.dtype),
               jax.ShapeDtypeStruct((_scratch("tjx_rmsnorm_gemm_workspace_bytes", M, D),), jnp.uint8))
    out, _ = jax.ffi.ffi_call("tjx_rmsnorm_gemm", results)(x, gamma, w, tm=np.int32(min(tm, M)), tn=np.int32(min(tn, N)),
                                                           tk=np.int32(min(tk, D)), eps=np.float32(eps))
    return out


def attention_block(q, k, v, gamma, w_up, w_down, block_q: int = 256, block_kv: int = 256, eps: float = 1e-6):
    """The two-phase attention block through `tjx_attention_block` (examples/attention_block.py:49-85)."""
    import jax
    import jax.numpy as jnp

    register()
    B, H, S, Dh = q.shape
    bq, bk = min(block_q, S), min(block_kv, S)
    sch = _schedule.causal_attention_schedule(B, H, S, bq, bk)
    if sch.step_tables:
        tile, code = sch.tables["step_tile"], sch.tables["step_code"]
    else:
        nq, nk = S // bq, S // bk
        tile, block = np.repeat(np.arange(nq, dtype=np.int32), nk), np.tile(np.arange(nk, dtype=np.int32), nq)
        code = (block << _schedule.CODE_SHIFT) | ((block == 0) << 1) | (block == nk - 1)
    scratch = _scratch("tjx_attention_block_workspace_bytes", B, H, S, Dh, w_up.shape[1])
    results = (jax.ShapeDtypeStruct((B, S, H * Dh), q.dtype), jax.ShapeDtypeStruct((scratch,), jnp.uint8))
    out, _ = jax.ffi.ffi_call("tjx_attention_block", results)(
        q, k, v, gamma, w_up, w_down, _i32(tile), _i32(code), block_q=np.int32(bq), block_kv=np.int32(bk),
        pattern_tiles=np.int32(S // bq), eps=np.float32(eps))
    return out


def mla_decode(q_c, q_r, c_kv, k_rope, lengths, block_kv: int = 512):
    """Absorbed MLA decode through `tjx_mla_decode` (examples/decode.py:226-250): (out, step_tile, step_code,
    step_count)."""
    import jax
    import jax.numpy as jnp

    register()
    B, T, H, _ = q_c.shape
    S = c_kv.shape[1]
    block = min(block_kv, S)
    n = B * (S // block)
    results = (jax.ShapeDtypeStruct(q_c.shape, q_c.dtype), jax.ShapeDtypeStruct((n,), jnp.int32),
               jax.ShapeDtypeStruct((n,), jnp.int32), jax.ShapeDtypeStruct((1,), jnp.int32),
               jax.ShapeDtypeStruct((B + 1,), jnp.int32),
               jax.ShapeDtypeStruct((_scratch("tjx_mla_decode_workspace_bytes", B, T, H, S, block),), jnp.uint8))
    out, tile, code, count, _, _ = jax.ffi.ffi_call("tjx_mla_decode", results)(q_c, q_r, c_kv, k_rope, lengths,
                                                                               block=np.int32(block))
    return out, tile, code, count


def ragged_paged_attention(q, keys, values, kv_cache, kv_lens, page_indices, cu_q_lens, distribution,
                           sm_scale: float = 1.0):
    """One ragged paged attention step through `tjx_ragged_paged_attention` (`autokernel_rpa`,
    examples/ragged_paged_attention.py:279-290): (out, the updated cache). The cache operand is aliased to the cache
    result, so under `jax.jit` with the cache donated the update is in place, as the reference's is."""
    import jax
    import jax.numpy as jnp

    register()
    T, H, D = q.shape
    S = kv_lens.shape[0]
    page_size = kv_cache.shape[1]
    scratch = _scratch("tjx_ragged_paged_attention_workspace_bytes", T, S, H, D, page_size, page_indices.shape[0] // S)
    results = (jax.ShapeDtypeStruct(q.shape, q.dtype), jax.ShapeDtypeStruct(kv_cache.shape, kv_cache.dtype),
               jax.ShapeDtypeStruct((scratch,), jnp.uint8))
    out, cache, _ = jax.ffi.ffi_call("tjx_ragged_paged_attention", results, input_output_aliases={3: 1})(
        q, keys, values, kv_cache, kv_lens, page_indices, cu_q_lens, distribution, sm_scale=np.float32(sm_scale))
    return out, cache
