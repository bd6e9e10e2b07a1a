"""Loads libtilejax_b200.so (built in-tree by `tilejax_b200.csrc.build`) and declares its C ABI for ctypes.

There is no fallback: if the library is missing or a call fails, an exception says so.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_int, c_size_t, c_void_p
from pathlib import Path

import os

# The library built in-tree; TILEJAX_B200_LIBRARY names another build of the same sources (a variant made with
# `python -m tilejax_b200.csrc.build -D... --output ...`) to load instead.
LIBRARY = Path(os.environ.get("TILEJAX_B200_LIBRARY") or Path(__file__).resolve().parent / "libtilejax_b200.so")

# Every symbol include/tilejax_b200.h declares: name -> (restype, argtypes).
_P = c_void_p
SYMBOLS: dict[str, tuple] = {
    "tjx_version": (c_int, []),
    "tjx_last_error": (c_char_p, []),
    "tjx_device_status": (c_int, [_P, ctypes.POINTER(c_int)]),
    "tjx_set_wait_limit_us": (c_int, [c_int]),
    "tjx_set_profile_buffer": (c_int, [_P, c_size_t]),
    "tjx_build_steps": (c_int, [_P, c_int, _P, c_int, c_int, c_int, c_int, _P, _P, _P, _P, _P]),
    "tjx_build_steps_from_runs": (c_int, [_P, c_int, c_int, _P, _P, _P, _P, _P]),
    "tjx_gemm_bf16": (c_int, [_P, _P, _P] + [c_int] * 10 + [_P, _P, c_int, _P, _P, c_int, _P]),
    "tjx_rmsnorm_gemm_workspace_bytes": (c_size_t, [c_int, c_int]),
    "tjx_rmsnorm_gemm_bf16": (c_int, [_P, _P, _P, _P, c_int, c_int, c_int, ctypes.c_float, c_int, c_int, c_int, c_int, _P,
                                      c_size_t, _P]),
    "tjx_attention_block_workspace_bytes": (c_size_t, [c_int] * 5),
    "tjx_attention_block_bf16": (c_int, [_P] * 7 + [c_int] * 7 + [ctypes.c_float, _P, _P, c_int, c_int, _P, c_size_t, _P]),
    "tjx_gemm_set_cta_limit": (c_int, [c_int]),
    "tjx_gemm_set_pair_mode": (c_int, [c_int]),
    "tjx_all_gather_gemm_bf16": (c_int, [_P] * 5 + [c_int] * 8 + [_P, _P, c_int, _P, c_int, _P]),
    "tjx_causal_attention_bf16": (c_int, [_P, _P, _P, _P] + [c_int] * 6 + [_P, _P, c_int, c_int, _P]),
    "tjx_paged_gqa_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "tjx_paged_gqa_decode_bf16": (c_int, [_P] * 6 + [c_int] * 8 + [_P] * 5 + [c_size_t, _P]),
    "tjx_rpa_write_bf16": (c_int, [_P] * 7 + [c_int] * 7 + [_P]),
    "tjx_rpa_write_runs_bf16": (c_int, [_P] * 9 + [c_int] * 7 + [_P]),
    "tjx_rpa_decode_workspace_bytes": (c_size_t, [c_int] * 6),
    "tjx_rpa_decode_bf16": (c_int, [_P] * 6 + [c_int] * 8 + [ctypes.c_float, _P, c_size_t, _P]),
    "tjx_rpa_prefill_workspace_bytes": (c_size_t, [c_int, c_int]),
    "tjx_rpa_prefill_bf16": (c_int, [_P] * 7 + [c_int] * 8 + [ctypes.c_float, _P, c_size_t, _P]),
    "tjx_rpa_prefill_tiles_workspace_bytes": (c_size_t, [c_int, c_int]),
    "tjx_rpa_prefill_tiles_bf16": (c_int, [_P] * 8 + [c_int] * 8 + [ctypes.c_float, _P, c_size_t, _P]),
    "tjx_ragged_paged_attention_workspace_bytes": (c_size_t, [c_int] * 6),
    "tjx_ragged_paged_attention_bf16": (c_int, [_P] * 9 + [c_int] * 8 + [ctypes.c_float, _P, c_size_t, _P]),
    "tjx_mla_set_mode": (c_int, [c_int]),
    "tjx_mla_decode_workspace_bytes": (c_size_t, [c_int] * 5),
    "tjx_mla_decode_bf16": (c_int, [_P] * 6 + [c_int] * 7 + [_P] * 5 + [c_size_t, _P]),
    "tjx_paged_gqa_decode_static_scratch_bytes": (c_size_t, []),
    "tjx_paged_gqa_decode_bf16_static": (c_int, [_P] * 6 + [c_int] * 8 + [_P] * 4 + [_P]),
}

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


class NativeError(RuntimeError):
    """A call into libtilejax_b200.so failed; `code` is its TJX_E_* return value."""

    def __init__(self, code: int, message: str):
        super().__init__(f"tilejax_b200: {message} (code {code})")
        self.code = code


def library() -> ctypes.CDLL:
    """The loaded library with argument types set. Raises if it has not been built."""
    global _lib
    with _lock:
        if _lib is None:
            if not LIBRARY.exists():
                raise RuntimeError(
                    f"{LIBRARY} is missing: build it with `python -m tilejax_b200.csrc.build` "
                    "(there is no CPU or PyTorch fallback for these kernels)"
                )
            lib = ctypes.CDLL(str(LIBRARY))
            for name, (restype, argtypes) in SYMBOLS.items():
                fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
                fn.restype = restype
                fn.argtypes = argtypes
            _lib = lib
        return _lib


def check(code: int) -> None:
    """Raise NativeError for a non-zero return code."""
    if code != 0:
        raise NativeError(code, library().tjx_last_error().decode() or "unknown error")
