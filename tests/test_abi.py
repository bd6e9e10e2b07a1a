"""The C ABI: the library builds, loads without a GPU, and exports every symbol the header declares."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "tilejax_b200.h"


def declared_symbols() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(tjx_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_entry_points():
    names = declared_symbols()
    for name in ("tjx_gemm_bf16", "tjx_build_steps", "tjx_paged_gqa_decode_bf16", "tjx_causal_attention_bf16",
                 "tjx_last_error", "tjx_device_status"):
        assert name in names


def test_library_exports_every_declared_symbol(native):
    from tilejax_b200 import _lib

    raw = ctypes.CDLL(str(_lib.LIBRARY))
    for name in declared_symbols():
        assert hasattr(raw, name), f"{name} is declared in the header but not exported"
    assert set(_lib.SYMBOLS) == set(declared_symbols())
    assert native.tjx_version() >= 100
    assert native.tjx_last_error() is not None


def test_every_declaration_cites_the_reference():
    text = HEADER.read_text()
    for name in ("tjx_build_steps", "tjx_gemm_bf16", "tjx_causal_attention_bf16", "tjx_paged_gqa_decode_bf16"):
        comment = text[: text.index(f"int {name}(")].rsplit("/*", 1)[1]
        assert re.search(r"(examples|src/autokernel)/\w+\.py:\d+", comment), name


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from tilejax_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIBRARY", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.library()


def test_operators_refuse_cpu_tensors():
    import torch

    from tilejax_b200 import ops

    x = torch.zeros(128, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="no CPU path"):
        ops.matmul(x, x)
