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


def test_the_no_allocation_decode_wrapper_checks_its_buffers_on_the_host():
    # Every buffer of ops.paged_gqa_decode_static is the caller's: a wrong dtype or a short buffer would become
    # out-of-bounds device writes, so each is refused before the library is called (no GPU needed to see that).
    import pytest
    import torch

    from tilejax_b200 import ops

    B, T, H, D, pages, page, num_pages, Hkv = 2, 1, 8, 128, 4, 16, 8, 2

    def good():
        i32 = lambda *shape: torch.zeros(shape, dtype=torch.int32)  # noqa: E731
        q = torch.zeros(B, T, H, D, dtype=torch.bfloat16)
        kp = torch.zeros(num_pages, page, Hkv * D, dtype=torch.bfloat16)
        return dict(q=q, k_pages=kp, v_pages=kp.clone(), block_tables=i32(B, pages), lengths=i32(B),
                    out=torch.zeros_like(q), step_tile=i32(B * pages), step_code=i32(B * pages), step_count=i32(1),
                    tile_first=i32(B + 1))

    bad = {
        "bfloat16": [("q", lambda a: a["q"].float()), ("out", lambda a: a["out"].float()),
                     ("v_pages", lambda a: a["v_pages"].half())],
        "int32": [("block_tables", lambda a: a["block_tables"].long()), ("lengths", lambda a: a["lengths"].long()),
                  ("step_tile", lambda a: a["step_tile"].long()), ("tile_first", lambda a: a["tile_first"].long())],
        "out must have q's shape": [("out", lambda a: a["out"][:1])],
        "both be": [("v_pages", lambda a: a["v_pages"][:4]), ("k_pages", lambda a: torch.zeros(8, 16, 200, dtype=torch.bfloat16))],
        "block_tables is": [("lengths", lambda a: a["lengths"][:1]), ("block_tables", lambda a: a["block_tables"][:1])],
        "too small": [("step_tile", lambda a: a["step_tile"][:-1]), ("step_code", lambda a: a["step_code"][:3]),
                      ("tile_first", lambda a: a["tile_first"][:B]), ("step_count", lambda a: a["step_count"][:0])],
    }
    for message, cases in bad.items():
        for name, change in cases:
            args = good()
            args[name] = change(args)
            with pytest.raises(ValueError, match=message):
                ops.paged_gqa_decode_static(**args)
    with pytest.raises(ValueError, match="CUDA tensors"):  # and only then: these operators have no CPU path
        ops.paged_gqa_decode_static(**good())
