"""The jax.ffi binding (tilejax_b200/xla_ffi.py over csrc/tjx_xla_ffi.cc). JAX is not installed where this suite
normally runs: the calls are then skipped, and what is checked is that the binding says so honestly and that the
handler source declares a handler for every target the Python side registers."""

import re
from pathlib import Path

import numpy as np
import pytest

from tilejax_b200 import xla_ffi
from tilejax_b200.csrc import build

SOURCE = Path(build.CSRC) / "tjx_xla_ffi.cc"


def test_every_registered_target_has_a_handler_symbol():
    text = SOURCE.read_text()
    defined = set(re.findall(r"XLA_FFI_DEFINE_HANDLER_SYMBOL\((\w+),", text))
    assert defined == set(xla_ffi.TARGETS.values())
    for entry in ("tjx_build_steps", "tjx_gemm_bf16", "tjx_causal_attention_bf16", "tjx_paged_gqa_decode_bf16",
                  "tjx_rmsnorm_gemm_bf16", "tjx_attention_block_bf16", "tjx_mla_decode_bf16",
                  "tjx_ragged_paged_attention_bf16"):
        assert f"{entry}(" in text  # each handler ends in the C ABI call it wraps
    assert "cudaMalloc" not in text and "cudaDeviceSynchronize" not in text  # enqueue only, no allocation


def test_without_jax_the_binding_is_unavailable_and_says_why():
    if build.ffi_include_dir() is not None:
        pytest.skip("JAX is installed here")
    assert not xla_ffi.available() and build.build_ffi() is None
    with pytest.raises(RuntimeError, match="needs JAX"):
        xla_ffi.register()


@pytest.mark.gpu
def test_custom_calls_agree_with_the_ctypes_path():
    if build.ffi_include_dir() is None:
        pytest.skip("JAX is not installed: the XLA FFI handlers cannot be built")
    import jax
    import jax.numpy as jnp
    import torch

    from tilejax_b200 import ops

    assert build.build_ffi() is not None
    rng = np.random.default_rng(0)
    x = jnp.asarray(rng.standard_normal((512, 256), np.float32), jnp.bfloat16)
    y = jnp.asarray(rng.standard_normal((256, 512), np.float32), jnp.bfloat16)
    got = np.asarray(jax.jit(lambda a, b: xla_ffi.causal_matmul(a, b, 128, 128, 128))(x, y).astype(jnp.float32))
    xt = torch.from_numpy(np.asarray(x.astype(jnp.float32))).cuda().bfloat16()
    yt = torch.from_numpy(np.asarray(y.astype(jnp.float32))).cuda().bfloat16()
    want = ops.causal_matmul(xt, yt, 128, 128, 128).float().cpu().numpy()
    np.testing.assert_array_equal(got, want)
