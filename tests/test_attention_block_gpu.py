"""`attention_block` (examples/attention_block.py:49-85) through the C ABI against the oracle and float64: attention
writing the heads side by side in f32, the row-wise RMSNorm, the matmul with tanh GELU in its epilogue, the matmul.
The reference's own tolerance against float64 is 3e-2 of the largest value (tests/test_examples.py:187); against the
oracle, the compare rule for bf16 outputs (rtol 2e-2, atol 2e-2 * max|want|)."""

import numpy as np
import pytest
import torch
from helpers import f64, to_device, to_host
from test_attention_block import make_inputs

import oracle
from oracle.attention_block import attention_block_f64, attention_block_ref
from tilejax_b200 import ops
from tilejax_b200._lib import NativeError, library
from tilejax_b200.autokernel import kernels as K

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize(("shape", "blocks"), [
    ((1, 2, 512, 128, 512), (128, 128, 1024)),    # tests/test_examples.py:179-198
    ((1, 2, 512, 128, 512), (256, 128, 1024)),
    ((1, 2, 256, 128, 1024), (128, 128, 256)),    # the feed-forward layer in four steps (:208-222)
    ((2, 4, 384, 128, 768), (128, 512, 256)),     # two batches; one key block spans the sequence; 3 weight steps
    ((1, 8, 1024, 128, 2048), (512, 512, 1024)),  # pair-MMA pieces in both matmuls
])
def test_matches_the_oracle_and_float64(shape, blocks):
    inputs = make_inputs(*shape)
    B, H, S, Dh, F = shape
    out = torch.full((B, S, H * Dh), float("nan"), dtype=torch.bfloat16, device="cuda")
    got = to_host(ops.attention_block(*(to_device(a) for a in inputs), *blocks, out=out))
    assert ops.device_status() == 0
    exact = attention_block_f64(*inputs)
    np.testing.assert_allclose(f64(got), exact, atol=3e-2 * np.abs(exact).max())
    if S * H <= 2048:  # the blockwise oracle in NumPy: seconds at these sizes
        oracle.compare("attention_block", got, attention_block_ref(*inputs, *blocks))


def test_the_rows_are_normalised_and_the_future_is_not_seen():
    inputs = list(make_inputs(1, 2, 256, 128, 256, seed=3))
    dev = [to_device(a) for a in inputs]
    base = to_host(ops.attention_block(*dev, 128, 128, 256))
    # Keys and values after position 100 only reach queries after position 100.
    k2, v2 = inputs[1].copy(), inputs[2].copy()
    k2[:, :, 101:] = -k2[:, :, 101:]
    v2[:, :, 101:] = 0
    changed = to_host(ops.attention_block(dev[0], to_device(k2), to_device(v2), *dev[3:], 128, 128, 256))
    np.testing.assert_array_equal(f64(changed[:, :101]), f64(base[:, :101]))
    assert np.abs(f64(changed[:, 101:]) - f64(base[:, 101:])).max() > 0
    # Scaling v by a power of two scales the attention output, and the norm takes it out again (up to eps).
    v4 = (inputs[2].astype(np.float32) * 4).astype(inputs[2].dtype)
    scaled = to_host(ops.attention_block(dev[0], dev[1], to_device(v4), *dev[3:], 128, 128, 256))
    assert np.abs(f64(scaled) - f64(base)).max() <= 2e-2 * np.abs(f64(base)).max()


def test_through_the_front_end():
    inputs = make_inputs(1, 2, 256, 128, 512, seed=5)
    tiles = K.BlockTiles(block_q=128, block_kv=128, block_f=256)
    assert K.attention_block.verify(*inputs, tiles) <= 0.1
    out = K.attention_block(*inputs, tiles)
    oracle.compare("attention_block", out, attention_block_ref(*inputs, 128, 128, 256))


def test_bad_arguments_are_errors():
    q, k, v, gamma, w_up, w_down = (to_device(a) for a in make_inputs(1, 2, 256, 128, 256))
    with pytest.raises(ValueError, match=r"gamma must be \(1, 256\)"):
        ops.attention_block(q, k, v, gamma[:, :128].contiguous(), w_up, w_down)
    with pytest.raises(ValueError, match="bfloat16"):
        ops.attention_block(q.float(), k, v, gamma, w_up, w_down)
    with pytest.raises(NativeError, match="head dimension must be 128"):
        q64 = torch.zeros(1, 4, 256, 64, dtype=torch.bfloat16, device="cuda")
        ops.attention_block(q64, q64, q64, gamma, w_up, w_down)
    need = int(library().tjx_attention_block_workspace_bytes(1, 2, 256, 128, 256))
    assert need == 256 * 256 * 4 + 256 * 256 * 2 + 256 * 256 * 2
    ws = torch.empty(need - 256, dtype=torch.uint8, device="cuda")
    out = torch.empty(1, 256, 256, dtype=torch.bfloat16, device="cuda")
    tile, code = ops._attention_tables(1, 2, 256, 128, 128, q.device)
    rc = library().tjx_attention_block_bf16(*(t.data_ptr() for t in (q, k, v, gamma, w_up, w_down, out)), 1, 2, 256, 128,
                                            256, 128, 128, 1e-6, tile.data_ptr(), code.data_ptr(), tile.numel(), 2,
                                            ws.data_ptr(), ws.numel(), None)
    assert rc != 0 and b"workspace is smaller" in library().tjx_last_error()
