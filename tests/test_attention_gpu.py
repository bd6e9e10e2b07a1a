"""Causal flash attention through the C ABI against the oracle (`causal_attention`,
examples/causal_attention.py:37-63). Tolerance: atol 2e-2 (tests/test_examples.py:86-87) and the reference's
compare rule (rtol 2e-2, atol 2e-2 * max|want|, src/autokernel/api.py:329-350)."""

import numpy as np
import pytest
import torch
from helpers import f64, to_device, to_host

import oracle
from tilejax_b200 import ops, synthetic
from tilejax_b200._lib import NativeError

pytestmark = pytest.mark.gpu


def run_attention(q, k, v, bq, bk):
    out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.causal_attention(to_device(q), to_device(k), to_device(v), bq, bk, out=out)
    assert ops.device_status() == 0
    return to_host(out)


@pytest.mark.parametrize(("shape", "blocks"), [
    ((2, 4, 512, 128), (128, 128)),   # tests/test_examples.py:80-95
    ((1, 2, 512, 128), (256, 128)),
    ((1, 2, 512, 128), (128, 256)),
    ((1, 2, 1024, 128), (512, 512)),
    ((1, 1, 128, 128), (128, 128)),   # a single block: one tile, one step
    ((1, 3, 384, 128), (128, 128)),   # an odd number of 128-row tiles: the last CTA has one slot
    ((1, 1, 1024, 128), (1024, 1024)),
])
def test_matches_the_oracle(shape, blocks):
    q, k, v = synthetic.attention_inputs(*shape)
    got = run_attention(q, k, v, *blocks)
    want = oracle.causal_attention_ref(q, k, v, *blocks)
    oracle.compare("causal_attention", got, want)
    np.testing.assert_allclose(f64(got), oracle.causal_attention_f64(q, k, v), atol=2e-2)


def test_benchmark_shape_against_float64_rows_and_causality():
    # BASELINE config 3 at full size: sampled (b, h) pairs against float64; and causality as a size-independent
    # property: changing keys and values at positions > t leaves out[..., :t + 1, :] bit-identical.
    B, H, S, D = 4, 16, 2048, 128
    q, k, v = synthetic.attention_inputs(B, H, S, D)
    got = run_attention(q, k, v, 512, 512)
    assert not np.isnan(f64(got)).any()
    for b, h in ((0, 0), (3, 15), (1, 7)):
        want = oracle.causal_attention_f64(q[b : b + 1, h : h + 1], k[b : b + 1, h : h + 1], v[b : b + 1, h : h + 1])
        np.testing.assert_allclose(f64(got[b, h]), want[0, 0], atol=2e-2)
    t = 1000
    k2, v2 = k.copy(), v.copy()
    k2[:, :, t + 1 :] = synthetic.normal_bf16(k2[:, :, t + 1 :].shape, 9)
    v2[:, :, t + 1 :] = synthetic.normal_bf16(v2[:, :, t + 1 :].shape, 10)
    again = run_attention(q, k2, v2, 512, 512)
    np.testing.assert_array_equal(f64(again[:, :, : t + 1]), f64(got[:, :, : t + 1]))
    # The user's blocks change the schedule, not the result beyond rounding.
    other = run_attention(q, k, v, 256, 256)
    assert np.abs(f64(other) - f64(got)).max() <= 2e-2


def test_second_benchmark_shape():
    q, k, v = synthetic.attention_inputs(1, 16, 4096, 128)
    got = run_attention(q, k, v, 512, 512)
    want = oracle.causal_attention_f64(q[:, 5:6], k[:, 5:6], v[:, 5:6])
    np.testing.assert_allclose(f64(got[0, 5]), want[0, 0], atol=2e-2)


def test_unsupported_shapes_are_errors():
    q = torch.zeros(1, 1, 192, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(NativeError, match="multiple of 128"):
        ops.causal_attention(q, q, q, 64, 64)
    q = torch.zeros(1, 1, 256, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(NativeError, match="head dimension"):
        ops.causal_attention(q, q, q, 128, 128)
