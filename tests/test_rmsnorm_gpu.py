"""`rmsnorm_matmul` (examples/rmsnorm_matmul.py:31-47) through the C ABI against the oracle and float64: one pass
over x for the gamma-scaled operand and the row scales, then the matmul step loop with the row scale in its
epilogue. bf16 outputs by the reference's compare rule (rtol 2e-2, atol 2e-2 * max|want|); f32 outputs within 1e-4 of
the largest value (the gamma-scaled operand is rounded to bf16 before the product, as the nest rounds it)."""

import numpy as np
import pytest
import torch
from helpers import BF16, f64, rand_bf16, to_device, to_host

import oracle
from tilejax_b200 import ops
from tilejax_b200._lib import NativeError
from tilejax_b200.autokernel import kernels as K

pytestmark = pytest.mark.gpu


def inputs(M, D, N, seed=0):
    rng = np.random.default_rng(seed)
    x = rand_bf16((M, D), seed)
    gamma = (1 + 0.1 * rng.standard_normal((1, D), np.float32)).astype(BF16)
    w = rand_bf16((D, N), seed + 2, D**-0.5)
    return x, gamma, w


@pytest.mark.parametrize(("shape", "tiles"), [
    ((256, 384, 256), (128, 128, 128)),     # single-CTA pieces
    ((1024, 1024, 512), (512, 512, 512)),   # the example's own sizes: one MMA per pair of SMs
    ((200, 72, 264), (512, 512, 512)),      # tiles clipped to a ragged matrix
    ((2048, 2048, 1536), (256, 512, 512)),
])
def test_matches_the_oracle_and_float64(shape, tiles):
    M, D, N = shape
    x, gamma, w = inputs(M, D, N)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    got = to_host(ops.rmsnorm_matmul(to_device(x), to_device(gamma), to_device(w), *tiles, out=out))
    assert ops.device_status() == 0
    oracle.compare("rmsnorm_matmul", got, oracle.rmsnorm_matmul_ref(x, gamma, w, *tiles))
    exact = oracle.rmsnorm_matmul_f64(x, gamma, w)
    np.testing.assert_allclose(f64(got), exact, rtol=2e-2, atol=2e-2 * np.abs(exact).max())


def test_f32_output_and_the_row_scale():
    x, gamma, w = inputs(512, 1024, 256, seed=3)
    x[7] = 0  # a row of zeros: scale = rsqrt(eps), output 0
    got = to_host(ops.rmsnorm_matmul(to_device(x), to_device(gamma), to_device(w), 256, 256, 512,
                                     out_dtype=torch.float32))
    want = f64(oracle.rmsnorm_matmul_ref(x, gamma, w, 256, 256, 512, out_dtype=np.float32))
    assert got.dtype == np.float32 and not got[7].any()
    assert np.abs(f64(got) - want).max() <= 1e-4 * np.abs(want).max()
    # Scaling x by a power of two leaves rmsnorm(x) @ w unchanged up to eps: the row scale really divides by rms(x).
    doubled = to_host(ops.rmsnorm_matmul(to_device((x.astype(np.float32) * 4).astype(BF16)), to_device(gamma),
                                         to_device(w), 256, 256, 512, out_dtype=torch.float32))
    assert np.abs(f64(doubled) - f64(got)).max() <= 1e-4 * np.abs(want).max()


def test_through_the_front_end():
    x, gamma, w = inputs(1024, 512, 768, seed=5)
    assert K.rmsnorm_matmul.verify(x, gamma, w, K.NormMatmulTiles(tm=256, tn=256, tk=256)) <= 0.1
    out = K.rmsnorm_matmul(x, gamma, w, K.NormMatmulTiles(tm=128, tn=128, tk=128))
    oracle.compare("rmsnorm_matmul", out, oracle.rmsnorm_matmul_ref(x, gamma, w, 128, 128, 128))


def test_bad_arguments_are_errors():
    x, gamma, w = (to_device(a) for a in inputs(256, 256, 256))
    with pytest.raises(ValueError, match=r"gamma \(1, D\)"):
        ops.rmsnorm_matmul(x, gamma[:, :128].contiguous(), w)
    with pytest.raises(ValueError, match="bfloat16"):
        ops.rmsnorm_matmul(x.float(), gamma, w)
    with pytest.raises(NativeError, match="multiple of 128"):
        ops.rmsnorm_matmul(x, gamma, w, 64, 128, 128)
