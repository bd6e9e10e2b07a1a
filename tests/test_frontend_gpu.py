"""The front end on a B200: `kernel(...)`, `.verify` and `.tuning` for each hot-path loop nest. `verify` compares
the CUDA kernel (through the C ABI) with the loop nest's reference on the CPU under the reference's tolerances."""

import numpy as np
import pytest
import torch
from helpers import f64, rand_bf16, to_device

import oracle
from tilejax_b200 import ops, synthetic
from tilejax_b200.autokernel import Config, Pipeline
from tilejax_b200.autokernel import kernels as K

pytestmark = pytest.mark.gpu
TILES = K.MatmulTiles(tm=128, tn=128, tk=128)


def test_matmul_verifies_and_takes_host_or_device_arrays():
    x, y = rand_bf16((256, 384), 0), rand_bf16((384, 256), 1)
    assert K.matmul.verify(x, y, TILES) <= 0.5
    on_host = K.matmul(x, y, TILES)
    assert isinstance(on_host, np.ndarray) and on_host.shape == (256, 256)
    on_device = K.matmul(to_device(x), to_device(y), TILES)
    assert isinstance(on_device, torch.Tensor) and on_device.is_cuda
    oracle.compare("matmul", on_host, oracle.matmul_ref(x, y, 128, 128, 128))
    # Every pipeline depth runs the same arithmetic.
    sig = K.matmul.signature(x, y)
    for pipeline in (Pipeline(2, 2), Pipeline(4, 3)):
        out = K.matmul.lowered(sig, Config(TILES, pipeline)).run(x, y)
        oracle.compare("matmul", out, oracle.matmul_ref(x, y, 128, 128, 128))


def test_every_loop_nest_verifies():
    x, y = rand_bf16((512, 256), 0), rand_bf16((256, 512), 1)
    assert K.causal_matmul.verify(x, y, TILES) <= 0.5
    assert K.causal_matmul.verify(x, y, K.MatmulTiles(tm=256, tn=512, tk=256)) <= 0.5
    q, k, v = synthetic.attention_inputs(1, 2, 512, 128)
    assert K.causal_attention.verify(q, k, v, K.AttentionBlocks(128, 256)) <= 2e-2
    q, kp, vp, bt, lengths = synthetic.decode_inputs(4, 8, 2, 128, 16, 32, 128, distinct_pages=True)
    lengths[:] = [0, 1, 300, 512]
    assert K.paged_gqa_decode.verify(q, kp, vp, bt, lengths) <= 2e-2
    assert not f64(K.paged_gqa_decode(q, kp, vp, bt, lengths)[0]).any()
    kc, vc = rand_bf16((4, 512, 256), 4), rand_bf16((4, 512, 256), 5)
    assert K.gqa_decode.verify(rand_bf16((4, 1, 8, 128), 6, 128**-0.5), kc, vc, lengths, K.DecodeTiles(block_kv=128)) <= 2e-2
    q_c, q_r = rand_bf16((4, 1, 16, 512), 7, 0.01), rand_bf16((4, 1, 16, 128), 8, 0.07)
    c_kv, k_rope = rand_bf16((4, 512, 512), 9), rand_bf16((4, 512, 128), 10)
    assert K.mla_decode.verify(q_c, q_r, c_kv, k_rope, lengths, K.DecodeTiles(block_kv=128)) <= 2e-2
    assert K.all_gather_matmul.verify(x, y, K.CollectiveTiles()) <= 0.5  # one rank: the gather is the identity


def test_tuning_tries_schedules_and_keeps_the_fastest():
    x, y = rand_bf16((1024, 1024), 0), rand_bf16((1024, 1024), 1)
    tuning = K.matmul.tuning(x, y)
    assert 1 <= len(tuning.trials) <= 12 and tuning.best in tuning.trials
    assert all(t.profile is not None or t.error for t in tuning.trials)
    assert tuning.best.seconds == min(t.seconds for t in tuning.trials) or tuning.best.seconds <= 1.02 * min(
        t.seconds for t in tuning.trials)
    text = str(tuning)
    assert text.startswith("chose MatmulTiles(") and text.count("*") == 1
    out = K.matmul(x, y)  # uses the tuned schedule
    oracle.compare("matmul", out, oracle.matmul_ref(x, y, 512, 512, 512))
    assert K.matmul.tuning(x, y) is tuning  # remembered per signature


def test_profile_says_where_the_time_goes():
    # autokernel.profile (src/autokernel/profiling.py:267-274): device time from CUDA events, the split from the
    # kernels' own counters. The parts are non-negative and add up to the device time.
    import tilejax_b200.autokernel as autokernel

    x, y = rand_bf16((2048, 2048), 0), rand_bf16((2048, 2048), 1)
    for tiles in (K.MatmulTiles(), TILES):  # one MMA per pair of SMs, and the single-CTA ring
        report = autokernel.profile(K.matmul, (x, y, tiles), runs=3)
        assert report.regions and report.calls == 3 and report.device_s > 0 and report.steps > 0
        parts = (report.wait_s, report.out_wait_s, report.compute_s, report.other_s)
        assert all(p >= 0 for p in parts) and sum(parts) == pytest.approx(report.device_s, rel=1e-6)
        assert report.fill_s <= report.wait_s and report.compute_s > 0
        assert report.bottleneck in ("dma", "overhead", "compute") and "bottleneck:" in str(report)
    q, k, v = synthetic.attention_inputs(1, 4, 1024, 128)
    report = autokernel.profile(K.causal_attention, (q, k, v, K.AttentionBlocks()))
    assert report.regions and report.compute_s > 0 and "softmax" in report.scopes
    q, kp, vp, bt, lengths = synthetic.decode_inputs(8, 32, 8, 128, 16, 64, 1024)
    report = autokernel.profile(K.paged_gqa_decode, (q, kp, vp, bt, lengths))
    assert report.regions and report.wait_s > 0 and report.steps == 8 * 64
    # The MLA decode kernel counts too: its issuing warp's waits for the cache blocks and for the softmax warps.
    lengths4 = np.array([0, 1, 300, 512], np.int32)
    q_c, q_r = rand_bf16((4, 1, 16, 512), 7, 0.01), rand_bf16((4, 1, 16, 128), 8, 0.07)
    c_kv, k_rope = rand_bf16((4, 512, 512), 9), rand_bf16((4, 512, 128), 10)
    report = autokernel.profile(K.mla_decode, (q_c, q_r, c_kv, k_rope, lengths4, K.DecodeTiles(block_kv=128)))
    assert report.regions and report.device_s > 0 and report.wait_s > 0
    # A kernel that carries no counters still reports its device time: the warp-level MLA kernel behind the switch.
    ops.set_mla_mode(0)
    try:
        blind = autokernel.profile(K.mla_decode, (q_c, q_r, c_kv, k_rope, lengths4, K.DecodeTiles(block_kv=128)))
    finally:
        ops.set_mla_mode(1)
    assert not blind.regions and blind.bottleneck is None and blind.device_s > 0
