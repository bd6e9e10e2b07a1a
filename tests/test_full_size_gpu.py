"""The benchmark's sizes of the newer operators, checked through properties that do not need the whole oracle: sampled
rows against float64, causality, bit-identical repeats. (The matmul, causal attention and paged decode have theirs
in their own test files.)"""

import numpy as np
import pytest
from helpers import f64, rand_bf16, to_device, to_host

import oracle
from oracle.attention_block import gelu_tanh
from tilejax_b200 import ops

pytestmark = pytest.mark.gpu


def test_mla_decode_at_the_benchmark_shape():
    # benchmarks/decode.py:152-173: batch 32, 64 heads, contexts 1024..3072 of a 4096-position cache.
    B, H, S = 32, 64, 4096
    lens = np.random.default_rng(0).integers(1024, 3073, B).astype(np.int32)
    q_c, q_r = rand_bf16((B, 1, H, 512), 3, 192**-0.5 * 0.1), rand_bf16((B, 1, H, 128), 4, 192**-0.5)
    c_kv, k_rope = rand_bf16((B, S, 512), 5), rand_bf16((B, S, 128), 6)
    dev = [to_device(a) for a in (q_c, q_r, c_kv, k_rope, lens)]
    got = to_host(ops.mla_decode(*dev, 512))
    assert ops.device_status() == 0
    again = to_host(ops.mla_decode(*dev, 512))
    np.testing.assert_array_equal(got.view(np.uint16), again.view(np.uint16))        # a repeat is bit-identical
    other = to_host(ops.mla_decode(*dev, 128))                                        # the block only shapes the tables
    np.testing.assert_array_equal(got.view(np.uint16), other.view(np.uint16))
    for b in (0, 7, 31):  # float64 on three sequences
        want = oracle.mla_decode_f64(q_c[b : b + 1], q_r[b : b + 1], c_kv[b : b + 1], k_rope[b : b + 1], lens[b : b + 1])
        assert np.abs(f64(got[b : b + 1]) - want).max() <= 2e-2
    # Positions at and after lengths[b] carry no weight: huge values there change nothing. (Not NaN: a masked
    # position's probability is an exact 0, and 0 * NaN is NaN in the reference's `p @ ct` too.)
    c2, r2 = c_kv.copy(), k_rope.copy()
    for b in range(B):
        c2[b, lens[b]:] = np.float32(1e30)
        r2[b, lens[b]:] = np.float32(-1e30)
    poisoned = to_host(ops.mla_decode(dev[0], dev[1], to_device(c2), to_device(r2), dev[4], 512))
    np.testing.assert_array_equal(got.view(np.uint16), poisoned.view(np.uint16))


def test_attention_block_at_the_benchmark_shape():
    # tests/test_examples.py:201-206: B 4, 8 heads of 128, S 2048, D 1024, F 4096.
    from test_attention_block import make_inputs

    B, H, S, Dh, F = 4, 8, 2048, 128, 4096
    q, k, v, gamma, w_up, w_down = make_inputs(B, H, S, Dh, F, seed=2)
    dev = [to_device(a) for a in (q, k, v, gamma, w_up, w_down)]
    got = to_host(ops.attention_block(*dev, 256, 512, 1024))
    assert ops.device_status() == 0 and not np.isnan(f64(got)).any()
    # Sampled (batch, position) rows in float64: attention over the keys up to the position, norm, feed-forward.
    g64, up64, down64 = f64(gamma), f64(w_up), f64(w_down)
    worst = 0.0
    for b, i in ((0, 0), (1, 127), (2, 1000), (3, 2047)):
        a = np.zeros(H * Dh)
        for h in range(H):
            s = f64(k[b, h, : i + 1]) @ f64(q[b, h, i])
            p = np.exp(s - s.max())
            a[h * Dh : (h + 1) * Dh] = (p / p.sum()) @ f64(v[b, h, : i + 1])
        n = a / np.sqrt(np.mean(a * a) + 1e-6) * g64[0]
        want = gelu_tanh(n @ up64) @ down64
        worst = max(worst, np.abs(f64(got[b, i]) - want).max() / np.abs(want).max())
    assert worst <= 3e-2  # tests/test_examples.py:187
    # Causality: keys and values after position 1000 cannot reach the positions up to 1000.
    k2, v2 = k.copy(), v.copy()
    k2[:, :, 1001:] = -k2[:, :, 1001:]
    v2[:, :, 1001:] = 0
    changed = to_host(ops.attention_block(dev[0], to_device(k2), to_device(v2), *dev[3:], 256, 512, 1024))
    np.testing.assert_array_equal(changed[:, :1001].view(np.uint16), got[:, :1001].view(np.uint16))


def test_ragged_paged_attention_at_the_benchmark_shape():
    # 32 decode sequences and 4 prefill sequences of 1024 tokens on a prefix of 1024, Llama-3-8B heads, pages of 128.
    rng = np.random.default_rng(0)
    q_lens = [1] * 32 + [1024] * 4
    kv_lens = [int(x) for x in rng.integers(1, 4097, 32)] + [2048] * 4
    inp = oracle.rpa_inputs(q_lens, kv_lens, max_len=4096, seed=5)
    dev = {name: to_device(a) for name, a in inp.items()}
    scale = 128**-0.5
    out, cache = ops.ragged_paged_attention(dev["q"], dev["keys"], dev["values"], dev["kv_cache"], dev["kv_lens"],
                                            dev["page_indices"], dev["cu_q_lens"], dev["distribution"], scale)
    assert ops.device_status() == 0
    got, host_cache = to_host(out), to_host(cache)
    want_cache = oracle.rpa_write_ref(inp["kv_cache"], inp["keys"], inp["values"], inp["kv_lens"], inp["page_indices"],
                                      inp["cu_q_lens"], inp["distribution"])
    np.testing.assert_array_equal(host_cache.view(np.uint16), want_cache.view(np.uint16))
    # Float64 on sampled tokens: three decode tokens, and prefill tokens at a tile's start, inside and at its end.
    pps, ps, G = 4096 // 128, 128, 4
    cu = inp["cu_q_lens"]
    samples = [(s, 0) for s in (0, 13, 31)] + [(32, 0), (33, 127), (34, 128), (35, 1023)]
    for s, i in samples:
        n, q_len = kv_lens[s], q_lens[s]
        seen = n - q_len + i + 1
        pages = [int(inp["page_indices"][s * pps + x]) for x in range((seen + ps - 1) // ps)]
        kv = np.concatenate([f64(want_cache[pg]) for pg in pages])[:seen]
        t = int(cu[s]) + i
        for h in (0, 5, 31):
            sc = kv[:, h // G, 0, :] @ f64(inp["q"][t, h]) * scale
            w = np.exp(sc - sc.max())
            want = (w / w.sum()) @ kv[:, h // G, 1, :]
            assert np.abs(f64(got[t, h]) - want).max() <= 2e-2, (s, i, h)

