"""Ragged paged attention's cache write and decode case through the C ABI (examples/ragged_paged_attention.py:33-79,
:121-149) against the oracle: the write bit for bit, the decode within the decode tolerance (2e-2,
tests/test_decode.py:235) of the oracle and of float64."""

import numpy as np
import pytest
import torch
from helpers import f64, to_device, to_host

import oracle
from tilejax_b200 import ops
from tilejax_b200._lib import NativeError

pytestmark = pytest.mark.gpu

NAMES = ("kv_cache", "keys", "values", "kv_lens", "page_indices", "cu_q_lens", "distribution")


def step(q_lens, kv_lens, **sizes):
    inp = oracle.rpa_inputs(q_lens, kv_lens, **sizes)
    dev = {k: to_device(v) for k, v in inp.items()}
    return inp, dev


@pytest.mark.parametrize(("q_lens", "kv_lens", "sizes"), [
    ([1, 1, 1, 300, 7, 130], [513, 1, 128, 300, 135, 400], dict(max_len=1024, max_tokens=448, max_seqs=8)),
    ([1] * 16, list(range(1, 1025, 64)), dict(max_len=1024)),                       # decode only
    ([5, 129], [5, 1000], dict(heads=8, kv_heads=2, max_len=1024, page_size=16)),   # no decode sequence; small pages
])
def test_the_write_is_bit_exact_and_touches_nothing_else(q_lens, kv_lens, sizes):
    inp, dev = step(q_lens, kv_lens, **sizes)
    want = oracle.rpa_write_ref(*(inp[n] for n in NAMES))
    got = to_host(ops.rpa_write(*(dev[n] for n in NAMES)))
    np.testing.assert_array_equal(got.view(np.uint16), want.view(np.uint16))
    assert ops.device_status() == 0


@pytest.mark.parametrize(("q_lens", "kv_lens", "sizes"), [
    ([1, 1, 1, 1, 9], [1, 128, 129, 700, 64], dict(max_len=1024, max_seqs=8)),      # Llama-3-8B heads: 32 / 8
    ([1] * 24, [int(x) for x in np.random.default_rng(0).integers(1, 2049, 24)], dict(max_len=2048)),
    ([1, 1, 40], [77, 513, 40], dict(heads=8, kv_heads=8, max_len=1024, page_size=64)),   # one query head per KV head
    ([6, 3], [6, 30], dict(heads=16, kv_heads=2, max_len=256)),                     # no decode sequence: q comes back
])
def test_decode_matches_the_oracle_and_float64(q_lens, kv_lens, sizes):
    inp, dev = step(q_lens, kv_lens, **sizes)
    cache = ops.rpa_write(*(dev[n] for n in NAMES))
    scale = 128**-0.5
    args = (dev["q"], cache, dev["kv_lens"], dev["page_indices"], dev["distribution"], scale)
    got = to_host(ops.rpa_decode(*args))
    assert ops.device_status() == 0
    host_cache = to_host(cache)
    want = oracle.rpa_decode_ref(inp["q"], host_cache, inp["kv_lens"], inp["page_indices"], inp["distribution"], scale)
    exact = oracle.rpa_decode_f64(inp["q"], host_cache, inp["kv_lens"], inp["page_indices"], inp["distribution"], scale)
    assert np.abs(f64(got) - f64(want)).max() <= 2e-2
    assert np.abs(f64(got) - exact).max() <= 2e-2
    d0 = int(inp["distribution"][0])
    np.testing.assert_array_equal(got[d0:].view(np.uint16), inp["q"][d0:].view(np.uint16))  # the other rows: the query
    # In place, as the reference's donated queries: the same values.
    q_in_place = dev["q"].clone()
    same = ops.rpa_decode(q_in_place, *args[1:], out=q_in_place)
    assert same.data_ptr() == q_in_place.data_ptr()
    np.testing.assert_array_equal(to_host(same).view(np.uint16), got.view(np.uint16))


def test_bad_arguments_are_errors():
    inp, dev = step([1, 2], [5, 9], max_len=256)
    with pytest.raises(ValueError, match="side by side"):
        ops.rpa_decode(dev["q"], dev["kv_cache"][:, :, :, 0], dev["kv_lens"], dev["page_indices"], dev["distribution"])
    with pytest.raises(ValueError, match=r"\(T, Hkv, D\)"):
        ops.rpa_write(dev["kv_cache"], dev["keys"][:, :4].contiguous(), dev["values"], dev["kv_lens"],
                      dev["page_indices"], dev["cu_q_lens"], dev["distribution"])
    cache64 = torch.zeros(4, 128, 8, 2, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(NativeError, match="head dimension must be 128"):
        ops.rpa_decode(torch.zeros(3, 32, 64, dtype=torch.bfloat16, device="cuda"), cache64, dev["kv_lens"],
                       dev["page_indices"], dev["distribution"])


@pytest.mark.parametrize(("q_lens", "kv_lens", "sizes"), [
    ([1, 1, 300, 7, 130], [513, 1, 300, 135, 400], dict(max_len=1024, max_tokens=448, max_seqs=8, seed=3)),
    ([128, 129, 1], [128, 1000, 1], dict(heads=8, kv_heads=4, max_len=1024)),   # a whole block; a prefix of 871; then...
    ([5], [5], dict(heads=4, kv_heads=2, max_len=256)),                           # fewer rows than a tile
    ([700, 3], [2048, 1500], dict(heads=16, kv_heads=2, max_len=2048)),           # chunked prefill deep in the cache
])
def test_prefill_matches_the_oracle_and_float64(q_lens, kv_lens, sizes):
    if q_lens == [128, 129, 1]:
        q_lens, kv_lens = [1, 128, 129], [1, 128, 1000]  # decode sequences come first in the ABI
    inp, dev = step(q_lens, kv_lens, **sizes)
    cache = ops.rpa_write(*(dev[n] for n in NAMES))
    scale = 128**-0.5
    args = (dev["q"], cache, dev["kv_lens"], dev["page_indices"], dev["cu_q_lens"], dev["distribution"], scale)
    got = to_host(ops.rpa_prefill(*args))
    assert ops.device_status() == 0
    host = (inp["q"], to_host(cache), inp["kv_lens"], inp["page_indices"], inp["cu_q_lens"], inp["distribution"], scale)
    want = oracle.rpa_prefill_ref(*host)
    exact = oracle.rpa_prefill_f64(*host)
    assert np.abs(f64(got) - f64(want)).max() <= 2e-2
    assert np.abs(f64(got) - exact).max() <= 2e-2
    d0, tokens = int(inp["distribution"][0]), int(inp["cu_q_lens"][-1])
    np.testing.assert_array_equal(got[:d0].view(np.uint16), inp["q"][:d0].view(np.uint16))      # decode rows: untouched
    np.testing.assert_array_equal(got[tokens:].view(np.uint16), inp["q"][tokens:].view(np.uint16))  # padding rows
    in_place = dev["q"].clone()
    same = ops.rpa_prefill(in_place, *args[1:], out=in_place)
    np.testing.assert_array_equal(to_host(same).view(np.uint16), got.view(np.uint16))


def test_the_whole_step_is_write_then_decode_then_prefill():
    inp, dev = step([1, 1, 1, 200, 64], [900, 1, 257, 200, 700], max_len=1024, max_tokens=320, max_seqs=8, seed=9)
    scale = 128**-0.5
    out, cache = ops.ragged_paged_attention(dev["q"], dev["keys"], dev["values"], dev["kv_cache"], dev["kv_lens"],
                                            dev["page_indices"], dev["cu_q_lens"], dev["distribution"], scale)
    assert ops.device_status() == 0
    want_cache = oracle.rpa_write_ref(*(inp[n] for n in NAMES))
    np.testing.assert_array_equal(to_host(cache).view(np.uint16), want_cache.view(np.uint16))
    want = oracle.rpa_decode_f64(inp["q"], want_cache, inp["kv_lens"], inp["page_indices"], inp["distribution"], scale)
    pre = oracle.rpa_prefill_f64(inp["q"], want_cache, inp["kv_lens"], inp["page_indices"], inp["cu_q_lens"],
                                 inp["distribution"], scale)
    want[3:] = pre[3:]
    assert np.abs(f64(to_host(out)) - want).max() <= 2e-2
    np.testing.assert_array_equal(to_host(dev["q"]).view(np.uint16), inp["q"].view(np.uint16))  # q itself is left alone


@pytest.mark.parametrize(("q_lens", "kv_lens", "sizes"), [
    ([1, 1, 1, 200, 64], [900, 1, 257, 200, 700], dict(max_len=1024, max_tokens=320, max_seqs=8, seed=9)),  # padding rows
    ([1] * 8 + [256, 130], [40 * i + 1 for i in range(8)] + [512, 130], dict(max_len=1024, seed=3)),        # every row used
    ([1] * 16, list(range(1, 1025, 64)), dict(max_len=1024, max_tokens=64)),                                # decode only
    ([129, 5], [1000, 5], dict(max_len=1024, max_tokens=256, seed=4)),                                      # no decode sequence
])
def test_the_one_call_step_equals_the_three_calls_bit_for_bit(q_lens, kv_lens, sizes):
    # tjx_ragged_paged_attention_bf16 against tjx_rpa_write_bf16, tjx_rpa_decode_bf16 and tjx_rpa_prefill_bf16 in that
    # order: the same cache and the same out, rows that no case writes (padding tokens) holding the query; q itself
    # untouched; three calls on one workspace.
    inp, dev = step(q_lens, kv_lens, **sizes)
    inp["q"][int(sum(q_lens)):] = 3.0  # the padding rows: something a fresh buffer does not hold by chance
    dev["q"] = to_device(inp["q"])
    scale = 128**-0.5
    index = [dev[n] for n in ("kv_lens", "page_indices")]
    cache3 = ops.rpa_write(dev["kv_cache"].clone(), dev["keys"], dev["values"], *index, dev["cu_q_lens"], dev["distribution"])
    out3 = ops.rpa_decode(dev["q"], cache3, *index, dev["distribution"], scale)
    out3 = ops.rpa_prefill(out3, cache3, *index, dev["cu_q_lens"], dev["distribution"], scale, out=out3)
    for _ in range(3):
        cache1 = dev["kv_cache"].clone()
        out1, same_cache = ops.ragged_paged_attention(dev["q"], dev["keys"], dev["values"], cache1, *index,
                                                      dev["cu_q_lens"], dev["distribution"], scale)
        assert ops.device_status() == 0
        assert same_cache is cache1
        assert torch.equal(cache1.view(torch.int16), cache3.view(torch.int16))
        assert torch.equal(out1.view(torch.int16), out3.view(torch.int16))
    np.testing.assert_array_equal(to_host(dev["q"]).view(np.uint16), inp["q"].view(np.uint16))
    # The update in place, as the reference's donated q gets it.
    in_place = dev["q"].clone()
    same, _ = ops.ragged_paged_attention(in_place, dev["keys"], dev["values"], dev["kv_cache"].clone(), *index,
                                         dev["cu_q_lens"], dev["distribution"], scale, out=in_place)
    assert same is in_place and torch.equal(in_place.view(torch.int16), out3.view(torch.int16))
    # Under the reference's name and signature (examples/ragged_paged_attention.py:279-290).
    from tilejax_b200.autokernel.kernels import autokernel_rpa

    named, _ = autokernel_rpa(dev["q"], dev["keys"], dev["values"], dev["kv_cache"].clone(), *index, dev["cu_q_lens"],
                              dev["distribution"], sm_scale=scale)
    assert torch.equal(named.view(torch.int16), out3.view(torch.int16))


def test_the_one_call_step_refuses_before_it_writes_the_cache():
    # More sequences than a device step table holds: refused by the call as a whole, the cache as it was.
    T = S = 8193
    zeros = lambda *shape: torch.zeros(shape, dtype=torch.int32, device="cuda")  # noqa: E731
    q = torch.zeros((T, 4, 128), dtype=torch.bfloat16, device="cuda")
    kv = torch.ones((T, 2, 128), dtype=torch.bfloat16, device="cuda")
    cache = torch.zeros((2, 128, 2, 2, 128), dtype=torch.bfloat16, device="cuda")
    lens = torch.ones(S, dtype=torch.int32, device="cuda")
    cu = torch.arange(S + 1, dtype=torch.int32, device="cuda")
    dist = torch.tensor([S, S, S], dtype=torch.int32, device="cuda")
    with pytest.raises(NativeError, match="more than 8192 tiles"):
        ops.ragged_paged_attention(q, kv, kv, cache, lens, zeros(S), cu, dist)
    torch.cuda.synchronize()
    assert not cache.any()


def test_prefill_limits_are_errors():
    inp, dev = step([4], [4], heads=4, kv_heads=4, max_len=256)  # one query head per KV head
    with pytest.raises(NativeError, match="even number of query heads per KV head"):
        ops.rpa_prefill(dev["q"], dev["kv_cache"], dev["kv_lens"], dev["page_indices"], dev["cu_q_lens"], dev["distribution"])
    inp, dev = step([4], [4], heads=4, kv_heads=2, max_len=256, page_size=64)
    with pytest.raises(NativeError, match="pages of 128 positions"):
        ops.rpa_prefill(dev["q"], dev["kv_cache"], dev["kv_lens"], dev["page_indices"], dev["cu_q_lens"], dev["distribution"])


def test_the_decode_nest_runs_through_the_front_end():
    # `@autokernel.kernel` on the loop nest (a trip count read from kv_lens as the kernel runs, q updated): the same
    # launch as ops.rpa_decode, found by recognising the nest; the caller's q is left alone (the reference donates it).
    from tilejax_b200.autokernel import kernels

    inp, dev = step([1, 1, 1, 1, 9], [1, 128, 129, 700, 64], max_len=1024, max_seqs=8)
    cache = ops.rpa_write(*(dev[n] for n in NAMES))
    scale = 128**-0.5
    kernel = kernels.make_rpa_decode(scale)
    q_before = dev["q"].clone()
    args = (dev["q"], cache, dev["kv_lens"], dev["page_indices"], dev["distribution"])
    got = kernel(*args)
    assert ops.device_status() == 0 and torch.equal(dev["q"], q_before)
    assert torch.equal(got, ops.rpa_decode(*args, scale))
    want = oracle.rpa_decode_ref(inp["q"], to_host(cache), inp["kv_lens"], inp["page_indices"], inp["distribution"], scale)
    assert np.abs(f64(to_host(got)) - f64(want)).max() <= 2e-2
    assert kernel.verify(*args) <= 2e-2
    assert "tjx_rpa_decode_bf16" in kernel.source(*args)


def test_the_write_nest_runs_through_the_front_end_and_the_run_kernel_writes_in_place():
    from tilejax_b200.autokernel import kernels

    inp, dev = step([1, 1, 1, 300, 7, 130], [513, 1, 128, 300, 135, 400], max_len=1024, max_tokens=448, max_seqs=8)
    runs = oracle.rpa_write_runs(inp["kv_lens"], inp["page_indices"], inp["cu_q_lens"], inp["distribution"], 128, 448)
    tables = [to_device(v) for v in runs.values()]
    want = oracle.rpa_write_ref(*(inp[n] for n in NAMES))
    before = dev["kv_cache"].clone()
    got = kernels.rpa_write(dev["kv_cache"], dev["keys"], dev["values"], dev["page_indices"], *tables)
    assert ops.device_status() == 0 and torch.equal(dev["kv_cache"], before)  # the caller's cache is left alone
    np.testing.assert_array_equal(to_host(got).view(np.uint16), want.view(np.uint16))
    same = ops.rpa_write_runs(dev["kv_cache"], dev["keys"], dev["values"], dev["page_indices"], *tables)
    assert same.data_ptr() == dev["kv_cache"].data_ptr() and torch.equal(same, got)     # the C entry: in place
    assert torch.equal(ops.rpa_write(*(dev[n] for n in NAMES)), got)                    # writing again changes nothing


def test_the_prefill_nest_runs_through_the_front_end():
    from tilejax_b200.autokernel import kernels

    inp, dev = step([1, 1, 300, 7, 130], [513, 1, 300, 135, 400], max_len=1024, max_tokens=448, max_seqs=8)
    cache = ops.rpa_write(*(dev[n] for n in NAMES))
    tiles = oracle.rpa_prefill_tiles(inp["kv_lens"], inp["page_indices"], inp["cu_q_lens"], inp["distribution"], 448)
    tables = [to_device(v) for v in tiles.values()]
    scale = 128**-0.5
    kernel = kernels.make_rpa_prefill(scale)
    q_before = dev["q"].clone()
    args = (dev["q"], cache, dev["page_indices"], *tables)
    got = kernel(*args)
    assert ops.device_status() == 0 and torch.equal(dev["q"], q_before)
    # The tiles of 256 cut in two are the tiles of 128 the other entry point builds itself: the same launch.
    assert torch.equal(got, ops.rpa_prefill(dev["q"], cache, dev["kv_lens"], dev["page_indices"], dev["cu_q_lens"],
                                            dev["distribution"], scale))
    host_cache = to_host(cache)
    exact = oracle.rpa_prefill_f64(inp["q"], host_cache, inp["kv_lens"], inp["page_indices"], inp["cu_q_lens"],
                                   inp["distribution"], scale)
    assert np.abs(f64(to_host(got)) - exact).max() <= 2e-2
    assert kernel.verify(*args) <= 2e-2
