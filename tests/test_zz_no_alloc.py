"""The decode entry point that allocates nothing (tjx_paged_gqa_decode_bf16_static), for callers that cannot call
cudaMalloc and have no scratch to lend: it must give what the ordinary entry point gives.

Collected last on purpose (the file name sorts after every other test file): a run that stops at the first
failure has then already run everything else. It passes alone in a fresh process and after the other tests: it
needs nothing they set up, and the library's built-in scratch keeps no state a call depends on.
"""

import numpy as np
import pytest
import torch
from helpers import f64, to_device, to_host

from tilejax_b200 import ops, synthetic
from tilejax_b200._lib import NativeError, library

pytestmark = pytest.mark.gpu

STATIC_CALLS: list[int] = []  # the first call of the process may still load the entry point's own code


def both_ways(q, kp, vp, bt, lengths):
    dev = [to_device(a) for a in (q, kp, vp, bt, lengths)]
    B, pages = bt.shape
    want = ops.paged_gqa_decode(*dev)
    want_tables = ops.paged_gqa_decode.last_buffers
    # Everything the static entry point touches is allocated here, by the caller, before the call.
    out = torch.full_like(dev[0], float("nan"))
    step_tile = torch.empty(B * pages, dtype=torch.int32, device="cuda")
    step_code = torch.empty(B * pages, dtype=torch.int32, device="cuda")
    step_count = torch.empty(1, dtype=torch.int32, device="cuda")
    tile_first = torch.empty(B + 1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]
    got = ops.paged_gqa_decode_static(*dev, out, step_tile, step_code, step_count, tile_first)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before  # no allocation through torch either
    # ... and none behind torch's back: the driver's count of free device memory (cudaMemGetInfo) has not moved,
    # which a cudaMalloc or cudaMallocAsync inside the library would have lowered. (The library's code and its
    # built-in scratch were loaded by the ordinary call above, which launches the same kernels.)
    if STATIC_CALLS:
        assert torch.cuda.mem_get_info()[0] == free_before
    STATIC_CALLS.append(1)
    assert ops.device_status() == 0
    # Same kernels, same order of operations: the results are bit-identical, well inside the decode tolerance
    # the other tests use (2e-2 of the largest value).
    assert np.abs(f64(to_host(got)) - f64(to_host(want))).max() <= 2e-2 * max(np.abs(f64(to_host(want))).max(), 1e-6)
    assert torch.equal(got, want)
    assert torch.equal(step_tile, want_tables.step_tile) and torch.equal(step_code, want_tables.step_code)
    assert int(step_count[0]) == int(want_tables.step_count[0])
    return to_host(got)


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    # First call: the reference's ragged case (an empty sequence, one token, a partial page, a full cache).
    q, kp, vp, bt, lengths = synthetic.decode_inputs(4, 8, 2, 128, 16, 32, 128, distinct_pages=True)
    lengths[:] = [0, 1, 300, 512]
    first = both_ways(q, kp, vp, bt, lengths)
    assert not f64(first[0]).any()
    # Second call, other sizes and data: the scratch still holds the first call's partials, and none may leak.
    q, kp, vp, bt, lengths = synthetic.decode_inputs(64, 32, 8, 128, 16, 256, 8192, seed=7)
    both_ways(q, kp, vp, bt, lengths)
    # And the first inputs once more, after the larger call overwrote the scratch.
    q, kp, vp, bt, lengths = synthetic.decode_inputs(4, 8, 2, 128, 16, 32, 128, distinct_pages=True)
    lengths[:] = [0, 1, 300, 512]
    np.testing.assert_array_equal(f64(both_ways(q, kp, vp, bt, lengths)), f64(first))


def test_sizes_beyond_the_built_in_scratch_are_refused():
    limit = int(library().tjx_paged_gqa_decode_static_scratch_bytes())
    assert limit == 36 * 1024 * 1024
    B, H, pages = 256, 32, 256  # four times the benchmark's batch: needs about 70 MB
    assert int(library().tjx_paged_gqa_decode_workspace_bytes(B, 1, H, 128, pages)) > limit
    q = torch.zeros(B, 1, H, 128, dtype=torch.bfloat16, device="cuda")
    kp = torch.zeros(16, 16, 8 * 128, dtype=torch.bfloat16, device="cuda")
    bt = torch.zeros(B, pages, dtype=torch.int32, device="cuda")
    lengths = torch.ones(B, dtype=torch.int32, device="cuda")
    tables = [torch.empty(n, dtype=torch.int32, device="cuda") for n in (B * pages, B * pages, 1, B + 1)]
    with pytest.raises(NativeError, match="more than the 37748736 bytes built into the library"):
        ops.paged_gqa_decode_static(q, kp, kp, bt, lengths, torch.empty_like(q), *tables)
