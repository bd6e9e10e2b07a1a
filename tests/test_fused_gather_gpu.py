"""The one-launch all-gather matmul (tjx_all_gather_gemm_bf16) on ONE GPU: the other "ranks" are ordinary buffers on
the same device, so the copier warps, the arrival counters, the epochs and the own-shard tensor map all run exactly
as they do across GPUs, only the loads do not cross NVLink. Expected values: the same GEMM on rows gathered
beforehand (bit-equal: same kernel, same order of summation) and float64 on sampled rows, as the reference tests
its collective matmul (tests/test_collective.py:61-76, rtol 2e-2 / atol 0.5).

Also the give-up path of a device-side wait: a launch whose epoch is one ahead of its arrival counters can never
see its remote rows arrive; with a short limit it must return, report code 105 through the status word, and leave
the GPU usable.
"""

import numpy as np
import pytest
import torch

from tilejax_b200 import collective, ops, schedule
from tilejax_b200._lib import NativeError

pytestmark = pytest.mark.gpu


def tile_tables(me, ranks, m, N, tm, tn):
    order = schedule.collective_row_blocks(me, ranks, m // tm)
    ti, tj = collective.banded_tiles(order, N // tn, max(1, 2048 // tn))
    return torch.from_numpy(ti).cuda(), torch.from_numpy(tj).cuda()


def shards_for(ranks, m, K, call):
    g = torch.Generator(device="cuda")
    g.manual_seed(1000 * call + ranks)
    return [torch.randn((m, K), generator=g, device="cuda").to(torch.bfloat16) for _ in range(ranks)]


@pytest.mark.parametrize(("ranks", "me", "m", "K", "N", "tiles"), [
    (2, 1, 512, 1024, 1024, (256, 512, 512)),
    (8, 5, 256, 512, 768, (256, 256, 512)),
    (4, 0, 1024, 256, 512, (512, 512, 256)),
    # w split by columns over the ranks, as the reference's example shards it (examples/collective_matmul.py:64): rank 3
    # of 8 holds 256 of 2048 columns, so there is less compute to hide the gather behind than rows to bring in.
    (8, 3, 512, 1024, 256, (256, 256, 512)),
])
def test_fused_gather_equals_gather_then_gemm_over_three_epochs(ranks, me, m, K, N, tiles):
    tm, tn, tk = tiles
    g = torch.Generator(device="cuda")
    g.manual_seed(7)
    w = torch.randn((K, N), generator=g, device="cuda").to(torch.bfloat16)
    ti, tj = tile_tables(me, ranks, m, N, tm, tn)
    arrivals = torch.zeros(ranks * m // 256, dtype=torch.int32, device="cuda")
    gathered = torch.full((ranks * m, K), float("nan"), dtype=torch.bfloat16, device="cuda")
    out = torch.empty((ranks * m, N), dtype=torch.bfloat16, device="cuda")
    for epoch in (1, 2, 3):  # one arrivals array across calls: the counters are never reset
        shards = shards_for(ranks, m, K, epoch)
        out.fill_(float("nan"))
        ops.all_gather_gemm(shards[me], shards, gathered, w, out, me, tm, tn, tk, ti, tj, arrivals, epoch)
        assert ops.device_status() == 0
        xs = torch.cat(shards)
        want = ops.gemm(xs, w, tm, tn, tk)
        assert torch.equal(out, want), (ranks, me, epoch)
        rows = slice(None, None, 61)
        exact = xs[rows].double() @ w.double()
        np.testing.assert_allclose(out[rows].double().cpu().numpy(), exact.cpu().numpy(), rtol=2e-2, atol=0.5)
        # The copier warps brought every other rank's rows in; the own rows are never written.
        for r in range(ranks):
            got = gathered[r * m : (r + 1) * m]
            if r == me:
                assert (torch.isnan(got).all() if epoch == 1 else True)
            else:
                assert torch.equal(got, shards[r])
        assert int(arrivals.min()) >= 0


def test_a_wait_that_cannot_end_gives_up_reports_105_and_leaves_the_gpu_usable():
    ranks, me, m, K, N, (tm, tn, tk) = 2, 0, 256, 256, 256, (256, 256, 256)
    shards = shards_for(ranks, m, K, 9)
    w = shards_for(1, K, N, 10)[0]
    ti, tj = tile_tables(me, ranks, m, N, tm, tn)
    arrivals = torch.zeros(ranks * m // 256, dtype=torch.int32, device="cuda")
    gathered = torch.zeros((ranks * m, K), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((ranks * m, N), dtype=torch.bfloat16, device="cuda")
    ops.set_wait_limit_us(50_000)
    try:
        # Epoch 2 on counters that have seen no call: the tiles of the other rank's rows wait for twice the
        # arrivals this launch's copier warps will ever post.
        ops.all_gather_gemm(shards[me], shards, gathered, w, out, me, tm, tn, tk, ti, tj, arrivals, 2)
        with pytest.raises(NativeError, match="code 105") as err:
            ops.device_status()
        assert err.value.code == -5  # TJX_E_KERNEL
        assert ops.device_status() == 0  # reading the status cleared it
    finally:
        ops.set_wait_limit_us(2_000_000)
    # The own shard's tiles ran before the wait; and the GPU still computes.
    assert torch.equal(out[:m], ops.gemm(shards[me], w, tm, tn, tk))
    assert torch.equal(ops.gemm(torch.cat(shards), w, tm, tn, tk)[m:], ops.gemm(shards[1], w, tm, tn, tk))
    assert ops.device_status() == 0


def test_headline_size_as_rank_4_of_8_on_one_gpu_and_where_its_producers_wait(capsys):
    # 16384 x 8192 x 8192 as eight shards of 2048 rows, walked a shard at a time as AllGatherMatmul walks them. The
    # result is bit-equal to the plain GEMM over the same rows; the kernel's counters say what the gather costs: the
    # producers barely wait for rows to arrive (the copier warps are far ahead), the MMA thread waits longer for its
    # ring slots than in the plain GEMM while the copy shares L2 and the SM-to-L2 paths with the tile loads.
    import ctypes

    from tilejax_b200._lib import check, library

    ranks, me, M, K, N, (tm, tn, tk) = 8, 4, 16384, 8192, 8192, (512, 512, 512)
    m = M // ranks
    shards = shards_for(ranks, m, K, 21)
    w = shards_for(1, K, N, 22)[0]
    order = schedule.collective_row_blocks(me, ranks, m // tm)
    per = m // tm
    parts = [collective.banded_tiles(order[s * per : (s + 1) * per], N // tn, 2048 // tn) for s in range(ranks)]
    ti = torch.from_numpy(np.concatenate([p[0] for p in parts])).cuda()
    tj = torch.from_numpy(np.concatenate([p[1] for p in parts])).cuda()
    arrivals = torch.zeros(M // 256, dtype=torch.int32, device="cuda")
    gathered = torch.zeros((M, K), dtype=torch.bfloat16, device="cuda")
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    xs = torch.cat(shards)

    def counters(launch):
        buf = torch.zeros(148 * 16, dtype=torch.int64, device="cuda")
        check(library().tjx_set_profile_buffer(ctypes.c_void_p(buf.data_ptr()), buf.numel() * 8))
        try:
            launch()
            torch.cuda.synchronize()
        finally:
            check(library().tjx_set_profile_buffer(None, 0))
        return buf.cpu().numpy().reshape(-1, 16)

    ops.all_gather_gemm(shards[me], shards, gathered, w, out, me, tm, tn, tk, ti, tj, arrivals, 1)  # warm
    fused = counters(lambda: ops.all_gather_gemm(shards[me], shards, gathered, w, out, me, tm, tn, tk, ti, tj, arrivals, 2))
    assert ops.device_status() == 0
    want = ops.gemm(xs, w, tm, tn, tk)
    plain = counters(lambda: ops.gemm(xs, w, tm, tn, tk))
    assert torch.equal(out, want)
    for r in range(ranks):
        if r != me:
            assert torch.equal(gathered[r * m : (r + 1) * m], shards[r])
    life, plain_life = fused[:, 7] - fused[:, 0], plain[:, 7] - plain[:, 0]
    issuing = fused[:, 6] > 0
    copier_done = fused[:, 11] - fused[:, 0]
    assert (copier_done > 0).all() and (copier_done <= life).all()
    assert (fused[:, 10] >= 0).all() and fused[:, 10].mean() < 0.05 * life.mean()
    with capsys.disabled():
        print(f"\n  cycles per CTA (mean): plain GEMM {plain_life.mean():.0f}, of which the MMA thread waits for inputs "
              f"{plain[plain[:, 6] > 0, 3].mean():.0f}; as rank {me} of {ranks}: {life.mean():.0f}, MMA thread waits "
              f"{fused[issuing, 3].mean():.0f}, producers wait for gathered rows {fused[:, 10].mean():.0f} "
              f"(max {fused[:, 10].max()}), copier warps done after {copier_done.mean():.0f} (max {copier_done.max()})")
