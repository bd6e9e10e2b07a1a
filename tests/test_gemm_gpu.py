"""The matmul step loop through the C ABI against the oracle: `matmul` (examples/matmul.py) and
`causal_matmul` (examples/causal_matmul.py) semantics, bf16 in, f32 accumulation.

Tolerances: bf16 outputs by the reference's compare rule (rtol 2e-2, atol 2e-2 * max|want|,
src/autokernel/api.py:329-350); f32 accumulators within 1e-5 of the largest value.
"""

import numpy as np
import pytest
import torch
from helpers import f64, rand_bf16, to_device, to_host

import oracle
from tilejax_b200 import ops, schedule
from tilejax_b200._lib import NativeError

pytestmark = pytest.mark.gpu


def run_matmul(x, y, tiles, **kw):
    out = ops.matmul(to_device(x), to_device(y), *tiles, **kw)
    assert ops.device_status() == 0
    return to_host(out)


@pytest.mark.parametrize(("shape", "tiles"), [
    ((256, 384, 256), (128, 128, 128)),   # tests/test_api.py:20-30
    ((128, 64, 128), (128, 128, 128)),    # one tile, one step
    ((512, 512, 512), (512, 512, 512)),   # one user tile of 8 CTA tiles
    ((1024, 256, 768), (256, 256, 128)),
    ((384, 1024, 640), (128, 128, 512)),
    ((200, 72, 264), (512, 512, 512)),    # tiles clipped to a ragged matrix
])
def test_matmul_matches_the_oracle(shape, tiles):
    M, K, N = shape
    x, y = rand_bf16((M, K), 0), rand_bf16((K, N), 1)
    want = oracle.matmul_ref(x, y, *tiles)
    got = run_matmul(x, y, tiles)
    oracle.compare("matmul", got, want)
    np.testing.assert_allclose(f64(got), f64(x) @ f64(y), rtol=2e-2, atol=0.5)  # and float64, as the reference tests


def test_f32_accumulators_are_within_1e5_relative():
    x, y = rand_bf16((512, 2048), 0), rand_bf16((2048, 512), 1)
    got = run_matmul(x, y, (256, 256, 512), out_dtype=torch.float32)
    want = f64(x) @ f64(y)
    assert got.dtype == np.float32
    assert np.abs(f64(got) - want).max() <= 1e-5 * np.abs(want).max()
    oracle.compare("matmul f32", got, oracle.matmul_ref(x, y, 256, 256, 512, out_dtype=np.float32),
                   input_dtypes=(x.dtype, y.dtype))


def test_x_times_y_transposed_reads_y_in_place():
    # `a @ b.T` contracts both last dimensions (src/autokernel/mxu.py:38-43).
    x, y = rand_bf16((256, 192), 0), rand_bf16((384, 192), 1)
    out = ops.gemm(to_device(x), to_device(y), 128, 128, 64, y_transposed=True)
    np.testing.assert_allclose(f64(to_host(out)), f64(x) @ f64(y).T, rtol=2e-2, atol=0.5)


@pytest.mark.parametrize(("n", "k", "tiles"), [(512, 256, (128, 128, 128)), (1024, 512, (512, 512, 512)),
                                               (1024, 256, (256, 512, 128)), (1024, 256, (512, 256, 256)),
                                               (128, 128, (128, 128, 128))])
def test_causal_matmul_matches_the_oracle_and_writes_every_fill(n, k, tiles):
    x, y = rand_bf16((n, k), 0), rand_bf16((k, n), 1)
    want = oracle.causal_matmul_ref(x, y, *tiles)
    # The output starts as NaN: a skipped tile the kernel did not fill, or any tile it missed, stays NaN.
    out = torch.full((n, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.causal_matmul(to_device(x), to_device(y), *tiles, out=out)
    assert ops.device_status() == 0
    got = to_host(out)
    oracle.compare("causal_matmul", got, want)
    assert not f64(got)[np.triu_indices(n, 1)].any()  # exact zeros above the diagonal


def test_tile_tables_are_walked_as_given():
    # Only the listed tiles are computed, only the listed fills are zeroed; the rest of `out` is untouched.
    x, y = rand_bf16((512, 128), 0), rand_bf16((128, 512), 1)
    tile_i = to_device(np.array([3, 0, 2], np.int32))
    tile_j = to_device(np.array([1, 0, 3], np.int32))
    fill_i = to_device(np.array([1], np.int32))
    fill_j = to_device(np.array([2], np.int32))
    out = torch.full((512, 512), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.gemm(to_device(x), to_device(y), 128, 128, 128, tile_i=tile_i, tile_j=tile_j, fill_i=fill_i, fill_j=fill_j,
             out=out)
    got = f64(to_host(out)).reshape(4, 128, 4, 128).transpose(0, 2, 1, 3)
    want = (f64(x) @ f64(y)).reshape(4, 128, 4, 128).transpose(0, 2, 1, 3)
    for i in range(4):
        for j in range(4):
            if (i, j) in ((3, 1), (0, 0), (2, 3)):
                np.testing.assert_allclose(got[i, j], want[i, j], rtol=2e-2, atol=0.5)
            elif (i, j) == (1, 2):
                assert not got[i, j].any()
            else:
                assert (got[i, j] == 7.0).all()


def test_collective_row_order_computes_shards_in_any_order():
    # all_gather_matmul walks row blocks a shard at a time, own shard first; the result does not depend on it.
    x, y = rand_bf16((1024, 256), 0), rand_bf16((256, 256), 1)
    order = schedule.collective_row_blocks(2, 4, 2)  # chip 2 of 4, 2 blocks of 128 rows per shard
    tile_i = to_device(np.repeat(order, 2).astype(np.int32))
    tile_j = to_device(np.tile(np.arange(2, dtype=np.int32), 8))
    out = ops.gemm(to_device(x), to_device(y), 128, 128, 256, tile_i=tile_i, tile_j=tile_j)
    plain = ops.gemm(to_device(x), to_device(y), 128, 128, 256)
    assert torch.equal(out, plain)


def test_full_size_causal_matmul_properties():
    # 8192^2 x 8192 at the benchmark's two tilings: exact zeros above the diagonal, exact agreement between the
    # tilings' computed entries being not required, sampled rows against float64, and bit-exact tables.
    n = 8192
    x, y = rand_bf16((n, n), 0), rand_bf16((n, n), 1)
    xd, yd = to_device(x), to_device(y)
    rows = np.array([0, 1, 127, 128, 511, 512, 1023, 1024, 4095, 4096, 6000, 8191])
    want = np.tril(f64(x)[rows] @ f64(y), 0)
    want = np.where(np.arange(n)[None, :] <= rows[:, None], f64(x)[rows] @ f64(y), 0.0)
    for tiles in ((512, 512, 512), (1024, 2048, 1024)):
        out = torch.full((n, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.causal_matmul(xd, yd, *tiles, out=out)
        assert ops.device_status() == 0
        assert not torch.isnan(out).any()
        assert not torch.triu(out, 1).any()
        got = f64(to_host(out[torch.from_numpy(rows).cuda()]))
        assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()
        sch = schedule.causal_matmul_schedule(n, n, n, *tiles)
        for name, values in oracle.causal_tile_tables(n, n, tiles[0], tiles[1]).items():
            np.testing.assert_array_equal(sch.tables[name], values)


def test_dense_4096_against_sampled_float64_rows_and_linearity():
    n = 4096
    x, y = rand_bf16((n, n), 0), rand_bf16((n, n), 1)
    xd, yd = to_device(x), to_device(y)
    out = ops.matmul(xd, yd, 512, 512, 512, out_dtype=torch.float32)
    rows = np.array([0, 777, 2048, 4095])
    want = f64(x)[rows] @ f64(y)
    assert np.abs(f64(to_host(out[torch.from_numpy(rows).cuda()])) - want).max() <= 1e-5 * np.abs(want).max()
    # Linearity in x: (2 x) @ y == 2 (x @ y) exactly (scaling by 2 is exact in bf16 and f32).
    twice = ops.matmul(xd * 2, yd, 512, 512, 512, out_dtype=torch.float32)
    assert torch.equal(twice, out * 2)
    # Tiling does not change which products are summed: other tiles agree within accumulation-order noise.
    other = ops.matmul(xd, yd, 1024, 2048, 1024, out_dtype=torch.float32)
    assert (other - out).abs().max().item() <= 1e-5 * np.abs(want).max()


@pytest.mark.parametrize(("shape", "tiles", "kw"), [
    ((256, 64, 256), (256, 256, 64), {}),                         # one 256 x 256 piece, one reduction block
    ((512, 512, 512), (512, 512, 512), {}),
    ((1024, 768, 1536), (256, 512, 256), {"out_f32": True}),
    ((1024, 8192, 512), (256, 256, 512), {}),                     # a long reduction: many trips round the ring
    ((2048, 256, 2048), (512, 256, 256), {"causal": True}),
    ((4096, 512, 4096), (512, 512, 512), {}),                     # more pieces than SM pairs: persistent loop
    # A last round that keeps at most half the SM pairs busy is run on half pieces (N = 128), two pairs a piece:
    ((2560, 256, 2560), (256, 256, 256), {}),                     # 100 pieces: 74 + 26
    ((2560, 320, 2560), (512, 256, 64), {"out_f32": True}),
    ((3584, 256, 3584), (512, 512, 256), {"causal": True}),       # 105 computing pieces: 74 + 31, dealt out from lists
    ((3328, 128, 3328), (256, 256, 128), {"causal": True}),       # 91 = 74 + 17
    ((2560, 200, 2816), (256, 256, 64), {}),                      # K not a multiple of the K block: 110 pieces = 74 + 36
])
def test_sm_pairs_and_single_ctas_agree_bit_for_bit(shape, tiles, kw):
    # One MMA per pair of SMs (256 x 256 pieces) and one per SM (128 x 256) sum K in the same order.
    M, K, N = shape
    x, y = to_device(rand_bf16((M, K), 0)), to_device(rand_bf16((K, N), 1))
    dtype = torch.float32 if kw.get("out_f32") else torch.bfloat16
    outs = []
    try:
        for pairs in (True, False):
            ops.set_gemm_pair_mode(pairs)
            out = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
            if kw.get("causal"):
                ops.causal_matmul(x, y, *tiles, out=out)
            else:
                ops.gemm(x, y, *tiles, out=out, out_dtype=dtype)
            assert ops.device_status() == 0
            outs.append(out)
    finally:
        ops.set_gemm_pair_mode(True)
    assert not torch.isnan(outs[0]).any()
    assert torch.equal(outs[0], outs[1])
    want = f64(to_host(x))[:8] @ f64(to_host(y))
    if kw.get("causal"):
        want = np.where(np.arange(N)[None, :] <= np.arange(8)[:, None], want, 0.0)
    got = f64(to_host(outs[0][:8]))
    assert np.abs(got - want).max() <= 2e-2 * max(np.abs(want).max(), 1.0)


def test_sm_pairs_with_y_transposed_tables_and_a_cta_limit():
    x, y = rand_bf16((1024, 256), 0), rand_bf16((512, 256), 1)
    xd, yd = to_device(x), to_device(y)
    tile_i = to_device(np.array([3, 0, 2, 1], np.int32))
    tile_j = to_device(np.array([1, 0, 1, 0], np.int32))
    fill_i = to_device(np.array([1, 2], np.int32))
    fill_j = to_device(np.array([1, 0], np.int32))
    outs = []
    try:
        for pairs, limit in ((True, 6), (True, 0), (False, 0)):
            ops.set_gemm_pair_mode(pairs)
            ops.set_gemm_cta_limit(limit)
            out = torch.full((1024, 512), 7.0, dtype=torch.bfloat16, device="cuda")
            ops.gemm(xd, yd, 256, 256, 256, y_transposed=True, tile_i=tile_i, tile_j=tile_j, fill_i=fill_i,
                     fill_j=fill_j, out=out)
            assert ops.device_status() == 0
            outs.append(out)
    finally:
        ops.set_gemm_pair_mode(True)
        ops.set_gemm_cta_limit(0)
    assert torch.equal(outs[0], outs[2]) and torch.equal(outs[1], outs[2])
    got = f64(to_host(outs[0])).reshape(4, 256, 2, 256).transpose(0, 2, 1, 3)
    want = (f64(x) @ f64(y).T).reshape(4, 256, 2, 256).transpose(0, 2, 1, 3)
    for i in range(4):
        for j in range(2):
            if (i, j) in ((3, 1), (0, 0), (2, 1), (1, 0)):
                np.testing.assert_allclose(got[i, j], want[i, j], rtol=2e-2, atol=0.5)
            elif (i, j) in ((1, 1), (2, 0)):
                assert not got[i, j].any()
            else:
                assert (got[i, j] == 7.0).all()


def test_host_pipeline_matches_the_device_call():
    # One rank: x and w from pinned host memory in pieces, result back to pinned host memory, against the plain call.
    from tilejax_b200.collective import AllGatherMatmul

    m, K, N = 2048, 512, 1024
    x, w = rand_bf16((m, K), 0), rand_bf16((K, N), 1)
    op = AllGatherMatmul(m, K, N, 256, 512, 512)
    want = op(to_device(x), to_device(w)).clone()
    x_host, w_host = to_device(x).cpu().pin_memory(), to_device(w).cpu().pin_memory()
    out_host = torch.empty((m, N), dtype=torch.bfloat16).pin_memory()
    for chunks in (8, 3, 1):  # 3 does not divide the 8 row blocks: the largest divisor below it is used
        out_host.fill_(float("nan"))
        op.from_host(x_host, w_host, out_host, chunks=chunks)
        op.host_done.synchronize()
        assert ops.device_status() == 0
        assert torch.equal(out_host, want.cpu())


def test_bad_arguments_are_errors():
    x = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(NativeError, match="multiple of 128"):
        ops.gemm(x, x, 64, 128, 128)
    with pytest.raises(NativeError, match="cover M and N"):
        ops.gemm(torch.zeros(384, 256, dtype=torch.bfloat16, device="cuda"), x, 256, 128, 128)
    with pytest.raises(NativeError, match="multiples of 8"):
        ops.gemm(torch.zeros(128, 100, dtype=torch.bfloat16, device="cuda"),
                 torch.zeros(100, 128, dtype=torch.bfloat16, device="cuda"), 128, 128, 100)
    with pytest.raises(ValueError, match="bfloat16"):
        ops.gemm(x.float(), x, 128, 128, 128)
    with pytest.raises(NativeError, match="mode must be 0"):
        ops.set_gemm_pair_mode(5)
    # The one-launch all-gather matmul checks its shapes before anything runs.
    tables = torch.zeros(4, dtype=torch.int32, device="cuda")
    arrivals = torch.zeros(2, dtype=torch.int32, device="cuda")
    big = torch.zeros(512, 256, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(512, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(NativeError, match="tile table must list every tile"):
        ops.all_gather_gemm(x, [None, x], big, x, out, 0, 256, 256, 256, tables[:3], tables[:3], arrivals, 1)
    with pytest.raises(NativeError, match="multiples of 256"):
        ops.all_gather_gemm(x, [None, x], big, x, out, 0, 128, 256, 256, tables, tables, arrivals, 1)
    with pytest.raises(NativeError, match="epoch"):
        ops.all_gather_gemm(x, [None, x], big, x, out, 0, 256, 256, 256, tables[:2], tables[:2], arrivals, 0)
