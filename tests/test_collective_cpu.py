"""The collective matmul's host logic on CPU: the exchange plan, and the shard exchange itself over gloo with two
ranks (the data movement is backend-agnostic; the GEMM it feeds has no CPU path and is not run here)."""

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np

from tilejax_b200 import schedule
from tilejax_b200.collective import banded_tiles, exchange_rounds, shard_order

ROOT = Path(__file__).resolve().parent.parent


def test_exchange_rounds_deliver_shards_in_the_reference_ring_order():
    # Round r receives the shard of rank (me - r) mod G: the order the reference's tiles walk
    # (src/autokernel/plan.py:225-238); sends and receives pair up across ranks in every round.
    for ranks in (1, 2, 4, 8):
        for me in range(ranks):
            rounds = exchange_rounds(me, ranks)
            assert [r.recv_from for r in rounds] == [(me - r) % ranks for r in range(1, ranks)]
            assert shard_order(me, ranks) == [int(b) for b in schedule.collective_row_blocks(me, ranks, 1)]
            for rnd in rounds:
                peer = exchange_rounds(rnd.send_to, ranks)[rnd.step - 1]
                assert peer.recv_from == me
    assert exchange_rounds(0, 1) == []


def test_banded_tile_tables_list_every_tile_once_shard_by_shard():
    # A shard's tiles in column bands: every (row block, column tile) exactly once, a band's tiles together, and
    # within a band row block by row block — for ragged band counts too.
    for col_tiles, band in ((16, 4), (6, 4), (3, 1), (5, 8)):
        rows = schedule.collective_row_blocks(1, 4, 3)[3:6]  # the second shard rank 1 of 4 computes
        ti, tj = banded_tiles(rows, col_tiles, band)
        assert ti.dtype == np.int32 and tj.dtype == np.int32
        assert sorted(zip(ti.tolist(), tj.tolist())) == sorted((int(r), c) for r in rows for c in range(col_tiles))
        bands = (tj // band).tolist()
        assert bands == sorted(bands)
        first_band = [(i, j) for i, j in zip(ti.tolist(), tj.tolist()) if j < band]
        assert first_band == [(int(r), c) for r in rows for c in range(min(band, col_tiles))]


WORKER = """
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, {root!r})
from tilejax_b200.collective import ShardExchange
from tilejax_b200.autokernel import kernels as K
dist.init_process_group("gloo")
me, ranks = dist.get_rank(), dist.get_world_size()
m, Kdim = 64, 32
x = torch.full((m, Kdim), float(me + 1)) + torch.arange(m)[:, None] / 1000
ex = ShardExchange(m, Kdim, torch.float32, torch.device("cpu"))
xs = ex.gather(x)
for r in range(ranks):
    want = torch.full((m, Kdim), float(r + 1)) + torch.arange(m)[:, None] / 1000
    assert torch.equal(xs[r * m : (r + 1) * m], want), (me, r)
# The loop nest as plain code gathers through the process group too, and plans for the gathered shape.
import ml_dtypes
xb = (np.arange(128 * 128, dtype=np.float32).reshape(128, 128) % 7 + me).astype(ml_dtypes.bfloat16)
wb = np.ones((128, 128), np.float32).astype(ml_dtypes.bfloat16)
out = K.all_gather_matmul.reference(xb, wb, K.CollectiveTiles(tm=128, tn=128, tk=128))
assert out.shape == (ranks * 128, 128)
for r in range(ranks):
    rows = (np.arange(128 * 128, dtype=np.float32).reshape(128, 128) % 7 + r)
    assert np.array_equal(out[r * 128 : (r + 1) * 128].astype(np.float32), (rows @ np.ones((128, 128), np.float32)).astype(ml_dtypes.bfloat16).astype(np.float32))
sig = K.all_gather_matmul.signature(xb, wb)
assert sig[-1][0] == (ranks * 128, 128)
plan, sch = K.all_gather_matmul.build(sig, K.CollectiveTiles(tm=128, tn=128, tk=128))
assert sch.steps == ranks and plan.params["chips"] == ranks
dist.barrier()
dist.destroy_process_group()
print("rank %d ok" % me, flush=True)
"""


def test_two_ranks_exchange_their_shards_over_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent(WORKER.format(root=str(ROOT))))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    out = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
         "127.0.0.1", "--master-port", "29533", str(script)],
        env=env, capture_output=True, text=True, timeout=240)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "rank 0 ok" in out.stdout and "rank 1 ok" in out.stdout
