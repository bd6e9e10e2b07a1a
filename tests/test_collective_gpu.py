"""The collective matmul on two B200s: both transports against a plain all-gather + the same GEMM, and against
float64 on sampled rows. Needs two GPUs (skipped on a one-GPU box); each rank is its own process."""

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu

WORKER = """
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, {root!r})
from tilejax_b200 import ops
from tilejax_b200.collective import AllGatherMatmul
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
m, K, N = 1024, 1024, 1536
g = torch.Generator(device="cuda"); g.manual_seed(100 + rank)
x = torch.randn((m, K), generator=g, device="cuda").to(torch.bfloat16)
g.manual_seed(7)
w = torch.randn((K, N), generator=g, device="cuda").to(torch.bfloat16)
parts = [torch.empty_like(x) for _ in range(world)]
dist.all_gather(parts, x)
xs = torch.cat(parts)
want = ops.gemm(xs, w, 256, 512, 512)                      # the same kernel on rows already gathered
exact = (xs[::97].double() @ w.double())
for transport in ("fused", "peer", "nccl"):
    op = AllGatherMatmul(m, K, N, 256, 512, 512, transport=transport)
    op.MAX_EPOCH = 2                                         # the arrival counters start over at the third call
    for call in range(3):                                    # several calls: both halves of the send buffer
        xc = (x * (call + 1)).to(torch.bfloat16)
        out = op(xc, w).clone()
        torch.cuda.synchronize()
        assert torch.equal(out, ops.gemm((xs * (call + 1)).to(torch.bfloat16), w, 256, 512, 512)), (transport, call)
    assert (out[::97].double() / 3 - exact).abs().max() <= 2e-2 * exact.abs().max()
    assert ops.device_status() == 0
    # Host buffers in, host result out, pipelined: the same bits, two calls (both halves of the send buffer).
    x_host, w_host = x.cpu().pin_memory(), w.cpu().pin_memory()
    out_host = torch.empty((world * m, N), dtype=torch.bfloat16).pin_memory()
    for call in range(2):
        out_host.fill_(float("nan"))
        op.from_host(x_host, w_host, out_host, chunks=4)
        op.host_done.synchronize()
        assert torch.equal(out_host, want.cpu()), (transport, "from_host", call)
    # The same with w read a part per rank and all-gathered over NVLink (w is the same on every rank here), own rows back.
    out_host.fill_(float("nan"))
    op.from_host(x_host, w_host, out_host, chunks=4, copy_back="own", w_replicated=True)
    op.host_done.synchronize()
    assert torch.equal(out_host[rank * m : (rank + 1) * m], want[rank * m : (rank + 1) * m].cpu()), (transport, "shared w")
    assert torch.equal(op.out, want), (transport, "shared w, device result")
dist.barrier()
dist.destroy_process_group()
sys.stdout.write("rank %d ok\\n" % rank)
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_agree_with_gather_then_matmul(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent(WORKER.format(root=str(ROOT))))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    out = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
         "127.0.0.1", "--master-port", "29541", str(script)],
        env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-3000:]
    assert "rank 0 ok" in out.stdout and "rank 1 ok" in out.stdout
