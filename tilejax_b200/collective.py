"""The collective matmul: `all_gather(x) @ w`, the gather overlapped with the tile compute.

Meaning as the reference's `all_gather_matmul` (examples/collective_matmul.py:44-59): every rank holds m rows of
x and computes all ranks' rows times its own w. The reference passes shards around a ring of chips inside its
kernel (src/autokernel/codegen.py:1156-1229) and walks the row blocks a shard at a time, its own first, then the
shard of rank (me - r) mod G at ring step r (src/autokernel/plan.py:225-238).

On NVLink 5 behind NVSwitch every peer is one hop away at full bandwidth, so the ring is unrolled into G - 1
direct exchanges: in round r a rank sends its own shard to (me + r) mod G and receives the shard of (me - r) mod G
straight into its place in the local gathered buffer `xs` — the same arrival order the reference's tile walk
expects. The rounds run on a communication stream over NCCL; the compute stream starts on the rank's own shard
at once and waits, per shard, only for that shard's round. The GEMM kernel always reads this GPU's own memory.

`ShardExchange` is the data movement alone and works on any backend (the host logic is tested with gloo on
CPU tensors); `AllGatherMatmul` adds the sm_100a GEMM and has no CPU path.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

from . import schedule as _schedule


@dataclass(frozen=True)
class Round:
    """One exchange: send the own shard to `send_to`, receive the shard of `recv_from` (its rows of xs)."""

    step: int
    send_to: int
    recv_from: int


def exchange_rounds(me: int, ranks: int) -> list[Round]:
    """Rounds 1 .. ranks - 1 of the unrolled ring: round r receives rank (me - r) mod ranks' shard."""
    return [Round(r, (me + r) % ranks, (me - r) % ranks) for r in range(1, ranks)]


def shard_order(me: int, ranks: int) -> list[int]:
    """Shards in the order rank `me` computes them: own first, then as the rounds deliver them."""
    return [me] + [r.recv_from for r in exchange_rounds(me, ranks)]


class ShardExchange:
    """Gathers every rank's [m, K] shard into a local [ranks * m, K] buffer, one round at a time."""

    def __init__(self, m: int, K: int, dtype: torch.dtype, device: torch.device, group=None):
        self.group = group
        self.ranks = dist.get_world_size(group) if dist.is_initialized() else 1
        self.me = dist.get_rank(group) if dist.is_initialized() else 0
        self.m, self.K = m, K
        self.xs = torch.empty((self.ranks * m, K), dtype=dtype, device=device)
        self.rounds = exchange_rounds(self.me, self.ranks)

    def rows(self, rank: int) -> torch.Tensor:
        return self.xs[rank * self.m : (rank + 1) * self.m]

    def _global(self, rank: int) -> int:
        return rank if self.group is None else dist.get_global_rank(self.group, rank)

    def start_round(self, x: torch.Tensor, rnd: Round) -> list:
        """Enqueue one round's send and receive; returns the requests to wait on."""
        ops = [
            dist.P2POp(dist.isend, x, self._global(rnd.send_to), self.group),
            dist.P2POp(dist.irecv, self.rows(rnd.recv_from), self._global(rnd.recv_from), self.group),
        ]
        return dist.batch_isend_irecv(ops)

    def gather(self, x: torch.Tensor) -> torch.Tensor:
        """The whole gather, blocking: xs with every rank's rows in rank order (all_gather, tiled)."""
        self.rows(self.me).copy_(x)
        for rnd in self.rounds:
            for req in self.start_round(x, rnd):
                req.wait()
        return self.xs


class AllGatherMatmul:
    """out = all_gather(x) @ w on each rank, [ranks * m, N] bf16, with the gather hidden behind the compute.

    Buffers (xs, out), the tile tables of each shard, the communication stream and the events are made once;
    a call only enqueues work. `reserve_sms` leaves that many SMs free of GEMM CTAs while exchanges are in
    flight, for NCCL's copy kernels to run beside the persistent GEMM.
    """

    def __init__(self, m: int, K: int, N: int, tm: int = 256, tn: int = 512, tk: int = 512, group=None,
                 device: torch.device | None = None, reserve_sms: int = 16):
        from . import ops  # needs the built library

        self._ops = ops
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.device = device
        self.exchange = ShardExchange(m, K, torch.bfloat16, device, group)
        self.ranks, self.me = self.exchange.ranks, self.exchange.me
        self.m, self.K, self.N = m, K, N
        self.tm, self.tn, self.tk = min(tm, m), min(tn, N), min(tk, K)
        if m % self.tm:
            raise ValueError("tile rows must divide a shard")  # src/autokernel/plan.py:845-871
        self.out = torch.empty((self.ranks * m, N), dtype=torch.bfloat16, device=device)
        self.comm_stream = torch.cuda.Stream(device=device)
        self.x_ready = torch.cuda.Event()
        self.arrived = [torch.cuda.Event() for _ in self.exchange.rounds]
        self.done = torch.cuda.Event()
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        self.cta_limit = max(1, sms - reserve_sms) if self.ranks > 1 and reserve_sms > 0 else 0
        # Tile tables per received shard: its row blocks (in order) x every column block, row-major. The own
        # shard needs none: its tiles are read straight from x.
        shard_blocks = m // self.tm
        cols = np.arange(N // self.tn, dtype=np.int32)
        order = _schedule.collective_row_blocks(self.me, self.ranks, shard_blocks)
        self.tables = []
        for s in range(1, self.ranks):
            rows = order[s * shard_blocks : (s + 1) * shard_blocks]
            ti = torch.from_numpy(np.repeat(rows, cols.size).astype(np.int32)).to(device)
            tj = torch.from_numpy(np.tile(cols, rows.size).astype(np.int32)).to(device)
            self.tables.append((ti, tj))

    @property
    def steps(self) -> int:
        """Steps of the reference's schedule: every (tile, reduction block)."""
        return (self.ranks * self.m // self.tm) * (self.N // self.tn) * (self.K // self.tk)

    def __call__(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        ops, ex = self._ops, self.exchange
        if x.shape != (self.m, self.K) or w.shape != (self.K, self.N):
            raise ValueError("x must be this rank's (m, K) shard and w (K, N)")
        compute = torch.cuda.current_stream(self.device)
        own_out = self.out[self.me * self.m : (self.me + 1) * self.m]
        if self.ranks == 1:
            ops.gemm(x, w, self.tm, self.tn, self.tk, out=own_out)
            return self.out
        # Communication stream: all rounds, in the order the tiles will want them.
        self.x_ready.record(compute)
        self.comm_stream.wait_event(self.x_ready)
        self.comm_stream.wait_event(self.done)  # the previous call's GEMMs have finished reading xs
        with torch.cuda.stream(self.comm_stream):
            for rnd, event in zip(ex.rounds, self.arrived, strict=True):
                for req in ex.start_round(x, rnd):
                    req.wait()
                event.record(self.comm_stream)
        # Compute stream: the own shard at once, straight from x (it is never copied), then each shard as its
        # round completes. While rounds are in flight the GEMM leaves a few SMs to the exchange's kernels.
        try:
            ops.set_gemm_cta_limit(self.cta_limit)
            ops.gemm(x, w, self.tm, self.tn, self.tk, out=own_out)
            for s, (ti, tj) in enumerate(self.tables):
                compute.wait_event(self.arrived[s])
                if s == len(self.tables) - 1:
                    ops.set_gemm_cta_limit(0)  # nothing is in flight behind the last shard
                ops.gemm(ex.xs, w, self.tm, self.tn, self.tk, tile_i=ti, tile_j=tj, out=self.out)
        finally:
            ops.set_gemm_cta_limit(0)
        self.done.record(compute)
        return self.out
