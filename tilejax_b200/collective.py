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

`ShardExchange` is that data movement over `torch.distributed` send / receive and works on any backend (the host
logic is tested with gloo on CPU tensors). `PeerExchange` does the same rounds as copy-engine pulls from the peers'
symmetric memory over NVLink, which take no SM away from the GEMM; it is the default on GPUs. `AllGatherMatmul`
adds the sm_100a GEMM and has no CPU path.
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


class PeerExchange:
    """The same gather over NVLink peer memory instead of NCCL kernels: every rank keeps its shard in a
    symmetric-memory buffer that its peers map, and each round is one device-to-device copy from the peer's
    buffer into this GPU's own `xs` — issued on the communication stream, carried by the copy engines, so the
    exchange takes no SM from the GEMM. A stream-ordered barrier over the buffer's signal pads (one tiny kernel)
    tells every rank that all shards of this call are in place; the send buffer is double-buffered so a rank may
    write call k + 1's shard while peers still read call k's."""

    def __init__(self, m: int, K: int, dtype: torch.dtype, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = dist.group.WORLD if group is None else group
        self.ranks, self.me = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.m, self.K = m, K
        self.send = symm_mem.empty((2, m, K), dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.send, self.group)
        self.peers = [self.handle.get_buffer(r, (2, m, K), dtype, 0) for r in range(self.ranks)]
        self.xs = torch.empty((self.ranks * m, K), dtype=dtype, device=device)
        self.rounds = exchange_rounds(self.me, self.ranks)
        self.calls = 0

    def rows(self, rank: int) -> torch.Tensor:
        return self.xs[rank * self.m : (rank + 1) * self.m]

    def shard_buffer(self) -> torch.Tensor:
        """Where the next call's shard goes: writing x here directly saves the copy into the send buffer."""
        return self.send[self.calls & 1]

    def barrier(self) -> None:
        """All ranks' current-stream work so far is done (enqueued on the current stream)."""
        self.handle.barrier(channel=0)

    def pull(self, rnd: Round, parity: int) -> None:
        """Round `rnd`: copy the shard of rank rnd.recv_from from its send buffer into this GPU's xs."""
        self.rows(rnd.recv_from).copy_(self.peers[rnd.recv_from][parity], non_blocking=True)


def banded_tiles(row_blocks: np.ndarray, col_tiles: int, band: int) -> tuple[np.ndarray, np.ndarray]:
    """(tile_i, tile_j) over `row_blocks` x all `col_tiles` column tiles, walked in column bands `band` tiles wide:
    within a band row block by row block. The CTAs in flight then share a band's slice of y, which stays in L2,
    instead of streaming all of y once per row block. Every tile appears exactly once."""
    ti, tj = [], []
    for first in range(0, col_tiles, band):
        cols = np.arange(first, min(first + band, col_tiles), dtype=np.int32)
        ti.append(np.repeat(row_blocks.astype(np.int32), cols.size))
        tj.append(np.tile(cols, row_blocks.size))
    return np.concatenate(ti), np.concatenate(tj)


def shard_groups(ranks: int) -> list[list[int]]:
    """Which shards (in arrival order: 0 is the own shard) each GEMM launch covers: the own shard alone first —
    nothing has arrived yet — then the shards that arrive while it runs, then the rest: three launches at most, so
    the later ones are long enough to fill their waves."""
    if ranks <= 2:
        return [[s] for s in range(ranks)]
    rest = ranks - 1
    first = -(-rest * 3 // 7)
    return [[0], list(range(1, 1 + first)), list(range(1 + first, ranks))]


class AllGatherMatmul:
    """out = all_gather(x) @ w on each rank, [ranks * m, N] bf16, with the gather hidden behind the compute.

    Buffers (xs, out), the tile tables, the communication stream and the events are made once; a call only enqueues
    work. `transport` is "fused" (the default: one GEMM launch whose copier warps pull the peers' shards out of
    symmetric memory; tiles that are not multiples of 256 fall back to "peer"), "peer" (copy-engine pulls from
    peers' symmetric memory on a second stream: no SMs) or "nccl" (send / receive rounds: NCCL's copy kernels need
    SMs, so `reserve_sms` of them are kept free of GEMM CTAs while rounds are in flight; "peer" keeps a few free for
    its barrier kernel).
    """

    MAX_EPOCH = 1 << 20  # calls of the one-launch kernel between resets of its arrival counters (the C ABI takes 2^22)

    def __init__(self, m: int, K: int, N: int, tm: int = 256, tn: int = 512, tk: int = 512, group=None,
                 device: torch.device | None = None, reserve_sms: int | None = None, transport: str = "fused"):
        from . import ops  # needs the built library

        self._ops = ops
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.device = device
        ranks = dist.get_world_size(group) if dist.is_initialized() else 1
        if transport not in ("fused", "peer", "nccl"):
            raise ValueError("transport is 'fused', 'peer' or 'nccl'")
        self.transport = transport if ranks > 1 else "none"
        if self.transport == "fused" and (min(tm, m) % 256 or min(tn, N) % 256):
            self.transport = "peer"  # the fused kernel works in 256 x 256 pieces
        if self.transport in ("peer", "fused"):
            self.exchange = PeerExchange(m, K, torch.bfloat16, device, group)
        else:
            self.exchange = ShardExchange(m, K, torch.bfloat16, device, group)
        self.ranks, self.me = self.exchange.ranks, self.exchange.me
        self.group = group
        self.m, self.K, self.N = m, K, N
        self.tm, self.tn, self.tk = min(tm, m), min(tn, N), min(tk, K)
        if m % self.tm:
            raise ValueError("tile rows must divide a shard")  # src/autokernel/plan.py:845-871
        self.out = torch.empty((self.ranks * m, N), dtype=torch.bfloat16, device=device)
        self.comm_stream = torch.cuda.Stream(device=device)
        self.x_ready = torch.cuda.Event()
        self.barrier_done = torch.cuda.Event()
        self.arrived = [torch.cuda.Event() for _ in self.exchange.rounds]
        self.done = torch.cuda.Event()
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        if reserve_sms is None:
            reserve_sms = {"peer": 4, "nccl": 32}.get(self.transport, 0)
        self.cta_limit = max(1, sms - reserve_sms) if self.ranks > 1 and reserve_sms > 0 else 0
        # One GEMM launch per group of shards; the tile table of a group lists its shards' row blocks, in arrival
        # order, times every column block, row-major. The own shard needs none: its tiles come straight from x.
        shard_blocks = m // self.tm
        col_tiles, band = N // self.tn, max(1, 2048 // self.tn)
        order = _schedule.collective_row_blocks(self.me, self.ranks, shard_blocks)
        self.groups = shard_groups(self.ranks)
        self.tables = []
        for group_shards in self.groups[1:]:
            rows = np.concatenate([order[s * shard_blocks : (s + 1) * shard_blocks] for s in group_shards])
            ti, tj = banded_tiles(rows, col_tiles, band)
            self.tables.append((group_shards[-1], torch.from_numpy(ti).to(device), torch.from_numpy(tj).to(device)))
        if self.transport == "fused":
            # One launch over every tile, a shard at a time — own first, then in arrival order — and in column
            # bands within a shard; the kernel's copier warps count every 256-row block they have brought in.
            parts = [banded_tiles(order[s * shard_blocks : (s + 1) * shard_blocks], col_tiles, band)
                     for s in range(self.ranks)]
            self.all_ti = torch.from_numpy(np.concatenate([p[0] for p in parts])).to(device)
            self.all_tj = torch.from_numpy(np.concatenate([p[1] for p in parts])).to(device)
            self.arrivals = torch.zeros(self.ranks * m // 256, dtype=torch.int32, device=device)
            self.epoch = 0

    @property
    def steps(self) -> int:
        """Steps of the reference's schedule: every (tile, reduction block)."""
        return (self.ranks * self.m // self.tm) * (self.N // self.tn) * (self.K // self.tk)

    def shard_buffer(self) -> torch.Tensor | None:
        """With the peer-memory transports: the buffer to write the next call's x into to save a copy (else None)."""
        return self.exchange.shard_buffer() if self.transport in ("peer", "fused") else None

    def __call__(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        ops = self._ops
        if x.shape != (self.m, self.K) or w.shape != (self.K, self.N):
            raise ValueError("x must be this rank's (m, K) shard and w (K, N)")
        compute = torch.cuda.current_stream(self.device)
        own_out = self.out[self.me * self.m : (self.me + 1) * self.m]
        if self.ranks == 1:
            ops.gemm(x, w, self.tm, self.tn, self.tk, out=own_out)
            return self.out
        if self.transport == "fused":
            staged = self.exchange.send[self.exchange.calls & 1]
            if x.data_ptr() != staged.data_ptr():
                staged.copy_(x, non_blocking=True)  # peers finished with this half before the previous barrier
            self._fused_launch(w)
            self.done.record(compute)
            return self.out
        if self.transport == "peer":
            staged = self.exchange.send[self.exchange.calls & 1]
            if x.data_ptr() != staged.data_ptr():
                # Peers finished reading this half two calls ago, before the previous call's barrier.
                compute.wait_event(self.barrier_done)
                staged.copy_(x, non_blocking=True)
        self.x_ready.record(compute)
        self._start_exchange(x)
        # Compute stream: the own shard at once, straight from x (it is never copied into xs), then each group of
        # shards once its last round has completed. While the exchange is in flight the GEMM leaves it a few SMs.
        try:
            ops.set_gemm_cta_limit(self.cta_limit)
            ops.gemm(x, w, self.tm, self.tn, self.tk, out=own_out)
            self._other_groups(w, compute)
        finally:
            ops.set_gemm_cta_limit(0)
        self.done.record(compute)
        return self.out

    def _fused_launch(self, w: torch.Tensor) -> None:
        """Current stream: a barrier (every rank's shard of this call is in its send buffer, and every rank has
        finished the previous call), then the one launch that gathers and multiplies."""
        ex = self.exchange
        parity = ex.calls & 1
        ex.calls += 1
        ex.barrier()
        self.barrier_done.record(torch.cuda.current_stream(self.device))
        if self.epoch >= self.MAX_EPOCH:
            # The arrival counters only ever grow (a launch waits for epoch x copier warps): start them over, in
            # stream order behind the previous launch, before the entry point's epoch limit is reached.
            self.arrivals.zero_()
            self.epoch = 0
        self.epoch += 1
        shards = [ex.peers[r][parity] for r in range(self.ranks)]
        self._ops.all_gather_gemm(ex.send[parity], shards, ex.xs, w, self.out, self.me, self.tm, self.tn, self.tk,
                                  self.all_ti, self.all_tj, self.arrivals, self.epoch)

    def _start_exchange(self, x: torch.Tensor) -> None:
        """Enqueue the exchange rounds on the communication stream, behind `x_ready` (this rank's shard is in place:
        in the send buffer for the peer transport, in x for nccl)."""
        ex, comm = self.exchange, self.comm_stream
        comm.wait_event(self.x_ready)
        comm.wait_event(self.done)  # the previous call's GEMMs have finished reading xs
        with torch.cuda.stream(comm):
            if self.transport in ("peer", "fused"):
                parity = ex.calls & 1
                ex.calls += 1
                ex.barrier()  # every rank's shard of this call is in its send buffer
                self.barrier_done.record(comm)
                for rnd, event in zip(ex.rounds, self.arrived, strict=True):
                    ex.pull(rnd, parity)
                    event.record(comm)
            else:
                for rnd, event in zip(ex.rounds, self.arrived, strict=True):
                    for req in ex.start_round(x, rnd):
                        req.wait()
                    event.record(comm)

    def _other_groups(self, w: torch.Tensor, compute, after_group=None) -> None:
        """The GEMM launches over the shards that arrive, each behind its last round; `after_group(shards)` is
        called after each launch is enqueued."""
        ops, ex = self._ops, self.exchange
        for n, (last_shard, ti, tj) in enumerate(self.tables):
            compute.wait_event(self.arrived[last_shard - 1])
            if n == len(self.tables) - 1:
                ops.set_gemm_cta_limit(0)  # nothing is in flight behind the last group
            ops.gemm(ex.xs, w, self.tm, self.tn, self.tk, tile_i=ti, tile_j=tj, out=self.out)
            if after_group is not None:
                after_group(self.groups[n + 1])

    def from_host(self, x_host: torch.Tensor, w_host: torch.Tensor, out_host: torch.Tensor, chunks: int = 8,
                  copy_back: str = "all", w_replicated: bool = False) -> None:
        """The same product for operands in pinned host memory, result into pinned host memory: the host-to-device
        copies, the GEMMs and the device-to-host copies run as a pipeline on three streams, so a step costs about
        its slower copy direction instead of the sum of both copies and the compute. w goes first (every tile needs
        it), then this rank's rows of x in `chunks` pieces, each multiplied as soon as it has landed and its rows of
        the result copied back while the next piece is still arriving; the other ranks' shards follow as in
        `__call__`. With `copy_back="own"` only this rank's m rows of the result are copied to `out_host` (where w is
        the same on every rank the result is too, and the ranks together hand the host every row once); the whole
        result stays in `self.out`. With `w_replicated=True` the caller states that w_host holds the same values on
        every rank (as `all_gather_matmul`'s replicated w does): each rank then reads only its 1 / ranks of w's rows from
        its host and the ranks all-gather the parts over NVLink, instead of every rank pulling all of w over PCIe.
        Enqueues only: `out_host` is complete once `host_done` has been synchronised."""
        if copy_back not in ("all", "own"):
            raise ValueError("copy_back is 'all' or 'own'")
        ops = self._ops
        if x_host.shape != (self.m, self.K) or w_host.shape != (self.K, self.N):
            raise ValueError("x must be this rank's (m, K) shard and w (K, N)")
        if out_host.shape != self.out.shape or out_host.dtype != self.out.dtype:
            raise ValueError("out_host must be [ranks * m, N] bfloat16")
        if not (x_host.is_pinned() and w_host.is_pinned() and out_host.is_pinned()):
            raise ValueError("the host buffers must be pinned")
        if not hasattr(self, "_stage"):
            # Two sets of device staging buffers, used alternately, so that the next call's copies never wait for
            # this call's GEMMs: (w, x, "the GEMMs that read this set are done"). With the peer transport x is
            # staged in the send buffer, which already has two halves.
            def stage():
                w = torch.empty((self.K, self.N), dtype=torch.bfloat16, device=self.device)
                x = None if self.transport in ("peer", "fused") else torch.empty(
                    (self.m, self.K), dtype=torch.bfloat16, device=self.device)
                return w, x, torch.cuda.Event()

            self._stage = [stage(), stage()]
            self._host_calls = 0
            self._h2d, self._d2h = torch.cuda.Stream(device=self.device), torch.cuda.Stream(device=self.device)
            self.host_done = torch.cuda.Event()
            self._w_ready = torch.cuda.Event()
        w_dev, x_stage, set_done = self._stage[self._host_calls & 1]
        self._host_calls += 1
        blocks = self.m // self.tm
        chunks = max(c for c in range(1, max(1, min(chunks, blocks)) + 1) if blocks % c == 0)
        rows = self.m // chunks
        compute = torch.cuda.current_stream(self.device)
        h2d, d2h = self._h2d, self._d2h
        # (With the fused transport the pieces of the own shard are multiplied as they land, so the other shards
        # take the copy-engine path here: one launch over everything could not start before the last piece.)
        peer_memory = self.transport in ("peer", "fused")
        x_dev = self.exchange.send[self.exchange.calls & 1] if peer_memory else x_stage
        base = self.me * self.m

        h2d.wait_event(set_done)  # the GEMMs of two calls ago have read this set's w and x
        compute.wait_event(self.host_done)  # the previous call's rows of `out` have all been copied back
        if peer_memory:
            h2d.wait_event(self.barrier_done)  # peers finished reading this half of the send buffer two calls ago
        with torch.cuda.stream(h2d):
            if w_replicated and self.ranks > 1 and self.K % self.ranks == 0:
                part = self.K // self.ranks
                mine = w_dev[self.me * part : (self.me + 1) * part]
                mine.copy_(w_host[self.me * part : (self.me + 1) * part], non_blocking=True)
                dist.all_gather_into_tensor(w_dev, mine, group=self.group)  # in place: each part lands where it belongs
            else:
                w_dev.copy_(w_host, non_blocking=True)
            self._w_ready.record(h2d)
        compute.wait_event(self._w_ready)
        try:
            ops.set_gemm_cta_limit(self.cta_limit)
            for c in range(chunks):
                lo, hi = c * rows, (c + 1) * rows
                landed, computed = torch.cuda.Event(), torch.cuda.Event()
                with torch.cuda.stream(h2d):
                    x_dev[lo:hi].copy_(x_host[lo:hi], non_blocking=True)
                    landed.record(h2d)
                compute.wait_event(landed)
                ops.gemm(x_dev[lo:hi], w_dev, self.tm, self.tn, self.tk, out=self.out[base + lo : base + hi])
                computed.record(compute)
                d2h.wait_event(computed)
                with torch.cuda.stream(d2h):
                    out_host[base + lo : base + hi].copy_(self.out[base + lo : base + hi], non_blocking=True)
            if self.ranks > 1:
                self.x_ready.record(h2d)  # the whole shard is in place
                self._start_exchange(x_dev)
                order = shard_order(self.me, self.ranks)

                def copy_rows_back(shards):
                    if copy_back == "own":
                        return
                    computed = torch.cuda.Event()
                    computed.record(compute)
                    d2h.wait_event(computed)
                    with torch.cuda.stream(d2h):
                        for s in shards:
                            lo = order[s] * self.m
                            out_host[lo : lo + self.m].copy_(self.out[lo : lo + self.m], non_blocking=True)

                self._other_groups(w_dev, compute, copy_rows_back)
        finally:
            ops.set_gemm_cta_limit(0)
        self.done.record(compute)
        set_done.record(compute)
        self.host_done.record(d2h)
