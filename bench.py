"""Benchmark of the step-loop hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-extras] [--only NAME]

Headline workload at every N: the collective matmul `all_gather(x) @ y` (examples/collective_matmul.py:44-59) —
x [16384 x 8192] bf16 row-sharded over the N GPUs, y [8192 x 8192] bf16 on every GPU, each GPU computing all
16384 rows (weak scaling: per-GPU work is constant), the all-gather overlapped with the tile compute. At N = 1 that
is one dense 16384 x 8192 x 8192 matmul through the persistent tcgen05 GEMM. `value` is whole-job TFLOP/s
(N x 2 M N K / step time). A step is one pass.

After the timed steps (outside every timed region) each rank checks its result: bit-equal to the same GEMM on rows
gathered beforehand with a plain all-gather, and sampled rows against float64; the line carries the outcome under
`parity` and the program exits non-zero on a mismatch.

At N = 1 the line also carries `workloads`: the other hot-path configurations (dense 4096^3 and 8192^3, causal
8192^3 at both tilings, causal attention, paged decode with shared and with distinct pages, MLA decode), each timed
on the device with its own roofline fractions and its own CPU baseline, and `cpu_baseline`: the NumPy port of the
headline loop nest timed on the host cores on a bounded sample.

`--impl reference` times the reference's CPU path (the port; the reference itself needs JAX, which is absent) on
the host cores for the same metric.

Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M_TOTAL, K_DIM, N_DIM = 16384, 8192, 8192
TILES = (256, 512, 512)  # CollectiveTiles defaults (examples/collective_matmul.py:35-41)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NOMINAL = {"bf16_tflops": 2250.0, "hbm_gbs": 8000.0}
CPU_SAMPLE_ROWS = 2048

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per launch of each workload's dominant kernel, from one
# ncu capture of `python bench.py --only <workload> --steps 1 --warmup 1` (one kernel, one launch,
# --clock-control none). A workload that has not been captured since its kernel last changed has no entry and
# reports `traffic: null`.
NCU_TRAFFIC_BYTES: dict[str, float] = {
    "gemm_16384x8192x8192": 2.299167e9 + 0.263586e9,
    "paged_gqa_decode_B64_H32_Hkv8_D128_page16_shared_pages": 467166208.0 + 4148480.0,
    "paged_gqa_decode_B64_H32_Hkv8_D128_page16_distinct_pages": 551334656.0 + 4222208.0,
    # profiles/attention_kernel_b4_h16_s2048_d128.md: 132.9 MB read + 13.9 MB written (134.2 MB algorithmic).
    "causal_attention_B4_H16_S2048_D128_blocks512": 132.940288e6 + 13.855488e6,
    # profiles/mla_tc_kernel_b32_h64_ctx1024to3072.md: the main kernel's 89.6 MB read + 3.7 MB written (the cache rows
    # as stored are 83.8 MB; 75.4 MB as the reference counts them).
    "mla_decode_B32_H64_ctx1024to3072": 89.602304e6 + 3.712512e6,
}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return FALLBACK_PEAKS, "fallback"


def host_threads() -> int:
    threads = os.cpu_count() or 1
    try:
        from threadpoolctl import threadpool_info

        blas = [p["num_threads"] for p in threadpool_info() if p.get("user_api") == "blas"]
        if blas:
            threads = max(blas)
    except Exception:
        pass
    return threads


# ----------------------------------------------------------------------------------------- clocks


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed regions run."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid: str):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", uuid, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, sm_max, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            cells = [c.strip() for c in line.split(",")]
            if len(cells) < 8:
                continue
            try:
                sm.append(float(cells[0]))
                sm_max.append(float(cells[1]))
                power.append(float(cells[2]))
            except ValueError:
                continue
            for name, cell in zip(names, cells[4:8]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        busy = [c for c, p in zip(sm, power) if p > 300.0] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "samples_under_load": len(busy),
                "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------------------- helpers


def to_device(a, device):
    import numpy as np
    import torch

    from tilejax_b200.synthetic import bf16_dtype

    a = np.ascontiguousarray(a)
    if a.dtype == bf16_dtype():
        return torch.from_numpy(a.view(np.uint16)).view(torch.bfloat16).to(device)
    return torch.from_numpy(a).to(device)


def device_randn_bf16(shape, seed, device, scale=1.0):
    """N(0, 1) bf16 generated on the device (large operands: the host generator would take minutes)."""
    import torch

    g = torch.Generator(device=device)
    g.manual_seed(seed)
    x = torch.randn(shape, generator=g, device=device, dtype=torch.float32)
    if scale != 1.0:
        x *= scale
    return x.to(torch.bfloat16)


def time_device(fn, iters: int, warmup: int, flush=None) -> float:
    """Median device time of fn() in ms over `iters` runs, each bracketed by CUDA events on the current stream;
    `flush()` (an L2 flush) runs untimed before each, then a spin kernel behind which the host queues the timed
    launches. (The median, as the reference's benchmarks take it,
    benchmarks/timing.py:12-22: under the board's power cap single launches scatter by several per cent.)"""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush()
        # Half a millisecond of spinning on the device ahead of the first event: the host queues the events and fn's
        # launches behind it, so the interval holds device time only and not the host's time to issue a launch
        # (tens of microseconds through Python, as long as the shortest kernels here run).
        torch.cuda._sleep(1_000_000)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        end.synchronize()
        times.append(start.elapsed_time(end))
    return statistics.median(times)


def time_sustained(fn, seconds: float, ms_hint: float) -> float:
    """Mean device time of fn() in ms over a back-to-back loop of at least `seconds`: the figure for a kernel under
    the power cap, next to the isolated-launch one."""
    import torch

    iters = max(10, int(seconds * 1e3 / max(ms_hint, 1e-3)))
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    end.synchronize()
    return start.elapsed_time(end) / iters


def tensor_roofline(tflops: float, pk: dict, pk_kind: str, sustained_tflops: float | None = None,
                    traffic: float | None = None, **more) -> dict:
    """The roofline record of a tensor-bound kernel: `frac` is against the burst cuBLAS figure (the kernel was timed
    in isolated launches); `frac_sustained` compares the back-to-back figure with the sustained cuBLAS one."""
    r = {"bound": "tensor", "achieved": tflops, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
         "frac": tflops / pk["bf16_tflops"], "frac_burst": tflops / pk["bf16_tflops"],
         "peak_kind": f"{pk_kind} cuBLAS bf16, burst", "peak_sustained": pk["bf16_tflops_sustained"],
         "achieved_sustained": sustained_tflops,
         "frac_sustained": None if sustained_tflops is None else sustained_tflops / pk["bf16_tflops_sustained"],
         "nominal_frac": tflops / NOMINAL["bf16_tflops"], "traffic": traffic}
    r.update(more)
    return r


def hbm_roofline(gbs: float, pk: dict, pk_kind: str, algorithmic_bytes: float, ms: float,
                 traffic: float | None = None) -> dict:
    """The roofline record of an HBM-bound kernel. `frac` uses the algorithmic bytes; where an ncu capture gave the
    DRAM bytes of the launch, `frac_dram` = those bytes / time / peak says how much of the figure L2 hits supply."""
    r = {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
         "peak_kind": f"{pk_kind} copy bandwidth", "nominal_frac": gbs / NOMINAL["hbm_gbs"],
         "algorithmic_bytes": algorithmic_bytes, "traffic": traffic,
         "frac_dram": None if traffic is None else traffic / ms / 1e6 / pk["hbm_gbs"]}
    return r


# ----------------------------------------------------------------------------------------- CPU baselines


def _timed(fn, repeats: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    return sum(times) / len(times)


def cpu_port_tflops(rows: int, repeats: int, warmup: int) -> tuple[float, float, int, str]:
    """The NumPy port of the matmul loop nest (oracle.matmul_ref) on `rows` rows of the workload's x against the
    full y, on the host cores. Returns (TFLOP/s, seconds per pass, threads, sample description)."""
    import oracle
    from tilejax_b200 import synthetic

    x = synthetic.normal_bf16((rows, K_DIM), 0)
    y = synthetic.normal_bf16((K_DIM, N_DIM), 1)
    sec = _timed(lambda: oracle.matmul_ref(x, y, *TILES), repeats, warmup)
    flops = 2.0 * rows * K_DIM * N_DIM
    sample = (f"{rows} of {M_TOTAL} rows of x against the full y [{K_DIM}x{N_DIM}], tiles {TILES}, "
              f"NumPy f32 BLAS on bf16-rounded inputs, mean of {repeats} passes")
    return flops / sec / 1e12, sec, host_threads(), sample


def cpu_baselines_for_workloads() -> dict:
    """The NumPy port of each side workload's loop nest on a bounded sample (a second or two each), on the host
    cores: {workload prefix: cpu_baseline record}."""
    import numpy as np

    import oracle
    from tilejax_b200 import synthetic

    threads = host_threads()
    out = {}
    n = 2048
    x, y = synthetic.normal_bf16((n, n), 0), synthetic.normal_bf16((n, n), 1)
    sec = _timed(lambda: oracle.matmul_ref(x, y, 512, 512, 512), 2, 1)
    out["dense_matmul"] = {"value": 2.0 * n**3 / sec / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                           "sample": f"a {n}^3 product (tiles 512^3) of the same loop nest, NumPy f32 BLAS, mean of 2"}
    sec = _timed(lambda: oracle.causal_matmul_ref(x, y, 512, 512, 512), 2, 1)
    out["causal_matmul"] = {"value": float(n) * n * (n + 1) / sec / 1e12, "unit": "TFLOP/s", "cores": threads,
                            "kind": "port", "sample": f"tril of a {n}^3 product (tiles 512^3), algorithmic flops "
                                                      "K*M*(M+1), NumPy f32 BLAS, mean of 2"}
    B, H, S, D = 1, 2, 2048, 128
    q, k, v = synthetic.attention_inputs(B, H, S, D)
    sec = _timed(lambda: oracle.causal_attention_ref(q, k, v, 512, 512), 1, 1)
    out["causal_attention"] = {"value": 4.0 * B * H * D * S * (S + 1) / 2 / sec / 1e12, "unit": "TFLOP/s",
                               "cores": threads, "kind": "port",
                               "sample": f"{H} of the 64 (batch, head) pairs at S {S}, blocks 512 x 512, one pass"}
    Bd = 8
    qd, kp, vp, bt, lengths = synthetic.decode_inputs(Bd, 32, 8, 128, 16, 256, 1024)
    sec = _timed(lambda: oracle.paged_gqa_decode_ref(qd, kp, vp, bt, lengths), 1, 0)
    out["paged_gqa_decode"] = {"value": float(np.sum(lengths)) * 4096.0 / sec / 1e9, "unit": "GB/s", "cores": threads,
                               "kind": "port", "sample": f"{Bd} of the 64 sequences (lengths uniform in 1..4096, "
                                                         "16-token pages), one pass of the NumPy loop nest"}
    n = 1024
    rng = np.random.default_rng(7)
    xr, wr = synthetic.normal_bf16((n, n), 0), synthetic.normal_bf16((n, n), 1)
    gamma = (1 + 0.1 * rng.standard_normal((1, n), np.float32)).astype(xr.dtype)
    sec = _timed(lambda: oracle.rmsnorm_matmul_ref(xr, gamma, wr, 512, 512, 512), 2, 1)
    out["rmsnorm_matmul"] = {"value": 2.0 * n**3 / sec / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                             "sample": f"a {n}^3 problem (tiles 512^3) of the same loop nest, NumPy f32, mean of 2"}
    from oracle.attention_block import attention_block_ref

    Bb, Hb, Sb, Db, Fb = 1, 2, 512, 128, 1024
    qb, kb, vb = synthetic.attention_inputs(Bb, Hb, Sb, Db)
    gb = (1 + 0.1 * rng.standard_normal((1, Hb * Db), np.float32)).astype(qb.dtype)
    up = (rng.standard_normal((Hb * Db, Fb), np.float32) / (Hb * Db) ** 0.5).astype(qb.dtype)
    down = (rng.standard_normal((Fb, Hb * Db), np.float32) / Fb**0.5).astype(qb.dtype)
    sec = _timed(lambda: attention_block_ref(qb, kb, vb, gb, up, down, 256, 256, 1024), 1, 0)
    flops = 4.0 * Bb * Hb * Db * Sb * (Sb + 1) / 2 + 4.0 * Bb * Sb * Hb * Db * Fb
    out["attention_block"] = {"value": flops / sec / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                              "sample": f"a block of {Hb} heads, S {Sb}, F {Fb} (blocks 256 x 256), one pass of the NumPy "
                                        "loop nest"}
    Bm, Hm, Sm = 2, 64, 2048
    lens = np.array([1500, 2048], np.int32)
    q_c, q_r = synthetic.normal_bf16((Bm, 1, Hm, 512), 3), synthetic.normal_bf16((Bm, 1, Hm, 128), 4)
    c_kv, k_rope = synthetic.normal_bf16((Bm, Sm, 512), 5), synthetic.normal_bf16((Bm, Sm, 128), 6)
    sec = _timed(lambda: oracle.mla_decode_ref(q_c, q_r, c_kv, k_rope, lens, 512), 1, 0)
    out["mla_decode"] = {"value": float(lens.sum()) * 576 * 2 / sec / 1e9, "unit": "GB/s", "cores": threads,
                         "kind": "port", "sample": f"{Bm} sequences of the 32 (64 heads, contexts 1500 and 2048), one "
                                                   "pass of the NumPy loop nest"}
    inp = oracle.rpa_inputs([1] * 4 + [256], [1000, 2000, 300, 4000, 512], max_len=4096, seed=0)
    cache = oracle.rpa_write_ref(inp["kv_cache"], inp["keys"], inp["values"], inp["kv_lens"], inp["page_indices"],
                                 inp["cu_q_lens"], inp["distribution"])

    def rpa_step():
        o = oracle.rpa_decode_ref(inp["q"], cache, inp["kv_lens"], inp["page_indices"], inp["distribution"], 128**-0.5)
        return oracle.rpa_prefill_ref(o, cache, inp["kv_lens"], inp["page_indices"], inp["cu_q_lens"],
                                      inp["distribution"], 128**-0.5)

    sec = _timed(rpa_step, 1, 0)
    seen = 256 * 256 + 256 * 257 // 2
    out["ragged_paged_attention"] = {"value": 4.0 * 32 * 128 * seen / sec / 1e12, "unit": "TFLOP/s", "cores": threads,
                                     "kind": "port", "sample": "4 decode sequences and one prefill sequence of 256 tokens "
                                                               "on a prefix of 256, one pass of the NumPy loop nests; "
                                                               "flops of the prefill tokens as in the GPU figure"}
    return out


def reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torch.distributed.run sets OMP_NUM_THREADS=1 for its workers; the reference arm uses every host core.
    cores = os.cpu_count() or 1
    try:
        from threadpoolctl import threadpool_limits

        threadpool_limits(limits=cores)
    except Exception:
        pass
    tflops, sec, threads, sample = cpu_port_tflops(CPU_SAMPLE_ROWS, max(args.steps, 1), max(args.warmup, 1))
    line = {
        "impl": "reference",
        "metric": "bf16_matmul_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(args.gpus), "tiles": list(TILES),
                   "note": "reference CPU path: NumPy port of examples/collective_matmul.py's loop nest "
                           "(the reference needs JAX, which is not installed); each step is a bounded sample; "
                           "one host runs it whatever N is"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_name(n: int) -> str:
    return (f"collective_matmul: all_gather(x[{M_TOTAL}x{K_DIM}] row-sharded over {n} GPU(s)) @ y[{K_DIM}x{N_DIM}] "
            f"replicated, bf16, f32 accumulation")


# ----------------------------------------------------------------------------------------- extra workloads


def extra_workloads(device, pk: dict, pk_kind: str, only: str | None = None, iters: int = 20, warm: int = 3,
                    quick: bool = False) -> dict:
    """The other hot-path configurations at one GPU, device-timed with an L2 flush before every run. `only` keeps
    the workloads whose name contains it and `quick` drops the sustained loops and the front-end timings (for
    profiling one kernel with few launches)."""
    import numpy as np
    import torch

    from tilejax_b200 import ops, synthetic
    from tilejax_b200.autokernel import kernels

    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    flush_mode = os.environ.get("TJX_FLUSH", "write_read")

    def flush():
        # Write a buffer larger than L2, then read it back: the write evicts every line of the workload, the read
        # sweep pushes the written (dirty) lines out to HBM, so the timed kernel starts on a cold L2 that owes HBM no
        # write-backs. (After the write alone, up to 126 MB of dirty lines are written back during the timed kernel,
        # which costs an HBM-bound kernel a fifth of its bandwidth.)
        if flush_mode == "none":
            return
        flush_buf.zero_()
        if flush_mode == "write_read":
            flush_buf.view(torch.int32).sum()

    out = {}
    want = lambda name: only is None or only in name  # noqa: E731

    later = []  # back-to-back loops of more than a second: run after every isolated timing, they heat the chip

    def tensor_entry(name, ms, flops, fn=None, extra=None, sustained=False):
        tf = flops / ms / 1e9
        out[name] = {"ms": ms, "value": tf, "unit": "TFLOP/s",
                     "roofline": tensor_roofline(tf, pk, pk_kind, None, NCU_TRAFFIC_BYTES.get(name))}
        if extra:
            out[name].update(extra)
        if sustained and not quick and fn is not None:
            later.append((name, fn, flops, ms))

    def frontend_ms(call):
        """The same launch through `@autokernel.kernel` (parse, plan and tables cached after the first call)."""
        if quick:
            return None
        try:
            return time_device(call, max(3, iters // 2), 2, flush)
        except Exception as e:  # report, do not hide
            return f"error: {str(e)[:160]}"

    for n in (4096, 8192):
        if not (want(f"dense_matmul_{n}") or (n == 8192 and want("causal_matmul"))):
            continue
        x = device_randn_bf16((n, n), 0, device)
        y = device_randn_bf16((n, n), 1, device)
        if want(f"dense_matmul_{n}"):
            fn = lambda x=x, y=y: ops.matmul(x, y, 512, 512, 512)  # noqa: E731
            ms = time_device(fn, iters, warm, flush)
            tensor_entry(f"dense_matmul_{n}_tiles512", ms, 2.0 * n**3, fn, sustained=True, extra={
                "via_autokernel_ms": frontend_ms(lambda: kernels.matmul(x, y, kernels.MatmulTiles()))})
        if n == 8192:
            for tiles in ((512, 512, 512), (1024, 2048, 1024)):
                name = f"causal_matmul_8192_tiles{tiles[0]}x{tiles[1]}x{tiles[2]}"
                if not want(name):
                    continue
                fn = lambda x=x, y=y, tiles=tiles: ops.causal_matmul(x, y, *tiles)  # noqa: E731
                ms = time_device(fn, iters, warm, flush)
                dense_ms = out.get("dense_matmul_8192_tiles512", {}).get("ms")
                tensor_entry(name, ms, float(n) * n * (n + 1), fn, extra={
                    "dense_equivalent_tflops": 2.0 * n**3 / ms / 1e9, "algorithmic_flops": "K*M*(M+1)",
                    "time_vs_dense": None if dense_ms is None else ms / dense_ms,
                    "via_autokernel_ms": frontend_ms(
                        lambda: kernels.causal_matmul(x, y, kernels.MatmulTiles(*tiles)))})

    if want("rmsnorm_matmul"):
        # RMSNorm fused with the projection after it (examples/rmsnorm_matmul.py:31-47) at the dense config's size:
        # the same product plus one pass over x (2 M D bytes read, 2 M D + 4 M written).
        n = 8192
        x = device_randn_bf16((n, n), 0, device)
        gamma = (1 + 0.1 * device_randn_bf16((1, n), 7, device).float()).to(torch.bfloat16)
        w = device_randn_bf16((n, n), 1, device, n**-0.5)
        ms = time_device(lambda: ops.rmsnorm_matmul(x, gamma, w, 512, 512, 512), iters, warm, flush)
        tensor_entry("rmsnorm_matmul_8192_tiles512", ms, 2.0 * n**3, extra={
            "includes": "the pass over x that writes the gamma-scaled operand and the row scales, then the matmul",
            "via_autokernel_ms": frontend_ms(lambda: kernels.rmsnorm_matmul(x, gamma, w, kernels.NormMatmulTiles()))})

    for (B, H, S, D) in ((4, 16, 2048, 128), (1, 16, 4096, 128)):
        if not want(f"causal_attention_B{B}"):
            continue
        name = f"causal_attention_B{B}_H{H}_S{S}_D{D}_blocks512"
        try:
            q = device_randn_bf16((B, H, S, D), 0, device, D**-0.5)
            k = device_randn_bf16((B, H, S, D), 1, device)
            v = device_randn_bf16((B, H, S, D), 2, device)
            fn = lambda: ops.causal_attention(q, k, v, 512, 512)  # noqa: E731
            ms = time_device(fn, iters, warm, flush)
            tensor_entry(name, ms, 4.0 * B * H * D * S * (S + 1) / 2, fn, extra={
                "algorithmic_flops": "4*B*H*D*S*(S+1)/2",
                "via_autokernel_ms": frontend_ms(
                    lambda: kernels.causal_attention(q, k, v, kernels.AttentionBlocks(512, 512)))})
        except Exception as e:  # not built yet, or failed: report, do not hide
            out[name] = {"error": str(e)[:200]}

    if want("attention_block"):
        # A whole attention block (examples/attention_block.py:49-85) at the size the reference lowers for its TPU
        # (tests/test_examples.py:201-206): B 4, 8 heads of 128, S 2048, D 1024, F 4096. Four launches: attention,
        # row norm, matmul + GELU, matmul. Flops: the causal attention's plus 4 * B * S * D * F for the two matmuls.
        name = "attention_block_B4_H8_S2048_D1024_F4096"
        try:
            B, H, S, Dh, F = 4, 8, 2048, 128, 4096
            D = H * Dh
            q = device_randn_bf16((B, H, S, Dh), 0, device, Dh**-0.5)
            k = device_randn_bf16((B, H, S, Dh), 1, device)
            v = device_randn_bf16((B, H, S, Dh), 2, device)
            gamma = (1 + 0.1 * device_randn_bf16((1, D), 7, device).float()).to(torch.bfloat16)
            w_up = device_randn_bf16((D, F), 8, device, D**-0.5)
            w_down = device_randn_bf16((F, D), 9, device, F**-0.5)
            fn = lambda: ops.attention_block(q, k, v, gamma, w_up, w_down, 256, 512, 1024)  # noqa: E731
            ms = time_device(fn, iters, warm, flush)
            tensor_entry(name, ms, 4.0 * B * H * Dh * S * (S + 1) / 2 + 4.0 * B * S * D * F, extra={
                "algorithmic_flops": "4*B*H*Dh*S*(S+1)/2 + 4*B*S*D*F",
                "launches": "attention_kernel, rmsnorm_rows_kernel, gemm (GELU epilogue), gemm",
                "via_autokernel_ms": frontend_ms(
                    lambda: kernels.attention_block(q, k, v, gamma, w_up, w_down, kernels.BlockTiles(256, 512, 1024)))})
        except Exception as e:
            out[name] = {"error": str(e)[:200]}

    if want("ragged_paged_attention"):
        # One step of ragged paged attention in RPA v3's layout (examples/ragged_paged_attention.py:279-290): 32 decode
        # sequences with caches uniform in 1..4096 and 4 prefill sequences of 1024 new tokens on a prefix of 1024,
        # Llama-3-8B heads (32 / 8 x 128), pages of 128: the cache write, the decode case, the prefill case.
        name = "ragged_paged_attention_decode32_prefill4x1024_H32_Hkv8_page128"
        try:
            rng = np.random.default_rng(0)
            H, Hkv, D, ps, max_len = 32, 8, 128, 128, 4096
            q_lens = [1] * 32 + [1024] * 4
            kv_lens = [int(x) for x in rng.integers(1, 4097, 32)] + [2048] * 4
            S, T, pps = len(q_lens), sum(q_lens), max_len // ps
            used = [-(-n // ps) for n in kv_lens]
            pages = sum(used) + 1
            table = np.zeros((S, pps), np.int32)
            pool, at = 1 + rng.permutation(pages - 1), 0
            for i, n in enumerate(used):
                table[i, :n] = pool[at:at + n]
                at += n
            cache = device_randn_bf16((pages, ps, Hkv, 2, D), 11, device)
            qd = device_randn_bf16((T, H, D), 12, device)
            kd2, vd2 = device_randn_bf16((T, Hkv, D), 13, device), device_randn_bf16((T, Hkv, D), 14, device)
            dev = lambda a: torch.from_numpy(np.asarray(a, np.int32)).to(device)  # noqa: E731
            lens_d, table_d = dev(kv_lens), dev(table.reshape(-1))
            cu_d, dist_d = dev(np.concatenate([[0], np.cumsum(q_lens)])), dev([32, 32, S])
            fn = lambda: ops.ragged_paged_attention(qd, kd2, vd2, cache, lens_d, table_d, cu_d, dist_d, D**-0.5)  # noqa: E731
            ms = time_device(fn, iters, warm, flush)
            seen = sum(q * (k - q) + q * (q + 1) // 2 for q, k in zip(q_lens[32:], kv_lens[32:], strict=True))
            tensor_entry(name, ms, 4.0 * H * D * seen, extra={
                "algorithmic_flops": "the prefill tokens' 4*H*D*(positions seen); the decode part reads "
                                     f"{sum(kv_lens[:32]) * Hkv * 2 * D * 2 / 1e6:.0f} MB of cache",
                "launches": "one call (tjx_ragged_paged_attention_bf16): rpa_write with decode lengths and prefill tiles beside it, step tables + decode, decode rows, attention (paged)",
                "new_tokens": T})
        except Exception as e:
            out[name] = {"error": str(e)[:200]}

    if want("mla_decode"):
        # The reference's MLA benchmark shape (benchmarks/decode.py:152-173): batch 32, contexts around 2048 of a
        # 4096-position cache, 64 heads, 512 latents + 64 RoPE columns (stored 128 wide), blocks of 512.
        # A second line at four times the batch: the same kernels once the fill of their pipeline and the tail of
        # partials are a smaller part of the call.
        for B in (32, 128):
            try:
                H, S = 64, 4096
                rng = np.random.default_rng(0)
                lens = rng.integers(1024, 3073, B).astype(np.int32)
                q_c = device_randn_bf16((B, 1, H, 512), 3, device, 192**-0.5 * 0.1)
                q_r = device_randn_bf16((B, 1, H, 128), 4, device, 192**-0.5)
                c_kv = device_randn_bf16((B, S, 512), 5, device)
                k_rope = device_randn_bf16((B, S, 128), 6, device)
                q_r[..., 64:] = 0
                k_rope[..., 64:] = 0
                lens_d = torch.from_numpy(lens).to(device)
                mbufs = ops.MlaBuffers(B, H, S, 512, device)
                mout = torch.empty_like(q_c)
                ms = time_device(lambda: ops.mla_decode(q_c, q_r, c_kv, k_rope, lens_d, 512, out=mout, buffers=mbufs),  # noqa: B023
                                 2 * iters, warm, flush)
                tokens = float(lens.sum())
                nbytes = tokens * 576 * 2  # what the math reads: 512 latents + 64 RoPE columns per position
                gbs = nbytes / ms / 1e6
                name = f"mla_decode_B{B}_H{H}_ctx1024to3072"
                out[name] = {
                    "ms": ms, "value": gbs, "unit": "GB/s",
                    "tflops": tokens * H * (2 * 576 + 2 * 512) / ms / 1e9,
                    "includes": "step-table kernel, the tcgen05 decode kernel and the kernel that merges its partials",
                    "roofline": hbm_roofline(gbs, pk, pk_kind, nbytes, ms, NCU_TRAFFIC_BYTES.get(name))}
                del c_kv, k_rope
            except Exception as e:  # report, do not hide
                out[f"mla_decode_B{B}"] = {"error": str(e)[:200]}

    # Paged GQA decode (examples/decode.py:199-223) on batch 64, 32 / 8 heads, 16-token pages, lengths uniform in
    # 1..4096: once with the block tables drawn with replacement from a pool of 8192 pages (sequences then share
    # pages, which L2 serves), once with a page of its own for every slot (examples/kv_cache.py:54-60: a permutation
    # of a pool of 16384), where every byte comes from HBM.
    for variant, num_pages, distinct in (("_shared_pages", 8192, False), ("_distinct_pages", 16384, True)):
        name = f"paged_gqa_decode_B64_H32_Hkv8_D128_page16{variant}"
        if not want(name):
            continue
        rng = np.random.default_rng(0)
        lengths = rng.integers(1, 4097, 64).astype(np.int32)
        if distinct:
            bt = rng.permutation(num_pages)[: 64 * 256].reshape(64, 256).astype(np.int32)
        else:
            bt = rng.integers(0, num_pages, (64, 256)).astype(np.int32)
        kd = device_randn_bf16((num_pages, 16, 1024), 1, device)
        vd = device_randn_bf16((num_pages, 16, 1024), 2, device)
        qd = device_randn_bf16((64, 1, 32, 128), 3, device, 128**-0.5)
        btd, ld = to_device(bt, device), to_device(lengths, device)
        bufs = ops.DecodeBuffers(64, 32, 128, 256, device)
        od = torch.empty_like(qd)
        ms = time_device(lambda: ops.paged_gqa_decode(qd, kd, vd, btd, ld, out=od, buffers=bufs), 2 * iters, warm,
                         flush)
        nbytes = float(lengths.sum()) * 4096.0
        gbs = nbytes / ms / 1e6
        out[name] = {
            "ms": ms, "value": gbs, "unit": "GB/s",
            "includes": "step-table kernel + decode (the merge of partials is fused into it)",
            "pages": "one page per (sequence, slot): no page is read twice" if distinct else
                     "block tables drawn with replacement: about 29 % of the page reads hit L2",
            "via_autokernel_ms": frontend_ms(lambda: kernels.paged_gqa_decode(qd, kd, vd, btd, ld)),
            "roofline": hbm_roofline(gbs, pk, pk_kind, nbytes, ms, NCU_TRAFFIC_BYTES.get(name))}
        del kd, vd
    for name, fn, flops, ms in later:
        sustained_tf = flops / time_sustained(fn, 1.2, ms) / 1e9
        out[name]["roofline"].update(achieved_sustained=sustained_tf,
                                     frac_sustained=sustained_tf / pk["bf16_tflops_sustained"])
    ops.device_status()
    return out


# ----------------------------------------------------------------------------------------- main arm


def check_parity(op, x, y, world: int, rank: int, device) -> dict:
    """Outside every timed region: this rank's result against the same GEMM on rows gathered beforehand (bit-equal:
    same kernel, same order of summation) and sampled rows against float64. Reduced over the ranks."""
    import torch
    import torch.distributed as dist

    from tilejax_b200 import ops

    out = op(x, y).clone()
    torch.cuda.synchronize()
    if world > 1:
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        xs = torch.cat(parts)
    else:
        xs = x
    want = ops.gemm(xs, y, op.tm, op.tn, op.tk)
    bit_equal = bool(torch.equal(out, want))
    rows = torch.arange(rank % 7, xs.shape[0], 521, device=device)
    exact = xs[rows].double() @ y.double()
    rel = float(((out[rows].double() - exact).abs().max() / exact.abs().max()).item())
    status = ops.device_status()
    flags = torch.tensor([0.0 if bit_equal else 1.0, rel, float(status)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(flags, op=dist.ReduceOp.MAX)
    ok = flags[0].item() == 0.0 and flags[1].item() <= 2e-2 and flags[2].item() == 0.0
    return {"bit_equal_to_gather_then_gemm": flags[0].item() == 0.0, "sampled_f64_max_rel": flags[1].item(),
            "tolerance": "2e-2 of the largest value (bf16 output)", "rows_sampled_per_rank": int(rows.numel()),
            "device_status": int(flags[2].item()), "ranks_checked": world, "ok": ok}


PEER_COPY_GBS = 770.0  # measured peer copy bandwidth per direction per GPU on this pool's NVLink 5 / NVSwitch


def reference_layout(world: int, rank: int, device, x, y, m: int, steps: int, warmup: int, pk: dict, barrier) -> dict:
    """The collective matmul as the reference's own example shards it (examples/collective_matmul.py:64, in_specs
    P("x", None) and P(None, "x")): w split by columns, so a rank computes all_gather(x) @ its N / G columns, 2 * G *
    m * K * n flops (benchmarks/collective_matmul.py:44) — 1 / G of the headline's — behind the same gathered bytes.
    With eight ranks the gather no longer hides: the bound is the slower of the tensor pipe and NVLink. Both
    transports are timed: the one-launch kernel, whose copier warps pull at about 400 GB/s, and the copy-engine one
    ("peer": a GEMM launch per group of shards behind copies on a second stream)."""
    import torch
    import torch.distributed as dist

    from tilejax_b200.collective import AllGatherMatmul

    n = N_DIM // world
    w = y[:, rank * n : (rank + 1) * n].contiguous()
    flops = 2.0 * M_TOTAL * K_DIM * n
    gathered = (world - 1) * m * K_DIM * 2
    tensor_ms = flops / (pk["bf16_tflops"] * 1e9)
    link_ms = gathered / (PEER_COPY_GBS * 1e6)
    by_transport, parity_ok = {}, True
    for transport in ("fused", "peer"):
        op = AllGatherMatmul(m, K_DIM, n, *TILES, transport=transport)
        for _ in range(warmup):
            op(x, w)
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            op(x, w)
        end.record()
        barrier()
        elapsed = torch.tensor([start.elapsed_time(end)], device=device)
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        ms = elapsed.item() / steps
        parity = check_parity(op, x, w, world, rank, device)
        barrier()
        parity_ok = parity_ok and parity["ok"]
        by_transport[op.transport] = {"ms_per_step": ms, "gather_gbs_per_gpu": gathered / ms / 1e6,
                                      "frac": max(tensor_ms, link_ms) / ms, "parity": parity}
        del op
    best = min(by_transport, key=lambda t: by_transport[t]["ms_per_step"])
    ms = by_transport[best]["ms_per_step"]
    return {"ms_per_step": ms, "steps": steps, "value": world * flops / ms / 1e9, "unit": "TFLOP/s",
            "per_gpu_tflops": flops / ms / 1e9, "columns_per_gpu": n, "transport": best,
            "gathered_bytes_per_gpu": gathered, "by_transport": by_transport,
            "roofline": {"bound": "tensor" if tensor_ms >= link_ms else "nvlink", "tensor_ms": tensor_ms,
                         "nvlink_ms": link_ms, "target_ms": max(tensor_ms, link_ms),
                         "frac": max(tensor_ms, link_ms) / ms,
                         "peaks": f"measured cuBLAS bf16 burst {pk['bf16_tflops']} TFLOP/s; measured peer copy "
                                  f"{PEER_COPY_GBS} GB/s per direction"},
            "parity": {"ok": parity_ok}}


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-extras", action="store_true", help="skip the other single-GPU workloads and the CPU baselines")
    parser.add_argument("--only", default=None, help="run only the single-GPU workloads whose name contains this "
                        "(dense_matmul_8192, causal_matmul, causal_attention_B4, paged_gqa_decode, ...) for "
                        "--steps runs after --warmup: a short command to profile one kernel")
    args = parser.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    if os.environ.get("TJX_GEMM_PAIRS") is not None:  # A/B switch: see tjx_gemm_set_pair_mode
        from tilejax_b200 import ops as _ops

        _ops.set_gemm_pair_mode(int(os.environ["TJX_GEMM_PAIRS"]))
    if args.only:
        import torch

        torch.cuda.set_device(0)
        pk, pk_kind = peaks()
        print(json.dumps(extra_workloads(torch.device("cuda", 0), pk, pk_kind, args.only, max(args.steps, 1),
                                         max(args.warmup, 0), quick=True)), flush=True)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist

    from tilejax_b200 import ops
    from tilejax_b200.collective import AllGatherMatmul

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(device).uuid).replace("GPU-", "")) if rank == 0 else None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=device)
    pk, pk_kind = peaks()

    m = M_TOTAL // world
    # Seeded synthetic operands: this rank's rows of x (seed 1000 + rank), y (seed 1) identical on every rank.
    x_host = device_randn_bf16((m, K_DIM), 1000 + rank, device).cpu().pin_memory()
    y_host = device_randn_bf16((K_DIM, N_DIM), 1, device).cpu().pin_memory()
    x = x_host.to(device)
    y = y_host.to(device)
    reserve = os.environ.get("TJX_RESERVE_SMS")
    op = AllGatherMatmul(m, K_DIM, N_DIM, *TILES, reserve_sms=None if reserve is None else int(reserve),
                         transport=os.environ.get("TJX_TRANSPORT", "fused"))
    op.exchange.rows(op.me).copy_(x)  # (only the kernel-alone timing below reads the own rows of xs)
    out_host = torch.empty((M_TOTAL, N_DIM), dtype=torch.bfloat16).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing
    for _ in range(args.warmup):
        op(x, y)
    barrier()
    if world > 1 and op.transport == "fused":
        # A bounded wait that gave up inside the one-launch kernel on any rank (it records a status and returns):
        # say so and measure the copy-engine transport instead of timing steps that each wait out their limit.
        try:
            status = ops.device_status()
        except Exception:  # the status call raises when a kernel recorded a code
            status = 1
        failed = torch.tensor([status], device=device)
        dist.all_reduce(failed, op=dist.ReduceOp.MAX)
        if failed.item() != 0:
            if rank == 0:
                print(f"fused transport reported device status {failed.item()} during warm-up; using peer",
                      file=sys.stderr, flush=True)
            op = AllGatherMatmul(m, K_DIM, N_DIM, *TILES, transport="peer")
            op.exchange.rows(op.me).copy_(x)
            for _ in range(args.warmup):
                op(x, y)
            barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        op(x, y)
    end.record()
    barrier()
    elapsed = torch.tensor([start.elapsed_time(end)], device=device)
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    ms_per_step = elapsed.item() / args.steps

    # ---- parity of what was just timed (not timed itself)
    parity = check_parity(op, x, y, world, rank, device)
    barrier()

    # ---- the dominant kernel alone, on its stream: isolated launches (the roofline's numerator, against the burst
    # peak) and a back-to-back loop of more than a second (against the sustained peak)
    alone = lambda: ops.gemm(op.exchange.xs, y, op.tm, op.tn, op.tk, out=op.out)  # noqa: E731
    gemm_ms = time_device(alone, min(max(args.steps, 5), 20), 1)
    ops.device_status()
    barrier()

    # ---- end to end: host buffers in, host result out, copies inside the timed region
    own_rows_only = world > 1

    def e2e_step():
        # Host shard and weights in, host result out: copies, GEMMs and copies back pipelined on three streams. With
        # several GPUs every rank computes the whole (replicated) result and hands the host its own rows of it, and
        # reads its 1 / N of the replicated y from the host (the ranks all-gather the parts over NVLink).
        op.from_host(x_host, y_host, out_host, copy_back="own" if own_rows_only else "all", w_replicated=world > 1)
        torch.cuda.current_stream().wait_event(op.host_done)

    for _ in range(2):
        e2e_step()
    barrier()
    e2e_steps = max(3, min(args.steps, 10))
    start.record()
    for _ in range(e2e_steps):
        e2e_step()
    end.record()
    barrier()
    e2e_elapsed = torch.tensor([start.elapsed_time(end)], device=device)
    if world > 1:
        dist.all_reduce(e2e_elapsed, op=dist.ReduceOp.MAX)
    e2e_ms = e2e_elapsed.item() / e2e_steps
    flops_per_gpu = 2.0 * M_TOTAL * K_DIM * N_DIM
    workloads = cpu = None
    if world == 1 and not args.no_extras:
        workloads = extra_workloads(device, pk, pk_kind)  # isolated launches first, its back-to-back loops last
    # The dominant kernel back to back for more than a second: last, so that it does not heat the chip under the
    # isolated timings above.
    gemm_sustained_ms = time_sustained(alone, 1.2, gemm_ms)
    ops.device_status()
    barrier()
    column_sharded = None
    if world > 1 and not args.no_extras:
        try:
            column_sharded = reference_layout(world, rank, device, x, y, m, min(args.steps, 20), args.warmup, pk, barrier)
        except Exception as exc:  # the headline line is still printed, with the failure in it; a result that is
            column_sharded = {"error": f"{type(exc).__name__}: {exc}"}  # wrong (parity) still ends the run non-zero
    clocks = sampler.stop() if sampler else None  # sampled over every timed region of this run

    value = world * flops_per_gpu / ms_per_step / 1e9
    gemm_tflops = flops_per_gpu / gemm_ms / 1e9
    line = {
        "metric": "bf16_matmul_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(world), "tiles": list(TILES), "rows_per_gpu": m,
                   "l2": "operands and output (671 MB) are larger than L2; no flush between steps",
                   "gather": "none (1 GPU)" if world == 1 else
                   "inside the one GEMM launch: copier warps pull the peers' shards over NVLink (transport fused)"
                   if op.transport == "fused" else
                   f"{world - 1} rounds on a second stream, transport {op.transport}, {len(op.groups)} GEMM launches"},
        "per_gpu_tflops": value / world,
        "parity": parity,
        "clocks": clocks,
        "e2e": {"value": world * flops_per_gpu / e2e_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": x_host.numel() * 2 + y_host.numel() * 2 // world,
                "d2h_bytes_per_step": (m if own_rows_only else M_TOTAL) * N_DIM * 2,
                "bytes_are": "per rank",
                "api": "tilejax_b200.collective.AllGatherMatmul.from_host with pinned host x, y and out"
                       + ("; each rank reads 1 / N of the replicated y from its host (all-gathered over NVLink) and returns "
                          "its own rows of the replicated result" if own_rows_only else "")},
        # Kernels of this library launched inside the timed region of `value`: GEMM launches per step x steps.
        "gpu_launches": args.steps * (1 if world == 1 or op.transport == "fused" else len(op.groups)),
        "roofline": tensor_roofline(
            gemm_tflops, pk, pk_kind, flops_per_gpu / gemm_sustained_ms / 1e9,
            NCU_TRAFFIC_BYTES["gemm_16384x8192x8192"], kernel="gemm_pair_kernel<256,3,2>", ms_per_launch=gemm_ms,
            ms_per_launch_sustained=gemm_sustained_ms, flops_per_launch=flops_per_gpu),
    }
    if column_sharded is not None:
        line["workloads"] = {f"collective_matmul_w_column_sharded_{world}gpus": column_sharded}
        parity = {**parity, "ok": parity["ok"] and column_sharded.get("parity", {}).get("ok", True)}
    if workloads is not None:
        line["workloads"] = workloads
        tflops, sec, threads, sample = cpu_port_tflops(CPU_SAMPLE_ROWS, 3, 1)
        line["cpu_baseline"] = {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample}
        for prefix, record in cpu_baselines_for_workloads().items():
            for name, entry in line["workloads"].items():
                if name.startswith(prefix) and isinstance(entry, dict) and "error" not in entry:
                    entry["cpu_baseline"] = record
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if not parity["ok"]:
        raise SystemExit("parity check failed: " + json.dumps(parity))


if __name__ == "__main__":
    main()
