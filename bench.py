"""Benchmark of the step-loop hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-extras]

Headline workload at every N: the collective matmul of BASELINE config 5 — x [16384 x 8192] bf16 row-sharded over
the N GPUs, y [8192 x 8192] bf16 on every GPU, each GPU computing all 16384 rows (weak scaling: per-GPU work is
constant), the all-gather overlapped with the tile compute. At N = 1 that is one dense 16384 x 8192 x 8192 matmul
through the persistent tcgen05 GEMM. `value` is whole-job TFLOP/s (N x 2 M N K / step time). A step is one pass.

At N = 1 the line also carries `workloads`: the other BASELINE configs (dense 4096^3 and 8192^3, causal 8192^3 at
both tilings, causal attention, paged decode), each timed on the device with its own roofline fraction, and
`cpu_baseline`: the NumPy port of the same loop nest timed on the host cores on a bounded sample.

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
CPU_SAMPLE_ROWS = 2048

# DRAM bytes (read + write) per launch of the dominant kernel from an ncu capture of this command's workload
# (profiles/gemm_pair_kernel_16384x8192x8192.md): dram__bytes_read.sum + dram__bytes_write.sum.
NCU_TRAFFIC_BYTES = {"gemm_16384x8192x8192": 2.299167e9 + 0.263586e9}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return FALLBACK_PEAKS, "fallback"


# ----------------------------------------------------------------------------------------- clocks


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

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
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


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
    """Mean device time of fn() in ms over `iters` runs, CUDA events on the current stream; `flush()` (an L2
    flush) runs untimed before each."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        end.synchronize()
        total += start.elapsed_time(end)
    return total / iters


# ----------------------------------------------------------------------------------------- reference arm


def cpu_port_tflops(rows: int, repeats: int, warmup: int) -> tuple[float, float, int, str]:
    """The NumPy port of the matmul loop nest (oracle.matmul_ref) on `rows` rows of the workload's x against the
    full y, on the host cores. Returns (TFLOP/s, seconds per pass, threads, sample description)."""
    import numpy as np

    import oracle
    from tilejax_b200 import synthetic

    x = synthetic.normal_bf16((rows, K_DIM), 0)
    y = synthetic.normal_bf16((K_DIM, N_DIM), 1)
    for _ in range(warmup):
        oracle.matmul_ref(x, y, *TILES)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.matmul_ref(x, y, *TILES)
        times.append(time.perf_counter() - t0)
    sec = float(np.mean(times))
    threads = os.cpu_count() or 1
    try:
        from threadpoolctl import threadpool_info

        blas = [p["num_threads"] for p in threadpool_info() if p.get("user_api") == "blas"]
        if blas:
            threads = max(blas)
    except Exception:
        pass
    flops = 2.0 * rows * K_DIM * N_DIM
    sample = (f"{rows} of {M_TOTAL} rows of x against the full y [{K_DIM}x{N_DIM}], tiles {TILES}, "
              f"NumPy f32 BLAS on bf16-rounded inputs, mean of {repeats} passes")
    return flops / sec / 1e12, sec, threads, sample


def reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tflops, sec, threads, sample = cpu_port_tflops(CPU_SAMPLE_ROWS, max(args.steps, 1), max(args.warmup, 1))
    line = {
        "impl": "reference",
        "metric": "bf16_matmul_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(args.gpus), "tiles": list(TILES),
                   "note": "reference CPU path: NumPy port of examples/collective_matmul.py's loop nest "
                           "(the reference needs JAX, which is not installed); each step is a bounded sample"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_name(n: int) -> str:
    return (f"collective_matmul: all_gather(x[{M_TOTAL}x{K_DIM}] row-sharded over {n} GPU(s)) @ y[{K_DIM}x{N_DIM}] "
            f"replicated, bf16, f32 accumulation (BASELINE config 5)")


# ----------------------------------------------------------------------------------------- extra workloads


def extra_workloads(device, pk: dict, pk_kind: str, only: str | None = None, iters: int = 10, warm: int = 3) -> dict:
    """The other BASELINE configs at one GPU, device-timed with an L2 flush before every run. `only` keeps the
    workloads whose name contains it (for profiling one kernel with few launches)."""
    import numpy as np
    import torch

    from tilejax_b200 import ops, synthetic

    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    flush = lambda: flush_buf.zero_()  # noqa: E731
    tf_peak, hbm_peak = pk["bf16_tflops"], pk["hbm_gbs"]
    out = {}
    want = lambda name: only is None or only in name  # noqa: E731

    def tensor_entry(name, ms, flops, extra=None):
        tf = flops / ms / 1e9
        out[name] = {"ms": ms, "value": tf, "unit": "TFLOP/s",
                     "roofline": {"bound": "tensor", "achieved": tf, "peak": tf_peak, "unit": "TFLOP/s",
                                  "frac": tf / tf_peak, "peak_kind": f"{pk_kind} burst", "traffic": None}}
        if extra:
            out[name].update(extra)

    for n in (4096, 8192):
        if not (want(f"dense_matmul_{n}") or (n == 8192 and want("causal_matmul"))):
            continue
        x = device_randn_bf16((n, n), 0, device)
        y = device_randn_bf16((n, n), 1, device)
        if want(f"dense_matmul_{n}"):
            ms = time_device(lambda: ops.matmul(x, y, 512, 512, 512), iters, warm, flush)
            tensor_entry(f"dense_matmul_{n}_tiles512", ms, 2.0 * n**3)
        if n == 8192:
            for tiles in ((512, 512, 512), (1024, 2048, 1024)):
                name = f"causal_matmul_8192_tiles{tiles[0]}x{tiles[1]}x{tiles[2]}"
                if not want(name):
                    continue
                ms = time_device(lambda: ops.causal_matmul(x, y, *tiles), iters, warm, flush)
                tensor_entry(name, ms, float(n) * n * (n + 1),
                             {"dense_equivalent_tflops": 2.0 * n**3 / ms / 1e9,
                              "algorithmic_flops": "K*M*(M+1)"})
        del x, y

    for (B, H, S, D) in ((4, 16, 2048, 128), (1, 16, 4096, 128)):
        if not want(f"causal_attention_B{B}"):
            continue
        try:
            q = device_randn_bf16((B, H, S, D), 0, device, D**-0.5)
            k = device_randn_bf16((B, H, S, D), 1, device)
            v = device_randn_bf16((B, H, S, D), 2, device)
            ms = time_device(lambda: ops.causal_attention(q, k, v, 512, 512), iters, warm, flush)
            tensor_entry(f"causal_attention_B{B}_H{H}_S{S}_D{D}_blocks512", ms, 4.0 * B * H * D * S * (S + 1) / 2,
                         {"algorithmic_flops": "4*B*H*D*S*(S+1)/2"})
        except Exception as e:  # not built yet, or failed: report, do not hide
            out[f"causal_attention_B{B}_H{H}_S{S}_D{D}_blocks512"] = {"error": str(e)[:200]}

    if want("mla_decode"):
        # The reference's MLA benchmark shape (benchmarks/decode.py:152-173): batch 32, contexts around 2048 of a
        # 4096-position cache, 64 heads, 512 latents + 64 RoPE columns (stored 128 wide), blocks of 512.
        try:
            B, H, S = 32, 64, 4096
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
            ms = time_device(lambda: ops.mla_decode(q_c, q_r, c_kv, k_rope, lens_d, 512, out=mout, buffers=mbufs),
                             2 * iters, warm, flush)
            tokens = float(lens.sum())
            nbytes = tokens * 576 * 2  # what the math reads: 512 latents + 64 RoPE columns per position
            gbs = nbytes / ms / 1e6
            out[f"mla_decode_B{B}_H{H}_ctx1024to3072"] = {
                "ms": ms, "value": gbs, "unit": "GB/s", "algorithmic_bytes": nbytes,
                "tflops": tokens * H * (2 * 576 + 2 * 512) / ms / 1e9,
                "includes": "step-table kernel + decode (the merge of partials is fused into it)",
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak,
                             "peak_kind": pk_kind, "traffic": None}}
        except Exception as e:  # report, do not hide
            out["mla_decode"] = {"error": str(e)[:200]}

    if not want("paged_gqa_decode"):
        ops.device_status()
        return out
    q, kp, vp, bt, lengths = synthetic.decode_inputs(64, 32, 8, 128, 16, 256, 8192)
    qd, kd, vd, btd, ld = (to_device(a, device) for a in (q, kp, vp, bt, lengths))
    bufs = ops.DecodeBuffers(64, 32, 128, 256, device)
    od = torch.empty_like(qd)
    ms = time_device(lambda: ops.paged_gqa_decode(qd, kd, vd, btd, ld, out=od, buffers=bufs), 2 * iters, warm, flush)
    nbytes = float(lengths.sum()) * 4096.0
    gbs = nbytes / ms / 1e6
    out["paged_gqa_decode_B64_H32_Hkv8_D128_page16"] = {
        "ms": ms, "value": gbs, "unit": "GB/s", "algorithmic_bytes": nbytes, "includes": "step-table kernel + decode (the merge of partials is fused into it)",
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak,
                     "peak_kind": pk_kind, "traffic": None}}
    ops.device_status()
    return out


# ----------------------------------------------------------------------------------------- main arm


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-extras", action="store_true", help="skip the other single-GPU workloads and the CPU baseline")
    parser.add_argument("--only", default=None, help="run only the single-GPU workloads whose name contains this "
                        "(dense_matmul_8192, causal_matmul, causal_attention_B4, paged_gqa_decode, ...) for "
                        "--steps runs after --warmup: a short command to profile one kernel")
    args = parser.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    if os.environ.get("TJX_GEMM_PAIRS") is not None:  # A/B switch: 0 = one MMA per SM instead of one per pair of SMs
        from tilejax_b200 import ops as _ops

        _ops.set_gemm_pair_mode(int(os.environ["TJX_GEMM_PAIRS"]))
    if args.only:
        import torch

        torch.cuda.set_device(0)
        pk, pk_kind = peaks()
        print(json.dumps(extra_workloads(torch.device("cuda", 0), pk, pk_kind, args.only, max(args.steps, 1),
                                         max(args.warmup, 0))), flush=True)
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
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=device)
    pk, pk_kind = peaks()

    m = M_TOTAL // world
    # Seeded synthetic operands: this rank's rows of x (seed 0 + rank), y (seed 1) identical on every rank.
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
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(device).uuid).replace("GPU-", "")) if rank == 0 else None
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

    # ---- the dominant kernel alone (its launches, timed on their stream): the roofline's numerator
    gemm_ms = time_device(lambda: ops.gemm(op.exchange.xs, y, op.tm, op.tn, op.tk, out=op.out), args.steps, 1)
    ops.device_status()

    # ---- end to end: host buffers in, host result out, copies inside the timed region
    def e2e_step():
        # Host shard and weights in, host result out: copies, GEMMs and copies back pipelined on three streams.
        op.from_host(x_host, y_host, out_host)
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
    clocks = sampler.stop() if sampler else None  # sampled over the device-timed, kernel-alone and e2e regions

    flops_per_gpu = 2.0 * M_TOTAL * K_DIM * N_DIM
    value = world * flops_per_gpu / ms_per_step / 1e9
    gemm_tflops = flops_per_gpu / gemm_ms / 1e9
    # The burst figure for a kernel that ran at boost clocks, the sustained one when the run was long enough for
    # the power cap to pull the SM clock down (as the peak measurement's own 4 s loop was).
    throttled = bool(clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz")
                     and clocks["sm_mhz"] < 0.85 * clocks["sm_max_mhz"])
    long_run = gemm_ms * args.steps > 1000.0 or throttled
    peak = pk["bf16_tflops_sustained"] if long_run else pk["bf16_tflops"]
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
        "clocks": clocks,
        "e2e": {"value": world * flops_per_gpu / e2e_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": x_host.numel() * 2 + y_host.numel() * 2, "d2h_bytes_per_step": out_host.numel() * 2,
                "api": "tilejax_b200.collective.AllGatherMatmul.from_host with pinned host x, y and out"},
        # Kernels of this library launched inside the timed region of `value`: GEMM launches per step x steps.
        "gpu_launches": args.steps * (1 if world == 1 or op.transport == "fused" else len(op.groups)),
        "roofline": {"bound": "tensor", "kernel": "gemm_pair_kernel<3,2>", "achieved": gemm_tflops, "peak": peak,
                     "unit": "TFLOP/s", "frac": gemm_tflops / peak,
                     "peak_kind": f"{pk_kind} cuBLAS bf16, {'sustained' if long_run else 'burst'}",
                     "ms_per_launch": gemm_ms, "flops_per_launch": flops_per_gpu,
                     "nominal_frac": gemm_tflops / 2250.0,
                     "traffic": NCU_TRAFFIC_BYTES["gemm_16384x8192x8192"]},
    }
    if world == 1 and not args.no_extras:
        line["workloads"] = extra_workloads(device, pk, pk_kind)
        tflops, sec, threads, sample = cpu_port_tflops(CPU_SAMPLE_ROWS, 3, 1)
        line["cpu_baseline"] = {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
