"""The hot-path operators on CUDA tensors: thin host wrappers that check shapes, keep the static tables on the
device and call the C ABI (include/tilejax_b200.h) on the current CUDA stream.

PyTorch is used for device memory and streams only. Nothing here computes on the CPU, and there is no fallback:
without the built library or an sm_100 GPU the calls raise.
"""

from __future__ import annotations

import ctypes
import hashlib
from functools import lru_cache

import numpy as np
import torch

from . import schedule as _schedule
from ._lib import check, library


def _ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors: torch.Tensor) -> torch.device:
    device = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise ValueError("tilejax_b200 operators take CUDA tensors (there is no CPU path)")
        if t.device != device:
            raise ValueError("all tensors must be on the same device")
        if not t.is_contiguous():
            raise ValueError("tensors must be contiguous (row-major)")
    return device


_table_cache: dict[tuple, torch.Tensor] = {}


def device_table(key: tuple, values: np.ndarray, device: torch.device) -> torch.Tensor:
    """A static int32 table on `device`, uploaded once per (contents, device). `key` only labels the entry: two
    kernels whose names and shapes agree but whose masks differ get different tables."""
    host = np.ascontiguousarray(values, np.int32)
    full = (key, host.shape, hashlib.blake2b(host.tobytes(), digest_size=16).digest(), str(device))
    t = _table_cache.get(full)
    if t is None:
        t = torch.from_numpy(host).to(device)
        _table_cache[full] = t
    return t


def device_status() -> int:
    """Synchronise the current stream and return (clearing it) the kernels' error word; raises if non-zero."""
    code = ctypes.c_int(0)
    check(library().tjx_device_status(_stream(), ctypes.byref(code)))
    return code.value


def set_wait_limit_us(microseconds: int) -> None:
    """How long a device-side wait may last on the current device before the kernel gives up and records its code
    (1000 .. 10,000,000 microseconds; 2 s unless changed). Synchronises the device."""
    check(library().tjx_set_wait_limit_us(int(microseconds)))


# ------------------------------------------------------------------------------------------ step tables


def build_steps(lengths: torch.Tensor, blocks: int, value0: int, value_step: int,
                tile_values: torch.Tensor | None = None):
    """Device step tables for the runtime mask `value0 + k * value_step >= lengths[tile]: continue`.
    Returns (step_tile, step_code, step_count, tile_first), all int32 on the device."""
    device = _need_cuda(lengths)
    if lengths.dtype != torch.int32:
        raise ValueError("lengths must be int32")
    tiles = int(lengths.numel() if tile_values is None else tile_values.numel())
    step_tile = torch.empty(tiles * blocks, dtype=torch.int32, device=device)
    step_code = torch.empty(tiles * blocks, dtype=torch.int32, device=device)
    step_count = torch.empty(1, dtype=torch.int32, device=device)
    tile_first = torch.empty(tiles + 1, dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        check(library().tjx_build_steps(_ptr(lengths), int(lengths.numel()), _ptr(tile_values), tiles, blocks,
                                        value0, value_step, _ptr(step_tile), _ptr(step_code), _ptr(step_count),
                                        _ptr(tile_first), _stream()))
    return step_tile, step_code, step_count, tile_first


def build_steps_from_runs(run: torch.Tensor):
    """Device step tables from an evaluated mask run[tiles, blocks] (uint8 / bool)."""
    device = _need_cuda(run)
    run = run.to(torch.uint8).contiguous()
    tiles, blocks = run.shape
    step_tile = torch.empty(tiles * blocks, dtype=torch.int32, device=device)
    step_code = torch.empty(tiles * blocks, dtype=torch.int32, device=device)
    step_count = torch.empty(1, dtype=torch.int32, device=device)
    tile_first = torch.empty(tiles + 1, dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        check(library().tjx_build_steps_from_runs(_ptr(run), tiles, blocks, _ptr(step_tile), _ptr(step_code),
                                                  _ptr(step_count), _ptr(tile_first), _stream()))
    return step_tile, step_code, step_count, tile_first


# ------------------------------------------------------------------------------------------ matmul


def gemm(x: torch.Tensor, y: torch.Tensor, tm: int, tn: int, tk: int, *, causal: bool = False,
         out_dtype: torch.dtype | None = None, y_transposed: bool = False, stages: int = 0,
         tile_i: torch.Tensor | None = None, tile_j: torch.Tensor | None = None,
         fill_i: torch.Tensor | None = None, fill_j: torch.Tensor | None = None,
         out: torch.Tensor | None = None) -> torch.Tensor:
    """out = x @ y (or x @ y.T), bf16 operands, f32 accumulation, by tiles of (tm, tn). With tile tables only the
    listed tiles are computed and the fill tiles are zeroed; other tiles of `out` are left as they are. K is always
    summed in one order, so a product computed in several launches over row ranges is bit-equal to the same product
    in one launch (the collective matmul relies on that)."""
    device = _need_cuda(x, y)
    if x.dtype != torch.bfloat16 or y.dtype != torch.bfloat16:
        raise ValueError("x and y must be bfloat16")
    M, K = x.shape
    N = y.shape[0] if y_transposed else y.shape[1]
    if (y.shape[1] if y_transposed else y.shape[0]) != K:
        raise ValueError("x and y do not share their reduction dimension")
    out_dtype = torch.bfloat16 if out_dtype is None else out_dtype
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("the output is bfloat16 or float32")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=device)
    elif out.shape != (M, N) or out.dtype != out_dtype or not out.is_contiguous() or out.device != device:
        raise ValueError("out has the wrong shape, dtype or layout")
    n_tiles = 0 if tile_i is None else int(tile_i.numel())
    n_fills = 0 if fill_i is None else int(fill_i.numel())
    with torch.cuda.device(device):
        check(library().tjx_gemm_bf16(_ptr(x), _ptr(y), _ptr(out), M, N, K, int(y_transposed), tm, tn, tk, stages,
                                      int(out_dtype == torch.float32), int(causal), _ptr(tile_i), _ptr(tile_j),
                                      n_tiles, _ptr(fill_i), _ptr(fill_j), n_fills, _stream()))
    return out


_rmsnorm_workspaces: dict[tuple, torch.Tensor] = {}


def rmsnorm_matmul(x: torch.Tensor, gamma: torch.Tensor, w: torch.Tensor, tm: int = 512, tn: int = 512, tk: int = 512,
                   eps: float = 1e-6, out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """The `rmsnorm_matmul` loop nest (examples/rmsnorm_matmul.py:31-47): rsqrt(mean(x^2) + eps) * ((x * gamma) @ w),
    x (M, D), gamma (1, D), w (D, N). The gamma-scaled operand and the row scales go through a scratch buffer kept
    per (M, D, device, stream)."""
    device = _need_cuda(x, gamma, w)
    if any(t.dtype != torch.bfloat16 for t in (x, gamma, w)):
        raise ValueError("x, gamma and w must be bfloat16")
    M, D = x.shape
    if gamma.shape != (1, D) or w.shape[0] != D or w.dim() != 2:
        raise ValueError("x is (M, D), gamma (1, D), w (D, N)")
    N = w.shape[1]
    out_dtype = torch.bfloat16 if out_dtype is None else out_dtype
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("the output is bfloat16 or float32")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=device)
    elif out.shape != (M, N) or out.dtype != out_dtype or not out.is_contiguous() or out.device != device:
        raise ValueError("out has the wrong shape, dtype or layout")
    with torch.cuda.device(device):
        key = (M, D, str(device), torch.cuda.current_stream(device).cuda_stream)
        ws = _rmsnorm_workspaces.get(key)
        if ws is None:
            ws = torch.empty(int(library().tjx_rmsnorm_gemm_workspace_bytes(M, D)), dtype=torch.uint8, device=device)
            _rmsnorm_workspaces.clear()  # one shape at a time: the scratch is as large as x
            _rmsnorm_workspaces[key] = ws
        check(library().tjx_rmsnorm_gemm_bf16(_ptr(x), _ptr(gamma), _ptr(w), _ptr(out), M, N, D, float(eps), min(tm, M),
                                              min(tn, N), min(tk, D), int(out_dtype == torch.float32), _ptr(ws),
                                              ws.numel(), _stream()))
    return out


def all_gather_gemm(x_own: torch.Tensor, peer_shards: list[torch.Tensor | None], gathered: torch.Tensor,
                    y: torch.Tensor, out: torch.Tensor, me: int, tm: int, tn: int, tk: int, tile_i: torch.Tensor,
                    tile_j: torch.Tensor, arrivals: torch.Tensor, epoch: int) -> torch.Tensor:
    """out = all_gather(x) @ y in one launch: the GEMM's copier warps pull `peer_shards[r]` (rank r's shard as
    mapped into this process; entry `me` is ignored) into `gathered` while the own shard's tiles run. The caller
    orders the launch against the peers with its own barrier (see `collective.AllGatherMatmul`)."""
    device = _need_cuda(x_own, y)
    ranks = len(peer_shards)
    m, K = x_own.shape
    N = y.shape[1]
    if gathered.shape != (ranks * m, K) or out.shape != (ranks * m, N) or y.shape[0] != K:
        raise ValueError("gathered is [ranks * m, K], y [K, N], out [ranks * m, N]")
    if any(t.dtype != torch.bfloat16 for t in (x_own, gathered, y, out)):
        raise ValueError("operands and output are bfloat16")
    if arrivals.dtype != torch.int32 or arrivals.numel() != ranks * m // 256:
        raise ValueError("arrivals is int32[ranks * m / 256]")
    pointers = (ctypes.c_void_p * ranks)(*[None if t is None or r == me else t.data_ptr()
                                           for r, t in enumerate(peer_shards)])
    with torch.cuda.device(device):
        check(library().tjx_all_gather_gemm_bf16(_ptr(x_own), pointers, _ptr(gathered), _ptr(y), _ptr(out), ranks, me,
                                                 m, N, K, tm, tn, tk, _ptr(tile_i), _ptr(tile_j),
                                                 int(tile_i.numel()), _ptr(arrivals), int(epoch), _stream()))
    return out


def set_gemm_cta_limit(max_ctas: int) -> None:
    """Cap the persistent GEMM's grid for this thread's following launches (0 = one CTA per SM)."""
    check(library().tjx_gemm_set_cta_limit(int(max_ctas)))


def set_gemm_pair_mode(mode: int | bool) -> None:
    """How this thread's GEMM launches map pieces to SMs: 1 / True (the default; 3 is the same) one MMA per pair of
    SMs in 256 x 256 pieces when the tiles allow it; 2 the same with 256 x 128 pieces (an A/B switch, slower);
    0 / False never pairs. Values do not depend on it."""
    check(library().tjx_gemm_set_pair_mode(int(mode)))


def matmul(x: torch.Tensor, y: torch.Tensor, tm: int = 512, tn: int = 512, tk: int = 512, **kw) -> torch.Tensor:
    """The `matmul` loop nest (examples/matmul.py:22-35): tiles clipped to the matrix as its prologue does."""
    M, K = x.shape
    N = y.shape[1]
    return gemm(x, y, min(tm, M), min(tn, N), min(tk, K), **kw)


def causal_matmul(x: torch.Tensor, y: torch.Tensor, tm: int = 512, tn: int = 512, tk: int = 512, **kw) -> torch.Tensor:
    """The `causal_matmul` loop nest (examples/causal_matmul.py:23-40): tril(x @ y); tiles wholly above the
    diagonal are never loaded or multiplied, only written with zeros."""
    M, K = x.shape
    N = y.shape[1]
    tm, tn, tk = min(tm, M), min(tn, N), min(tk, K)
    sch = _schedule.causal_matmul_schedule(M, N, K, tm, tn, tk)
    tables = {}
    for name, values in sch.tables.items():
        tables[name] = device_table(("causal_matmul", M, N, tm, tn, name), values, x.device)
    return gemm(x, y, tm, tn, tk, causal=True, **tables, **kw)


# ------------------------------------------------------------------------------------------ attention


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, block_q: int = 512, block_kv: int = 512,
                     out: torch.Tensor | None = None) -> torch.Tensor:
    """The `causal_attention` loop nest (examples/causal_attention.py:37-63); q pre-scaled by the caller."""
    device = _need_cuda(q, k, v)
    B, H, S, D = q.shape
    if k.shape != q.shape or v.shape != q.shape:
        raise ValueError("q, k, v must have the same shape (B, H, S, D)")
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise ValueError("q, k, v must be bfloat16")
    bq, bk = min(block_q, S), min(block_kv, S)
    step_tile, step_code = _attention_tables(B, H, S, bq, bk, device)
    if out is None:
        out = torch.empty_like(q)
    with torch.cuda.device(device):
        check(library().tjx_causal_attention_bf16(_ptr(q), _ptr(k), _ptr(v), _ptr(out), B, H, S, D, bq, bk,
                                                  _ptr(step_tile), _ptr(step_code), step_tile.numel(), S // bq, _stream()))
    return out


def _attention_tables(B: int, H: int, S: int, bq: int, bk: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """The causal step tables of one (batch, head): which key blocks each query tile visits, on the device."""
    sch = _schedule.causal_attention_schedule(B, H, S, bq, bk)
    if sch.step_tables:
        tile, code = sch.tables["step_tile"], sch.tables["step_code"]
    else:  # the mask skips nothing (one query block, or one key block): every (tile, block) step, written out
        nq, nk = S // bq, S // bk
        tile = np.repeat(np.arange(nq, dtype=np.int32), nk)
        block = np.tile(np.arange(nk, dtype=np.int32), nq)
        code = (block << _schedule.CODE_SHIFT) | ((block == 0) << 1) | (block == nk - 1)
    return (device_table(("attn", S, bq, bk, "tile"), tile, device), device_table(("attn", S, bq, bk, "code"), code, device))


_block_workspaces: dict[tuple, torch.Tensor] = {}


def attention_block(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gamma: torch.Tensor, w_up: torch.Tensor,
                    w_down: torch.Tensor, block_q: int = 256, block_kv: int = 256, block_f: int = 1024,
                    eps: float = 1e-6, out: torch.Tensor | None = None) -> torch.Tensor:
    """The `attention_block` loop nest (examples/attention_block.py:49-85): causal attention over all heads, RMSNorm
    of the heads side by side, then gelu(n @ w_up) @ w_down; q pre-scaled by the caller. `block_f` is accepted for
    the nest's signature: it orders the reference's f32 additions, nothing else."""
    tensors = (q, k, v, gamma, w_up, w_down)
    if any(t.dtype != torch.bfloat16 for t in tensors):
        raise ValueError("q, k, v, gamma, w_up and w_down must be bfloat16")
    if q.ndim != 4 or k.shape != q.shape or v.shape != q.shape:
        raise ValueError("q, k, v must have the same shape (B, H, S, Dh)")
    B, H, S, Dh = q.shape
    D = H * Dh
    if gamma.shape != (1, D) or w_up.ndim != 2 or w_up.shape[0] != D or w_down.shape != (w_up.shape[1], D):
        raise ValueError(f"gamma must be (1, {D}), w_up ({D}, F) and w_down (F, {D})")
    F = w_up.shape[1]
    if block_f <= 0:
        raise ValueError("block_f must be positive")
    device = _need_cuda(*tensors)
    bq, bk = min(block_q, S), min(block_kv, S)
    step_tile, step_code = _attention_tables(B, H, S, bq, bk, device)
    if out is None:
        out = torch.empty(B, S, D, dtype=torch.bfloat16, device=device)
    with torch.cuda.device(device):
        need = int(library().tjx_attention_block_workspace_bytes(B, H, S, Dh, F))
        key = (device, need)
        ws = _block_workspaces.get(key)
        if ws is None:
            _block_workspaces.clear()  # one shape at a time: the scratch holds every intermediate of the block
            ws = _block_workspaces[key] = torch.empty(max(need, 256), dtype=torch.uint8, device=device)
        check(library().tjx_attention_block_bf16(_ptr(q), _ptr(k), _ptr(v), _ptr(gamma), _ptr(w_up), _ptr(w_down), _ptr(out),
                                                 B, H, S, Dh, F, bq, bk, float(eps), _ptr(step_tile), _ptr(step_code),
                                                 step_tile.numel(), S // bq, _ptr(ws), ws.numel(), _stream()))
    return out


# ------------------------------------------------------------------------------------------ decode


@lru_cache(maxsize=None)
def _decode_workspace_bytes(B: int, T: int, H: int, D: int, pages: int) -> int:
    return int(library().tjx_paged_gqa_decode_workspace_bytes(B, T, H, D, pages))


class DecodeBuffers:
    """The step tables and scratch one `paged_gqa_decode` call fills; reusable across calls of the same sizes."""

    def __init__(self, B: int, H: int, D: int, pages_per_seq: int, device: torch.device, T: int = 1):
        n = B * pages_per_seq
        self.key = (B, T, H, D, pages_per_seq, str(device))
        self.step_tile = torch.empty(n, dtype=torch.int32, device=device)
        self.step_code = torch.empty(n, dtype=torch.int32, device=device)
        self.step_count = torch.empty(1, dtype=torch.int32, device=device)
        self.tile_first = torch.empty(B + 1, dtype=torch.int32, device=device)
        self.workspace_bytes = _decode_workspace_bytes(B, T, H, D, pages_per_seq)
        self.workspace = torch.empty(self.workspace_bytes + 256, dtype=torch.uint8, device=device)

    def workspace_ptr(self) -> int:
        return (self.workspace.data_ptr() + 255) & ~255


def paged_gqa_decode(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_tables: torch.Tensor,
                     lengths: torch.Tensor, out: torch.Tensor | None = None,
                     buffers: DecodeBuffers | None = None) -> torch.Tensor:
    """The `paged_gqa_decode` loop nest (examples/decode.py:199-223): q (B, T, H, D) holds T new tokens per
    sequence (`lengths` counts them; token t sits at position lengths[b] - T + t and sees the positions up to its
    own). The step tables the call built on the device are left in `buffers` (pass one to inspect or reuse them)."""
    device = _need_cuda(q, k_pages, v_pages, block_tables, lengths)
    B, T, H, D = q.shape
    num_pages, page_size, W = k_pages.shape
    if v_pages.shape != k_pages.shape or W % D != 0:
        raise ValueError("k_pages and v_pages must both be (num_pages, page_size, Hkv * D)")
    if block_tables.dtype != torch.int32 or lengths.dtype != torch.int32:
        raise ValueError("block_tables and lengths must be int32")
    if block_tables.shape[0] != B or lengths.shape != (B,):
        raise ValueError("block_tables is (B, pages_per_seq) and lengths (B,)")
    Hkv = W // D
    pages_per_seq = block_tables.shape[1]
    if not q.is_contiguous():
        raise ValueError("q must be contiguous (B, T, H, D)")
    if buffers is None or buffers.key != (B, T, H, D, pages_per_seq, str(device)):
        buffers = DecodeBuffers(B, H, D, pages_per_seq, device, T)
    if out is None:
        out = torch.empty_like(q)
    with torch.cuda.device(device):
        check(library().tjx_paged_gqa_decode_bf16(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_tables), _ptr(lengths), _ptr(out), B, T, H, Hkv, D,
            page_size, pages_per_seq, num_pages, _ptr(buffers.step_tile), _ptr(buffers.step_code),
            _ptr(buffers.step_count), _ptr(buffers.tile_first), ctypes.c_void_p(buffers.workspace_ptr()),
            buffers.workspace_bytes, _stream()))
    paged_gqa_decode.last_buffers = buffers
    return out


@lru_cache(maxsize=16)
def _identity_block_table(B: int, blocks: int, device: str) -> torch.Tensor:
    return torch.arange(B * blocks, dtype=torch.int32, device=device).reshape(B, blocks)


def gqa_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, lengths: torch.Tensor,
               block_kv: int = 512, out: torch.Tensor | None = None,
               buffers: DecodeBuffers | None = None) -> torch.Tensor:
    """The `gqa_decode` loop nest (examples/decode.py:176-196), T new tokens per sequence: the contiguous cache
    (B, S, Hkv * D) is the page pool whose block table is the identity — sequence b's block j is page
    b * (S / block) + j — so the paged kernel runs unchanged, device step tables included."""
    _need_cuda(q, k_cache, v_cache, lengths)
    B, S, W = k_cache.shape
    block = min(block_kv, S)
    if v_cache.shape != k_cache.shape or S % block or not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("caches are contiguous (B, S, Hkv * D) with S a multiple of the block")
    blocks = S // block
    table = _identity_block_table(B, blocks, str(q.device))
    return paged_gqa_decode(q, k_cache.view(B * blocks, block, W), v_cache.view(B * blocks, block, W), table, lengths,
                            out=out, buffers=buffers)


class MlaBuffers:
    """The step tables and scratch one `mla_decode` call fills; reusable across calls of the same sizes."""

    def __init__(self, B: int, H: int, S: int, block: int, device: torch.device, T: int = 1):
        n = B * (S // block)
        self.key = (B, T, H, S, block, str(device))
        self.step_tile = torch.empty(n, dtype=torch.int32, device=device)
        self.step_code = torch.empty(n, dtype=torch.int32, device=device)
        self.step_count = torch.empty(1, dtype=torch.int32, device=device)
        self.tile_first = torch.empty(B + 1, dtype=torch.int32, device=device)
        self.workspace_bytes = int(library().tjx_mla_decode_workspace_bytes(B, T, H, S, block))
        self.workspace = torch.empty(self.workspace_bytes + 256, dtype=torch.uint8, device=device)

    def workspace_ptr(self) -> int:
        return (self.workspace.data_ptr() + 255) & ~255


def set_mla_mode(mode: int) -> None:
    """Which kernel `mla_decode` launches: 1 (the default) tcgen05 with 64 rows per CTA, 0 warp-level MMA with 16.
    Values agree to rounding."""
    check(library().tjx_mla_set_mode(int(mode)))


def mla_decode(q_c: torch.Tensor, q_r: torch.Tensor, c_kv: torch.Tensor, k_rope: torch.Tensor, lengths: torch.Tensor,
               block_kv: int = 512, out: torch.Tensor | None = None, buffers: MlaBuffers | None = None) -> torch.Tensor:
    """The `mla_decode` loop nest (examples/decode.py:226-250) for T new tokens per sequence: q_c (B, T, H, 512),
    q_r (B, T, H, 128), the latent cache (B, S, 512) and the RoPE key cache (B, S, 128); out (B, T, H, 512), each
    head's softmax-weighted latents. New token t sees the positions up to lengths[b] - T + t."""
    device = _need_cuda(q_c, q_r, c_kv, k_rope, lengths)
    B, T, H, C = q_c.shape
    S, R = c_kv.shape[1], k_rope.shape[2]
    if q_r.shape != (B, T, H, R) or c_kv.shape != (B, S, C) or k_rope.shape != (B, S, R) or lengths.shape != (B,):
        raise ValueError("q_c (B, T, H, C), q_r (B, T, H, R), c_kv (B, S, C), k_rope (B, S, R), lengths (B,)")
    if lengths.dtype != torch.int32 or any(t.dtype != torch.bfloat16 for t in (q_c, q_r, c_kv, k_rope)):
        raise ValueError("lengths is int32, the other operands bfloat16")
    if not all(t.is_contiguous() for t in (q_c, q_r, c_kv, k_rope)):
        raise ValueError("operands must be contiguous")
    block = min(block_kv, S)
    if S % block:
        raise ValueError("the block must divide the cache length")
    if buffers is None or buffers.key != (B, T, H, S, block, str(device)):
        buffers = MlaBuffers(B, H, S, block, device, T)
    if out is None:
        out = torch.empty_like(q_c)
    with torch.cuda.device(device):
        check(library().tjx_mla_decode_bf16(
            _ptr(q_c), _ptr(q_r), _ptr(c_kv), _ptr(k_rope), _ptr(lengths), _ptr(out), B, T, H, S, C, R, block,
            _ptr(buffers.step_tile), _ptr(buffers.step_code), _ptr(buffers.step_count), _ptr(buffers.tile_first),
            ctypes.c_void_p(buffers.workspace_ptr()), buffers.workspace_bytes, _stream()))
    mla_decode.last_buffers = buffers
    return out


# ------------------------------------------------------------------------------------------ ragged paged attention


def _rpa_sizes(kv_cache: torch.Tensor, kv_lens: torch.Tensor, page_indices: torch.Tensor) -> tuple[int, ...]:
    if kv_cache.dim() != 5 or kv_cache.shape[3] != 2 or kv_cache.dtype != torch.bfloat16:
        raise ValueError("the cache is (pages, page_size, Hkv, 2, D) bfloat16: each head's key and value side by side")
    num_pages, page_size, Hkv, _, D = kv_cache.shape
    S = kv_lens.shape[0]
    if page_indices.dim() != 1 or S == 0 or page_indices.shape[0] % S:
        raise ValueError("page_indices is (S * pages_per_seq,), sequence s's pages at s * pages_per_seq")
    if any(t.dtype != torch.int32 for t in (kv_lens, page_indices)):
        raise ValueError("kv_lens and page_indices must be int32")
    return num_pages, page_size, Hkv, D, S, page_indices.shape[0] // S


def rpa_write(kv_cache: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, kv_lens: torch.Tensor,
              page_indices: torch.Tensor, cu_q_lens: torch.Tensor, distribution: torch.Tensor) -> torch.Tensor:
    """`write_new_tokens` (examples/ragged_paged_attention.py:74-79): the step's new keys and values (T, Hkv, D)
    written IN PLACE into the cache at positions [kv_len - q_len, kv_len) of their sequences; returns the cache."""
    num_pages, page_size, Hkv, D, S, pps = _rpa_sizes(kv_cache, kv_lens, page_indices)
    device = _need_cuda(kv_cache, keys, values, kv_lens, page_indices, cu_q_lens, distribution)
    if keys.shape != values.shape or keys.dim() != 3 or keys.shape[1:] != (Hkv, D) or keys.dtype != torch.bfloat16 \
            or values.dtype != torch.bfloat16:
        raise ValueError("keys and values are (T, Hkv, D) bfloat16")
    if cu_q_lens.shape != (S + 1,) or distribution.shape != (3,) or cu_q_lens.dtype != torch.int32 \
            or distribution.dtype != torch.int32:
        raise ValueError("cu_q_lens is int32 (S + 1,), distribution int32 (3,)")
    with torch.cuda.device(device):
        check(library().tjx_rpa_write_bf16(_ptr(kv_cache), _ptr(keys), _ptr(values), _ptr(kv_lens), _ptr(page_indices),
                                           _ptr(cu_q_lens), _ptr(distribution), keys.shape[0], S, Hkv, D, page_size, pps,
                                           num_pages, _stream()))
    return kv_cache


def rpa_write_runs(kv_cache: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, page_indices: torch.Tensor,
                   write_page: torch.Tensor, write_rows: torch.Tensor, write_first: torch.Tensor,
                   write_stop: torch.Tensor, n_writes: torch.Tensor) -> torch.Tensor:
    """The reference's `rpa_write` kernel (examples/ragged_paged_attention.py:33-47) on its own run tables: run
    w < n_writes[0] copies the tokens from write_rows[w] on to rows write_first[w] .. write_stop[w] - 1 of page
    page_indices[write_page[w]] of the cache (pages, page_size, Hkv, 2, D), IN PLACE; returns the cache."""
    device = _need_cuda(kv_cache, keys, values, page_indices, write_page, write_rows, write_first, write_stop, n_writes)
    if kv_cache.dim() != 5 or kv_cache.shape[3] != 2 or kv_cache.dtype != torch.bfloat16 or not kv_cache.is_contiguous():
        raise ValueError("kv_cache is a contiguous (pages, page_size, Hkv, 2, D) bfloat16 tensor")
    num_pages, page_size, Hkv, _, D = kv_cache.shape
    if keys.shape != values.shape or keys.dim() != 3 or keys.shape[1:] != (Hkv, D) or keys.dtype != torch.bfloat16 \
            or values.dtype != torch.bfloat16:
        raise ValueError("keys and values are (T, Hkv, D) bfloat16")
    tables = (write_page, write_rows, write_first, write_stop)
    if any(t.dtype != torch.int32 or t.dim() != 1 or t.shape != write_page.shape for t in tables) \
            or page_indices.dtype != torch.int32 or page_indices.dim() != 1 or n_writes.dtype != torch.int32 \
            or n_writes.numel() < 1:
        raise ValueError("the run tables are int32 vectors of one length, page_indices an int32 vector, n_writes int32 (1,)")
    with torch.cuda.device(device):
        check(library().tjx_rpa_write_runs_bf16(_ptr(kv_cache), _ptr(keys), _ptr(values), _ptr(page_indices),
                                                _ptr(write_page), _ptr(write_rows), _ptr(write_first), _ptr(write_stop),
                                                _ptr(n_writes), keys.shape[0], page_indices.numel(), write_page.numel(),
                                                Hkv, D, page_size, num_pages, _stream()))
    return kv_cache


_rpa_workspaces: dict[tuple, torch.Tensor] = {}


def rpa_decode(q: torch.Tensor, kv_cache: torch.Tensor, kv_lens: torch.Tensor, page_indices: torch.Tensor,
               distribution: torch.Tensor, sm_scale: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """`rpa_decode` (examples/ragged_paged_attention.py:121-149): q (T, H, D); sequence s < distribution[0] is token
    s, whose row becomes its attention output over the kv_lens[s] cached positions (scores times sm_scale); every
    other row stays the query. `out=q` updates the queries in place, as the reference's donated buffer is."""
    num_pages, page_size, Hkv, D, S, pps = _rpa_sizes(kv_cache, kv_lens, page_indices)
    device = _need_cuda(q, kv_cache, kv_lens, page_indices, distribution)
    if q.dim() != 3 or q.shape[2] != D or q.dtype != torch.bfloat16:
        raise ValueError("q is (T, H, D) bfloat16")
    if distribution.shape != (3,) or distribution.dtype != torch.int32:
        raise ValueError("distribution is int32 (3,)")
    T, H, _ = q.shape
    if out is None:
        out = torch.empty_like(q)
    elif out.shape != q.shape or out.dtype != q.dtype or not out.is_contiguous() or out.device != q.device:
        raise ValueError("out must look like q")
    with torch.cuda.device(device):
        need = int(library().tjx_rpa_decode_workspace_bytes(T, S, H, D, page_size, pps))
        key = (str(device), need)
        ws = _rpa_workspaces.get(key)
        if ws is None:
            _rpa_workspaces.clear()
            ws = _rpa_workspaces[key] = torch.empty(need + 256, dtype=torch.uint8, device=device)
        ws_ptr = (ws.data_ptr() + 255) & ~255
        check(library().tjx_rpa_decode_bf16(_ptr(q), _ptr(out), _ptr(kv_cache), _ptr(kv_lens), _ptr(page_indices),
                                            _ptr(distribution), T, S, H, Hkv, D, page_size, pps, num_pages,
                                            float(sm_scale), ctypes.c_void_p(ws_ptr), need, _stream()))
    return out


def rpa_prefill(q: torch.Tensor, kv_cache: torch.Tensor, kv_lens: torch.Tensor, page_indices: torch.Tensor,
                cu_q_lens: torch.Tensor, distribution: torch.Tensor, sm_scale: float = 1.0,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """`rpa_prefill` with its tiles (examples/ragged_paged_attention.py:196-275): the new tokens of every sequence in
    [distribution[0], distribution[2]) attend causally over their sequence's cache; their rows of q (T, H, D) become the
    outputs, every other row stays. `out=q` updates in place."""
    num_pages, page_size, Hkv, D, S, pps = _rpa_sizes(kv_cache, kv_lens, page_indices)
    device = _need_cuda(q, kv_cache, kv_lens, page_indices, cu_q_lens, distribution)
    if q.dim() != 3 or q.shape[2] != D or q.dtype != torch.bfloat16:
        raise ValueError("q is (T, H, D) bfloat16")
    if cu_q_lens.shape != (S + 1,) or distribution.shape != (3,) or cu_q_lens.dtype != torch.int32 \
            or distribution.dtype != torch.int32:
        raise ValueError("cu_q_lens is int32 (S + 1,), distribution int32 (3,)")
    T, H, _ = q.shape
    if out is None:
        out = torch.empty_like(q)
    elif out.shape != q.shape or out.dtype != q.dtype or not out.is_contiguous() or out.device != q.device:
        raise ValueError("out must look like q")
    with torch.cuda.device(device):
        need = int(library().tjx_rpa_prefill_workspace_bytes(T, S))
        ws = torch.empty(need + 256, dtype=torch.uint8, device=device)
        ws_ptr = (ws.data_ptr() + 255) & ~255
        check(library().tjx_rpa_prefill_bf16(_ptr(q), _ptr(out), _ptr(kv_cache), _ptr(kv_lens), _ptr(page_indices),
                                             _ptr(cu_q_lens), _ptr(distribution), T, S, H, Hkv, D, page_size, pps,
                                             num_pages, float(sm_scale), ctypes.c_void_p(ws_ptr), need, _stream()))
        ws.record_stream(torch.cuda.current_stream(device))
    return out


def rpa_prefill_tiles(q: torch.Tensor, kv_cache: torch.Tensor, page_indices: torch.Tensor, tile_page: torch.Tensor,
                      tile_rows: torch.Tensor, tile_pos: torch.Tensor, n_tiles: torch.Tensor, sm_scale: float = 1.0,
                      out: torch.Tensor | None = None) -> torch.Tensor:
    """The reference's `rpa_prefill` kernel (examples/ragged_paged_attention.py:204-243) on its own tile tables: tile
    k < n_tiles[0] is the rows tile_rows[k] .. tile_rows[k + 1] - 1 of q (T, H, D), the first at cache position
    tile_pos[k], of the sequence whose pages start at page_indices[tile_page[k]]; those rows become their causal
    attention outputs, every other row stays. `out=q` updates in place."""
    device = _need_cuda(q, kv_cache, page_indices, tile_page, tile_rows, tile_pos, n_tiles)
    if kv_cache.dim() != 5 or kv_cache.shape[3] != 2 or kv_cache.dtype != torch.bfloat16 or not kv_cache.is_contiguous():
        raise ValueError("kv_cache is a contiguous (pages, page_size, Hkv, 2, D) bfloat16 tensor")
    num_pages, page_size, Hkv, _, D = kv_cache.shape
    if q.dim() != 3 or q.shape[2] != D or q.dtype != torch.bfloat16:
        raise ValueError("q is (T, H, D) bfloat16")
    max_tiles = tile_page.numel()
    if any(t.dtype != torch.int32 or t.dim() != 1 for t in (page_indices, tile_page, tile_rows, tile_pos, n_tiles)) \
            or tile_pos.numel() != max_tiles or tile_rows.numel() != max_tiles + 1 or n_tiles.numel() < 1:
        raise ValueError("tile_page and tile_pos are int32 (tiles,), tile_rows int32 (tiles + 1,), n_tiles int32 (1,)")
    T, H, _ = q.shape
    if out is None:
        out = torch.empty_like(q)
    elif out.shape != q.shape or out.dtype != q.dtype or not out.is_contiguous() or out.device != q.device:
        raise ValueError("out must look like q")
    with torch.cuda.device(device):
        need = int(library().tjx_rpa_prefill_tiles_workspace_bytes(T, max_tiles))
        ws = torch.empty(need + 256, dtype=torch.uint8, device=device)
        ws_ptr = (ws.data_ptr() + 255) & ~255
        check(library().tjx_rpa_prefill_tiles_bf16(_ptr(q), _ptr(out), _ptr(kv_cache), _ptr(page_indices), _ptr(tile_page),
                                                   _ptr(tile_rows), _ptr(tile_pos), _ptr(n_tiles), T, max_tiles,
                                                   page_indices.numel(), H, Hkv, D, page_size, num_pages, float(sm_scale),
                                                   ctypes.c_void_p(ws_ptr), need, _stream()))
        ws.record_stream(torch.cuda.current_stream(device))
    return out


def ragged_paged_attention(q: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, kv_cache: torch.Tensor,
                           kv_lens: torch.Tensor, page_indices: torch.Tensor, cu_q_lens: torch.Tensor,
                           distribution: torch.Tensor, sm_scale: float = 1.0,
                           out: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """RPA v3's step (`autokernel_rpa`, examples/ragged_paged_attention.py:279-290): the new tokens' keys and values
    written into the cache in place, the decode sequences' attention, then the others'. Returns (out (T, H, D), the
    cache); q is left as it was unless `out=q` asks for the update in place. One call into the library (tjx_ragged_paged_attention_bf16): the same results as
    rpa_write, rpa_decode and rpa_prefill one after the other, without their copy of q into out."""
    num_pages, page_size, Hkv, D, S, pps = _rpa_sizes(kv_cache, kv_lens, page_indices)
    device = _need_cuda(q, keys, values, kv_cache, kv_lens, page_indices, cu_q_lens, distribution)
    if q.dim() != 3 or q.shape[2] != D or q.dtype != torch.bfloat16 or not q.is_contiguous():
        raise ValueError("q is a contiguous (T, H, D) bfloat16 tensor")
    T, H, _ = q.shape
    if keys.shape != (T, Hkv, D) or values.shape != (T, Hkv, D) or keys.dtype != torch.bfloat16 \
            or values.dtype != torch.bfloat16:
        raise ValueError("keys and values are (T, Hkv, D) bfloat16")
    if cu_q_lens.shape != (S + 1,) or distribution.shape != (3,) or cu_q_lens.dtype != torch.int32 \
            or distribution.dtype != torch.int32:
        raise ValueError("cu_q_lens is int32 (S + 1,), distribution int32 (3,)")
    if out is None:
        out = torch.empty_like(q)
    elif out.shape != q.shape or out.dtype != q.dtype or not out.is_contiguous() or out.device != q.device:
        raise ValueError("out must look like q")
    with torch.cuda.device(device):
        need = int(library().tjx_ragged_paged_attention_workspace_bytes(T, S, H, D, page_size, pps))
        key = ("step", str(device), need)
        ws = _rpa_workspaces.get(key)
        if ws is None:
            _rpa_workspaces.clear()
            ws = _rpa_workspaces[key] = torch.empty(need + 256, dtype=torch.uint8, device=device)
        ws_ptr = (ws.data_ptr() + 255) & ~255
        check(library().tjx_ragged_paged_attention_bf16(
            _ptr(q), _ptr(keys), _ptr(values), _ptr(kv_cache), _ptr(kv_lens), _ptr(page_indices), _ptr(cu_q_lens),
            _ptr(distribution), _ptr(out), T, S, H, Hkv, D, page_size, pps, num_pages, float(sm_scale),
            ctypes.c_void_p(ws_ptr), need, _stream()))
    return out, kv_cache


def paged_gqa_decode_static(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_tables: torch.Tensor,
                            lengths: torch.Tensor, out: torch.Tensor, step_tile: torch.Tensor, step_code: torch.Tensor,
                            step_count: torch.Tensor, tile_first: torch.Tensor) -> torch.Tensor:
    """`paged_gqa_decode` for a caller that may not allocate: every buffer, the output and the step tables
    included, is passed in, and the kernels' scratch is the fixed array inside the library
    (tjx_paged_gqa_decode_bf16_static). This wrapper allocates nothing either. Sizes whose scratch would exceed
    the built-in 36 MiB raise; calls that overlap on the GPU race on the shared scratch."""
    if q.dim() != 4 or k_pages.dim() != 3 or block_tables.dim() != 2:
        raise ValueError("q is (B, T, H, D), the pages (num_pages, page_size, Hkv * D), block_tables (B, pages_per_seq)")
    B, T, H, D = q.shape
    num_pages, page_size, W = k_pages.shape
    pages_per_seq = block_tables.shape[1]
    if any(t.dtype != torch.bfloat16 for t in (q, k_pages, v_pages, out)):
        raise ValueError("q, k_pages, v_pages and out must be bfloat16")
    if any(t.dtype != torch.int32 for t in (block_tables, lengths, step_tile, step_code, step_count, tile_first)):
        raise ValueError("block_tables, lengths and the step table buffers must be int32")
    if out.shape != q.shape:
        raise ValueError("out must have q's shape (B, T, H, D)")
    if v_pages.shape != k_pages.shape or W % D != 0:
        raise ValueError("k_pages and v_pages must both be (num_pages, page_size, Hkv * D)")
    if block_tables.shape[0] != B or lengths.shape != (B,):
        raise ValueError("block_tables is (B, pages_per_seq) and lengths (B,)")
    if step_tile.numel() < B * pages_per_seq or step_code.numel() < B * pages_per_seq or tile_first.numel() < B + 1 \
            or step_count.numel() < 1:
        raise ValueError("the step table buffers are too small")
    device = _need_cuda(q, k_pages, v_pages, block_tables, lengths, out, step_tile, step_code, step_count, tile_first)
    with torch.cuda.device(device):
        check(library().tjx_paged_gqa_decode_bf16_static(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_tables), _ptr(lengths), _ptr(out), B, T, H, W // D, D,
            page_size, pages_per_seq, num_pages, _ptr(step_tile), _ptr(step_code), _ptr(step_count),
            _ptr(tile_first), _stream()))
    return out
