"""The recogniser is strict: a loop nest reaches a kernel only if that kernel computes exactly what the nest says.

Matmul tile code is matched statement by statement; attention and decode code by fingerprint (the kernel function
and every helper it calls, modulo local names). The reference compiles anything; this backend has five fixed
kernels, so everything else must be a KernelError ("not a recognised schedule"), never a silently wrong result.
The last tests take the reference's OWN example sources (when its tree is at hand), build kernels from them with
the NumPy-backed stand-ins bound as `jax` / `jnp`, and check that they are recognised and mean what the oracle says.
"""

import os

import numpy as np
import pytest
from helpers import BF16, f64, make_kernel, rand_bf16, spec

import oracle
import tilejax_b200.autokernel as autokernel
from tilejax_b200 import synthetic
from tilejax_b200.autokernel import KernelError, fingerprint, jaxlike
from tilejax_b200.autokernel import kernels as K
from tilejax_b200.autokernel.recognised import RECOGNISED

MATMUL = """
def f(x, y):
    M, K = x.shape
    N = y.shape[1]
    out = {alloc}
    for i in range(0, M, 128):
        for j in range(0, N, 128):
            {mask}
            acc = jnp.zeros((128, 128), jnp.float32)
            for k in range(0, K, 128):
                acc += x[i : i + 128, k : k + 128] @ y[k : k + 128, j : j + 128]
            {after}
            out = out.at[i : i + 128, j : j + 128].set({value})
    return out
"""
TRIL_MASK = "if j > i + 127:\n                continue"
ROWS_COLS = ("rows = i + jax.lax.broadcasted_iota(jnp.int32, (128, 128), 0)\n"
             "            cols = j + jax.lax.broadcasted_iota(jnp.int32, (128, 128), 1)")


def matmul_like(value, mask="pass", after="pass", alloc="jnp.zeros((M, N), x.dtype)"):
    return make_kernel(MATMUL.format(value=value, mask=mask, after=after, alloc=alloc))


def test_the_matmul_forms_are_recognised():
    specs = (spec(256, 256), spec(256, 256))
    assert not matmul_like("acc.astype(x.dtype)").lower(*specs).plan.params["causal"]
    causal = matmul_like("jnp.where(cols <= rows, acc, 0.0).astype(x.dtype)", TRIL_MASK, ROWS_COLS).lower(*specs)
    assert causal.plan.params["causal"] and (causal.tiles, causal.total_tiles) == (3, 4)
    flipped = matmul_like("jnp.where(rows >= cols, acc, 0).astype(x.dtype)", TRIL_MASK, ROWS_COLS).lower(*specs)
    assert flipped.plan.params["causal"]
    f32 = matmul_like("acc", alloc="jnp.zeros((M, N), jnp.float32)").lower(*specs)
    assert np.dtype(f32.plan.params["out_dtype"]) == np.float32
    assert not matmul_like("acc.astype(x.dtype)", alloc="jnp.full((M, N), 0, x.dtype)").lower(*specs).plan.params["causal"]


@pytest.mark.parametrize(("value", "mask", "after", "alloc", "why"), [
    # Both compile and run correctly on the reference; a fixed matmul kernel would return other numbers.
    ("(acc * 2.0 + 1.0).astype(x.dtype)", "pass", "pass", None, "other epilogues are not built"),
    ("jnp.where(cols >= rows, acc, 7.0).astype(x.dtype)", TRIL_MASK, ROWS_COLS, None, "other epilogues are not built"),
    ("jnp.where(cols <= rows, acc, 0.0).astype(x.dtype)", TRIL_MASK,
     ROWS_COLS.replace("j + jax", "j + 1 + jax"), None, "other epilogues are not built"),
    ("jnp.where(cols <= rows, acc, 0.0).astype(x.dtype)", "pass",
     ROWS_COLS + "\n            acc = acc * 2.0", None, "other epilogues are not built"),
    ("acc.astype(x.dtype)", "pass", "acc = acc + 1.0", None, "a fused epilogue"),
    ("acc.astype(x.dtype)", "pass", "pass", "jnp.full((M, N), 1.0, x.dtype)", "allocated with zeros"),
    ("acc.astype(jnp.float32)", "pass", "pass", None, "cast to the output's dtype"),
    ("jnp.where(cols <= rows, acc, 0.0).astype(x.dtype)", "if j > i + 255:\n                continue", ROWS_COLS,
     None, "tile mask"),
])
def test_other_tile_code_is_refused_not_sent_to_the_matmul_kernel(value, mask, after, alloc, why):
    kernel = matmul_like(value, mask, after, alloc or "jnp.zeros((M, N), x.dtype)")
    with pytest.raises(KernelError, match="not a recognised schedule") as e:
        kernel.lower(spec(512, 256), spec(256, 512))
    assert why in str(e.value)


ATTENTION = """
MASK_VALUE = {mask_value}


def f(q, k, v):
    B, H, S, D = q.shape
    bq, bk = 128, 128
    dtype = q.dtype
    out = jnp.zeros((B, H, S, D), dtype)
    for b in range(B):
        for h in range(H):
            for i in range(0, S, bq):
                row_max = jnp.full((bq, 1), MASK_VALUE, jnp.float32)
                row_sum = jnp.zeros((bq, 1), jnp.float32)
                acc = jnp.zeros((bq, D), jnp.float32)
                for j in range(0, S, bk):
                    if j > i + bq - 1:
                        continue
                    s = q[b, h, i : i + bq, :] @ k[b, h, j : j + bk, :].T{scale}
                    rows = i + jax.lax.broadcasted_iota(jnp.int32, (bq, bk), 0)
                    cols = j + jax.lax.broadcasted_iota(jnp.int32, (bq, bk), 1)
                    s = jnp.where(cols <= rows, s, MASK_VALUE)
                    max_new = jnp.maximum(row_max, jnp.max(s, axis=1, keepdims=True))
                    p = jnp.exp(s - max_new)
                    alpha = jnp.exp(row_max - max_new)
                    row_sum = alpha * row_sum + jnp.sum(p, axis=1, keepdims=True)
                    acc = alpha * acc + {p} @ v[b, h, j : j + bk, :]
                    row_max = max_new
                out = out.at[b, h, i : i + bq, :].set((acc / row_sum).astype(dtype))
    return out
"""


def test_attention_is_accepted_by_what_it_computes_not_by_what_it_mentions():
    qkv = [spec(1, 2, 256, 128)] * 3
    # Local names do not matter: this is kernels.causal_attention with its tunable's blocks written out... but the
    # block sizes are part of the code, so it is a form of its own and unknown.
    same = make_kernel(ATTENTION.format(mask_value="-1e30", scale="", p="p.astype(dtype)"), name="f")
    with pytest.raises(KernelError, match="not a form of it this backend's kernel is known to compute"):
        same.lower(*qkv)
    # The package's own nest is known; a different mask value, an extra scale or an unrounded P are not — each would
    # have been sent to the fixed kernel by a recogniser that only looked for `@`, `.T`, `exp` and `maximum`.
    assert K.causal_attention.lower(*qkv, K.AttentionBlocks(128, 128)).plan.family == "attention"
    base = fingerprint.fingerprint(K.causal_attention)
    assert base in RECOGNISED["attention"]
    variants = [dict(mask_value="-1e9", scale="", p="p.astype(dtype)"), dict(mask_value="-1e30", scale=" * 0.5", p="p.astype(dtype)"),
                dict(mask_value="-1e30", scale="", p="p")]
    prints = {fingerprint.fingerprint(make_kernel(ATTENTION.format(**v), name="f")) for v in variants}
    assert len(prints) == 3 and not prints & set(RECOGNISED["attention"])
    for v in variants:
        with pytest.raises(KernelError, match="not a recognised schedule"):
            make_kernel(ATTENTION.format(**v), name="f").lower(*qkv)


def test_every_nest_of_this_package_is_in_the_table():
    for family, names in (("attention", ["causal_attention"]), ("decode", ["paged_gqa_decode", "gqa_decode"]),
                          ("mla", ["mla_decode"]), ("rmsnorm", ["rmsnorm_matmul"])):
        for name in names:
            assert fingerprint.fingerprint(getattr(K, name)) in RECOGNISED[family], name


# ----------------------------------------------------------------------------- the reference's own example sources

# The reference's examples, when its tree sits beside this repository (or where AUTOKERNEL_EXAMPLES points).
EXAMPLES = os.environ.get("AUTOKERNEL_EXAMPLES") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference", "examples")
needs_reference = pytest.mark.skipif(not os.path.isdir(EXAMPLES), reason="the reference's tree is not on this machine")


def example(file: str, **imported) -> dict:
    """The example's definitions; `imported` stands for what the file imports from its neighbours."""
    stand_ins = {"jax": jaxlike, "jnp": jaxlike.numpy, "autokernel": autokernel, "__name__": "example", **imported}
    return fingerprint.load_example(os.path.join(EXAMPLES, file), stand_ins)


@needs_reference
def test_the_references_matmul_examples_run_unmodified():
    ns = example("matmul.py")
    x, y = rand_bf16((256, 384), 0), rand_bf16((384, 256), 1)
    tiles = ns["MatmulTiles"](tm=128, tn=128, tk=128)
    lowered = ns["matmul"].lower(x, y, tiles)
    assert (lowered.steps, lowered.tiles, lowered.total_tiles) == (12, 4, 4)  # tests/test_api.py:22
    np.testing.assert_array_equal(f64(ns["matmul"].reference(x, y, tiles)), f64(oracle.matmul_ref(x, y, 128, 128, 128)))
    ns = example("causal_matmul.py", MatmulTiles=ns["MatmulTiles"])  # (`from matmul import MatmulTiles`)
    causal = ns["causal_matmul"]
    x, y = rand_bf16((512, 256), 0), rand_bf16((256, 512), 1)
    tiles = type(causal.default_tunable)(tm=128, tn=128, tk=128)
    lowered = causal.lower(x, y, tiles)
    assert lowered.plan.params["causal"] and (lowered.tiles, lowered.total_tiles, lowered.steps) == (10, 16, 20)
    np.testing.assert_array_equal(f64(causal.reference(x, y, tiles)), f64(oracle.causal_matmul_ref(x, y, 128, 128, 128)))


@needs_reference
def test_the_references_attention_example_runs_unmodified():
    ns = example("causal_attention.py")
    attention = ns["causal_attention"]  # lane-replicated row statistics, widened with jnp.tile
    assert fingerprint.fingerprint(attention) in RECOGNISED["attention"]
    q, k, v = synthetic.attention_inputs(1, 2, 512, 128)
    blocks = ns["AttentionBlocks"](block_q=128, block_kv=256)
    lowered = attention.lower(q, k, v, blocks)
    assert lowered.plan.family == "attention" and lowered.steps == 2 * (1 + 1 + 2 + 2)
    np.testing.assert_array_equal(f64(attention.reference(q, k, v, blocks)), f64(oracle.causal_attention_ref(q, k, v, 128, 256)))


@needs_reference
def test_the_references_decode_examples_run_unmodified():
    ns = example("decode.py")  # block-diagonal queries, own_blocks, lane-wide statistics
    q, kp, vp, bt, lengths = synthetic.decode_inputs(4, 8, 2, 128, 16, 32, 128, distinct_pages=True)
    lengths[:] = [0, 1, 300, 512]
    paged = ns["paged_gqa_decode"]
    assert fingerprint.fingerprint(paged) in RECOGNISED["decode"]
    lowered = paged.lower(q, kp, vp, bt, lengths)
    assert lowered.plan.family == "decode" and lowered.schedule.runtime and lowered.steps == 4 * 32
    want = oracle.paged_gqa_decode_ref(q, kp, vp, bt, lengths)
    oracle.compare("paged_gqa_decode.reference", paged.reference(q, kp, vp, bt, lengths), want, rtol=1e-6, atol=1e-6)
    kc, vc = rand_bf16((4, 512, 256), 4), rand_bf16((4, 512, 256), 5)
    tiles = ns["DecodeTiles"](block_kv=128)
    flat = ns["gqa_decode"]
    assert flat.lower(q, kc, vc, lengths, tiles).plan.params["contiguous"]
    oracle.compare("gqa_decode.reference", flat.reference(q, kc, vc, lengths, tiles),
                   oracle.gqa_decode_ref(q, kc, vc, lengths, 128), rtol=1e-6, atol=1e-6)
    q_c, q_r = rand_bf16((4, 1, 16, 512), 7, 0.01), rand_bf16((4, 1, 16, 128), 8, 0.07)
    c_kv, k_rope = rand_bf16((4, 512, 512), 9), rand_bf16((4, 512, 128), 10)
    mla = ns["mla_decode"]
    assert mla.lower(q_c, q_r, c_kv, k_rope, lengths, tiles).plan.params["mla"]
    oracle.compare("mla_decode.reference", mla.reference(q_c, q_r, c_kv, k_rope, lengths, tiles),
                   oracle.mla_decode_ref(q_c, q_r, c_kv, k_rope, lengths, 128), rtol=1e-6, atol=1e-6)


@needs_reference
def test_the_references_rmsnorm_matmul_example_runs_unmodified():
    ns = example("rmsnorm_matmul.py")  # the sum of squares kept lane-wide, (tm, 128), widened with jnp.tile
    kernel = ns["rmsnorm_matmul"]
    assert fingerprint.fingerprint(kernel) in RECOGNISED["rmsnorm"]
    rng = np.random.default_rng(0)
    x = rand_bf16((256, 384), 0)
    gamma = (1 + 0.1 * rng.standard_normal((1, 384), np.float32)).astype(BF16)
    w = rand_bf16((384, 256), 2, 1 / 16)
    tiles = ns["NormMatmulTiles"](tm=128, tn=128, tk=128)
    lowered = kernel.lower(x, gamma, w, tiles)
    assert lowered.plan.family == "rmsnorm_gemm" and (lowered.tiles, lowered.steps) == (4, 12)
    assert "tjx_rmsnorm_gemm_bf16" in lowered.source
    want = oracle.rmsnorm_matmul_ref(x, gamma, w, 128, 128, 128)
    np.testing.assert_array_equal(f64(kernel.reference(x, gamma, w, tiles)), f64(want))
    np.testing.assert_allclose(f64(want), oracle.rmsnorm_matmul_f64(x, gamma, w), rtol=2e-2, atol=0.05)
    # This package's own form of the nest means the same.
    np.testing.assert_array_equal(f64(K.rmsnorm_matmul.reference(x, gamma, w, K.NormMatmulTiles(128, 128, 128))), f64(want))


def test_a_norm_matmul_with_other_tile_code_is_refused():
    source = """
        def f(x, gamma, w):
            M, D = x.shape
            N = w.shape[1]
            out = jnp.zeros((M, N), x.dtype)
            for i in range(0, M, 128):
                for j in range(0, N, 128):
                    acc = jnp.zeros((128, 128), jnp.float32)
                    sum_sq = jnp.zeros((128, 1), jnp.float32)
                    for k in range(0, D, 128):
                        xk = x[i : i + 128, k : k + 128].astype(jnp.float32)
                        sum_sq += jnp.sum(xk * xk, axis=1, keepdims=True)
                        acc += (xk * gamma[0:1, k : k + 128].astype(jnp.float32)).astype(x.dtype) @ w[k : k + 128, j : j + 128]
                    scale = jax.lax.rsqrt(sum_sq / D + 1e-5)
                    out = out.at[i : i + 128, j : j + 128].set((acc * scale).astype(x.dtype))
            return out
        """
    with pytest.raises(KernelError, match="not a form of it this backend's kernel is known to compute"):
        make_kernel(source).lower(spec(256, 256), spec(1, 256), spec(256, 256))  # another eps: another function


@needs_reference
def test_the_references_collective_example_is_recognised():
    ns = example("collective_matmul.py")
    kernel = ns["all_gather_matmul"]
    lowered = kernel.lower(spec(512, 256), spec(256, 512), type(kernel.default_tunable)())
    assert lowered.plan.params["gathered"] == "xs" and "all_gather" in lowered.source
    x, w = rand_bf16((512, 256), 0), rand_bf16((256, 512), 1)
    np.testing.assert_array_equal(f64(kernel.reference(x, w, type(kernel.default_tunable)())),
                                  f64(oracle.matmul_ref(x, w, 256, 512, 256)))
