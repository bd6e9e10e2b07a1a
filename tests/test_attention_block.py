"""`attention_block` (examples/attention_block.py:49-85) on the CPU side: the oracle against float64, the loop nest's
own meaning against the oracle, what the front end plans for it (phases, steps — the reference's known answers,
tests/test_examples.py:179-216), and what it refuses."""

import os

import numpy as np
import pytest
from helpers import BF16, f64, make_kernel, rand_bf16, spec

import tilejax_b200.autokernel as autokernel
from oracle.attention_block import attention_block_f64, attention_block_ref
from tilejax_b200.autokernel import KernelError, fingerprint, jaxlike
from tilejax_b200.autokernel import kernels as K
from tilejax_b200.autokernel.recognised import RECOGNISED


def make_inputs(B, H, S, Dh, F, seed=0):
    """Shapes and scales of examples/attention_block.py:122-130."""
    rng = np.random.default_rng(seed)
    D = H * Dh
    q = rand_bf16((B, H, S, Dh), seed, Dh**-0.5)
    k, v = rand_bf16((B, H, S, Dh), seed + 1), rand_bf16((B, H, S, Dh), seed + 2)
    gamma = (1 + 0.1 * rng.standard_normal((1, D), np.float32)).astype(BF16)
    w_up = rand_bf16((D, F), seed + 4, D**-0.5)
    w_down = rand_bf16((F, D), seed + 5, F**-0.5)
    return q, k, v, gamma, w_up, w_down


@pytest.mark.parametrize(("block_q", "block_kv", "block_f"), [(128, 128, 1024), (256, 128, 1024), (128, 128, 128)])
def test_the_oracle_agrees_with_float64_and_the_nest_with_the_oracle(block_q, block_kv, block_f):
    inputs = make_inputs(1, 2, 256, 128, 256)
    want = attention_block_ref(*inputs, block_q, block_kv, block_f)
    exact = attention_block_f64(*inputs)
    np.testing.assert_allclose(f64(want), exact, atol=3e-2 * np.abs(exact).max())  # tests/test_examples.py:187
    tiles = K.BlockTiles(block_q=block_q, block_kv=block_kv, block_f=max(block_f, 256))
    if block_f >= 256:
        np.testing.assert_array_equal(f64(K.attention_block.reference(*inputs, tiles)), f64(want))


@pytest.mark.parametrize(("block_q", "block_kv"), [(128, 128), (256, 128)])
def test_one_block_of_hidden_units_takes_no_step_of_its_own(block_q, block_kv):
    # tests/test_examples.py:183-198: F = 512 under the default block_f, so the feed-forward loop runs inline.
    specs = (spec(1, 2, 512, 128),) * 3 + (spec(1, 256), spec(256, 512), spec(512, 256))
    lowered = K.attention_block.lower(*specs, K.BlockTiles(block_q=block_q, block_kv=block_kv))
    assert lowered.plan.family == "attention_block" and lowered.plan.params["phases"] == ("j",)
    assert lowered.steps == sum(i // block_kv + 1 for i in range(block_q - 1, 512, block_q))
    assert lowered.tiles == 512 // block_q
    assert "tjx_attention_block_bf16" in lowered.source


def test_streamed_weights_are_a_second_phase():
    # tests/test_examples.py:208-222: the feed-forward layer in four steps.
    specs = (spec(1, 2, 256, 128),) * 3 + (spec(1, 256), spec(256, 1024), spec(1024, 256))
    lowered = K.attention_block.lower(*specs, K.BlockTiles(block_q=128, block_kv=128, block_f=256))
    assert lowered.plan.params["phases"] == ("j", "f")
    assert lowered.steps == (1 + 2) + 2 * 4
    sch = lowered.plan.params["schedule"]
    assert sch.phase_counts == (2, 4) and sch.fills == 0


def test_what_the_kernels_cannot_run_is_a_kernel_error():
    with pytest.raises(KernelError, match="head_dim 128"):
        K.attention_block.lower(*((spec(1, 4, 256, 64),) * 3 + (spec(1, 256), spec(256, 1024), spec(1024, 256))))
    with pytest.raises(KernelError, match="bfloat16"):
        K.attention_block.lower(*((spec(1, 2, 256, 128, dtype=np.float32),) * 3
                                  + (spec(1, 256, dtype=np.float32), spec(256, 512, dtype=np.float32),
                                     spec(512, 256, dtype=np.float32))))
    with pytest.raises(KernelError, match=r"gamma \(1, 256\)"):
        K.attention_block.lower(*((spec(1, 2, 256, 128),) * 3 + (spec(1, 128), spec(256, 512), spec(512, 256))))


def renamed(**edits) -> str:
    """This package's nest as source text, its locals renamed (which changes nothing), then `edits` applied."""
    import inspect
    import textwrap

    source = textwrap.dedent(inspect.getsource(K.attention_block.fn))
    source = source.replace("@autokernel.kernel\n", "").replace("def attention_block(", "def f(")
    for old, new in (("row_max", "m"), ("row_sum", "l"), ("acc", "o"), ("normed", "n"), ("hidden", "u"), ("tiles", "t")):
        source = source.replace(old, new)
    for old, new in edits.values():
        assert old in source, old
        source = source.replace(old, new)
    return source


def test_the_same_code_under_other_names_is_accepted_and_other_arithmetic_is_refused():
    specs = (spec(1, 2, 256, 128),) * 3 + (spec(1, 256), spec(256, 512), spec(512, 256))
    names = dict(BlockTiles=K.BlockTiles, MASK_VALUE=K.MASK_VALUE, EPS=K.EPS)
    lowered = make_kernel(renamed(), **names).lower(*specs, K.BlockTiles(128, 128, 256))
    assert lowered.plan.family == "attention_block" and lowered.steps == 3 + 2 * 2
    for edit in (("+ EPS)", "+ 1e-5)"),                                              # another eps
                 ("* jax.lax.rsqrt(jnp.mean(a * a, axis=1, keepdims=True) + EPS)", ""),  # no norm at all
                 ("jax.nn.gelu(n @ w_up[:, f : f + bf])", "jax.nn.gelu(n @ w_up[:, f : f + bf], approximate=False)"),
                 ("jax.nn.gelu(n @ w_up[:, f : f + bf])", "jnp.maximum(n @ w_up[:, f : f + bf], 0.0)"),  # a ReLU
                 ("p[h].astype(dtype) @ vt[h]", "p[h] @ vt[h]")):                   # P not rounded before P @ v
        with pytest.raises(KernelError, match="not a form of it this backend's kernel is known to compute"):
            make_kernel(renamed(edit=edit), **names).lower(*specs, K.BlockTiles(128, 128, 256))


def test_this_packages_nest_is_in_the_table():
    assert fingerprint.fingerprint(K.attention_block) in RECOGNISED["attention_block"]


# The reference's examples, when its tree sits beside this repository (or where AUTOKERNEL_EXAMPLES points).
EXAMPLES = os.environ.get("AUTOKERNEL_EXAMPLES") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference", "examples")


@pytest.mark.skipif(not os.path.isdir(EXAMPLES), reason="the reference's tree is not on this machine")
def test_the_references_example_runs_unmodified():
    stand_ins = {"jax": jaxlike, "jnp": jaxlike.numpy, "autokernel": autokernel, "__name__": "example"}
    ns = fingerprint.load_example(os.path.join(EXAMPLES, "attention_block.py"), stand_ins)
    kernel = ns["attention_block"]  # row statistics lane-wide, (H, bq, 128), widened with `widen`
    assert fingerprint.fingerprint(kernel) in RECOGNISED["attention_block"]
    inputs = make_inputs(1, 2, 256, 128, 512)
    tiles = ns["BlockTiles"](block_q=128, block_kv=128, block_f=256)
    lowered = kernel.lower(*inputs, tiles)
    assert lowered.plan.family == "attention_block" and (lowered.tiles, lowered.steps) == (2, 3 + 2 * 2)
    want = attention_block_ref(*inputs, 128, 128, 256)
    np.testing.assert_array_equal(f64(kernel.reference(*inputs, tiles)), f64(want))
    np.testing.assert_array_equal(f64(K.attention_block.reference(*inputs, K.BlockTiles(128, 128, 256))), f64(want))
