"""The `autokernel` front end on CPU: parsing, planning, the schedules' counts, the recogniser's refusals, the
meaning of `.fn` / `.reference`, tunables and the tuner's search — modelled on the reference's tests/test_api.py,
test_parse.py, test_tunable.py, test_tune.py and test_examples.py."""

import dataclasses

import numpy as np
import pytest
from helpers import BF16, f64, rand_bf16

import oracle
import tilejax_b200.autokernel as autokernel
from tilejax_b200 import synthetic
from tilejax_b200.autokernel import Config, KernelError, KernelProfile, Pipeline, Trial, jaxlike
from tilejax_b200.autokernel import kernels as K
from tilejax_b200.autokernel.plan import Spec
from tilejax_b200.autokernel.tunable import choices, is_tunable, neighbours
from tilejax_b200.autokernel.tune import proposals, search

jnp = jaxlike.numpy
TILES = K.MatmulTiles(tm=128, tn=128, tk=128)


def spec(*shape, dtype=BF16):
    return Spec(tuple(shape), np.dtype(dtype))


# ----------------------------------------------------------------------------- lowering describes the kernel


def test_lowered_describes_the_kernel():
    # tests/test_api.py:20-30
    lowered = K.matmul.lower(spec(256, 384), spec(384, 256), TILES)
    assert (lowered.steps, lowered.tiles, lowered.total_tiles) == (12, 4, 4)
    assert lowered.pipeline == Pipeline(3, 2) and str(lowered.pipeline) == "3 input / 2 output buffers"
    assert lowered.config.tunable == TILES and str(lowered.config).startswith("MatmulTiles(tm=128")
    assert K.matmul.lower(spec(256, 384), spec(384, 256), TILES) is lowered  # built once per signature
    assert repr(K.matmul) == "<autokernel.Kernel matmul>" and K.matmul.__name__ == "matmul"
    assert K.matmul.source(spec(256, 384), spec(384, 256), TILES) == lowered.source
    assert "MatmulTiles(tm=128, tn=128, tk=128); 3 input / 2 output buffers" in lowered.source
    assert "tjx_gemm_bf16" in lowered.source and "ring of 4 slots" in lowered.source
    # Tiles that are multiples of 256 run one MMA per pair of SMs unless the pipeline asks for a ring depth.
    big = K.matmul.lower(spec(1024, 512), spec(512, 1024))
    assert "CTA pair    256 x 256 x 64" in big.source
    deep = K.matmul.lowered(K.matmul.signature(spec(1024, 512), spec(512, 1024)), Config(K.MatmulTiles(), Pipeline(4, 2)))
    assert "CTA tile    128 x 256 x 64, ring of 4 slots" in deep.source


def test_causal_matmul_skips_tiles_above_the_diagonal():
    # tests/test_examples.py:56-63
    lowered = K.causal_matmul.lower(spec(512, 256), spec(256, 512), TILES)
    assert (lowered.tiles, lowered.total_tiles, lowered.steps) == (10, 16, 20)
    want = oracle.causal_tile_tables(512, 512, 128, 128)
    for name, values in want.items():
        np.testing.assert_array_equal(lowered.schedule.tables[name], values)
    one = K.causal_matmul.lower(spec(128, 128), spec(128, 128), TILES)
    assert one.schedule.tables == {}  # tests/test_schedule.py:189-198


def test_attention_tables_hold_one_batch_heads_pattern():
    # tests/test_examples.py:91-95
    lowered = K.causal_attention.lower(*[spec(2, 4, 512, 128)] * 3, K.AttentionBlocks(128, 128))
    assert lowered.steps == 2 * 4 * (1 + 2 + 3 + 4) and lowered.schedule.repeats == 8
    assert len(lowered.schedule.tables["step_tile"]) == 10
    big = K.causal_attention.lower(*[spec(4, 16, 2048, 128)] * 3, K.AttentionBlocks())
    assert (big.tiles, big.steps) == (256, 640)


def test_decode_steps_are_found_on_the_device():
    lowered = K.paged_gqa_decode.lower(spec(4, 1, 8, 128), spec(16, 128, 256), spec(16, 128, 256),
                                       spec(4, 4, dtype=np.int32), spec(4, dtype=np.int32))
    assert lowered.schedule.runtime and lowered.schedule.empty and lowered.steps == 16  # at most
    assert "built on the device from lengths" in lowered.source
    # The contiguous cache is the same kernel over the identity block table (examples/decode.py:176-196).
    flat = K.gqa_decode.lower(spec(4, 1, 8, 128), spec(4, 1024, 256), spec(4, 1024, 256), spec(4, dtype=np.int32),
                              K.DecodeTiles(block_kv=256))
    assert flat.schedule.runtime and flat.steps == 4 * 4 and "identity block table" in flat.source
    assert flat.plan.params["page"] == 256 and flat.plan.params["num_pages"] == 16
    # Absorbed MLA decode (examples/decode.py:226-250): its own kernel, the same device tables.
    mla = K.mla_decode.lower(spec(4, 1, 16, 512), spec(4, 1, 16, 128), spec(4, 1024, 512), spec(4, 1024, 128),
                             spec(4, dtype=np.int32), K.DecodeTiles(block_kv=256))
    assert mla.schedule.runtime and mla.steps == 4 * 4 and "tjx_mla_decode_bf16" in mla.source


def test_tiles_clamp_to_the_matrix_and_neighbours_that_build_the_same_kernel_are_skipped():
    kernel, sig = K.matmul, K.matmul.signature(spec(256, 256), spec(256, 256))
    plan, _ = kernel.build(sig, K.MatmulTiles())  # 512 clamps to 256
    assert [(r.step, r.count) for r in plan.loops] == [(256, 1)] * 3
    trial = Trial(Config(K.MatmulTiles(), Pipeline()), KernelProfile(1e-5, 0.5, 0.1, 1))
    steps = [c.tunable for c in proposals(kernel, sig, trial)]
    assert K.MatmulTiles(tm=1024) not in steps and K.MatmulTiles(tm=256) not in steps  # the same kernel


# ----------------------------------------------------------------------------- the meaning of a kernel


def test_reference_accumulates_in_f32_and_fn_runs_as_written():
    x, y = rand_bf16((256, 384), 0), rand_bf16((384, 256), 1)
    ref = K.matmul.reference(x, y, TILES)
    np.testing.assert_array_equal(f64(ref), f64(oracle.matmul_ref(x, y, 128, 128, 128)))
    fn = jaxlike.to_numpy(K.matmul.fn(jaxlike.Array(x), jaxlike.Array(y), TILES))
    assert fn.dtype == BF16  # plain `bf16 @ bf16` rounds each block product to bf16
    np.testing.assert_allclose(f64(fn), f64(x) @ f64(y), rtol=5e-2, atol=2.0)


def test_references_equal_the_oracle_for_every_nest():
    x, y = rand_bf16((512, 256), 0), rand_bf16((256, 512), 1)
    np.testing.assert_array_equal(f64(K.causal_matmul.reference(x, y, TILES)),
                                  f64(oracle.causal_matmul_ref(x, y, 128, 128, 128)))
    q, k, v = synthetic.attention_inputs(1, 2, 256, 128)
    np.testing.assert_array_equal(f64(K.causal_attention.reference(q, k, v, K.AttentionBlocks(128, 128))),
                                  f64(oracle.causal_attention_ref(q, k, v, 128, 128)))
    q, kp, vp, bt, lengths = synthetic.decode_inputs(4, 8, 2, 128, 16, 8, 32)
    lengths[:] = [0, 1, 100, 128]
    got = K.paged_gqa_decode.reference(q, kp, vp, bt, lengths)
    np.testing.assert_array_equal(f64(got), f64(oracle.paged_gqa_decode_ref(q, kp, vp, bt, lengths)))
    assert not f64(got[0]).any()
    kc, vc = rand_bf16((3, 512, 256), 4), rand_bf16((3, 512, 256), 5)
    qc, lens = rand_bf16((3, 1, 8, 128), 6, 128**-0.5), np.array([0, 300, 512], np.int32)
    np.testing.assert_array_equal(f64(K.gqa_decode.reference(qc, kc, vc, lens, K.DecodeTiles(block_kv=128))),
                                  f64(oracle.gqa_decode_ref(qc, kc, vc, lens, 128)))
    q_c, q_r = rand_bf16((3, 1, 16, 512), 7, 0.01), rand_bf16((3, 1, 16, 128), 8, 0.07)
    c_kv, k_rope = rand_bf16((3, 512, 512), 9), rand_bf16((3, 512, 128), 10)
    np.testing.assert_array_equal(f64(K.mla_decode.reference(q_c, q_r, c_kv, k_rope, lens, K.DecodeTiles(block_kv=128))),
                                  f64(oracle.mla_decode_ref(q_c, q_r, c_kv, k_rope, lens, 128)))
    np.testing.assert_array_equal(f64(K.all_gather_matmul.reference(x, y, K.CollectiveTiles())),
                                  f64(oracle.matmul_ref(x, y, 256, 512, 256)))


# ----------------------------------------------------------------------------- errors, before anything runs


def test_inputs_are_arrays_of_the_right_count():
    # tests/test_api.py:33-43
    x = rand_bf16((256, 256), 0)
    with pytest.raises(KernelError, match=r"takes 2 input arrays \(x, y\), then optionally `tiles`; got 1"):
        K.matmul(x)
    with pytest.raises(KernelError, match="input `y` must be an array, got float"):
        K.matmul(x, 1.0)
    with pytest.raises(KernelError, match="`tiles` must be a MatmulTiles, not tuple"):
        K.matmul(x, x, (128, 128, 128))


def make(source, **names):
    ns = {"jnp": jnp, "jax": jaxlike, "autokernel": autokernel, **names}
    import linecache

    filename = f"<test kernel {abs(hash(source))}>"
    linecache.cache[filename] = (len(source), None, source.splitlines(keepends=True), filename)
    exec(compile(source, filename, "exec"), ns)
    return ns["f"]


def error(source, **names):
    with pytest.raises(KernelError) as e:
        autokernel.kernel(make(source, **names))
    return str(e.value)


def test_the_function_shape():
    # tests/test_parse.py:81-156
    assert "no `for` loop" in error("def f(x):\n    return x\n")
    assert "assignments and asserts" in error("def f(x):\n    if x:\n        pass\n    for i in range(1):\n        pass\n    return x\n")
    assert "followed by `return`" in error("def f(x):\n    out = jnp.zeros(1)\n    for i in range(1):\n        pass\n")
    assert "return the outputs by name" in error("def f(x):\n    for i in range(1):\n        pass\n    return x + 1\n")
    assert "must be allocated before the loops" in error("def f(x):\n    for i in range(1):\n        pass\n    return out\n")
    assert "its input arrays, then optionally a tunable" in error("def f(x, *rest):\n    pass\n")
    assert "loops are `for v in range(...)`" in error(
        "def f(x):\n    out = jnp.zeros(1)\n    for i in x:\n        out = out.at[i].set(1)\n    return out\n")
    assert "the only `if` is a mask" in error(
        "def f(x):\n    out = jnp.zeros(8)\n    for i in range(8):\n        acc = x[i]\n        if acc:\n            acc = 0\n"
        "        out = out.at[i].set(acc)\n    return out\n")
    assert "is never stored" in error("def f(x):\n    out = jnp.zeros(8)\n    for i in range(8):\n        acc = x[i]\n    return out\n")
    message = error("def f(x):\n    out = jnp.zeros(1)\n    for i in range(1):\n        pass\n")
    assert message.startswith("<test kernel") and ":3:" in message.splitlines()[0]  # names the file and line


def test_a_kernels_tunable_must_be_a_tunable():
    source = ("def f(x, tiles=(128, 128)):\n    out = jnp.zeros((8, 128))\n    for i in range(0, 8, 8):\n"
              "        out = out.at[i : i + 8, :].set(x[i : i + 8, :])\n    return out\n")
    assert "default must be an @autokernel.tunable" in error(source)


def test_unrecognised_schedules_are_refused_not_emulated():
    scale = autokernel.kernel(make(
        "def f(x):\n    out = jnp.zeros((8, 128))\n    for i in range(0, 8, 8):\n"
        "        out = out.at[i : i + 8, :].set(x[i : i + 8, :] * 2)\n    return out\n"))
    with pytest.raises(KernelError, match="not a recognised schedule.*no\n?.*fallback|not a recognised schedule"):
        scale.lower(spec(8, 128))
    banded = autokernel.kernel(make(
        "def f(x, y):\n    out = jnp.zeros((512, 512), x.dtype)\n    for i in range(0, 512, 128):\n"
        "        for j in range(0, 512, 128):\n            if j > i:\n                continue\n"
        "            acc = jnp.zeros((128, 128), jnp.float32)\n            for k in range(0, 256, 128):\n"
        "                acc += x[i : i + 128, k : k + 128] @ y[k : k + 128, j : j + 128]\n"
        "            out = out.at[i : i + 128, j : j + 128].set(acc.astype(x.dtype))\n    return out\n"))
    lowered = banded.lower(spec(512, 256), spec(256, 512))  # any tile mask is fine for the table-walking GEMM
    assert (lowered.tiles, lowered.total_tiles) == (10, 16)
    with pytest.raises(KernelError, match="whole number of steps"):
        K.matmul.build(K.matmul.signature(spec(320, 256), spec(256, 320)), TILES)  # 320 = 2.5 tiles
    with pytest.raises(KernelError, match="multiples of 128"):
        K.matmul.build(K.matmul.signature(spec(192, 256), spec(256, 192)), dataclasses.replace(TILES, tm=64, tn=64))
    with pytest.raises(KernelError, match="skip every output tile"):
        autokernel.kernel(make(
            "def f(x, y):\n    out = jnp.zeros((128, 128), x.dtype)\n    for i in range(0, 128, 128):\n"
            "        for j in range(0, 128, 128):\n            if j >= 0:\n                continue\n"
            "            acc = jnp.zeros((128, 128), jnp.float32)\n            for k in range(0, 128, 128):\n"
            "                acc += x[i : i + 128, k : k + 128] @ y[k : k + 128, j : j + 128]\n"
            "            out = out.at[i : i + 128, j : j + 128].set(acc.astype(x.dtype))\n    return out\n")
        ).lower(spec(128, 128), spec(128, 128))


# ----------------------------------------------------------------------------- tunables and the search


@autokernel.tunable
class Tiles:
    tm: int = autokernel.choice(128, 256, 512, default=256)
    tk: int = autokernel.choice(128, 256)


def test_a_tunable_is_a_frozen_dataclass_of_choices():
    # tests/test_tunable.py:18-46
    t = Tiles()
    assert (t.tm, t.tk) == (256, 128) and is_tunable(t) and not is_tunable(3) and not is_tunable(Tiles)
    with pytest.raises(dataclasses.FrozenInstanceError):
        t.tm = 512
    assert hash(t) == hash(Tiles()) and choices(t) == {"tm": (128, 256, 512), "tk": (128, 256)}
    assert list(neighbours(Tiles())) == [Tiles(tm=512), Tiles(tm=128), Tiles(tk=256)]
    assert list(neighbours(Tiles(tm=384))) == [Tiles(tm=384, tk=256)]  # a value off the choices stays put
    with pytest.raises(TypeError, match=r"declare tunable fields with autokernel\.choice"):
        @autokernel.tunable
        class Bad:
            tm: int = 128
    with pytest.raises(ValueError, match="at least one value"):
        autokernel.choice()
    with pytest.raises(ValueError, match="isn't one of the choices"):
        autokernel.choice(1, 2, default=3)


def profile(seconds, config=None, steps=4, wait=0.0, out_wait=0.0, compute=None, regions=True):
    """A KernelProfile with these times; `compute` defaults to all of the time not waiting (tests/test_tune.py:44-47)."""
    compute = seconds - wait - out_wait if compute is None else compute
    return KernelProfile("f", config, 1, seconds, regions, steps, wait, 0.0, out_wait, compute)


def test_search_climbs_to_the_fastest_and_stops():
    # tests/test_tune.py:51-91
    times = {1: 9.0, 2: 7.0, 3: 8.0, 4: 6.0}
    tuning = search(1, lambda c: Trial(c, profile(times[c])),
                    lambda trial: [trial.config + 1, trial.config + 2] if trial.config < 4 else [], 10)
    assert tuning.config == 4 and [t.config for t in tuning.trials] == [1, 2, 3, 4]
    assert "chose 4" in str(tuning) and str(tuning).count("*") == 1
    # A gain under 1% does not move; the budget stops the search; failures are infinitely slow.
    flat = search(1, lambda c: Trial(c, profile(1.0 - 0.001 * c)), lambda t: [t.config + 1], 10)
    assert flat.config == 1
    capped = search(1, lambda c: Trial(c, profile(1.0 / c)), lambda t: [t.config + 1], 3)
    assert len(capped.trials) == 3
    rescued = search(1, lambda c: Trial(c, error="boom") if c == 1 else Trial(c, profile(1.0)), lambda t: [2], 5)
    assert rescued.config == 2
    with pytest.raises(KernelError, match="no schedule tried ran"):
        search(1, lambda c: Trial(c, error="boom"), lambda t: [], 5)


def test_proposals_follow_the_bottleneck():
    # tests/test_tune.py:97-120, on the matmul nest: what the counters say decides what is tried next.
    kernel = K.matmul
    sig = kernel.signature(spec(2048, 2048), spec(2048, 2048))
    here = Config(K.MatmulTiles(), Pipeline(3, 2))
    steps = kernel.build(sig, here.tunable)[1].steps
    # Exposed input copies: a deeper ring first, then only schedules that move fewer bytes (bigger tiles).
    dma = proposals(kernel, sig, Trial(here, profile(10.0, here, wait=5.0)))
    assert dma[0] == Config(K.MatmulTiles(), Pipeline(4, 2))
    assert dma[1:] and all(c.pipeline == here.pipeline and c.tunable in (K.MatmulTiles(tm=1024), K.MatmulTiles(tn=1024))
                           for c in dma[1:])
    # Per-step overhead: bigger tiles only, fewest steps first.
    overhead = proposals(kernel, sig, Trial(here, profile(10.0, here, compute=1.0)))
    assert overhead and all(kernel.build(sig, c.tunable)[1].steps < steps for c in overhead)
    # Compute-bound, or no counters: every neighbour that launches something else, fewest steps first.
    compute = proposals(kernel, sig, Trial(here, profile(10.0, here)))
    assert {c.tunable for c in compute} == {K.MatmulTiles(tm=1024), K.MatmulTiles(tn=1024), K.MatmulTiles(tm=256),
                                            K.MatmulTiles(tn=256)}
    assert [kernel.build(sig, c.tunable)[1].steps for c in compute] == sorted(
        kernel.build(sig, c.tunable)[1].steps for c in compute)
    blind = proposals(kernel, sig, Trial(here, profile(10.0, here, wait=5.0, regions=False)))
    assert blind == compute
    # The kernel walks K in its own blocks: a neighbour that only changes tk launches the same thing and is never
    # proposed; nor is a deeper output buffering, which no kernel here has.
    assert all(c.tunable.tk == 512 for c in compute)
    outs = proposals(kernel, sig, Trial(here, profile(10.0, here, out_wait=5.0)))
    assert all(c.pipeline == here.pipeline for c in outs)
    # At the deepest ring there is, no deeper one is proposed.
    deepest = Config(K.MatmulTiles(), Pipeline(4, 2))
    assert all(c.pipeline == deepest.pipeline for c in proposals(kernel, sig, Trial(deepest, profile(10.0, deepest, wait=3.0))))
    failed = proposals(kernel, sig, Trial(here, error="boom"))
    assert failed[0] == Config(K.MatmulTiles(), Pipeline(2, 2))
    with pytest.raises(KernelError, match="1 to 4 input buffers"):
        Pipeline(5, 1)


def test_schedules_that_launch_the_same_kernel_are_not_tuned_over():
    # The attention kernel visits the same keys whatever the block sizes: nothing to propose, one trial at most.
    attention = K.causal_attention
    sig = attention.signature(*[spec(1, 2, 1024, 128)] * 3)
    here = Config(K.AttentionBlocks(), Pipeline())
    assert proposals(attention, sig, Trial(here, profile(1.0, here))) == []
    # Contiguous decode walks blocks of the chosen size: its neighbours are real candidates.
    decode = K.gqa_decode
    sig = decode.signature(spec(4, 1, 8, 128), spec(4, 2048, 256), spec(4, 2048, 256), spec(4, dtype=np.int32))
    here = Config(K.DecodeTiles(), Pipeline())
    assert {c.tunable.block_kv for c in proposals(decode, sig, Trial(here, profile(1.0, here)))} == {256, 1024}


def test_a_profile_names_its_bottleneck():
    # src/autokernel/profiling.py:128-140: exposed copies above 20 % -> dma; else time outside waits and compute
    # above 30 % -> overhead; else compute; nothing without counters.
    assert profile(10.0, wait=2.5).bottleneck == "dma" and profile(10.0, out_wait=2.5).bottleneck == "dma"
    filling = KernelProfile("f", None, 1, 10.0, True, 4, 2.5, 2.0, 0.0, 7.5)  # most of the wait fills the ring
    assert filling.exposed_wait_s == 0.5 and filling.bottleneck == "compute"
    assert profile(10.0, compute=6.0).bottleneck == "overhead" and profile(10.0, compute=6.0).other_s == 4.0
    assert profile(10.0).bottleneck == "compute" and profile(10.0, regions=False).bottleneck is None
    text = str(profile(10e-6, Config(None), steps=4, wait=2e-6))
    assert "input waits" in text and "bottleneck: compute" in text and "4" in text
    # The counters of three CTAs (one of them without work) as shares of a CTA's lifetime.
    from tilejax_b200.autokernel.profiling import shares

    records = np.zeros((3, 16), np.int64)
    records[0, :8] = [100, 150, 1050, 200, 50, 100, 5, 1100]   # lifetime 1000: wait 200 (50 filling), room 100
    records[1, :8] = [0, 100, 900, 0, 0, 0, 2, 1000]
    records[2, :8] = [0, 0, 0, 0, 0, 0, 0, 1000]                 # the odd CTA of a pair: no issuing thread
    found = shares(records)
    assert found["ctas"] == 2 and found["wait"] == pytest.approx(0.1) and found["fill"] == pytest.approx(0.025)
    assert found["out_wait"] == pytest.approx(0.05) and found["compute"] == pytest.approx((0.6 + 0.8) / 2)
    assert found["outside"] == pytest.approx((0.1 + 0.2) / 2) and shares(records[2:]) is None


def test_without_a_gpu_tuning_returns_the_defaults(monkeypatch):
    from tilejax_b200.autokernel import tune as tune_module

    monkeypatch.setattr(tune_module, "can_time", lambda: False)
    tuning = K.causal_matmul.tuning(spec(1024, 1024), spec(1024, 1024))
    assert tuning.config == Config(K.MatmulTiles(), Pipeline()) and not tuning.trials
    assert "the defaults" in str(tuning)


def test_compare_tolerances():
    # tests/test_api.py:87-108
    a = np.array([1.0, 2.0, np.nan, np.inf], np.float32)
    assert autokernel.compare("f32", a, a) == 0.0
    assert autokernel.compare("f32", a + np.array([1e-5, 0, 0, 0], np.float32), a) == pytest.approx(1e-5, rel=1e-2)
    with pytest.raises(AssertionError, match="1 of 4 elements"):
        autokernel.compare("f32", a + np.array([1.0, 0, 0, 0], np.float32), a)
    b = np.array([100.0, 1.0], np.float32).astype(BF16)
    assert autokernel.compare("bf16", (b.astype(np.float32) + np.array([0, 1.0], np.float32)).astype(BF16), b) == 1.0
    i = np.array([1, 2], np.int32)
    with pytest.raises(AssertionError):
        autokernel.compare("i32", i + 1, i)
