"""The Dutivik decoder through the framework (configuration, loader, cache manager, step function,
scheduler, entry point) against the plain statement in tests/plain_dutivik.py, on the host with the
stand-in kernels and on the GPU with the CUDA kernels, in 32-bit and in bfloat16.

Small configurations of their own and random weights: whole prompts against token-by-token decoding,
portions down to one and two tokens, mixed batches against each request alone, pages and state slots used
again (freed pages overwritten), the first tokens of a request (the convolution's zeros, a window that is not
full yet), long decoding across the window and across pages, layers that run another layer's tensors with a
state of their own, sizes that make mechanisms coincide (one head a group, equal key and value sizes, the
whole head turned or nothing turned, a window of one position, one tap, no feed-forward, scales of one), and
greedy generation through the entry point."""
from __future__ import annotations

import json

import numpy as np
import pytest
import torch

import plain_dutivik as P
import plain_kernels
import replay_cases as rc
from kvcore_b200 import (CacheConfig, DeviceConfig, KVCoreConfig, ModelConfig, SamplingParams, SchedulerConfig)
from kvcore_b200.config import ConfigError
from kvcore_b200.config.registry import model_spec_from_config, model_spec_from_folder
from kvcore_b200.engine.llm_engine import GenerationRequest, LLMEngine
from kvcore_b200.weights.safetensors_io import write_safetensors

BACKENDS = [pytest.param("cpu", id="host"), pytest.param("cuda:0", id="gpu", marks=pytest.mark.gpu)]
# largest |difference| of a row over the request's largest |logit|; in bfloat16 also the root mean square of a
# row's difference (its mean taken off) over that of the request's logits
TOLERANCE = {"float32": 3e-5}
# What bfloat16 costs these tiny models depends on the model and on the position: a state's read-out or a unit
# vector that happens to be small is divided by its own size, which multiplies whatever rounding it carries.
# Measured with the stand-in kernels, which round where the product rounds (worst row / median row, root mean
# square): both_kinds 3.3e-2 / 0.8e-2, coincide 1.8e-1 / 1.2e-2 (vectors of 6 entries), serving_sizes 1.3e-2 /
# 0.6e-2.  So a single row may stray to about 1.7 times the worst seen, while the median row of a trace must stay
# below 2e-2: a kernel that is a little wrong everywhere fails the second, a wrong key or a lost state the
# first (and the 32-bit runs, at 3e-5).
BF16_ROW_TOLERANCE = {"both_kinds": 6e-2, "coincide": 3e-1, "serving_sizes": 3e-2}
BF16_MEDIAN_RMS_TOLERANCE = 2e-2


@pytest.fixture(params=BACKENDS)
def device(request, monkeypatch):
    if request.param == "cpu":
        plain_kernels.install(monkeypatch)
    return request.param


G, S = P.gla_layer, P.parallel_layer
CONFIGS = {
    # both kinds of layer, two heads a group on either side, layers that run another layer's tensors
    "both_kinds": P.model_config([
        G(heads=2, dim=16, vdim=24, tau=8.0, rank=4),
        S(heads=4, kv_heads=2, dim=16, vdim=24, window=12, rot_dims=8, base=100.0, factor=2.0,
          r_heads=4, r_kv_heads=2, r_dim=16, r_vdim=8, conv=4, left_scale=0.7, right_scale=1.3),
        G(heads=2, dim=16, vdim=24, weights_of=0),
        S(heads=4, kv_heads=2, dim=16, vdim=24, window=12, r_heads=4, r_kv_heads=2, r_dim=16, r_vdim=8, weights_of=1),
        S(heads=2, kv_heads=1, dim=24, vdim=8, window=21, rot_dims=24, base=10000.0, r_heads=2, r_kv_heads=2,
          r_dim=8, r_vdim=20, conv=2, left_scale=1.1, right_scale=0.5, ff=40),
    ], vocab=83, width=48),
    # what the first makes unequal is equal or 1 here and the other way round: one head a group, one head, equal
    # key and value sizes, nothing turned, no scaling of the frequencies, a window of one position and one longer
    # than any request, one tap (no convolution state), scales of one, tau of one, no feed-forward, sizes no
    # 16-byte vector fits, the parallel layer first and a borrowed one behind its owner at once
    "coincide": P.model_config([
        S(heads=2, kv_heads=2, dim=10, vdim=10, window=1, rot_dims=0, r_heads=1, r_kv_heads=1, r_dim=6, r_vdim=6,
          conv=1, ff=None),
        S(heads=2, kv_heads=2, dim=10, vdim=10, window=1, r_heads=1, r_kv_heads=1, r_dim=6, r_vdim=6, weights_of=0),
        G(heads=1, dim=12, vdim=12, tau=1.0, rank=1, ff=24),
        S(heads=1, kv_heads=1, dim=20, vdim=6, window=500, rot_dims=20, base=50.0, r_heads=3, r_kv_heads=3,
          r_dim=10, r_vdim=10, conv=3, ff=20),
        G(heads=3, dim=6, vdim=10, tau=3.0, rank=5, ff=None),
    ], vocab=61, width=40, eps=1e-6, embedding_scale=1.0),
    # sizes the tensor-core attention takes (widths in steps of 16), windows across several pages, key sizes that
    # fill the state kernel's registers and ones that are shared by two threads a column
    "serving_sizes": P.model_config([
        S(heads=4, kv_heads=1, dim=64, vdim=128, window=44, rot_dims=32, base=500000.0, factor=4.0,
          r_heads=4, r_kv_heads=2, r_dim=128, r_vdim=64, conv=4),
        G(heads=2, dim=192, vdim=32, tau=12.0, rank=16),
        S(heads=4, kv_heads=2, dim=32, vdim=48, window=70, rot_dims=32, base=10000.0,
          r_heads=2, r_kv_heads=1, r_dim=64, r_vdim=288, conv=3, left_scale=1.4, right_scale=0.6),
        G(heads=2, dim=192, vdim=32, weights_of=1),
    ], vocab=128, width=64),
}
LENGTHS = {"both_kinds": (1, 23, 45, 70, 37, 2), "coincide": (64, 1, 30, 50), "serving_sizes": (150, 3, 97, 61)}


def write_folder(folder, cfg, seed):
    weights = P.random_weights(cfg, seed)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(P.public_config(cfg)))
    write_safetensors(folder / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in weights.items()})
    return {k: v.double() for k, v in weights.items()}


@pytest.fixture(scope="module", params=list(CONFIGS))
def case(request, tmp_path_factory):
    name = request.param
    cfg = CONFIGS[name]
    folder = tmp_path_factory.mktemp(f"dutivik_{name}")
    weights = write_folder(folder, cfg, seed=len(name))
    requests = {f"q{i}": rc.random_tokens(cfg["vocab"], n, 30 + i) for i, n in enumerate(LENGTHS[name])}
    reference = {rid: P.forward(cfg, weights, toks).numpy() for rid, toks in requests.items()}
    return dict(name=name, cfg=cfg, folder=folder, weights=weights, requests=requests, reference=reference)


def compare(rows, reference, dtype, name="both_kinds"):
    assert rows
    spread = []
    bound = TOLERANCE[dtype] if dtype == "float32" else BF16_ROW_TOLERANCE[name]
    for (rid, pos), row in sorted(rows.items()):
        assert np.isfinite(row).all(), f"non-finite logits for {rid}@{pos}"
        err = np.abs(row - reference[rid][pos]).max() / np.abs(reference[rid]).max()
        assert err <= bound, f"{rid}: first wrong position {pos} (error {err:.3e})"
        if dtype == "bfloat16":
            diff = row - reference[rid][pos]
            rms = np.sqrt(np.mean((diff - diff.mean()) ** 2)) / reference[rid].std()
            assert rms <= bound, f"{rid}: first wrong position {pos} (rms error {rms:.3e})"
            spread.append(rms)
    if spread:
        assert np.median(spread) <= BF16_MEDIAN_RMS_TOLERANCE, f"median rms error {np.median(spread):.3e}"


# ---- configuration -----------------------------------------------------------------------------------
def test_config_names_the_tensors_of_the_plain_statement(case):
    from kvcore_b200.parts.model import build_model

    spec = model_spec_from_folder(case["folder"])
    assert spec.architecture == "Dutivik"
    model = build_model(spec, dtype=torch.float32, device="meta")
    assert {slot.name: slot.shape for slot in model.weight_slots()} == P.tensor_shapes(case["cfg"])


def test_config_gives_every_constant_to_the_parts(tmp_path):
    cfg = CONFIGS["both_kinds"]
    write_folder(tmp_path / "m", cfg, 1)
    spec = model_spec_from_folder(tmp_path / "m")
    assert [entry.layer for entry in spec.schedule] == [0, 1, 0, 1, 2] and len(spec.layers) == 3
    assert all(entry.cache_of is None for entry in spec.schedule)
    assert spec.embedding.params["scale"] == cfg["embedding"]["scale"]
    gla = spec.layers[0].mixer.params
    assert (gla["num_heads"], gla["head_dim"], gla["value_dim"], gla["tau"], gla["decay_rank"], gla["eps"]) == (2, 16, 24, 8.0, 4, 1e-5)
    left, right = spec.layers[1].mixer.params["members"]
    assert spec.layers[1].mixer.params["scales"] == (0.7, 1.3)
    assert (left.params["window"], left.params["rot_dims"], left.params["rot_base"], left.params["rot_factor"],
            left.params["scale"], left.params["value_dim"]) == (12, 8, 100.0, 2.0, 0.25, 24)
    assert (right.params["num_heads"], right.params["num_kv_heads"], right.params["conv_taps"], right.params["value_dim"]) == (4, 2, 4, 8)
    assert spec.layers[2].mixer.params["members"][0].params["rot_factor"] == 1.0       # no scaling key: none
    assert set(spec.layers[0].norms) == {"mixer_norm"} and spec.layers[0].norms["mixer_norm"].params["bias"]
    assert spec.final_norm.params["bias_tensor"] == "final.norm.b"
    assert spec.layers[2].feed_forward.params["intermediate_size"] == 40
    # without tensors to ask, the inner size of the decay's projection is a key of its own
    with pytest.raises(ConfigError, match="decay_rank"):
        model_spec_from_config(P.public_config(cfg))
    keyed = json.loads(json.dumps(P.public_config(cfg)))
    keyed["layers"][0]["mixer"]["decay_rank"] = keyed["layers"][2]["mixer"]["decay_rank"] = 7
    assert model_spec_from_config(keyed).layers[0].mixer.params["decay_rank"] == 7


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="attention"), "mixer of this design"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "feed-forward of this design"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=18), "at most dim"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(conv=12), "taps"),
    (lambda c: c["layers"][2].update(weights_of=9), "names no layer"),
    (lambda c: c["layers"][2]["mixer"].update(tau=4.0), "describes another layer"),
    (lambda c: c["layers"][0]["mixer"].pop("tau"), "tau"),
    (lambda c: c["layers"][1]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c.pop("embedding"), "embedding"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_config_refuses(change, message):
    cfg = json.loads(json.dumps(P.public_config(CONFIGS["both_kinds"])))
    for layer in cfg["layers"]:
        if layer["type"] == "gla":
            layer["mixer"] = dict(layer["mixer"], decay_rank=4)
    cfg["layers"][2]["mixer"] = cfg["layers"][0]["mixer"] = dict(cfg["layers"][0]["mixer"])
    cfg["layers"][2]["mixer"] = dict(cfg["layers"][0]["mixer"])
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        model_spec_from_config(cfg)


def test_cache_groups_and_state(tmp_path):
    """A token's keys and values are one cached row of the attention beside the delta rule; layers of one size
    share a page group, also when they run the same tensors; every run of a layer has a state of its own."""
    from kvcore_b200.cache.kv_manager import group_entries
    from kvcore_b200.parts.model import build_model

    write_folder(tmp_path / "m", CONFIGS["both_kinds"], 1)
    model = build_model(model_spec_from_folder(tmp_path / "m"), dtype=torch.float32, device="meta")
    requirements = model.entry_requirements()
    groups, entry_group = group_entries(requirements)
    assert [(g.planes, g.heads, g.width, g.window, g.entries) for g in groups] == [
        (1, 1, 2 * 16 + 2 * 24, 12, (1, 3)), (1, 1, 24 + 8, 21, (4,))]
    assert entry_group == {1: 0, 3: 0, 4: 1}
    delta = 4 * 16 * 8 + (2 * 2 * 16 + 4 * 8) * 3
    assert [req.state_spec.shape for req in requirements] == [
        (2 * 16 * 24,), (delta,), (2 * 16 * 24,), (delta,), (2 * 8 * 20 + (2 * 2 * 8 + 2 * 20) * 1,)]
    assert all(req.state_spec.dtype == torch.float32 and req.cache_of is None for req in requirements)


# ---- the cuttings ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuttings_match_the_plain_statement(case, dtype, device, tmp_path):
    cfg, requests = case["cfg"], case["requests"]
    traces = {
        "whole": rc.trace_whole(requests),
        "tail": rc.trace_decode_tail(requests, tail=20),
        "chunks": rc.trace_chunks(requests, sizes=(7, 3, 16, 2, 5, 1, 9, 2, 31)),
        "mixed": rc.trace_mixed(requests, max_live=4, seed=3),
    }
    results = {}
    for name, steps in traces.items():
        out = tmp_path / name
        rc.run_inprocess(case["folder"], dtype, steps, out, rc.peak_tokens(steps), device=device,
                         fill_freed_pages="poison" if name == "mixed" else None)
        rows = rc.collect(steps, out, cfg["vocab"])
        assert len(rows) == sum(len(t) for t in requests.values())
        compare(rows, case["reference"], dtype, case["name"])
        results[name] = rows
    if dtype == "float32" and device != "cpu":
        # every kernel of the 32-bit path sums in an order that depends on the position only
        for name in ("tail", "chunks", "mixed"):
            for key, row in results["whole"].items():
                assert np.array_equal(row, results[name][key]), f"{name} differs from whole at {key}"


def test_residual_stream_after_every_layer(case, device):
    """Layer by layer: the 32-bit stream that each block hands on against the plain statement's, in two portions
    (the second begins inside a window and inside the convolution's reach)."""
    from kvcore_b200.engine.step import StepEntry
    from kvcore_b200.engine.trace_replay import build_replay

    tokens = case["requests"]["q1"] if len(case["requests"]["q1"]) > 2 else case["requests"]["q2"]
    step_function, kv = build_replay(str(case["folder"]), "float32", 256, device=device)
    seen = []
    for block in step_function.model.blocks:
        original = block.forward

        def recording(h, residual, ctx, cache, original=original):
            out = original(h, residual, ctx, cache)
            seen.append(out[1].detach().clone().cpu())
            return out
        block.forward = recording
    cut = len(tokens) // 3 + 1
    runs = len(case["cfg"]["layers"])
    assert kv.allocate_slots("x", cut)
    step_function.step([StepEntry("x", tokens[:cut], [])])
    assert kv.allocate_slots("x", len(tokens) - cut)
    step_function.step([StepEntry("x", tokens[cut:], [len(tokens) - cut - 1])])
    collected = []
    P.forward(case["cfg"], case["weights"], tokens, collected)
    assert len(seen) == 2 * runs and len(collected) == runs
    for index, want in enumerate(collected):
        got = torch.cat([seen[index], seen[runs + index]])
        assert got.dtype == torch.float32
        torch.testing.assert_close(got.double(), want, rtol=3e-5, atol=3e-5, msg=lambda m: f"layer run {index}: {m}")


def test_pages_and_slots_are_used_again(case, device, tmp_path):
    """A pool for the largest live set only: the trace needs more pages over its life than the pool has and
    more requests than state slots in a row, so a new request finds a page and a state row that another has
    left (the row must read as zeros, the page must not be read before it is written)."""
    requests = dict(case["requests"])
    requests.update({f"again{i}": toks for i, toks in enumerate(case["requests"].values())})
    steps = rc.trace_mixed(requests, max_live=3, seed=11)
    peak = rc.peak_tokens(steps)
    assert sum(-(-len(t) // 16) * 16 for t in requests.values()) > peak
    out = tmp_path / "o"
    step_function, kv = rc.run_inprocess(case["folder"], "float32", steps, out, peak, device=device,
                                         fill_freed_pages="poison")
    assert all(pool.num_free == pool.num_usable for pool in kv.pools)
    reference = dict(case["reference"])
    reference.update({f"again{i}": ref for i, ref in enumerate(case["reference"].values())})
    compare(rc.collect(steps, out, case["cfg"]["vocab"]), reference, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, device, tmp_path):
    """Two prompt tokens, then single tokens: the windows pass over decoded tokens only, pages behind them are
    handed back, the states run on (on the GPU: decode graphs captured and replayed)."""
    cfg = CONFIGS["serving_sizes"] if device != "cpu" else CONFIGS["both_kinds"]
    folder = tmp_path / "m"
    weights = write_folder(folder, cfg, seed=5)
    tokens = rc.random_tokens(cfg["vocab"], 150 if device != "cpu" else 60, 77)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:2], "want": [0, 1]}], "end": []}]
    for pos in range(2, len(tokens)):
        steps.append({"step": pos - 1, "entries": [{"id": "a", "tokens": [tokens[pos]], "want": [0]}],
                      "end": ["a"] if pos == len(tokens) - 1 else []})
    out = tmp_path / "o"
    rc.run_inprocess(folder, dtype, steps, out, 192, device=device, fill_freed_pages="poison")
    compare(rc.collect(steps, out, cfg["vocab"]), {"a": P.forward(cfg, weights, tokens).numpy()}, dtype,
            "serving_sizes" if device != "cpu" else "both_kinds")


def test_each_mechanism_changes_the_logits():
    """The plain statement itself: leaving a mechanism out moves the logits by far more than any tolerance
    here, so a test that passes has seen it.  (Guards the tests, not the product.)"""
    cfg = CONFIGS["both_kinds"]
    weights = P.random_weights(cfg, 9, dtype=torch.float64)
    tokens = rc.random_tokens(cfg["vocab"], 40, 3)
    base = P.forward(cfg, weights, tokens)

    def moved(config=None, **tensors):
        other = dict(weights)
        other.update(tensors)
        return float((P.forward(config or cfg, other, tokens) - base).abs().max() / base.abs().max())

    def changed(change):
        other = json.loads(json.dumps(cfg))
        change(other)
        return other

    zeros, ones = torch.zeros_like, torch.ones_like
    left = lambda c, i=1: c["layers"][i]["mixer"]["left"]
    assert moved(**{"l1.mix.left.g": zeros(weights["l1.mix.left.g"])}) > 1e-3              # the gate per head
    assert moved(**{"l1.mix.right.q.conv": ones(weights["l1.mix.right.q.conv"])}) > 1e-3   # the convolution
    assert moved(**{"l1.mix.right.A_log": weights["l1.mix.right.A_log"] + 1.0}) > 1e-3     # the decay per head
    assert moved(**{"l1.mix.right.dt_bias": weights["l1.mix.right.dt_bias"] + 1.0}) > 1e-3
    assert moved(**{"l1.mix.right.b": zeros(weights["l1.mix.right.b"])}) > 1e-3            # beta
    assert moved(**{"l1.mix.right.norm": ones(weights["l1.mix.right.norm"])}) > 1e-3
    assert moved(**{"l0.mix.a2.b": weights["l0.mix.a2.b"] - 3.0}) > 1e-3                   # the decay per channel
    assert moved(**{"l0.mix.a1": zeros(weights["l0.mix.a1"])}) > 1e-3
    assert moved(**{"l0.mix.norm": ones(weights["l0.mix.norm"])}) > 1e-3
    assert moved(**{"l0.norm1.b": zeros(weights["l0.norm1.b"])}) > 1e-3                    # the norm's bias
    assert moved(**{"final.norm.b": zeros(weights["final.norm.b"])}) > 1e-3
    assert moved(changed(lambda c: c["embedding"].update(scale=1.0))) > 1e-3
    assert moved(changed(lambda c: c["layers"][0]["mixer"].update(tau=1.0))) > 1e-3
    for key, value in (("size", 11), ("size", 13)):                                         # one position either way
        assert moved(changed(lambda c: (left(c)["mask"].update({key: value}), left(c, 3)["mask"].update({key: value})))) > 1e-4
    assert moved(changed(lambda c: (left(c)["rot"].update(dims=4), left(c, 3)["rot"].update(dims=4)))) > 1e-3
    assert moved(changed(lambda c: (left(c)["rot"].update(base=77.0), left(c, 3)["rot"].update(base=77.0)))) > 1e-3
    assert moved(changed(lambda c: (left(c)["rot"]["scaling"].update(factor=1.0), left(c, 3)["rot"]["scaling"].update(factor=1.0)))) > 1e-3
    assert moved(changed(lambda c: (left(c).update(scale=0.5), left(c, 3).update(scale=0.5)))) > 1e-3
    assert moved(changed(lambda c: (c["layers"][1]["mixer"].update(left_scale=1.0), c["layers"][3]["mixer"].update(left_scale=1.0)))) > 1e-3
    assert moved(changed(lambda c: (c["layers"][1]["mixer"].update(right_scale=1.0), c["layers"][3]["mixer"].update(right_scale=1.0)))) > 1e-3
    # a layer that runs another's tensors keeps a state of its own: running it on tensors of its own moves the logits
    own = changed(lambda c: c["layers"][2].pop("weights_of"))
    extra = {name: t for name, t in P.random_weights(own, 10, dtype=torch.float64).items() if name not in weights}
    assert extra and moved(own, **extra) > 1e-3


# ---- the entry point and the scheduler -------------------------------------------------------------------
def plain_greedy(cfg, weights, prompt, steps):
    tokens = list(prompt)
    for _ in range(steps):
        tokens.append(int(P.forward(cfg, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]


@pytest.mark.parametrize("name,budget", [("both_kinds", 16), ("coincide", 7)])
def test_greedy_generation_through_the_entry_point(device, tmp_path, name, budget):
    cfg = CONFIGS[name]
    folder = tmp_path / "m"
    weights = write_folder(folder, cfg, seed=21)
    prompts = [rc.random_tokens(cfg["vocab"], n, 60 + i) for i, n in enumerate((5, 19, 33))]
    config = KVCoreConfig(
        model_config=ModelConfig(model=str(folder), dtype="float32", max_model_len=128),
        cache_config=CacheConfig(block_size=16, num_gpu_blocks=24),
        scheduler_config=SchedulerConfig(max_num_seqs=4, max_num_scheduled_tokens=budget,
                                         max_num_partial_prefills=4, max_long_partial_prefills=4),
        device_config=DeviceConfig(device=device),
    )
    engine = LLMEngine(config)
    requests = [GenerationRequest(f"g{i}", SamplingParams(max_tokens=12, temperature=0.0), tuple(p))
                for i, p in enumerate(prompts)]
    outputs = engine.generate(requests)
    for prompt, output in zip(prompts, outputs):
        assert list(output.output_token_ids) == plain_greedy(cfg, weights, prompt, 12)
    kv = engine.engine_core.model_runner.kv_manager
    kv.check_invariants()
    assert not kv.live_requests()


def test_generation_with_few_pages_and_preemption(device, tmp_path):
    """So few pages that a running request is preempted and computed again from its first token: its state
    row must read as new (an empty state, the convolution's zeros), not as what it left."""
    cfg = CONFIGS["both_kinds"]
    folder = tmp_path / "m"
    weights = write_folder(folder, cfg, seed=22)
    prompts = [rc.random_tokens(cfg["vocab"], n, 90 + i) for i, n in enumerate((30, 28, 26))]
    config = KVCoreConfig(
        model_config=ModelConfig(model=str(folder), dtype="float32", max_model_len=64),
        cache_config=CacheConfig(block_size=4, num_gpu_blocks=16),
        scheduler_config=SchedulerConfig(max_num_seqs=3, max_num_scheduled_tokens=32,
                                         max_num_partial_prefills=3, max_long_partial_prefills=3),
        device_config=DeviceConfig(device=device),
    )
    engine = LLMEngine(config)
    requests = [GenerationRequest(f"g{i}", SamplingParams(max_tokens=10, temperature=0.0), tuple(p))
                for i, p in enumerate(prompts)]
    for prompt, output in zip(prompts, engine.generate(requests)):
        assert list(output.output_token_ids) == plain_greedy(cfg, weights, prompt, 10)


# ---- the programs, each in a process of its own ------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_program_on_a_dutivik_folder(case, dtype, tmp_path):
    """``bin/trace_run`` as a user drives it: a step, its ``done`` line, the next step."""
    if case["name"] != "serving_sizes":
        pytest.skip("one configuration is enough for the subprocess run")
    steps = rc.trace_mixed(case["requests"], max_live=3, seed=5)
    steps.insert(1, {"step": 1000, "entries": [], "end": []})      # a step that brings nothing
    out = tmp_path / "out"
    rc.run_subprocess(case["folder"], dtype, steps, out, rc.peak_tokens(steps))
    rows = rc.collect(steps, out, case["cfg"]["vocab"])
    assert len(rows) == sum(len(t) for t in case["requests"].values())
    compare(rows, case["reference"], dtype, case["name"])


@pytest.mark.gpu
def test_offline_batch_program_on_a_dutivik_folder(tmp_path):
    import ast
    import re
    import subprocess
    import sys

    cfg = CONFIGS["serving_sizes"]
    folder = tmp_path / "m"
    weights = write_folder(folder, cfg, seed=4)
    prompts = {f"req-{i}": rc.random_tokens(cfg["vocab"], n, 80 + i) for i, n in enumerate((70, 9, 33))}
    (tmp_path / "requests.json").write_text(json.dumps(
        [dict(request_id=rid, prompt_token_ids=tokens) for rid, tokens in prompts.items()]))
    command = [sys.executable, str(rc.ROOT / "bin" / "kvcore_offline_batch"), "--model", str(folder), "--dtype", "float32",
               "--prompt-tokens-file", str(tmp_path / "requests.json"), "--max-tokens", "6", "--block-size", "16",
               "--num-gpu-blocks", "64", "--max-model-len", "256", "--max-num-seqs", "4",
               "--max-num-scheduled-tokens", "48", "--max-num-partial-prefills", "4", "--max-long-partial-prefills", "4",
               "--log-level", "WARNING"]
    result = subprocess.run(command, capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stderr[-2000:]
    found = {m["id"]: list(ast.literal_eval(m["ids"])) for m in re.finditer(
        r"^\[(?P<id>[^\]]+)\] finish_reason=\S+\ntoken_ids=(?P<ids>\(.*\))$", result.stdout, re.M)}
    assert list(found) == list(prompts)
    for rid, prompt in prompts.items():
        assert found[rid] == plain_greedy(cfg, weights, prompt, 6)
