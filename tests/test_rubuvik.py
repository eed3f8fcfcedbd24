"""The Rubuvik decoder through the framework (configuration, loader, cache manager, step function,
scheduler, entry point) against the plain statement in tests/plain_rubuvik.py, on the host with the
stand-in kernels and on the GPU with the CUDA kernels, in 32-bit and in bfloat16.

Small configurations of their own and random weights: whole prompts against token-by-token decoding,
portions down to one and two tokens, mixed batches against each request alone, pages and state slots used
again (freed pages overwritten), the first tokens of a request (a window that is not full yet, the first
period of the query temperature), long decoding across the windows and across pages, every order of the
three mixers, sizes that make mechanisms coincide (one head a group, one head, equal key and value sizes,
a window of one position and one longer than any request, a temperature period of one, every expert
chosen, every group kept, no shared expert, no feed-forward, no token side, factors of one, decays of zero
and one), and greedy generation through the entry point."""
from __future__ import annotations

import json

import numpy as np
import pytest
import torch

import plain_kernels
import plain_rubuvik as P
import replay_cases as rc
from kvcore_b200 import (CacheConfig, DeviceConfig, KVCoreConfig, ModelConfig, SamplingParams, SchedulerConfig)
from kvcore_b200.config import ConfigError
from kvcore_b200.config.registry import model_spec_from_config, model_spec_from_folder
from kvcore_b200.engine.llm_engine import GenerationRequest, LLMEngine
from kvcore_b200.weights.safetensors_io import write_safetensors

BACKENDS = [pytest.param("cpu", id="host"), pytest.param("cuda:0", id="gpu", marks=pytest.mark.gpu)]
# largest |difference| of a row over the request's largest |logit|; in bfloat16 also the root mean square of a
# row's difference (its mean taken off) over that of the request's logits.  A wrong key, a lost state or a
# window one position off moves a row by 1e-2 and more (test_each_mechanism_changes_the_logits); the 32-bit
# runs hold every position to 5e-5.  In bfloat16 a single row may stray further than the median row.
TOLERANCE = {"float32": 5e-5}
BF16_ROW_TOLERANCE = 8e-2
BF16_MEDIAN_RMS_TOLERANCE = 2.5e-2
# a position where a router's choice hangs on less than this is left out of the bfloat16 comparisons
BF16_ROUTER_MARGIN = 4e-2


@pytest.fixture(params=BACKENDS)
def device(request, monkeypatch):
    if request.param == "cpu":
        plain_kernels.install(monkeypatch)
    return request.param


L, A = P.lightning_layer, P.attention_layer
CONFIGS = {
    # all three mixers, both feed-forwards, value mixing across both kinds of attention, a token side input
    "all_kinds": P.model_config([
        A(heads=4, kv_heads=2, dim=16, vdim=24, window=12, q_temp=(0.4, 7), v_mix=True, mlp=P.dense(40)),
        L(heads=2, dim=16, vdim=24, mlp=P.moe(experts=8, top=3, ff=16, groups=(4, 2), scale=1.7, shared=24)),
        A(kind="attention_2", heads=4, kv_heads=2, dim=8, vdim=24, window=21, scale=0.6, v_mix=True, mlp=P.dense(32)),
        L(heads=3, dim=8, vdim=16, decay=(0.5, 0.93, 0.999), mlp=P.dense(24)),
        A(heads=2, kv_heads=2, dim=16, vdim=24, window=5, q_temp=(1.1, 16), v_mix=True,
          mlp=P.moe(experts=6, top=2, ff=24, groups=(2, 1), scale=0.8)),
    ], vocab=83, width=48, eps=1e-5, embedding_scale=0.6, residual_mult=0.8, side=6),
    # what the first makes unequal is equal or 1 here and the other way round: one head a group, one head, equal
    # key and value sizes, a window of one position and one longer than any request, no window at all, a period of
    # one, no mixing, every expert chosen, every group kept, no groups, no feed-forward, no token side input,
    # factors of one, decays of zero and one, sizes no 16-byte vector fits, attention_2 first
    "coincide": P.model_config([
        A(kind="attention_2", heads=2, kv_heads=2, dim=10, vdim=10, window=1, q_temp=(0.3, 1), mlp=None),
        L(heads=1, dim=6, vdim=6, decay=(1.0,), mlp=P.moe(experts=4, top=4, ff=12, groups=(2, 2))),
        A(heads=1, kv_heads=1, dim=20, vdim=6, window=500, mlp=P.moe(experts=3, top=1, ff=10)),
        L(heads=3, dim=10, vdim=6, decay=(0.0, 0.5, 0.97), mlp=None),
        A(kind="attention_2", heads=3, kv_heads=1, dim=6, vdim=10, v_mix=True, mlp=P.dense(20)),
        A(heads=2, kv_heads=2, dim=8, vdim=5, v_mix=True, mlp=None),      # the same width of values, cut into other heads
    ], vocab=61, width=40, eps=1e-6),
    # sizes the tensor-core attention takes (widths in steps of 16), windows across several pages, key sizes that
    # fill the state kernel's registers and ones that are shared by two threads a column
    "serving_sizes": P.model_config([
        L(heads=2, dim=128, vdim=64, mlp=P.dense(96)),
        A(kind="attention_2", heads=4, kv_heads=1, dim=64, vdim=128, window=44, v_mix=True,
          mlp=P.moe(experts=8, top=2, ff=32, groups=(4, 3), scale=2.5, shared=64)),
        A(heads=4, kv_heads=1, dim=32, vdim=128, window=70, q_temp=(0.5, 32), v_mix=True, mlp=P.dense(64)),
        L(heads=2, dim=192, vdim=32, decay=(0.9, 0.9995), mlp=None),
    ], vocab=128, width=64, embedding_scale=2.0, residual_mult=0.5, side=16),
}
LENGTHS = {"all_kinds": (1, 23, 45, 70, 37, 2), "coincide": (64, 1, 30, 50), "serving_sizes": (150, 3, 97, 61)}


def write_folder(folder, cfg, seed):
    weights = P.random_weights(cfg, seed)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in weights.items()})
    return {k: v.double() for k, v in weights.items()}


@pytest.fixture(scope="module", params=list(CONFIGS))
def case(request, tmp_path_factory):
    name = request.param
    cfg = CONFIGS[name]
    folder = tmp_path_factory.mktemp(f"rubuvik_{name}")
    weights = write_folder(folder, cfg, seed=len(name))
    requests = {f"q{i}": rc.random_tokens(cfg["vocab"], n, 30 + i) for i, n in enumerate(LENGTHS[name])}
    reference, margins = {}, {}
    for rid, toks in requests.items():
        seen = []
        reference[rid] = P.forward(cfg, weights, toks, margins=seen).numpy()
        margins[rid] = seen[0].numpy()
    return dict(name=name, cfg=cfg, folder=folder, weights=weights, requests=requests, reference=reference,
                margins=margins)


def compare(rows, reference, dtype, margins=None):
    """32-bit: every row within TOLERANCE.  bfloat16: rows whose own router margin is small are left out; a row
    in front of which some router chose otherwise (these models' streams carry a percent of rounding, and a
    state or a cached key hands a changed row on) may stray, so up to 6 % of the rows may lie beyond the row
    tolerance, while the median row must stay within BF16_MEDIAN_RMS_TOLERANCE: a kernel that is a little
    wrong everywhere fails the second, a wrong key or a lost state the 32-bit runs and the kernels' own tests."""
    assert rows
    spread, beyond = [], []
    for (rid, pos), row in sorted(rows.items()):
        assert np.isfinite(row).all(), f"non-finite logits for {rid}@{pos}"
        err = np.abs(row - reference[rid][pos]).max() / np.abs(reference[rid]).max()
        if dtype == "float32":
            assert err <= TOLERANCE[dtype], f"{rid}: first wrong position {pos} (error {err:.3e})"
            continue
        if margins is not None and margins[rid][pos] < BF16_ROUTER_MARGIN:
            continue
        diff = row - reference[rid][pos]
        rms = np.sqrt(np.mean((diff - diff.mean()) ** 2)) / reference[rid].std()
        spread.append(rms)
        if max(err, rms) > BF16_ROW_TOLERANCE:
            beyond.append((rid, pos, float(max(err, rms))))
    if spread:
        assert len(beyond) <= max(2, 0.06 * len(spread)), f"{len(beyond)} of {len(spread)} rows stray: {beyond[:8]}"
        assert np.median(spread) <= BF16_MEDIAN_RMS_TOLERANCE, f"median rms error {np.median(spread):.3e}"


# ---- configuration -----------------------------------------------------------------------------------
def test_config_names_the_tensors_of_the_plain_statement(case):
    from kvcore_b200.parts.model import build_model

    spec = model_spec_from_folder(case["folder"])
    assert spec.architecture == "Rubuvik"
    model = build_model(spec, dtype=torch.float32, device="meta")
    assert {slot.name: slot.shape for slot in model.weight_slots()} == P.tensor_shapes(case["cfg"])


def test_config_gives_every_constant_to_the_parts():
    cfg = CONFIGS["all_kinds"]
    spec = model_spec_from_config(cfg)
    assert [entry.layer for entry in spec.schedule] == [0, 1, 2, 3, 4]
    assert spec.embedding.params["scale"] == 0.6 and spec.embedding.params["side_width"] == 6 * 5
    first, light, second = (spec.layers[i].mixer for i in (0, 1, 2))
    assert first.kind == second.kind == "gated_window_attention" and light.kind == "lightning_attention"
    p = first.params
    assert (p["num_heads"], p["num_kv_heads"], p["head_dim"], p["value_dim"], p["window"], p["scale"], p["q_temp"]) == \
        (4, 2, 16, 24, 12, 0.25, (0.4, 7))
    assert (p["bias"], p["sink"], p["qk_norm"], p["head_gate"], p["value_mix"], p["slope_exponent"]) == \
        (False, False, False, False, "first", 8.0)
    p = second.params
    assert (p["bias"], p["sink"], p["qk_norm"], p["head_gate"], p["value_mix"], p["q_temp"], p["window"], p["scale"]) == \
        (True, True, True, True, "later", None, 21, 0.6)
    assert spec.layers[4].mixer.params["value_mix"] == "later"
    assert light.params["decay"] == tuple(cfg["layers"][1]["mixer"]["decay"]) and light.params["eps"] == 1e-5
    assert spec.layers[3].mixer.params["decay"] == (0.5, 0.93, 0.999)
    moe = spec.layers[1].feed_forward.params
    assert (moe["num_experts"], moe["top_k"], moe["expert_size"], moe["group_count"], moe["group_keep"], moe["weight_scale"],
            moe["score"], moe["weight_on"], moe["renormalize"]) == (8, 3, 16, 4, 2, 1.7, "softmax", "output", False)
    assert moe["shared"].params["intermediate_size"] == 24 and spec.layers[4].feed_forward.params["shared"] is None
    norms = spec.layers[0].norms
    assert set(norms) == {"mixer_norm", "mixer_out_norm", "feed_forward_norm", "feed_forward_out_norm"}
    assert all(n.params["offset"] == 1.0 and n.params["eps"] == 1e-5 for n in norms.values())
    assert [norms[k].params["multiplier"] for k in sorted(norms)] == [1.0, 0.8, 1.0, 0.8]
    side = spec.layers[3].block.params["token_side"]
    assert (side["dim"], side["index"], side["scale"], side["eps"]) == (6, 3, 0.8, 1e-5)
    # keys that a model may leave out
    plain = model_spec_from_config(CONFIGS["coincide"])
    assert "token_side" not in plain.layers[0].block.params and plain.embedding.params.get("side_width", 0) == 0
    assert plain.layers[4].mixer.params["window"] is None and plain.layers[4].mixer.params["value_mix"] == "first"
    assert plain.layers[2].feed_forward.params["group_count"] == 1 and plain.layers[2].feed_forward.params["weight_scale"] == 1.0
    assert plain.layers[0].feed_forward is None and set(plain.layers[0].norms) == {"mixer_norm", "mixer_out_norm"}


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="gla"), "mixer of this design"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "feed-forward of this design"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "one a head"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5, -0.5]), "one a head"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "exceeds experts"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3), "equal groups"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=1), "must hold"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=8), "values of other sizes"),
    (lambda c: c["layers"][0]["mixer"]["q_temp"].update(every=0), "every"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c.pop("embedding"), "embedding"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["token_side"].pop("dim"), "dim"),
])
def test_config_refuses(change, message):
    cfg = json.loads(json.dumps(CONFIGS["all_kinds"]))
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        model_spec_from_config(cfg)


def test_cache_groups_and_state(tmp_path):
    """A token's keys and values are one cached row; layers of one size and window share a page group; a
    lightning layer keeps no pages and one state row a request."""
    from kvcore_b200.cache.kv_manager import group_entries
    from kvcore_b200.parts.model import build_model

    model = build_model(model_spec_from_config(CONFIGS["all_kinds"]), dtype=torch.float32, device="meta")
    requirements = model.entry_requirements()
    groups, entry_group = group_entries(requirements)
    assert [(g.planes, g.heads, g.width, g.window, g.entries) for g in groups] == [
        (1, 1, 2 * 16 + 2 * 24, 12, (0,)), (1, 1, 2 * 8 + 2 * 24, 21, (2,)), (1, 1, 2 * 16 + 2 * 24, 5, (4,))]
    assert entry_group == {0: 0, 2: 1, 4: 2}
    assert [None if r.state_spec is None else r.state_spec.shape for r in requirements] == [
        None, (2 * 16 * 24,), None, (3 * 8 * 16,), None]


def test_unused_tensors_of_a_checkpoint_are_accepted(device, tmp_path):
    """A layer that mixes no values in may carry the number anyway, a layer without feed-forward its norms."""
    from kvcore_b200.engine.trace_replay import build_replay

    cfg = CONFIGS["coincide"]
    weights = P.random_weights(cfg, 3)
    weights.update({"l0.mix.vmix": torch.tensor(0.5), "l0.norm2": torch.zeros(cfg["width"]),
                    "l0.norm2b": torch.zeros(cfg["width"])})
    folder = tmp_path / "m"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in weights.items()})
    build_replay(str(folder), "float32", 64, device=device)


# ---- the cuttings ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuttings_match_the_plain_statement(case, dtype, device, tmp_path):
    cfg, requests = case["cfg"], case["requests"]
    traces = {
        "whole": rc.trace_whole(requests),
        "tail": rc.trace_decode_tail(requests, tail=26),
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
        compare(rows, case["reference"], dtype, case["margins"])
        results[name] = rows
    if dtype == "float32" and device != "cpu":
        # every kernel of the 32-bit path sums in an order that depends on the position only
        for name in ("tail", "chunks", "mixed"):
            for key, row in results["whole"].items():
                assert np.array_equal(row, results[name][key]), f"{name} differs from whole at {key}"


def test_residual_stream_after_every_layer(case, device):
    """Layer by layer: the 32-bit stream that each block hands on against the plain statement's, in two portions
    (the second begins inside a window and carries a state over)."""
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
    P.forward(case["cfg"], case["weights"], tokens, streams=collected)
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
    handed back, the states run on, the query temperature steps up (on the GPU: decode graphs captured and
    replayed)."""
    cfg = CONFIGS["serving_sizes"] if device != "cpu" else CONFIGS["all_kinds"]
    folder = tmp_path / "m"
    weights = write_folder(folder, cfg, seed=5)
    tokens = rc.random_tokens(cfg["vocab"], 150 if device != "cpu" else 60, 77)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:2], "want": [0, 1]}], "end": []}]
    for pos in range(2, len(tokens)):
        steps.append({"step": pos - 1, "entries": [{"id": "a", "tokens": [tokens[pos]], "want": [0]}],
                      "end": ["a"] if pos == len(tokens) - 1 else []})
    out = tmp_path / "o"
    rc.run_inprocess(folder, dtype, steps, out, 192, device=device, fill_freed_pages="poison")
    margins = []
    reference = P.forward(cfg, weights, tokens, margins=margins).numpy()
    compare(rc.collect(steps, out, cfg["vocab"]), {"a": reference}, dtype, {"a": margins[0].numpy()})


def test_each_mechanism_changes_the_logits():
    """The plain statement itself: leaving a mechanism out moves the logits by far more than any tolerance
    here, so a test that passes has seen it.  (Guards the tests, not the product.)"""
    cfg = CONFIGS["all_kinds"]
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
    mixer = lambda c, i: c["layers"][i]["mixer"]
    assert moved(**{"l2.mix.g": zeros(weights["l2.mix.g"])}) > 1e-3                        # the gate per head
    assert moved(**{"l2.mix.sink": weights["l2.mix.sink"] + 2.0}) > 1e-3                   # the sink
    assert moved(**{"l2.mix.q.b": zeros(weights["l2.mix.q.b"])}) > 1e-3                    # the biases
    assert moved(**{"l2.mix.v.b": zeros(weights["l2.mix.v.b"])}) > 1e-3
    assert moved(**{"l2.mix.vmix": zeros(weights["l2.mix.vmix"])}) > 1e-3                  # value mixing
    assert moved(**{"l4.mix.vmix": zeros(weights["l4.mix.vmix"])}) > 1e-3
    assert moved(**{"l0.mix.vmix": ones(weights["l0.mix.vmix"])}) == 0.0                   # the first one's is unused
    assert moved(**{"l1.mix.norm": ones(weights["l1.mix.norm"])}) > 1e-3
    assert moved(**{"l1.mix.g": zeros(weights["l1.mix.g"])}) > 1e-3
    assert moved(**{"l1.mlp.correction": zeros(weights["l1.mlp.correction"])}) > 1e-3
    assert moved(**{"l1.norm1b": zeros(weights["l1.norm1b"])}) > 1e-3                      # weights around zero
    assert moved(**{"final.norm": zeros(weights["final.norm"])}) > 1e-3
    assert moved(**{"l3.side.norm": ones(weights["l3.side.norm"])}) > 1e-3
    assert moved(**{"side.embed": ones(weights["side.embed"])}) > 1e-3
    assert moved(changed(lambda c: c.pop("token_side"))) > 1e-3
    assert moved(changed(lambda c: c["embedding"].update(scale=1.0))) > 1e-3
    assert moved(changed(lambda c: c.update(residual_mult=1.0))) > 1e-3
    assert moved(changed(lambda c: mixer(c, 1).update(decay=[0.5, 0.5]))) > 1e-3
    assert moved(changed(lambda c: mixer(c, 0)["q_temp"].update(every=8))) > 1e-4
    assert moved(changed(lambda c: mixer(c, 0)["q_temp"].update(coef=0.0))) > 1e-3
    for size in (11, 13):                                                                   # one position either way
        assert moved(changed(lambda c: mixer(c, 0)["mask"].update(size=size))) > 1e-4
    for size in (20, 22):
        assert moved(changed(lambda c: mixer(c, 2)["mask"].update(size=size))) > 1e-4
    assert moved(changed(lambda c: mixer(c, 2).update(scale=0.3))) > 1e-3
    assert moved(changed(lambda c: c["layers"][1]["mlp"]["router"].update(scale=1.0))) > 1e-3
    assert moved(changed(lambda c: c["layers"][1]["mlp"]["router"].pop("groups"))) > 1e-3
    assert moved(changed(lambda c: c["layers"][1]["mlp"]["router"].update(top=2))) > 1e-3
    assert moved(changed(lambda c: c["layers"][1]["mlp"].pop("shared"))) > 1e-3


# ---- configurations drawn at random ------------------------------------------------------------------------
def drawn_config(seed):
    """Another model of the design: sizes, head counts, order of layers, windows and constants all drawn."""
    import random

    rng = random.Random(seed)
    fast = seed % 2 == 0                       # every other model has widths the tensor-core attention takes
    width = rng.choice([32, 48, 64, 96] if fast else [24, 40, 56, 72])
    mixing_kv, mixing_vdim = rng.choice([1, 2, 3]), rng.choice([8, 16, 24, 40] if fast else [6, 10, 12, 20])
    layers = []
    for _ in range(rng.randrange(2, 6)):
        kind = rng.choice(["lightning", "attention", "attention_2"])
        mlp = rng.choice([None, "dense", "moe", "moe"])
        if mlp == "dense":
            mlp = P.dense(rng.choice([16, 24, 40, 52]))
        elif mlp == "moe":
            count = rng.choice([1, 2, 3, 4])
            per = rng.choice([1, 2, 3])
            keep = rng.randrange(1, count + 1)
            top = rng.randrange(1, keep * per + 1)
            mlp = P.moe(experts=count * per, top=top, ff=rng.choice([8, 12, 16, 20]),
                        groups=None if count == 1 and rng.random() < 0.5 else (count, keep), scale=rng.choice([1.0, 0.5, 2.5]),
                        shared=rng.choice([None, 16, 24]))
        if kind == "lightning":
            heads = rng.choice([1, 2, 3, 4])
            layers.append(L(heads=heads, dim=rng.choice([16, 32, 64] if fast else [4, 6, 10, 24]),
                            vdim=rng.choice([8, 16, 32, 40] if fast else [5, 6, 12, 20]),
                            decay=[rng.choice([0.0, 0.3, 0.8, 0.95, 0.999, 1.0]) for _ in range(heads)], mlp=mlp))
            continue
        mixes = rng.random() < 0.7
        kv_heads = mixing_kv if mixes else rng.choice([1, 2])
        layers.append(A(kind=kind, heads=kv_heads * rng.choice([1, 2, 3]), kv_heads=kv_heads,
                        dim=rng.choice([16, 32, 48, 64] if fast else [6, 10, 20, 28]),
                        vdim=mixing_vdim if mixes else rng.choice([8, 24] if fast else [7, 9]),
                        window=rng.choice([None, 1, 2, 5, 16, 17, 31, 40, 64]), scale=rng.choice([None, 0.2, 0.05]),
                        q_temp=rng.choice([None, (0.5, 1), (0.25, 7), (1.0, 16), (0.1, 300)]), v_mix=mixes, mlp=mlp))
    return P.model_config(layers, vocab=rng.randrange(40, 160), width=width, eps=rng.choice([1e-6, 1e-5]),
                          embedding_scale=rng.choice([1.0, 0.5, 3.0]), residual_mult=rng.choice([1.0, 0.7, 0.4]),
                          side=rng.choice([None, 4, 6, 8, 16]))


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(seed, device, tmp_path):
    """Eight other models of the design through the framework: in 32-bit every position of every cutting against
    the plain statement (and, on the GPU, bit-equal between cuttings); in bfloat16 the mixed cutting."""
    cfg = drawn_config(seed)
    folder = tmp_path / "m"
    weights = write_folder(folder, cfg, seed=100 + seed)
    requests = {f"d{i}": rc.random_tokens(cfg["vocab"], n, 500 + 10 * seed + i) for i, n in enumerate((1, 2, 47, 90, 33))}
    reference, margins = {}, {}
    for rid, toks in requests.items():
        seen = []
        reference[rid] = P.forward(cfg, weights, toks, margins=seen).numpy()
        margins[rid] = seen[0].numpy()
    traces = {"whole": rc.trace_whole(requests), "tail": rc.trace_decode_tail(requests, tail=40),
              "chunks": rc.trace_chunks(requests, sizes=(2, 13, 1, 5, 32, 3)),
              "mixed": rc.trace_mixed(requests, max_live=3, seed=seed)}
    results = {}
    for name, steps in traces.items():
        out = tmp_path / name
        rc.run_inprocess(folder, "float32", steps, out, rc.peak_tokens(steps), device=device,
                         fill_freed_pages="poison" if name == "mixed" else None)
        results[name] = rc.collect(steps, out, cfg["vocab"])
        compare(results[name], reference, "float32")
    if device != "cpu":
        for name in ("tail", "chunks", "mixed"):
            for key, row in results["whole"].items():
                assert np.array_equal(row, results[name][key]), f"{name} differs from whole at {key}"
    steps = traces["mixed"]
    rc.run_inprocess(folder, "bfloat16", steps, tmp_path / "b", rc.peak_tokens(steps), device=device, fill_freed_pages="poison")
    compare(rc.collect(steps, tmp_path / "b", cfg["vocab"]), reference, "bfloat16", margins)


# ---- the entry point and the scheduler -------------------------------------------------------------------
def plain_greedy(cfg, weights, prompt, steps):
    tokens = list(prompt)
    for _ in range(steps):
        tokens.append(int(P.forward(cfg, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]


@pytest.mark.parametrize("name,budget", [("all_kinds", 16), ("coincide", 7)])
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
    row must read as new (an empty state), not as what it left."""
    cfg = CONFIGS["all_kinds"]
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
def test_trace_program_on_a_rubuvik_folder(case, dtype, tmp_path):
    """``bin/trace_run`` as a user drives it: a step, its ``done`` line, the next step."""
    if case["name"] != "serving_sizes":
        pytest.skip("one configuration is enough for the subprocess run")
    steps = rc.trace_mixed(case["requests"], max_live=3, seed=5)
    steps.insert(1, {"step": 1000, "entries": [], "end": []})      # a step that brings nothing
    out = tmp_path / "out"
    rc.run_subprocess(case["folder"], dtype, steps, out, rc.peak_tokens(steps))
    rows = rc.collect(steps, out, case["cfg"]["vocab"])
    assert len(rows) == sum(len(t) for t in case["requests"].values())
    compare(rows, case["reference"], dtype, case["margins"])


@pytest.mark.gpu
def test_offline_batch_program_on_a_rubuvik_folder(tmp_path):
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
