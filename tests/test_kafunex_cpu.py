"""Kafunex on a machine without a GPU: configuration, plan, loader, cache rules and the engine's host side (step
function, state slots, pages, scheduler) over the plain kernel statements of tests/kernel_refs.py, against the plain
implementation of tests/plain_kafunex.py.  The CUDA kernels themselves are the business of test_kafunex_gpu.py."""
import copy

import pytest
import torch

import plain_kafunex as P
import tiny
import tiny_kafunex as TK
from kernel_refs import ReferenceKernels
from infurnace_b200.cache import CacheManager
from infurnace_b200.config.specs import (GatedRecurrenceSpec, KVCacheNeed, PostNormBlockSpec, StateNeed,
                                         TalkingAttentionSpec)
from infurnace_b200.engine import Engine, EngineOptions, SamplingParams
from infurnace_b200.errors import ModelConfigError, WeightError
from infurnace_b200.models import config_from_dict, plan_for

TOL = 2e-5      # float32 engine against the float64 oracle, logits of size one


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("kafunex"))
    return {n: TK.make_model_dir(n, root) for n in ("K1", "K2")}


def engine(model_dir, name, pool=320, **kw):
    ps = TK.TINY[name]["page_size"]
    opts = dict(dtype="float32", device="cpu", page_size=ps, num_pages=pool // ps, max_num_seqs=4, max_num_batched_tokens=pool)
    opts.update(kw)
    return Engine.from_model_dir(model_dir, EngineOptions(**opts), kernels=ReferenceKernels(torch.float64))


# ------------------------------------------------------------------------------ configuration, plan, weights
def test_configuration_round_trip_and_plan():
    for name, spec in TK.TINY.items():
        cfg = config_from_dict(spec["config"])
        assert cfg.to_dict() == spec["config"]
        plan = plan_for(cfg)
        assert set(plan.tensors()) == set(TK.make_weights(spec["config"], 0)), name
        for (tname, tspec), (_, t) in zip(sorted(plan.tensors().items()), sorted(TK.make_weights(spec["config"], 0).items())):
            assert tuple(tspec.shape) == tuple(t.shape), tname
        for layer, entry in zip(plan.layers, spec["config"]["layers"]):
            assert isinstance(layer, PostNormBlockSpec) and (layer.ffn is None) == (entry["mlp"] is None)
            if entry["type"] == "attention":
                assert isinstance(layer.mixer, TalkingAttentionSpec)
                need = layer.cache_need()
                assert isinstance(need, KVCacheNeed) and need.chunk == (entry["mixer"].get("mask") or {}).get("size")
                assert layer.mixer.scale == entry["mixer"]["scale"] and layer.mixer.values_are_keys
            else:
                assert isinstance(layer.mixer, GatedRecurrenceSpec)
                m = entry["mixer"]
                assert layer.cache_need() == StateNeed((m["heads"], m["dim"], m["vdim"]))


def test_configuration_faults_are_named():
    base = TK.TINY["K1"]["config"]

    def broken(edit):
        c = copy.deepcopy(base)
        edit(c)
        with pytest.raises(ModelConfigError) as e:
            config_from_dict(c)
        return str(e.value)

    assert "type" in broken(lambda c: c["layers"][0].update(type="mamba"))
    assert "vdim" in broken(lambda c: c["layers"][1]["mixer"].update(vdim=8))
    assert "kv_heads" in broken(lambda c: c["layers"][1]["mixer"].update(kv_heads=3))
    assert "dense" in broken(lambda c: c["layers"][0]["mlp"].update(kind="experts"))
    assert "eps" in broken(lambda c: c.update(norm={}))
    assert "width" in broken(lambda c: c.pop("width"))
    assert "mask.size" in broken(lambda c: c["layers"][1]["mixer"].update(mask={"size": 0}))


def test_loader_lists_what_is_wrong(models, tmp_path):
    from safetensors.torch import load_file, save_file
    import os, shutil
    d = str(tmp_path / "bad")
    shutil.copytree(models["K1"], d)
    t = load_file(os.path.join(d, "model.safetensors"))
    del t["l0.mix.lower"]
    t["l1.mix.talk"] = torch.zeros(3, 3)
    t["l2.norm2"] = torch.ones(())          # layer 2 has no feed-forward
    save_file(t, os.path.join(d, "model.safetensors"))
    with pytest.raises(WeightError) as e:
        engine(d, "K1")
    msg = str(e.value)
    assert "l0.mix.lower" in msg and "l1.mix.talk" in msg and "l2.norm2" in msg


# ------------------------------------------------------------------------------ the cache's chunk rule
def test_pages_of_a_finished_chunk_go_back_and_state_slots_are_zeroed():
    cfg = config_from_dict(TK._config(50, 16, 1e-5, [TK._attn(2, 1, 8, 0.3, 24, None), TK._rec(1, 4, 4, None)]))
    plan = plan_for(cfg)
    cache = CacheManager(plan, page_size=8, num_pages=5, max_requests=2, dtype=torch.float32, device="cpu")
    (group,) = cache.kv_groups
    assert group.need.chunk == 24
    cache.add_request("a")
    for step in range(12):                           # 96 tokens through a pool of 40: only the live chunk is held
        cache.allocate("a", 8)
        cache.commit("a", 8)
        cache.check()
        done = 8 * (step + 1)
        held = [i for i, p in enumerate(cache.block_table("a", 0)) if p >= 0]
        assert held == list(range((done // 24) * 24 // 8, -(-done // 8))) or held == list(range((done // 24) * 24 // 8, done // 8))
    state = cache.state_groups[0].tensors[1]
    state[cache.slot_of("a")].fill_(3.0)
    slot = cache.slot_of("a")
    cache.free_request("a")
    assert cache.free_pages() == [5]
    cache.add_request("b")
    assert cache.slot_of("b") == slot and float(state[slot].abs().max()) == 0.0      # a slot that is used again starts at zero


# ------------------------------------------------------------------------------ the engine's host side
LENS = [37, 100, 64, 19, 85, 50, 1, 2, 3]


def _requests(vocab, seed=0):
    return {f"r{i}": tiny.random_tokens(vocab, n, seed + i) for i, n in enumerate(LENS)}


@pytest.mark.parametrize("name", ["K1", "K2"])
@pytest.mark.parametrize("mode", ["whole", "bulk_tail", "portions", "mixed"])
def test_cutting_modes_on_the_host_path(models, name, mode):
    cfg, w = P.read_model(models[name])
    reqs = _requests(cfg["vocab"])
    steps = {"whole": tiny.schedule_whole, "bulk_tail": lambda r: tiny.schedule_bulk_tail(r, tail=40),
             "portions": lambda r: tiny.schedule_portions(r, seed=3),
             "mixed": lambda r: tiny.schedule_mixed(r, max_tokens=320, seed=4)}[mode](reqs)
    eng = engine(models[name], name)
    out = tiny.collect(steps, tiny.run_inprocess(eng.runner, steps), cfg["vocab"])
    for rid, toks in reqs.items():
        assert (out[rid] - P.forward(cfg, w, toks)).abs().max() < TOL, (rid, mode)
    assert eng.runner.cache.num_free_slots == 4
    assert eng.runner.cache.free_pages() == [g.pool.num_pages for g in eng.runner.cache.kv_groups]


def test_the_oracle_would_show_a_wrong_chunk_edge_a_lost_bias_or_unmixed_heads(models):
    """The tiny models are made so that these faults move the logits by far more than the tolerance."""
    cfg, w = P.read_model(models["K1"])
    toks = tiny.random_tokens(cfg["vocab"], 60, 9)
    ref = P.forward(cfg, w, toks)
    wider = copy.deepcopy(cfg)
    wider["layers"][1]["mixer"]["mask"]["size"] += 1
    assert (P.forward(wider, w, toks) - ref).abs().max() > 1000 * TOL
    unmixed = dict(w)
    unmixed["l1.mix.talk"] = torch.eye(4)
    assert (P.forward(cfg, unmixed, toks) - ref).abs().max() > 1000 * TOL
    flat = dict(w)
    flat["l0.mix.lower"] = torch.zeros_like(w["l0.mix.lower"])
    assert (P.forward(cfg, flat, toks) - ref).abs().max() > 1000 * TOL


def test_prefill_equals_token_by_token_decoding(models):
    cfg, w = P.read_model(models["K1"])
    toks = tiny.random_tokens(cfg["vocab"], 75, 21)              # past three edges of the chunk of 24, ten of the chunk of 7
    ref = P.forward(cfg, w, toks)
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    eng = engine(models["K1"], "K1")
    out = tiny.collect(steps, tiny.run_inprocess(eng.runner, steps), cfg["vocab"])["x"]
    assert (out - ref).abs().max() < TOL


def test_a_small_pool_is_enough_when_every_layer_is_chunked(tmp_path):
    """With a chunk rule on every attention layer the pages of finished chunks are used again by the same request."""
    conf = TK._config(40, 24, 1e-5, [TK._attn(2, 2, 8, 0.3, 16, 16), TK._rec(2, 4, 8, None), TK._attn(4, 1, 4, 0.5, 5, None)])
    TK.TINY["_small"] = dict(config=conf, page_size=4, store="float32", seed=12)
    try:
        d = TK.make_model_dir("_small", str(tmp_path))
        cfg, w = P.read_model(d)
        toks = tiny.random_tokens(40, 90, 2)
        steps = tiny.schedule_portions({"a": toks}, seed=7)
        eng = engine(d, "_small", pool=40, max_num_batched_tokens=64)         # 10 pages per group for 90 tokens
        out = tiny.collect(steps, tiny.run_inprocess(eng.runner, steps), 40)["a"]
        assert (out - P.forward(cfg, w, toks)).abs().max() < TOL
    finally:
        del TK.TINY["_small"]


@pytest.mark.parametrize("layers", [[TK._rec(2, 4, 8, 16), TK._rec(1, 6, 5, None)],
                                    [TK._attn(2, 2, 8, 0.3, 9, None), TK._attn(4, 1, 4, 0.5, None, 12)],
                                    [TK._rec(1, 3, 7, None)]])
def test_models_of_one_kind_of_mixer(tmp_path, layers):
    """Only recurrences (no key/value group at all), only attention (no state), a single layer without feed-forward."""
    TK.TINY["_v"] = dict(config=TK._config(50, 24, 1e-5, layers), page_size=4, store="float32", seed=3)
    try:
        d = TK.make_model_dir("_v", str(tmp_path))
    finally:
        del TK.TINY["_v"]
    cfg, w = P.read_model(d)
    reqs = {f"r{i}": tiny.random_tokens(50, n, i) for i, n in enumerate([20, 1, 33, 7, 2, 15])}
    steps = tiny.schedule_mixed(reqs, max_tokens=128, seed=1)
    eng = Engine.from_model_dir(d, EngineOptions(dtype="float32", device="cpu", page_size=4, num_pages=32, max_num_seqs=4,
                                                 max_num_batched_tokens=128), kernels=ReferenceKernels(torch.float64))
    out = tiny.collect(steps, tiny.run_inprocess(eng.runner, steps), 50)
    for rid, toks in reqs.items():
        assert (out[rid] - P.forward(cfg, w, toks)).abs().max() < TOL
    prompt = tiny.random_tokens(50, 5, 9)
    assert eng.generate([prompt], SamplingParams(max_tokens=6)) == [P.greedy(cfg, w, prompt, 6)]


def test_greedy_generation_through_the_scheduler(models):
    cfg, w = P.read_model(models["K2"])
    eng = engine(models["K2"], "K2", max_num_batched_tokens=24)          # prompts go in as portions beside decoded tokens
    prompts = [tiny.random_tokens(cfg["vocab"], n, 40 + n) for n in (1, 9, 33, 70, 5, 18)]      # six requests, four slots
    outs = eng.generate(prompts, SamplingParams(max_tokens=20))
    for p, o in zip(prompts, outs):
        assert o == P.greedy(cfg, w, p, 20)
    eng.runner.cache.check()
    assert eng.runner.cache.num_free_slots == 4


def test_the_new_parts_in_another_arrangement():
    """The attention part with values of its own and without head mixing, gate, norms, distance bias or chunk rule, and the
    feed-forward with another activation, in a post-norm block behind a plain embedding: what a different design would
    put together from the same descriptions.  Compared with the formulas written out in tiny_kafunex.another_arrangement."""
    from infurnace_b200.engine.runner import ModelRunner, StepEntry
    from infurnace_b200.parts import DecoderModel, Runtime
    plan, w, toks, want = TK.another_arrangement()
    assert set(plan.tensors()) == set(w)
    rt = Runtime(device=torch.device("cpu"), act_dtype=torch.float32, kernels=ReferenceKernels(torch.float64))
    cache = CacheManager(plan, page_size=4, num_pages=16, max_requests=2, dtype=torch.float32, device="cpu")
    runner = ModelRunner(DecoderModel(plan, w, rt), cache, rt, 64, 64)
    cache.add_request("a")
    got = torch.cat([runner.step([StepEntry("a", toks[:13], list(range(13)))]).clone(),
                     runner.step([StepEntry("a", toks[13:], list(range(len(toks) - 13)))]).clone()]).double()
    assert (got - want).abs().max() < TOL
