"""Lunelorn on a machine without a GPU: configuration, plan, loader, cache entries and the engine's host side (step
function, state slots, pages, scheduler) over the plain kernel statements of tests/kernel_refs.py, against the plain
implementation of tests/plain_lunelorn.py.  The CUDA kernels themselves are the business of test_lunelorn_gpu.py."""
import copy

import pytest
import torch

import plain_lunelorn as P
import tiny
import tiny_lunelorn as TL
from kernel_refs import ReferenceKernels
from infurnace_b200.cache import CacheLayout, CacheManager
from infurnace_b200.config.specs import (KVCacheNeed, ParallelMixerSpec, RetentionSpec, SandwichBlockSpec, StateNeed,
                                         StreamInjectSpec, TimeMixSpec)
from infurnace_b200.engine import Engine, EngineOptions, SamplingParams
from infurnace_b200.errors import ModelConfigError, WeightError
from infurnace_b200.models import config_from_dict, plan_for

TOL = 1e-4      # float32 stream and buffers against the float64 oracle, logits of size seven, layers that run up to three times


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("lunelorn"))
    return {n: TL.make_model_dir(n, root) for n in ("L1", "L2")}


def engine(model_dir, name, pool=320, **kw):
    ps = TL.TINY[name]["page_size"]
    opts = dict(dtype="float32", device="cpu", page_size=ps, num_pages=pool // ps, max_num_seqs=4, max_num_batched_tokens=pool)
    opts.update(kw)
    return Engine.from_model_dir(model_dir, EngineOptions(**opts), kernels=ReferenceKernels(torch.float64))


# ------------------------------------------------------------------------------ configuration, plan, weights
def test_configuration_round_trip_and_plan():
    for name, spec in TL.TINY.items():
        cfg = config_from_dict(spec["config"])
        assert cfg.to_dict() == spec["config"]
        plan = plan_for(cfg)
        made = TL.make_weights(spec["config"], 0)
        assert set(n for n, t in plan.tensors().items() if not t.optional) == set(made), name
        for tname, t in made.items():
            assert tuple(plan.tensors()[tname].shape) == tuple(t.shape), tname
        blocks = [layer for layer in plan.layers if isinstance(layer, SandwichBlockSpec)]
        for layer, entry in zip(blocks, spec["config"]["layers"]):
            assert (layer.ffn is None) == (entry["mlp"] is None) and (layer.side is None) == ("token_side" not in spec["config"])
            kind = {"retention": RetentionSpec, "parallel": ParallelMixerSpec, "wkv": TimeMixSpec}[entry["type"]]
            assert isinstance(layer.mixer, kind)
        loop = spec["config"].get("loop")
        order = [c.layer for c in plan.resolved_schedule()]
        injects = [i for i in order if isinstance(plan.layers[i], StreamInjectSpec)]
        if loop is None:
            assert order == list(range(len(blocks))) and not injects
        else:
            span = list(range(loop["start"], loop["stop"]))
            assert len(injects) == loop["times"] and [plan.layers[i].add_embedding for i in injects] == [t > 0 for t in range(loop["times"])]
            assert [i for i in order if i not in injects] == list(range(loop["start"])) + span * loop["times"] + list(range(loop["stop"], len(blocks)))
            assert plan.embedding.keep == (loop["times"] > 1)


def test_every_layer_run_has_cache_entries_of_its_own():
    cfg = config_from_dict(TL.TINY["L1"]["config"])          # layers 1 and 2 run three times
    plan = plan_for(cfg)
    layout = CacheLayout(plan)
    (kv_need, kv_ids), = layout.kv.values()
    assert isinstance(kv_need, KVCacheNeed) and kv_need.value_head_dim == 8 and len(kv_ids) == 1
    states = {need.shape: len(ids) for need, ids in layout.state.values()}
    assert states == {(40,): 1, (3, 8, 8): 3, (48,): 3, (2, 8, 12): 3}
    cache = CacheManager(plan, page_size=8, num_pages=4, max_requests=2, dtype=torch.float32, device="cpu")
    cache.add_request("a")
    for g in cache.state_groups:
        for t in g.tensors.values():
            t[cache.slot_of("a")].fill_(2.0)
    slot = cache.slot_of("a")
    cache.free_request("a")
    cache.add_request("b")
    assert cache.slot_of("b") == slot
    assert all(float(t[slot].abs().max()) == 0.0 for g in cache.state_groups for t in g.tensors.values())


def test_configuration_faults_are_named():
    base = TL.TINY["L1"]["config"]

    def broken(edit):
        c = copy.deepcopy(base)
        edit(c)
        with pytest.raises(ModelConfigError) as e:
            config_from_dict(c)
        return str(e.value)

    assert "type" in broken(lambda c: c["layers"][0].update(type="mamba"))
    assert "decay" in broken(lambda c: c["layers"][2]["mixer"].update(decay=[0.5]))
    assert "kv_heads" in broken(lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3))
    assert "rot.dims" in broken(lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18))
    assert "moe" in broken(lambda c: c["layers"][0]["mlp"].update(kind="dense"))
    assert "top" in broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=6))
    assert "eps" in broken(lambda c: c.update(norm={}))
    assert "loop" in broken(lambda c: c["loop"].update(stop=4))
    assert "token_side.dim" in broken(lambda c: c.update(token_side={}))


def test_loader_lists_what_is_wrong_and_takes_sizes_from_the_file(models, tmp_path):
    from safetensors.torch import load_file, save_file
    import json, os, shutil
    d = str(tmp_path / "bad")
    shutil.copytree(models["L1"], d)
    t = load_file(os.path.join(d, "model.safetensors"))
    del t["l2.mix.g"]
    t["l0.mix.right.z.b"] = torch.zeros(3)
    t["l1.mlp.router"] = torch.ones(2, 48)          # layer 1 has no feed-forward
    save_file(t, os.path.join(d, "model.safetensors"))
    with pytest.raises(WeightError) as e:
        engine(d, "L1")
    msg = str(e.value)
    assert "l2.mix.g" in msg and "l0.mix.right.z.b" in msg and "l1.mlp.router" in msg
    # the width of the decay's bottleneck comes from the stored tensors when the configuration does not name it, and the
    # norms of a layer without feed-forward may be stored although nothing reads them
    d2 = str(tmp_path / "open")
    shutil.copytree(models["L1"], d2)
    cfg = json.load(open(os.path.join(d2, "config.json")))
    del cfg["layers"][1]["mixer"]["rank"]
    json.dump(cfg, open(os.path.join(d2, "config.json"), "w"))
    t = load_file(os.path.join(d2, "model.safetensors"))
    t["l1.norm2"], t["l1.norm2b"] = torch.ones(48), torch.ones(48)
    save_file(t, os.path.join(d2, "model.safetensors"))
    toks = tiny.random_tokens(97, 12, 1)
    a, b = engine(models["L1"], "L1"), engine(d2, "L1")
    steps = tiny.schedule_whole({"a": toks})
    assert torch.equal(tiny.collect(steps, tiny.run_inprocess(a.runner, steps), 97)["a"],
                       tiny.collect(steps, tiny.run_inprocess(b.runner, steps), 97)["a"])


# ------------------------------------------------------------------------------ the engine's host side
LENS = [37, 100, 64, 19, 85, 50, 1, 2, 3]


def _requests(vocab, seed=0):
    return {f"r{i}": tiny.random_tokens(vocab, n, seed + i) for i, n in enumerate(LENS)}


@pytest.mark.parametrize("name", ["L1", "L2"])
@pytest.mark.parametrize("mode", ["whole", "bulk_tail", "portions", "mixed"])
def test_cutting_modes_on_the_host_path(models, name, mode):
    cfg, w = TL.load_model_dir(models[name])
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


def test_the_oracle_would_show_a_lost_mechanism(models):
    """The tiny models are made so that these faults move the logits by far more than the tolerance."""
    cfg, w = TL.load_model_dir(models["L1"])
    toks = tiny.random_tokens(cfg["vocab"], 60, 9)
    ref = P.forward(cfg, w, toks)

    def moved(cfg2=None, **tensors):
        w2 = dict(w)
        w2.update(tensors)
        return float((P.forward(cfg2 or cfg, w2, toks) - ref).abs().max()) > 1000 * TOL

    assert moved(**{"l1.mix.u": torch.zeros_like(w["l1.mix.u"])})                      # the bonus of the current token
    assert moved(**{"l1.mix.mu.k": torch.zeros_like(w["l1.mix.mu.k"])})                # the blend with the token before
    assert moved(**{"loop.step": torch.zeros_like(w["loop.step"])})                    # the per-pass vector
    assert moved(**{"l0.mix.right.x.b": w["l0.mix.right.x.b"] + 1.0})
    other = copy.deepcopy(cfg)
    other["layers"][2]["mixer"]["decay"] = [0.6, 0.9]
    assert moved(other)
    other = copy.deepcopy(cfg)
    other["layers"][0]["mixer"]["left"]["rot"]["base"] = 900.0                         # the angles of keys and values
    assert moved(other)
    other = copy.deepcopy(cfg)
    other["loop"]["times"] = 2
    assert moved(other)
    other = copy.deepcopy(cfg)
    other["layers"][0]["mlp"]["router"]["top"] = 1
    assert moved(other)
    other = copy.deepcopy(cfg)
    other["logit_softcap"] = 5.0
    assert moved(other)


def test_prefill_equals_token_by_token_decoding(models):
    cfg, w = TL.load_model_dir(models["L1"])
    toks = tiny.random_tokens(cfg["vocab"], 75, 21)
    ref = P.forward(cfg, w, toks)
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    eng = engine(models["L1"], "L1")
    out = tiny.collect(steps, tiny.run_inprocess(eng.runner, steps), cfg["vocab"])["x"]
    assert (out - ref).abs().max() < TOL


@pytest.mark.parametrize("layers,loop", [
    ([TL._ret(2, 4, 8, [0.9, 0.5], TL._moe(3, 1, 8)), TL._ret(1, 6, 5, [1.0], None)], None),          # state only: no pages at all
    ([TL._par(2, 2, 8, 8, 4, 100.0, 0.3, 1, 1.0, 0.5, None)], (0, 1, 1)),                             # a loop of one pass
    ([TL._wkv(1, 3, 2, None), TL._wkv(2, 4, 1, TL._moe(2, 2, 4))], (1, 2, 2)),                        # heads of three rows
    ([TL._ret(1, 4, 4, [0.0], None), TL._par(3, 1, 4, 6, 2, 10.0, 1.0, 5, 0.0, 1.0, TL._moe(1, 1, 4))], (0, 2, 2)),
])
def test_other_arrangements_of_the_layers(tmp_path, layers, loop):
    """Only recurrences, a single layer, a loop that runs once, a loop over everything, one expert, a decay of zero
    and of one, a mixer scale of zero, one rotated pair: values that make mechanisms coincide or vanish."""
    conf = TL._config(50, 24, 1e-5, layers, loop=loop, side=3 if loop else None, cap=None if loop else 4.0)
    d = TL.make_model_dir("_v", str(tmp_path), config=conf, seed=3, store="float32")
    cfg, w = TL.load_model_dir(d)
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
    cfg, w = TL.load_model_dir(models["L2"])
    eng = engine(models["L2"], "L2", max_num_batched_tokens=24)          # prompts go in as portions beside decoded tokens
    prompts = [tiny.random_tokens(cfg["vocab"], n, 40 + n) for n in (1, 9, 33, 70, 5, 18)]      # six requests, four slots
    outs = eng.generate(prompts, SamplingParams(max_tokens=12))
    for p, o in zip(prompts, outs):
        assert o == P.greedy(cfg, w, p, 12)
    eng.runner.cache.check()
    assert eng.runner.cache.num_free_slots == 4
