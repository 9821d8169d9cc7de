"""Filorax on a machine without a GPU: configuration, plan, loader, cache entries and the engine's host side (step
function, state slots, pages, scheduler) over the plain kernel statements of tests/kernel_refs.py, against the plain
implementation of tests/plain_filorax.py.  The CUDA kernels themselves are the business of test_filorax_gpu.py."""
import copy

import pytest
import torch

import plain_filorax as P
import tiny
import tiny_filorax as TF
from kernel_refs import ReferenceKernels
from infurnace_b200.cache import CacheLayout, CacheManager
from infurnace_b200.config.specs import DepthAverageBlockSpec, LatentAttentionSpec, PagedCacheNeed, RoutedExpertsSpec
from infurnace_b200.engine import Engine, EngineOptions, SamplingParams
from infurnace_b200.errors import ModelConfigError, WeightError
from infurnace_b200.models import config_from_dict, plan_for

TOL = 2e-5      # float32 stream and buffers against the float64 oracle


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("filorax"))
    return {n: TF.make_model_dir(n, root) for n in ("F1", "F2")}


def engine(model_dir, page_size, pool=320, **kw):
    opts = dict(dtype="float32", device="cpu", page_size=page_size, num_pages=pool // page_size, max_num_seqs=4,
                max_num_batched_tokens=pool)
    opts.update(kw)
    return Engine.from_model_dir(model_dir, EngineOptions(**opts), kernels=ReferenceKernels(torch.float64))


def tolerance(ref):
    return TOL * max(1.0, float(ref.abs().max()))


# ------------------------------------------------------------------------------ configuration, plan, weights
def test_configuration_round_trip_and_plan():
    for name, spec in TF.TINY.items():
        cfg = config_from_dict(spec["config"])
        assert cfg.to_dict() == spec["config"], name
        plan = plan_for(cfg)
        made = TF.make_weights(spec["config"], 0)
        assert set(n for n, t in plan.tensors().items() if not t.optional) == set(made), name
        for tname, t in made.items():
            assert tuple(plan.tensors()[tname].shape) == tuple(t.shape), tname
        assert [c.layer for c in plan.resolved_schedule()] == list(range(len(spec["config"]["layers"])))
        for depth, (layer, entry) in enumerate(zip(plan.layers, spec["config"]["layers"])):
            assert isinstance(layer, DepthAverageBlockSpec) and layer.depth == depth and layer.depths == len(plan.layers)
            assert layer.residual_mult == spec["config"]["residual_mult"]
            mixer, m = layer.mixer, entry["mixer"]
            assert isinstance(mixer, LatentAttentionSpec)
            assert (mixer.num_heads, mixer.head_dim, mixer.value_head_dim, mixer.kv_rank, mixer.scale) == \
                (m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["scale"])
            assert mixer.window == (m["mask"]["size"] if "mask" in m else None)
            assert mixer.rot_dim == m.get("rot_dim", 0) and (mixer.position is None) == ("rot" not in m)
            assert (mixer.sink is None) == (entry["type"] == "latent_attention_3") == (mixer.gate is None)
            assert (layer.ffn is None) == (entry["mlp"] is None)
            if layer.ffn is not None:
                r = entry["mlp"]["router"]
                assert isinstance(layer.ffn, RoutedExpertsSpec) and layer.ffn.scoring == "all" and layer.ffn.top == r["top"]
                assert layer.ffn.weight_scale == r.get("scale", 1.0) and len(layer.ffn.experts) == r["experts"]
                assert layer.ffn.groups == ((r["groups"]["count"], r["groups"]["keep"]) if "groups" in r else None)
                assert (layer.ffn.shared is None) == ("shared" not in entry["mlp"])


def test_cache_entries_hold_the_latent_and_the_convolutions_inputs():
    conf = TF.TINY["F1"]["config"]
    plan = plan_for(config_from_dict(conf))
    layout = CacheLayout(plan)
    groups = {(need.window, tuple((s.name, s.heads, s.width) for s in need.streams)): ids for need, ids in layout.kv.values()}
    assert all(isinstance(need, PagedCacheNeed) for need, _ in layout.kv.values())
    # layers share pages only where window and widths agree; pages below a window go back early, so windows keep apart
    assert set(groups) == {(None, (("latent", 1, 12), ("rotated_key", 1, 6))), (7, (("latent", 1, 16),)), (20, (("latent", 1, 8),)),
                           (None, (("latent", 1, 10), ("rotated_key", 1, 2)))}
    assert all(len(ids) == 1 for ids in groups.values())
    taps, width = conf["canon"]["taps"], conf["width"]
    states = {need.shape: len(ids) for need, ids in layout.state.values()}
    assert states == {(taps - 1, width): 7}                     # two per layer, one for the layer without feed-forward
    cache = CacheManager(plan, page_size=8, num_pages=6, max_requests=2, dtype=torch.float32, device="cpu")
    cache.add_request("a")
    slot = cache.slot_of("a")
    for g in cache.state_groups:
        for t in g.tensors.values():
            t[slot].fill_(2.0)
    cache.free_request("a")
    cache.add_request("b")
    assert cache.slot_of("b") == slot
    assert all(float(t[slot].abs().max()) == 0.0 for g in cache.state_groups for t in g.tensors.values())


def test_a_latent_and_a_rotated_key_of_one_width_keep_a_dense_tensor_each():
    """Streams of equal shape would share one tensor with a stream axis; the latent kernels address a stream as
    [pages * page_size, width], so this need asks for a tensor per stream."""
    conf = TF._config(30, 16, 1e-5, 1, 1.0, 2, [TF._rot(2, 8, 12, 8, 12, 0.3, 100.0, None)])
    plan = plan_for(config_from_dict(conf))
    cache = CacheManager(plan, page_size=4, num_pages=5, max_requests=2, dtype=torch.float32, device="cpu")
    (g,) = cache.kv_groups
    (streams,) = g.streams.values()
    assert set(streams) == {"latent", "rotated_key"}
    assert all(t.is_contiguous() and tuple(t.shape) == (5, 1, 4, 12) for t in streams.values())
    assert streams["latent"].data_ptr() != streams["rotated_key"].data_ptr()


def test_configuration_faults_are_named():
    base = TF.TINY["F1"]["config"]

    def broken(edit):
        c = copy.deepcopy(base)
        edit(c)
        with pytest.raises(ModelConfigError) as e:
            config_from_dict(c)
        return str(e.value)

    assert "type" in broken(lambda c: c["layers"][0].update(type="latent_attention_4"))
    assert "kv_rank" in broken(lambda c: c["layers"][1]["mixer"].pop("kv_rank"))
    assert "mask" in broken(lambda c: c["layers"][1]["mixer"].pop("mask"))
    assert "rot.dims" in broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=8))
    assert "rot.dims" in broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3))
    assert "moe" in broken(lambda c: c["layers"][0]["mlp"].update(kind="dense"))
    assert "groups" in broken(lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4))
    assert "top" in broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=5))
    assert "eps" in broken(lambda c: c.update(norm={"groups": 3}))
    assert "norm.groups" in broken(lambda c: c["norm"].update(groups=5))
    assert "taps" in broken(lambda c: c.update(canon={}))
    assert "layers" in broken(lambda c: c.update(layers=[]))


def test_loader_lists_what_is_wrong(models, tmp_path):
    import os
    import shutil
    from safetensors.torch import load_file, save_file
    d = str(tmp_path / "bad")
    shutil.copytree(models["F1"], d)
    t = load_file(os.path.join(d, "model.safetensors"))
    del t["l0.mix.sink"]
    t["l2.mix.g"] = torch.zeros(16, 48)             # the mixer with the ordinary softmax has no gate
    t["l1.mlp.router"] = torch.ones(2, 48)          # layer 1 has no feed-forward
    t["l3.dwa"] = torch.ones(4)                     # five results are averaged after the fourth layer
    save_file(t, os.path.join(d, "model.safetensors"))
    with pytest.raises(WeightError) as e:
        engine(d, 16)
    msg = str(e.value)
    assert all(name in msg for name in ("l0.mix.sink", "l2.mix.g", "l1.mlp.router", "l3.dwa"))


# ------------------------------------------------------------------------------ the engine's host side
LENS = [37, 100, 64, 19, 85, 50, 1, 2, 3]


def _requests(vocab, seed=0):
    return {f"r{i}": tiny.random_tokens(vocab, n, seed + i) for i, n in enumerate(LENS)}


@pytest.mark.parametrize("name", ["F1", "F2"])
@pytest.mark.parametrize("mode", ["whole", "bulk_tail", "portions", "mixed"])
def test_cutting_modes_on_the_host_path(models, name, mode):
    cfg, w = TF.load_model_dir(models[name])
    reqs = _requests(cfg["vocab"])
    steps = {"whole": tiny.schedule_whole, "bulk_tail": lambda r: tiny.schedule_bulk_tail(r, tail=40),
             "portions": lambda r: tiny.schedule_portions(r, seed=3),
             "mixed": lambda r: tiny.schedule_mixed(r, max_tokens=320, seed=4)}[mode](reqs)
    eng = engine(models[name], TF.TINY[name]["page_size"])
    out = tiny.collect(steps, tiny.run_inprocess(eng.runner, steps), cfg["vocab"])
    for rid, toks in reqs.items():
        ref = P.forward(cfg, w, toks)
        assert (out[rid] - ref).abs().max() < tolerance(ref), (rid, mode)
    eng.runner.cache.check()
    assert eng.runner.cache.num_free_slots == 4
    assert eng.runner.cache.free_pages() == [g.pool.num_pages for g in eng.runner.cache.kv_groups]


def test_the_stream_after_every_layer(models):
    """The residual stream that each block hands on, not only the logits, is the plain implementation's."""
    cfg, w = TF.load_model_dir(models["F1"])
    toks = tiny.random_tokens(cfg["vocab"], 30, 5)
    _, layers = P.forward(cfg, w, toks, return_layers=True)
    eng = engine(models["F1"], 16)
    seen = []
    for i, layer in enumerate(eng.runner.model.layers):
        inner = layer.forward

        def spy(x, pending, ctx, call, next_layer=None, inner=inner):
            out = inner(x, pending, ctx, call, next_layer=next_layer)
            seen.append(x[:len(toks)].clone())
            return out
        layer.forward = spy
    steps = tiny.schedule_whole({"a": toks})
    tiny.run_inprocess(eng.runner, steps)
    assert len(seen) == len(cfg["layers"])
    for i, got in enumerate(seen):
        assert (got.double() - layers[i]).abs().max() < tolerance(layers[i]), i


def test_the_oracle_would_show_a_lost_mechanism(models):
    """The tiny models are made so that these faults move the logits by far more than the tolerance."""
    cfg, w = TF.load_model_dir(models["F1"])
    toks = tiny.random_tokens(cfg["vocab"], 60, 9)
    ref = P.forward(cfg, w, toks)

    def moved(cfg2=None, **tensors):
        w2 = dict(w)
        w2.update(tensors)
        return float((P.forward(cfg2 or cfg, w2, toks) - ref).abs().max()) > 1000 * tolerance(ref)

    def edited(edit):
        other = copy.deepcopy(cfg)
        edit(other)
        return other

    assert moved(**{"l0.mix.sink": w["l0.mix.sink"] - 30.0})                               # a sink that is left out
    assert moved(**{"l1.mix.sink": w["l1.mix.sink"] - 30.0})
    assert moved(edited(lambda c: c["layers"][1]["mixer"]["mask"].update(size=8)))          # a window one token off
    assert moved(edited(lambda c: c["layers"][1]["mixer"]["mask"].update(size=6)))
    assert moved(edited(lambda c: c["layers"][2]["mixer"]["mask"].update(size=21)))
    assert moved(edited(lambda c: c["layers"][0]["mixer"]["rot"].update(base=90.0)))        # the angles
    assert moved(edited(lambda c: c["layers"][0]["mixer"].update(scale=0.8)))
    assert moved(edited(lambda c: c.update(residual_mult=0.6)))
    assert moved(edited(lambda c: c["norm"].update(groups=1)))
    assert moved(edited(lambda c: c["norm"].update(eps=1e-2)))
    assert moved(edited(lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=3)))  # every group may be chosen
    assert moved(edited(lambda c: c["layers"][3]["mlp"]["router"]["groups"].update(keep=2)))
    assert moved(edited(lambda c: c["layers"][0]["mlp"]["router"].update(scale=1.0)))
    assert moved(edited(lambda c: c["layers"][0]["mlp"]["router"].update(top=1)))
    shifted = torch.roll(w["l1.canon1"], 1, dims=1)                                         # the taps in the other order
    assert moved(**{"l1.canon1": shifted})
    assert moved(**{"l3.canon2": torch.zeros_like(w["l3.canon2"])})
    assert moved(**{"l2.dwa": torch.roll(w["l2.dwa"], 1)})                                  # the average over depth
    assert moved(**{"l0.dwa": torch.tensor([0.0, 1.0])})
    assert moved(**{"l0.mlp.shared.sg": torch.zeros_like(w["l0.mlp.shared.sg"])})           # the shared expert's gate
    assert moved(**{"l3.mix.g": torch.zeros_like(w["l3.mix.g"])})                           # the output gate
    assert moved(**{"l0.mix.dkv.norm": torch.ones_like(w["l0.mix.dkv.norm"])})


def test_prefill_equals_token_by_token_decoding(models):
    for name in ("F1", "F2"):
        cfg, w = TF.load_model_dir(models[name])
        toks = tiny.random_tokens(cfg["vocab"], 75, 21)
        ref = P.forward(cfg, w, toks)
        steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
        eng = engine(models[name], TF.TINY[name]["page_size"])
        out = tiny.collect(steps, tiny.run_inprocess(eng.runner, steps), cfg["vocab"])["x"]
        assert (out - ref).abs().max() < tolerance(ref), name


@pytest.mark.parametrize("pattern", [[2] * 40, [3, 2, 5, 2, 2, 7, 1, 1, 2, 30, 2, 23], [1, 79], [78, 2], [6] * 13 + [2]])
def test_portions_down_to_two_tokens(models, pattern):
    """Portions shorter than the convolutions' reach and than every window; windows' and pages' edges fall inside them."""
    cfg, w = TF.load_model_dir(models["F1"])
    toks = tiny.random_tokens(cfg["vocab"], sum(pattern), 31)
    ref = P.forward(cfg, w, toks)
    steps, at = [], 0
    for i, n in enumerate(pattern):
        steps.append({"step": i, "entries": [{"id": "x", "tokens": toks[at:at + n], "want": list(range(n))}], "end": []})
        at += n
    eng = engine(models["F1"], 16)
    out = tiny.collect(steps, tiny.run_inprocess(eng.runner, steps), cfg["vocab"])["x"]
    assert (out - ref).abs().max() < tolerance(ref)


def test_pages_below_a_window_go_back_and_are_used_again(models):
    """A request far longer than its windows holds few pages of the windowed groups; another request then takes them."""
    cfg, w = TF.load_model_dir(models["F1"])
    long_toks, short = tiny.random_tokens(cfg["vocab"], 200, 1), tiny.random_tokens(cfg["vocab"], 40, 2)
    eng = engine(models["F1"], 16, pool=256)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": long_toks[:150], "want": list(range(150))}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": long_toks[150:], "want": list(range(50))},
                                     {"id": "b", "tokens": short, "want": list(range(40))}], "end": []}]
    outs = tiny.run_inprocess(eng.runner, steps[:1])
    held = {g.need.window: g.pool.num_pages - g.pool.num_free for g in eng.runner.cache.kv_groups}
    assert held[None] == 10 and held[7] <= 2 and held[20] <= 3
    outs.update(tiny.run_inprocess(eng.runner, steps[1:]))
    out = tiny.collect(steps, outs, cfg["vocab"])
    for rid, toks in (("a", long_toks), ("b", short)):
        ref = P.forward(cfg, w, toks)
        assert (out[rid] - ref).abs().max() < tolerance(ref), rid


VARIANTS = {
    # one layer, one head, one expert that every token takes, no shared expert, a window of two, two taps
    "single": TF._config(30, 16, 1e-5, 1, 0.7, 2, [TF._win(1, 4, 4, 4, 0.5, 2, TF._moe(1, 1, 8))]),
    # no feed-forward anywhere, only the rotated mixer, groups as wide as the row (a norm per element pair)
    "mixers_only": TF._config(41, 24, 1e-6, 12, 1.3, 4, [TF._rot(2, 4, 8, 6, 6, 0.3, 50.0, None), TF._rot(3, 2, 2, 4, 5, 0.9, 2.0, None)]),
    # every group kept (no limit), as many groups as experts, top = all experts of the kept groups, six taps
    "groups": TF._config(64, 40, 1e-5, 2, 0.2, 6, [
        TF._win(2, 8, 8, 8, 0.4, 5, TF._moe(6, 3, 12, groups=(2, 2), scale=0.5, shared=4), plain=True),
        TF._win(5, 4, 6, 8, 0.4, 64, TF._moe(6, 2, 12, groups=(6, 2), scale=3.0)),
        TF._rot(2, 6, 4, 4, 8, 0.5, 300.0, TF._moe(8, 4, 8, groups=(4, 2)))]),
}


@pytest.mark.parametrize("name", list(VARIANTS))
def test_other_arrangements_of_the_layers(tmp_path, name):
    """Values that make mechanisms coincide or vanish, other sizes and orders, in a mixed schedule over a small pool, and
    greedy generation through the scheduler."""
    conf = VARIANTS[name]
    d = TF.make_model_dir("_" + name, str(tmp_path), config=conf, seed=3, store="float32")
    cfg, w = TF.load_model_dir(d)
    V = conf["vocab"]
    reqs = {f"r{i}": tiny.random_tokens(V, n, i) for i, n in enumerate([20, 1, 33, 7, 2, 15, 70])}
    steps = tiny.schedule_mixed(reqs, max_tokens=192, seed=1)
    eng = Engine.from_model_dir(d, EngineOptions(dtype="float32", device="cpu", page_size=4, num_pages=48, max_num_seqs=4,
                                                 max_num_batched_tokens=192), kernels=ReferenceKernels(torch.float64))
    out = tiny.collect(steps, tiny.run_inprocess(eng.runner, steps), V)
    for rid, toks in reqs.items():
        ref = P.forward(cfg, w, toks)
        assert (out[rid] - ref).abs().max() < tolerance(ref), rid
    prompt = tiny.random_tokens(V, 5, 9)
    assert eng.generate([prompt], SamplingParams(max_tokens=6)) == [P.greedy(cfg, w, prompt, 6)]


def test_greedy_generation_through_the_scheduler(models):
    cfg, w = TF.load_model_dir(models["F1"])
    eng = engine(models["F1"], 16, max_num_batched_tokens=24)          # prompts go in as portions beside decoded tokens
    prompts = [tiny.random_tokens(cfg["vocab"], n, 40 + n) for n in (1, 9, 33, 70, 5, 18)]      # six requests, four slots
    outs = eng.generate(prompts, SamplingParams(max_tokens=12))
    for p, o in zip(prompts, outs):
        assert o == P.greedy(cfg, w, p, 12)
    eng.runner.cache.check()
    assert eng.runner.cache.num_free_slots == 4
