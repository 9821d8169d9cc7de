"""Golonex on a machine without a GPU: configuration, plan, loader, cache entries and the engine's host side (step
function, state slots, pages, scheduler) over the plain kernel statements of tests/kernel_refs.py, against the plain
implementation of tests/plain_golonex.py.  The CUDA kernels themselves are the business of test_golonex_gpu.py."""
import copy

import pytest
import torch

import plain_golonex as P
import tiny
import tiny_golonex as TG
from kernel_refs import ReferenceKernels
from infurnace_b200.cache import CacheLayout, CacheManager
from infurnace_b200.config.specs import (
    KVCacheNeed, LatentAttentionSpec, PagedCacheNeed, PreNormBlockSpec, RealGatedRecurrenceSpec, RotaryValueAttentionSpec,
    RoutedExpertsSpec,
)
from infurnace_b200.engine import Engine, EngineOptions, SamplingParams
from infurnace_b200.errors import ModelConfigError, WeightError
from infurnace_b200.models import config_from_dict, plan_for

TOL = 2e-5      # float32 stream and buffers against the float64 oracle


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("golonex"))
    return {n: TG.make_model_dir(n, root) for n in ("G1", "G2")}


def engine(model_dir, page_size, pool=320, **kw):
    opts = dict(dtype="float32", device="cpu", page_size=page_size, num_pages=pool // page_size, max_num_seqs=4,
                max_num_batched_tokens=pool)
    opts.update(kw)
    return Engine.from_model_dir(model_dir, EngineOptions(**opts), kernels=ReferenceKernels(torch.float64))


def tolerance(ref):
    return TOL * max(1.0, float(ref.abs().max()))


# ------------------------------------------------------------------------------ each mechanism of the oracle alone
def test_the_oracles_mechanisms_alone():
    g = torch.Generator().manual_seed(0)
    # rotation: a pair turns by position * frequency; position 0 leaves the vector alone; lengths are kept without stretching
    v = torch.randn(5, 2, 6, generator=g, dtype=torch.float64)
    rot = {"base": 10.0, "dims": 4}
    t = P.rotate_pairs(v, rot)
    assert torch.equal(t[0], v[0]) and torch.equal(t[..., 4:], v[..., 4:])
    assert torch.allclose(t[..., :4].norm(dim=-1), v[..., :4].norm(dim=-1))
    a = 3 * 10.0 ** (-2 / 4)                      # pair 1 at position 3
    assert torch.allclose(t[3, 0, 2], v[3, 0, 2] * torch.cos(torch.tensor(a)) - v[3, 0, 3] * torch.sin(torch.tensor(a)))
    # stretched frequencies: fast pairs keep theirs, slow ones are divided, cosine and sine carry the factor
    plain, one = P.rotary_frequencies({"base": 100.0, "dims": 8})
    freq, gain = P.rotary_frequencies({"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}})
    assert one == 1.0 and abs(gain - (0.1 * 1.3862943611198906 + 1)) < 1e-12
    assert torch.allclose(freq[0], plain[0]) and torch.allclose(freq[-1], plain[-1] / 4.0) and bool((freq <= plain).all())
    # the window and the sink
    q = torch.zeros(4, 1, 2, dtype=torch.float64)
    k = torch.zeros(4, 1, 2, dtype=torch.float64)
    val = torch.arange(4, dtype=torch.float64).view(4, 1, 1)
    assert torch.allclose(P.softmax_attention(q, k, val, 1.0, 2)[:, 0, 0], torch.tensor([0.0, 0.5, 1.5, 2.5], dtype=torch.float64))
    assert torch.allclose(P.softmax_attention(q, k, val, 1.0, None)[:, 0, 0], torch.tensor([0.0, 0.5, 1.0, 1.5], dtype=torch.float64))
    sunk = P.softmax_attention(q, k, val, 1.0, 2, sink=torch.zeros(1, dtype=torch.float64))[:, 0, 0]
    assert torch.allclose(sunk, torch.tensor([0.0, 1.0 / 3, 1.0, 5.0 / 3], dtype=torch.float64))
    # the convolution: the last column is the current token's
    x = torch.tensor([[1.0], [10.0], [100.0]], dtype=torch.float64)
    u = P.short_convolution(x, torch.tensor([[3.0, 2.0]], dtype=torch.float64), torch.tensor([0.5], dtype=torch.float64))
    assert torch.allclose(u[:, 0], torch.tensor([2.5, 23.5, 230.5], dtype=torch.float64))
    # the recurrence: a gate of zero keeps nothing of the past and passes sqrt(1 - 1) = 0 of the input; from S = 0
    ones = torch.ones(3, 2, dtype=torch.float64)
    S = P.real_gated_recurrence(ones, ones, ones, torch.tensor([-30.0, 30.0], dtype=torch.float64))
    assert float(S[:, 0].abs().max()) < 1e-5 and float((S[:, 1] - 1.0).abs().max()) < 1e-9
    S = P.real_gated_recurrence(0.5 * ones, ones, ones, torch.zeros(2, dtype=torch.float64))
    a = torch.exp(torch.tensor(-8 * 0.5 * 0.6931471805599453, dtype=torch.float64))
    assert torch.allclose(S[1, 0], a * torch.sqrt(1 - a * a) + torch.sqrt(1 - a * a))
    # the router: sigmoid scores, the lower index among equals, weights not renormalised
    router = torch.tensor([[1.0, 1.0, -1.0], [1.0, 2.0, 0.0]], dtype=torch.float64)          # [experts, width]
    idx, wt = P.route(torch.eye(3, dtype=torch.float64), router, 1)
    assert idx[:, 0].tolist() == [0, 1, 1] and torch.allclose(wt[:, 0], torch.sigmoid(torch.tensor([1.0, 2.0, 0.0], dtype=torch.float64)))


# ------------------------------------------------------------------------------ configuration, plan, weights
def test_configuration_round_trip_and_plan():
    for name, spec in TG.TINY.items():
        conf = spec["config"]
        cfg = config_from_dict(conf)
        assert cfg.to_dict() == conf, name
        plan = plan_for(cfg)
        made = TG.make_weights(conf, 0)
        assert set(n for n, t in plan.tensors().items() if not t.optional) == set(made), name
        for tname, t in made.items():
            assert tuple(plan.tensors()[tname].shape) == tuple(t.shape), tname
        assert plan.lm_head.tied and plan.lm_head.weight == plan.embedding.weight and plan.lm_head.softcap == conf.get("logit_softcap")
        for layer, entry in zip(plan.layers, conf["layers"]):
            assert isinstance(layer, PreNormBlockSpec)
            m, mixer = entry["mixer"], layer.mixer
            assert (layer.ffn is None) == (entry["mlp"] is None) == (layer.ffn_norm is None)
            assert (layer.side is None) == ("token_side" not in conf)
            if entry["type"] == "rglru":
                assert isinstance(mixer, RealGatedRecurrenceSpec)
                assert (mixer.width, mixer.blocks, mixer.taps, mixer.decay_scale) == (m["width"], m["blocks"], m["conv"], 8.0)
            elif entry["type"] == "latent_attention":
                assert isinstance(mixer, LatentAttentionSpec) and mixer.gate_per_head and mixer.sink is not None
                assert (mixer.num_heads, mixer.head_dim, mixer.rot_dim, mixer.value_head_dim, mixer.kv_rank, mixer.q_rank, mixer.scale) == \
                    (m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"], m["scale"])
                assert mixer.window == (m["mask"]["size"] if "mask" in m else None)
                assert (mixer.position is None) == (m["rot_dim"] == 0)
                if mixer.position is not None:
                    assert mixer.position.interleaved and mixer.position.rotary_dim == m["rot"]["dims"]
            else:
                assert isinstance(mixer, RotaryValueAttentionSpec) and mixer.v_proj is None and mixer.position.interleaved
                assert (mixer.num_heads, mixer.num_kv_heads, mixer.head_dim, mixer.scale) == (m["heads"], m["kv_heads"], m["dim"], m["scale"])
                sc = m["rot"].get("scaling")
                assert mixer.position.scaling == ((sc["factor"], sc["original"], sc["fast"], sc["slow"]) if sc else None)
            if layer.ffn is not None:
                r = entry["mlp"]["router"]
                assert isinstance(layer.ffn, RoutedExpertsSpec) and layer.ffn.scoring == "sigmoid" and layer.ffn.weight_on == "input"
                assert layer.ffn.top == r["top"] and len(layer.ffn.experts) == r["experts"]
                assert (layer.ffn.shared is None) == ("shared" not in entry["mlp"])


def test_cache_entries_pages_and_states():
    conf = TG.TINY["G1"]["config"]
    plan = plan_for(config_from_dict(conf))
    layout = CacheLayout(plan)
    kinds = sorted((type(need).__name__, need.window) for need, _ in layout.kv.values())
    assert kinds == [("KVCacheNeed", 9), ("PagedCacheNeed", 7), ("PagedCacheNeed", 20)]
    states = {need.shape: len(ids) for need, ids in layout.state.values()}
    assert states == {(36,): 1, (2, 36): 1, (24,): 1, (4, 24): 1}          # per recurrent layer: the state and taps - 1 inputs
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
    assert any(isinstance(n, KVCacheNeed) for n, _ in layout.kv.values()) and any(isinstance(n, PagedCacheNeed) for n, _ in layout.kv.values())


def test_configuration_faults_are_named():
    base = TG.TINY["G1"]["config"]

    def broken(edit):
        c = copy.deepcopy(base)
        edit(c)
        with pytest.raises(ModelConfigError) as e:
            config_from_dict(c)
        return str(e.value)

    assert "type" in broken(lambda c: c["layers"][0].update(type="lstm"))
    assert "blocks" in broken(lambda c: c["layers"][0]["mixer"].update(blocks=5))
    assert "conv" in broken(lambda c: c["layers"][0]["mixer"].pop("conv"))
    assert "q_rank" in broken(lambda c: c["layers"][1]["mixer"].pop("q_rank"))
    assert "rot.dims" in broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=8))
    assert "rot.dims" in broken(lambda c: c["layers"][2]["mixer"]["rot"].update(dims=3))
    assert "scaling.factor" in broken(lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("factor"))
    assert "kv_heads" in broken(lambda c: c["layers"][2]["mixer"].update(kv_heads=3))
    assert "vdim" in broken(lambda c: c["layers"][2]["mixer"].update(vdim=8))
    assert "mask.size" in broken(lambda c: c["layers"][2]["mixer"].update(mask={}))
    assert "moe" in broken(lambda c: c["layers"][0]["mlp"].update(kind="dense"))
    assert "top" in broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=6))
    assert "eps" in broken(lambda c: c.update(norm={}))
    assert "token_side" in broken(lambda c: c.update(token_side={}))
    assert "layers" in broken(lambda c: c.update(layers=[]))


def test_loader_lists_what_is_wrong(models, tmp_path):
    import os
    import shutil
    from safetensors.torch import load_file, save_file
    d = str(tmp_path / "bad")
    shutil.copytree(models["G1"], d)
    t = load_file(os.path.join(d, "model.safetensors"))
    del t["l1.mix.sink"]
    t["l2.mix.v"] = torch.zeros(24, 48)             # the values are the keys: there is no v matrix
    t["l3.mlp.router"] = torch.ones(2, 48)          # layer 3 has no feed-forward
    t["l0.mix.ra"] = torch.ones(3, 12, 11)          # square matrices per block
    t["head"] = torch.ones(101, 48)                 # the head is the embedding table
    save_file(t, os.path.join(d, "model.safetensors"))
    with pytest.raises(WeightError) as e:
        engine(d, 16)
    msg = str(e.value)
    assert all(name in msg for name in ("l1.mix.sink", "l2.mix.v", "l3.mlp.router", "l0.mix.ra", "head"))


# ------------------------------------------------------------------------------ the engine's host side
LENS = [37, 100, 64, 19, 85, 50, 1, 2, 3]


def _requests(vocab, seed=0):
    return {f"r{i}": tiny.random_tokens(vocab, n, seed + i) for i, n in enumerate(LENS)}


@pytest.mark.parametrize("name", ["G1", "G2"])
@pytest.mark.parametrize("mode", ["whole", "bulk_tail", "portions", "mixed"])
def test_cutting_modes_on_the_host_path(models, name, mode):
    cfg, w = TG.load_model_dir(models[name])
    reqs = _requests(cfg["vocab"])
    steps = {"whole": tiny.schedule_whole, "bulk_tail": lambda r: tiny.schedule_bulk_tail(r, tail=40),
             "portions": lambda r: tiny.schedule_portions(r, seed=3),
             "mixed": lambda r: tiny.schedule_mixed(r, max_tokens=320, seed=4)}[mode](reqs)
    eng = engine(models[name], TG.TINY[name]["page_size"])
    out = tiny.collect(steps, tiny.run_inprocess(eng.runner, steps), cfg["vocab"])
    for rid, toks in reqs.items():
        ref = P.forward(cfg, w, toks)
        assert (out[rid] - ref).abs().max() < tolerance(ref), (rid, mode)
    eng.runner.cache.check()
    assert eng.runner.cache.num_free_slots == 4
    assert eng.runner.cache.free_pages() == [g.pool.num_pages for g in eng.runner.cache.kv_groups]


def test_the_stream_after_every_layer(models):
    """The residual stream after each block, not only the logits, is the plain implementation's."""
    cfg, w = TG.load_model_dir(models["G1"])
    toks = tiny.random_tokens(cfg["vocab"], 30, 5)
    _, layers = P.forward(cfg, w, toks, return_layers=True)
    eng = engine(models["G1"], 16)
    seen = []
    for layer in eng.runner.model.layers:
        inner = layer.forward

        def spy(x, pending, ctx, call, next_layer=None, inner=inner):
            out = inner(x, pending, ctx, call, next_layer=next_layer)
            seen.append(x[:len(toks)].clone())           # a block with a side input leaves the stream up to date
            return out
        layer.forward = spy
    tiny.run_inprocess(eng.runner, tiny.schedule_whole({"a": toks}))
    assert len(seen) == len(cfg["layers"])
    for i, got in enumerate(seen):
        assert (got.double() - layers[i]).abs().max() < tolerance(layers[i]), i


def test_the_oracle_would_show_a_lost_mechanism(models):
    """The tiny models are made so that these faults move the logits by far more than the tolerance."""
    cfg, w = TG.load_model_dir(models["G1"])
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

    assert moved(**{"l1.mix.sink": w["l1.mix.sink"] - 30.0})                               # a sink that is left out
    assert moved(**{"l4.mix.sink": w["l4.mix.sink"] - 30.0})
    assert moved(edited(lambda c: c["layers"][1]["mixer"]["mask"].update(size=8)))          # a window one token off
    assert moved(edited(lambda c: c["layers"][1]["mixer"]["mask"].update(size=6)))
    assert moved(edited(lambda c: c["layers"][2]["mixer"]["mask"].update(size=10)))
    assert moved(edited(lambda c: c["layers"][2]["mixer"]["mask"].update(size=8)))
    assert moved(edited(lambda c: c["layers"][4]["mixer"]["mask"].update(size=21)))
    assert moved(edited(lambda c: c["layers"][1]["mixer"]["rot"].update(base=90.0)))        # the angles
    assert moved(edited(lambda c: c["layers"][2]["mixer"]["rot"].update(dims=12)))
    assert moved(edited(lambda c: c["layers"][2]["mixer"]["rot"].pop("scaling")))
    assert moved(edited(lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].update(factor=2.0)))
    assert moved(edited(lambda c: c["layers"][4]["mixer"]["rot"].update(dims=4)))
    assert moved(edited(lambda c: c["layers"][1]["mixer"].update(scale=0.8)))
    assert moved(edited(lambda c: c["norm"].update(eps=1e-2)))
    assert moved(edited(lambda c: c["layers"][0]["mlp"]["router"].update(top=1)))
    assert moved(edited(lambda c: c.update(logit_softcap=5.0)))
    assert moved(**{"l0.mix.conv": torch.roll(w["l0.mix.conv"], 1, dims=1)})                # the taps in the other order
    assert moved(**{"l3.mix.conv.b": torch.zeros_like(w["l3.mix.conv.b"])})
    assert moved(**{"l0.mix.lam": w["l0.mix.lam"] + 1.0})                                   # the decays
    assert moved(**{"l0.mix.ra": torch.roll(w["l0.mix.ra"], 1, dims=0)})                    # the blocks of the gates
    assert moved(**{"l3.mix.ri.b": torch.zeros_like(w["l3.mix.ri.b"])})
    assert moved(**{"l0.mix.y.b": torch.zeros_like(w["l0.mix.y.b"])})
    assert moved(**{"l0.mlp.shared.sg": torch.zeros_like(w["l0.mlp.shared.sg"])})           # the shared expert's gate
    assert moved(**{"l1.mix.g": torch.zeros_like(w["l1.mix.g"])})                           # the output gate
    assert moved(**{"l1.mix.dq.norm": torch.ones_like(w["l1.mix.dq.norm"])})
    assert moved(**{"side.embed": torch.roll(w["side.embed"], 5, dims=1)})                  # each layer its own slice
    assert moved(**{"embed.norm": torch.ones_like(w["embed.norm"])})
    # the weight on the expert's input is not the weight on its output
    def output_weighted(h, weights, p, mlp):
        chosen, weight = P.route(h, P.w64(weights, p + "router"), int(mlp["router"]["top"]))
        out = torch.zeros(h.shape[0], h.shape[1], dtype=torch.float64)
        for t in range(h.shape[0]):
            for e, g in zip(chosen[t].tolist(), weight[t]):
                out[t] += g * P.gated_expert(h[t:t + 1], weights, f"{p}e{e}.")[0]
        if mlp.get("shared"):
            out = out + torch.sigmoid(h @ P.w64(weights, p + "shared.sg").T) * P.gated_expert(h, weights, p + "shared.")
        return out
    inner = P.mixture
    P.mixture = output_weighted
    try:
        assert float((P.forward(cfg, w, toks) - ref).abs().max()) > 1000 * tolerance(ref)
    finally:
        P.mixture = inner


def test_prefill_equals_token_by_token_decoding(models):
    for name in ("G1", "G2"):
        cfg, w = TG.load_model_dir(models[name])
        toks = tiny.random_tokens(cfg["vocab"], 75, 21)
        ref = P.forward(cfg, w, toks)
        steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
        eng = engine(models[name], TG.TINY[name]["page_size"])
        out = tiny.collect(steps, tiny.run_inprocess(eng.runner, steps), cfg["vocab"])["x"]
        assert (out - ref).abs().max() < tolerance(ref), name


@pytest.mark.parametrize("pattern", [[2] * 40, [3, 2, 5, 2, 2, 7, 1, 1, 2, 30, 2, 23], [1, 79], [78, 2], [6] * 13 + [2]])
def test_portions_down_to_two_tokens(models, pattern):
    """Portions shorter than the convolutions' reach and than every window; windows' and pages' edges fall inside them."""
    cfg, w = TG.load_model_dir(models["G1"])
    toks = tiny.random_tokens(cfg["vocab"], sum(pattern), 31)
    ref = P.forward(cfg, w, toks)
    steps, at = [], 0
    for i, n in enumerate(pattern):
        steps.append({"step": i, "entries": [{"id": "x", "tokens": toks[at:at + n], "want": list(range(n))}], "end": []})
        at += n
    eng = engine(models["G1"], 16)
    out = tiny.collect(steps, tiny.run_inprocess(eng.runner, steps), cfg["vocab"])["x"]
    assert (out - ref).abs().max() < tolerance(ref)


def test_pages_below_a_window_go_back_and_are_used_again(models):
    """A request far longer than its windows holds few pages; another request then takes them, and its slot."""
    cfg, w = TG.load_model_dir(models["G1"])
    long_toks, short = tiny.random_tokens(cfg["vocab"], 200, 1), tiny.random_tokens(cfg["vocab"], 40, 2)
    third = tiny.random_tokens(cfg["vocab"], 30, 3)
    eng = engine(models["G1"], 16, pool=208)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": long_toks[:150], "want": list(range(150))}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": long_toks[150:], "want": list(range(50))},
                                     {"id": "b", "tokens": short, "want": list(range(40))}], "end": ["a"]},
             {"step": 2, "entries": [{"id": "c", "tokens": third, "want": list(range(30))}], "end": ["b", "c"]}]
    outs = tiny.run_inprocess(eng.runner, steps[:1])
    held = {g.need.window: g.pool.num_pages - g.pool.num_free for g in eng.runner.cache.kv_groups}
    assert held[7] <= 2 and held[9] <= 2 and held[20] <= 3
    outs.update(tiny.run_inprocess(eng.runner, steps[1:]))
    out = tiny.collect(steps, outs, cfg["vocab"])
    for rid, toks in (("a", long_toks), ("b", short), ("c", third)):
        ref = P.forward(cfg, w, toks)
        assert (out[rid] - ref).abs().max() < tolerance(ref), rid


VARIANTS = {
    # one layer of each kind alone; one head, one expert that every token takes, a window of two, two taps
    "recurrent_only": TG._config(30, 16, 1e-5, [TG._rec(16, 2, 2, TG._moe(1, 1, 8))]),
    "latent_only": TG._config(41, 24, 1e-6, [TG._lat(1, 4, 2, 4, 4, 3, 0.5, 2, 50.0, None)], side=3),
    "attention_only": TG._config(33, 16, 1e-5, [TG._att(1, 1, 6, 0.6, 2, 2.0, 6, TG._moe(2, 2, 4, shared=4))], cap=3.0),
    # no feed-forward anywhere, blocks as small as one channel, seven taps (longer than most portions)
    "mixers_only": TG._config(50, 24, 1e-6, [TG._rec(12, 12, 7, None), TG._att(6, 3, 4, 0.9, 5, 100.0, 2, None),
                                             TG._lat(3, 2, 2, 4, 5, 4, 0.9, 64, 2.0, None)]),
    # another order: attention first and last, recurrences side by side, eight experts of which all but one run
    "order": TG._config(64, 40, 1e-5, [
        TG._att(5, 5, 8, 0.4, 5, 300.0, 4, TG._moe(8, 7, 8, shared=4), scaling=(8.0, 32, 4.0, 0.5)),
        TG._rec(40, 5, 4, TG._moe(3, 2, 12)), TG._rec(20, 2, 2, None),
        TG._lat(5, 4, 6, 6, 8, 9, 0.4, 11, 300.0, TG._moe(6, 2, 12, shared=8)),
        TG._att(2, 1, 10, 0.4, 64, 9.0, 10, None)], cap=20.0, side=2),
}


@pytest.mark.parametrize("name", list(VARIANTS))
def test_other_arrangements_of_the_layers(tmp_path, name):
    """Values that make mechanisms coincide or vanish, other sizes and orders, in a mixed schedule over a small pool, and
    greedy generation through the scheduler."""
    conf = VARIANTS[name]
    d = TG.make_model_dir("_" + name, str(tmp_path), config=conf, seed=3, store="float32")
    cfg, w = TG.load_model_dir(d)
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
    cfg, w = TG.load_model_dir(models["G1"])
    eng = engine(models["G1"], 16, max_num_batched_tokens=24)          # prompts go in as portions beside decoded tokens
    prompts = [tiny.random_tokens(cfg["vocab"], n, 40 + n) for n in (1, 9, 33, 70, 5, 18)]      # six requests, four slots
    outs = eng.generate(prompts, SamplingParams(max_tokens=12))
    for p, o in zip(prompts, outs):
        assert o == P.greedy(cfg, w, p, 12)
    eng.runner.cache.check()
    assert eng.runner.cache.num_free_slots == 4
