"""Tiny Filorax configurations and model folders with weights drawn here (not by the package), shaped so that a fault
shows: query matrices are scaled up (peaked attention: a wrong, missing or stale latent moves the logits), sinks are of
the size of the scores, the taps of the short convolutions and the weights of the average over depth are far from 0,
router matrices are large enough that the choice of experts is no close call, and the shared expert's gate is neither
open nor shut."""
from __future__ import annotations

import json
import os

import torch


def _moe(experts, top, ff, groups=None, scale=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        router["scale"] = scale
    m = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def _win(heads, dim, vdim, rank, scale, window, mlp, plain=False):
    """A windowed latent attention: with sink and gate, or (``plain``) with the ordinary softmax and no gate."""
    return {"type": "latent_attention_3" if plain else "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "mask": {"size": window}}, "mlp": mlp}


def _rot(heads, dim, rot, vdim, rank, scale, base, mlp):
    """The causal latent attention with a rotated key part shared by the heads, sink and gate."""
    return {"type": "latent_attention_2",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "rot": {"base": base, "dims": rot}, "vdim": vdim, "kv_rank": rank,
                      "scale": scale}, "mlp": mlp}


def _config(vocab, width, eps, groups, mult, taps, layers):
    return {"architecture": "Filorax", "canon": {"taps": taps}, "layers": layers, "norm": {"eps": eps, "groups": groups},
            "residual_mult": mult, "vocab": vocab, "width": width}


TINY = {
    # all three mixers, a layer without feed-forward, three norm groups, three taps, groups of experts of which two of three
    # are kept, a shared expert in one layer only, float32 storage
    "F1": dict(config=_config(101, 48, 1e-5, 3, 0.5, 3, [
        _rot(3, 8, 6, 10, 12, 0.4, 100.0, _moe(6, 3, 20, groups=(3, 2), scale=1.5, shared=28)),
        _win(2, 12, 8, 16, 0.35, 7, None),
        _win(4, 4, 4, 8, 0.6, 20, _moe(4, 4, 12), plain=True),
        _rot(2, 6, 2, 6, 10, 0.5, 7.0, _moe(4, 2, 16, groups=(2, 1), scale=2.5, shared=8))]),
               page_size=16, store="float32", seed=21),
    # values that make mechanisms coincide or vanish: one norm group, one tap (no state to carry), a multiplier of one, a
    # window of one token and one longer than any test sequence, one expert group, top 1, pages of 8; bfloat16 storage
    "F2": dict(config=_config(77, 32, 1e-6, 1, 1.0, 1, [
        _win(2, 8, 8, 8, 0.5, 1, _moe(3, 1, 8, shared=8)),
        _win(1, 16, 12, 24, 0.3, 4096, _moe(2, 2, 24, groups=(1, 1))),
        _rot(4, 4, 4, 8, 6, 0.7, 10000.0, None),
        _win(2, 8, 4, 8, 0.4, 9, None, plain=True)]),
               page_size=8, store="bfloat16", seed=22),
    # wider, sizes the tensor-core routes take: products with k of 256 and 64, five taps, windows of 33 and 50
    "F3": dict(config=_config(331, 256, 1e-5, 4, 0.25, 5, [
        _win(4, 32, 64, 64, 0.2, 33, _moe(8, 2, 64, groups=(4, 2), scale=2.0, shared=128)),
        _rot(4, 64, 32, 32, 96, 0.12, 10000.0, _moe(4, 3, 128, shared=64)),
        _win(8, 16, 16, 32, 0.3, 50, _moe(8, 3, 32, groups=(2, 1), scale=1.0), plain=True)]),
               page_size=16, store="bfloat16", seed=23),
}


def make_weights(cfg, seed, sharpen=3.0):
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    taps = cfg["canon"]["taps"]

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * (gain / i ** 0.5)

    def near_one(*shape, spread=0.2):
        return 1.0 + spread * torch.randn(tuple(shape), generator=g)

    w = {"embed": torch.randn(V, W, generator=g), "head": mat(V, W, 2.0), "final.norm": near_one(W)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, D, Vd, R, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m.get("rot_dim", 0)
        w[p + "norm1"] = near_one(W)
        w[p + "canon1"] = 0.4 * torch.randn(W, taps, generator=g)
        w[p + "dwa"] = 1.0 / (i + 2) + 0.3 * torch.randn(i + 2, generator=g)
        w[p + "mix.q"] = mat(H * (D + r), W, sharpen)
        w[p + "mix.dkv"] = mat(R + r, W, 1.5)
        w[p + "mix.dkv.norm"] = near_one(R)
        w[p + "mix.uk"], w[p + "mix.uv"], w[p + "mix.o"] = mat(H * D, R, 1.5), mat(H * Vd, R), mat(W, H * Vd)
        if layer["type"] != "latent_attention_3":
            w[p + "mix.sink"] = 1.5 + 2.0 * torch.randn(H, generator=g)
            w[p + "mix.g"] = mat(H * Vd, W, 2.0)
        mlp = layer["mlp"]
        if mlp is not None:
            e, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            w[p + "norm2"] = near_one(W)
            w[p + "canon2"] = 0.4 * torch.randn(W, taps, generator=g)
            w[p + "mlp.router"] = mat(e, W, 3.0)
            for j in range(e):
                w[f"{p}mlp.e{j}.gate"], w[f"{p}mlp.e{j}.up"], w[f"{p}mlp.e{j}.down"] = mat(ff, W, 2.0), mat(ff, W), mat(W, ff)
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                w[p + "mlp.shared.gate"], w[p + "mlp.shared.up"], w[p + "mlp.shared.down"] = mat(sf, W, 2.0), mat(sf, W), mat(W, sf)
                w[p + "mlp.shared.sg"] = mat(1, W, 1.5)
    return w


def make_model_dir(name, root, config=None, seed=None, store=None):
    """Write tiny model ``name`` under ``root`` (config.json, model.safetensors) and return the folder.  The values
    are rounded to the storage dtype before they are written, so the oracle and the engine read the same numbers."""
    from safetensors.torch import save_file
    spec = TINY.get(name, {})
    config = config or spec["config"]
    d = os.path.join(root, f"tiny{name}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(config, f)
    dt = getattr(torch, store or spec["store"])
    save_file({k: v.to(dt).contiguous() for k, v in make_weights(config, seed if seed is not None else spec["seed"]).items()},
              os.path.join(d, "model.safetensors"))
    return d


def load_model_dir(d):
    """(config mapping, weights as float64-ready tensors) of a folder written by :func:`make_model_dir`."""
    from safetensors.torch import load_file
    with open(os.path.join(d, "config.json")) as f:
        cfg = json.load(f)
    return cfg, {k: v.float() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
