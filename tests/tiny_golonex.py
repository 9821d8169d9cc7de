"""Tiny Golonex configurations and model folders with weights drawn here (not by the package), shaped so that a fault
shows: query matrices are scaled up (peaked attention: a wrong, missing or stale key moves the logits), sinks are of the
size of the scores, the decays of the recurrence are spread from fast to slow, the taps of its convolution are far from
0, router matrices are large enough that the choice of experts is no close call, and the gates are neither open nor shut."""
from __future__ import annotations

import json
import os

import torch


def _moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def _lat(heads, dim, rot, vdim, rank, qrank, scale, window, base, mlp, dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "q_rank": qrank, "scale": scale}
    if rot:
        m["rot"] = {"base": base, "dims": dims or rot}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def _att(heads, kv, dim, scale, window, base, dims, mlp, scaling=None):
    rot = {"base": base, "dims": dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale, "rot": rot}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _rec(width, blocks, taps, mlp):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": taps}, "mlp": mlp}


def _config(vocab, width, eps, layers, cap=None, side=None):
    c = {"architecture": "Golonex", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if cap is not None:
        c["logit_softcap"] = cap
    if side is not None:
        c["token_side"] = {"dim": side}
    return c


TINY = {
    # all three mixers, the recurrence first, a layer without feed-forward, two of five experts, a shared expert in some
    # layers, partly rotated heads with stretched frequencies, a token side input, a soft cap; float32 storage
    "G1": dict(config=_config(101, 48, 1e-5, [
        _rec(36, 3, 3, _moe(5, 2, 20, shared=28)),
        _lat(3, 8, 6, 10, 12, 20, 0.4, 7, 100.0, _moe(4, 3, 12)),
        _att(4, 2, 12, 0.3, 9, 50.0, 8, None, scaling=(4.0, 64, 8.0, 1.0)),
        _rec(24, 1, 5, None),
        _lat(2, 6, 4, 6, 10, 7, 0.5, 20, 7.0, _moe(4, 1, 16, shared=8), dims=2)], cap=6.0, side=5),
               page_size=16, store="float32", seed=31),
    # values that make mechanisms coincide or vanish: one tap (no inputs to carry), one block, as many key/value heads as
    # heads, heads rotated whole without stretching, a window of one token and windows longer than any test sequence or
    # none at all, no rotated part, top = all experts, no side input, no cap; pages of 8; bfloat16 storage
    "G2": dict(config=_config(77, 32, 1e-6, [
        _att(2, 2, 8, 0.5, 1, 10000.0, 8, _moe(3, 3, 8)),
        _rec(32, 1, 1, _moe(2, 1, 24, shared=8)),
        _lat(1, 16, 0, 12, 24, 5, 0.3, 4096, 1.0, None),
        _att(4, 1, 4, 0.7, None, 30.0, 2, None),
        _lat(2, 4, 8, 4, 8, 16, 0.4, None, 500.0, _moe(2, 2, 8))]),
               page_size=8, store="bfloat16", seed=32),
    # wider, sizes the tensor-core routes take: heads of 48 and 24, latents of 72 and 96, windows of 33, 50 and 120
    "G3": dict(config=_config(331, 320, 1e-6, [
        _lat(5, 24, 16, 48, 72, 88, 0.2, 33, 10000.0, _moe(6, 2, 40, shared=96)),
        _rec(224, 4, 3, _moe(4, 3, 128, shared=64)),
        _att(6, 3, 48, 0.14, 50, 10000.0, 16, _moe(7, 1, 24), scaling=(3.0, 200, 12.0, 1.5)),
        _lat(8, 16, 16, 16, 96, 48, 0.3, 120, 5000.0, None)], cap=10.0, side=12),
               page_size=16, store="bfloat16", seed=33, sharpen=2.0),       # run in bfloat16 over hundreds of tokens
}


def make_weights(cfg, seed, sharpen=3.0):
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    n = len(cfg["layers"])
    side = cfg["token_side"]["dim"] if cfg.get("token_side") else None

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * (gain / i ** 0.5)

    def near_one(*shape, spread=0.2):
        return 1.0 + spread * torch.randn(tuple(shape), generator=g)

    def vec(size, spread):
        return spread * torch.randn(size, generator=g)

    # the table is also the head: rows of length two keep the logits of size two (the embedding's norm undoes the scale)
    w = {"embed": mat(V, W, 2.0), "embed.norm": near_one(W), "final.norm": near_one(W)}
    if side is not None:
        w["side.embed"] = torch.randn(V, n * side, generator=g)
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        w[p + "norm1"] = near_one(W)
        q = p + "mix."
        if kind == "rglru":
            C, B, taps = m["width"], m["blocks"], m["conv"]
            bs = C // B
            w[q + "y"], w[q + "y.b"], w[q + "x"], w[q + "x.b"] = mat(C, W, 1.5), vec(C, 0.3), mat(C, W, 1.5), vec(C, 0.3)
            w[q + "conv"], w[q + "conv.b"] = 0.5 * torch.randn(C, taps, generator=g), vec(C, 0.2)
            w[q + "ra"], w[q + "ra.b"] = torch.randn(B, bs, bs, generator=g) * (1.5 / bs ** 0.5), vec(B * bs, 0.7).view(B, bs)
            w[q + "ri"], w[q + "ri.b"] = torch.randn(B, bs, bs, generator=g) * (1.5 / bs ** 0.5), vec(B * bs, 0.7).view(B, bs)
            w[q + "lam"] = torch.linspace(-6.0, 0.5, C)[torch.randperm(C, generator=g)]      # decays from slow to fast
            w[q + "o"] = mat(W, C)
        elif kind == "latent_attention":
            H, D, R, Vd, rank, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            w[q + "dq"], w[q + "dq.norm"], w[q + "uq"] = mat(qr, W), near_one(qr), mat(H * (D + R), qr, sharpen)
            w[q + "dkv"], w[q + "dkv.norm"] = mat(rank + R, W, 1.5), near_one(rank)
            w[q + "uk"], w[q + "uv"], w[q + "o"] = mat(H * D, rank, 1.5), mat(H * Vd, rank), mat(W, H * Vd)
            w[q + "sink"] = 1.5 + 2.0 * torch.randn(H, generator=g)
            w[q + "g"] = mat(H, W, 2.0)
        else:
            H, G, D = m["heads"], m["kv_heads"], m["dim"]
            w[q + "q"], w[q + "k"], w[q + "o"] = mat(H * D, W, sharpen), mat(G * D, W, 1.5), mat(W, H * D)
        mlp = layer["mlp"]
        if mlp is not None:
            e, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            w[p + "norm2"] = near_one(W)
            w[p + "mlp.router"] = mat(e, W, 3.0)
            for j in range(e):
                w[f"{p}mlp.e{j}.gate"], w[f"{p}mlp.e{j}.up"], w[f"{p}mlp.e{j}.down"] = mat(ff, W, 2.0), mat(ff, W), mat(W, ff)
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                w[p + "mlp.shared.gate"], w[p + "mlp.shared.up"], w[p + "mlp.shared.down"] = mat(sf, W, 2.0), mat(sf, W), mat(W, sf)
                w[p + "mlp.shared.sg"] = mat(1, W, 1.5)
        if side is not None:
            w[p + "side.gate"], w[p + "side.proj"], w[p + "side.norm"] = mat(side, W, 1.5), mat(W, side), 0.5 * near_one(W)
    return w


def make_model_dir(name, root, config=None, seed=None, store=None, sharpen=None):
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
    made = make_weights(config, seed if seed is not None else spec["seed"], sharpen=sharpen or spec.get("sharpen", 3.0))
    save_file({k: v.to(dt).contiguous() for k, v in made.items()},
              os.path.join(d, "model.safetensors"))
    return d


def load_model_dir(d):
    """(config mapping, weights as float64-ready tensors) of a folder written by :func:`make_model_dir`."""
    from safetensors.torch import load_file
    with open(os.path.join(d, "config.json")) as f:
        cfg = json.load(f)
    return cfg, {k: v.float() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
