"""The Filorax decoder, stated plainly: one function per mechanism, float64, whole sequences, no cache.

It shares no code with the package.  ``weights`` maps tensor names to tensors; ``cfg`` is config.json as a mapping.
A sequence is run from its first token; every function takes [T, ...] tensors of one sequence.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def w64(weights, name):
    return weights[name].to(F64)


def group_rms_norm(x, weight, groups, eps):
    """The row in ``groups`` equal consecutive parts, each divided by its own sqrt(mean(part^2) + eps); then times weight."""
    T, W = x.shape
    parts = x.reshape(T, groups, W // groups)
    parts = parts / torch.sqrt(parts.pow(2).mean(-1, keepdim=True) + eps)
    return parts.reshape(T, W) * weight


def causal_conv_add(h, taps_weight):
    """h_t + sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the sequence's start.  ``taps_weight`` [W, taps]."""
    T, W = h.shape
    taps = taps_weight.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += taps_weight[:, j] * h[s]
    return out


def rotate_half_split(v, positions, base, dims):
    """The first ``dims`` entries of the last axis, entry i paired with i + dims/2, turned by position * base^(-2i/dims)."""
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    ang = positions.to(F64)[:, None] * torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)
    while ang.dim() < v.dim():
        ang = ang.unsqueeze(1)
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat((a * c - b * s, b * c + a * s, v[..., dims:]), dim=-1)


def sink_softmax_attention(q, k, v, scale, window, sink):
    """q [T, H, D], k [T, H, D], v [T, H, V] -> [T, H, V].  Position i sees j <= i, and with a window only i - j < window.
    ``sink`` [H] or None: exp(sink_h) joins the denominator, with no value."""
    T, H, _ = q.shape
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        s = torch.einsum("hd,jhd->hj", q[i], k[lo:i + 1]) * scale          # [H, keys]
        m = s.max(dim=1).values
        if sink is not None:
            m = torch.maximum(m, sink)
        e = torch.exp(s - m[:, None])
        den = e.sum(dim=1)
        if sink is not None:
            den = den + torch.exp(sink - m)
        out[i] = torch.einsum("hj,jhv->hv", e / den[:, None], v[lo:i + 1])
    return out


def latent_attention(h, weights, prefix, mixer, kind, eps):
    """The three latent mixers.  kind 'latent_attention': window, sink, gate; 'latent_attention_2': a rotated part,
    causal, sink, gate; 'latent_attention_3': window, ordinary softmax, no gate."""
    T = h.shape[0]
    H, D, V, R = mixer["heads"], mixer["dim"], mixer["vdim"], mixer["kv_rank"]
    r = int(mixer.get("rot_dim", 0) or 0)
    q = (h @ w64(weights, prefix + "q").T).reshape(T, H, D + r)
    down = h @ w64(weights, prefix + "dkv").T                                     # [T, R + r]
    c = down[:, :R]
    c = c / torch.sqrt(c.pow(2).mean(-1, keepdim=True) + eps) * w64(weights, prefix + "dkv.norm")
    k = (c @ w64(weights, prefix + "uk").T).reshape(T, H, D)
    v = (c @ w64(weights, prefix + "uv").T).reshape(T, H, V)
    if r:
        pos = torch.arange(T)
        rot = mixer["rot"]
        q_rot = rotate_half_split(q[..., D:], pos, rot["base"], int(rot["dims"]))
        k_rot = rotate_half_split(down[:, R:].reshape(T, 1, r), pos, rot["base"], int(rot["dims"]))
        q = torch.cat((q[..., :D], q_rot), dim=-1)
        k = torch.cat((k, k_rot.expand(T, H, r)), dim=-1)
    window = mixer["mask"]["size"] if mixer.get("mask") else None
    has_sink = kind in ("latent_attention", "latent_attention_2")
    sink = w64(weights, prefix + "sink") if has_sink else None
    o = sink_softmax_attention(q, k, v, float(mixer["scale"]), window, sink).reshape(T, H * V)
    if has_sink:                                                                  # these two kinds also gate their output
        o = o * torch.sigmoid(h @ w64(weights, prefix + "g").T)
    return o @ w64(weights, prefix + "o").T


def gated_expert(h, weights, prefix):
    g = h @ w64(weights, prefix + "gate").T
    return ((g * torch.sigmoid(g)) * (h @ w64(weights, prefix + "up").T)) @ w64(weights, prefix + "down").T


def route(h, router_weight, router):
    """-> (chosen experts [T, top], weights [T, top]).  Softmax over all experts; only experts of the ``keep`` groups
    with the largest best score can be chosen; the weights are the chosen scores times ``scale``."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    s = torch.softmax(h @ router_weight.T, dim=-1)                                 # [T, E]
    T = s.shape[0]
    per = E // groups["count"]
    best = s.reshape(T, groups["count"], per).max(dim=-1).values
    kept = torch.topk(best, groups["keep"], dim=-1).indices
    allowed = torch.zeros(T, groups["count"], dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    allowed = allowed[:, :, None].expand(T, groups["count"], per).reshape(T, E)
    chosen = torch.topk(torch.where(allowed, s, torch.full_like(s, -1.0)), top, dim=-1).indices
    return chosen, torch.gather(s, 1, chosen) * float(router.get("scale", 1.0))


def mixture(h, weights, prefix, mlp):
    chosen, gates = route(h, w64(weights, prefix + "router"), mlp["router"])
    out = torch.zeros(h.shape[0], w64(weights, prefix + "e0.down").shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), gates[t]):
            out[t] += g * gated_expert(h[t:t + 1], weights, f"{prefix}e{e}.")[0]
    if mlp.get("shared"):
        share = torch.sigmoid(h @ w64(weights, prefix + "shared.sg").T)          # [T, 1]
        out = out + share * gated_expert(h, weights, prefix + "shared.")
    return out


def forward(cfg, weights, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence from its first token (and the stream after every layer)."""
    eps, groups, m = float(cfg["norm"]["eps"]), int(cfg["norm"]["groups"]), float(cfg["residual_mult"])
    x = w64(weights, "embed")[torch.as_tensor(tokens, dtype=torch.long)]
    history = [x]                                                                 # X_0, X_1, ...
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = causal_conv_add(group_rms_norm(x, w64(weights, p + "norm1"), groups, eps), w64(weights, p + "canon1"))
        x = x + m * latent_attention(h, weights, p + "mix.", layer["mixer"], layer["type"], eps)
        if layer.get("mlp") is not None:
            h = causal_conv_add(group_rms_norm(x, w64(weights, p + "norm2"), groups, eps), w64(weights, p + "canon2"))
            x = x + m * mixture(h, weights, p + "mlp.", layer["mlp"])
        history.append(x)
        mix = w64(weights, p + "dwa")
        x = sum(mix[j] * history[j] for j in range(i + 2))
        after.append(x)
    logits = group_rms_norm(x, w64(weights, "final.norm"), groups, eps) @ w64(weights, "head").T
    return (logits, torch.stack(after)) if return_layers else logits


def greedy(cfg, weights, prompt, n):
    """The ``n`` tokens that follow ``prompt`` when the largest logit is always taken (the lowest index among equals);
    every token is computed from the whole sequence again."""
    toks = list(prompt)
    out = []
    for _ in range(n):
        nxt = int(torch.argmax(forward(cfg, weights, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
