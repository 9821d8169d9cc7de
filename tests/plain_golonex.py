"""The Golonex decoder, stated plainly: one function per mechanism, float64, whole sequences, no cache.

It shares no code with the package.  ``weights`` maps tensor names to tensors; ``cfg`` is config.json as a mapping.
A sequence is run from its first token; every function takes [T, ...] tensors of one sequence.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def w64(weights, name):
    return weights[name].to(F64)


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis (weight None: no weight)."""
    y = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_frequencies(rot):
    """(frequency of every rotated pair, the factor on cosine and sine)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    freq = base ** (-2.0 * i / dims)
    scaling = rot.get("scaling")
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(v, rot):
    """v [T, heads, d]: entries 2i and 2i + 1 (i < dims / 2) of every head turned by position * frequency_i."""
    dims = int(rot["dims"])
    freq, gain = rotary_frequencies(rot)
    angle = torch.arange(v.shape[0], dtype=F64)[:, None] * freq[None, :]
    c, s = (torch.cos(angle) * gain)[:, None, :], (torch.sin(angle) * gain)[:, None, :]
    out = v.clone()
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def softmax_attention(q, k, v, scale, window, sink=None):
    """q, k [T, H, d], v [T, H, dv].  Position i sees j with 0 <= i - j < window (window None: every j <= i).  ``sink``
    [H]: exp(sink) joins the denominator and nothing else."""
    T = q.shape[0]
    out = torch.zeros(T, q.shape[1], v.shape[2], dtype=F64)
    for i in range(T):
        first = 0 if window is None else max(0, i - window + 1)
        s = torch.einsum("hd,jhd->hj", q[i], k[first:i + 1]) * scale
        top = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            top = torch.maximum(top, sink[:, None])
        e = torch.exp(s - top)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[:, None] - top)
        out[i] = torch.einsum("hj,jhv->hv", e / den, v[first:i + 1])
    return out


def window_of(m):
    return int(m["mask"]["size"]) if m.get("mask") else None


def grouped_attention(h, weights, p, m):
    """Grouped-query attention whose values are its keys as projected (before the rotation)."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w64(weights, p + "q").T).view(T, H, D)
    k = (h @ w64(weights, p + "k").T).view(T, G, D)
    v = k
    if m.get("rot"):
        q, k = rotate_pairs(q, m["rot"]), rotate_pairs(k, m["rot"])
    rep = H // G
    o = softmax_attention(q, k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1), float(m["scale"]), window_of(m))
    return o.reshape(T, -1) @ w64(weights, p + "o").T


def latent_attention(h, weights, p, m, eps):
    """Queries through a latent; keys and values from a latent c, beside one rotated key part shared by the heads."""
    T = h.shape[0]
    H, D, R, V, rank = m["heads"], m["dim"], int(m.get("rot_dim") or 0), m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ w64(weights, p + "dq").T, w64(weights, p + "dq.norm"), eps)
    q = (cq @ w64(weights, p + "uq").T).view(T, H, D + R)
    down = h @ w64(weights, p + "dkv").T
    c = rms_norm(down[:, :rank], w64(weights, p + "dkv.norm"), eps)
    k = (c @ w64(weights, p + "uk").T).view(T, H, D)
    v = (c @ w64(weights, p + "uv").T).view(T, H, V)
    if R:
        shared = rotate_pairs(down[:, rank:].view(T, 1, R), m["rot"])
        q = torch.cat((q[..., :D], rotate_pairs(q[..., D:], m["rot"])), dim=-1)
        k = torch.cat((k, shared.expand(T, H, R)), dim=-1)
    o = softmax_attention(q, k, v, float(m["scale"]), window_of(m), w64(weights, p + "sink"))
    gate = torch.sigmoid(h @ w64(weights, p + "g").T)                              # [T, H]
    return (o * gate[:, :, None]).reshape(T, H * V) @ w64(weights, p + "o").T


def short_convolution(x, taps_weight, bias):
    """u_t = bias + sum_j w[:, j] * x_(t - taps + 1 + j): the last column is the current token's; zeros before the start."""
    T = x.shape[0]
    taps = taps_weight.shape[1]
    u = bias.expand(T, -1).clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                u[t] += taps_weight[:, j] * x[s]
    return u


def block_diagonal(u, matrices, bias):
    """u [T, width] in ``blocks`` equal parts, part b through matrices[b] ([out, in]) plus bias[b]."""
    T = u.shape[0]
    B = matrices.shape[0]
    parts = u.view(T, B, -1)
    return (torch.einsum("boi,tbi->tbo", matrices, parts) + bias).reshape(T, -1)


def real_gated_recurrence(r, i, u, lam, scale=8.0):
    """S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t from S = 0, a_t = exp(-scale * r_t * softplus(lam))."""
    a = torch.exp(-scale * r * torch.nn.functional.softplus(lam))
    S = torch.zeros(u.shape[1], dtype=F64)
    out = []
    for t in range(u.shape[0]):
        S = a[t] * S + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out.append(S)
    return torch.stack(out)


def recurrent_block(h, weights, p, m):
    y = gelu_tanh(h @ w64(weights, p + "y").T + w64(weights, p + "y.b"))
    u = short_convolution(h @ w64(weights, p + "x").T + w64(weights, p + "x.b"), w64(weights, p + "conv"), w64(weights, p + "conv.b"))
    r = torch.sigmoid(block_diagonal(u, w64(weights, p + "ra"), w64(weights, p + "ra.b")))
    i = torch.sigmoid(block_diagonal(u, w64(weights, p + "ri"), w64(weights, p + "ri.b")))
    S = real_gated_recurrence(r, i, u, w64(weights, p + "lam"))
    return (S * y) @ w64(weights, p + "o").T


def gated_expert(h, weights, p):
    a = h @ w64(weights, p + "gate").T
    return (a * torch.sigmoid(a) * (h @ w64(weights, p + "up").T)) @ w64(weights, p + "down").T


def route(h, router, top):
    """(chosen experts [T, top], their weights): sigmoid scores, the ``top`` largest (the lower index among equals), the
    scores themselves as weights."""
    score = torch.sigmoid(h @ router.T)
    order = torch.sort(score, dim=-1, descending=True, stable=True)
    return order.indices[:, :top], order.values[:, :top]


def mixture(h, weights, p, mlp):
    chosen, weight = route(h, w64(weights, p + "router"), int(mlp["router"]["top"]))
    out = torch.zeros(h.shape[0], w64(weights, p + "e0.down").shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            out[t] += gated_expert((g * h[t])[None, :], weights, f"{p}e{e}.")[0]           # the weight goes into the input
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w64(weights, p + "shared.sg").T) * gated_expert(h, weights, p + "shared.")
    return out


def token_side(x, ids, weights, p, layer, dim, eps):
    e = w64(weights, "side.embed")[ids][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w64(weights, p + "side.gate").T) * e) @ w64(weights, p + "side.proj").T
    return rms_norm(y, w64(weights, p + "side.norm"), eps)


def forward(cfg, weights, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence from its first token (and the stream after every layer)."""
    eps = float(cfg["norm"]["eps"])
    ids = torch.as_tensor(tokens, dtype=torch.long)
    side = cfg["token_side"]["dim"] if cfg.get("token_side") else None
    x = rms_norm(w64(weights, "embed")[ids], w64(weights, "embed.norm"), eps)
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p, kind, m = f"l{i}.", layer["type"], layer["mixer"]
        h = rms_norm(x, w64(weights, p + "norm1"), eps)
        if kind == "rglru":
            x = x + recurrent_block(h, weights, p + "mix.", m)
        elif kind == "latent_attention":
            x = x + latent_attention(h, weights, p + "mix.", m, eps)
        elif kind == "attention":
            x = x + grouped_attention(h, weights, p + "mix.", m)
        else:
            raise ValueError(kind)
        if layer.get("mlp") is not None:
            x = x + mixture(rms_norm(x, w64(weights, p + "norm2"), eps), weights, p + "mlp.", layer["mlp"])
        if side is not None:
            x = x + token_side(x, ids, weights, p, i, side, eps)
        after.append(x)
    logits = rms_norm(x, w64(weights, "final.norm"), eps) @ w64(weights, "embed").T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
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
