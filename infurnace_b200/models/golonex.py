"""Golonex: the plan builder (configuration -> layers, order, tensor names).

A pre-norm decoder over a float32 residual stream.  The embedding's rows are normalised.  A layer is
x += mixer(norm1(x)), x += ffn(norm2(x)) where it has a feed-forward, then a per-layer token input (a slice of a second
table's row of the token, gated by gelu_tanh of a small product of the stream, projected back, divided by its root mean
square and added).  Three mixers, in any order given by config.json's ``layers``: ``rglru`` (the recurrent block around a
real-gated linear recurrent unit: a gelu branch beside a short causal convolution and a per-channel gated recurrence
whose gates are block-diagonal products); ``latent_attention`` (queries through a latent of their own; keys and values
from a small cached latent beside one rotated key part shared by the heads; sliding window, a sink in the softmax, one
output gate per head); ``attention`` (grouped-query attention whose values are its keys before rotation, rotated on part
of each head in the interleaved pairing with stretched slow frequencies, sliding window).  The feed-forward is a mixture
of gated experts chosen by sigmoid scores, which multiply what the expert READS, beside a shared expert with a per-token
gate.  A final norm, the embedding table as the head and a soft cap on the logits follow.  Tensor names: ``embed``,
``embed.norm``, ``side.embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.gate|up|down``,
``l<i>.mlp.shared.gate|up|down|sg``, ``l<i>.side.gate|proj|norm``, ``final.norm``.
"""
from __future__ import annotations

from ..config.golonex import ATTENTION, LATENT, RGLRU, GolonexConfig
from ..config.specs import (
    GatedMLPSpec, LatentAttentionSpec, LayerCall, LMHeadSpec, ModelPlan, NormedEmbeddingSpec, PreNormBlockSpec,
    RealGatedRecurrenceSpec, RMSNormSpec, RotarySpec, RotaryValueAttentionSpec, RoutedExpertsSpec, TokenSideSpec,
)
from .registry import register_architecture

MAX_POSITIONS = 1 << 20        # positions have no end in this design; block tables need one
EXPERT_ACTIVATION = "silu"
SIDE_ACTIVATION = "gelu_tanh"
DECAY_SCALE = 8.0              # log a = -8 * r * softplus(lam)
WEIGHT_TERMS = 2               # softmax weights and the recurrence's gates are 32-bit in this design: on tensor cores they (and what
                               # the gates read) enter their products as two bfloat16 terms


def _rotary(rot, width):
    sc = rot.get("scaling")
    scaling = (float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"])) if sc else None
    return RotarySpec(width, int(rot["dims"]), float(rot["base"]), interleaved=True, scaling=scaling, frequency_dtype="float64")


def _window(m):
    return int(m["mask"]["size"]) if m.get("mask") else None


def _mixer(kind, m, p, W, eps):
    if kind == RGLRU:
        return RealGatedRecurrenceSpec(
            hidden_size=W, width=m["width"], blocks=m["blocks"], taps=m["conv"], decay_scale=DECAY_SCALE, y_proj=p + "y",
            y_bias=p + "y.b", x_proj=p + "x", x_bias=p + "x.b", conv=p + "conv", conv_bias=p + "conv.b", a_gate=p + "ra",
            a_bias=p + "ra.b", x_gate=p + "ri", x_bias_gate=p + "ri.b", decay=p + "lam", o_proj=p + "o", gate_terms=WEIGHT_TERMS)
    if kind == LATENT:
        rot_dim = int(m.get("rot_dim") or 0)
        return LatentAttentionSpec(
            hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], rot_dim=rot_dim, value_head_dim=m["vdim"],
            kv_rank=m["kv_rank"], scale=float(m["scale"]), eps=eps, q_proj=p + "uq", down_proj=p + "dkv",
            latent_norm=p + "dkv.norm", k_up=p + "uk", v_up=p + "uv", o_proj=p + "o",
            position=_rotary(m["rot"], rot_dim) if rot_dim else None, window=_window(m), sink=p + "sink", gate=p + "g",
            gate_per_head=True, q_rank=m["q_rank"], q_down=p + "dq", q_norm=p + "dq.norm", weight_terms=WEIGHT_TERMS)
    assert kind == ATTENTION
    return RotaryValueAttentionSpec(
        hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], value_head_dim=m["dim"],
        scale=float(m["scale"]), eps=eps, q_proj=p + "q", k_proj=p + "k", v_proj=None, o_proj=p + "o",
        position=_rotary(m["rot"], m["dim"]) if m.get("rot") else None, window=_window(m), weight_terms=WEIGHT_TERMS)


def _mlp(mlp, p, W):
    router, shared = mlp["router"], mlp.get("shared")
    return RoutedExpertsSpec(
        W, mlp["expert"]["ff"], router["top"], EXPERT_ACTIVATION, p + "router",
        tuple((f"{p}e{j}.gate", f"{p}e{j}.up", f"{p}e{j}.down") for j in range(router["experts"])),
        scoring="sigmoid", weight_on="input",
        shared=GatedMLPSpec(W, shared["ff"], EXPERT_ACTIVATION, p + "shared.gate", p + "shared.up", p + "shared.down") if shared else None,
        shared_gate=p + "shared.sg" if shared else None)


def build_golonex_plan(cfg: GolonexConfig) -> ModelPlan:
    W, eps, V = cfg.hidden_size, cfg.norm_eps, cfg.vocab_size
    n = len(cfg.layers)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        has_ffn = layer["mlp"] is not None
        side = None
        if cfg.token_side_dim is not None:
            sd = cfg.token_side_dim
            side = TokenSideSpec(W, sd, V, "side.embed", n * sd, i * sd, SIDE_ACTIVATION, p + "side.gate", p + "side.proj",
                                 RMSNormSpec(W, eps, p + "side.norm"))
        layers.append(PreNormBlockSpec(
            mixer_norm=RMSNormSpec(W, eps, p + "norm1"), mixer=_mixer(layer["type"], layer["mixer"], p + "mix.", W, eps),
            ffn_norm=RMSNormSpec(W, eps, p + "norm2") if has_ffn else None, ffn=_mlp(layer["mlp"], p + "mlp.", W) if has_ffn else None,
            side=side, unused=() if has_ffn else ((p + "norm2", W),)))
    return ModelPlan(
        architecture=cfg.architecture, vocab_size=V, hidden_size=W, max_positions=MAX_POSITIONS,
        embedding=NormedEmbeddingSpec(V, W, "embed", RMSNormSpec(W, eps, "embed.norm")), layers=tuple(layers),
        schedule=tuple(LayerCall(i) for i in range(n)), final_norm=RMSNormSpec(W, eps, "final.norm"),
        lm_head=LMHeadSpec(V, W, "embed", tied=True, softcap=cfg.logit_softcap))


register_architecture("Golonex", GolonexConfig, build_golonex_plan)
