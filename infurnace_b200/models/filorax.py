"""Filorax: the plan builder (configuration -> layers, order, tensor names).

A pre-norm decoder over a float32 residual stream.  Every norm works in groups (the row in equal parts, each with its
own statistic).  A layer is x += m * mixer(conv1(norm1(x))), x += m * ffn(conv2(norm2(x))) with m one number for the whole
model and conv a short causal convolution over time that is added to its input (its last inputs are part of a
sequence's state); what goes on to the next layer is a weighted average over the embedding's output and the results of
all layers so far.  The mixers, in any order given by config.json's ``layers``, are three kinds of attention whose keys
and values come from a small cached latent: with a sliding window, a sink in the softmax and an output gate
(``latent_attention``); with a rotated key part shared by the heads, causal, sink and gate (``latent_attention_2``); with
a window and the ordinary softmax (``latent_attention_3``).  The feed-forward is a mixture of gated experts whose scores
are the softmax over all experts, chosen within the best groups of neighbouring experts, beside a shared expert with a
per-token gate.  A final norm and an untied head follow.  Tensor names: ``embed``, ``l<i>.norm1|norm2``,
``l<i>.canon1|canon2``, ``l<i>.dwa``, ``l<i>.mix.q|dkv|dkv.norm|uk|uv|sink|g|o``, ``l<i>.mlp.router``,
``l<i>.mlp.e<j>.gate|up|down``, ``l<i>.mlp.shared.gate|up|down|sg``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.filorax import ROTATED_SINK_GATE, WINDOW_PLAIN, FiloraxConfig
from ..config.specs import (
    CausalConvSpec, DepthAverageBlockSpec, EmbeddingSpec, GatedMLPSpec, GroupRMSNormSpec, LatentAttentionSpec, LayerCall,
    LMHeadSpec, ModelPlan, RotarySpec, RoutedExpertsSpec,
)
from .registry import register_architecture

MAX_POSITIONS = 1 << 20        # positions have no end in this design; block tables need one
EXPERT_ACTIVATION = "silu"


def _mixer(kind, m, p, W, eps):
    rot_dim = int(m.get("rot_dim") or 0)
    position = None
    if rot_dim:
        position = RotarySpec(rot_dim, int(m["rot"]["dims"]), float(m["rot"]["base"]))
    plain = kind == WINDOW_PLAIN                      # the ordinary softmax, no gate
    return LatentAttentionSpec(
        hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], rot_dim=rot_dim, value_head_dim=m["vdim"], kv_rank=m["kv_rank"],
        scale=float(m["scale"]), eps=eps, q_proj=p + "q", down_proj=p + "dkv", latent_norm=p + "dkv.norm", k_up=p + "uk",
        v_up=p + "uv", o_proj=p + "o", position=position, window=int(m["mask"]["size"]) if m.get("mask") else None,
        sink=None if plain else p + "sink", gate=None if plain else p + "g")


def _mlp(mlp, p, W):
    router = mlp["router"]
    groups = router.get("groups")
    shared = mlp.get("shared")
    return RoutedExpertsSpec(
        W, mlp["expert"]["ff"], router["top"], EXPERT_ACTIVATION, p + "router",
        tuple((f"{p}e{j}.gate", f"{p}e{j}.up", f"{p}e{j}.down") for j in range(router["experts"])),
        scoring="all", weight_scale=float(router["scale"]) if router.get("scale") is not None else 1.0,
        groups=(int(groups["count"]), int(groups["keep"])) if groups else None,
        shared=GatedMLPSpec(W, shared["ff"], EXPERT_ACTIVATION, p + "shared.gate", p + "shared.up", p + "shared.down") if shared else None,
        shared_gate=p + "shared.sg" if shared else None)


def build_filorax_plan(cfg: FiloraxConfig) -> ModelPlan:
    W, eps, V, G = cfg.hidden_size, cfg.norm_eps, cfg.vocab_size, cfg.norm_groups
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        has_ffn = layer["mlp"] is not None
        layers.append(DepthAverageBlockSpec(
            hidden_size=W, depth=i, depths=len(cfg.layers), residual_mult=cfg.residual_mult,
            mixer_norm=GroupRMSNormSpec(W, eps, G, p + "norm1"), mixer=_mixer(layer["type"], layer["mixer"], p + "mix.", W, eps),
            mixer_conv=CausalConvSpec(W, cfg.conv_taps, p + "canon1"),
            ffn_norm=GroupRMSNormSpec(W, eps, G, p + "norm2") if has_ffn else None,
            ffn=_mlp(layer["mlp"], p + "mlp.", W) if has_ffn else None,
            ffn_conv=CausalConvSpec(W, cfg.conv_taps, p + "canon2") if has_ffn else None,
            average=p + "dwa"))
    return ModelPlan(
        architecture=cfg.architecture, vocab_size=V, hidden_size=W, max_positions=MAX_POSITIONS,
        embedding=EmbeddingSpec(V, W, "embed"), layers=tuple(layers), schedule=tuple(LayerCall(i) for i in range(len(layers))),
        final_norm=GroupRMSNormSpec(W, eps, G, "final.norm"), lm_head=LMHeadSpec(V, W, "head", tied=False))


register_architecture("Filorax", FiloraxConfig, build_filorax_plan)
