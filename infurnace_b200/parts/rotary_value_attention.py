"""Softmax attention over the paged cache whose values are normalised and rotated by their position."""
from __future__ import annotations

import torch

from ..config.specs import RotaryValueAttentionSpec
from .registry import build_part, register_part


class RotaryValueAttention:
    """h -> o_proj(unrotate(attention(q, K, V))).

    q | k | v run as one product (q | k where the description has no value projection: a value head is then its key head
    as projected, before the rotation).  One kernel rotates the q and k heads on their first rotary_dim entries, divides
    each value head by its root mean square and rotates it over its whole width by the token's position, writes q
    in the cache's dtype and k and v into their page streams (which may differ in width).  The attention kernel reads
    every key and value from the pages, this step's included, keeps scores, softmax weights and sums in float32,
    and rotates each head's summed output back by the query's position before it stores it.  The angles come from
    the rotary parts' per-step tables (cosine and sine of every token's angles, float32)."""

    graph_safe = True

    def __init__(self, spec: RotaryValueAttentionSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        self.values_are_keys = spec.v_proj is None
        if self.values_are_keys and (spec.value_head_dim != spec.head_dim or spec.value_norm or spec.value_position is not None):
            raise ValueError("values that are the keys have the keys' width, no norm and no rotation of their own")
        names = (spec.q_proj, spec.k_proj) if self.values_are_keys else (spec.q_proj, spec.k_proj, spec.v_proj)
        self.w_qkv = torch.cat([weights[n] for n in names], dim=0).contiguous()
        self.w_o = weights[spec.o_proj]
        self.position = build_part(spec.position, weights, runtime) if spec.position is not None else None
        self.value_position = build_part(spec.value_position, weights, runtime) if spec.value_position is not None else None
        if self.value_position is not None and spec.value_position.rotary_dim != spec.value_head_dim:
            raise ValueError("the values are rotated over their whole width")
        import os
        self.exact_weights = os.environ.get("INFURNACE_EXACT_ATTENTION", "0") not in ("", "0")
        self.width = spec.num_heads * spec.head_dim + spec.num_kv_heads * (
            spec.head_dim + (0 if self.values_are_keys else spec.value_head_dim))

    def _on_tensor_cores(self, kv):
        """bfloat16 with keys and values of one width in one tensor: the framework's tensor-core attention kernels run
        (scores and softmax in float32; the weights are rounded to bfloat16 as the left operand of the P V product, which
        accumulates in float32).  Everything else, and every step when ``exact_weights`` is set, runs the plain kernel,
        which keeps the weights in float32 through the sum."""
        s = self.spec
        group = s.num_heads // s.num_kv_heads
        return (not self.exact_weights and self.rt.act_dtype == torch.bfloat16 and kv.pages is not None
                and s.head_dim == s.value_head_dim and s.head_dim % 16 == 0 and s.head_dim <= 256 and group <= 16
                and hasattr(self.k, "rotate_rows"))

    def forward(self, h, ctx, call):
        s, k = self.spec, self.k
        n = h.shape[0]
        qkv = ctx.buffer("rva_qkv", (n, self.width), torch.float32)
        k.linear(h, self.w_qkv, qkv)
        kv = ctx.kv(call.cache)
        pk, pv = kv.streams["k"], kv.streams["v"]
        q = ctx.buffer("rva_q", (n, s.num_heads * s.head_dim), self.rt.act_dtype)
        qk_table = self.position.table(ctx) if self.position is not None else None
        v_table = self.value_position.table(ctx) if self.value_position is not None else None
        k.rotary_store(qkv, s.num_heads, s.num_kv_heads, s.head_dim, s.value_head_dim, qk_table,
                       s.position.rotary_dim if s.position is not None else 0,
                       bool(s.position.interleaved) if s.position is not None else False,
                       s.eps if s.value_norm else None, v_table,
                       bool(s.value_position.interleaved) if s.value_position is not None else False,
                       q, pk, pv, kv.slot_mapping if call.store else None, **({"values_are_keys": True} if self.values_are_keys else {}))
        out = ctx.buffer("rva_out", (n, s.num_heads * s.value_head_dim), self.rt.act_dtype)
        if self._on_tensor_cores(kv):
            # the framework's tensor-core attention over the entry's one tensor of keys and values, then the turn back
            k.paged_attention(q, s.num_heads, s.num_kv_heads, s.head_dim, kv.pages, kv.block_tables, ctx.cu_q, ctx.seq_lens, out,
                              s.scale, s.window or 0, ctx.max_q_len, ctx.max_seq_len, min_q_len=ctx.min_q_len,
                              **({"weight_terms": s.weight_terms} if s.weight_terms != 1 else {}))
            if v_table is not None:
                k.rotate_rows(out, v_table, s.num_heads, s.value_head_dim, s.value_head_dim, bool(s.value_position.interleaved),
                              back=True)
        else:
            k.paged_attention_streams(q, s.num_heads, s.num_kv_heads, s.head_dim, s.value_head_dim, pk, pv, kv.block_tables,
                                      ctx.cu_q, ctx.seq_lens, out, s.scale, s.window or 0, v_table,
                                      bool(s.value_position.interleaved) if s.value_position is not None else False,
                                      max_q_len=ctx.max_q_len, max_seq_len=ctx.max_seq_len)
        delta = ctx.buffer("delta_mixer", (n, s.hidden_size), torch.float32)
        k.linear(out, self.w_o, delta)
        return delta


register_part(RotaryValueAttentionSpec, RotaryValueAttention)
