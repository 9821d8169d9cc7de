"""Softmax attention whose keys and values come from a small cached latent."""
from __future__ import annotations

import torch

from ..config.specs import LatentAttentionSpec
from .registry import build_part, register_part


class LatentAttention:
    """h -> o_proj(gate * concat_h UV_h (sum_j p_hj c_j)), p_h = softmax_j(scale * ((UK_h^T q_h) . c_j + q_rot_h . k_rot_j)).

    The keys k_h = UK_h c and values v_h = UV_h c of the context are never formed: q_h . (UK_h c) = (UK_h^T q_h) . c, and
    the weighted sum of values is UV_h applied to the weighted sum of latents.  So the pages hold the normalised latent
    (and the small rotated key part shared by the heads) and nothing else, every head of a token attends over the same
    rows, and a step's cost in memory traffic is the latents' bytes whatever the number of heads.

    A step: one product q | latent, rotated key | gate against the concatenated matrices (float32 out); one kernel that
    normalises the latent, turns the rotated parts by the token's angles, stores latent and rotated key in their page
    streams and lays the heads' unrotated query parts out head-major; a grouped product over the heads with UK_h^T
    (the framework's grouped product, a head being what an expert is there); the attention kernel over the pages, this
    step's tokens included, with window and sink; a grouped product with UV_h; one kernel that applies the output gate
    and puts the heads side by side; the output product.  Where the queries have a latent of their own, they are two more
    products with an RMS norm between them, and the first product holds latent, rotated key | gate only."""

    graph_safe = True

    def __init__(self, spec: LatentAttentionSpec, weights, runtime):
        self.spec = s = spec
        self.rt = runtime
        self.k = runtime.kernels
        H, D, V, R = s.num_heads, s.head_dim, s.value_head_dim, s.kv_rank
        # with a latent of their own the queries are two products with a norm between them, and the step's first product
        # holds latent, rotated key | gate only
        self.q_latent = bool(s.q_rank)
        parts = [weights[s.down_proj]] if self.q_latent else [weights[s.q_proj], weights[s.down_proj]]
        if s.gate is not None:
            parts.append(weights[s.gate])
        self.w_in = torch.cat(parts, dim=0).contiguous()
        if self.q_latent:
            self.w_q_down, self.w_q_up, self.q_norm_w = weights[s.q_down], weights[s.q_proj], weights[s.q_norm]
        self.down_col = 0 if self.q_latent else H * (D + s.rot_dim)
        self.gate_col = self.down_col + R + s.rot_dim
        self.gate_width = H if s.gate_per_head else H * V
        self.norm_w = weights[s.latent_norm]
        # UK_h^T as the matrix of a product x W^T: [heads, rank, dim]; UV_h as it is stored: [heads, vdim, rank]
        self.w_absorb = weights[s.k_up].view(H, D, R).transpose(1, 2).contiguous()
        self.w_values = weights[s.v_up].view(H, V, R).contiguous()
        self.w_o = weights[s.o_proj]
        self.sink = weights[s.sink] if s.sink is not None else None
        self.position = build_part(s.position, weights, runtime) if s.position is not None else None
        import os
        self.exact_weights = os.environ.get("INFURNACE_EXACT_ATTENTION", "0") not in ("", "0")
        self.terms = {"weight_terms": s.weight_terms} if s.weight_terms != 1 else {}

    def _segment(self, n):
        """Rows of a head's segment in the grouped products, and the tile of the tcgen05 route (0: the other route)."""
        k, s = self.k, self.spec
        ok = getattr(k, "moe_grouped_tc_ok", None)
        if ok is not None and ok(n * s.num_heads, self.rt.act_dtype, self.w_absorb, self.w_values):
            t = k.MOE_TILE
            return -(-n // t) * t, t
        return n, 0

    def forward(self, h, ctx, call):
        s, k = self.spec, self.k
        n = h.shape[0]
        H, D, V, R, r = s.num_heads, s.head_dim, s.value_head_dim, s.kv_rank, s.rot_dim
        act = self.rt.act_dtype
        proj = ctx.buffer("la_proj", (n, self.w_in.shape[0]), torch.float32)
        k.linear(h, self.w_in, proj)
        q = None
        if self.q_latent:
            cq_raw = ctx.buffer("la_cq_raw", (n, s.q_rank), torch.float32)
            k.linear(h, self.w_q_down, cq_raw)
            cq = ctx.buffer("la_cq", (n, s.q_rank), act)
            k.rmsnorm(cq_raw, self.q_norm_w, s.eps, cq)
            q = ctx.buffer("la_q", (n, H * (D + r)), torch.float32)
            k.linear(cq, self.w_q_up, q)
        extra = {}
        if q is not None:
            extra["q"] = q
        if s.position is not None and s.position.interleaved:
            extra["interleaved"] = True
        kv = ctx.kv(call.cache)
        lat_pages = kv.streams["latent"]
        rot_pages = kv.streams["rotated_key"] if r else None
        seg, tile = self._segment(n)
        cap, _ = self._segment(ctx.max_rows)
        q_plain = ctx.buffer("la_q_plain", (H * seg, D), act, rows=H * cap).view(H, seg, D)
        q_rot = ctx.buffer("la_q_rot", (n, H, r), torch.float32) if r else None
        offsets = ctx.buffer("la_offsets", (H + 1,), torch.int32, rows=H + 1)
        tiles = ctx.buffer("la_tiles", (H * seg // tile,), torch.int32, rows=H * cap // tile) if tile else None
        table = self.position.table(ctx) if self.position is not None else None
        k.latent_prepare(proj, H, D, r, R, self.down_col, self.norm_w, s.eps, table, s.position.rotary_dim if table is not None else 0,
                         q_plain, q_rot, lat_pages, rot_pages, kv.slot_mapping if call.store else None, offsets, tiles, tile, **extra)
        q_lat = ctx.buffer("la_q_lat", (H * seg, R), torch.float32, rows=H * cap)
        if tile:
            k.moe_linear_grouped(q_plain.view(H * seg, D), self.w_absorb, tiles, q_lat)
        else:
            k.moe_linear(q_plain.view(H * seg, D), self.w_absorb, offsets, None, 1, q_lat)
        o_lat = ctx.buffer("la_o_lat", (H * seg, R), act, rows=H * cap)
        k.latent_attention(q_lat.view(H, seg, R), q_rot, lat_pages, rot_pages, kv.block_tables, ctx.cu_q, ctx.seq_lens, ctx.req_index,
                           self.sink, o_lat.view(H, seg, R), s.scale, s.window or 0, n, max_q_len=ctx.max_q_len,
                           max_seq_len=ctx.max_seq_len, exact=self.exact_weights, **self.terms)
        y = ctx.buffer("la_y", (H * seg, V), torch.float32, rows=H * cap)
        if tile:
            k.moe_linear_grouped(o_lat, self.w_values, tiles, y)
        else:
            k.moe_linear(o_lat, self.w_values, offsets, None, 1, y)
        out = ctx.buffer("la_out", (n, H * V), act)
        gate = proj[:, self.gate_col:self.gate_col + self.gate_width] if s.gate is not None else None
        if s.gate_per_head and gate is not None:
            k.gate_heads(y.view(H, seg, V), gate, out, n, per_head=True)
        else:
            k.gate_heads(y.view(H, seg, V), gate, out, n)
        delta = ctx.buffer("delta_mixer", (n, s.hidden_size), torch.float32)
        k.linear(out, self.w_o, delta)
        return delta


register_part(LatentAttentionSpec, LatentAttention)
