"""Recurrent mixers whose state lives in the request's state slot: the HGRN2 gated recurrence, retention with a fixed
decay per head, RWKV-style time mixing (all three a matrix state per head), the element-wise minGRU and the real-gated
linear recurrent unit behind a short convolution."""
from __future__ import annotations

import torch

from ..config.specs import GatedRecurrenceSpec, GatedUnitSpec, RealGatedRecurrenceSpec, RetentionSpec, TimeMixSpec
from .registry import register_part


class GatedRecurrence:
    """h -> o_proj(norm(S^T q)) with S <- diag(f) S + (1 - f) v^T per head.

    The three projections run as one product against their row-wise concatenation (exact) into float32, because
    everything that enters the recurrence is 32-bit.  One kernel then applies silu to q and the gate formula to f,
    walks this step's tokens of every request in order from the state its slot holds (zero when the slot was
    granted), writes the state back and normalises each head's output.  A whole prompt, a portion and a single
    decoded token are the same call: the state carries what came before."""

    graph_safe = True     # launches depend on the step's sizes only

    def __init__(self, spec: GatedRecurrenceSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        self.w_qfv = torch.cat((weights[spec.q_proj], weights[spec.f_proj], weights[spec.v_proj]), dim=0).contiguous()
        self.w_o = weights[spec.o_proj]
        self.bias, self.lower, self.norm_w = weights[spec.f_bias], weights[spec.lower], weights[spec.out_norm]
        self.hd = spec.num_heads * spec.head_dim
        self.hv = spec.num_heads * spec.value_head_dim
        slabs = getattr(self.k, "gated_scan_slabs", None)
        self.slabs = slabs(spec.head_dim, spec.value_head_dim) if slabs else 1

    def forward(self, h, ctx, call):
        s, k = self.spec, self.k
        n = h.shape[0]
        proj = ctx.buffer("gr_proj", (n, 2 * self.hd + self.hv), torch.float32)
        k.linear(h, self.w_qfv, proj)
        out = ctx.buffer("gr_out", (n, self.hv), self.rt.act_dtype)
        raw = ctx.buffer("gr_raw", (n, self.hv), torch.float32) if self.slabs > 1 else None
        k.gated_scan(proj, 0, self.hd, 2 * self.hd, self.bias, self.lower, self.norm_w, s.eps, ctx.state(call.cache),
                     ctx.state_slots, ctx.cu_q, ctx.seq_lens, out, s.num_heads, s.head_dim, s.value_head_dim, raw=raw,
                     max_q_len=ctx.max_q_len)
        delta = ctx.buffer("delta_mixer", (n, s.hidden_size), torch.float32)
        k.linear(out, self.w_o, delta)
        return delta


register_part(GatedRecurrenceSpec, GatedRecurrence)


class Retention:
    """h -> o_proj(unit_norm(S^T q) * silu(G h)) with S <- decay_h S + (k * key_scale) v^T per head.

    q | k | v | g run as one product into float32 (what enters the recurrence is 32-bit).  The recurrence kernel is
    the framework's walk of a matrix state per head (``linear_scan``) with a constant decay per head; it divides each
    head's output by its root mean square and multiplies by silu of the gate columns before it writes the rows that
    ``o_proj`` reads.  A prompt, a portion and a decoded token are the same call: the slot's state carries the past."""

    graph_safe = True

    def __init__(self, spec: RetentionSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        self.w_all = torch.cat([weights[n] for n in (spec.q_proj, spec.k_proj, spec.v_proj, spec.g_proj)], dim=0).contiguous()
        self.w_o = weights[spec.o_proj]
        self.decay = torch.tensor(spec.decay, dtype=torch.float32, device=runtime.device)
        self.hd = spec.num_heads * spec.head_dim
        self.hv = spec.num_heads * spec.value_head_dim

    def forward(self, h, ctx, call):
        s, k, hd, hv = self.spec, self.k, self.hd, self.hv
        n = h.shape[0]
        proj = ctx.buffer("ret_proj", (n, 2 * hd + 2 * hv), torch.float32)
        k.linear(h, self.w_all, proj)
        out = ctx.buffer("ret_out", (n, hv), self.rt.act_dtype)
        k.linear_scan(proj[:, :hd], proj[:, hd:2 * hd], proj[:, 2 * hd:2 * hd + hv], None, s.num_heads, s.head_dim,
                      s.value_head_dim, ctx.state(call.cache), ctx.state_slots, ctx.cu_q, ctx.seq_lens, out, s.eps,
                      decay=self.decay, key_scale=s.key_scale, gate=proj[:, 2 * hd + hv:], max_q_len=ctx.max_q_len)
        delta = ctx.buffer("delta_mixer", (n, s.hidden_size), torch.float32)
        k.linear(out, self.w_o, delta)
        return delta


register_part(RetentionSpec, Retention)


class TimeMix:
    """RWKV-style time mixing over two cache entries: the matrix state per head, and the previous token's input.

    One kernel forms the five blends of each token with the one before it (the slot's saved row for the first token
    of a step) and saves the step's last row.  r, k, v, g and the decay's bottleneck read their blends through the
    framework's products (into float32; the bottleneck's tanh is its product's epilogue); the recurrence kernel
    turns the raw decay into exp(-exp(. + w0)), reads each output from the state BEFORE the token's update with the
    bonus on the token's own k v^T, and finishes with the per-head unit norm, the stored norm weight and the gate."""

    graph_safe = True

    def __init__(self, spec: TimeMixSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        self.mu = torch.stack([weights[n].to(torch.float32) for n in spec.mu], dim=0).contiguous()
        self.w_r, self.w_k, self.w_v, self.w_g = (weights[n] for n in (spec.r_proj, spec.k_proj, spec.v_proj, spec.g_proj))
        self.w1, self.w2, self.w0 = weights[spec.w1], weights[spec.w2], weights[spec.w0]
        self.rank = self.w1.shape[0]
        self.bonus = weights[spec.bonus].reshape(-1).contiguous()
        self.norm_w = weights[spec.out_norm]
        self.w_o = weights[spec.o_proj]
        self.hd = spec.num_heads * spec.head_dim

    def forward(self, h, ctx, call):
        s, k, hd = self.spec, self.k, self.hd
        n, W = h.shape
        mixes = ctx.buffer("tm_mixes", (5 * n, W), self.rt.act_dtype).view(5, n, W)
        k.token_shift_mix(h, ctx.state((call.cache, 1)), ctx.state_slots, ctx.cu_q, ctx.seq_lens, self.mu, mixes)
        proj = [ctx.buffer("tm_" + name, (n, hd), torch.float32) for name in ("r", "k", "v", "g", "w")]
        for j, w in enumerate((self.w_r, self.w_k, self.w_v, self.w_g)):
            k.linear(mixes[j], w, proj[j])
        low = ctx.buffer("tm_low", (n, self.rank), self.rt.act_dtype)
        k.linear(mixes[4], self.w1, low, epilogue="tanh")
        k.linear(low, self.w2, proj[4])
        out = ctx.buffer("tm_out", (n, hd), self.rt.act_dtype)
        k.linear_scan(proj[0], proj[1], proj[2], proj[4], s.num_heads, s.head_dim, s.head_dim, ctx.state((call.cache, 0)),
                      ctx.state_slots, ctx.cu_q, ctx.seq_lens, out, s.eps, w_bias=self.w0, bonus=self.bonus,
                      norm_weight=self.norm_w, gate=proj[3], max_q_len=ctx.max_q_len)
        delta = ctx.buffer("delta_mixer", (n, s.hidden_size), torch.float32)
        k.linear(out, self.w_o, delta)
        return delta


register_part(TimeMixSpec, TimeMix)


class GatedUnit:
    """minGRU: z | x | g run as one product into float32; one kernel adds the biases, forms gate and candidate,
    walks each request's tokens element by element from the slot's state and writes S * silu(g)."""

    graph_safe = True

    def __init__(self, spec: GatedUnitSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        self.w_all = torch.cat([weights[n] for n in (spec.z_proj, spec.x_proj, spec.g_proj)], dim=0).contiguous()
        self.z_bias, self.x_bias = weights[spec.z_bias], weights[spec.x_bias]
        self.w_o = weights[spec.o_proj]

    def forward(self, h, ctx, call):
        s, k = self.spec, self.k
        n = h.shape[0]
        proj = ctx.buffer("gu_proj", (n, 3 * s.width), torch.float32)
        k.linear(h, self.w_all, proj)
        out = ctx.buffer("gu_out", (n, s.width), self.rt.act_dtype)
        k.gated_unit_scan(proj, self.z_bias, self.x_bias, ctx.state(call.cache), ctx.state_slots, ctx.cu_q, ctx.seq_lens, out,
                          max_q_len=ctx.max_q_len)
        delta = ctx.buffer("delta_unit", (n, s.hidden_size), torch.float32)
        k.linear(out, self.w_o, delta)
        return delta


register_part(GatedUnitSpec, GatedUnit)


class RealGatedRecurrence:
    """h -> o_proj(S * gelu_tanh(Y h + by)), S <- a S + sqrt(1 - a^2) * i * u per channel, u = conv(X h + bx).

    y | x run as one product into float32.  One kernel adds the x bias, runs the short causal convolution over each
    request's tokens from the inputs its slot kept (cache entry 1) and writes u twice: float32 for the recurrence and, in the
    products' dtype, block by block for the gates.  The two block-diagonal gate matrices are one grouped product (the
    framework's grouped product with a block in an expert's place: r | i of a block are the rows of one matrix) into
    float32 (where the operands are bfloat16 and the description asks for two terms, u enters as its rounding and what the
    rounding left out against the matrix repeated along k).  The recurrence kernel adds the gates' biases, forms sigmoid, softplus, the decay and the input term in float32,
    walks each request's tokens from the slot's state (cache entry 0; long portions in chunks side by side) and multiplies
    by the gelu branch.  A prompt, a portion and a decoded token are the same calls: the slot carries the past."""

    graph_safe = True

    def __init__(self, spec: RealGatedRecurrenceSpec, weights, runtime):
        self.spec = s = spec
        self.rt = runtime
        self.k = runtime.kernels
        f32 = lambda name: weights[name].to(torch.float32).contiguous()      # small vectors: the kernels read float32
        self.w_yx = torch.cat((weights[s.y_proj], weights[s.x_proj]), dim=0).contiguous()
        self.y_bias, self.x_bias = f32(s.y_bias), f32(s.x_bias)
        self.conv_w, self.conv_b = f32(s.conv), f32(s.conv_bias)
        self.w_gates = torch.cat((weights[s.a_gate], weights[s.x_gate]), dim=1).contiguous()      # [blocks, 2 bs, bs]
        # two terms of u (bfloat16 operands only): the matrix repeated along k meets [roundings | what they left out]
        self.terms = 2 if s.gate_terms == 2 and runtime.act_dtype == torch.bfloat16 else 1
        if self.terms == 2:
            self.w_gates = torch.cat((self.w_gates, self.w_gates), dim=2).contiguous()           # [blocks, 2 bs, 2 bs]
        self.a_bias, self.i_bias = f32(s.a_bias).reshape(-1), f32(s.x_bias_gate).reshape(-1)
        self.decay = f32(s.decay)
        self.w_o = weights[s.o_proj]

    def _segment(self, n):
        """Rows of a block's segment in the grouped product, and the tile of the tcgen05 route (0: the other route)."""
        k = self.k
        ok = getattr(k, "moe_grouped_tc_ok", None)
        if ok is not None and ok(n * self.spec.blocks, self.rt.act_dtype, self.w_gates):
            t = k.MOE_TILE
            return -(-n // t) * t, t
        return n, 0

    def forward(self, h, ctx, call):
        s, k = self.spec, self.k
        n = h.shape[0]
        W, B = s.width, s.blocks
        bs = W // B
        act = self.rt.act_dtype
        proj = ctx.buffer("rg_proj", (n, 2 * W), torch.float32)
        k.linear(h, self.w_yx, proj)
        seg, tile = self._segment(n)
        cap, _ = self._segment(ctx.max_rows)
        u = ctx.buffer("rg_u", (n, W), torch.float32)
        kb = self.terms * bs
        ub = ctx.buffer("rg_u_blocks", (B * seg, kb), act, rows=B * cap).view(B, seg, kb)
        offsets = ctx.buffer("rg_offsets", (B + 1,), torch.int32, rows=B + 1)
        tiles = ctx.buffer("rg_tiles", (B * seg // tile,), torch.int32, rows=B * cap // tile) if tile else None
        k.rglru_conv(proj, W, self.x_bias, self.conv_w, self.conv_b, ctx.state((call.cache, 1)), ctx.state_slots, ctx.cu_q,
                     ctx.seq_lens, ctx.req_index, u, ub, offsets, tiles, tile)
        gates = ctx.buffer("rg_gates", (B * seg, 2 * bs), torch.float32, rows=B * cap)
        if tile:
            k.moe_linear_grouped(ub.view(B * seg, kb), self.w_gates, tiles, gates)
        else:
            k.moe_linear(ub.view(B * seg, kb), self.w_gates, offsets, None, 1, gates)
        out = ctx.buffer("rg_out", (n, W), act)
        k.rglru_scan(gates.view(B, seg, 2 * bs), self.a_bias, self.i_bias, self.decay, s.decay_scale, u, proj, 0, self.y_bias,
                     ctx.state((call.cache, 0)), ctx.state_slots, ctx.cu_q, ctx.seq_lens, out, max_q_len=ctx.max_q_len)
        delta = ctx.buffer("delta_mixer", (n, s.hidden_size), torch.float32)
        k.linear(out, self.w_o, delta)
        return delta


register_part(RealGatedRecurrenceSpec, RealGatedRecurrence)
