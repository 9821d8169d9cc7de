"""A mixture of gated feed-forwards."""
from __future__ import annotations

import torch

from ..config.specs import RoutedExpertsSpec
from ..errors import ModelConfigError
from .registry import register_part


class RoutedExperts:
    """h -> sum over a token's ``top`` experts of weight * down_e(act(gate_e h) * up_e h).

    The router's logits are a product into float32.  One kernel picks each token's ``top`` largest logits and takes
    the softmax over them; one lists, per expert, the (token, choice) pairs that chose it, in token order (all on the
    device: the step's launches depend on its sizes only).  The experts' products then run as two grouped launches
    over that list (gate | up with the activation in the epilogue, then down) against the experts' matrices stacked
    along a leading axis, and one kernel sums each token's results in the order of its choices, in float32.  bfloat16
    steps of more than 256 pairs (prompts) take the tcgen05 kernel in its grouped mode, over a list whose segments are
    padded to that kernel's tile of 128 rows (``_forward_padded``); fewer pairs, float32 and odd sizes the kernels of
    csrc/moe.cu.

    The description's ``scoring``, ``groups`` and ``weight_scale`` go to the router kernel as they are.  With ``weight_on``
    "input" an expert reads weight * h: the tokens' rows are gathered into the list's order times their weights (one
    kernel, which the padded route runs anyway), and the combining kernel adds the results as they are.  A ``shared``
    expert is two dense products on every row; its result joins the weighted sum in the combining kernel, times
    sigmoid of the row's ``shared_gate`` logit when there is one.  That logit is one more row of the router's matrix, so
    it costs no product of its own."""

    graph_safe = True

    def __init__(self, spec: RoutedExpertsSpec, weights, runtime):
        if spec.activation != "silu":
            raise ModelConfigError(f"activation {spec.activation!r}: only 'silu' has a kernel")
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        self.router = weights[spec.router]
        self.w_shared_gate_up = self.w_shared_down = None
        if spec.shared is not None:
            if spec.shared.activation != "silu":
                raise ModelConfigError(f"activation {spec.shared.activation!r}: only 'silu' has a kernel")
            self.w_shared_gate_up = torch.cat((weights[spec.shared.gate_proj], weights[spec.shared.up_proj]), dim=0).contiguous()
            self.w_shared_down = weights[spec.shared.down_proj]
            if spec.shared_gate is not None:
                self.router = torch.cat((self.router, weights[spec.shared_gate].to(self.router.dtype)), dim=0).contiguous()
        elif spec.shared_gate is not None:
            raise ModelConfigError("a gate of the shared expert needs a shared expert")
        self.route_args = dict(scoring=spec.scoring, groups=spec.groups, weight_scale=spec.weight_scale)
        if spec.weight_on not in ("output", "input"):
            raise ModelConfigError(f"weight_on {spec.weight_on!r}: an expert's weight multiplies its 'output' or its 'input'")
        self.weight_input = spec.weight_on == "input"
        self.w_gate_up = torch.stack([torch.cat((weights[g], weights[u]), dim=0) for g, u, _ in spec.experts], dim=0).contiguous()
        self.w_down = torch.stack([weights[d] for _, _, d in spec.experts], dim=0).contiguous()
        self.num_experts = len(spec.experts)

    def forward(self, h, ctx, fold=None):
        s, k, E = self.spec, self.k, self.num_experts
        n = h.shape[0]
        logits = ctx.buffer("moe_logits", (n, self.router.shape[0]), torch.float32)
        k.linear(h, self.router, logits)
        shared = self._shared(h, ctx, logits)
        ids = ctx.buffer("moe_ids", (n, s.top), torch.int32)
        gates = ctx.buffer("moe_gates", (n, s.top), torch.float32)
        pairs = n * s.top
        ok = getattr(k, "moe_grouped_tc_ok", None)
        if ok is not None and ok(pairs, h.dtype, self.w_gate_up, self.w_down):
            k.moe_route(logits, s.top, ids, gates, experts=E, **self.route_args)
            return self._forward_padded(h, ctx, ids, gates, shared)
        offsets = ctx.buffer("moe_offsets", (E + 1,), torch.int32, rows=E + 1)
        perm = ctx.buffer("moe_perm", (pairs,), torch.int32, rows=ctx.max_rows * s.top)
        pos = ctx.buffer("moe_pos", (pairs,), torch.int32, rows=ctx.max_rows * s.top)
        k.moe_route_plan(logits, s.top, ids, gates, offsets, perm, pos, experts=E, **self.route_args)   # one launch for few pairs
        act = ctx.buffer("moe_act", (pairs, s.intermediate_size), self.rt.act_dtype, rows=ctx.max_rows * s.top)
        if self.weight_input:        # the experts read weight * h: the rows are gathered and scaled into the list's order first
            xs = ctx.buffer("moe_xs_scaled", (pairs, h.shape[1]), h.dtype, rows=ctx.max_rows * s.top)
            k.moe_gather_scaled(h, perm, s.top, gates, xs)
            k.moe_linear(xs, self.w_gate_up, offsets, None, 1, act, epilogue="silu_gate")
        else:
            k.moe_linear(h, self.w_gate_up, offsets, perm, s.top, act, epilogue="silu_gate")
        y = ctx.buffer("moe_y", (pairs, s.hidden_size), torch.float32, rows=ctx.max_rows * s.top)
        k.moe_linear(act, self.w_down, offsets, None, 1, y)
        delta = ctx.buffer("delta_ffn", (n, s.hidden_size), torch.float32)
        k.moe_combine(y, pos, None if self.weight_input else gates, delta, *shared)
        return delta

    def _shared(self, h, ctx, logits):
        """(result of the shared expert [n, hidden] float32, its gate's logits [n]) or (None, None)."""
        s = self.spec
        if s.shared is None:
            return None, None
        n = h.shape[0]
        act = ctx.buffer("moe_shared_act", (n, s.shared.intermediate_size), self.rt.act_dtype)
        self.k.linear(h, self.w_shared_gate_up, act, epilogue="silu_gate")
        out = ctx.buffer("moe_shared", (n, s.hidden_size), torch.float32)
        self.k.linear(act, self.w_shared_down, out)
        return out, (logits[:, self.num_experts] if s.shared_gate is not None else None)

    def _forward_padded(self, h, ctx, ids, gates, shared=(None, None)):
        """A prompt's experts on the tcgen05 kernel: the pair list with every expert's segment padded to the kernel's row
        tile, the tokens' rows gathered into that order, the two products as grouped launches whose row tiles each belong to
        one expert, the weighted sum through the padded places."""
        s, k, E = self.spec, self.k, self.num_experts
        n = h.shape[0]
        pairs = n * s.top
        places, cap = k.moe_padded_rows(pairs, E), k.moe_padded_rows(ctx.max_rows * s.top, E)
        offsets = ctx.buffer("moe_offsets", (E + 1,), torch.int32, rows=E + 1)
        perm = ctx.buffer("moe_perm_padded", (places,), torch.int32, rows=cap)
        pos = ctx.buffer("moe_pos", (pairs,), torch.int32, rows=ctx.max_rows * s.top)
        tiles = ctx.buffer("moe_tiles", (places // k.MOE_TILE,), torch.int32, rows=cap // k.MOE_TILE)
        k.moe_plan_padded(ids, E, offsets, perm, pos, tiles)
        xs = ctx.buffer("moe_xs", (places, h.shape[1]), self.rt.act_dtype, rows=cap)
        if self.weight_input:
            k.moe_gather_scaled(h, perm, s.top, gates, xs, tile_expert=tiles)
        else:
            k.moe_gather(h, perm, s.top, tiles, xs)
        act = ctx.buffer("moe_act_padded", (places, s.intermediate_size), self.rt.act_dtype, rows=cap)
        k.moe_linear_grouped(xs, self.w_gate_up, tiles, act, epilogue="silu_gate")
        y = ctx.buffer("moe_y_padded", (places, s.hidden_size), torch.float32, rows=cap)
        k.moe_linear_grouped(act, self.w_down, tiles, y)
        delta = ctx.buffer("delta_ffn", (n, s.hidden_size), torch.float32)
        k.moe_combine(y, pos, None if self.weight_input else gates, delta, *shared)
        return delta


register_part(RoutedExpertsSpec, RoutedExperts)
