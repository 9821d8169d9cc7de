"""The short causal convolution in front of a sublayer."""
from __future__ import annotations

from ..config.specs import CausalConvSpec
from .registry import register_part


class CausalConvAdd:
    """h_t -> h_t + sum_j w[:, j] * h_(t - taps + 1 + j) on each channel, over each request's tokens in order; zeros stand
    before a sequence's start.  The taps - 1 inputs before a portion come from the request's row of the cache entry
    ``cache_id`` (float32 [slots, taps - 1, width], zeroed when the slot is granted), which then takes the portion's
    last inputs: however a sequence is cut into steps, a token sees the same inputs.  Products and sums are float32."""

    graph_safe = True

    def __init__(self, spec: CausalConvSpec, weights, runtime):
        self.spec = spec
        self.weight = weights[spec.weight]
        self.k = runtime.kernels

    def forward(self, h, ctx, cache_id, name="conv_out"):
        out = ctx.buffer(name, h.shape, h.dtype)
        self.k.causal_conv(h, self.weight, ctx.state(cache_id), ctx.state_slots, ctx.cu_q, ctx.seq_lens, ctx.req_index, out)
        return out


register_part(CausalConvSpec, CausalConvAdd)
