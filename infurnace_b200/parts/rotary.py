"""Rotary position encoding."""
from __future__ import annotations

import torch

from ..config.specs import RotarySpec
from ..errors import ModelConfigError
from .registry import register_part


def rotary_frequencies(spec: RotarySpec):
    """(float32 frequencies of the rotated pairs, the factor on cosine and sine).  With ``scaling`` the slow ones are
    stretched as the description says."""
    import math
    if spec.scaling is None and spec.frequency_dtype == "float32":
        exponent = torch.arange(0, spec.rotary_dim, 2, dtype=torch.float32) / spec.rotary_dim
        return 1.0 / (spec.theta ** exponent), 1.0
    i = torch.arange(0, spec.rotary_dim // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * i / spec.rotary_dim)
    gain = 1.0
    if spec.scaling is not None:
        factor, original, fast, slow = (float(v) for v in spec.scaling)

        def dim_of(turns):
            return spec.rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(spec.theta))
        lo = max(math.floor(dim_of(fast)), 0)
        hi = min(math.ceil(dim_of(slow)), spec.rotary_dim - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        freq = freq / factor * ramp + freq * (1.0 - ramp)
        gain = 0.1 * math.log(factor) + 1.0
    return freq.to(torch.float32), float(gain)


class Rotary:
    """inv_freq_i = 1 / theta^(2i / rotary_dim), angle = position * inv_freq_i, both in
    float32 (src/infurnace/executor/tinygrad/model.py:18-22); the rotation itself runs
    inside the attention part's fused kernel, which takes the frequencies, the rotated
    width and the pairing as arguments (model.py:24-27 is the half-split pairing)."""

    graph_safe = True     # launches depend on the step's sizes only, never on values read on the host

    def __init__(self, spec: RotarySpec, weights, runtime):
        if spec.rotary_dim % 2 or not 0 < spec.rotary_dim <= spec.head_dim:
            raise ModelConfigError(f"rotary_dim {spec.rotary_dim} must be even and at most head_dim {spec.head_dim}")
        self.spec = spec
        self.k = runtime.kernels
        freq, self.gain = rotary_frequencies(spec)
        self.inv_freq = freq.to(runtime.device)

    def fused_rotary(self):
        if self.gain != 1.0:
            return None                       # the fused kernels form plain cosines and sines themselves
        return self.inv_freq, self.spec.rotary_dim, self.spec.interleaved

    def table(self, ctx):
        """(cos, sin) of every token's angles, computed once per step and shared by all layers with the same
        base and rotated width (the angles do not depend on the layer)."""
        key = ("rope_table", self.spec.theta, self.spec.rotary_dim, self.spec.scaling, self.spec.frequency_dtype)
        t = ctx.shared.get(key)
        if t is None:
            tag = "" if self.spec.scaling is None else "_" + "_".join(repr(v) for v in self.spec.scaling)
            tag += "" if self.spec.frequency_dtype == "float32" else "_" + self.spec.frequency_dtype
            t = ctx.buffer(f"rope_table_{self.spec.theta}_{self.spec.rotary_dim}{tag}", (ctx.num_tokens, self.spec.rotary_dim),
                           torch.float32)
            if self.gain != 1.0:
                self.k.rope_table(ctx.positions, self.inv_freq, t, gain=self.gain)
            else:
                self.k.rope_table(ctx.positions, self.inv_freq, t)
            ctx.shared[key] = t
        return t

    def apply(self, qkv, num_heads, num_kv_heads, head_dim, positions):
        if self.gain != 1.0:
            raise ModelConfigError("a rotation whose cosine and sine carry a factor runs from its per-step table only")
        self.k.qk_norm_rope_store(qkv, num_heads, num_kv_heads, head_dim, None, None, 0.0,
                                  self.inv_freq, self.spec.rotary_dim, self.spec.interleaved,
                                  positions, None, None)


register_part(RotarySpec, Rotary)
