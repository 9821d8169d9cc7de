"""RMSNorm with the residual addition folded in."""
from __future__ import annotations

from ..config.specs import GroupRMSNormSpec, RMSNormSpec, ScalarRMSNormSpec
from .registry import register_part


class RMSNorm:
    """out = (x + delta) * rsqrt(mean((x + delta)^2) + eps) * weight, statistics in 32-bit
    (src/infurnace/executor/tinygrad/model.py:11-13).  x is the float32 residual stream;
    without ``rows`` the sum is written back to x, which is the reference's ``x = x + ...``
    (model.py:143,148) done in the same pass."""

    graph_safe = True     # launches depend on the step's sizes only, never on values read on the host
    foldable = True       # weight and spec.eps are all that a neighbouring product needs to do this norm

    def __init__(self, spec: RMSNormSpec, weights, runtime):
        self.spec = spec
        self.weight = weights[spec.weight]
        self.k = runtime.kernels

    def forward(self, x, out, delta=None, rows=None):
        self.k.rmsnorm(x, self.weight, self.spec.eps, out, delta=delta, rows=rows)
        return out


register_part(RMSNormSpec, RMSNorm)


class ScalarRMSNorm:
    """out = x * rsqrt(mean(x^2) + eps) * g with one number g, as the last norm of a model (``rows``) or
    before a product.  It runs the RMSNorm kernel with g repeated along the row, which is the same
    arithmetic element by element.  As the norm of a sublayer's result inside a residual update it is not
    called at all: the block's update kernel reads ``weight`` and ``spec.eps``."""

    graph_safe = True

    def __init__(self, spec: ScalarRMSNormSpec, weights, runtime):
        self.spec = spec
        self.weight = weights[spec.weight].reshape(1).contiguous()
        self.k = runtime.kernels
        self._row = None

    def forward(self, x, out, delta=None, rows=None):
        if self._row is None or self._row.numel() != x.shape[1]:
            self._row = self.weight.expand(x.shape[1]).contiguous()
        self.k.rmsnorm(x, self._row, self.spec.eps, out, delta=delta, rows=rows)
        return out


register_part(ScalarRMSNormSpec, ScalarRMSNorm)


class GroupRMSNorm:
    """The RMS norm in groups: the row in ``groups`` equal consecutive parts, each divided by its own
    sqrt(mean(part^2) + eps), the whole times the weight; statistics in float32.  With ``delta`` the float32 stream first
    becomes x + mult * delta (in place, unless ``rows`` picks the rows that are normed); ``keep`` also gets the updated
    rows."""

    graph_safe = True

    def __init__(self, spec: GroupRMSNormSpec, weights, runtime):
        self.spec = spec
        self.weight = weights[spec.weight]
        self.k = runtime.kernels

    def forward(self, x, out, delta=None, rows=None, mult=1.0, keep=None):
        self.k.group_rmsnorm(x, self.weight, self.spec.groups, self.spec.eps, out, delta=delta, mult=mult, rows=rows, keep=keep)
        return out


register_part(GroupRMSNormSpec, GroupRMSNorm)
