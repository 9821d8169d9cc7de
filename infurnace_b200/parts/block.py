"""How a layer's parts are arranged."""
from __future__ import annotations

import torch

from ..config.specs import (
    DepthAverageBlockSpec, LayerCall, PostNormBlockSpec, PreNormBlockSpec, SandwichBlockSpec, StreamInjectSpec, TokenSideSpec,
)
from .parallel import WeightedSum
from .registry import Folded, build_part, register_part


class PreNormBlock:
    """x += mixer(norm(x)); x += ffn(norm(x))
    (src/infurnace/executor/tinygrad/model.py:101,143,145,148).  Each addition happens in
    the kernel of the norm that follows it, so the block takes the previous block's last
    delta as ``pending`` and hands its own on.

    A block without feed-forward hands on the mixer's delta.  A block with a per-layer token input
    (``side``) ends with the stream up to date: the last delta is added in a pass that also leaves
    the stream in the products' dtype for the side input's gate product, the side input's result is
    normalised and added by the framework's stream update kernel, which in the same pass writes the
    NEXT block's first norm when a block of this kind follows (it gets a :class:`ReadyInput`)."""

    def __init__(self, spec: PreNormBlockSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        self.mixer_norm = build_part(spec.mixer_norm, weights, runtime)
        self.mixer = build_part(spec.mixer, weights, runtime)
        self.ffn_norm = build_part(spec.ffn_norm, weights, runtime) if spec.ffn is not None else None
        self.ffn = build_part(spec.ffn, weights, runtime) if spec.ffn is not None else None
        self.side = build_part(spec.side, weights, runtime) if spec.side is not None else None

    @property
    def graph_safe(self):
        parts = [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn, self.side) if p is not None]
        return all(getattr(p, "graph_safe", False) for p in parts)

    folds_norms = True

    def takes_folded(self, n):
        """Whether the block before this one may hand over x already updated and this block's
        first norm folded (a :class:`Folded` as ``pending``) for a step of n tokens."""
        take = getattr(self.mixer, "can_take_folded", None)
        return bool(getattr(self.mixer_norm, "foldable", False) and take and take(n))

    def forward(self, x, pending, ctx, call, next_layer=None):
        n = x.shape[0]
        if isinstance(pending, ReadyInput):          # x is up to date and our first norm is written
            h = pending.values
        elif isinstance(pending, Folded):            # x is up to date and our first norm is folded
            h = pending
        else:
            h = ctx.buffer("h", x.shape, self.rt.act_dtype)
            self.mixer_norm.forward(x, h, delta=pending)
        if self.ffn is None:
            d = self.mixer.forward(h, ctx, call)
            return self._finish(x, d, ctx, next_layer)
        take = getattr(self.ffn, "can_take_folded", None)
        if getattr(self.mixer, "can_fold_output", False) and getattr(self.ffn_norm, "foldable", False) and take and take(n):
            d = self.mixer.forward(h, ctx, call, fold=(x, self.ffn_norm))
        else:
            d = self.mixer.forward(h, ctx, call)
        if isinstance(d, Folded):
            h = d
        else:
            h = ctx.buffer("h", x.shape, self.rt.act_dtype)
            self.ffn_norm.forward(x, h, delta=d)
        if self.side is None and next_layer is not None and getattr(self.ffn, "can_fold_output", False) and next_layer.takes_folded(n):
            return self.ffn.forward(h, ctx, fold=(x, next_layer.mixer_norm))
        return self._finish(x, self.ffn.forward(h, ctx), ctx, next_layer)

    def _finish(self, x, d, ctx, next_layer):
        """The block's last delta: handed on as it is, or, with a side input, added here before that input reads the stream."""
        if self.side is None:
            return d
        k = self.k
        if self.rt.act_dtype == torch.float32:
            k.scaled_sum(x, d, 1.0)
            xa = x
        else:
            xa = ctx.buffer("stream_copy", x.shape, self.rt.act_dtype)
            k.scaled_sum(x, d, 1.0, copy=xa)
        y = self.side.forward(xa, ctx)
        ahead = None
        if isinstance(next_layer, PreNormBlock) and hasattr(next_layer.mixer_norm, "weight") \
                and type(next_layer.mixer_norm) is type(self.side.norm):
            ahead = next_layer.mixer_norm
        norm = self.side.norm
        if ahead is not None and ahead.spec.eps == norm.spec.eps:
            out = ctx.buffer("h", x.shape, self.rt.act_dtype)
            k.residual_norm_update(x, y, norm.weight, norm.spec.eps, out=out, next_weight=ahead.weight)
            return ReadyInput(out)
        k.residual_norm_update(x, y, norm.weight, norm.spec.eps)
        return None


register_part(PreNormBlockSpec, PreNormBlock)


class PostNormBlock:
    """x += ls1 * norm(mixer(x)); x += ls2 * norm(ffn(x)): no norm stands before a sublayer, and the norm
    (one number as weight) is applied to their result.  Norm, layer scale and addition are one kernel, which in
    bfloat16 mode also leaves the bfloat16 copy of the stream that the next product reads.  The block hands on
    no pending delta: x is up to date when it returns."""

    def __init__(self, spec: PostNormBlockSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        self.mixer = build_part(spec.mixer, weights, runtime)
        self.mixer_norm = build_part(spec.mixer_norm, weights, runtime)
        self.mixer_scale = weights[spec.mixer_scale]
        self.ffn = build_part(spec.ffn, weights, runtime) if spec.ffn is not None else None
        self.ffn_norm = build_part(spec.ffn_norm, weights, runtime) if spec.ffn is not None else None
        self.ffn_scale = weights[spec.ffn_scale] if spec.ffn is not None else None

    @property
    def graph_safe(self):
        parts = [self.mixer] + ([self.ffn] if self.ffn is not None else [])
        return all(getattr(p, "graph_safe", False) for p in parts)

    def _input(self, x, ctx):
        """What the sublayer's products read: x itself in float32 mode, else its bfloat16 copy."""
        from .model import STREAM_COPY
        if self.rt.act_dtype == torch.float32:
            return x
        h = ctx.shared.get(STREAM_COPY)
        if h is None or h.shape != x.shape:
            h = ctx.buffer("stream_copy", x.shape, torch.bfloat16)
            self.k.cast_rows(x, h)
            ctx.shared[STREAM_COPY] = h
        return h

    def _update(self, x, y, norm, scale, ctx):
        from .model import STREAM_COPY
        half = None
        if self.rt.act_dtype == torch.bfloat16:
            half = ctx.buffer("stream_copy", x.shape, torch.bfloat16)
        self.k.residual_postnorm(x, y, norm.weight, scale, norm.spec.eps, half)
        if half is not None:
            ctx.shared[STREAM_COPY] = half

    def forward(self, x, pending, ctx, call):
        from .model import STREAM_COPY
        if pending is not None:                      # a block of another kind ran before and left its last delta
            if isinstance(pending, Folded):
                raise TypeError("a post-norm block cannot take a folded norm from the block before it")
            x.add_(pending)
            ctx.shared.pop(STREAM_COPY, None)
        self._update(x, self.mixer.forward(self._input(x, ctx), ctx, call), self.mixer_norm, self.mixer_scale, ctx)
        if self.ffn is not None:
            self._update(x, self.ffn.forward(self._input(x, ctx), ctx), self.ffn_norm, self.ffn_scale, ctx)
        return None


register_part(PostNormBlockSpec, PostNormBlock)


class TokenSide:
    """x += norm(proj(act(gate x) * e)) with e a slice of the token's row of a table shared by the layers.  ``xa`` is
    the stream in the dtype the products read.  The gate product writes float32; one kernel applies the activation
    and the token's slice; the stream's update is the block's update kernel."""

    graph_safe = True

    def __init__(self, spec: TokenSideSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        self.table = weights[spec.table]
        self.w_gate, self.w_proj = weights[spec.gate], weights[spec.proj]
        self.norm = build_part(spec.norm, weights, runtime)

    def forward(self, xa, ctx):
        s, k = self.spec, self.k
        n = xa.shape[0]
        z = ctx.buffer("side_z", (n, s.dim), torch.float32)
        k.linear(xa, self.w_gate, z)
        g = ctx.buffer("side_g", (n, s.dim), self.rt.act_dtype)
        k.token_side_gate(z, self.table, ctx.token_ids, s.offset, s.activation, g)
        y = ctx.buffer("delta_side", (n, s.hidden_size), torch.float32)
        k.linear(g, self.w_proj, y)
        return y


register_part(TokenSideSpec, TokenSide)


class ReadyInput:
    """What a sandwich block hands to the sandwich block after it instead of a pending delta: x is up to date, and
    ``values`` already holds the next block's first pre-norm of it (written by this block's last stream update)."""
    __slots__ = ("values",)

    def __init__(self, values):
        self.values = values


class SandwichBlock:
    """x += post1(mixer(pre1(x))); x += post2(ffn(pre2(x))); then the token side input.  Every update of the stream
    is one kernel that normalises the sublayer's float32 result, adds it to x in float32 and, in the same pass, writes
    what the next product reads: the next pre-norm of x (the next BLOCK's first norm too, when a block of this kind
    follows directly: it gets a :class:`ReadyInput`), or x itself in the products' dtype.  x is up to date when the
    block returns; it hands on no pending delta."""

    hands_over_input = True          # the decoder passes ``next_layer`` when the next layer call is a block of this kind

    def __init__(self, spec: SandwichBlockSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        self.mixer_norm = build_part(spec.mixer_norm, weights, runtime)
        self.mixer = build_part(spec.mixer, weights, runtime)
        self.mixer_post = build_part(spec.mixer_post_norm, weights, runtime)
        self.ffn = build_part(spec.ffn, weights, runtime) if spec.ffn is not None else None
        self.ffn_norm = build_part(spec.ffn_norm, weights, runtime) if spec.ffn is not None else None
        self.ffn_post = build_part(spec.ffn_post_norm, weights, runtime) if spec.ffn is not None else None
        self.side = build_part(spec.side, weights, runtime) if spec.side is not None else None

    @property
    def graph_safe(self):
        parts = [self.mixer] + [p for p in (self.ffn, self.side) if p is not None]
        return all(getattr(p, "graph_safe", False) for p in parts)

    def _update(self, x, y, post, ctx, then_norm=None, then_copy=False):
        """x += y / rms(y) * post.weight; returns the next product's input if one was asked for."""
        out = None
        if then_norm is not None or then_copy:
            out = ctx.buffer("h", x.shape, self.rt.act_dtype)
        nxt = then_norm.weight if then_norm is not None else None
        if isinstance(y, WeightedSum):               # two mixers side by side: their weighted sum is formed in this pass
            (y1, s1), (y2, s2) = y.terms
            self.k.residual_norm_update(x, y1, post.weight, post.spec.eps, out=out, next_weight=nxt, y2=y2, scale=s1, scale2=s2)
        else:
            self.k.residual_norm_update(x, y, post.weight, post.spec.eps, out=out, next_weight=nxt)
        return out

    def forward(self, x, pending, ctx, call, next_layer=None):
        if isinstance(pending, ReadyInput):          # the block before this one wrote our first norm already
            h = pending.values
        else:
            if pending is not None:                  # a block of another kind ran before and left its last delta
                if isinstance(pending, Folded):
                    raise TypeError("a sandwich block cannot take a folded norm from the block before it")
                x.add_(pending)
            h = ctx.buffer("h", x.shape, self.rt.act_dtype)
            self.mixer_norm.forward(x, h)
        ahead = next_layer.mixer_norm if isinstance(next_layer, SandwichBlock) else None
        if getattr(self.mixer, "can_return_weighted", False):
            y = self.mixer.forward(h, ctx, call, weighted=True)
        else:
            y = self.mixer.forward(h, ctx, call)
        last_norm = None if self.side is not None else ahead        # the block's last update also writes the next block's norm
        if self.ffn is not None:
            h = self._update(x, y, self.mixer_post, ctx, then_norm=self.ffn_norm)
            y = self.ffn.forward(h, ctx)
            xa = self._update(x, y, self.ffn_post, ctx, then_norm=last_norm, then_copy=self.side is not None)
        else:
            xa = self._update(x, y, self.mixer_post, ctx, then_norm=last_norm, then_copy=self.side is not None)
        if self.side is not None:
            xa = self._update(x, self.side.forward(xa, ctx), self.side.norm, ctx, then_norm=ahead)
        return ReadyInput(xa) if ahead is not None else None


register_part(SandwichBlockSpec, SandwichBlock)


# key of ``ctx.shared`` under which the blocks that average over depth keep every token's earlier block results of the step
DEPTH_HISTORY = ("depth_history",)


class DepthAverageBlock:
    """x += m * mixer(conv1(norm1(x))); x += m * ffn(conv2(norm2(x))); then x <- sum_j a[j] * X_j over the embedding's
    output X_0 and the results X_1 .. of all blocks so far, this one's included.

    The X_j of a step's tokens live in one float32 buffer [tokens, depths, hidden] shared by the blocks of the model
    (scratch of the step, not state: an average reads the same token's rows only).  The block at depth 0 puts the
    embedding's output there while it forms its first norm.  The mixer's delta is added in the kernel of the second
    norm; the last delta is added in the averaging kernel, which stores the block's result, writes the average over x
    and, when a block of this kind follows, also that block's first norm of the new x (it gets a :class:`ReadyInput`).
    Each convolution keeps its last inputs in a state entry of its own: entry 0 of the call's cache is the mixer's,
    entries 1 and 2 the convolutions'.  x is up to date when the block returns."""

    hands_over_input = True

    def __init__(self, spec: DepthAverageBlockSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        self.mixer_norm = build_part(spec.mixer_norm, weights, runtime)
        self.mixer = build_part(spec.mixer, weights, runtime)
        self.mixer_conv = build_part(spec.mixer_conv, weights, runtime) if spec.mixer_conv is not None else None
        has_ffn = spec.ffn is not None
        self.ffn = build_part(spec.ffn, weights, runtime) if has_ffn else None
        self.ffn_norm = build_part(spec.ffn_norm, weights, runtime) if has_ffn else None
        self.ffn_conv = build_part(spec.ffn_conv, weights, runtime) if has_ffn and spec.ffn_conv is not None else None
        self.average = weights[spec.average] if spec.average is not None else None

    @property
    def graph_safe(self):
        parts = [self.mixer] + [p for p in (self.ffn, self.mixer_conv, self.ffn_conv) if p is not None]
        return all(getattr(p, "graph_safe", False) for p in parts)

    def _history(self, x, ctx):
        """The step's [tokens, depths, hidden] buffer; every block asks for the same one (``depths`` is the plan's)."""
        hist = ctx.shared.get(DEPTH_HISTORY)
        if hist is None:
            if self.spec.depth != 0:
                raise RuntimeError("a block that averages over depth found no history: the block at depth 0 has not run in this step")
            hist = ctx.buffer("depth_history", (x.shape[0], self.spec.depths + 1, x.shape[1]), torch.float32)
            ctx.shared[DEPTH_HISTORY] = hist
        return hist

    def forward(self, x, pending, ctx, call, next_layer=None):
        s, k = self.spec, self.k
        m = s.residual_mult
        hist = self._history(x, ctx) if self.average is not None else None
        if isinstance(pending, ReadyInput):          # the block before this one wrote our first norm already
            h = pending.values
        else:
            if isinstance(pending, Folded):
                raise TypeError("a block that averages over depth cannot take a folded norm from the block before it")
            if hist is not None and s.depth != 0:
                raise RuntimeError("the average over depth needs every earlier block's result: only the block at depth 0 may "
                                   "start from a plain stream")
            h = ctx.buffer("h", x.shape, self.rt.act_dtype)
            self.mixer_norm.forward(x, h, delta=pending, keep=hist[:, 0] if hist is not None else None)
        if self.mixer_conv is not None:
            h = self.mixer_conv.forward(h, ctx, (call.cache, 1))
        d = self.mixer.forward(h, ctx, LayerCall(call.layer, (call.cache, 0), call.store))
        if self.ffn is not None:
            h = ctx.buffer("h", x.shape, self.rt.act_dtype)
            self.ffn_norm.forward(x, h, delta=d, mult=m)
            if self.ffn_conv is not None:
                h = self.ffn_conv.forward(h, ctx, (call.cache, 2))
            d = self.ffn.forward(h, ctx)
        ahead = next_layer.mixer_norm if isinstance(next_layer, DepthAverageBlock) else None
        out = ctx.buffer("h", x.shape, self.rt.act_dtype) if ahead is not None else None
        if hist is not None:
            k.depth_average(x, d, m, hist, s.depth + 1, self.average, out=out, next_weight=ahead.weight if ahead is not None else None,
                            groups=ahead.spec.groups if ahead is not None else 1, eps=ahead.spec.eps if ahead is not None else 0.0)
        elif ahead is not None:
            ahead.forward(x, out, delta=d, mult=m)
        else:
            k.scaled_sum(x, d, m)
        return ReadyInput(out) if ahead is not None else None


register_part(DepthAverageBlockSpec, DepthAverageBlock)


class StreamInject:
    """x += table[row] (+ the rows the embedding kept): the step that opens a pass over a range of layers that runs
    several times.  It stands in the schedule like a layer."""

    graph_safe = True

    def __init__(self, spec: StreamInjectSpec, weights, runtime):
        from .model import EMBEDDING_ROWS
        self.spec = spec
        self.k = runtime.kernels
        self.vec = weights[spec.table][spec.row].contiguous()
        self._key = EMBEDDING_ROWS

    def forward(self, x, pending, ctx, call):
        if pending is not None:
            if isinstance(pending, Folded):
                raise TypeError("an injection step cannot take a folded norm from the block before it")
            x.add_(pending)
        rows = None
        if self.spec.add_embedding:
            rows = ctx.shared.get(self._key)
            if rows is None:
                raise RuntimeError("the embedding kept no rows for this step (its description needs keep=True)")
        self.k.add_rows(x, rows, self.vec)
        return None


register_part(StreamInjectSpec, StreamInject)
