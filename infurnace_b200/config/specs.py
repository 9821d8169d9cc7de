"""Architecture-independent descriptions of a model: parts, layers and their order.

A model's ``config.json`` is turned, by the architecture's plan builder, into a
:class:`ModelPlan`: a tuple of layer descriptions, each put together from part
descriptions (norm, mixer, feed-forward, position encoding), and a *schedule*: the
list of layer calls in the order in which they run.  Everything below is plain data
(frozen dataclasses, no tensors), so it imports without torch, as the reference's
model contract does (tests/test_model_config.py:118).

Every part description

* carries its sizes and constants as fields (nothing is a literal in a kernel call),
* names its tensors (``tensors()``: name -> :class:`TensorSpec`), which is what the
  weight loader checks a model folder against, and
* says what it needs from the cache manager (``cache_need()``).

The implementation class of a description is looked up in
``infurnace_b200.parts.registry`` by the description's type, so a new mixer is a new
dataclass plus a class registered for it; neither this file nor the engine changes.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional, Tuple


# --------------------------------------------------------------------------- tensors
@dataclass(frozen=True)
class TensorSpec:
    """One tensor of a model folder.  ``kind`` is "float" (kept in the engine's weight
    dtype, see weights/loader.py) or "int" (an integer table, kept as int32).  ``init``:
    (mean, standard deviation) of the tensor in random-weights mode, where its shape alone
    would give the wrong idea (a single number that is a norm weight, a lower bound in (0, 1)).  An entry of
    ``shape`` may be None: the file gives that size (the part reads it from the tensor).  ``optional``: a folder
    may hold the tensor or not; no part needs it."""
    shape: Tuple[Optional[int], ...]
    kind: str = "float"
    init: Optional[Tuple[float, float]] = None
    optional: bool = False


# --------------------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class PagedStream:
    """One thing a mixer keeps per token in the pages: ``heads`` rows of ``width`` elements."""
    name: str
    heads: int
    width: int


@dataclass(frozen=True)
class KVCacheNeed:
    """Keys and values that grow with the sequence, kept in pages.

    ``window`` None: every earlier key stays visible.  ``window`` w: a query at
    position p sees keys at positions p-w+1 .. p, and pages that lie wholly below
    that range are given back while the request still runs.  ``value_head_dim``: the
    width of a value head where it differs from a key head's.  ``chunk`` c: a query at
    position p sees the keys of its own chunk only, positions (p // c) * c .. p, and the
    pages of a chunk are given back once the request's next position lies in a later one."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_head_dim: Optional[int] = None
    chunk: Optional[int] = None

    @property
    def streams(self) -> Tuple[PagedStream, ...]:
        return (PagedStream("k", self.num_kv_heads, self.head_dim),
                PagedStream("v", self.num_kv_heads, self.value_head_dim or self.head_dim))

    @property
    def group_key(self):
        return ("kv", self.streams, self.window) if self.chunk is None else ("kv", self.streams, self.window, ("chunk", self.chunk))


@dataclass(frozen=True)
class PagedCacheNeed:
    """Per-token entries of any shape, kept in pages: a tuple of streams (a compressed latent and a
    small rotated key, say, instead of full keys and values), with the same window rule as
    :class:`KVCacheNeed`.  A cache entry then has one tensor per stream,
    ``[pages, heads, page_size, width]``; streams of equal shape share one tensor
    ``[pages, streams, heads, page_size, width]`` (which is the layout of keys and values) unless ``separate`` asks
    for a dense tensor per stream whatever the shapes (kernels that address a stream as ``[pages * page_size, width]``)."""
    streams: Tuple[PagedStream, ...]
    window: Optional[int] = None
    separate: bool = False

    @property
    def group_key(self):
        return ("kv", self.streams, self.window, self.separate)


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size (``shape`` float32 elements per request)."""
    shape: Tuple[int, ...]

    @property
    def group_key(self):
        return ("state", self.shape)


# --------------------------------------------------------------------------- parts
@dataclass(frozen=True)
class RMSNormSpec:
    """y = x * rsqrt(mean(x^2) + eps) * weight, statistics in 32-bit
    (src/infurnace/executor/tinygrad/model.py:11-13)."""
    size: int
    eps: float
    weight: str  # tensor name

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {self.weight: TensorSpec((self.size,))}


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding of the first ``rotary_dim`` elements of a head.

    ``interleaved`` False pairs element i with i + rotary_dim/2 (the half-split form
    of model.py:24-27); True pairs 2i with 2i+1.  ``theta`` is the base of the
    frequencies inv_freq_i = theta^(-2i/rotary_dim) (model.py:18-22).

    ``scaling`` = (factor, original, fast, slow) stretches the slow frequencies (YaRN): with
    d(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(d(fast)), 0),
    hi = min(ceil(d(slow)), rotary_dim - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i
    turns at inv_freq_i / factor * ramp_i + inv_freq_i * (1 - ramp_i), and cosine and sine are both
    multiplied by 0.1 * ln(factor) + 1.  ``frequency_dtype`` "float32": theta^(-2i/rotary_dim) is formed in float32, as
    the reference forms it (model.py:18-22); "float64": formed in float64 and rounded to float32 once (always so with
    ``scaling``)."""
    head_dim: int
    rotary_dim: int
    theta: float
    interleaved: bool = False
    scaling: Optional[Tuple[float, float, float, float]] = None
    frequency_dtype: str = "float32"

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {}


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over the paged cache.

    q/k/v/o projections without bias (model.py:102-104,143); optional per-head
    RMSNorm of q and k before the position encoding (model.py:110-114); scores are
    scaled by ``scale`` (the reference leaves it at its attention routine's default,
    1/sqrt(head_dim), model.py:118); causal; optional window."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    q_proj: str
    k_proj: str
    v_proj: str
    o_proj: str
    q_norm: Optional[RMSNormSpec] = None
    k_norm: Optional[RMSNormSpec] = None
    position: Optional[RotarySpec] = None
    window: Optional[int] = None

    def tensors(self) -> Mapping[str, TensorSpec]:
        t = {
            self.q_proj: TensorSpec((self.num_heads * self.head_dim, self.hidden_size)),
            self.k_proj: TensorSpec((self.num_kv_heads * self.head_dim, self.hidden_size)),
            self.v_proj: TensorSpec((self.num_kv_heads * self.head_dim, self.hidden_size)),
            self.o_proj: TensorSpec((self.hidden_size, self.num_heads * self.head_dim)),
        }
        for part in (self.q_norm, self.k_norm, self.position):
            if part is not None:
                t.update(part.tensors())
        return t

    def cache_need(self):
        return KVCacheNeed(self.num_kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class GatedMLPSpec:
    """x -> down(act(gate(x)) * up(x)), no bias (model.py:146-148).  ``activation``
    names the gate's function; "silu" is z * sigmoid(z)."""
    hidden_size: int
    intermediate_size: int
    activation: str
    gate_proj: str
    up_proj: str
    down_proj: str

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {
            self.gate_proj: TensorSpec((self.intermediate_size, self.hidden_size)),
            self.up_proj: TensorSpec((self.intermediate_size, self.hidden_size)),
            self.down_proj: TensorSpec((self.hidden_size, self.intermediate_size)),
        }

    def cache_need(self):
        return None


@dataclass(frozen=True)
class PreNormBlockSpec:
    """x += mixer(norm1(x)); x += ffn(norm2(x))  (model.py:101,143,145,148).  ``ffn`` None: the block has no
    feed-forward (``ffn_norm`` is then None too, and ``unused`` may name norm weights that a folder stores all the
    same).  ``side``: a per-layer token input (a ``TokenSideSpec``) that follows the feed-forward."""
    mixer_norm: object
    mixer: object
    ffn_norm: Optional[object] = None
    ffn: Optional[object] = None
    side: Optional[object] = None
    unused: Tuple[Tuple[str, int], ...] = ()      # (name, length) of vectors a folder may hold that no part reads

    def tensors(self) -> Mapping[str, TensorSpec]:
        t = {}
        for part in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn, self.side):
            if part is not None:
                t.update(part.tensors())
        for name, size in self.unused:
            t.setdefault(name, TensorSpec((size,), optional=True))
        return t

    def cache_need(self):
        return self.mixer.cache_need()


@dataclass(frozen=True)
class EmbeddingSpec:
    """x[t] = table[id_t], no scaling (model.py:95)."""
    vocab_size: int
    hidden_size: int
    weight: str

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {self.weight: TensorSpec((self.vocab_size, self.hidden_size))}


@dataclass(frozen=True)
class LMHeadSpec:
    """logits = x @ W^T in 32-bit (model.py:151).  ``tied`` True: ``weight`` names the
    embedding table, which is read in place (weights.py:68), and is no tensor of its own;
    ``stored_as`` is then the name under which a model folder may nevertheless store the
    head, which is accepted only as an exact copy of the table (the reference's rule is
    identity of the two, model.py:34-36)."""
    vocab_size: int
    hidden_size: int
    weight: str
    tied: bool
    stored_as: Optional[str] = None
    softcap: Optional[float] = None       # c: logits <- c * tanh(logits / c)

    def tensors(self) -> Mapping[str, TensorSpec]:
        if self.tied:
            return {}
        return {self.weight: TensorSpec((self.vocab_size, self.hidden_size))}


# --------------------------------------------------------------------------- parts of post-norm decoders
@dataclass(frozen=True)
class ScalarRMSNormSpec:
    """y = x / sqrt(mean(x^2) + eps) * g with g a single number (a tensor of shape ())."""
    eps: float
    weight: str

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {self.weight: TensorSpec((), init=(1.0, 0.1))}


@dataclass(frozen=True)
class SinusoidEmbeddingSpec:
    """x[t] = table[id_t] + e(position_t), e[2i] = sin(p * base^(-2i/width)), e[2i+1] = cos of the same angle."""
    vocab_size: int
    hidden_size: int
    weight: str
    base: float = 10000.0

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {self.weight: TensorSpec((self.vocab_size, self.hidden_size))}


@dataclass(frozen=True)
class DenseMLPSpec:
    """x -> down(act(up(x))), no gate, no bias.  ``activation``: "relu2" (the square of relu), "silu",
    "gelu_tanh"."""
    hidden_size: int
    intermediate_size: int
    activation: str
    up_proj: str
    down_proj: str

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {self.up_proj: TensorSpec((self.intermediate_size, self.hidden_size)),
                self.down_proj: TensorSpec((self.hidden_size, self.intermediate_size))}

    def cache_need(self):
        return None


@dataclass(frozen=True)
class GatedRecurrenceSpec:
    """The HGRN2 mixer: a gated linear recurrence in which one gate f both decays the state and, as 1 - f, weighs the new value.

    Per head a float32 state S [dim, vdim], zero at the start of a sequence:
    q = silu(Q h), f = lower + (1 - lower) * sigmoid(F h + bias), v = V h;
    S <- diag(f) S + (1 - f) v^T;  o = S^T q;  each head's o is RMS-normalised over vdim with the
    weight ``out_norm`` (shared by the heads) and the heads side by side go through ``o_proj``."""
    hidden_size: int
    num_heads: int
    head_dim: int
    value_head_dim: int
    eps: float
    q_proj: str
    f_proj: str
    f_bias: str
    lower: str
    v_proj: str
    out_norm: str
    o_proj: str

    def tensors(self) -> Mapping[str, TensorSpec]:
        hd, hv = self.num_heads * self.head_dim, self.num_heads * self.value_head_dim
        return {
            self.q_proj: TensorSpec((hd, self.hidden_size)),
            self.f_proj: TensorSpec((hd, self.hidden_size)),
            self.f_bias: TensorSpec((hd,), init=(0.0, 0.5)),
            self.lower: TensorSpec((hd,), init=(0.5, 0.1)),
            self.v_proj: TensorSpec((hv, self.hidden_size)),
            self.out_norm: TensorSpec((self.value_head_dim,)),
            self.o_proj: TensorSpec((self.hidden_size, hv)),
        }

    def cache_need(self):
        return StateNeed((self.num_heads, self.head_dim, self.value_head_dim))


@dataclass(frozen=True)
class TalkingAttentionSpec:
    """Grouped-query softmax attention whose heads' scores are mixed before the softmax.

    q = Q h, k = K h.  ``q_norm`` / ``k_norm``: RMSNorm of the WHOLE projection (one statistic per token
    over all heads) with a weight of that length.  ``values_are_keys``: the unnormalised k doubles as the
    value and the model has no v matrix.  No rotation; the position enters as a bias:
    a[j] = scale * q_j . k - slope_j * (distance), slope_j = 2^(-slope_exponent * (j + 1) / heads)
    (``slope_exponent`` None: no bias).  ``talk`` [heads, heads]: b[j] = sum_i talk[j, i] a[i]
    (None: b = a).  ``chunk`` c: position p sees s <= p with s // c == p // c (None: every s <= p).
    ``gate``: the heads side by side are multiplied by sigmoid(G h) before ``o_proj``."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    eps: float
    q_proj: str
    k_proj: str
    o_proj: str
    v_proj: Optional[str] = None
    q_norm: Optional[str] = None
    k_norm: Optional[str] = None
    talk: Optional[str] = None
    gate: Optional[str] = None
    chunk: Optional[int] = None
    slope_exponent: Optional[float] = 8.0

    @property
    def values_are_keys(self) -> bool:
        return self.v_proj is None

    def tensors(self) -> Mapping[str, TensorSpec]:
        qw, kw = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        t = {self.q_proj: TensorSpec((qw, self.hidden_size)), self.k_proj: TensorSpec((kw, self.hidden_size)),
             self.o_proj: TensorSpec((self.hidden_size, qw))}
        if self.v_proj is not None:
            t[self.v_proj] = TensorSpec((kw, self.hidden_size))
        if self.q_norm is not None:
            t[self.q_norm] = TensorSpec((qw,))
        if self.k_norm is not None:
            t[self.k_norm] = TensorSpec((kw,))
        if self.talk is not None:
            t[self.talk] = TensorSpec((self.num_heads, self.num_heads), init=(0.0, 0.35))
        if self.gate is not None:
            t[self.gate] = TensorSpec((qw, self.hidden_size))
        return t

    def cache_need(self):
        return KVCacheNeed(self.num_kv_heads, self.head_dim, chunk=self.chunk)


@dataclass(frozen=True)
class PostNormBlockSpec:
    """x += scale1 * norm1(mixer(x)); x += scale2 * norm2(ffn(x)).  No norm stands before a sublayer: what it
    returns is normalised before it is added; ``mixer_scale`` / ``ffn_scale`` name per-feature vectors (layer scale).
    ``ffn`` None: the block has no feed-forward (and neither its norm nor its scale)."""
    hidden_size: int
    mixer: object
    mixer_norm: object
    mixer_scale: str
    ffn: Optional[object] = None
    ffn_norm: Optional[object] = None
    ffn_scale: Optional[str] = None

    def tensors(self) -> Mapping[str, TensorSpec]:
        t = {}
        for part in (self.mixer, self.mixer_norm, self.ffn, self.ffn_norm):
            if part is not None:
                t.update(part.tensors())
        t[self.mixer_scale] = TensorSpec((self.hidden_size,))
        if self.ffn is not None:
            t[self.ffn_scale] = TensorSpec((self.hidden_size,))
        return t

    def cache_need(self):
        return self.mixer.cache_need()


# --------------------------------------------------------------------------- parts of sandwich-norm hybrid decoders
@dataclass(frozen=True)
class NormedEmbeddingSpec:
    """x[t] = norm(table[id_t]).  ``keep``: the rows are also kept for the step (a later part adds them to the
    stream again, see :class:`StreamInjectSpec`)."""
    vocab_size: int
    hidden_size: int
    weight: str
    norm: object
    keep: bool = False
    unused: Tuple[str, ...] = ()          # tables [rows, width] a folder may hold although no part reads them

    def tensors(self) -> Mapping[str, TensorSpec]:
        t = {self.weight: TensorSpec((self.vocab_size, self.hidden_size)), **self.norm.tensors()}
        for name in self.unused:
            t[name] = TensorSpec((None, self.hidden_size), optional=True)
        return t


@dataclass(frozen=True)
class StreamInjectSpec:
    """A step between layers that only adds to the stream: x += row ``row`` of the table ``table`` [rows, width]
    (one vector for all tokens), and, with ``add_embedding``, the rows the embedding kept.  It stands in the
    schedule like a layer and keeps nothing in the cache."""
    hidden_size: int
    table: str
    rows: int
    row: int
    add_embedding: bool = False

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {self.table: TensorSpec((self.rows, self.hidden_size), init=(0.0, 0.3))}

    def cache_need(self):
        return None


@dataclass(frozen=True)
class RetentionSpec:
    """Linear attention with one fixed decay per head, no softmax and no denominator.  Per head a float32 state
    S [dim, vdim], zero at the start of a sequence: S <- decay_h S + (k * key_scale) v^T, o = S^T q.  Each head's o
    is divided by its root mean square (no weight), the heads side by side are multiplied by silu(G h) and go
    through ``o_proj``."""
    hidden_size: int
    num_heads: int
    head_dim: int
    value_head_dim: int
    decay: Tuple[float, ...]
    key_scale: float
    eps: float
    q_proj: str
    k_proj: str
    v_proj: str
    g_proj: str
    o_proj: str

    def tensors(self) -> Mapping[str, TensorSpec]:
        hd, hv = self.num_heads * self.head_dim, self.num_heads * self.value_head_dim
        return {self.q_proj: TensorSpec((hd, self.hidden_size)), self.k_proj: TensorSpec((hd, self.hidden_size)),
                self.v_proj: TensorSpec((hv, self.hidden_size)), self.g_proj: TensorSpec((hv, self.hidden_size)),
                self.o_proj: TensorSpec((self.hidden_size, hv))}

    def cache_need(self):
        return StateNeed((self.num_heads, self.head_dim, self.value_head_dim))


@dataclass(frozen=True)
class TimeMixSpec:
    """RWKV-style time mixing.  With h' the previous token's input (zeros before the first), each of r, k, v, g, w
    reads its own blend h + (h' - h) * mu_s.  Per head a float32 state S [dim, dim]: the decay is
    w = exp(-exp(W2 tanh(W1 mix_w) + w0)) per token, head and key channel; o = (S + diag(u) k v^T)^T r (the bonus u
    for the current token only), then S <- diag(w) S + k v^T.  Each head's o is divided by its root mean square,
    times ``out_norm`` (per head and channel), times silu(G mix_g), then ``o_proj``.  The previous token's input is
    part of the state.  ``rank`` (the width of the decay's bottleneck) None: the stored tensors give it."""
    hidden_size: int
    num_heads: int
    head_dim: int
    eps: float
    mu: Tuple[str, str, str, str, str]        # the blends of r, k, v, g, w
    r_proj: str
    k_proj: str
    v_proj: str
    g_proj: str
    w1: str
    w2: str
    w0: str
    bonus: str
    out_norm: str
    o_proj: str
    rank: Optional[int] = None

    def tensors(self) -> Mapping[str, TensorSpec]:
        hd, W = self.num_heads * self.head_dim, self.hidden_size
        t = {name: TensorSpec((W,), init=(0.5, 0.25)) for name in self.mu}
        for name in (self.r_proj, self.k_proj, self.v_proj, self.g_proj):
            t[name] = TensorSpec((hd, W))
        t[self.w1] = TensorSpec((self.rank, W))
        t[self.w2] = TensorSpec((hd, self.rank))
        t[self.w0] = TensorSpec((hd,), init=(-1.5, 1.0))
        t[self.bonus] = TensorSpec((self.num_heads, self.head_dim), init=(0.3, 0.3))
        t[self.out_norm] = TensorSpec((hd,))
        t[self.o_proj] = TensorSpec((W, hd))
        return t

    def cache_need(self):
        return (StateNeed((self.num_heads, self.head_dim, self.head_dim)), StateNeed((self.hidden_size,)))


@dataclass(frozen=True)
class GatedUnitSpec:
    """minGRU: an element-wise gated recurrence whose gates read only the current token.  z = sigmoid(Z h + bz),
    u = X h + bx, candidate = u + 1/2 where u >= 0 and sigmoid(u) where u < 0; S <- (1 - z) S + z * candidate per
    element of a float32 state [width]; the output is ``o_proj``(S * silu(G h))."""
    hidden_size: int
    width: int
    z_proj: str
    z_bias: str
    x_proj: str
    x_bias: str
    g_proj: str
    o_proj: str

    def tensors(self) -> Mapping[str, TensorSpec]:
        n, W = self.width, self.hidden_size
        return {self.z_proj: TensorSpec((n, W)), self.z_bias: TensorSpec((n,), init=(0.0, 0.5)),
                self.x_proj: TensorSpec((n, W)), self.x_bias: TensorSpec((n,), init=(0.0, 0.5)),
                self.g_proj: TensorSpec((n, W)), self.o_proj: TensorSpec((W, n))}

    def cache_need(self):
        return StateNeed((self.width,))


@dataclass(frozen=True)
class RealGatedRecurrenceSpec:
    """The recurrent block around a real-gated linear recurrent unit (RG-LRU).  Two branches of ``width`` channels:
    y = gelu_tanh(``y_proj`` h + ``y_bias``) and u = conv(``x_proj`` h + ``x_bias``), a causal convolution per channel
    over time (``conv`` [width, taps], the last column is the current token's, zeros before the start, plus
    ``conv_bias``; no activation).  u in ``blocks`` equal parts: r = sigmoid(``a_gate``[b] u_b + ``a_bias``[b]),
    i = sigmoid(``x_gate``[b] u_b + ``x_bias_gate``[b]) with square matrices [out, in] per part.
    log a = -``decay_scale`` * r * softplus(``decay``); S <- a S + sqrt(1 - a^2) * i * u per channel of a float32 state
    that starts at zero; the output is ``o_proj``(S * y).  The convolution's last taps - 1 inputs are state too.
    ``gate_terms`` 2: where the gate products' operands are bfloat16, u enters them as two terms (its rounding and what the
    rounding left out), so that the gates see 16 bits of u instead of 8."""
    hidden_size: int
    width: int
    blocks: int
    taps: int
    decay_scale: float
    y_proj: str
    y_bias: str
    x_proj: str
    x_bias: str
    conv: str
    conv_bias: str
    a_gate: str
    a_bias: str
    x_gate: str
    x_bias_gate: str
    decay: str
    o_proj: str
    gate_terms: int = 1

    def tensors(self) -> Mapping[str, TensorSpec]:
        n, W, B = self.width, self.hidden_size, self.blocks
        bs = n // B
        return {self.y_proj: TensorSpec((n, W)), self.y_bias: TensorSpec((n,), init=(0.0, 0.3)),
                self.x_proj: TensorSpec((n, W)), self.x_bias: TensorSpec((n,), init=(0.0, 0.3)),
                self.conv: TensorSpec((n, self.taps), init=(0.0, 0.4)), self.conv_bias: TensorSpec((n,), init=(0.0, 0.3)),
                self.a_gate: TensorSpec((B, bs, bs), init=(0.0, 0.2)), self.a_bias: TensorSpec((B, bs), init=(0.0, 0.5)),
                self.x_gate: TensorSpec((B, bs, bs), init=(0.0, 0.2)), self.x_bias_gate: TensorSpec((B, bs), init=(0.0, 0.5)),
                self.decay: TensorSpec((n,), init=(0.0, 1.0)), self.o_proj: TensorSpec((W, n))}

    def cache_need(self):
        """Entry 0: the recurrence's state; entry 1: the convolution's last inputs."""
        return (StateNeed((self.width,)), StateNeed((max(self.taps - 1, 1), self.width)))


@dataclass(frozen=True)
class RotaryValueAttentionSpec:
    """Grouped-query softmax attention whose values carry positions too.  q and k are rotated on their first
    ``position.rotary_dim`` entries (:class:`RotarySpec`).  ``value_norm``: each value head is divided by its root
    mean square (no weight) before it is cached.  ``value_position``: the value of position j is rotated by j over
    that description's width before it is cached, and each head's summed output at position i is rotated back by
    -i.  Causal, optional window, plain softmax; key and value heads may differ in width.  ``v_proj`` None: the
    values are the keys as projected, before their rotation, and the model has no v matrix.  ``weight_terms``: on the
    tensor-core routes a softmax weight, formed in float32, enters the weighted sum as one bfloat16 number or as two
    (its rounding and what the rounding left out: 16 bits of the float32 weight, two products)."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_head_dim: int
    scale: float
    eps: float
    q_proj: str
    k_proj: str
    v_proj: Optional[str]
    o_proj: str
    position: Optional[RotarySpec] = None
    value_norm: bool = False
    value_position: Optional[RotarySpec] = None
    window: Optional[int] = None
    weight_terms: int = 1

    def tensors(self) -> Mapping[str, TensorSpec]:
        W = self.hidden_size
        t = {self.q_proj: TensorSpec((self.num_heads * self.head_dim, W)),
             self.k_proj: TensorSpec((self.num_kv_heads * self.head_dim, W)),
             self.o_proj: TensorSpec((W, self.num_heads * self.value_head_dim))}
        if self.v_proj is not None:
            t[self.v_proj] = TensorSpec((self.num_kv_heads * self.value_head_dim, W))
        return t

    def cache_need(self):
        return KVCacheNeed(self.num_kv_heads, self.head_dim, self.window,
                           None if self.value_head_dim == self.head_dim else self.value_head_dim)


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Several mixers side by side that read the same input; the result is the sum of ``scales[i] * mixers[i](h)``.
    Each keeps its own cache entry (``cache_need`` is the tuple of theirs)."""
    mixers: Tuple[object, ...]
    scales: Tuple[float, ...]

    def tensors(self) -> Mapping[str, TensorSpec]:
        t = {}
        for m in self.mixers:
            t.update(m.tensors())
        return t

    def cache_need(self):
        return tuple(m.cache_need() for m in self.mixers)


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """A mixture of gated feed-forwards without biases.  Router logits z = R h in 32-bit; an expert is
    down(act(gate h) * (up h)).  ``experts`` names each expert's (gate, up, down) tensors.

    ``scoring`` "chosen" (the default): each token runs the ``top`` experts with the largest logits, weighted by the
    softmax over those logits only.  ``scoring`` "all": the scores are the softmax over all experts, the ``top`` largest
    scores are chosen and the weights are those scores times ``weight_scale``, not renormalised.  ``scoring`` "sigmoid":
    the scores are sigmoid(z) per expert, chosen and weighted like "all".  ``weight_on`` "output" (the default): the
    weight multiplies the expert's result; "input": it multiplies what the expert reads, and the results are summed as
    they are (the two differ because an expert is not linear).  ``groups`` =
    (count, keep): the experts form ``count`` equal groups of neighbours, a group's score is its largest score, and only
    experts of the ``keep`` best groups can be chosen (None: no such limit).  ``shared``: a gated feed-forward that
    every token runs, added to the sum; with ``shared_gate`` (a tensor [1, hidden]) it is first multiplied by
    sigmoid(shared_gate . h), one number per token."""
    hidden_size: int
    intermediate_size: int
    top: int
    activation: str
    router: str
    experts: Tuple[Tuple[str, str, str], ...]
    scoring: str = "chosen"
    weight_scale: float = 1.0
    groups: Optional[Tuple[int, int]] = None
    shared: Optional[GatedMLPSpec] = None
    shared_gate: Optional[str] = None
    weight_on: str = "output"

    def tensors(self) -> Mapping[str, TensorSpec]:
        t = {self.router: TensorSpec((len(self.experts), self.hidden_size), init=(0.0, 0.3))}
        for gate, up, down in self.experts:
            t[gate] = TensorSpec((self.intermediate_size, self.hidden_size))
            t[up] = TensorSpec((self.intermediate_size, self.hidden_size))
            t[down] = TensorSpec((self.hidden_size, self.intermediate_size))
        if self.shared is not None:
            t.update(self.shared.tensors())
        if self.shared_gate is not None:
            t[self.shared_gate] = TensorSpec((1, self.hidden_size), init=(0.0, 0.1))
        return t

    def cache_need(self):
        return None


@dataclass(frozen=True)
class TokenSideSpec:
    """A per-layer token input: e = columns ``offset`` .. ``offset + dim`` of row id_t of ``table``;
    g = act(``gate`` x) * e; y = ``proj`` g; x += y / rms(y) * ``norm``."""
    hidden_size: int
    dim: int
    vocab_size: int
    table: str
    table_width: int
    offset: int
    activation: str
    gate: str
    proj: str
    norm: RMSNormSpec

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {self.table: TensorSpec((self.vocab_size, self.table_width)), self.gate: TensorSpec((self.dim, self.hidden_size)),
                self.proj: TensorSpec((self.hidden_size, self.dim)), **self.norm.tensors()}


@dataclass(frozen=True)
class SandwichBlockSpec:
    """x += post1(mixer(pre1(x))); x += post2(ffn(pre2(x))); then the token side input, if any.  A norm stands
    before and after each sublayer.  ``ffn`` None: no feed-forward; its norms may then still be stored
    (``unused``: tensors a folder may hold that no part reads)."""
    hidden_size: int
    mixer_norm: object
    mixer: object
    mixer_post_norm: object
    ffn_norm: Optional[object] = None
    ffn: Optional[object] = None
    ffn_post_norm: Optional[object] = None
    side: Optional[TokenSideSpec] = None
    unused: Tuple[str, ...] = ()

    def tensors(self) -> Mapping[str, TensorSpec]:
        t = {}
        for part in (self.mixer_norm, self.mixer, self.mixer_post_norm, self.ffn_norm, self.ffn, self.ffn_post_norm, self.side):
            if part is not None:
                t.update(part.tensors())
        for name in self.unused:
            t.setdefault(name, TensorSpec((self.hidden_size,), optional=True))
        return t

    def cache_need(self):
        return self.mixer.cache_need()


# --------------------------------------------------------------------------- parts of latent-attention decoders
@dataclass(frozen=True)
class GroupRMSNormSpec:
    """RMS norm in groups: the row is split into ``groups`` equal consecutive parts, each divided by its own
    sqrt(mean(part^2) + eps); the whole row is then multiplied by ``weight``.  One group is the plain RMS norm."""
    size: int
    eps: float
    groups: int
    weight: str

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {self.weight: TensorSpec((self.size,))}


@dataclass(frozen=True)
class CausalConvSpec:
    """A short causal convolution over time on each channel, added to its input:
    y_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the sequence's start; ``weight`` [width, taps], no
    bias.  The last taps - 1 inputs of a sequence are its state."""
    width: int
    taps: int
    weight: str

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {self.weight: TensorSpec((self.width, self.taps), init=(0.0, 0.2))}

    def cache_need(self):
        return StateNeed((max(self.taps - 1, 1), self.width))


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Softmax attention whose keys and values are made from a small latent per token, which is all that is cached.

    q = Q h, laid out head by head as [head_dim unrotated, rot_dim rotated].  D h has kv_rank + rot_dim rows: the first
    kv_rank, RMS-normalised with ``latent_norm`` (a plain weight), are the latent c; the last rot_dim are one rotated key
    part shared by all heads.  Per head k = UK c and v = UV c; score = (q_unrotated . k + q_rotated . k_rotated) * scale.
    ``position`` (a :class:`RotarySpec` over the rot_dim part) turns the rotated parts of q and of the key by the token's
    position.  ``window`` w: position i sees j with 0 <= i - j < w (None: every j <= i).  ``sink``: a tensor [heads]; exp
    of it joins the softmax's denominator, with no key and no value.  ``gate``: the heads side by side are multiplied by
    sigmoid(G h) before ``o_proj``; with ``gate_per_head`` G has one row per head and the whole head takes one number.
    ``q_rank`` r: the queries go through a latent of their own, q = ``q_proj`` (rmsnorm(``q_down`` h) * ``q_norm``),
    with ``q_down`` [r, hidden], ``q_norm`` [r] and ``q_proj`` [heads * (head_dim + rot_dim), r].  ``weight_terms``: as
    :class:`RotaryValueAttentionSpec`'s."""
    hidden_size: int
    num_heads: int
    head_dim: int
    rot_dim: int
    value_head_dim: int
    kv_rank: int
    scale: float
    eps: float
    q_proj: str
    down_proj: str
    latent_norm: str
    k_up: str
    v_up: str
    o_proj: str
    position: Optional[RotarySpec] = None
    window: Optional[int] = None
    sink: Optional[str] = None
    gate: Optional[str] = None
    gate_per_head: bool = False
    q_rank: Optional[int] = None
    q_down: Optional[str] = None
    q_norm: Optional[str] = None
    weight_terms: int = 1

    def tensors(self) -> Mapping[str, TensorSpec]:
        W, H = self.hidden_size, self.num_heads
        t = {self.q_proj: TensorSpec((H * (self.head_dim + self.rot_dim), self.q_rank or W)),
             self.down_proj: TensorSpec((self.kv_rank + self.rot_dim, W)),
             self.latent_norm: TensorSpec((self.kv_rank,)),
             self.k_up: TensorSpec((H * self.head_dim, self.kv_rank)),
             self.v_up: TensorSpec((H * self.value_head_dim, self.kv_rank)),
             self.o_proj: TensorSpec((W, H * self.value_head_dim))}
        if self.sink is not None:
            t[self.sink] = TensorSpec((H,), init=(0.0, 1.0))
        if self.gate is not None:
            t[self.gate] = TensorSpec((H if self.gate_per_head else H * self.value_head_dim, W))
        if self.q_rank:
            t[self.q_down] = TensorSpec((self.q_rank, W))
            t[self.q_norm] = TensorSpec((self.q_rank,))
        return t

    def cache_need(self):
        streams = (PagedStream("latent", 1, self.kv_rank),)
        if self.rot_dim:
            streams += (PagedStream("rotated_key", 1, self.rot_dim),)
        return PagedCacheNeed(streams, self.window, separate=True)      # also where kv_rank == rot_dim


@dataclass(frozen=True)
class DepthAverageBlockSpec:
    """A pre-norm block with a residual multiplier, an input convolution before each sublayer and a weighted average
    over depth.  x += mult * mixer(conv1(norm1(x))); x += mult * ffn(conv2(norm2(x))) (``ffn`` None: no feed-forward).
    With X_0 the embedding's output and X_(d) the result of the block at depth d - 1 before averaging, the block at
    depth ``depth`` hands on sum_j ``average``[j] * X_j, j = 0 .. depth + 1 (``average`` None: no averaging).  ``depths`` is
    the number of such blocks in the model: a step keeps depths + 1 rows per token.  ``mixer_conv`` / ``ffn_conv`` may be
    None."""
    hidden_size: int
    depth: int
    depths: int
    residual_mult: float
    mixer_norm: object
    mixer: object
    mixer_conv: Optional[CausalConvSpec] = None
    ffn_norm: Optional[object] = None
    ffn: Optional[object] = None
    ffn_conv: Optional[CausalConvSpec] = None
    average: Optional[str] = None

    def tensors(self) -> Mapping[str, TensorSpec]:
        t = {}
        for part in (self.mixer_norm, self.mixer, self.mixer_conv, self.ffn_norm, self.ffn, self.ffn_conv):
            if part is not None:
                t.update(part.tensors())
        if self.average is not None:
            t[self.average] = TensorSpec((self.depth + 2,), init=(1.0 / (self.depth + 2), 0.1))
        return t

    def cache_need(self):
        """Entry 0: the mixer's; entries 1 and 2: the states of the two convolutions (None where there is none)."""
        return (self.mixer.cache_need(), self.mixer_conv.cache_need() if self.mixer_conv is not None else None,
                self.ffn_conv.cache_need() if self.ffn_conv is not None and self.ffn is not None else None)


# --------------------------------------------------------------------------- the order
@dataclass(frozen=True)
class LayerCall:
    """One entry of the schedule: run ``layer`` (an index into ``ModelPlan.layers``).

    ``cache`` is the id of the cache entry the layer's mixer reads; it defaults to a
    fresh id per call.  Two calls may name the same layer (shared weights, each with a
    cache of its own) and a call may name another call's cache id with ``store`` False:
    then it reads what that call stored and stores nothing itself."""
    layer: int
    cache: Optional[object] = None       # an int; parts that keep several entries derive (cache, j) for entry j
    store: bool = True


@dataclass(frozen=True)
class ModelPlan:
    """All of a model that the loader, the cache manager and the engine need."""
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: EmbeddingSpec
    layers: Tuple[object, ...]
    schedule: Tuple[LayerCall, ...]
    final_norm: object
    lm_head: LMHeadSpec
    extra: Mapping[str, object] = field(default_factory=dict)

    def resolved_schedule(self) -> Tuple[LayerCall, ...]:
        """The schedule with every ``cache`` id filled in: a call without one gets the
        smallest id that no call names."""
        named = {c.cache for c in self.schedule if c.cache is not None}
        out, nxt = [], 0
        for call in self.schedule:
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"schedule names layer {call.layer}; the model has {len(self.layers)}")
            if call.cache is None:
                while nxt in named:
                    nxt += 1
                named.add(nxt)
                call = LayerCall(call.layer, nxt, call.store)
            out.append(call)
        stored = {c.cache for c in out if c.store}
        for call in out:
            if not call.store and call.cache not in stored:
                raise ValueError(f"layer call reads cache {call.cache}, which no call stores")
        return tuple(out)

    def duplicates(self) -> Mapping[str, str]:
        """Names a model folder may hold beside the inventory, each with the tensor it must be an exact
        copy of: the head of a tied model stored under a name of its own."""
        if self.lm_head.tied and self.lm_head.stored_as and self.lm_head.stored_as != self.lm_head.weight:
            return {self.lm_head.stored_as: self.lm_head.weight}
        return {}

    def tensors(self) -> Mapping[str, TensorSpec]:
        t = dict(self.embedding.tensors())
        for layer in self.layers:
            for name, spec in layer.tensors().items():
                if name in t and t[name] != spec:
                    raise ValueError(f"tensor {name} is described twice with different shapes")
                t[name] = spec
        t.update(self.final_norm.tensors())
        t.update(self.lm_head.tensors())
        return t
