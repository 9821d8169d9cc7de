"""Typed configuration of the Golonex decoder, read from config.json's own keys.

config.json of this design is nested: ``vocab``, ``width``, ``norm.eps``, optionally ``logit_softcap`` and
``token_side.dim`` (a per-layer token input), and a list ``layers`` whose entries give ``type`` ("rglru",
"latent_attention" or "attention"), the mixer's sizes and constants under ``mixer`` and the feed-forward under ``mlp``
(null: the layer has none; else ``kind`` "moe" with ``expert.ff``, ``router.experts``, ``router.top`` and optionally
``shared.ff``).  Mixer keys: ``rglru``: ``width``, ``blocks``, ``conv`` (taps); ``latent_attention``: ``heads``, ``dim``,
``rot_dim``, ``vdim``, ``kv_rank``, ``q_rank``, ``scale``, ``rot.base`` / ``rot.dims``, ``mask.size``; ``attention``: ``heads``,
``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot.base`` / ``rot.dims`` / ``rot.scaling`` (``factor``, ``original``, ``fast``,
``slow``), ``mask.size``.  Every size and every constant that can differ between two models of the design comes from
the file; what the design fixes is in the plan builder.  The layers are kept as validated plain mappings, so
``to_dict`` gives back what ``from_dict`` read.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import ModelConfigError
from .lunelorn import _int, _map, _num

RGLRU, LATENT, ATTENTION = "rglru", "latent_attention", "attention"
MIXERS = (RGLRU, LATENT, ATTENTION)


def _check_rot(m, where, widest):
    rot = _map(m, "rot", where)
    dims = _int(rot, "dims", where + "rot.", least=2)
    _num(rot, "base", where + "rot.", positive=True)
    if dims % 2 or dims > widest:
        raise ModelConfigError(f"config.json: {where}rot.dims {dims} must be even and at most {widest}")
    if rot.get("scaling") is not None:
        sc = _map(rot, "scaling", where + "rot.")
        for key in ("factor", "original", "fast", "slow"):
            _num(sc, key, where + "rot.scaling.", positive=True)


def _check_mask(m, where):
    if m.get("mask") is not None:
        _int(_map(m, "mask", where), "size", where + "mask.")


def _check_mixer(kind, m, where):
    if kind not in MIXERS:
        raise ModelConfigError(f"config.json: {where[:-6]}type {kind!r} is no mixer of this design ({', '.join(map(repr, MIXERS))})")
    if kind == RGLRU:
        width, blocks = _int(m, "width", where), _int(m, "blocks", where)
        _int(m, "conv", where)
        if width % blocks:
            raise ModelConfigError(f"config.json: {where}blocks {blocks} does not divide width {width}")
        return
    _num(m, "scale", where)
    _check_mask(m, where)
    if kind == LATENT:
        for key in ("heads", "dim", "vdim", "kv_rank", "q_rank"):
            _int(m, key, where)
        rot_dim = _int(m, "rot_dim", where, least=0) if m.get("rot_dim") is not None else 0
        if rot_dim:
            _check_rot(m, where, rot_dim)
        return
    heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv:
        raise ModelConfigError(f"config.json: {where}heads {heads} is not a multiple of kv_heads {kv}")
    dim = _int(m, "dim", where)
    vdim = _int(m, "vdim", where) if m.get("vdim") is not None else dim
    if vdim != dim:
        raise ModelConfigError(f"config.json: {where}vdim {vdim} differs from dim {dim}, but this mixer's values are its keys")
    if m.get("rot") is not None:
        _check_rot(m, where, dim)


def _check_mlp(mlp, where):
    if mlp is None:
        return
    if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
        raise ModelConfigError(f"config.json: {where}mlp.kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r}: "
                               "only 'moe' feed-forwards exist in this design")
    _int(_map(mlp, "expert", where + "mlp."), "ff", where + "mlp.expert.")
    router = _map(mlp, "router", where + "mlp.")
    experts, top = _int(router, "experts", where + "mlp.router."), _int(router, "top", where + "mlp.router.")
    if top > experts:
        raise ModelConfigError(f"config.json: {where}mlp.router.top {top} exceeds experts {experts}")
    if mlp.get("shared") is not None:
        _int(_map(mlp, "shared", where + "mlp."), "ff", where + "mlp.shared.")


@dataclass(frozen=True)
class GolonexConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    logit_softcap: Optional[float]
    token_side_dim: Optional[int]
    layers: Tuple[Mapping[str, Any], ...]

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "GolonexConfig":
        if not isinstance(d, Mapping):
            raise ModelConfigError("config.json must hold a JSON object")
        arch = d.get("architecture")
        if not isinstance(arch, str):
            archs = d.get("architectures")
            arch = archs[0] if isinstance(archs, (list, tuple)) and archs else None
        if not isinstance(arch, str):
            raise ModelConfigError("config.json lacks required key 'architecture'")
        eps = _num(_map(d, "norm", ""), "eps", "norm.", positive=True)
        width = _int(d, "width", "")
        cap = _num(d, "logit_softcap", "", positive=True) if d.get("logit_softcap") is not None else None
        side = _int(_map(d, "token_side", ""), "dim", "token_side.") if d.get("token_side") is not None else None
        entries = d.get("layers")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ModelConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(e, Mapping):
                raise ModelConfigError(f"config.json: {where[:-1]} must be an object")
            _check_mixer(e.get("type"), _map(e, "mixer", where), where + "mixer.")
            _check_mlp(e.get("mlp"), where)
            layers.append(copy.deepcopy({"type": e["type"], "mixer": dict(e["mixer"]), "mlp": e.get("mlp")}))
        return cls(architecture=arch, vocab_size=_int(d, "vocab", ""), hidden_size=width, norm_eps=eps, logit_softcap=cap,
                   token_side_dim=side, layers=tuple(layers))

    def to_dict(self):
        out = {"architecture": self.architecture, "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
               "vocab": self.vocab_size, "width": self.hidden_size}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.token_side_dim is not None:
            out["token_side"] = {"dim": self.token_side_dim}
        return out
