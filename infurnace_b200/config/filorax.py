"""Typed configuration of the Filorax decoder, read from config.json's own keys.

config.json of this design is nested: ``vocab``, ``width``, ``residual_mult``, ``norm.eps`` and ``norm.groups`` (the
norms work in that many equal parts of the row), ``canon.taps`` (the length of the short causal convolution in front of
every sublayer) and a list ``layers`` whose entries give ``type`` ("latent_attention", "latent_attention_2" or
"latent_attention_3"), the mixer's sizes and constants under ``mixer`` (``heads``, ``dim``, ``vdim``, ``kv_rank``,
``scale``; ``mask.size`` for a sliding window; ``rot_dim`` with ``rot.base`` and ``rot.dims`` for a rotated part) and the
feed-forward under ``mlp`` (null: the layer has none; else ``kind`` "moe" with ``expert.ff``, ``router.experts``,
``router.top``, ``router.scale``, ``router.groups.count`` / ``keep`` and optionally ``shared.ff``).  Every size and every
constant that can differ between two models of the design comes from the file; what the design fixes is in the plan
builder.  The layers are kept as validated plain mappings, so ``to_dict`` gives back what ``from_dict`` read.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping, Tuple

from ..errors import ModelConfigError
from .lunelorn import _int, _map, _num

WINDOW_SINK_GATE, ROTATED_SINK_GATE, WINDOW_PLAIN = "latent_attention", "latent_attention_2", "latent_attention_3"
MIXERS = (WINDOW_SINK_GATE, ROTATED_SINK_GATE, WINDOW_PLAIN)


def _check_mixer(kind, m, where):
    if kind not in MIXERS:
        raise ModelConfigError(f"config.json: {where[:-6]}type {kind!r} is no mixer of this design ({', '.join(map(repr, MIXERS))})")
    for key in ("heads", "dim", "vdim", "kv_rank"):
        _int(m, key, where)
    _num(m, "scale", where)
    rot_dim = m.get("rot_dim")
    if kind == ROTATED_SINK_GATE or rot_dim:
        rot_dim = _int(m, "rot_dim", where)
        rot = _map(m, "rot", where)
        dims = _int(rot, "dims", where + "rot.", least=2)
        _num(rot, "base", where + "rot.", positive=True)
        if dims % 2 or dims > rot_dim:
            raise ModelConfigError(f"config.json: {where}rot.dims {dims} must be even and at most rot_dim {rot_dim}")
    if kind != ROTATED_SINK_GATE or m.get("mask") is not None:
        _int(_map(m, "mask", where), "size", where + "mask.")


def _check_mlp(mlp, where, width):
    if mlp is None:
        return
    if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
        raise ModelConfigError(f"config.json: {where}mlp.kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r}: "
                               "only 'moe' feed-forwards exist in this design")
    _int(_map(mlp, "expert", where + "mlp."), "ff", where + "mlp.expert.")
    router = _map(mlp, "router", where + "mlp.")
    experts, top = _int(router, "experts", where + "mlp.router."), _int(router, "top", where + "mlp.router.")
    if router.get("scale") is not None:
        _num(router, "scale", where + "mlp.router.")
    count = keep = 1
    if router.get("groups") is not None:
        groups = _map(router, "groups", where + "mlp.router.")
        count, keep = _int(groups, "count", where + "mlp.router.groups."), _int(groups, "keep", where + "mlp.router.groups.")
    if experts % count or keep > count:
        raise ModelConfigError(f"config.json: {where}mlp.router.groups: {count} groups must divide the {experts} experts, and keep "
                               f"{keep} cannot exceed them")
    if top > keep * (experts // count):
        raise ModelConfigError(f"config.json: {where}mlp.router.top {top} exceeds the experts of the {keep} groups that are kept")
    if mlp.get("shared") is not None:
        _int(_map(mlp, "shared", where + "mlp."), "ff", where + "mlp.shared.")


@dataclass(frozen=True)
class FiloraxConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    norm_groups: int
    residual_mult: float
    conv_taps: int
    layers: Tuple[Mapping[str, Any], ...]

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "FiloraxConfig":
        if not isinstance(d, Mapping):
            raise ModelConfigError("config.json must hold a JSON object")
        arch = d.get("architecture")
        if not isinstance(arch, str):
            archs = d.get("architectures")
            arch = archs[0] if isinstance(archs, (list, tuple)) and archs else None
        if not isinstance(arch, str):
            raise ModelConfigError("config.json lacks required key 'architecture'")
        norm = _map(d, "norm", "")
        eps = _num(norm, "eps", "norm.", positive=True)
        groups = _int(norm, "groups", "norm.") if norm.get("groups") is not None else 1
        width = _int(d, "width", "")
        if width % groups:
            raise ModelConfigError(f"config.json: norm.groups {groups} does not divide width {width}")
        taps = _int(_map(d, "canon", ""), "taps", "canon.") if d.get("canon") is not None else 1
        mult = _num(d, "residual_mult", "") if d.get("residual_mult") is not None else 1.0
        entries = d.get("layers")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ModelConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(e, Mapping):
                raise ModelConfigError(f"config.json: {where[:-1]} must be an object")
            _check_mixer(e.get("type"), _map(e, "mixer", where), where + "mixer.")
            _check_mlp(e.get("mlp"), where, width)
            layers.append(copy.deepcopy({"type": e["type"], "mixer": dict(e["mixer"]), "mlp": e.get("mlp")}))
        return cls(architecture=arch, vocab_size=_int(d, "vocab", ""), hidden_size=width, norm_eps=eps, norm_groups=groups,
                   residual_mult=mult, conv_taps=taps, layers=tuple(layers))

    def to_dict(self):
        return {"architecture": self.architecture, "canon": {"taps": self.conv_taps}, "layers": copy.deepcopy(list(self.layers)),
                "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "residual_mult": self.residual_mult,
                "vocab": self.vocab_size, "width": self.hidden_size}
