"""Typed configuration of the Nunivik decoder.

Its config.json is nested: ``architecture`` (the name), ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``
and ``layers``, a list whose entries give ``type`` (``attention``, ``delta`` or ``mamba2``), the mixer's sizes under
``mixer`` and the feed-forward under ``mlp`` (``{"kind": "dense", "ff": n}`` or null).  Every size and every constant
is read from there; nothing is assumed equal between layers.  A key that is missing or of the wrong kind is
refused by name.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Optional

from .base import ConfigError

ARCHITECTURE = "Nunivik"


def _get(document: Any, path: str, key: str) -> Any:
    if not isinstance(document, dict) or key not in document:
        raise ConfigError(f"{path}{key}", "is missing")
    return document[key]


def _positive_int(document: Any, path: str, key: str) -> int:
    value = _get(document, path, key)
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"{path}{key}", f"must be a positive integer, got {value!r}")
    return value


def _positive_number(document: Any, path: str, key: str) -> float:
    value = _get(document, path, key)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not value > 0 or math.isinf(value):
        raise ConfigError(f"{path}{key}", f"must be a finite positive number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float  # 0: scores are not capped
    window: int  # 0: every earlier key is seen
    rot_dims: int  # 0: no rotation
    rot_base: float
    rot_factor: float
    v_mix: bool


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class Mamba2Mixer:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int


@dataclass(frozen=True)
class NunivikLayer:
    type: str
    mixer: Any
    ff: Optional[int]  # the dense feed-forward's inner width, None for a layer without one


@dataclass(frozen=True)
class NunivikConfig:
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    layers: tuple[NunivikLayer, ...]
    eos_token_ids: tuple[int, ...] = ()
    architecture: str = field(default=ARCHITECTURE)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, document: dict[str, Any]) -> "NunivikConfig":
        if not isinstance(document, dict):
            raise ConfigError("<root>", "must be a JSON object")
        if document.get("architecture") != ARCHITECTURE:
            raise ConfigError("architecture", f"must be {ARCHITECTURE!r}, got {document.get('architecture')!r}")
        entries = _get(document, "", "layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("layers", "must be a non-empty list")
        layers = []
        for index, entry in enumerate(entries):
            path = f"layers[{index}]."
            kind = _get(entry, path, "type")
            mixer = _get(entry, path, "mixer")
            if kind == "attention":
                parsed = _attention(mixer, path + "mixer.")
            elif kind == "delta":
                parsed = _delta(mixer, path + "mixer.")
            elif kind == "mamba2":
                parsed = _mamba2(mixer, path + "mixer.")
            else:
                raise ConfigError(path + "type", f"{kind!r} is not a mixer of this design (attention, delta, mamba2)")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                if _get(mlp, path + "mlp.", "kind") != "dense":
                    raise ConfigError(path + "mlp.kind", f"{mlp.get('kind')!r} is not supported (only 'dense')")
                ff = _positive_int(mlp, path + "mlp.", "ff")
            layers.append(NunivikLayer(kind, parsed, ff))
        mixing = [(i, l.mixer.kv_heads * l.mixer.vdim) for i, l in enumerate(layers) if l.type == "attention" and l.mixer.v_mix]
        for index, width in mixing[1:]:  # a later layer adds the first one's values to its own, head by head
            if width != mixing[0][1]:
                raise ConfigError(f"layers[{index}].mixer.v_mix", f"values of kv_heads * vdim = {width}, the first mixing layer has {mixing[0][1]}")
        eos = document.get("eos_token_id")
        eos_ids = tuple(eos if isinstance(eos, list) else [eos]) if eos is not None else ()
        return cls(vocab=_positive_int(document, "", "vocab"), width=_positive_int(document, "", "width"),
                   embedding_scale=_positive_number(_get(document, "", "embedding"), "embedding.", "scale"),
                   eps=_positive_number(_get(document, "", "norm"), "norm.", "eps"), layers=tuple(layers), eos_token_ids=eos_ids)

    def to_dict(self) -> dict[str, Any]:
        """The config.json document this configuration is read back from."""
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "attention":
                mixer: dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale, "v_mix": m.v_mix}
                if m.softcap:
                    mixer["softcap"] = m.softcap
                if m.window:
                    mixer["mask"] = {"size": m.window}
                if m.rot_dims:
                    mixer["rot"] = {"dims": m.rot_dims, "base": m.rot_base, "scaling": {"factor": m.rot_factor}}
            elif layer.type == "delta":
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv}
            else:
                mixer = {"heads": m.heads, "vdim": m.vdim, "state": m.state, "groups": m.groups, "norm_groups": m.norm_groups, "conv": m.conv}
            layers.append({"type": layer.type, "mixer": mixer, "mlp": {"kind": "dense", "ff": layer.ff} if layer.ff is not None else None})
        document: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                                    "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.eps}, "layers": layers}
        if self.eos_token_ids:
            document["eos_token_id"] = list(self.eos_token_ids)
        return document


def _attention(m: Any, path: str) -> AttentionMixer:
    heads, kv_heads = _positive_int(m, path, "heads"), _positive_int(m, path, "kv_heads")
    if heads % kv_heads:
        raise ConfigError(path + "kv_heads", f"{kv_heads} does not divide heads {heads}")
    dim = _positive_int(m, path, "dim")
    rot = m.get("rot")
    rot_dims, rot_base, rot_factor = 0, 1.0, 1.0
    if rot is not None:
        rot_dims = _positive_int(rot, path + "rot.", "dims")
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(path + "rot.dims", f"{rot_dims} must be even and at most dim {dim}")
        rot_base = _positive_number(rot, path + "rot.", "base")
        if rot.get("scaling") is not None:
            rot_factor = _positive_number(rot["scaling"], path + "rot.scaling.", "factor")
    mask = m.get("mask")
    window = _positive_int(mask, path + "mask.", "size") if mask is not None else 0
    softcap = _positive_number(m, path, "softcap") if m.get("softcap") is not None else 0.0
    return AttentionMixer(heads=heads, kv_heads=kv_heads, dim=dim, vdim=_positive_int(m, path, "vdim"), scale=_positive_number(m, path, "scale"),
                          softcap=softcap, window=window, rot_dims=rot_dims, rot_base=rot_base, rot_factor=rot_factor, v_mix=bool(m.get("v_mix", False)))


def _delta(m: Any, path: str) -> DeltaMixer:
    heads, kv_heads = _positive_int(m, path, "heads"), _positive_int(m, path, "kv_heads")
    if heads % kv_heads:
        raise ConfigError(path + "kv_heads", f"{kv_heads} does not divide heads {heads}")
    return DeltaMixer(heads=heads, kv_heads=kv_heads, dim=_positive_int(m, path, "dim"), vdim=_positive_int(m, path, "vdim"),
                      conv=_positive_int(m, path, "conv"))


def _mamba2(m: Any, path: str) -> Mamba2Mixer:
    heads, groups = _positive_int(m, path, "heads"), _positive_int(m, path, "groups")
    if heads % groups:
        raise ConfigError(path + "groups", f"{groups} does not divide heads {heads}")
    norm_groups = _positive_int(m, path, "norm_groups")
    vdim = _positive_int(m, path, "vdim")
    if (heads * vdim) % norm_groups:
        raise ConfigError(path + "norm_groups", f"{norm_groups} does not divide heads * vdim = {heads * vdim}")
    return Mamba2Mixer(heads=heads, vdim=vdim, state=_positive_int(m, path, "state"), groups=groups, norm_groups=norm_groups,
                       conv=_positive_int(m, path, "conv"))
