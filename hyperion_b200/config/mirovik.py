"""Typed configuration of the Mirovik decoder.

Its config.json is nested: ``architecture`` (the name), ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, ``layers`` and
``loop``.  An entry of ``layers`` gives ``type`` (``parallel`` or ``mamba1``), the mixer's sizes under ``mixer`` and the
feed-forward under ``mlp``: ``{"kind": "dense", "ff": n}``, ``{"kind": "moe", "router": {"experts": E, "top": k}, "expert":
{"ff": n}, "shared": {"ff": m}}`` or null.  A ``parallel`` mixer holds ``left`` (attention with a learned distance bias:
``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``bias_max``), ``right`` (retention: ``heads``, ``dim``, ``vdim``, ``decay`` per
head, ``rot.dims``, ``rot.base``) and the two scales.  ``loop`` = ``{"start": a, "stop": b, "times": n}``: the layers a .. b - 1 are
passed n times in a row with the same weights.  Every size and constant is read from there; nothing is assumed equal between
layers.  A key that is missing or of the wrong kind is refused by name.  ``buckets`` under ``left`` is this package's own
key: the rows of the distance-bias tensor when random weights are made (a checkpoint's tensor decides otherwise).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from .base import ConfigError
from .nunivik import _get, _positive_int, _positive_number

ARCHITECTURE = "Mirovik"


@dataclass(frozen=True)
class BiasedAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: int
    buckets: int = 32


@dataclass(frozen=True)
class RetentionSizes:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]
    rot_dims: int  # 0: no rotation
    rot_base: float


@dataclass(frozen=True)
class ParallelMixer:
    left: BiasedAttentionSizes
    right: RetentionSizes
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class SelectiveMixer:
    inner: int
    state: int
    dt_rank: int
    conv: int


@dataclass(frozen=True)
class DenseFF:
    ff: int


@dataclass(frozen=True)
class ExpertsFF:
    experts: int
    top: int
    ff: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class MirovikLayer:
    type: str
    mixer: Any
    mlp: Any  # DenseFF, ExpertsFF or None


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class MirovikConfig:
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    layers: tuple[MirovikLayer, ...]
    loop: Optional[Loop] = None
    eos_token_ids: tuple[int, ...] = ()
    architecture: str = field(default=ARCHITECTURE)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def runs(self) -> list[tuple[int, Optional[int]]]:
        """(layer, number of the pass it opens or None) in the order the layers run."""
        count = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(count)]
        a, b = self.loop.start, self.loop.stop
        order: list[tuple[int, Optional[int]]] = [(i, None) for i in range(a)]
        for t in range(self.loop.times):
            order += [(i, t if i == a else None) for i in range(a, b)]
        return order + [(i, None) for i in range(b, count)]

    @classmethod
    def from_dict(cls, document: dict[str, Any]) -> "MirovikConfig":
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
            if kind == "parallel":
                parsed: Any = _parallel(mixer, path + "mixer.")
            elif kind == "mamba1":
                parsed = SelectiveMixer(inner=_positive_int(mixer, path + "mixer.", "inner"), state=_positive_int(mixer, path + "mixer.", "state"),
                                        dt_rank=_positive_int(mixer, path + "mixer.", "dt_rank"), conv=_positive_int(mixer, path + "mixer.", "conv"))
            else:
                raise ConfigError(path + "type", f"{kind!r} is not a mixer of this design (parallel, mamba1)")
            layers.append(MirovikLayer(kind, parsed, _mlp(entry.get("mlp"), path + "mlp.")))
        loop = None
        if document.get("loop") is not None:
            raw = document["loop"]
            start, stop = _get(raw, "loop.", "start"), _get(raw, "loop.", "stop")
            for name, value in (("start", start), ("stop", stop)):
                if isinstance(value, bool) or not isinstance(value, int):
                    raise ConfigError("loop." + name, f"must be an integer, got {value!r}")
            if not 0 <= start < stop <= len(layers):
                raise ConfigError("loop.stop", f"the layers {start} .. {stop} - 1 are not a run of the model's {len(layers)} layers")
            loop = Loop(start, stop, _positive_int(raw, "loop.", "times"))
        eos = document.get("eos_token_id")
        eos_ids = tuple(eos if isinstance(eos, list) else [eos]) if eos is not None else ()
        return cls(vocab=_positive_int(document, "", "vocab"), width=_positive_int(document, "", "width"),
                   embedding_scale=_positive_number(_get(document, "", "embedding"), "embedding.", "scale"),
                   eps=_positive_number(_get(document, "", "norm"), "norm.", "eps"), layers=tuple(layers), loop=loop, eos_token_ids=eos_ids)

    def to_dict(self) -> dict[str, Any]:
        """The config.json document this configuration is read back from."""
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "parallel":
                right: dict[str, Any] = {"heads": m.right.heads, "dim": m.right.dim, "vdim": m.right.vdim, "decay": list(m.right.decay)}
                if m.right.rot_dims:
                    right["rot"] = {"dims": m.right.rot_dims, "base": m.right.rot_base}
                mixer: dict[str, Any] = {"left": {"heads": m.left.heads, "kv_heads": m.left.kv_heads, "dim": m.left.dim, "vdim": m.left.vdim,
                                                  "scale": m.left.scale, "bias_max": m.left.bias_max, "buckets": m.left.buckets},
                                         "right": right, "left_scale": m.left_scale, "right_scale": m.right_scale}
            else:
                mixer = {"inner": m.inner, "state": m.state, "dt_rank": m.dt_rank, "conv": m.conv}
            if layer.mlp is None:
                mlp: Any = None
            elif isinstance(layer.mlp, DenseFF):
                mlp = {"kind": "dense", "ff": layer.mlp.ff}
            else:
                mlp = {"kind": "moe", "router": {"experts": layer.mlp.experts, "top": layer.mlp.top}, "expert": {"ff": layer.mlp.ff}}
                if layer.mlp.shared_ff is not None:
                    mlp["shared"] = {"ff": layer.mlp.shared_ff}
            layers.append({"type": layer.type, "mixer": mixer, "mlp": mlp})
        document: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                                    "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.eps}, "layers": layers}
        if self.loop is not None:
            document["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.eos_token_ids:
            document["eos_token_id"] = list(self.eos_token_ids)
        return document


def _number(document: Any, path: str, key: str) -> float:
    value = _get(document, path, key)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or value != value or value in (float("inf"), float("-inf")):
        raise ConfigError(f"{path}{key}", f"must be a finite number, got {value!r}")
    return float(value)


def _parallel(m: Any, path: str) -> ParallelMixer:
    left, right = _get(m, path, "left"), _get(m, path, "right")
    lp, rp = path + "left.", path + "right."
    heads, kv_heads = _positive_int(left, lp, "heads"), _positive_int(left, lp, "kv_heads")
    if heads % kv_heads:
        raise ConfigError(lp + "kv_heads", f"{kv_heads} does not divide heads {heads}")
    attention = BiasedAttentionSizes(heads=heads, kv_heads=kv_heads, dim=_positive_int(left, lp, "dim"), vdim=_positive_int(left, lp, "vdim"),
                                     scale=_positive_number(left, lp, "scale"), bias_max=_positive_int(left, lp, "bias_max"),
                                     buckets=_positive_int(left, lp, "buckets") if left.get("buckets") is not None else 32)
    r_heads, dim = _positive_int(right, rp, "heads"), _positive_int(right, rp, "dim")
    decay = _get(right, rp, "decay")
    if not isinstance(decay, list) or len(decay) != r_heads or any(isinstance(d, bool) or not isinstance(d, (int, float)) or not 0 <= d <= 1 for d in decay):
        raise ConfigError(rp + "decay", f"must list one decay in 0..1 per head ({r_heads}), got {decay!r}")
    rot = right.get("rot")
    rot_dims, rot_base = 0, 1.0
    if rot is not None:
        rot_dims = _positive_int(rot, rp + "rot.", "dims")
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(rp + "rot.dims", f"{rot_dims} must be even and at most dim {dim}")
        rot_base = _positive_number(rot, rp + "rot.", "base")
    retention = RetentionSizes(heads=r_heads, dim=dim, vdim=_positive_int(right, rp, "vdim"), decay=tuple(float(d) for d in decay),
                               rot_dims=rot_dims, rot_base=rot_base)
    return ParallelMixer(attention, retention, _number(m, path, "left_scale"), _number(m, path, "right_scale"))


def _mlp(mlp: Any, path: str):
    if mlp is None:
        return None
    kind = _get(mlp, path, "kind")
    if kind == "dense":
        return DenseFF(_positive_int(mlp, path, "ff"))
    if kind == "moe":
        router = _get(mlp, path, "router")
        experts, top = _positive_int(router, path + "router.", "experts"), _positive_int(router, path + "router.", "top")
        if top > experts:
            raise ConfigError(path + "router.top", f"{top} is more than the {experts} experts")
        shared = mlp.get("shared")
        return ExpertsFF(experts=experts, top=top, ff=_positive_int(_get(mlp, path, "expert"), path + "expert.", "ff"),
                         shared_ff=_positive_int(shared, path + "shared.", "ff") if shared is not None else None)
    raise ConfigError(path + "kind", f"{kind!r} is not a feed-forward of this design (dense, moe)")
