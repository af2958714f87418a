"""Typed configuration of the Kafunex decoder, read from config.json's own keys.

config.json of this design is nested: ``vocab``, ``width``, ``norm.eps`` and a list ``layers`` whose
entries give ``type`` ("attention" or "hgrn2"), the mixer's sizes under ``mixer`` and the feed-forward
under ``mlp`` (null: the layer has none).  Every size and every constant that can differ between two
models of the design comes from the file; what the design fixes (the base of the position vector,
the exponent of the distance slopes, the activation of the feed-forward) is in the plan builder.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import ModelConfigError

ATTENTION = "attention"
HGRN2 = "hgrn2"


def _int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = d.get(key) if isinstance(d, Mapping) else None
    if v is None or isinstance(v, bool) or not isinstance(v, int) or v < 1:
        raise ModelConfigError(f"config.json: {where}{key} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class KafunexMLP:
    kind: str
    ff: int


@dataclass(frozen=True)
class KafunexLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    kv_heads: Optional[int] = None          # attention only
    scale: Optional[float] = None           # attention only
    chunk: Optional[int] = None             # attention only: mask.size (None: every earlier key is visible)
    mlp: Optional[KafunexMLP] = None

    def to_dict(self):
        mixer = {"dim": self.dim, "heads": self.heads, "vdim": self.vdim}
        if self.type == ATTENTION:
            mixer.update(kv_heads=self.kv_heads, scale=self.scale)
            if self.chunk is not None:
                mixer["mask"] = {"size": self.chunk}
        return {"type": self.type, "mixer": mixer,
                "mlp": None if self.mlp is None else {"kind": self.mlp.kind, "ff": self.mlp.ff}}


@dataclass(frozen=True)
class KafunexConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: Tuple[KafunexLayer, ...]

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "KafunexConfig":
        if not isinstance(d, Mapping):
            raise ModelConfigError("config.json must hold a JSON object")
        arch = d.get("architecture")
        if not isinstance(arch, str):
            archs = d.get("architectures")
            arch = archs[0] if isinstance(archs, (list, tuple)) and archs else None
        if not isinstance(arch, str):
            raise ModelConfigError("config.json lacks required key 'architecture'")
        norm = d.get("norm")
        eps = norm.get("eps") if isinstance(norm, Mapping) else None
        if isinstance(eps, bool) or not isinstance(eps, (int, float)) or not math.isfinite(eps) or eps <= 0:
            raise ModelConfigError(f"config.json: norm.eps must be a positive number, got {eps!r}")
        entries = d.get("layers")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ModelConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(e, Mapping) or not isinstance(e.get("mixer"), Mapping):
                raise ModelConfigError(f"config.json: {where}mixer is missing")
            kind, m = e.get("type"), e["mixer"]
            heads, dim, vdim = _int(m, "heads", where + "mixer."), _int(m, "dim", where + "mixer."), _int(m, "vdim", where + "mixer.")
            mlp = e.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ModelConfigError(f"config.json: {where}mlp.kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r}: "
                                           "only 'dense' feed-forwards exist in this design")
                mlp = KafunexMLP("dense", _int(mlp, "ff", where + "mlp."))
            if kind == ATTENTION:
                kv = heads if m.get("kv_heads") is None else _int(m, "kv_heads", where + "mixer.")      # absent: one per query head
                if heads % kv:
                    raise ModelConfigError(f"config.json: {where}mixer.heads {heads} is not a multiple of kv_heads {kv}")
                if vdim != dim:
                    raise ModelConfigError(f"config.json: {where}mixer.vdim {vdim} differs from dim {dim}, but the values of "
                                           "this attention are its keys")
                scale = m.get("scale")
                if isinstance(scale, bool) or not isinstance(scale, (int, float)) or not math.isfinite(scale):
                    raise ModelConfigError(f"config.json: {where}mixer.scale must be a number, got {scale!r}")
                mask = m.get("mask")
                chunk = None if mask is None else _int(mask, "size", where + "mixer.mask.")
                layers.append(KafunexLayer(ATTENTION, heads, dim, vdim, kv, float(scale), chunk, mlp))
            elif kind == HGRN2:
                layers.append(KafunexLayer(HGRN2, heads, dim, vdim, mlp=mlp))
            else:
                raise ModelConfigError(f"config.json: {where}type {kind!r} is no mixer of this design "
                                       f"({ATTENTION!r}, {HGRN2!r})")
        return cls(architecture=arch, vocab_size=_int(d, "vocab", ""), hidden_size=_int(d, "width", ""),
                   norm_eps=float(eps), layers=tuple(layers))

    def to_dict(self):
        return {"architecture": self.architecture, "layers": [layer.to_dict() for layer in self.layers],
                "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size, "width": self.hidden_size}
