"""Typed configuration of the Lunelorn decoder, read from config.json's own keys.

config.json of this design is nested: ``vocab``, ``width``, ``norm.eps``, optionally ``logit_softcap``,
``token_side.dim`` (a per-layer token input) and ``loop`` (``start``, ``stop``, ``times``: layers start .. stop-1
run ``times`` times in a row with the same weights), and a list ``layers`` whose entries give ``type``
("retention", "parallel" or "wkv"), the mixer's sizes and constants under ``mixer`` and the feed-forward under
``mlp`` (null: the layer has none; else ``kind`` "moe" with ``expert.ff``, ``router.experts``, ``router.top``).
Every size and every constant that can differ between two models of the design comes from the file (one size,
the width of the wkv mixer's decay bottleneck, is given by a tensor's shape unless ``mixer.rank`` names it); what
the design fixes is in the plan builder.  The configuration keeps the layers as validated plain mappings, so
``to_dict`` gives back what ``from_dict`` read.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import ModelConfigError

RETENTION, PARALLEL, WKV = "retention", "parallel", "wkv"


def _int(d, key, where, least=1):
    v = d.get(key) if isinstance(d, Mapping) else None
    if v is None or isinstance(v, bool) or not isinstance(v, int) or v < least:
        raise ModelConfigError(f"config.json: {where}{key} must be an integer of at least {least}, got {v!r}")
    return v


def _num(d, key, where, positive=False):
    v = d.get(key) if isinstance(d, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or (positive and v <= 0):
        raise ModelConfigError(f"config.json: {where}{key} must be a {'positive ' if positive else ''}number, got {v!r}")
    return float(v)


def _map(d, key, where):
    v = d.get(key) if isinstance(d, Mapping) else None
    if not isinstance(v, Mapping):
        raise ModelConfigError(f"config.json: {where}{key} is missing")
    return v


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


def _check_mixer(kind, m, where):
    if kind == RETENTION:
        heads = _int(m, "heads", where)
        _int(m, "dim", where), _int(m, "vdim", where)
        decay = m.get("decay")
        if not isinstance(decay, (list, tuple)) or len(decay) != heads or any(
                isinstance(x, bool) or not isinstance(x, (int, float)) or not 0.0 <= x <= 1.0 for x in decay):
            raise ModelConfigError(f"config.json: {where}decay must list one number in [0, 1] for each of the {heads} heads")
    elif kind == PARALLEL:
        left, right = _map(m, "left", where), _map(m, "right", where)
        heads, kv = _int(left, "heads", where + "left."), _int(left, "kv_heads", where + "left.")
        if heads % kv:
            raise ModelConfigError(f"config.json: {where}left.heads {heads} is not a multiple of kv_heads {kv}")
        dim, vdim = _int(left, "dim", where + "left."), _int(left, "vdim", where + "left.")
        rot = _map(left, "rot", where + "left.")
        dims = _int(rot, "dims", where + "left.rot.", least=2)
        _num(rot, "base", where + "left.rot.", positive=True)
        if dims % 2 or dims > dim:
            raise ModelConfigError(f"config.json: {where}left.rot.dims {dims} must be even and at most dim {dim}")
        if vdim % 2:
            raise ModelConfigError(f"config.json: {where}left.vdim {vdim} must be even: the values are rotated in pairs")
        _num(left, "scale", where + "left.")
        _int(right, "width", where + "right.")
        _num(m, "left_scale", where), _num(m, "right_scale", where)
    elif kind == WKV:
        _int(m, "heads", where), _int(m, "dim", where)
        if m.get("rank") is not None:
            _int(m, "rank", where)
    else:
        raise ModelConfigError(f"config.json: {where[:-6]}type {kind!r} is no mixer of this design "
                               f"({RETENTION!r}, {PARALLEL!r}, {WKV!r})")


@dataclass(frozen=True)
class LunelornLoop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class LunelornConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: Tuple[Mapping[str, Any], ...]
    logit_softcap: Optional[float] = None
    token_side_dim: Optional[int] = None
    loop: Optional[LunelornLoop] = None

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LunelornConfig":
        if not isinstance(d, Mapping):
            raise ModelConfigError("config.json must hold a JSON object")
        arch = d.get("architecture")
        if not isinstance(arch, str):
            archs = d.get("architectures")
            arch = archs[0] if isinstance(archs, (list, tuple)) and archs else None
        if not isinstance(arch, str):
            raise ModelConfigError("config.json lacks required key 'architecture'")
        eps = _num(_map(d, "norm", ""), "eps", "norm.", positive=True)
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
        cap = d.get("logit_softcap")
        if cap is not None:
            cap = _num(d, "logit_softcap", "", positive=True)
        side = d.get("token_side")
        side_dim = None if side is None else _int(side, "dim", "token_side.")
        loop = d.get("loop")
        if loop is not None:
            loop = LunelornLoop(_int(loop, "start", "loop.", least=0), _int(loop, "stop", "loop.", least=0),
                                _int(loop, "times", "loop."))
            if not loop.start <= loop.stop <= len(layers):
                raise ModelConfigError(f"config.json: loop.start {loop.start} .. loop.stop {loop.stop} is no range of the "
                                       f"{len(layers)} layers")
        return cls(architecture=arch, vocab_size=_int(d, "vocab", ""), hidden_size=_int(d, "width", ""), norm_eps=eps,
                   layers=tuple(layers), logit_softcap=cap, token_side_dim=side_dim, loop=loop)

    def to_dict(self):
        d = {"architecture": self.architecture, "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
             "vocab": self.vocab_size, "width": self.hidden_size}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.token_side_dim is not None:
            d["token_side"] = {"dim": self.token_side_dim}
        if self.loop is not None:
            d["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return d
