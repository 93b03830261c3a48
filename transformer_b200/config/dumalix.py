"""Typed configuration of the Dumalix decoder.

``config.json`` of this design is nested; every size and every constant that may differ between models is read
from it:

    architecture: "Dumalix"     vocab, width     norm: {eps}     canon: {taps}
    loop: {start, stop, times}          layers start .. stop-1 run `times` times in a row (absent: every layer once)
    layers: [ {type, mixer: {...}, mlp: {kind: "dense", ff, limit} | null}, ... ]
      type "attention":        mixer {heads, kv_heads, dim, vdim, scale, conv, mask: {size},
                                      rot: {base, dims, scaling: {factor, original, fast, slow}}}
      type "latent_attention": mixer {heads, dim, rot_dim, vdim, kv_rank, scale,
                                      rot: {base, dims, scaling: {factor, original, fast, slow}}}
      (mask absent: plain causal; rot.scaling absent: none; conv absent: no convolution on the projections, 1: one tap,
       a weight per channel;
       canon absent: no convolution on what the mixers read)
    max_context (optional): the longest sequence, default 32768.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .registry import ConfigError
from .salepel import _num, _sub

DEFAULT_CONTEXT = 32768


@dataclass(frozen=True)
class RotRamp:
    factor: float
    original: float
    fast: float
    slow: float

    def as_tuple(self):
        return (self.factor, self.original, self.fast, self.slow)


def _rot(m, where):
    rot = _sub(m, "rot", where)
    sc = rot.get("scaling")
    ramp = None
    if sc is not None:
        w = where + ".rot.scaling"
        ramp = RotRamp(_num(sc, "factor", w, float), _num(sc, "original", w, float), _num(sc, "fast", w, float),
                       _num(sc, "slow", w, float))
    return _num(rot, "base", where + ".rot", float), _num(rot, "dims", where + ".rot"), ramp


def _rot_dict(base, dims, ramp):
    out = {"base": base, "dims": dims}
    if ramp is not None:
        out["scaling"] = {"factor": ramp.factor, "original": ramp.original, "fast": ramp.fast, "slow": ramp.slow}
    return out


@dataclass(frozen=True)
class ChunkAttentionMeta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int               # taps of the convolutions on q, k, v; 0: none
    chunk: int              # 0: plain causal
    rot_base: float
    rot_dims: int
    rot_ramp: Optional[RotRamp] = None

    @classmethod
    def from_dict(cls, m, where):
        base, dims, ramp = _rot(m, where)
        mask = m.get("mask")
        if mask is not None and not isinstance(mask, Mapping):
            raise ConfigError(f"{where}.mask must be an object")
        heads, dim = _num(m, "heads", where), _num(m, "dim", where)
        m = dict(m, kv_heads=m.get("kv_heads", heads), vdim=m.get("vdim", dim), scale=m.get("scale", dim ** -0.5),
                 conv=m.get("conv", 0))
        return cls(heads, _num(m, "kv_heads", where), dim, _num(m, "vdim", where), _num(m, "scale", where, float),
                   _num(m, "conv", where), 0 if mask is None else _num(mask, "size", where + ".mask"), base, dims, ramp)

    def to_dict(self):
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
               "rot": _rot_dict(self.rot_base, self.rot_dims, self.rot_ramp)}
        if self.conv:
            out["conv"] = self.conv
        if self.chunk:
            out["mask"] = {"size": self.chunk}
        return out


@dataclass(frozen=True)
class CausalLatentMeta:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    rot_ramp: Optional[RotRamp] = None

    @classmethod
    def from_dict(cls, m, where):
        base, dims, ramp = _rot(m, where)
        return cls(_num(m, "heads", where), _num(m, "dim", where), _num(m, "rot_dim", where), _num(m, "vdim", where),
                   _num(m, "kv_rank", where), _num(m, "scale", where, float), base, dims, ramp)

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                "kv_rank": self.kv_rank, "scale": self.scale, "rot": _rot_dict(self.rot_base, self.rot_dims, self.rot_ramp)}


@dataclass(frozen=True)
class ClampedDenseMeta:
    ff: int
    limit: float

    @classmethod
    def from_dict(cls, m, where):
        if m.get("kind") != "dense":
            raise ConfigError(f"{where}.kind must be 'dense', got {m.get('kind')!r}")
        return cls(_num(m, "ff", where), _num(m, "limit", where, float))

    def to_dict(self):
        return {"kind": "dense", "ff": self.ff, "limit": self.limit}


@dataclass(frozen=True)
class DumalixLayer:
    type: str                     # "attention" | "latent_attention"
    mixer: Any
    mlp: Optional[ClampedDenseMeta]


@dataclass(frozen=True)
class LoopMeta:
    start: int
    stop: int
    times: int


_MIXERS = {"attention": ChunkAttentionMeta, "latent_attention": CausalLatentMeta}


@dataclass(frozen=True)
class DumalixMeta:
    vocab: int
    width: int
    eps: float
    canon_taps: int               # 0: what the mixers read is not convolved
    loop: Optional[LoopMeta]
    layers: Tuple[DumalixLayer, ...]
    max_context: int = DEFAULT_CONTEXT
    eos: tuple = ()

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "DumalixMeta":
        layers_in = cfg.get("layers")
        if not isinstance(layers_in, (list, tuple)) or not layers_in:
            raise ConfigError("config.json lacks the list 'layers'")
        layers = []
        for i, entry in enumerate(layers_in):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping):
                raise ConfigError(f"{where} must be an object")
            kind = entry.get("type")
            if kind not in _MIXERS:
                raise ConfigError(f"{where}.type must be one of {sorted(_MIXERS)}, got {kind!r}")
            mixer = _MIXERS[kind].from_dict(_sub(entry, "mixer", where), where + ".mixer")
            mlp = entry.get("mlp")
            if mlp is not None and not isinstance(mlp, Mapping):
                raise ConfigError(f"{where}.mlp must be an object or null")
            layers.append(DumalixLayer(kind, mixer, None if mlp is None else ClampedDenseMeta.from_dict(mlp, where + ".mlp")))
        eos = cfg.get("eos_token_id", ())
        if isinstance(eos, bool) or not isinstance(eos, (int, list, tuple)):
            raise ConfigError(f"eos_token_id must be an integer or a list of integers, got {eos!r}")
        eos = (eos,) if isinstance(eos, int) else tuple(int(e) for e in eos)
        loop = cfg.get("loop")
        if loop is not None:
            if not isinstance(loop, Mapping):
                raise ConfigError("loop must be an object")
            loop = LoopMeta(_num(loop, "start", "loop"), _num(loop, "stop", "loop"), _num(loop, "times", "loop"))
        canon = cfg.get("canon")
        taps = 0 if canon is None else _num(canon, "taps", "canon")
        meta = cls(_num(cfg, "vocab", "config"), _num(cfg, "width", "config"),
                   _num(_sub(cfg, "norm", "config"), "eps", "norm", float), taps, loop, tuple(layers),
                   _num({"max_context": cfg.get("max_context", DEFAULT_CONTEXT)}, "max_context", "config"), eos)
        meta.validate()
        return meta

    @classmethod
    def from_folder(cls, folder: str) -> "DumalixMeta":
        with open(os.path.join(folder, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def run_order(self):
        """[(layer, first of a pass over the repeated group)] in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        a, b = self.loop.start, self.loop.stop
        order = [(i, False) for i in range(a)]
        for _ in range(self.loop.times):
            order += [(i, i == a) for i in range(a, b)]
        return order + [(i, False) for i in range(b, n)]

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or self.max_context <= 0:
            raise ConfigError("vocab, width and max_context must be positive")
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.eps}")
        if self.canon_taps < 0 or self.canon_taps > 16:
            raise ConfigError(f"canon.taps must lie in 1..16, got {self.canon_taps}")
        if self.loop is not None:
            lp = self.loop
            if not (0 <= lp.start < lp.stop <= len(self.layers)) or lp.times < 1:
                raise ConfigError(f"loop: 0 <= start < stop <= {len(self.layers)} and times >= 1 "
                                  f"(got {lp.start}, {lp.stop}, {lp.times})")
        for i, layer in enumerate(self.layers):
            m, where = layer.mixer, f"layers[{i}].mixer"
            names = ("heads", "kv_heads", "dim", "vdim") if isinstance(m, ChunkAttentionMeta) else \
                ("heads", "dim", "rot_dim", "vdim", "kv_rank")
            for n in names:
                if getattr(m, n) <= 0:
                    raise ConfigError(f"{where}.{n} must be positive, got {getattr(m, n)}")
            if not m.rot_base > 0:
                raise ConfigError(f"{where}.rot.base must be positive, got {m.rot_base}")
            r = m.rot_ramp
            if r is not None and (not r.factor > 0 or not r.original > 0 or not r.fast > 0 or not r.slow > 0):
                raise ConfigError(f"{where}.rot.scaling: factor, original, fast and slow must be positive")
            if isinstance(m, ChunkAttentionMeta):
                if m.heads % m.kv_heads:
                    raise ConfigError(f"{where}: {m.heads} heads cannot share {m.kv_heads} key heads")
                if m.rot_dims < 0 or m.rot_dims > m.dim or m.rot_dims % 2:
                    raise ConfigError(f"{where}.rot.dims must be even and at most dim ({m.rot_dims}, {m.dim})")
                if m.vdim % 2:
                    raise ConfigError(f"{where}.vdim must be even (the values rotate in pairs), got {m.vdim}")
                if m.conv < 0 or m.conv > 16 or m.chunk < 0:
                    raise ConfigError(f"{where}: conv must lie in 0..16, mask.size must not be negative")
            else:
                if m.rot_dims < 0 or m.rot_dims > m.rot_dim or m.rot_dims % 2:
                    raise ConfigError(f"{where}.rot.dims must be even and at most rot_dim ({m.rot_dims}, {m.rot_dim})")
            if layer.mlp is not None and (layer.mlp.ff <= 0 or not layer.mlp.limit > 0):
                raise ConfigError(f"layers[{i}].mlp: ff and limit must be positive")
        for e in self.eos:
            if not (0 <= e < self.vocab):
                raise ConfigError(f"eos token {e} lies outside the vocabulary of {self.vocab}")

    def to_dict(self) -> dict:
        out = {"architecture": "Dumalix", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "max_context": self.max_context,
               "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                          for l in self.layers]}
        if self.canon_taps:
            out["canon"] = {"taps": self.canon_taps}
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.eos:
            out["eos_token_id"] = list(self.eos)
        return out
