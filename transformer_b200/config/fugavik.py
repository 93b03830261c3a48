"""Typed configuration of the Fugavik decoder.

``config.json`` of this design is nested; every size and every constant that may differ between models is
read from it:

    architecture: "Fugavik"     vocab, width     norm: {eps}
    layers: [ {type, mixer: {...}, mlp: {...} | null}, ... ]
      type "attention":         mixer {heads, kv_heads, dim, vdim, scale, v_mix,
                                       rot: {base, dims, scaling: {factor}}}
                                (rot absent or dims 0: no rotation; rot.scaling absent: factor 1; v_mix absent: false)
      type "latent_attention":  mixer {heads, dim, vdim, kv_rank, scale}
      type "delta":             mixer {heads, kv_heads, dim, vdim, conv}
      mlp {kind: "dense", ff}  |  {kind: "moe", expert: {ff}, router: {experts, top}}
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
class AttentionMeta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int           # 0: no rotation
    rot_factor: float       # every frequency is divided by it
    v_mix: bool

    @classmethod
    def from_dict(cls, m, where):
        heads, dim = _num(m, "heads", where), _num(m, "dim", where)
        m = dict(m, kv_heads=m.get("kv_heads", heads), vdim=m.get("vdim", dim), scale=m.get("scale", dim ** -0.5))
        rot = m.get("rot")
        base, dims, factor = 10000.0, 0, 1.0
        if rot is not None:
            if not isinstance(rot, Mapping):
                raise ConfigError(f"{where}.rot must be an object")
            dims = _num(rot, "dims", where + ".rot")
            if dims:
                base = _num(rot, "base", where + ".rot", float)
            sc = rot.get("scaling")
            if sc is not None:
                if not isinstance(sc, Mapping):
                    raise ConfigError(f"{where}.rot.scaling must be an object")
                factor = _num(sc, "factor", where + ".rot.scaling", float)
        v_mix = m.get("v_mix", False)
        if not isinstance(v_mix, bool):
            raise ConfigError(f"{where}.v_mix must be true or false, got {v_mix!r}")
        return cls(heads, _num(m, "kv_heads", where), dim, _num(m, "vdim", where), _num(m, "scale", where, float),
                   base, dims, factor, v_mix)

    def to_dict(self):
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot_dims:
            out["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.rot_factor != 1.0:
                out["rot"]["scaling"] = {"factor": self.rot_factor}
        if self.v_mix:
            out["v_mix"] = True
        return out


@dataclass(frozen=True)
class LatentMeta:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float

    @classmethod
    def from_dict(cls, m, where):
        dim = _num(m, "dim", where)
        m = dict(m, vdim=m.get("vdim", dim), scale=m.get("scale", dim ** -0.5))
        return cls(_num(m, "heads", where), dim, _num(m, "vdim", where), _num(m, "kv_rank", where),
                   _num(m, "scale", where, float))

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "kv_rank": self.kv_rank, "scale": self.scale}


@dataclass(frozen=True)
class DeltaMeta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, m, where):
        heads, dim = _num(m, "heads", where), _num(m, "dim", where)
        m = dict(m, kv_heads=m.get("kv_heads", heads), vdim=m.get("vdim", dim))
        return cls(heads, _num(m, "kv_heads", where), dim, _num(m, "vdim", where), _num(m, "conv", where))

    def to_dict(self):
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


@dataclass(frozen=True)
class DenseMeta:
    ff: int

    def to_dict(self):
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class ExpertsMeta:
    ff: int
    experts: int
    top: int

    def to_dict(self):
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}


def _mlp(m, where):
    kind = m.get("kind")
    if kind == "dense":
        return DenseMeta(_num(m, "ff", where))
    if kind == "moe":
        router = _sub(m, "router", where)
        return ExpertsMeta(_num(_sub(m, "expert", where), "ff", where + ".expert"),
                           _num(router, "experts", where + ".router"), _num(router, "top", where + ".router"))
    raise ConfigError(f"{where}.kind must be 'dense' or 'moe', got {kind!r}")


@dataclass(frozen=True)
class FugavikLayer:
    type: str                     # "attention" | "latent_attention" | "delta"
    mixer: Any
    mlp: Any                      # DenseMeta | ExpertsMeta | None


_MIXERS = {"attention": AttentionMeta, "latent_attention": LatentMeta, "delta": DeltaMeta}


@dataclass(frozen=True)
class FugavikMeta:
    vocab: int
    width: int
    eps: float
    layers: Tuple[FugavikLayer, ...]
    max_context: int = DEFAULT_CONTEXT
    eos: tuple = ()

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "FugavikMeta":
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
            layers.append(FugavikLayer(kind, mixer, None if mlp is None else _mlp(mlp, where + ".mlp")))
        eos = cfg.get("eos_token_id", ())
        if isinstance(eos, bool) or not isinstance(eos, (int, list, tuple)):
            raise ConfigError(f"eos_token_id must be an integer or a list of integers, got {eos!r}")
        eos = (eos,) if isinstance(eos, int) else tuple(int(e) for e in eos)
        meta = cls(_num(cfg, "vocab", "config"), _num(cfg, "width", "config"),
                   _num(_sub(cfg, "norm", "config"), "eps", "norm", float), tuple(layers),
                   _num({"max_context": cfg.get("max_context", DEFAULT_CONTEXT)}, "max_context", "config"), eos)
        meta.validate()
        return meta

    @classmethod
    def from_folder(cls, folder: str) -> "FugavikMeta":
        with open(os.path.join(folder, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def first_v_mix(self) -> Optional[int]:
        """The first layer whose attention blends values: the others blend theirs with its values."""
        for i, layer in enumerate(self.layers):
            if isinstance(layer.mixer, AttentionMeta) and layer.mixer.v_mix:
                return i
        return None

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or self.max_context <= 0:
            raise ConfigError("vocab, width and max_context must be positive")
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.eps}")
        first = self.first_v_mix()
        for i, layer in enumerate(self.layers):
            m, where = layer.mixer, f"layers[{i}].mixer"
            for n in ("heads", "dim", "vdim"):
                if getattr(m, n) <= 0:
                    raise ConfigError(f"{where}.{n} must be positive, got {getattr(m, n)}")
            if not isinstance(m, LatentMeta):
                if m.kv_heads <= 0 or m.heads % m.kv_heads:
                    raise ConfigError(f"{where}: {m.heads} heads cannot share {m.kv_heads} key heads")
            if isinstance(m, AttentionMeta):
                if m.rot_dims < 0 or m.rot_dims > m.dim or m.rot_dims % 2:
                    raise ConfigError(f"{where}.rot.dims must be even and at most dim ({m.rot_dims}, {m.dim})")
                if not m.rot_base > 0 or not m.rot_factor > 0:
                    raise ConfigError(f"{where}.rot: base and scaling.factor must be positive")
                if m.v_mix and i != first:
                    f = self.layers[first].mixer
                    if (m.kv_heads, m.vdim) != (f.kv_heads, f.vdim):
                        raise ConfigError(f"{where}: values of {m.kv_heads} x {m.vdim} cannot be blended with layer "
                                          f"{first}'s {f.kv_heads} x {f.vdim}")
            elif isinstance(m, LatentMeta):
                if m.kv_rank <= 0:
                    raise ConfigError(f"{where}.kv_rank must be positive, got {m.kv_rank}")
            else:
                if m.conv < 1:
                    raise ConfigError(f"{where}.conv must be at least 1, got {m.conv}")
            f = layer.mlp
            if f is not None and f.ff <= 0:
                raise ConfigError(f"layers[{i}].mlp: ff must be positive")
            if isinstance(f, ExpertsMeta) and not (0 < f.top <= f.experts):
                raise ConfigError(f"layers[{i}].mlp.router: top {f.top} must lie in 1..{f.experts}")
        for e in self.eos:
            if not (0 <= e < self.vocab):
                raise ConfigError(f"eos token {e} lies outside the vocabulary of {self.vocab}")

    def to_dict(self) -> dict:
        out = {"architecture": "Fugavik", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "max_context": self.max_context,
               "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                          for l in self.layers]}
        if self.eos:
            out["eos_token_id"] = list(self.eos)
        return out
