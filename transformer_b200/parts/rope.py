"""Rotary position encoding: the angle table (the rotation itself is fused with the cache write).

angle(p, i) = p * theta^(-2i/dh), i in [0, dh/2).  The reference builds sin/cos tables [nctx, dh]
once per model (models/llama/common/src/compute.rs:41-53, models/llama/cuda/src/infer.rs:89-90) and
passes theta along; pairing and the frequency formula are inside its external operator.  Here the
table is computed in double precision on the host and stored as float [positions, dh/2], so the
angle itself carries no 32-bit rounding at large positions.
"""
from __future__ import annotations

import math

import torch

from .base import POSITIONS, Position

_TABLES = {}


@POSITIONS.register("rope")
class Rope(Position):
    """params: dh, theta, pairing ("adjacent" | "half"), positions (table length); optional: scaling, ramp, linear.

    ``scaling`` = (factor, low, high, original) rescales the frequencies by wavelength l = 2 pi / f against a context
    of ``original`` tokens: f stays where l < original / high, becomes f / factor where l > original / low, and
    between the two is (1 - s) f / factor + s f with s = (original / l - low) / (high - low).

    ``ramp`` = (factor, original, fast, slow) rescales them by their index instead: with
    n(t) = dh ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)), dh - 1) and
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency is f_i / factor * r_i + f_i (1 - r_i), and cos
    and sin are both multiplied by 0.1 ln(factor) + 1.

    ``linear`` = factor divides every frequency by the same number (positions stretched by it); it may stand beside
    either of the other two and is applied first."""
    graph_safe = True
    launches_only = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.dh = int(params["dh"])
        self.theta = float(params["theta"])
        self.pairing = params.get("pairing", "adjacent")
        self.positions = int(params["positions"])
        sc = params.get("scaling")
        self.scaling = None if sc is None else tuple(float(v) for v in sc)
        if self.scaling is not None and len(self.scaling) != 4:
            raise ValueError(f"rope scaling is (factor, low, high, original), got {sc!r}")
        rp = params.get("ramp")
        self.ramp = None if rp is None else tuple(float(v) for v in rp)
        if self.ramp is not None and (len(self.ramp) != 4 or self.scaling is not None):
            raise ValueError(f"rope ramp is (factor, original, fast, slow) and excludes 'scaling', got {rp!r}")
        self.linear = float(params.get("linear") or 1.0)
        if not self.linear > 0:
            raise ValueError(f"a linear rescaling divides by a positive factor, got {self.linear}")
        if self.dh % 2:
            raise ValueError(f"rotary pairs need an even head size, got {self.dh}")
        if self.pairing not in ("adjacent", "half"):
            raise ValueError(f"unknown rope pairing {self.pairing!r}")

    @property
    def half_pairing(self) -> int:
        return 1 if self.pairing == "half" else 0

    def rotation(self):
        cos, sin = self.tables()
        return cos, sin, self.half_pairing

    def tables(self):
        key = (self.dh, self.theta, self.positions, self.scaling, self.ramp, self.linear, str(self.device))
        if key not in _TABLES:
            i = torch.arange(self.dh // 2, dtype=torch.float64)
            inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.dh) / self.linear
            if self.scaling is not None:
                factor, low, high, original = self.scaling
                turns = original * inv_freq / (2.0 * torch.pi)          # original / wavelength
                blend = ((turns - low) / (high - low)).clamp(0.0, 1.0)  # 0: long waves (scaled), 1: short (kept)
                inv_freq = (1.0 - blend) * inv_freq / factor + blend * inv_freq
            mult = 1.0
            if self.ramp is not None:
                factor, original, fast, slow = self.ramp
                at = lambda turns: self.dh * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
                lo = max(math.floor(at(fast)), 0)
                hi = min(math.ceil(at(slow)), self.dh - 1)
                r = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
                inv_freq = inv_freq / factor * r + inv_freq * (1.0 - r)
                mult = 0.1 * math.log(factor) + 1.0
            ang = torch.arange(self.positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
            _TABLES[key] = ((torch.cos(ang) * mult).float().contiguous().to(self.device),
                            (torch.sin(ang) * mult).float().contiguous().to(self.device))
        return _TABLES[key]
