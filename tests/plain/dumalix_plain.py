"""A plain, slow implementation of the Dumalix decoder: one function per mechanism, whole sequences,
no cache, loops where loops are clearest.  It shares no code with the package under test, reads
``config.json`` and ``model.safetensors`` by itself and works on CPU tensors (float64 by default).

The design in short (n tokens of one sequence, positions 0 .. n-1, width d):

    e = E[tokens]                                             the embedding output
    run order: layers[0 .. start-1], then `times` passes over layers[start .. stop-1] (same weights, a cache and
        state of its own for every pass), then layers[stop ..];  before the first layer of every pass:
        x <- W_in [x ; e]
    every layer:  x <- x + mixer(c(N1(x))) + ff(N2(x)),   N(u) = u / sqrt(mean(u^2) + eps) * (1 + w),
        c(h) = h + causal convolution of h over time, per channel          (ff may be absent)
    logits = head . Nf(x)

Mixers: grouped-query attention with short convolutions on q, k, v, a norm per head, a partial rotary
encoding with rescaled frequencies, rotated values, a temperature per head, a mask of chunks and a sink in
the softmax ("attention"); attention through a shared low-rank latent with one rotated key part for all
heads ("latent_attention").  The feed-forward is a clamped gated pair.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch
from safetensors import safe_open

GLU_ALPHA = 1.702       # the design fixes the gate's slope


def read_folder(folder: str, dtype=torch.float64):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            t = f.get_tensor(name)
            tensors[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, tensors


def _keep(x, store):
    """``store``: what a 16-bit path does where it writes an activation to memory (round and come back)."""
    return x if store is None else store(x)


# ----------------------------------------------------------------------------------------------
# small parts
# ----------------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float, one_plus: bool = False) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    if w is None:
        return y
    return y * (1.0 + w) if one_plus else y * w


def causal_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [n, C], w [C, taps]:  y[t] = sum_j w[:, j] * u[t - taps + 1 + j], zeros before the start."""
    n, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(n):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def rescaled_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(frequencies [dims / 2], multiplier of cos and sin)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_adjacent(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, mult: float = 1.0,
                    sign: float = 1.0) -> torch.Tensor:
    """x [n, heads, D]; the first 2 * len(freqs) entries of every head turn in the pairs (2i, 2i + 1)."""
    out = x.clone()
    ang = sign * positions.to(torch.float64)[:, None] * freqs[None, :]
    cos, sin = (torch.cos(ang) * mult)[:, None, :], (torch.sin(ang) * mult)[:, None, :]
    r = 2 * freqs.shape[0]
    u, v = x[..., 0:r:2], x[..., 1:r:2]
    out[..., 0:r:2] = u * cos - v * sin
    out[..., 1:r:2] = v * cos + u * sin
    return out


def chunk_visible(i: int, j: int, size: Optional[int]) -> bool:
    return j <= i and (size is None or i // size == j // size)


# ----------------------------------------------------------------------------------------------
# mixers
# ----------------------------------------------------------------------------------------------
def attention(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, m: dict, eps: float, store=None) -> torch.Tensor:
    n = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(n)
    q = _keep(h @ t[p + "q"].T, store)
    k = _keep(h @ t[p + "k"].T, store)
    v = _keep(h @ t[p + "v"].T, store)
    if (p + "q.conv") in t:
        q, k, v = causal_conv(q, t[p + "q.conv"]), causal_conv(k, t[p + "k.conv"]), causal_conv(v, t[p + "v.conv"])
    q = rms_norm(q.view(n, H, D), t[p + "q.norm"], eps)
    k = rms_norm(k.view(n, G, D), t[p + "k.norm"], eps)
    v = v.view(n, G, V)
    rot = m["rot"]
    freqs, mult = rescaled_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    q = rotate_adjacent(q, pos, freqs, mult)
    k = _keep(rotate_adjacent(k, pos, freqs, mult), store)
    vfreqs, _ = rescaled_frequencies(V, rot["base"], None)
    v = _keep(rotate_adjacent(v, pos, vfreqs), store)
    size = (m.get("mask") or {}).get("size")
    temp, sink = t[p + "temp"], t[p + "sink"]
    seen = torch.tensor([[chunk_visible(i, j, size) for j in range(n)] for i in range(n)])
    o = torch.zeros((n, H, V), dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"] * temp[hd]
        s = s.masked_fill(~seen, float("-inf"))
        s = torch.cat([s, sink[hd].expand(n, 1)], dim=1)        # the sink: a column without key and value
        w = torch.softmax(s, dim=-1)[:, :n]
        o[:, hd] = w @ v[:, g]
    o = rotate_adjacent(o, pos, vfreqs, sign=-1.0)
    return _keep(o.reshape(n, H * V), store) @ t[p + "o"].T


def latent_attention(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, m: dict, eps: float, store=None) -> torch.Tensor:
    n = h.shape[0]
    H, D, R, V, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(n)
    q = _keep(h @ t[p + "q"].T, store).view(n, H, D + R)
    z = _keep(h @ t[p + "dkv"].T, store)
    c = _keep(rms_norm(z[:, :rank], t[p + "dkv.norm"], eps), store)
    rot = m["rot"]
    freqs, mult = rescaled_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    kr = _keep(rotate_adjacent(z[:, None, rank:], pos, freqs, mult), store)[:, 0]
    qr = rotate_adjacent(q[..., D:], pos, freqs, mult)
    kp = (c @ t[p + "uk"].T).view(n, H, D)
    vv = (c @ t[p + "uv"].T).view(n, H, V)
    o = torch.zeros((n, H, V), dtype=h.dtype)
    for hd in range(H):
        s = (q[:, hd, :D] @ kp[:, hd].T + qr[:, hd] @ kr.T) * m["scale"]
        s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool), 1), float("-inf"))
        o[:, hd] = torch.softmax(s, dim=-1) @ vv[:, hd]
    return _keep(o.reshape(n, H * V), store) @ t[p + "o"].T


def feed_forward(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, f: dict, store=None) -> torch.Tensor:
    limit = float(f["limit"])
    g = (h @ t[p + "gate"].T).clamp(max=limit)
    u = (h @ t[p + "up"].T).clamp(-limit, limit)
    y = g * torch.sigmoid(GLU_ALPHA * g) * (u + 1.0)
    return _keep(y, store) @ t[p + "down"].T


# ----------------------------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------------------------
def run_order(cfg: dict) -> List[tuple]:
    """[(layer, first of a pass)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def layer(x: torch.Tensor, t: Dict[str, torch.Tensor], i: int, cfg: dict, store=None) -> torch.Tensor:
    L, p, eps = cfg["layers"][i], f"l{i}.", cfg["norm"]["eps"]
    h = _keep(rms_norm(x, t[p + "norm1"], eps, one_plus=True), store)
    if (p + "canon1") in t:
        h = _keep(h + causal_conv(h, t[p + "canon1"]), store)
    mix = {"attention": attention, "latent_attention": latent_attention}[L["type"]]
    out = _keep(mix(h, t, p + "mix.", L["mixer"], eps, store), store)
    if L.get("mlp") is not None:
        h2 = _keep(rms_norm(x, t[p + "norm2"], eps, one_plus=True), store)
        out = out + _keep(feed_forward(h2, t, p + "mlp.", L["mlp"], store), store)
    return x + out


def forward(cfg: dict, t: Dict[str, torch.Tensor], tokens: Sequence[int], store=None, streams: Optional[list] = None
            ) -> torch.Tensor:
    """Logits [n, vocab] of one whole sequence.  ``streams``: a list that receives the stream after every layer run."""
    e = t["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
    x = e
    for i, first in run_order(cfg):
        if first:
            x = _keep(torch.cat([x, e], dim=-1), store) @ t["loop.in"].T
        x = layer(x, t, i, cfg, store)
        if streams is not None:
            streams.append(x.clone())
    xn = _keep(rms_norm(x, t["final.norm"], cfg["norm"]["eps"], one_plus=True), store)
    return xn @ t["head"].T
