"""A plain, slow implementation of the Fugavik decoder: one function per mechanism, whole sequences,
no cache, loops where loops are clearest.  It shares no code with the package under test, reads
``config.json`` and ``model.safetensors`` by itself and works on CPU tensors (float64 by default).

The design in short (n tokens of one sequence, positions 0 .. n-1, width d):

    x_0[t] = E[tok_t]
    every layer:  x <- x + s1 * LN1(mixer(x));  x <- x + s2 * LN2(ff(x))      (a layer may have no ff; nothing on the way in)
    logits = head . LNf(x)
    LN(u) = (u - mean u) / sqrt(var u + eps) * w + b         s1, s2: one multiplier per channel

Mixers: grouped-query attention with a norm per head on queries and keys, a rotation of halves with
all frequencies divided by one factor, a sink in the softmax and values blended with those of the first
blending layer ("attention"); causal attention through a cached latent with a sink and one sigmoid gate
per head ("latent_attention"); a gated delta rule with one decay per head, short causal convolutions
and a silu gate on its normed output ("delta").  Feed-forwards: a dense pair with a squared relu
between, or sigmoid-scored experts whose weight multiplies what the chosen expert reads.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch
from safetensors import safe_open

UNIT_EPS = 1e-6        # added under the root when queries and keys of the delta rule are made unit vectors


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
def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


# ----------------------------------------------------------------------------------------------
# rotation of halves: entry i turns with entry i + dims/2
# ----------------------------------------------------------------------------------------------
def rotary_frequencies(dims: int, base: float, scaling: Optional[dict]) -> List[float]:
    factor = 1.0 if not scaling else float(scaling["factor"])
    return [base ** (-2.0 * i / dims) / factor for i in range(dims // 2)]


def rotate_halves(v: torch.Tensor, position: int, freqs: Sequence[float]) -> torch.Tensor:
    """v [..., >= 2 len(freqs)]; entries beyond the rotated ones pass unchanged."""
    half = len(freqs)
    out = v.clone()
    for i, f in enumerate(freqs):
        ang = position * f
        c, s = math.cos(ang), math.sin(ang)
        a, b = v[..., i], v[..., i + half]
        out[..., i] = a * c - b * s
        out[..., i + half] = b * c + a * s
    return out


# ----------------------------------------------------------------------------------------------
# softmax whose denominator holds one more term that has no value
# ----------------------------------------------------------------------------------------------
def sink_softmax(scores: torch.Tensor, sink) -> torch.Tensor:
    """scores [m]; returns the weights of the m keys: exp(s_j) / (sum_j exp(s_j) + exp(sink))."""
    top = max(float(scores.max()), float(sink))
    e = torch.exp(scores - top)
    return e / (e.sum() + math.exp(float(sink) - top))


# ----------------------------------------------------------------------------------------------
# attention
# ----------------------------------------------------------------------------------------------
def attention_values(h, w, m, v_first: Optional[torch.Tensor], store=None) -> torch.Tensor:
    """The values [n, G, vdim] that a layer caches: its own projection, blended with ``v_first`` (the values of
    the first blending layer for the same tokens) when there is one."""
    n = h.shape[0]
    v = _keep(h @ w["v"].T, store).view(n, m["kv_heads"], m["vdim"])
    if v_first is not None:
        lam = float(w["vmix"])
        v = (1.0 - lam) * v + lam * v_first
    return v


def attention_mixer(h, w, m, eps, v, store=None) -> torch.Tensor:
    """``v``: the values of :func:`attention_values`."""
    n = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot")
    freqs = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling")) if rot else []
    q = rms_norm(_keep(h @ w["q"].T, store).view(n, H, dim), w["q.norm"], eps)
    k = rms_norm(_keep(h @ w["k"].T, store).view(n, G, dim), w["k.norm"], eps)
    q = _keep(torch.stack([rotate_halves(q[t], t, freqs) for t in range(n)]), store)
    k = _keep(torch.stack([rotate_halves(k[t], t, freqs) for t in range(n)]), store)
    v = _keep(v, store)
    out = torch.zeros(n, H, vdim, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        sc = (q[:, hd] @ k[:, g].T) * m["scale"]
        for t in range(n):
            p = sink_softmax(sc[t, :t + 1], w["sink"][hd])
            out[t, hd] = p @ v[:t + 1, g]
    return _keep(_keep(out.reshape(n, H * vdim), store) @ w["o"].T, store)


# ----------------------------------------------------------------------------------------------
# attention through a latent
# ----------------------------------------------------------------------------------------------
def latent_attention_mixer(h, w, m, eps, store=None) -> torch.Tensor:
    n = h.shape[0]
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = _keep(h @ w["q"].T, store).view(n, H, dim)
    c = _keep(rms_norm(_keep(h @ w["dkv"].T, store), w["dkv.norm"], eps), store)       # [n, kv_rank]: what is cached
    k = (c @ w["uk"].T).view(n, H, dim)
    v = (c @ w["uv"].T).view(n, H, vdim)
    gate = torch.sigmoid(_keep(h @ w["g"].T, store))                                   # [n, H]
    out = torch.zeros(n, H, vdim, dtype=h.dtype)
    for hd in range(H):
        sc = (q[:, hd] @ k[:, hd].T) * m["scale"]
        for t in range(n):
            p = sink_softmax(sc[t, :t + 1], w["sink"][hd])
            out[t, hd] = (p @ v[:t + 1, hd]) * gate[t, hd]
    return _keep(_keep(out.reshape(n, H * vdim), store) @ w["o"].T, store)


# ----------------------------------------------------------------------------------------------
# gated delta rule with one decay per head
# ----------------------------------------------------------------------------------------------
def causal_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [n, channels], taps [channels, T]: y_t = sum_j taps[:, j] * x_{t - (T - 1 - j)}, zeros before the start."""
    n, T = x.shape[0], taps.shape[1]
    y = torch.zeros_like(x)
    for t in range(n):
        for j in range(T):
            src = t - (T - 1 - j)
            if src >= 0:
                y[t] = y[t] + taps[:, j] * x[src]
    return y


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + UNIT_EPS)


def delta_mixer(h, w, m, eps, store=None) -> torch.Tensor:
    """Per head, with S [dim, vdim] zero at the start:
        S <- g_t S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t"""
    n = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(_keep(h @ w["q"].T, store), w["q.conv"])).view(n, G, dim)
    k = silu(causal_conv(_keep(h @ w["k"].T, store), w["k.conv"])).view(n, G, dim)
    v = silu(causal_conv(_keep(h @ w["v"].T, store), w["v.conv"])).view(n, H, vdim)
    q = unit(q) * dim ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ w["b"].T)                                               # [n, H]
    g = torch.exp(-torch.exp(w["A_log"]) * softplus(h @ w["a"].T + w["dt_bias"]))    # [n, H]
    gate = silu(_keep(h @ w["g"].T, store)).view(n, H, vdim)
    out = torch.zeros(n, H, vdim, dtype=h.dtype)
    for hd in range(H):
        kv = hd // (H // G)
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        for t in range(n):
            S = g[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            out[t, hd] = S.T @ q[t, kv]
    o = rms_norm(out, w["norm"], eps) * gate
    return _keep(_keep(o.reshape(n, H * vdim), store) @ w["o"].T, store)


# ----------------------------------------------------------------------------------------------
# feed-forwards
# ----------------------------------------------------------------------------------------------
def dense_ff(h, w, store=None) -> torch.Tensor:
    a = torch.relu(_keep(h @ w["up"].T, store)) ** 2
    return _keep(_keep(a, store) @ w["down"].T, store)


def router_choice(h, w_router, top: int):
    """(experts [n, top], weights [n, top]): the ``top`` largest sigmoid scores of every token, as they are."""
    s = torch.sigmoid(h @ w_router.T)
    weights, experts = torch.topk(s, top, dim=-1)
    return experts, weights


def expert_ff(h, w, store=None) -> torch.Tensor:
    a = silu(_keep(h @ w["gate"].T, store)) * _keep(h @ w["up"].T, store)
    return _keep(a, store) @ w["down"].T


def moe_ff(h, w, f, store=None, choice=None) -> torch.Tensor:
    """The weight multiplies what the expert reads:  out = sum over the chosen e of expert_e(weight_e * h)."""
    experts, weights = router_choice(h, w["router"], f["router"]["top"]) if choice is None else choice
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, a in zip(experts[t].tolist(), weights[t]):
            we = {k[len(f"e{e}."):]: v for k, v in w.items() if k.startswith(f"e{e}.")}
            out[t] = out[t] + expert_ff(_keep(a * h[t], store)[None], we, store)[0]
    return _keep(out, store)


# ----------------------------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------------------------
def sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: Sequence[int], store=None, layers_out=None,
            choices=None, scores_out=None) -> torch.Tensor:
    """Logits [n, vocab] of one sequence from its first token.  ``layers_out``: a list that receives the stream
    after every layer.  ``choices``: per layer with experts, (experts, weights or None) to use instead of the
    router's own pick (weights None: the router's scores of the given experts).  ``scores_out``: a dict that
    receives every such layer's router scores [n, experts]."""
    eps = cfg["norm"]["eps"]
    x = tensors["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = _keep(x, store)
        w, m = sub(tensors, p + "mix."), layer["mixer"]
        if layer["type"] == "attention":
            blend = bool(m.get("v_mix"))
            v = attention_values(h, w, m, v_first if blend else None, store)
            if blend and v_first is None:
                v_first = v
            y = attention_mixer(h, w, m, eps, v, store)
        elif layer["type"] == "latent_attention":
            y = latent_attention_mixer(h, w, m, eps, store)
        elif layer["type"] == "delta":
            y = delta_mixer(h, w, m, eps, store)
        else:
            raise ValueError(layer["type"])
        x = x + tensors[p + "ls1"] * layer_norm(y, tensors[p + "norm1"], tensors[p + "norm1.b"], eps)
        f = layer.get("mlp")
        if f is not None:
            h = _keep(x, store)
            wf = sub(tensors, p + "mlp.")
            if f["kind"] == "dense":
                y = dense_ff(h, wf, store)
            elif f["kind"] == "moe":
                choice = None
                if scores_out is not None:
                    scores_out[i] = torch.sigmoid(h @ wf["router"].T)
                if choices is not None and i in choices:
                    experts, weights = choices[i]
                    if weights is None:
                        weights = torch.gather(torch.sigmoid(h @ wf["router"].T), 1, experts)
                    choice = (experts, weights)
                y = moe_ff(h, wf, f, store, choice)
            else:
                raise ValueError(f["kind"])
            x = x + tensors[p + "ls2"] * layer_norm(y, tensors[p + "norm2"], tensors[p + "norm2.b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    xn = _keep(layer_norm(x, tensors["final.norm"], tensors["final.norm.b"], eps), store)
    return xn @ tensors["head"].T
