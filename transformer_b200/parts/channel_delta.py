"""A gated delta rule with one decay per key channel, as a mixer with per-sequence state.

    q = Wq x1, k = Wk x1  (kv_heads x dim),   v = Wv x1  (heads x vdim);   head h reads key head h / (heads / kv_heads)
    each passes a short causal convolution over time (per channel, ``taps`` wide, zeros before the start), then silu
    q, k unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q times dim^-1/2
    beta = sigmoid(Wb x1)  per head;    g = exp(-exp(A_log_h) softplus(Wa2 (Wa1 x1) + dt_bias))  per head and key channel
    per head:  S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
    out = Wo (o / rms_head(o) * norm * sigmoid(Wg2 (Wg1 x1)))

Variants by parameter: ``decay`` = "head": one decay per head instead of one per key channel,
g = exp(-exp(A_log_h) softplus(a_h + dt_bias_h)), the same for every key channel of the head; ``decay_rank`` 0: the
decay's pre-activation comes straight from one projection (``wa``; it shares a float-output product with beta's);
``gate_rank`` 0: the gate's pre-activation comes straight from one projection whose rows ride in the merged first
product; ``gate_act`` = "silu": the gate is silu(.) instead of sigmoid(.).

S is zero when a sequence starts, float, and carried from step to step together with the last ``taps - 1`` inputs
of the convolutions in the engine's per-sequence state (one row per slot).  Decays, their logarithms and
exponentials, beta, the unit norms, the state and the per-head norm are float on both paths; the bfloat16 path
differs in the type of the projections' results.  The projections of beta and of the decay write float (their
error would add up along the sequence).  Kernels: csrc/channel_delta.cu.
"""
from __future__ import annotations

import torch

from ..csrc import lib
from .base import MIXERS, Mixer, ParamDecl, StateNeed
from .linear import matmul_nt


@MIXERS.register("channel_delta")
class ChannelDelta(Mixer):
    """params: width, heads, kv_heads, dim, vdim, taps, decay_rank, gate_rank, eps; optional: decay ("channel" |
    "head"), gate_act ("sigmoid" | "silu")."""
    graph_safe = True
    launches_only = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        g = lambda n: int(params[n])
        self.d, self.H, self.G, self.dim, self.vdim = g("width"), g("heads"), g("kv_heads"), g("dim"), g("vdim")
        self.taps, self.ra, self.rg = g("taps"), g("decay_rank"), g("gate_rank")
        self.eps = float(params["eps"])
        self.decay = params.get("decay", "channel")
        self.gate_act = params.get("gate_act", "sigmoid")
        if self.decay not in ("channel", "head") or self.gate_act not in ("sigmoid", "silu"):
            raise ValueError(f"decay is 'channel' or 'head' and gate_act 'sigmoid' or 'silu'; got {self.decay!r}, "
                             f"{self.gate_act!r}")
        if self.ra < 0 or self.rg < 0:
            raise ValueError("the ranks of the decay's and the gate's first projections must not be negative")
        if self.H % self.G:
            raise ValueError(f"{self.H} heads cannot share {self.G} key heads")
        if self.dim > 256:
            raise ValueError(f"the delta-rule kernel takes heads of up to 256 query/key entries, got {self.dim}")
        if not (1 <= self.taps <= 16):
            raise ValueError(f"the convolution takes 1 to 16 taps, got {self.taps}")
        self.hk, self.hv = self.G * self.dim, self.H * self.vdim
        self.C = 2 * self.hk + self.hv                       # channels that pass the convolution: q, k, v
        self.n_decay = self.H if self.decay == "head" else self.H * self.dim       # decays per token
        # rows of the first product: q, k, v, then the decay's first projection (low rank) and the gate's (its first
        # projection, or without a low rank the gate's own rows)
        self.z_width = self.C + self.ra + (self.rg if self.rg else self.hv)

    def parameters(self):
        decl = {
            "win": ParamDecl((self.z_width, self.d)),
            "conv": ParamDecl((self.C, self.taps), "norm", "normal"),
            "wb": ParamDecl((self.H, self.d)),
            "dt_bias": ParamDecl((self.n_decay,), "norm", "normal"),
            "A_log": ParamDecl((self.H,), "norm", "normal"),
            "norm": ParamDecl((self.vdim,), "norm", "ones"),
            "wo": ParamDecl((self.d, self.hv)),
        }
        if self.ra:
            decl["a2"] = ParamDecl((self.n_decay, self.ra))
        else:
            decl["wa"] = ParamDecl((self.n_decay, self.d))
        if self.rg:
            decl["g2"] = ParamDecl((self.hv, self.rg))
        return decl

    def bind(self, tensors) -> None:
        super().bind(tensors)
        # the kernel that norms the heads' outputs takes one weight per (head, entry): the shared one, repeated
        self.weights["norm"] = self.weights["norm"].float().repeat(self.H).contiguous()
        if not self.ra:
            # beta's and the decay's pre-activations: one float-output product, beta's rows first
            self.weights["wb"] = torch.cat([self.weights["wb"], self.weights.pop("wa")], dim=0).contiguous()

    def state_need(self):
        return StateNeed((lib.delta_state_size(self.G, self.H, self.dim, self.vdim, self.taps),), torch.float32)

    def forward(self, ctx, x1, out, cache, state) -> None:
        nt, H = x1.shape[0], self.H
        sfx = lib.suffix(self.dtype)
        w = self.weights
        z = ctx.scratch("delta.z", (nt, self.z_width), self.dtype)
        matmul_nt(x1, w["win"], z)
        if self.ra:
            bz = ctx.scratch("delta.bz", (nt, H), torch.float32)
            matmul_nt(x1, w["wb"], bz)                                          # float out on both paths
            a = ctx.scratch("delta.a", (nt, self.n_decay), torch.float32)
            matmul_nt(z[:, self.C:self.C + self.ra], w["a2"], a)               # float out
        else:
            bz = ctx.scratch("delta.bz", (nt, H + self.n_decay), torch.float32)
            matmul_nt(x1, w["wb"], bz)                                          # [beta | decay], float out
            a = bz[:, H:]
        if self.rg:
            gz = ctx.scratch("delta.gz", (nt, self.hv), self.dtype)
            matmul_nt(z[:, self.C + self.ra:], w["g2"], gz)
        else:
            gz = z[:, self.C + self.ra:]
        # what enters the recurrence, float: one record per (token, head) [q | k | decay | beta, k.q], and the values
        rec = ctx.scratch("delta.rec", (nt, H, lib.delta_record_size(self.dim)), torch.float32)
        vals = ctx.scratch("delta.v", (nt, H, lib.delta_value_pitch(self.vdim)), torch.float32)
        lib.call("tb_delta_prep_" + sfx, lib.ptr(z), self.z_width, lib.ptr(w["conv"]), lib.ptr(state), lib.ptr(a),
                 lib.ptr(w["dt_bias"]), lib.ptr(w["A_log"]), lib.ptr(bz), lib.ptr(rec), lib.ptr(vals),
                 lib.ptr(ctx.tok_seq), lib.ptr(ctx.seq_start), lib.ptr(ctx.slots), nt, ctx.B, self.G, H,
                 self.dim, self.vdim, self.taps, 1 if ctx.decode else 0, a.stride(0), bz.stride(0),
                 1 if self.decay == "head" else 0)
        o = ctx.scratch("delta.o", (nt, self.hv), torch.float32)
        lib.call("tb_delta_scan", lib.ptr(rec), lib.ptr(vals), lib.ptr(state), lib.ptr(o),
                 lib.ptr(ctx.seq_start), lib.ptr(ctx.slots), nt, ctx.B, self.G, H, self.dim, self.vdim, self.taps)
        y = ctx.scratch("delta.y", (nt, self.hv), self.dtype)
        lib.call("tb_mlstm_out_" + sfx, lib.ptr(o), lib.ptr(gz), gz.stride(0), lib.ptr(w["norm"]), lib.ptr(y), nt, H,
                 self.vdim, self.eps, 1 if self.gate_act == "silu" else 0)
        matmul_nt(y, w["wo"], out)
