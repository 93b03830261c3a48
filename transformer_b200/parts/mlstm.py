"""A matrix memory with exponential gates (the mLSTM cell of xLSTM) as a mixer with per-sequence state.

    q = Wq x1 * dim^-1/2,  k = Wk x1  (heads x dim),   v = Wv x1  (heads x vdim)
    i = cap tanh((Wi x1 + bi) / cap),   f = logsigmoid(cap tanh((Wf x1 + bf) / cap))          per head, float
    m_t = max(f_t + m_{t-1}, i_t)
    S_t = e^{f_t + m_{t-1} - m_t} S_{t-1} + e^{i_t - m_t} k_t v_t^T       n_t alike with k_t alone
    o_t = S_t^T q_t / (max(|n_t . q_t|, e^{-m_t}) + 1e-6)
    out = Wo (o / rms_per_head(o) * norm * sigmoid(Wg x1))

S, n and m are zero when a sequence starts, are float, and are carried from step to step in the
engine's per-sequence state (one row per slot); the gates' projections are a float product of their
own, since their error would add up along the sequence.  The kernels are in csrc/mlstm.cu: token by
token for decoding, 64 tokens at a time (the recurrence's closed form inside a chunk) for prompts.
"""
from __future__ import annotations

import torch

from ..csrc import lib
from .base import MIXERS, Mixer, ParamDecl, StateNeed
from .linear import matmul_nt


USE_CHUNKS = True      # prompts: the kernel that takes 64 tokens at a time


@MIXERS.register("mlstm")
class MatrixMemory(Mixer):
    """params: width, heads, dim, vdim, gate_cap, eps."""
    graph_safe = True
    launches_only = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        g = lambda n: int(params[n])
        self.d, self.H, self.dim, self.vdim = g("width"), g("heads"), g("dim"), g("vdim")
        self.cap, self.eps = float(params["gate_cap"]), float(params["eps"])
        if not self.cap > 0:
            raise ValueError(f"the gates' cap must be positive, got {self.cap}")
        if self.dim > 256:
            raise ValueError(f"the matrix-memory kernel takes heads of up to 256 query/key entries, got {self.dim}")
        self.z_width = 2 * self.H * self.dim + 2 * self.H * self.vdim

    def parameters(self):
        hv = self.H * self.vdim
        return {
            "wqkvg": ParamDecl((self.z_width, self.d)),            # rows: q heads, k heads, v heads, output gate
            "wif": ParamDecl((2 * self.H, self.d)),                # rows: input gates, forget gates
            "bif": ParamDecl((2 * self.H,), "norm", "normal"),
            "norm": ParamDecl((hv,), "norm", "ones"),
            "wo": ParamDecl((self.d, hv)),
        }

    def state_need(self):
        return StateNeed((self.H, lib.mlstm_state_size(self.dim, self.vdim)), torch.float32)

    def forward(self, ctx, x1, out, cache, state) -> None:
        nt, H = x1.shape[0], self.H
        sfx = lib.suffix(self.dtype)
        w = self.weights
        z = ctx.scratch("mlstm.z", (nt, self.z_width), self.dtype)
        matmul_nt(x1, w["wqkvg"], z)
        gates = ctx.scratch("mlstm.gates", (nt, 2 * H), torch.float32)
        matmul_nt(x1, w["wif"], gates)         # float out on both paths
        o = ctx.scratch("mlstm.o", (nt, H * self.vdim), torch.float32)
        # prompts: 64 tokens of a sequence side by side; decoding: token by token, the state in registers
        kernel = "tb_mlstm_scan_" if ctx.decode or not USE_CHUNKS else "tb_mlstm_chunk_"
        lib.call(kernel + sfx, lib.ptr(z), lib.ptr(gates), lib.ptr(w["bif"]), lib.ptr(state), lib.ptr(o),
                 lib.ptr(ctx.seq_start), lib.ptr(ctx.slots), ctx.B, self.z_width, H, self.dim, self.vdim, self.cap,
                 self.dim ** -0.5)
        y = ctx.scratch("mlstm.y", (nt, H * self.vdim), self.dtype)
        g = z[:, 2 * H * self.dim + H * self.vdim:]
        lib.call("tb_mlstm_out_" + sfx, lib.ptr(o), lib.ptr(g), self.z_width, lib.ptr(w["norm"]), lib.ptr(y), nt, H,
                 self.vdim, self.eps, 0)
        matmul_nt(y, w["wo"], out)
