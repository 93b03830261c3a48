"""Parts that work on the stream between the norms and the mixers, or between two runs of the model.

* input filter **"causal_conv"**: what a part reads, h, becomes h + conv(h) (or conv(h) alone), a causal
  convolution over time on every channel, ``taps`` wide, zeros before the sequence's start.  The last
  ``taps - 1`` inputs of every sequence are its state (float, one row per slot), so a prompt may be cut anywhere
  and decoding goes on from it.  Kernel: csrc/stream_pair.cu.
* joint **"reinject"**: x <- W [x ; e] with e the embedding output of the step's tokens: a projection of twice the
  width that mixes the embedding back into the stream (before every pass over a group of layers that runs several
  times).  The sum that is still pending joins the stream in the kernel that also lays [x ; e] out for the product;
  the product writes the new stream in float.
"""
from __future__ import annotations

import torch

from ..csrc import lib
from .base import INPUT_FILTERS, JOINTS, InputFilter, Joint, ParamDecl, StateNeed
from .linear import matmul_nt
from .norm import pair_add_rmsnorm


@INPUT_FILTERS.register("causal_conv")
class CausalConv(InputFilter):
    """params: width, taps, residual (default True: out = y + conv(y))."""
    graph_safe = True
    launches_only = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.width, self.taps = int(params["width"]), int(params["taps"])
        self.residual = bool(params.get("residual", True))
        if not (1 <= self.taps <= 16):
            raise ValueError(f"the convolution takes 1 to 16 taps, got {self.taps}")

    def parameters(self):
        return {"weight": ParamDecl((self.width, self.taps), "norm", "normal")}

    def state_need(self):
        return StateNeed((max(self.taps - 1, 1) * self.width,), torch.float32)

    def forward(self, ctx, y, out, state) -> None:
        lib.call("tb_causal_conv_" + lib.suffix(self.dtype), lib.ptr(y), y.stride(0), lib.ptr(self.weights["weight"]),
                 lib.ptr(state), state.stride(0), lib.ptr(out), out.stride(0), lib.ptr(ctx.tok_seq),
                 lib.ptr(ctx.seq_start), lib.ptr(ctx.slots), y.shape[0], ctx.B, self.width, self.taps,
                 1 if self.residual else 0, 1 if ctx.decode else 0)


@JOINTS.register("reinject")
class Reinject(Joint):
    """params: width.  x <- weight [x ; e], weight [width, 2 width] with the stream's columns first."""
    graph_safe = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.width = int(params["width"])

    def parameters(self):
        return {"weight": ParamDecl((self.width, 2 * self.width))}

    def _pair(self, ctx, nt):
        return ctx.scratch("reinject.pair", (nt, 2 * self.width), self.dtype)

    def begin(self, ctx, x) -> None:
        # the embedding output, in the type the product reads, in the right half of every row
        pair_add_rmsnorm(self.dtype, x, None, None, None, self._pair(ctx, x.shape[0])[:, self.width:], None, None, 0.0)

    def forward(self, ctx, x, pending):
        pair = self._pair(ctx, x.shape[0])
        pair_add_rmsnorm(self.dtype, x, pending, None, None, pair[:, :self.width], None, None, 0.0)
        matmul_nt(pair, self.weights["weight"], x)       # float out: the stream itself
        return None
