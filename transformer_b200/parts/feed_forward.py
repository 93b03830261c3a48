"""Feed-forward parts: a dense SwiGLU and a softmax-top-k mixture of SwiGLU experts.

The reference runs the experts as a host loop over tokens and chosen experts with one product
each and a device-to-host copy of the router logits in every layer
(models/llama/common/src/compute.rs:294-333).  Here the tokens are sorted by expert on the device
and every expert runs once over all of its tokens (a grouped product); nothing touches the host.
"""
from __future__ import annotations

import torch

from ..csrc import lib
from .base import FEED_FORWARDS, FeedForward, NormTail, ParamDecl, WeightedRows
from . import linear
from .linear import gemm_skinny, grouped_matmul, matmul_nt

ROUTER_ROWS_FROM = 256      # above this many tokens the router works on tiles of 16 tokens (tensor cores)
ROUTER_TAIL_ROWS = 256      # up to this many tokens the norm before the experts also routes


@FEED_FORWARDS.register("swiglu")
class DenseSwiGLU(FeedForward):
    """params: width, di, bias (default False).  gate_up = x1 Wgu^T (gate rows first), h = silu(gate) * up,
    out = h Wd^T (compute.rs:278-292).  With ``bias`` all three projections have one: ``bgu`` (gate's, then up's)
    and ``bd``, float.  The down projection's bias rides inside its product: the bound weight gets the bias as one
    more column (and zeros up to a multiple of eight), and the kernel that applies the pair's biases and the
    activation writes a one into that column of ``h``.  ``glu_limit`` (with ``glu_alpha``, default 1): the pair
    becomes g' * sigmoid(alpha g') * (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit) instead of
    silu(g) * u, in the product's epilogue."""
    graph_safe = True
    launches_only = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.d = int(params["width"])
        self.di = int(params["di"])
        self.bias = bool(params.get("bias", False))
        limit = params.get("glu_limit")
        self.glu = None if limit is None else (float(params.get("glu_alpha", 1.0)), float(limit))
        if self.glu is not None and self.bias:
            raise ValueError("the clamped pair has no form with biases")

    def parameters(self):
        decl = {"wgu": ParamDecl((2 * self.di, self.d)), "wd": ParamDecl((self.d, self.di))}
        if self.bias:
            decl["bgu"] = ParamDecl((2 * self.di,), "norm", "normal")
            decl["bd"] = ParamDecl((self.d,), "norm", "normal")
        return decl

    def bind(self, tensors) -> None:
        super().bind(tensors)
        if self.bias:
            wd, bd = self.weights["wd"], self.weights.pop("bd")
            pad = (self.di + 1 + 7) // 8 * 8 - self.di - 1
            self.weights["wd"] = torch.cat([wd, bd.to(wd.dtype)[:, None], wd.new_zeros((self.d, pad))], dim=1).contiguous()

    def forward(self, ctx, x1, out) -> None:
        nt = x1.shape[0]
        if self.bias:
            wide = self.weights["wd"].shape[1]
            gu = ctx.scratch("ff.gu", (nt, 2 * self.di), self.dtype)
            matmul_nt(x1, self.weights["wgu"], gu)
            h = ctx.scratch("ff.h1", (nt, wide), self.dtype)
            lib.call("tb_bias_glu_" + lib.suffix(self.dtype), lib.ptr(gu), lib.ptr(self.weights["bgu"]), lib.ptr(h), nt,
                     self.di, wide)
            matmul_nt(h, self.weights["wd"], out)
            return
        h = ctx.scratch("ff.h", (nt, self.di), self.dtype)
        grouped_matmul(x1, self.weights["wgu"], h, swiglu=True, glu=self.glu)
        matmul_nt(h, self.weights["wd"], out)


@FEED_FORWARDS.register("mlp")
class DenseMLP(FeedForward):
    """params: width, di, act ("relu2").  A feed-forward without a gate: out = act(x1 Wu^T) Wd^T, with
    relu2(z) = max(z, 0)^2 (float, one rounding).  The activation sits in the epilogue of this package's own products
    (decoding, and the 32-bit path); behind the library's product of many bfloat16 rows it is a pass of its own over
    the result, in place."""
    graph_safe = True
    launches_only = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.d = int(params["width"])
        self.di = int(params["di"])
        self.act = params.get("act", "relu2")
        if self.act != "relu2":
            raise ValueError(f"unknown activation {self.act!r}; this part has 'relu2'")

    def parameters(self):
        return {"wu": ParamDecl((self.di, self.d)), "wd": ParamDecl((self.d, self.di))}

    def forward(self, ctx, x1, out) -> None:
        nt = x1.shape[0]
        h = ctx.scratch("ff.h", (nt, self.di), self.dtype)
        if self.dtype == torch.float32:
            linear.gemm_simt(x1, self.weights["wu"], h, out_kind=3)
        elif not (nt <= linear.SKINNY_MAX_ROWS and gemm_skinny(x1, self.weights["wu"], h, out_kind=3)):
            matmul_nt(x1, self.weights["wu"], h)
            lib.call("tb_relu2_" + lib.suffix(self.dtype), lib.ptr(h), nt * self.di)
        matmul_nt(h, self.weights["wd"], out)


@FEED_FORWARDS.register("moe")
class MoE(FeedForward):
    """params: width, di, nexp, nexp_use; optional: scoring, correction, identity, glu_alpha, glu_limit.

    router logits (float) -> the nexp_use largest, equal logits to the lower expert -> softmax over
    the kept logits (compute.rs:375-394) -> expert SwiGLU (compute.rs:320-328) -> weighted sum in
    descending-logit order, in float (compute.rs:329-330).

    Other routers and experts, by parameter:
    * ``scoring`` = "all": scores = softmax over ALL router outputs; the nexp_use largest of score + correction
      are chosen (``correction`` = True: a learned float vector, one entry per router output; equal values to the
      lower index); the weights are the chosen scores as they are.
    * ``identity`` = n: the router has nexp + n outputs, and the last n stand for experts without weights whose
      output is their input.
    * ``glu_limit`` (with ``glu_alpha``): the expert's pair becomes g' * sigmoid(alpha g') * (u' + 1) with
      g' = min(g, limit), u' = clamp(u, -limit, limit), instead of silu(g) * u.
    * ``scoring`` = "sigmoid": scores = sigmoid(logit), each by itself; the nexp_use largest are chosen (equal values
      to the lower index); the weights are the chosen scores as they are.
    * ``weight_on`` = "input": the weight multiplies what the expert reads, out = sum_e expert_e(w_e x1), instead of
      what it returns.  Every (token, choice) pair gets its own scaled copy of the token's row (one kernel, which
      also puts the rows in the experts' order), the experts run on those, and their results are summed unweighted."""
    graph_safe = True
    launches_only = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.d = int(params["width"])
        self.di = int(params["di"])
        self.E = int(params["nexp"])
        self.k = int(params["nexp_use"])
        if not (0 < self.k <= self.E + int(params.get("identity", 0))):
            raise ValueError(f"experts per token {self.k} must lie in 1..{self.E + int(params.get('identity', 0))}")
        self.identity = int(params.get("identity", 0))
        self.R = self.E + self.identity           # router outputs
        if self.R > 1024:
            raise ValueError(f"the routing kernels take up to 1024 experts, got {self.R}")
        self.scoring = params.get("scoring", "kept")
        if self.scoring not in ("kept", "all", "sigmoid"):
            raise ValueError(f"unknown router scoring {self.scoring!r}")
        self.weight_on = params.get("weight_on", "output")
        if self.weight_on not in ("output", "input"):
            raise ValueError(f"the router's weight multiplies the expert's 'output' or 'input', got {self.weight_on!r}")
        if self.weight_on == "input" and self.identity:
            raise ValueError("pass-through experts and weights on the input are not combined")
        self.correction = bool(params.get("correction", False))
        if self.correction and self.scoring != "all":
            raise ValueError("a correction of the choice goes with scoring 'all'")
        limit = params.get("glu_limit")
        self.glu = None if limit is None else (float(params.get("glu_alpha", 1.0)), float(limit))
        self.plain_router = self.scoring == "kept" and not self.identity

    def parameters(self):
        decl = {
            "router": ParamDecl((self.R, self.d)),
            "wgu": ParamDecl((self.E, 2 * self.di, self.d)),
            "wd": ParamDecl((self.E, self.d, self.di)),
        }
        if self.correction:
            decl["correction"] = ParamDecl((self.R,), "norm", "normal")
        return decl

    def early_weights(self):
        """The router's matrix: small, and every token's block waits for all of it."""
        r = self.weights.get("router")
        return r if r is not None and r.numel() * r.element_size() <= (1 << 20) else None

    def route(self, ctx, x1, logits_out=None, lists=None):
        """Experts and weights of every token.  With ``lists`` = (offsets, sorted_token, pair_row) the dispatch lists
        are wanted too; returns (idx, w, whether the lists were built along the way)."""
        nt = x1.shape[0]
        idx = ctx.scratch("moe.topk_idx", (nt, self.k), torch.int32)
        w = ctx.scratch("moe.topk_w", (nt, self.k), torch.float32)
        if self.scoring == "all":
            # scores over all outputs, choice with the correction, the block that finishes last builds the lists
            done = ctx.scratch("moe.done", (1,), torch.int32, zero=True) if lists is not None else None
            offsets, sorted_token, pair_row = lists if lists is not None else (None, None, None)
            if self.dtype == torch.bfloat16 and nt > ROUTER_ROWS_FROM and self.R <= 64 and \
                    lib.try_call("tb_router_rows_scored_bf16", lib.ptr(x1), lib.ptr(self.weights["router"]),
                                 lib.ptr(self.weights.get("correction")), lib.ptr(idx), lib.ptr(w), lib.ptr(offsets),
                                 lib.ptr(sorted_token), lib.ptr(pair_row), lib.ptr(done), nt, self.d, self.R, self.k):
                return idx, w, lists is not None
            lib.call("tb_router_scored_" + lib.suffix(self.dtype), lib.ptr(x1), lib.ptr(self.weights["router"]),
                     lib.ptr(self.weights.get("correction")), lib.ptr(idx), lib.ptr(w), lib.ptr(offsets),
                     lib.ptr(sorted_token), lib.ptr(pair_row), lib.ptr(done), nt, self.d, self.R, self.k)
            return idx, w, lists is not None
        if self.scoring == "sigmoid":
            # the same kernels with another rule for the weights; the block that finishes last builds the lists
            done = ctx.scratch("moe.done", (1,), torch.int32, zero=True) if lists is not None else None
            offsets, sorted_token, pair_row = lists if lists is not None else (None, None, None)
            if self.dtype == torch.bfloat16 and nt > ROUTER_ROWS_FROM and self.R <= 64 and \
                    lib.try_call("tb_router_rows_sigmoid_bf16", lib.ptr(x1), lib.ptr(self.weights["router"]),
                                 lib.ptr(idx), lib.ptr(w), lib.ptr(offsets), lib.ptr(sorted_token), lib.ptr(pair_row),
                                 lib.ptr(done), nt, self.d, self.R, self.k):
                return idx, w, lists is not None
            lib.call("tb_router_sigmoid_" + lib.suffix(self.dtype), lib.ptr(x1), lib.ptr(self.weights["router"]),
                     lib.ptr(idx), lib.ptr(w), lib.ptr(offsets), lib.ptr(sorted_token), lib.ptr(pair_row),
                     lib.ptr(done), nt, self.d, self.R, self.k)
            return idx, w, lists is not None
        if self.dtype == torch.bfloat16 and nt > ROUTER_ROWS_FROM and self.R <= 64:
            # many tokens, few experts: 16 tokens' logits are a tensor-core tile, the activations are read once, and
            # the block that finishes last builds the dispatch lists
            done = ctx.scratch("moe.done", (1,), torch.int32, zero=True) if lists is not None else None
            offsets, sorted_token, pair_row = lists if lists is not None else (None, None, None)
            if lib.try_call("tb_router_rows_bf16", lib.ptr(x1), lib.ptr(self.weights["router"]), lib.ptr(idx), lib.ptr(w),
                            lib.ptr(logits_out), lib.ptr(offsets), lib.ptr(sorted_token), lib.ptr(pair_row),
                            lib.ptr(done), nt, self.d, self.R, self.k):
                return idx, w, lists is not None
        # a few tokens: the block that finishes last builds the lists, which saves a kernel on the way to the experts
        fused = lists is not None and nt <= ROUTER_ROWS_FROM
        done = ctx.scratch("moe.done", (1,), torch.int32, zero=True) if fused else None
        offsets, sorted_token, pair_row = lists if fused else (None, None, None)
        lib.call("tb_router_" + lib.suffix(self.dtype), lib.ptr(x1), lib.ptr(self.weights["router"]),
                 lib.ptr(idx), lib.ptr(w), lib.ptr(logits_out), lib.ptr(offsets), lib.ptr(sorted_token),
                 lib.ptr(pair_row), lib.ptr(done), nt, self.d, self.R, self.k)
        return idx, w, fused

    def norm_tail(self, ctx, nt):
        """For a few tokens the router rides along with the norm before this part."""
        if nt > ROUTER_TAIL_ROWS:
            return None
        return NormTail("router", weights=self.weights["router"], k=self.k,
                        index=ctx.scratch("moe.topk_idx", (nt, self.k), torch.int32),
                        scores=ctx.scratch("moe.topk_w", (nt, self.k), torch.float32),
                        scored=self.scoring == "all", bias=self.weights.get("correction"),
                        sigmoid=self.scoring == "sigmoid")

    def forward(self, ctx, x1, out, tail=None) -> None:
        nt = x1.shape[0]
        M = nt * self.k
        sfx = lib.suffix(self.dtype)
        if self.dtype == torch.bfloat16 and M <= linear.SKINNY_MAX_PAIRS and self.d % 8 == 0 and self.di % 8 == 0:
            # a few tokens: no dispatch lists.  Row p = t * k + j of the experts' products is the pair (token t,
            # its j-th choice); every block of the product kernel finds its expert's pairs in the router's answer
            idx, w = (tail.index, tail.scores) if tail is not None else self.route(ctx, x1)[:2]
            h = ctx.scratch("moe.h", (M, self.di), self.dtype)
            y = ctx.scratch("moe.y", (M, self.d), self.dtype)
            pairs = idx.view(-1)
            src, x_div = x1, self.k
            if self.weight_on == "input":       # a scaled copy of the token's row for each of its pairs
                src, x_div = ctx.scratch("moe.scaled_rows", (M, self.d), self.dtype), 1
                lib.call("tb_moe_scaled_rows_" + sfx, lib.ptr(x1), lib.ptr(w), 0, lib.ptr(src), M, self.d, self.k)
                w = _ones(nt, self.k, x1.device)
            if gemm_skinny(src, self.weights["wgu"], h, groups=self.E, out_kind=2, max_group_rows=nt, row_group=pairs,
                           x_div=x_div, glu=self.glu) and \
                    gemm_skinny(h, self.weights["wd"], y, groups=self.E, max_group_rows=nt, row_group=pairs):
                ctx.record("moe.topk_idx", idx)
                if self.identity:       # pairs that chose an expert without weights: the token's own row
                    lib.call("tb_moe_identity_rows_" + sfx, lib.ptr(x1), lib.ptr(y), 0, 0, lib.ptr(pairs), self.k, M,
                             self.d, self.E)
                return WeightedRows(y, _identity_rows(M, x1.device), w, self.k)
        offsets = ctx.scratch("moe.offsets", (self.R + 1,), torch.int32)
        sorted_token = ctx.scratch("moe.sorted_token", (M,), torch.int32)
        pair_row = ctx.scratch("moe.pair_row", (M,), torch.int32)
        if tail is not None:
            idx, w, listed = tail.index, tail.scores, False
        else:
            idx, w, listed = self.route(ctx, x1, lists=(offsets, sorted_token, pair_row))
        ctx.record("moe.topk_idx", idx)
        if not listed:
            lib.call("tb_moe_dispatch", lib.ptr(idx), lib.ptr(offsets), lib.ptr(sorted_token), lib.ptr(pair_row),
                     M, self.k, self.R)
        h = ctx.scratch("moe.h", (M, self.di), self.dtype)
        if self.weight_on == "input":
            # the pairs' scaled rows, already in the experts' order (what the gather before the product does else)
            src = ctx.scratch("grouped.sorted_rows", (M, self.d), self.dtype)
            lib.call("tb_moe_scaled_rows_" + sfx, lib.ptr(x1), lib.ptr(w), lib.ptr(pair_row), lib.ptr(src), M, self.d,
                     self.k)
            w = _ones(nt, self.k, x1.device)
            grouped_matmul(src, self.weights["wgu"], h, group_offsets=offsets, groups=self.E, swiglu=True,
                           max_group_rows=nt, scratch=ctx.scratch, glu=self.glu)
        else:
            grouped_matmul(x1, self.weights["wgu"], h, a_rows=sorted_token, group_offsets=offsets, groups=self.E,
                           swiglu=True, max_group_rows=nt, scratch=ctx.scratch, glu=self.glu)
        y = ctx.scratch("moe.y", (M, self.d), self.dtype)
        grouped_matmul(h, self.weights["wd"], y, group_offsets=offsets, groups=self.E, max_group_rows=nt)
        if self.identity:               # the rows after the last real expert's: their tokens' own rows
            lib.call("tb_moe_identity_rows_" + sfx, lib.ptr(x1), lib.ptr(y), lib.ptr(offsets), lib.ptr(sorted_token),
                     0, 1, M, self.d, self.E)
        # the weighted sum over the chosen experts is left to the norm that follows (fused there)
        return WeightedRows(y, pair_row, w, self.k)


_IDENTITY_ROWS = {}


def _identity_rows(n: int, device) -> torch.Tensor:
    """0 .. n-1 as int32, made once per size."""
    key = (n, str(device))
    if key not in _IDENTITY_ROWS:
        _IDENTITY_ROWS[key] = torch.arange(n, dtype=torch.int32, device=device)
    return _IDENTITY_ROWS[key]


_ONES = {}


def _ones(nt: int, k: int, device) -> torch.Tensor:
    """[nt, k] float ones, made once per size: the weights of a sum whose terms were weighted on the way in."""
    key = (nt, k, str(device))
    if key not in _ONES:
        _ONES[key] = torch.ones((nt, k), dtype=torch.float32, device=device)
    return _ONES[key]


def sum_weighted_rows(wr: WeightedRows, out) -> None:
    """out[t] = sum_j weights[t, j] * rows[index[t, j]], for a consumer that wants a plain tensor."""
    nt, d = out.shape
    lib.call("tb_moe_combine_" + lib.suffix(out.dtype), lib.ptr(wr.rows), lib.ptr(wr.index), lib.ptr(wr.weights),
             lib.ptr(out), nt, d, wr.k)
