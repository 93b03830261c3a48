"""RMSNorm fused with the residual sum (models/llama/common/src/compute.rs:207,275,362); a layer norm (mean taken
off, weight and bias, an optional multiplier per channel) with the same fusions; and no norm at all."""
from __future__ import annotations

from ..csrc import lib
from .base import NORMS, Norm, NormedDelta, PairDelta, ParamDecl, WeightedRows


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """params: width, eps, mult (default 1), one_plus (default False).  y = v / rms(v) * weight * mult, or with
    ``one_plus`` (a weight stored around zero) v / rms(v) * (1 + weight) * mult.  Statistics and the residual sum are
    float; one rounding at the store.  The multiplier and the one are folded into the bound weight (float, once).
    A :class:`PairDelta` (two parts' outputs, both still to be added) is summed in the same kernel."""

    graph_safe = True
    launches_only = True
    takes_weighted_rows = True
    takes_normed_delta = True
    takes_pair_delta = True
    can_warm = True
    tails = ("router",)

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.mult = float(params.get("mult", 1.0))
        self.one_plus = bool(params.get("one_plus", False))

    def parameters(self):
        return {"weight": ParamDecl((self.width,), "norm", "normal" if self.one_plus else "ones")}

    def bind(self, tensors) -> None:
        super().bind(tensors)
        if self.one_plus:
            self.weights["weight"] = self.weights["weight"].float() + 1.0
        if self.mult != 1.0:
            self.weights["weight"] = self.weights["weight"].float() * self.mult

    def forward(self, ctx, x, delta, rows, y, warm=None, tail=None) -> None:
        if tail is not None and tail.sigmoid and not (isinstance(delta, NormedDelta) and delta.center):
            # this norm's own kernels know the two other rules of choice: the router runs behind it
            self.forward(ctx, x, delta, rows, y, warm=warm)
            _route(lib.suffix(self.dtype), y, tail, y.shape[0], self.width)
            return
        if isinstance(delta, NormedDelta):
            post_add_rmsnorm(self.dtype, x, delta, rows, self.weights["weight"], self.eps, y, tail=tail)
            return
        if isinstance(delta, PairDelta):
            pair_add_rmsnorm(self.dtype, x, delta, rows, self.weights["weight"], y, None, None, self.eps)
            if tail is not None:
                _route(lib.suffix(self.dtype), y, tail, y.shape[0], self.width)
            return
        n_out = y.shape[0]
        wy = idx = wts = None
        k = 0
        if isinstance(delta, WeightedRows):
            wy, idx, wts, k, delta = delta.rows, delta.index, delta.weights, delta.k, None
        if tail is not None:
            # the router of the normalized rows in the same kernel; what that form does not take (many rows, odd
            # widths) gets the norm alone and the router's own kernel
            E = tail.weights.shape[0]
            sfx = lib.suffix(self.dtype)
            if tail.scored:
                if lib.try_call("tb_add_rmsnorm_router_scored_" + sfx, lib.ptr(x), lib.ptr(delta), lib.ptr(wy),
                                lib.ptr(idx), lib.ptr(wts), k, lib.ptr(rows), lib.ptr(self.weights["weight"]), self.eps,
                                lib.ptr(y), lib.ptr(tail.weights), lib.ptr(tail.bias), lib.ptr(tail.index),
                                lib.ptr(tail.scores), n_out, self.width, E, tail.k):
                    return
                lib.call("tb_add_rmsnorm_" + sfx, lib.ptr(x), lib.ptr(delta), lib.ptr(wy), lib.ptr(idx), lib.ptr(wts), k,
                         lib.ptr(rows), lib.ptr(self.weights["weight"]), self.eps, lib.ptr(y), n_out, self.width, 0, 0)
                _route(sfx, y, tail, n_out, self.width)
                return
            if lib.try_call("tb_add_rmsnorm_router_" + sfx, lib.ptr(x), lib.ptr(delta), lib.ptr(wy), lib.ptr(idx),
                            lib.ptr(wts), k, lib.ptr(rows), lib.ptr(self.weights["weight"]), self.eps, lib.ptr(y),
                            lib.ptr(tail.weights), lib.ptr(tail.index), lib.ptr(tail.scores), n_out, self.width, E,
                            tail.k):
                return
            lib.call("tb_add_rmsnorm_" + sfx, lib.ptr(x), lib.ptr(delta), lib.ptr(wy), lib.ptr(idx), lib.ptr(wts), k,
                     lib.ptr(rows), lib.ptr(self.weights["weight"]), self.eps, lib.ptr(y), n_out, self.width,
                     lib.ptr(tail.weights), tail.weights.numel() * tail.weights.element_size())
            lib.call("tb_router_" + sfx, lib.ptr(y), lib.ptr(tail.weights), lib.ptr(tail.index), lib.ptr(tail.scores),
                     0, 0, 0, 0, 0, n_out, self.width, E, tail.k)
            return
        lib.call("tb_add_rmsnorm_" + lib.suffix(self.dtype), lib.ptr(x), lib.ptr(delta), lib.ptr(wy), lib.ptr(idx),
                 lib.ptr(wts), k, lib.ptr(rows), lib.ptr(self.weights["weight"]), self.eps, lib.ptr(y), n_out,
                 self.width, lib.ptr(warm), 0 if warm is None else warm.numel() * warm.element_size())


@NORMS.register("layernorm")
class LayerNorm(Norm):
    """params: width, eps, bias (default True), scale (default False).  y = (v - mean v) / sqrt(var v + eps) * weight
    + bias, the variance being the mean of the squared deviations.  With ``scale`` the result is multiplied channel
    by channel by a further learned vector ("scale": a block's layer scale), which is folded into the bound weight
    and bias (float, once).  Statistics and the residual sum are float; one rounding at the store.  A pending
    :class:`NormedDelta` of either kind is normed, added and normed again in the same kernel."""
    graph_safe = True
    launches_only = True
    takes_weighted_rows = True
    takes_normed_delta = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.bias = bool(params.get("bias", True))
        self.scale = bool(params.get("scale", False))

    def parameters(self):
        decl = {"weight": ParamDecl((self.width,), "norm", "ones")}
        if self.bias:
            decl["bias"] = ParamDecl((self.width,), "norm", "normal")
        if self.scale:
            decl["scale"] = ParamDecl((self.width,), "norm", "ones")
        return decl

    def bind(self, tensors) -> None:
        super().bind(tensors)
        if self.scale:
            s = self.weights.pop("scale").float()
            self.weights["weight"] = (self.weights["weight"].float() * s).contiguous()
            if self.bias:
                self.weights["bias"] = (self.weights["bias"].float() * s).contiguous()

    def as_normed(self, delta) -> NormedDelta:
        """``delta`` as something that this norm is still to be applied to before it joins the stream."""
        return NormedDelta(delta, self.weights["weight"], self.eps, self.weights.get("bias"), True)

    def forward(self, ctx, x, delta, rows, y) -> None:
        post = None
        if isinstance(delta, NormedDelta):
            post, delta = delta, delta.delta
        post_add_layernorm(self.dtype, x, delta, post, rows, self.weights["weight"], self.weights.get("bias"), self.eps,
                           True, y)


@NORMS.register("none")
class NoNorm(Norm):
    """params: width.  No norm at all, for blocks whose parts read the residual stream as it is: the pending
    contribution joins the stream (float sum; a :class:`NormedDelta` is normed on the way) and y is the sum, rounded
    once to the activation type.  The same kernels as the norm's, without weights."""
    graph_safe = True
    launches_only = True
    takes_weighted_rows = True
    takes_normed_delta = True
    takes_pair_delta = True
    tails = ("router",)

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.width = int(params["width"])

    def forward(self, ctx, x, delta, rows, y, tail=None) -> None:
        """``tail``: the router of the part that reads y; it rides in the kernel that norms a layer-normed delta, and
        runs behind any other."""
        if isinstance(delta, NormedDelta):
            post_add_rmsnorm(self.dtype, x, delta, rows, None, 0.0, y, tail=tail)
            return
        if tail is not None:
            self.forward(ctx, x, delta, rows, y)
            _route(lib.suffix(self.dtype), y, tail, y.shape[0], self.width)
            return
        if isinstance(delta, PairDelta):
            pair_add_rmsnorm(self.dtype, x, delta, rows, None, y, None, None, 0.0)
            return
        wy = idx = wts = None
        k = 0
        if isinstance(delta, WeightedRows):
            wy, idx, wts, k, delta = delta.rows, delta.index, delta.weights, delta.k, None
        lib.call("tb_add_rmsnorm_" + lib.suffix(self.dtype), lib.ptr(x), lib.ptr(delta), lib.ptr(wy), lib.ptr(idx),
                 lib.ptr(wts), k, lib.ptr(rows), 0, 0.0, lib.ptr(y), y.shape[0], self.width, 0, 0)


def _route(sfx, y, tail, n_out, width) -> None:
    """The router of the rows ``y`` by a kernel of its own, into the tail's index and scores."""
    E = tail.weights.shape[0]
    if tail.sigmoid:
        lib.call("tb_router_sigmoid_" + sfx, lib.ptr(y), lib.ptr(tail.weights), lib.ptr(tail.index), lib.ptr(tail.scores),
                 0, 0, 0, 0, n_out, width, E, tail.k)
    elif tail.scored:
        lib.call("tb_router_scored_" + sfx, lib.ptr(y), lib.ptr(tail.weights), lib.ptr(tail.bias), lib.ptr(tail.index),
                 lib.ptr(tail.scores), 0, 0, 0, 0, n_out, width, E, tail.k)
    else:
        lib.call("tb_router_" + sfx, lib.ptr(y), lib.ptr(tail.weights), lib.ptr(tail.index), lib.ptr(tail.scores),
                 0, 0, 0, 0, 0, n_out, width, E, tail.k)


def post_add_rmsnorm(dtype, x, pending: NormedDelta, rows, weight, eps, y, tail=None) -> None:
    """x[rows] += pending.delta / rms(pending.delta) * pending.weight (written back when ``rows`` is None), then
    y = x / rms(x) * weight; with ``y`` None only the sum.  ``tail``: a "router" NormTail computed along the way."""
    if pending.center or pending.bias is not None:
        post_add_layernorm(dtype, x, pending.delta, pending, rows, weight, None, eps, False, y, tail=tail)
        return
    delta, wy, idx, wts, k = pending.delta, None, None, None, 0
    if isinstance(delta, WeightedRows):
        wy, idx, wts, k, delta = delta.rows, delta.index, delta.weights, delta.k, None
    n_out = x.shape[0] if y is None else y.shape[0]
    sfx = lib.suffix(dtype)
    if tail is not None and rows is None and y is not None and weight is not None and not tail.sigmoid:
        if lib.try_call("tb_post_add_rmsnorm_router_" + sfx, lib.ptr(x), lib.ptr(delta), lib.ptr(wy), lib.ptr(idx),
                        lib.ptr(wts), k, lib.ptr(pending.weight), float(pending.eps), lib.ptr(weight), float(eps),
                        lib.ptr(y), lib.ptr(tail.weights), lib.ptr(tail.bias), lib.ptr(tail.index), lib.ptr(tail.scores),
                        n_out, x.shape[1], tail.weights.shape[0], tail.k, 1 if tail.scored else 0):
            return
    lib.call("tb_post_add_rmsnorm_" + sfx, lib.ptr(x), lib.ptr(delta), lib.ptr(wy), lib.ptr(idx),
             lib.ptr(wts), k, lib.ptr(pending.weight), float(pending.eps), lib.ptr(rows), lib.ptr(weight), float(eps),
             lib.ptr(y), n_out, x.shape[1])
    if tail is not None:
        _route(sfx, y, tail, n_out, x.shape[1])


def post_add_layernorm(dtype, x, delta, post, rows, weight, bias, eps, center, y, tail=None) -> None:
    """x[rows] += N_post(delta) (written back when ``rows`` is None), then y = N(x[rows]; weight, bias, eps, center).
    ``delta``: a tensor, a :class:`WeightedRows` or None; ``post``: the :class:`NormedDelta` whose norm the delta
    still has to pass (None: it joins as it is); ``weight`` None: y is the sum itself; ``y`` None: only the sum.
    ``tail``: a "router" NormTail of the rows y, in the same kernel where its form takes the sizes, else behind it."""
    wy = idx = wts = None
    k = 0
    if isinstance(delta, WeightedRows):
        wy, idx, wts, k, delta = delta.rows, delta.index, delta.weights, delta.k, None
    n_out = x.shape[0] if y is None else y.shape[0]
    pw = pb = None
    pe, pc = 0.0, 0
    if post is not None:
        pw, pb, pe, pc = post.weight, post.bias, float(post.eps), 1 if post.center else 0
    if tail is not None and y is not None:
        if lib.try_call("tb_post_add_layernorm_router_" + lib.suffix(dtype), lib.ptr(x), lib.ptr(delta), lib.ptr(wy),
                        lib.ptr(idx), lib.ptr(wts), k, lib.ptr(pw), lib.ptr(pb), pe, pc, lib.ptr(rows), lib.ptr(weight),
                        lib.ptr(bias), float(eps), 1 if center else 0, lib.ptr(y), n_out, x.shape[1],
                        lib.ptr(tail.weights), lib.ptr(tail.bias), lib.ptr(tail.index), lib.ptr(tail.scores),
                        tail.weights.shape[0], tail.k, tail.rule):
            return
    lib.call("tb_post_add_layernorm_" + lib.suffix(dtype), lib.ptr(x), lib.ptr(delta), lib.ptr(wy), lib.ptr(idx),
             lib.ptr(wts), k, lib.ptr(pw), lib.ptr(pb), pe, pc, lib.ptr(rows), lib.ptr(weight), lib.ptr(bias), float(eps),
             1 if center else 0, lib.ptr(y), n_out, x.shape[1])
    if tail is not None and y is not None:
        _route(lib.suffix(dtype), y, tail, n_out, x.shape[1])


def pair_add_rmsnorm(dtype, x, pending, rows, w1, y1, w2, y2, eps) -> None:
    """x[rows] += pending.first + pending.second (float; written back when ``rows`` is None; ``pending`` may be a
    tensor, a :class:`PairDelta` or None), then y1 = x / rms(x) * w1 and y2 = x / rms(x) * w2: one statistic, two
    weights.  A null weight gives the sum itself, rounded once; a null output is left out."""
    d1 = d2 = None
    if isinstance(pending, PairDelta):
        d1, d2 = pending.first, pending.second
    elif pending is not None:
        d1 = pending
    n_out = x.shape[0] if rows is None else rows.shape[0]
    lib.call("tb_pair_add_rmsnorm_" + lib.suffix(dtype), lib.ptr(x), lib.ptr(d1), lib.ptr(d2), lib.ptr(rows), lib.ptr(w1),
             lib.ptr(y1), 0 if y1 is None else y1.stride(0), lib.ptr(w2), lib.ptr(y2), 0 if y2 is None else y2.stride(0),
             float(eps), n_out, x.shape[1])
