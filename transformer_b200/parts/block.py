"""The arrangement of a layer's parts in a block.

"pre_norm" (models/llama/common/src/compute.rs:204-336):

    x += mixer(norm_m(x));   x += feed_forward(norm_f(x))

The residual stream ``x`` is float.  A part writes its contribution ``delta``; the sum into ``x``
is fused into the NEXT norm (of this block or the following one, or the final norm), so a block
takes the pending delta of the block before it and returns its own.

Arrangements are registered like parts (:data:`ARRANGEMENTS`): a class built from (LayerSpec, dtype, device)
that offers ``parts()`` (name -> part: the names under which the weights are bound), ``mixer`` (whose cache
and state needs the engine serves) and ``forward(ctx, x, pending, cache_view, state)`` with the contract
above: ``pending`` is what the block before left to be added to ``x`` (a tensor, a WeightedRows, or None), the
return value is what this block leaves.  A block that wants its sums done at once can call
:func:`add_pending` and return None.
"""
from __future__ import annotations

from .base import ARRANGEMENTS, FEED_FORWARDS, INPUT_FILTERS, MIXERS, NORMS, NormedDelta, PairDelta, WeightedRows


def build_layer(spec, dtype, device):
    """The block of one LayerSpec, by its arrangement."""
    return ARRANGEMENTS.get(spec.arrangement)(spec, dtype, device)


@ARRANGEMENTS.register("pre_norm")
class Layer:
    """The parts of one LayerSpec, built, in the pre-norm arrangement."""

    def __init__(self, spec, dtype, device):
        if spec.mixer_norm is None or spec.feed_forward_norm is None:
            raise ValueError("the pre_norm arrangement needs a norm before the mixer and one before the feed-forward")
        self.spec = spec
        self.mixer_norm = NORMS.build(spec.mixer_norm, dtype, device)
        self.mixer = MIXERS.build(spec.mixer, dtype, device)
        self.feed_forward_norm = NORMS.build(spec.feed_forward_norm, dtype, device)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, dtype, device)

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in self.parts().values())

    @property
    def launches_only(self) -> bool:
        return all(p.launches_only for p in self.parts().values())

    def parts(self):
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer,
                "feed_forward_norm": self.feed_forward_norm, "feed_forward": self.feed_forward}

    def forward(self, ctx, x, pending, cache_view, state):
        """x: float [nt, d]; pending: the previous block's delta or None.  Returns this block's
        pending delta (the feed-forward's output)."""
        nt, d = x.shape
        x1 = ctx.scratch("block.x1", (nt, d), ctx.dtype)
        delta = ctx.scratch("block.delta", (nt, d), ctx.dtype)
        pending = resolve(pending, self.mixer_norm, delta, x=x, ctx=ctx)
        self._norm(self.mixer_norm, self.mixer, ctx, x, pending, x1)
        self.mixer.forward(ctx, x1, delta, cache_view, state)
        tail = self.feed_forward.norm_tail(ctx, nt)
        if tail is not None and tail.kind in self.feed_forward_norm.tails:
            # the feed-forward's first small step rides along with the norm before it
            self.feed_forward_norm.forward(ctx, x, delta, None, x1, tail=tail)
            lazy = self.feed_forward.forward(ctx, x1, delta, tail=tail)
        else:
            self._norm(self.feed_forward_norm, self.feed_forward, ctx, x, delta, x1)
            lazy = self.feed_forward.forward(ctx, x1, delta)
        return delta if lazy is None else lazy


    @staticmethod
    def _norm(norm, then, ctx, x, delta, y) -> None:
        """The norm before the part ``then``; a norm that can do so starts fetching what that part reads first."""
        early = then.early_weights() if norm.can_warm else None
        if early is not None:
            norm.forward(ctx, x, delta, None, y, warm=early)
        else:
            norm.forward(ctx, x, delta, None, y)


@ARRANGEMENTS.register("sandwich")
class SandwichLayer:
    """A block that norms what its parts produce as well as what they read:

        x += norm_mb(mixer(norm_m(x)));   x += norm_fb(feed_forward(norm_f(x)))

    ``LayerSpec.extra`` names the two further norms, "mixer_post_norm" and "feed_forward_post_norm"; a layer may
    have no feed-forward (then it needs neither "feed_forward_post_norm" nor a feed-forward norm).  The mixer's
    output is handed to the feed-forward's norm as a :class:`NormedDelta`, so its norm, the sum into the stream and
    the next norm are one kernel; the feed-forward's output (the experts' weighted rows, unsummed) is normed and
    added by the block's last kernel, or, in a step of one token per sequence, left to the next block's first
    norm as a :class:`NormedDelta`."""

    def __init__(self, spec, dtype, device):
        extra = dict(spec.extra)
        if spec.mixer_norm is None or "mixer_post_norm" not in extra:
            raise ValueError("the sandwich arrangement needs a norm before the mixer and a 'mixer_post_norm'")
        self.spec = spec
        self.mixer_norm = NORMS.build(spec.mixer_norm, dtype, device)
        self.mixer = MIXERS.build(spec.mixer, dtype, device)
        self.mixer_post_norm = NORMS.build(extra["mixer_post_norm"], dtype, device)
        self.feed_forward = self.feed_forward_norm = self.feed_forward_post_norm = None
        if spec.feed_forward is not None:
            if spec.feed_forward_norm is None or "feed_forward_post_norm" not in extra:
                raise ValueError("a sandwich block with a feed-forward needs its norm and a 'feed_forward_post_norm'")
            self.feed_forward_norm = NORMS.build(spec.feed_forward_norm, dtype, device)
            self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, dtype, device)
            self.feed_forward_post_norm = NORMS.build(extra["feed_forward_post_norm"], dtype, device)

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in self.parts().values())

    @property
    def launches_only(self) -> bool:
        return all(p.launches_only for p in self.parts().values())

    def parts(self):
        out = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "mixer_post_norm": self.mixer_post_norm}
        if self.feed_forward is not None:
            out.update({"feed_forward_norm": self.feed_forward_norm, "feed_forward": self.feed_forward,
                        "feed_forward_post_norm": self.feed_forward_post_norm})
        return out

    @staticmethod
    def _normed(out, post) -> NormedDelta:
        if hasattr(post, "as_normed"):       # a norm of another kind says itself what is left to be done
            return post.as_normed(out)
        return NormedDelta(out, post.weights["weight"], post.eps)

    def forward(self, ctx, x, pending, cache_view, state):
        from .norm import post_add_rmsnorm
        nt, d = x.shape
        x1 = ctx.scratch("block.x1", (nt, d), ctx.dtype)
        delta = ctx.scratch("block.delta", (nt, d), ctx.dtype)
        pending = resolve(pending, self.mixer_norm, delta, x=x, ctx=ctx)
        Layer._norm(self.mixer_norm, self.mixer, ctx, x, pending, x1)
        self.mixer.forward(ctx, x1, delta, cache_view, state)
        pending = self._normed(delta, self.mixer_post_norm)
        if self.feed_forward is not None:
            pending = resolve(pending, self.feed_forward_norm, delta, x=x, ctx=ctx)
            tail = self.feed_forward.norm_tail(ctx, nt)
            if tail is not None and tail.kind in self.feed_forward_norm.tails:
                # the feed-forward's router rides along with the kernel that norms the mixer's output, adds it and
                # norms the sum
                self.feed_forward_norm.forward(ctx, x, pending, None, x1, tail=tail)
                lazy = self.feed_forward.forward(ctx, x1, delta, tail=tail)
            else:
                self.feed_forward_norm.forward(ctx, x, pending, None, x1)
                lazy = self.feed_forward.forward(ctx, x1, delta)
            pending = self._normed(delta if lazy is None else lazy, self.feed_forward_post_norm)
        if ctx.decode:
            # one token per sequence: the step is a chain of small kernels, and the last norm, the sum and the next
            # block's (or the model's last) norm are one of them instead of two
            return pending
        # many tokens: the sum is done here, so that the layer's launches name no tensor of another layer (layers of
        # equal parts are then replayed with their own tensors put in)
        post_add_rmsnorm(ctx.dtype, x, pending, None, None, 0.0, None)
        return None


@ARRANGEMENTS.register("parallel")
class ParallelLayer:
    """A block whose mixer and feed-forward read the same stream, each through a norm of its own:

        x += mixer(f(norm_m(x))) + feed_forward(norm_f(x))

    ``f`` is an optional input filter of the mixer's side, named "mixer_input_filter" in ``LayerSpec.extra`` (a
    causal convolution over time, with per-sequence state).  A layer may have no feed-forward.  The two norms share
    their statistic: one kernel adds what the block before left pending (a pair of outputs, summed in float),
    and writes both normed rows.  The block leaves its own two outputs pending as a :class:`PairDelta`."""

    def __init__(self, spec, dtype, device):
        if spec.mixer_norm is None:
            raise ValueError("the parallel arrangement needs a norm before the mixer")
        extra = dict(spec.extra)
        self.spec = spec
        self.mixer_norm = NORMS.build(spec.mixer_norm, dtype, device)
        self.mixer = MIXERS.build(spec.mixer, dtype, device)
        self.filter = INPUT_FILTERS.build(extra["mixer_input_filter"], dtype, device) \
            if "mixer_input_filter" in extra else None
        self.feed_forward = self.feed_forward_norm = None
        if spec.feed_forward is not None:
            if spec.feed_forward_norm is None:
                raise ValueError("a parallel block with a feed-forward needs its norm")
            self.feed_forward_norm = NORMS.build(spec.feed_forward_norm, dtype, device)
            self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, dtype, device)
        # both norms in one kernel: two plain RMS norms over the same row with the same eps
        self._fused = all(n is None or (type(n).__name__ == "RMSNorm") for n in (self.mixer_norm, self.feed_forward_norm)) \
            and (self.feed_forward_norm is None or self.feed_forward_norm.eps == self.mixer_norm.eps)

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in self.parts().values())

    @property
    def launches_only(self) -> bool:
        return all(p.launches_only for p in self.parts().values())

    def parts(self):
        out = {"mixer_norm": self.mixer_norm, "mixer": self.mixer}
        if self.filter is not None:
            out["mixer_input_filter"] = self.filter
        if self.feed_forward is not None:
            out.update({"feed_forward_norm": self.feed_forward_norm, "feed_forward": self.feed_forward})
        return out

    def state_needs(self):
        """Per-sequence state by the name of the part that carries it."""
        out = {}
        if self.mixer.state_need() is not None:
            out["mixer"] = self.mixer.state_need()
        if self.filter is not None and self.filter.state_need() is not None:
            out["mixer_input_filter"] = self.filter.state_need()
        return out

    def forward(self, ctx, x, pending, cache_view, state):
        from .norm import pair_add_rmsnorm
        nt, d = x.shape
        state = state or {}
        h1 = ctx.scratch("block.x1", (nt, d), ctx.dtype)
        h2 = ctx.scratch("block.x2", (nt, d), ctx.dtype) if self.feed_forward is not None else None
        out_m = ctx.scratch("block.delta", (nt, d), ctx.dtype)
        out_f = ctx.scratch("block.delta2", (nt, d), ctx.dtype) if self.feed_forward is not None else None
        if isinstance(pending, (NormedDelta, WeightedRows)):
            pending = resolve(pending, None, out_m, x=x, ctx=ctx)
        if self._fused:
            pair_add_rmsnorm(ctx.dtype, x, pending, None, self.mixer_norm.weights["weight"], h1,
                             None if h2 is None else self.feed_forward_norm.weights["weight"], h2, self.mixer_norm.eps)
        else:
            pending = resolve(pending, self.mixer_norm, out_m, x=x, ctx=ctx)
            self.mixer_norm.forward(ctx, x, pending, None, h1)
            if h2 is not None:
                self.feed_forward_norm.forward(ctx, x, None, None, h2)
        if self.filter is not None:
            f1 = ctx.scratch("block.x1f", (nt, d), ctx.dtype)
            self.filter.forward(ctx, h1, f1, state.get("mixer_input_filter"))
            h1 = f1
        self.mixer.forward(ctx, h1, out_m, cache_view, state.get("mixer"))
        if self.feed_forward is None:
            return out_m
        lazy = self.feed_forward.forward(ctx, h2, out_f)
        if lazy is not None:
            from .feed_forward import sum_weighted_rows
            sum_weighted_rows(lazy, out_f)
        return PairDelta(out_m, out_f)


def add_pending(ctx, x, pending) -> None:
    """x += pending, at once and in float, for an arrangement that does not leave the sum to a norm."""
    if pending is None:
        return
    if isinstance(pending, NormedDelta):
        from .norm import post_add_rmsnorm
        post_add_rmsnorm(ctx.dtype, x, pending, None, None, 0.0, None)
        return
    if isinstance(pending, PairDelta):
        from .norm import pair_add_rmsnorm
        pair_add_rmsnorm(ctx.dtype, x, pending, None, None, None, None, None, 0.0)
        return
    if isinstance(pending, WeightedRows):
        from .feed_forward import sum_weighted_rows
        into = ctx.scratch("block.delta", tuple(x.shape), ctx.dtype)
        sum_weighted_rows(pending, into)
        pending = into
    x.add_(pending.float())


def resolve(pending, norm, into, x=None, ctx=None):
    """A pending WeightedRows stays as it is for a norm that sums it itself; else it is summed into ``into``.  A
    pending NormedDelta stays for a norm that takes one; else it is normed and added to the stream ``x`` now."""
    if isinstance(pending, NormedDelta):
        if getattr(norm, "takes_normed_delta", False):
            return pending
        if x is None or ctx is None:
            raise ValueError("a normed delta can only be resolved with the stream at hand")
        add_pending(ctx, x, pending)
        return None
    if isinstance(pending, PairDelta):
        if getattr(norm, "takes_pair_delta", False):
            return pending
        if x is None or ctx is None:
            raise ValueError("a pair of outputs can only be resolved with the stream at hand")
        add_pending(ctx, x, pending)
        return None
    if isinstance(pending, WeightedRows) and not getattr(norm, "takes_weighted_rows", False):
        from .feed_forward import sum_weighted_rows
        sum_weighted_rows(pending, into)
        return into
    return pending
