"""The Fugavik decoder: blocks that read the residual stream as it is and pass what their parts produce through a
layer norm (mean taken off, weight and bias) and a learned multiplier per channel before it joins the stream.
Three kinds of mixer: grouped-query attention with a norm per head on queries and keys, a rotation of halves whose
frequencies are all divided by one factor, a sink in the softmax, and values blended with those of the first
blending layer; causal attention through a cached latent with a sink and one sigmoid gate per head; a gated delta
rule with one decay per head and a silu gate on its normed output.  Two kinds of feed-forward: a dense pair with a
squared relu between, and sigmoid-scored experts whose weight multiplies what the chosen expert reads.

Everything particular to the design lives here: how its configuration becomes a :class:`ModelSpec`, and which
file tensors fill which parameters.  Tensor names of a model file (linear weights [out, in]):

    embed [vocab, width]    final.norm, final.norm.b [width]    head [vocab, width]
    l<i>.norm1, .norm1.b, .ls1 [width]     norm and multiplier of the mixer's output;  .norm2, .norm2.b, .ls2 the same
                                           for the feed-forward's
    attention:         l<i>.mix.q [heads dim, width]  .k [kv_heads dim, width]  .v [kv_heads vdim, width]
                       .q.norm, .k.norm [dim]  .sink [heads]  .vmix []  .o [width, heads vdim]
    latent_attention:  l<i>.mix.q [heads dim, width]  .dkv [kv_rank, width]  .dkv.norm [kv_rank]
                       .uk [heads dim, kv_rank]  .uv [heads vdim, kv_rank]  .sink [heads]  .g [heads, width]
                       .o [width, heads vdim]
    delta:             l<i>.mix.q, .k [kv_heads dim, width]  .v [heads vdim, width]  .q.conv, .k.conv, .v.conv [rows, taps]
                       .b, .a [heads, width]  .A_log, .dt_bias [heads]  .g [heads vdim, width]  .norm [vdim]
                       .o [width, heads vdim]
    dense:             l<i>.mlp.up [ff, width]  .down [width, ff]
    moe:               l<i>.mlp.router [experts, width]  .e<j>.gate, .e<j>.up [ff, width]  .e<j>.down [width, ff]
"""
from __future__ import annotations

from typing import List

from ..config.fugavik import AttentionMeta, DenseMeta, FugavikMeta, LatentMeta
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..weights.plan import Source, TensorRule, single


def build_spec(m: FugavikMeta) -> ModelSpec:
    read = PartSpec.of("none", width=m.width)                                   # the parts read the stream as it is
    post = PartSpec.of("layernorm", width=m.width, eps=m.eps, bias=True, scale=True)
    source = m.first_v_mix()
    layers, order = [], []
    for i, layer in enumerate(m.layers):
        x = layer.mixer
        if isinstance(x, AttentionMeta):
            rope = PartSpec.of("rope", dh=x.rot_dims, theta=x.rot_base, pairing="half", positions=m.max_context,
                               linear=x.rot_factor)
            mixer = PartSpec.of("attention", width=m.width, nh=x.heads, nkvh=x.kv_heads, dh=x.dim, dv=x.vdim,
                                scale=x.scale, qk_norm="head", eps=m.eps, sink=True, position=rope,
                                value_mix=None if not x.v_mix else "source" if i == source else "blend")
        elif isinstance(x, LatentMeta):
            none = PartSpec.of("rope", dh=0, theta=10000.0, pairing="half", positions=m.max_context)
            mixer = PartSpec.of("latent_attention", width=m.width, heads=x.heads, dim=x.dim, rot_dim=0, vdim=x.vdim,
                                kv_rank=x.kv_rank, q_rank=0, window=0, scale=x.scale, eps=m.eps, sink=True,
                                head_gate=True, position=none)
        else:
            mixer = PartSpec.of("channel_delta", width=m.width, heads=x.heads, kv_heads=x.kv_heads, dim=x.dim,
                                vdim=x.vdim, taps=x.conv, decay="head", decay_rank=0, gate_rank=0, gate_act="silu",
                                eps=m.eps)
        order.append(RunEntry(i))
        extra = [("mixer_post_norm", post)]
        ff = None
        f = layer.mlp
        if f is not None:
            if isinstance(f, DenseMeta):
                ff = PartSpec.of("mlp", width=m.width, di=f.ff, act="relu2")
            else:
                ff = PartSpec.of("moe", width=m.width, di=f.ff, nexp=f.experts, nexp_use=f.top, scoring="sigmoid",
                                 weight_on="input")
            extra.append(("feed_forward_post_norm", post))
        layers.append(LayerSpec(mixer=mixer, feed_forward=ff, mixer_norm=read,
                                feed_forward_norm=read if ff is not None else None, arrangement="sandwich",
                                extra=tuple(extra)))
    return ModelSpec(
        width=m.width, vocab=m.vocab, max_context=m.max_context, layers=tuple(layers), order=tuple(order),
        embedding=PartSpec.of("lookup", vocab=m.vocab, width=m.width),
        final_norm=PartSpec.of("layernorm", width=m.width, eps=m.eps, bias=True),
        head=PartSpec.of("linear", vocab=m.vocab, width=m.width, tied=False),
        stop_tokens=tuple(m.eos),
    )


def tensor_plan(m: FugavikMeta) -> List[TensorRule]:
    d = m.width
    source = m.first_v_mix()
    rules = [TensorRule(("embedding", "table"), (m.vocab, d), "matrix", (single("embed", (m.vocab, d)),))]
    for i, layer in enumerate(m.layers):
        p, L = f"l{i}.", ("layers", i)
        mx = L + ("mixer",)

        def vec(dest, name, n, init="normal"):
            shape = (n,) if n is not None else ()
            rules.append(TensorRule(dest, shape, "norm", (single(p + name, shape),), init=init))

        def mat(dest, name, shape):
            rules.append(TensorRule(dest, tuple(shape), "matrix", (single(p + name, shape),)))

        def post_norm(part, n):
            vec(L + (part, "weight"), f"norm{n}", d, "ones")
            vec(L + (part, "bias"), f"norm{n}.b", d)
            vec(L + (part, "scale"), f"ls{n}", d, "ones")

        post_norm("mixer_post_norm", 1)
        x = layer.mixer
        if isinstance(x, AttentionMeta):
            hq, hk, hv, ho = x.heads * x.dim, x.kv_heads * x.dim, x.kv_heads * x.vdim, x.heads * x.vdim
            rules.append(TensorRule(mx + ("wqkv",), (hq + hk + hv, d), "matrix", (
                Source((p + "mix.q", p + "mix.k", p + "mix.v"), ((hq, d), (hk, d), (hv, d)), "cat0"),)))
            vec(mx + ("q_norm",), "mix.q.norm", x.dim, "ones")
            vec(mx + ("k_norm",), "mix.k.norm", x.dim, "ones")
            vec(mx + ("sink",), "mix.sink", x.heads)
            if x.v_mix and i != source:
                vec(mx + ("vmix",), "mix.vmix", None)
            else:       # the first blending layer's number is not used; a layer that does not blend has no use for one
                rules.append(TensorRule(mx + ("vmix",), (), "norm", (single(p + "mix.vmix", ()),), unused=True))
            mat(mx + ("wo",), "mix.o", (d, ho))
        elif isinstance(x, LatentMeta):
            hq, r = x.heads * x.dim, x.kv_rank
            rules.append(TensorRule(mx + ("wdown",), (hq + r, d), "matrix", (
                Source((p + "mix.q", p + "mix.dkv"), ((hq, d), (r, d)), "cat0"),)))
            vec(mx + ("c_norm",), "mix.dkv.norm", r, "ones")
            mat(mx + ("uk",), "mix.uk", (hq, r))
            mat(mx + ("uv",), "mix.uv", (x.heads * x.vdim, r))
            vec(mx + ("sink",), "mix.sink", x.heads)
            mat(mx + ("wg",), "mix.g", (x.heads, d))
            mat(mx + ("wo",), "mix.o", (d, x.heads * x.vdim))
        else:
            hk, hv, T = x.kv_heads * x.dim, x.heads * x.vdim, x.conv
            rules.append(TensorRule(mx + ("win",), (2 * hk + 2 * hv, d), "matrix", (
                Source((p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g"), ((hk, d), (hk, d), (hv, d), (hv, d)),
                       "cat0"),)))
            rules.append(TensorRule(mx + ("conv",), (2 * hk + hv, T), "norm", (
                Source((p + "mix.q.conv", p + "mix.k.conv", p + "mix.v.conv"), ((hk, T), (hk, T), (hv, T)), "cat0"),)))
            mat(mx + ("wb",), "mix.b", (x.heads, d))
            mat(mx + ("wa",), "mix.a", (x.heads, d))
            vec(mx + ("dt_bias",), "mix.dt_bias", x.heads)
            vec(mx + ("A_log",), "mix.A_log", x.heads)
            vec(mx + ("norm",), "mix.norm", x.vdim, "ones")
            mat(mx + ("wo",), "mix.o", (d, hv))
        f = layer.mlp
        if f is None:
            continue
        post_norm("feed_forward_post_norm", 2)
        ff = L + ("feed_forward",)
        if isinstance(f, DenseMeta):
            mat(ff + ("wu",), "mlp.up", (f.ff, d))
            mat(ff + ("wd",), "mlp.down", (d, f.ff))
        else:
            E = f.experts
            mat(ff + ("router",), "mlp.router", (E, d))
            rules.append(TensorRule(ff + ("wgu",), (E, 2 * f.ff, d), "matrix", (
                Source(tuple(p + f"mlp.e{e}.{which}" for e in range(E) for which in ("gate", "up")),
                       ((f.ff, d),) * (2 * E), "stack0_of_row_pairs"),)))
            rules.append(TensorRule(ff + ("wd",), (E, d, f.ff), "matrix", (
                Source(tuple(p + f"mlp.e{e}.down" for e in range(E)), ((d, f.ff),) * E, "stack0"),)))
    rules.append(TensorRule(("final_norm", "weight"), (d,), "norm", (single("final.norm", (d,)),), init="ones"))
    rules.append(TensorRule(("final_norm", "bias"), (d,), "norm", (single("final.norm.b", (d,)),)))
    rules.append(TensorRule(("head", "weight"), (m.vocab, d), "matrix", (single("head", (m.vocab, d)),)))
    return rules


FUGAVIK = register_architecture(Architecture(
    name="fugavik",
    config_cls=FugavikMeta,
    build_spec=build_spec,
    tensor_plan=tensor_plan,
    names=("fugavik", "Fugavik"),
))
