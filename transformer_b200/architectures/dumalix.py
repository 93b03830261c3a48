"""The Dumalix decoder: blocks whose mixer and feed-forward read the same stream in parallel, each through a norm
with a weight stored around zero; what the mixer reads passes a short causal convolution over time first; a group
of layers may run several times in a row with the same weights, each pass with a cache and state of its own and
preceded by a projection that mixes the embedding output back into the stream.  Two kinds of mixer: grouped-query
attention with convolutions on its projections, a norm per head, rescaled rotary frequencies, rotated values, a
temperature per head, a mask of chunks and a sink in the softmax; and causal attention through a shared latent.
The feed-forward is a clamped gated pair.

Everything particular to the design lives here: how its configuration becomes a :class:`ModelSpec`, and which
file tensors fill which parameters.  Tensor names of a model file (linear weights [out, in]):

    embed [vocab, width]    loop.in [width, 2 width]    final.norm [width]    head [vocab, width]
    l<i>.norm1, .norm2 [width]      l<i>.canon1 [width, taps]
    attention:         l<i>.mix.q [heads dim, width]  .k [kv_heads dim, width]  .v [kv_heads vdim, width]
                       .q.conv, .k.conv, .v.conv [rows, taps]  .q.norm, .k.norm [dim]  .temp, .sink [heads]
                       .o [width, heads vdim]
    latent_attention:  l<i>.mix.q [heads (dim + rot_dim), width]  .dkv [kv_rank + rot_dim, width]  .dkv.norm [kv_rank]
                       .uk [heads dim, kv_rank]  .uv [heads vdim, kv_rank]  .o [width, heads vdim]
    feed-forward:      l<i>.mlp.gate, .up [ff, width]  .down [width, ff]
"""
from __future__ import annotations

from typing import List

from ..config.dumalix import ChunkAttentionMeta, DumalixMeta
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..weights.plan import Source, TensorRule, single

GLU_ALPHA = 1.702      # the slope of the gate's sigmoid: the design fixes it


def build_spec(m: DumalixMeta) -> ModelSpec:
    norm = PartSpec.of("rmsnorm", width=m.width, eps=m.eps, one_plus=True)
    layers = []
    for layer in m.layers:
        x = layer.mixer
        ramp = None if x.rot_ramp is None else x.rot_ramp.as_tuple()
        rope = PartSpec.of("rope", dh=x.rot_dims, theta=x.rot_base, pairing="adjacent", positions=m.max_context,
                           ramp=ramp) if x.rot_dims else None
        if isinstance(x, ChunkAttentionMeta):
            mixer = PartSpec.of("attention", width=m.width, nh=x.heads, nkvh=x.kv_heads, dh=x.dim, dv=x.vdim,
                                scale=x.scale, qk_norm="head", eps=m.eps, conv_taps=x.conv,
                                temperature=True, sink=True, value_rotation=True, chunk=x.chunk,
                                position=rope if rope is not None else
                                PartSpec.of("rope", dh=0, theta=x.rot_base, pairing="adjacent", positions=m.max_context))
        else:
            mixer = PartSpec.of("latent_attention", width=m.width, heads=x.heads, dim=x.dim, rot_dim=x.rot_dim,
                                vdim=x.vdim, kv_rank=x.kv_rank, q_rank=0, window=0, scale=x.scale, eps=m.eps,
                                position=rope if rope is not None else
                                PartSpec.of("rope", dh=0, theta=x.rot_base, pairing="adjacent", positions=m.max_context))
        ff = None
        if layer.mlp is not None:
            ff = PartSpec.of("swiglu", width=m.width, di=layer.mlp.ff, glu_alpha=GLU_ALPHA, glu_limit=layer.mlp.limit)
        extra = ()
        if m.canon_taps:
            extra = (("mixer_input_filter", PartSpec.of("causal_conv", width=m.width, taps=m.canon_taps)),)
        layers.append(LayerSpec(mixer=mixer, feed_forward=ff, mixer_norm=norm,
                                feed_forward_norm=norm if ff is not None else None, arrangement="parallel",
                                extra=extra))
    joints = (PartSpec.of("reinject", width=m.width),) if m.loop is not None else ()
    order = tuple(RunEntry(i, joint=0 if first else None) for i, first in m.run_order())
    return ModelSpec(
        width=m.width, vocab=m.vocab, max_context=m.max_context, layers=tuple(layers), order=order,
        embedding=PartSpec.of("lookup", vocab=m.vocab, width=m.width), final_norm=norm,
        head=PartSpec.of("linear", vocab=m.vocab, width=m.width, tied=False),
        stop_tokens=tuple(m.eos), joints=joints,
    )


def tensor_plan(m: DumalixMeta) -> List[TensorRule]:
    d = m.width
    rules = [TensorRule(("embedding", "table"), (m.vocab, d), "matrix", (single("embed", (m.vocab, d)),))]
    if m.loop is not None:
        rules.append(TensorRule(("joints", 0, "weight"), (d, 2 * d), "matrix", (single("loop.in", (d, 2 * d)),)))
    for i, layer in enumerate(m.layers):
        p, L = f"l{i}.", ("layers", i)
        mx = L + ("mixer",)

        def vec(dest, name, n, init="normal"):
            rules.append(TensorRule(dest, (n,), "norm", (single(p + name, (n,)),), init=init))

        def mat(dest, name, shape):
            rules.append(TensorRule(dest, tuple(shape), "matrix", (single(p + name, shape),)))

        vec(L + ("mixer_norm", "weight"), "norm1", d)
        if m.canon_taps:
            rules.append(TensorRule(L + ("mixer_input_filter", "weight"), (d, m.canon_taps), "norm",
                                    (single(p + "canon1", (d, m.canon_taps)),)))
        x = layer.mixer
        if isinstance(x, ChunkAttentionMeta):
            hq, hk, hv, ho = x.heads * x.dim, x.kv_heads * x.dim, x.kv_heads * x.vdim, x.heads * x.vdim
            rules.append(TensorRule(mx + ("wqkv",), (hq + hk + hv, d), "matrix", (
                Source((p + "mix.q", p + "mix.k", p + "mix.v"), ((hq, d), (hk, d), (hv, d)), "cat0"),)))
            if x.conv:
                T = x.conv
                rules.append(TensorRule(mx + ("conv",), (hq + hk + hv, T), "norm", (
                    Source((p + "mix.q.conv", p + "mix.k.conv", p + "mix.v.conv"), ((hq, T), (hk, T), (hv, T)), "cat0"),)))
            vec(mx + ("q_norm",), "mix.q.norm", x.dim, "ones")
            vec(mx + ("k_norm",), "mix.k.norm", x.dim, "ones")
            vec(mx + ("temp",), "mix.temp", x.heads, "ones")
            vec(mx + ("sink",), "mix.sink", x.heads)
            mat(mx + ("wo",), "mix.o", (d, ho))
        else:
            hq, lat = x.heads * (x.dim + x.rot_dim), x.kv_rank + x.rot_dim
            rules.append(TensorRule(mx + ("wdown",), (hq + lat, d), "matrix", (
                Source((p + "mix.q", p + "mix.dkv"), ((hq, d), (lat, d)), "cat0"),)))
            vec(mx + ("c_norm",), "mix.dkv.norm", x.kv_rank, "ones")
            mat(mx + ("uk",), "mix.uk", (x.heads * x.dim, x.kv_rank))
            mat(mx + ("uv",), "mix.uv", (x.heads * x.vdim, x.kv_rank))
            mat(mx + ("wo",), "mix.o", (d, x.heads * x.vdim))
        f = layer.mlp
        if f is None:
            continue
        vec(L + ("feed_forward_norm", "weight"), "norm2", d)
        ff = L + ("feed_forward",)
        rules.append(TensorRule(ff + ("wgu",), (2 * f.ff, d), "matrix", (
            Source((p + "mlp.gate", p + "mlp.up"), ((f.ff, d), (f.ff, d)), "cat0"),)))
        mat(ff + ("wd",), "mlp.down", (d, f.ff))
    rules.append(TensorRule(("final_norm", "weight"), (d,), "norm", (single("final.norm", (d,)),)))
    rules.append(TensorRule(("head", "weight"), (m.vocab, d), "matrix", (single("head", (m.vocab, d)),)))
    return rules


DUMALIX = register_architecture(Architecture(
    name="dumalix",
    config_cls=DumalixMeta,
    build_spec=build_spec,
    tensor_plan=tensor_plan,
    names=("dumalix", "Dumalix"),
))
