"""Attention through a low-rank latent, with a sliding window and a rotated key part that all heads share.

    zq = Wdq x1,  cq = zq / rms(zq) * wq_norm,  q = Wuq cq                   per head: [dim plain | rot_dim rotated]
    [zc | zr] = Wdkv x1,  c = zc / rms(zc) * wc_norm,  kr = rotate(zr)      one row per token, cached: [c | kr]
    head h:  k_plain = Wuk_h c,  v = Wuv_h c
    score_h(t, j) = (q_plain . k_plain_j + rotate(q_rot) . kr_j) * scale,   j visible iff 0 <= t - j < window
    out = Wo concat_h(softmax(score_h) v_h)

Nothing per head is cached or formed for cached tokens: the query goes to the latent's side
(Wuk_h^T q_plain, a product batched over the heads), the attention kernel runs over the shared rows
[c | kr] with c as the value as well, and Wuv_h is applied to the attention's result (csrc/latent.cu).
A layer with ``own_latent`` False makes no latent: it reads the cache of the run named by its
``RunEntry.cache_of``, with its own Wuk, Wuv, queries and window.

Variants by parameter: ``q_rank`` 0: the queries come straight from one projection, q = Wq x1 (no low-rank step and
no query norm; Wq rides in the merged first product); ``window`` 0: plain causal attention; a rotary part with
adjacent pairs (2i, 2i + 1): the kernels pair entry i with i + dims/2, so the rows of the projections that make
the rotated entries are reordered once at binding (evens, then odds) -- a permutation applied to queries and
keys alike, which leaves every score as it was; ``sink``: a learned number per head (weights ``sink``) that joins
the softmax's denominator once, with no key and no value; ``head_gate``: head h's output is multiplied by
sigmoid(Wg x1)_h, one number per head, whose projection (weights ``wg`` [heads, width]) rides in the merged first
product, behind the latent's rows.
"""
from __future__ import annotations

import torch

from ..csrc import lib
from .base import MIXERS, POSITIONS, CacheNeed, Mixer, ParamDecl
from .linear import batched_matmul, matmul_nt
from .spec import PartSpec


USE_TENSOR_CORES = True    # bfloat16: the mma.sync kernel before the general one


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """params: width, heads, dim, rot_dim, vdim, kv_rank, q_rank, window, scale, eps, own_latent, position (a
    PartSpec of a rotary encoding of the first ``dh`` entries of the rotated part, pairing "half")."""
    launches_only = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        g = lambda n: int(params[n])
        self.d, self.H, self.dim, self.rot, self.vdim = g("width"), g("heads"), g("dim"), g("rot_dim"), g("vdim")
        self.rank, self.q_rank, self.window = g("kv_rank"), g("q_rank"), g("window")
        self.scale, self.eps = float(params["scale"]), float(params["eps"])
        self.own_latent = bool(params.get("own_latent", True))
        self.sink = bool(params.get("sink", False))
        self.head_gate = bool(params.get("head_gate", False))
        pos = params.get("position")
        if not isinstance(pos, PartSpec):
            raise ValueError("latent attention needs the rotary encoding of its rotated part ('position')")
        self.position = POSITIONS.build(pos, dtype, device)
        self.rdims = int(pos.get()["dh"])
        self.adjacent = pos.get().get("pairing", "adjacent") == "adjacent"
        if self.adjacent:       # the tables are the same; the pairing is met by reordering the projections' rows
            self.position = POSITIONS.build(PartSpec.of("rope", **dict(pos.get(), pairing="half")), dtype, device)
        if self.rdims > self.rot or self.rdims % 2:
            raise ValueError(f"the rotated part of {self.rot} entries takes a rotation of an even number of them, "
                             f"got {self.rdims}")
        if self.adjacent and not self.own_latent:
            raise ValueError("adjacent pairs are met in the layer that makes the latent; a reader needs halves paired")
        if self.window < 0:
            raise ValueError(f"the window must not be negative, got {self.window}")
        if self.window == 0:
            self.window = 1 << 30      # plain causal: the mask never cuts
        if self.rank > 512:
            raise ValueError(f"the latent attention kernel takes latents of up to 512 entries, got {self.rank}")
        self.q_head = self.dim + self.rot
        self.tile = lib.latent_attention_tile_tokens(self.H)
        self.tile_sizes = [self.tile]

    @property
    def graph_safe(self) -> bool:
        return self.position.graph_safe

    def parameters(self):
        first = self.q_rank if self.q_rank else self.H * self.q_head
        down = first + (self.rank + self.rot if self.own_latent else 0)
        decl = {
            "wdown": ParamDecl((down, self.d)),            # rows: Wdq (or Wq itself without a low-rank step), then (own latent) Wdkv
            "uk": ParamDecl((self.H * self.dim, self.rank)),
            "uv": ParamDecl((self.H * self.vdim, self.rank)),
            "wo": ParamDecl((self.d, self.H * self.vdim)),
        }
        if self.q_rank:
            decl["q_norm"] = ParamDecl((self.q_rank,), "norm", "ones")
            decl["uq"] = ParamDecl((self.H * self.q_head, self.q_rank))
        if self.own_latent:
            decl["c_norm"] = ParamDecl((self.rank,), "norm", "ones")
        if self.sink:
            decl["sink"] = ParamDecl((self.H,), "norm", "normal")
        if self.head_gate:
            decl["wg"] = ParamDecl((self.H, self.d))
        return decl

    def _halves(self, rows: torch.Tensor) -> torch.Tensor:
        """Rows of a rotated part [..., rot, in]: the rotated entries' evens first, then their odds."""
        r = self.rdims
        order = list(range(0, r, 2)) + list(range(1, r, 2)) + list(range(r, self.rot))
        return rows[..., order, :]

    def bind(self, tensors) -> None:
        super().bind(tensors)
        # the product that takes the queries to the latent's side wants Wuk_h^T as its [out, in] matrix
        uk = self.weights.pop("uk")
        self.weights["ukT"] = uk.view(self.H, self.dim, self.rank).transpose(1, 2).contiguous()
        if self.adjacent and self.rdims:
            qname = "uq" if self.q_rank else "wdown"
            wq = self.weights[qname].clone()
            nq = self.H * self.q_head
            heads = wq[:nq].view(self.H, self.q_head, -1)
            heads[:, self.dim:] = self._halves(heads[:, self.dim:].clone())
            if self.own_latent:
                wd = wq if qname == "wdown" else self.weights["wdown"].clone()
                wd[-self.rot:] = self._halves(wd[-self.rot:].clone())
                self.weights["wdown"] = wd
            self.weights[qname] = wq
        if self.head_gate:
            # the gates' rows join the first product, behind everything else, so that they cost no launch of their
            # own; zero rows up to a multiple of eight keep the rows of its result 16-byte aligned
            wd, wg = self.weights["wdown"], self.weights.pop("wg")
            self.gate_at = wd.shape[0]
            pad = (-(wd.shape[0] + self.H)) % 8
            self.weights["wdown"] = torch.cat([wd, wg, wd.new_zeros((pad, self.d))], dim=0).contiguous()

    def cache_need(self):
        return CacheNeed("latent", 1, self.rank + self.rot, (("rank", self.rank), ("rot", self.rot)))

    def forward(self, ctx, x1, out, cache, state) -> None:
        nt, H = x1.shape[0], self.H
        sfx = lib.suffix(self.dtype)
        w = self.weights
        wa = w["wdown"].shape[0]
        a = ctx.scratch("latent.a", (nt, wa), self.dtype)
        matmul_nt(x1, w["wdown"], a)
        table = ctx.page_table(cache)
        cos, sin, _ = self.position.rotation()
        write = self.own_latent and cache.writable
        if self.q_rank:
            cq = ctx.scratch("latent.cq", (nt, self.q_rank), self.dtype)
            lib.call("tb_latent_prep_" + sfx, lib.ptr(a), wa, lib.ptr(w["q_norm"]), lib.ptr(w.get("c_norm")), self.eps,
                     lib.ptr(cq), lib.ptr(cache.kv) if write else 0, lib.ptr(ctx.tok_seq), lib.ptr(ctx.tok_pos),
                     lib.ptr(table), ctx.max_pages, lib.ptr(cos), lib.ptr(sin), nt, self.q_rank, self.rank, self.rot,
                     self.rdims)
            q = ctx.scratch("latent.q", (nt, H * self.q_head), self.dtype)
            matmul_nt(cq, w["uq"], q)
        else:
            # the queries are the first columns of the merged product; the latent's part follows them
            q = a[:, :H * self.q_head]
            if write:
                lib.call("tb_latent_prep_" + sfx, lib.ptr(a[:, H * self.q_head:]), wa, 0, lib.ptr(w.get("c_norm")),
                         self.eps, 0, lib.ptr(cache.kv), lib.ptr(ctx.tok_seq), lib.ptr(ctx.tok_pos), lib.ptr(table),
                         ctx.max_pages, lib.ptr(cos), lib.ptr(sin), nt, 0, self.rank, self.rot, self.rdims)
        ldq = q.stride(0)
        sinks = w.get("sink")
        gate = a[:, self.gate_at:] if self.head_gate else None
        qa = ctx.scratch("latent.qa", (nt, H, self.rank), self.dtype)
        batched_matmul(q.as_strided((nt, H, self.dim), (ldq, self.q_head, 1)), w["ukT"], qa)
        ol = ctx.scratch("latent.ol", (nt, H, self.rank), self.dtype)
        tiles = ctx.tiles(self.tile)
        done = False
        if self.dtype == torch.bfloat16 and USE_TENSOR_CORES:
            # Slices of the key range, so that a few sequences still fill the GPU: a function of the batch's shape
            # alone (a captured graph keeps it), at most one slice per page of the window
            blocks = tiles.count * ((H + 15) // 16)
            splits = int(max(1, min(16, (min(self.window, ctx.engine.spec.max_context) + 63) // 64 + 1,
                                    (2 * ctx.engine.sm_count) // max(1, blocks))))
            partial = ctx.scratch("latent.partial", (nt, H, splits, self.rank + 2), torch.float32) if splits > 1 else None
            done = lib.try_call("tb_latent_attention_mma_bf16", lib.ptr(qa), lib.ptr(q), lib.ptr(ol), lib.ptr(partial),
                                lib.ptr(cache.kv), lib.ptr(tiles.seq), lib.ptr(tiles.t0), lib.ptr(tiles.nq),
                                lib.ptr(ctx.tok_pos), lib.ptr(table), lib.ptr(cos), lib.ptr(sin), tiles.count, nt,
                                ctx.max_pages, ldq, self.q_head, H, self.rank, self.rot, self.rdims,
                                self.window, splits, self.scale, lib.ptr(sinks), lib.ptr(gate), wa)
        if not done:
            lib.call("tb_latent_attention_" + sfx, lib.ptr(qa), lib.ptr(q), lib.ptr(ol), lib.ptr(cache.kv),
                     lib.ptr(tiles.seq), lib.ptr(tiles.t0), lib.ptr(tiles.nq), lib.ptr(ctx.tok_pos), lib.ptr(table),
                     lib.ptr(cos), lib.ptr(sin), tiles.count, ctx.max_pages, ldq, self.q_head, self.dim, H,
                     self.rank, self.rot, self.rdims, self.window, self.scale, lib.ptr(sinks), lib.ptr(gate), wa)
        o = ctx.scratch("latent.o", (nt, H, self.vdim), self.dtype)
        batched_matmul(ol, w["uv"].view(H, self.vdim, self.rank), o)
        matmul_nt(o.view(nt, H * self.vdim), w["wo"], out)
