"""Grouped-query attention over the paged cache (models/llama/common/src/compute.rs:210-270).

qkv = x1 Wqkv^T (one merged product, heads ordered q, k, v); rotary encoding of q and k fused with
the write of k and v into the cache; causal attention of the step's tokens over everything their
sequences hold; out = o Wo^T.  The residual sum is the caller's (the block's) business.

Further mechanisms, each a parameter of the same mixer (a model that names none of them runs exactly the path
above): value heads of a size of their own (``dv``); a score multiplier other than dh^-1/2 (``scale``); capped
scores, cap * tanh(score / cap) (``softcap``); a sliding window (``window``: position i sees j iff i - j < window)
that keeps the sequence's first tokens visible (``keep_first``), the cache keeping every position; an RMS norm over
the WHOLE query projection and the whole key projection before the rotation (``qk_norm="whole"``, weights
``q_norm`` / ``k_norm``, ``eps``); a rotation of only the first entries of every head (the rotary part's ``dh``
below the head's); a gate on the output, o * sigmoid(Wg x1), whose projection rides in the merged product
(``gate``).  With any of them the step runs  merged product -> norm + rotation + cache write (one kernel) ->
windowed attention with the gate in its epilogue -> output product  (csrc/attention_window.cu, rope_cache.cu).

A second family, again parameters of the same mixer: a short causal convolution over time on every channel of the
q, k and v projections, ``conv_taps`` wide (weights ``conv``; the last ``conv_taps - 1`` projected rows are state of
the sequence; one tap is a weight per channel); an RMS norm per head with one weight of the head's size shared by all heads (``qk_norm="head"``); a
learned multiplier of every query head's scores (``temperature``, weights ``temp``); values that are cached rotated
by their own position over all of their entries, in adjacent pairs, with the rotary part's base and no rescaling,
and an output that is turned back by the query's position (``value_rotation``); a mask of chunks (``chunk``:
position i sees j <= i iff i // chunk == j // chunk); a learned number per head that joins the softmax's
denominator (``sink``, weights ``sink``); values blended with those that an earlier layer made for the same token
(``value_mix``: the layer that says "source" leaves its values, as they are after the convolution and before any
rotation, in float scratch memory of the step; a layer that says "blend" caches (1 - l) v + l v_source with its own
learned number l, weights ``vmix``).  With any of these the kernel between the product and the attention is
``tb_head_prep`` (csrc/head_prep.cu): convolution, norms, temperature, the blend, both rotations and the cache write
at once.  That kernel turns adjacent pairs; a rotary part that pairs entry i with i + dims/2 is met by reordering,
once at binding, the rows of the query and key projections (and of their norm weights and convolutions) that make the
rotated entries: a permutation applied to queries and keys alike, which leaves every score as it was.
"""
from __future__ import annotations

import math

import torch

from ..csrc import lib
from .base import MIXERS, POSITIONS, CacheNeed, Mixer, ParamDecl, StateNeed
from .linear import matmul_nt
from .spec import PartSpec


USE_TCGEN05 = True     # prompts: the tcgen05 kernel before the mma.sync one
USE_DECODE_RING = True  # decoding: the kernel with a ring of cache pages (TMA, tensor cores) before the register-staged one
FUSE_DECODE_ROPE = True # decoding: that kernel also rotates q and k and writes the cache (no rotary kernel)
RING_BLOCKS_PER_SM = 2  # decoding: the keys are sliced until that kernel has this many blocks per SM
USE_WINDOW_MMA = True   # the windowed path, bfloat16: the tensor-core kernel before the general one


@MIXERS.register("attention")
class Attention(Mixer):
    """params: width, nh, nkvh, dh, position (a PartSpec of a rotary encoding, or None); optional: dv, scale, softcap,
    window, keep_first, qk_norm, eps, gate (see the head of this file)."""

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.d = int(params["width"])
        self.nh = int(params["nh"])
        self.nkvh = int(params["nkvh"])
        self.dh = int(params["dh"])
        if self.nh % self.nkvh:
            raise ValueError(f"{self.nh} heads cannot share {self.nkvh} key/value heads")
        if self.dh <= 0 or self.dh > 256:
            raise ValueError(f"the attention kernels take head sizes up to 256; got {self.dh}")
        pos = params.get("position")
        self.position = POSITIONS.build(pos, dtype, device) if isinstance(pos, PartSpec) else None
        self.dv = int(params.get("dv") or self.dh)
        self.softcap = float(params.get("softcap") or 0.0)
        self.window = int(params.get("window") or 0)            # 0: no window
        self.keep_first = int(params.get("keep_first") or 0)
        self.qk_norm = params.get("qk_norm")
        self.gate = bool(params.get("gate", False))
        self.eps = float(params.get("eps", 0.0))
        if self.qk_norm not in (None, "whole", "head"):
            raise ValueError(f"unknown query/key norm {self.qk_norm!r}")
        self.conv_taps = int(params.get("conv_taps") or 0)          # 0: no convolution on the projections
        self.temperature = bool(params.get("temperature", False))
        self.value_rotation = bool(params.get("value_rotation", False))
        self.chunk = int(params.get("chunk") or 0)
        self.sink = bool(params.get("sink", False))
        self.value_mix = params.get("value_mix")
        if self.value_mix not in (None, "source", "blend"):
            raise ValueError(f"value_mix is 'source', 'blend' or absent, got {self.value_mix!r}")
        if self.conv_taps < 0 or self.conv_taps > 16 or self.chunk < 0:
            raise ValueError("convolutions of 1 to 16 taps; chunk not negative")
        # the second family of mechanisms: its own kernel between the product and the attention
        self.prepared = bool(self.conv_taps or self.qk_norm == "head" or self.temperature or self.value_rotation or
                             self.value_mix)
        if self.prepared and (self.gate or self.qk_norm == "whole"):
            raise ValueError("a norm over the whole projection or an output gate does not go with the per-head family")
        if self.dv <= 0 or self.dv > 256 or self.window < 0 or self.keep_first < 0 or self.softcap < 0:
            raise ValueError("value heads of 1..256 entries; window, keep_first and softcap not negative")
        # any of the further mechanisms takes the step to the windowed kernels
        self.extended = bool(self.dv != self.dh or self.softcap or self.window or self.qk_norm or self.gate or
                             "scale" in params or self.prepared or self.chunk or self.sink)
        if not self.extended and (self.dh % 16):
            raise ValueError(f"the attention kernels take head sizes 16, 32, ..., 256; got {self.dh}")
        self.rdims = 0
        if self.extended and self.position is not None:
            if device.type == "cuda" and self.position.rotation() is None:
                raise ValueError("the windowed attention takes a rotary position encoding or none")
            self.rdims = int(pos.get()["dh"])
            if self.rdims > self.dh:
                raise ValueError(f"a rotation of {self.rdims} entries does not fit heads of {self.dh}")
        self.value_position = None
        if self.value_rotation:
            if self.dv % 2 or not isinstance(pos, PartSpec):
                raise ValueError("rotated values need an even value size and the rotary part whose base they share")
            pp = pos.get()
            self.value_position = POSITIONS.build(PartSpec.of("rope", dh=self.dv, theta=pp["theta"], pairing="adjacent",
                                                              positions=pp["positions"]), dtype, device)
        self.qkv_width = (self.nh + self.nkvh) * self.dh + self.nkvh * self.dv + (self.nh * self.dv if self.gate else 0)
        self.scale = float(params["scale"]) if "scale" in params else 1.0 / math.sqrt(self.dh)
        # query tiles this mixer asks the step to plan: the general kernel's, and the prompt kernel's
        self.general_tile = lib.attention_tile_tokens(self.nh, self.nkvh)
        # bfloat16 prompts: the mma.sync kernel takes every head size, the tcgen05 kernel heads of 64 and 128
        self.prompt_tile = lib.attention_prefill_tile_tokens() if dtype == torch.bfloat16 else 0
        self.tc_tile = lib.attention_tc_tile_tokens() if (self.prompt_tile and self.dh in (64, 128)) else 0
        # the windowed path on the tensor cores: a block takes all query heads of a key head, 64 rows in all
        self.window_tile = lib.attention_window_mma_tile_tokens(self.nh, self.nkvh) \
            if (self.extended and dtype == torch.bfloat16) else 0
        if self.extended:
            self.prompt_tile = self.tc_tile = 0
        self.tile_sizes = [t for t in (self.general_tile, self.prompt_tile, self.tc_tile, self.window_tile) if t]

    @property
    def graph_safe(self) -> bool:
        return self.position is None or self.position.graph_safe

    @property
    def launches_only(self) -> bool:
        return self.position is None or self.position.launches_only

    def parameters(self):
        decl = {
            "wqkv": ParamDecl((self.qkv_width, self.d)),
            "wo": ParamDecl((self.d, self.nh * self.dv)),
        }
        if self.qk_norm == "whole":
            decl["q_norm"] = ParamDecl((self.nh * self.dh,), "norm", "ones")
            decl["k_norm"] = ParamDecl((self.nkvh * self.dh,), "norm", "ones")
        elif self.qk_norm == "head":
            decl["q_norm"] = ParamDecl((self.dh,), "norm", "ones")
            decl["k_norm"] = ParamDecl((self.dh,), "norm", "ones")
        if self.conv_taps:
            decl["conv"] = ParamDecl((self.qkv_width, self.conv_taps), "norm", "normal")
        if self.temperature:
            decl["temp"] = ParamDecl((self.nh,), "norm", "ones")
        if self.sink:
            decl["sink"] = ParamDecl((self.nh,), "norm", "normal")
        if self.value_mix == "blend":
            decl["vmix"] = ParamDecl((), "norm", "normal")
        if self.position is not None:      # what the position encoding has learned travels with its mixer
            decl.update({"position." + n: d for n, d in self.position.parameters().items()})
        return decl

    def bind(self, tensors) -> None:
        super().bind(tensors)
        if self.position is not None:
            self.position.bind({n: tensors["position." + n] for n in self.position.parameters()})
        if "vmix" in self.weights:
            self.weights["vmix"] = self.weights["vmix"].float().reshape(1).contiguous()
        if self.prepared and self.rdims and self.position.rotation()[2]:
            # halves paired: entry i of the rotated part goes to 2i, entry i + rdims/2 to 2i + 1, in every query and
            # key head, so that the kernel's adjacent pairs are the design's pairs
            r = self.rdims
            order = [j for i in range(r // 2) for j in (i, i + r // 2)] + list(range(r, self.dh))
            rows = [h * self.dh + j for h in range(self.nh + self.nkvh) for j in order]
            rows += list(range(len(rows), self.qkv_width))
            at = torch.tensor(rows, device=self.weights["wqkv"].device)
            self.weights["wqkv"] = self.weights["wqkv"][at].contiguous()
            if "conv" in self.weights:
                self.weights["conv"] = self.weights["conv"][at].contiguous()
            if self.qk_norm == "head":
                one = torch.tensor(order, device=self.weights["q_norm"].device)
                self.weights["q_norm"] = self.weights["q_norm"][one].contiguous()
                self.weights["k_norm"] = self.weights["k_norm"][one].contiguous()

    def cache_need(self):
        if self.dv != self.dh:
            return CacheNeed("full", self.nkvh, self.dh, (("dv", self.dv),))
        return CacheNeed("full", self.nkvh, self.dh)

    def state_need(self):
        if self.conv_taps > 1:      # the convolutions' last inputs: the projected rows before the step's first
            return StateNeed(((self.conv_taps - 1) * self.qkv_width,), torch.float32)
        return None

    def _forward_prepared(self, ctx, x1, out, cache, state) -> None:
        """The step of the per-head family: see the head of this file."""
        nt = x1.shape[0]
        sfx = lib.suffix(self.dtype)
        w = self.weights
        z = ctx.scratch("attn.qkv", (nt, self.qkv_width), self.dtype)        # q | k | v as the product leaves them
        matmul_nt(x1, w["wqkv"], z)
        table = ctx.page_table(cache)
        cos = sin = vcos = vsin = None
        if self.rdims:
            cos, sin, _ = self.position.rotation()      # halves paired: the rows were reordered at binding
        if self.value_position is not None:
            vcos, vsin, _ = self.value_position.rotation()
        kc, vc = (cache.k, cache.v) if cache.writable else (None, None)
        q = ctx.scratch("attn.q", (nt, self.nh * self.dh), self.dtype)
        # the values of the blend's source: written by the source's run, read by the later runs of the same step
        vfirst = ctx.scratch("attn.v_source", (nt, self.nkvh * self.dv), torch.float32) if self.value_mix else None
        lib.call("tb_head_prep_" + sfx, lib.ptr(z), self.qkv_width, lib.ptr(w.get("conv")), lib.ptr(state),
                 0 if state is None else state.stride(0), lib.ptr(w.get("q_norm")), lib.ptr(w.get("k_norm")),
                 lib.ptr(w.get("temp")), self.eps, lib.ptr(cos), lib.ptr(sin), lib.ptr(vcos), lib.ptr(vsin), lib.ptr(q),
                 lib.ptr(kc), lib.ptr(vc), lib.ptr(ctx.tok_seq), lib.ptr(ctx.tok_pos), lib.ptr(ctx.seq_start),
                 lib.ptr(ctx.slots), lib.ptr(table), ctx.max_pages, nt, self.nh, self.nkvh, self.dh, self.dv,
                 self.rdims, max(self.conv_taps, 1), 1 if ctx.decode else 0, lib.ptr(vfirst),
                 lib.ptr(w["vmix"]) if self.value_mix == "blend" else 0)
        if self.conv_taps > 1 and not ctx.decode:
            # every token has read the old inputs: the state moves on to the step's last rows
            lib.call("tb_conv_roll_" + sfx, lib.ptr(z), self.qkv_width, lib.ptr(state), state.stride(0),
                     lib.ptr(ctx.seq_start), lib.ptr(ctx.slots), ctx.B, self.qkv_width, self.conv_taps)
        o = ctx.scratch("attn.o", (nt, self.nh * self.dv), self.dtype)
        window = self.window if self.window else 1 << 30
        run_window_attention(ctx, self, q, o, None, cache, table, nt, window, q_stride=self.nh * self.dh,
                             sinks=w.get("sink"), ocos=vcos, osin=vsin)
        matmul_nt(o, w["wo"], out)

    def _forward_window(self, ctx, x1, out, cache) -> None:
        """The step with the further mechanisms: see the head of this file."""
        nt = x1.shape[0]
        sfx = lib.suffix(self.dtype)
        w = self.weights
        z = ctx.scratch("attn.qkv", (nt, self.qkv_width), self.dtype)        # q | k | v | gate
        matmul_nt(x1, w["wqkv"], z)
        table = ctx.page_table(cache)
        cos = sin = None
        half = 0
        if self.rdims:
            cos, sin, half = self.position.rotation()
        kc, vc = (cache.k, cache.v) if cache.writable else (None, None)
        lib.call("tb_qknorm_rope_cache_" + sfx, lib.ptr(z), self.qkv_width, lib.ptr(w.get("q_norm")),
                 lib.ptr(w.get("k_norm")), self.eps, lib.ptr(ctx.tok_seq), lib.ptr(ctx.tok_pos), lib.ptr(table),
                 ctx.max_pages, lib.ptr(cos), lib.ptr(sin), lib.ptr(kc), lib.ptr(vc), nt, self.nh, self.nkvh, self.dh,
                 self.dv, self.rdims, half)
        o = ctx.scratch("attn.o", (nt, self.nh * self.dv), self.dtype)
        gate = z[:, (self.nh + self.nkvh) * self.dh + self.nkvh * self.dv:] if self.gate else None
        window = self.window if self.window else 1 << 30
        run_window_attention(ctx, self, z, o, gate, cache, table, nt, window,
                             sinks=w.get("sink") if self.sink else None)
        matmul_nt(o, w["wo"], out)

    def forward(self, ctx, x1, out, cache, state) -> None:
        if self.prepared:
            self._forward_prepared(ctx, x1, out, cache, state)
            return
        if self.extended:
            self._forward_window(ctx, x1, out, cache)
            return
        nt = x1.shape[0]
        sfx = lib.suffix(self.dtype)
        qkv = ctx.scratch("attn.qkv", (nt, self.qkv_width), self.dtype)
        matmul_nt(x1, self.weights["wqkv"], qkv)
        table = ctx.page_table(cache)
        rotation = self.position.rotation() if self.position is not None else None
        if rotation is not None:
            cos, sin, half = rotation      # a rotary encoding: fused with the cache write below
        else:
            if self.position is not None:
                self.position.apply(ctx, qkv, self.nh, self.nkvh, self.dh)     # any other: by its own means
            cos, sin = ctx.identity_rotation(self.dh)
            half = 0
        o = ctx.scratch("attn.o", (nt, self.nh * self.dh), self.dtype)
        if ctx.decode and self._decode_fused(ctx, qkv, o, cache, table, nt, cos, sin, half):
            matmul_nt(o, self.weights["wo"], out)      # rotation and cache write happened inside the attention kernel
            return
        kc, vc = (cache.k, cache.v) if cache.writable else (None, None)
        lib.call("tb_rope_cache_" + sfx, lib.ptr(qkv), lib.ptr(ctx.tok_seq), lib.ptr(ctx.tok_pos),
                 lib.ptr(table), ctx.max_pages, lib.ptr(cos), lib.ptr(sin), lib.ptr(kc), lib.ptr(vc),
                 nt, self.nh, self.nkvh, self.dh, half)
        if ctx.decode and self._decode_kernel(ctx, qkv, o, cache, table, nt, sfx):
            matmul_nt(o, self.weights["wo"], out)
            return
        if self.tc_tile and nt >= 2 * ctx.B and USE_TCGEN05:
            # prompts: S and O in tensor memory, K and V pages by TMA
            tiles = ctx.tiles(self.tc_tile)
            if lib.try_call("tb_attention_tc_bf16", lib.ptr(qkv), lib.ptr(o), lib.ptr(cache.k), lib.ptr(cache.v),
                            lib.ptr(tiles.seq), lib.ptr(tiles.t0), lib.ptr(tiles.nq), lib.ptr(ctx.tok_pos),
                            lib.ptr(table), tiles.count, nt, ctx.max_pages, self.qkv_width, self.nh, self.nkvh,
                            self.dh, cache.k.shape[0], self.scale):
                matmul_nt(o, self.weights["wo"], out)
                return
        if self.prompt_tile and nt >= 2 * ctx.B:
            tiles = ctx.tiles(self.prompt_tile)
            if lib.try_call("tb_attention_prefill_bf16", lib.ptr(qkv), lib.ptr(o), lib.ptr(cache.k), lib.ptr(cache.v),
                            lib.ptr(tiles.seq), lib.ptr(tiles.t0), lib.ptr(tiles.nq), lib.ptr(ctx.tok_pos),
                            lib.ptr(table), tiles.count, ctx.max_pages, self.qkv_width, self.nh, self.nkvh, self.dh,
                            self.scale):
                matmul_nt(o, self.weights["wo"], out)
                return
        tiles = ctx.tiles(self.general_tile)
        splits = ctx.attention_splits(tiles.count, self.nh, self.nkvh)
        partial = None
        if splits > 1:
            partial = ctx.scratch("attn.partial", (nt, self.nh, splits, self.dh + 2), torch.float32)
        lib.call("tb_attention_" + sfx, lib.ptr(qkv), lib.ptr(o), lib.ptr(cache.k), lib.ptr(cache.v),
                 lib.ptr(tiles.seq), lib.ptr(tiles.t0), lib.ptr(tiles.nq), lib.ptr(ctx.tok_pos), lib.ptr(table),
                 lib.ptr(partial), tiles.count, nt, ctx.max_pages, self.qkv_width, self.nh, self.nkvh, self.dh,
                 splits, self.scale)
        matmul_nt(o, self.weights["wo"], out)

    def _ring(self) -> bool:
        """Whether decoding runs the kernel with a ring of cache pages (TMA, tensor cores)."""
        return USE_DECODE_RING and self.dtype == torch.bfloat16 and self.dh in (64, 128, 192, 256)

    def _decode_plan(self, ctx, nt, ring):
        """Slices of the keys, and the scratch they need: (splits, partial results, counters of finished slices)."""
        group = self.nh // self.nkvh
        gc = 16 if ring else 1 if group == 1 else 2 if group == 2 else 4       # query heads of a group per block
        blocks = nt * self.nkvh * ((group + gc - 1) // gc)
        # Slices of the keys so that the blocks fill the GPU: as many blocks as are resident at once for the kernel
        # that keeps a ring of pages in shared memory (two per SM: measured best in the step at batch 1 to 16, also with
        # lengths that differ 16-fold; alone, the kernel would rather have one per SM), eight times the SMs for the register-staged one.  A function of the batch's shape
        # alone, since a captured graph keeps it for as long as the sequences grow (the kernels cut short sequences
        # into fewer slices by themselves).
        splits = int(max(1, min(32, ((RING_BLOCKS_PER_SM if ring else 8) * ctx.engine.sm_count) // blocks)))
        partial = done = None
        if splits > 1:
            partial = ctx.scratch("attn.partial", (nt, self.nh, splits, self.dh + 2), torch.float32)
            if ring:    # the block that finishes a head group's last slice merges them
                done = ctx.scratch("attn.done", (nt * self.nh,), torch.int32, zero=True)
        return splits, partial, done

    def _decode_fused(self, ctx, qkv, o, cache, table, nt, cos, sin, half) -> bool:
        """One token per sequence, straight from the q-k-v product: the ring kernel also rotates the queries and the
        new key and writes key and value into the cache.  False (and nothing done) if it refuses."""
        if not (self._ring() and FUSE_DECODE_ROPE):
            return False
        splits, partial, done = self._decode_plan(ctx, nt, True)
        return lib.try_call("tb_attention_decode_rope_bf16", lib.ptr(qkv), lib.ptr(o), lib.ptr(cache.k), lib.ptr(cache.v),
                            lib.ptr(ctx.tok_seq), lib.ptr(ctx.tok_pos), lib.ptr(table), lib.ptr(partial), lib.ptr(done),
                            lib.ptr(cos), lib.ptr(sin), nt, ctx.max_pages, self.qkv_width, self.nh, self.nkvh, self.dh,
                            splits, cache.k.shape[0], half, 1 if cache.writable else 0, self.scale)

    def _decode_kernel(self, ctx, qkv, o, cache, table, nt, sfx) -> bool:
        """One token per sequence, queries rotated and the cache written: the kernels that stream the cache.  False if
        they refuse the head size."""
        ring = self._ring()
        splits, partial, done = self._decode_plan(ctx, nt, ring)
        if ring:
            if lib.try_call("tb_attention_decode_mma_bf16", lib.ptr(qkv), lib.ptr(o), lib.ptr(cache.k),
                            lib.ptr(cache.v), lib.ptr(ctx.tok_seq), lib.ptr(ctx.tok_pos), lib.ptr(table),
                            lib.ptr(partial), lib.ptr(done), nt, ctx.max_pages, self.qkv_width, self.nh, self.nkvh,
                            self.dh, splits, cache.k.shape[0], self.scale):
                return True
        return lib.try_call("tb_attention_decode_" + sfx, lib.ptr(qkv), lib.ptr(o), lib.ptr(cache.k), lib.ptr(cache.v),
                            lib.ptr(ctx.tok_seq), lib.ptr(ctx.tok_pos), lib.ptr(table), lib.ptr(partial), nt,
                            ctx.max_pages, self.qkv_width, self.nh, self.nkvh, self.dh, splits, self.scale)


def run_window_attention(ctx, m, z, o, gate, cache, table, nt, window, q_stride=None, sinks=None, ocos=None,
                         osin=None) -> None:
    """The windowed attention of the step's rotated queries ``z`` over the cache, into ``o`` (gate applied).
    ``sinks``: a number per head in the softmax's denominator; ``ocos, osin``: tables that turn the output back."""
    sfx = lib.suffix(m.dtype)
    q_stride = m.qkv_width if q_stride is None else q_stride
    if m.window_tile and USE_WINDOW_MMA:
        # bfloat16: the tensor-core kernel, for prompts and decoding alike.  Slices of the visited pages so that a few
        # sequences still fill the GPU: a function of the batch's shape alone (a captured graph keeps it)
        tiles = ctx.tiles(m.window_tile)
        reach = min(window, ctx.engine.spec.max_context) if not m.chunk else min(window, m.chunk)
        pages = (reach + m.keep_first + 63) // 64 + 2
        splits = int(max(1, min(16, pages, (2 * ctx.engine.sm_count) // max(1, tiles.count * m.nkvh))))
        partial = ctx.scratch("attn.partial", (nt, m.nh, splits, m.dv + 2), torch.float32) if splits > 1 else None
        if lib.try_call("tb_attention_window_mma_bf16", lib.ptr(z), lib.ptr(o), lib.ptr(cache.k), lib.ptr(cache.v),
                        lib.ptr(gate), lib.ptr(tiles.seq), lib.ptr(tiles.t0), lib.ptr(tiles.nq), lib.ptr(ctx.tok_pos),
                        lib.ptr(table), lib.ptr(partial), tiles.count, nt, ctx.max_pages, q_stride, m.qkv_width,
                        m.nh, m.nkvh, m.dh, m.dv, splits, window, m.keep_first, m.scale, m.softcap, m.chunk,
                        lib.ptr(sinks), lib.ptr(ocos), lib.ptr(osin)):
            return
    tiles = ctx.tiles(m.general_tile)
    # slices of the visited keys so that a few sequences still fill the GPU: a function of the batch's shape alone (a
    # captured graph keeps it), and no more than the window has 32-key tiles
    splits = ctx.attention_splits(tiles.count, m.nh, m.nkvh)
    reach = min(window, 1 << 20) if not m.chunk else min(window, m.chunk)
    splits = int(max(1, min(splits, (reach + m.keep_first + 31) // 32 + 1)))
    partial = ctx.scratch("attn.partial", (nt, m.nh, splits, m.dv + 2), torch.float32) if splits > 1 else None
    lib.call("tb_attention_window_" + sfx, lib.ptr(z), lib.ptr(o), lib.ptr(cache.k), lib.ptr(cache.v), lib.ptr(gate),
             lib.ptr(tiles.seq), lib.ptr(tiles.t0), lib.ptr(tiles.nq), lib.ptr(ctx.tok_pos), lib.ptr(table),
             lib.ptr(partial), tiles.count, nt, ctx.max_pages, q_stride, m.qkv_width, m.nh, m.nkvh, m.dh, m.dv,
             splits, window, m.keep_first, m.scale, m.softcap, m.chunk, lib.ptr(sinks), lib.ptr(ocos), lib.ptr(osin))
