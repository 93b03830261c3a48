"""Small Fugavik configurations, random model folders in the design's own tensor names, and the comparison of the
engine with the plain implementation (tests/plain/fugavik_plain.py)."""
import json
import os

import torch
from safetensors.torch import save_file

from plain import fugavik_plain as FP


def attention(heads, kv_heads, dim, vdim, dims=None, base=10000.0, factor=None, scale=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if dims != 0:
        m["rot"] = {"base": base, "dims": dim if dims is None else dims}
        if factor is not None:
            m["rot"]["scaling"] = {"factor": factor}
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m}


def latent(heads, dim, vdim, kv_rank, scale=None):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank,
                                                  "scale": dim ** -0.5 if scale is None else scale}}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(vocab, width, layers, eps=1e-6):
    return {"architecture": "Fugavik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "max_context": 1024,
            "layers": [dict(l[0], mlp=l[1]) for l in layers]}


# Sizes differ from one another wherever the design lets them: query and key heads, the two head sizes, groups of
# one and of several, a rotation of a part of the head, of all of it and of none, frequencies divided by 1, 2.5 and
# 4, blending layers with a plain one between them and before them, one to five taps, one to three experts per
# token, layers with and without a feed-forward, every kind of mixer first and last.
MIXED = config(101, 64, [
    (attention(4, 2, 16, 24, dims=8, factor=2.5), dense(40)),
    (delta(4, 2, 16, 24, 3), moe(24, 5, 2)),
    (attention(6, 3, 16, 8, factor=4.0, scale=0.4, v_mix=True), None),
    (latent(4, 16, 24, 32, scale=0.3), moe(16, 3, 3)),
    (attention(3, 3, 32, 8, dims=0, v_mix=True), dense(48)),
    (delta(2, 2, 24, 8, 2), None),
    (attention(3, 3, 8, 8, dims=4, v_mix=True), moe(32, 4, 1)),
], eps=1e-5)
NO_EXPERTS = config(90, 64, [
    (delta(4, 2, 16, 24, 4), dense(40)),
    (attention(4, 2, 16, 16, v_mix=True, factor=2.0), dense(32)),
    (latent(2, 32, 16, 64), None),
    (attention(4, 2, 16, 16, v_mix=True, dims=8), dense(32)),
], eps=1e-5)
ONLY_ATTENTION = config(64, 48, [(attention(4, 2, 16, 32, dims=8, factor=3.0, v_mix=True), None),
                                 (attention(2, 2, 24, 32, v_mix=True), None)])
ONLY_LATENT = config(64, 48, [(latent(3, 16, 20, 24, scale=0.5), None)])
ONLY_DELTA = config(64, 48, [(delta(4, 2, 12, 20, 4), None)])
ONLY_DENSE = config(64, 48, [(delta(1, 1, 8, 8, 1), dense(56))])
ONLY_EXPERTS = config(64, 48, [(delta(1, 1, 8, 8, 2), moe(24, 6, 2))])
# sizes the vector and tensor-core forms take, sequences across several pages
WIDE = config(128, 128, [
    (attention(4, 2, 64, 64, factor=2.0, v_mix=True), moe(64, 8, 2)),
    (delta(2, 1, 64, 64, 4), dense(96)),
    (latent(8, 32, 64, 96, scale=0.2), moe(64, 8, 1)),
    (attention(8, 2, 128, 64, dims=64, base=5e5, v_mix=True), dense(96)),
    (latent(4, 64, 32, 64), None),
    (delta(2, 2, 128, 128, 4), None),
])
# sizes that are multiples of nothing: every vectorized or tensor-core form refuses them
ODD = config(77, 50, [
    (attention(3, 1, 10, 7, dims=6, factor=1.5, v_mix=True), dense(22)),
    (delta(3, 3, 10, 7, 1), moe(9, 3, 2)),
    (latent(5, 6, 7, 11), None),
    (delta(6, 2, 36, 33, 5), dense(30)),
    (attention(5, 5, 12, 6, dims=12), moe(7, 2, 1)),
    (attention(1, 1, 14, 7, dims=2, v_mix=True), None),
], eps=1e-4)
CONFIGS = {"mixed": (MIXED, 1), "no_experts": (NO_EXPERTS, 2), "attention": (ONLY_ATTENTION, 3),
           "latent": (ONLY_LATENT, 4), "delta": (ONLY_DELTA, 5), "dense": (ONLY_DENSE, 6), "experts": (ONLY_EXPERTS, 7),
           "wide": (WIDE, 8), "odd": (ODD, 9)}
STD = {"wide": 0.08}


def random_config(rng, nice):
    """A configuration drawn with ``rng`` (random.Random): 3 to 8 layers of every kind in any order, sizes that the
    vector and tensor-core forms take (``nice``) or that are multiples of nothing."""
    pick = rng.choice
    width = pick([64, 128, 192, 256, 320]) if nice else pick([50, 72, 100, 136, 200])
    vm = (pick([1, 2, 4]), pick([16, 32, 64, 80]) if nice else pick([6, 20, 24, 40]))     # what blending layers share
    layers = []
    for _ in range(rng.randrange(3, 9)):
        kind = pick(["attention", "attention", "latent", "delta"])
        if kind == "attention":
            v_mix = rng.random() < 0.7
            kv = vm[0] if v_mix else pick([1, 2, 3, 4])
            dim = pick([16, 32, 64, 128]) if nice else pick([8, 12, 24, 40, 72])
            vdim = vm[1] if v_mix else (pick([16, 32, 64, 128]) if nice else pick([10, 24, 36]))
            mix = attention(kv * pick([1, 2, 4]), kv, dim, vdim, dims=pick([0, dim, dim // 2, dim]) // 2 * 2,
                            base=pick([10000.0, 500000.0, 100.0]), factor=pick([None, 2.0, 4.0, 1.0, 8.0]),
                            scale=pick([None, 0.1, 0.2]), v_mix=v_mix)
        elif kind == "latent":
            mix = latent(pick([1, 2, 4, 8, 16]) if nice else pick([3, 5, 6]), pick([16, 32, 64]) if nice else pick([8, 12, 24]),
                         pick([16, 32, 64, 80, 128]) if nice else pick([10, 20, 36]),
                         pick([32, 64, 96, 128, 256]) if nice else pick([24, 40, 72, 200]), scale=pick([None, 0.15]))
        else:
            kv = pick([1, 2, 4])
            mix = delta(kv * pick([1, 2]), kv, pick([16, 32, 64, 128]) if nice else pick([8, 24, 40]),
                        pick([16, 32, 64, 128]) if nice else pick([12, 20, 33]), pick([1, 2, 3, 4, 4, 5]))
        r = rng.random()
        if r < 0.15:
            mlp = None
        elif r < 0.55:
            mlp = dense(pick([64, 128, 320]) if nice else pick([30, 52, 100]))
        else:
            e = pick([2, 4, 8, 16]) if nice else pick([3, 5, 7])
            mlp = moe(pick([32, 64, 128]) if nice else pick([12, 20, 44]), e, rng.randrange(1, min(e, 4) + 1))
        layers.append((mix, mlp))
    return config(rng.randrange(90, 700), width, layers, eps=pick([1e-6, 1e-5]))


def random_tensors(cfg, seed, std=0.15):
    """Every tensor of a model file, by the design's names.  Nothing is left where it would hide a fault: norm
    weights around one, norm biases and layer scales away from zero and one, sinks of the size of the scores, blending
    numbers around a half, decays that neither keep everything nor forget at once, routers with clear preferences."""
    g = torch.Generator().manual_seed(seed)
    d = cfg["width"]
    out = {}

    def mat(name, *shape, s=std):
        out[name] = (torch.randn(*shape, generator=g) * s).bfloat16()

    def around_one(name, n, spread=0.3):
        out[name] = (1.0 + spread * torch.randn(n, generator=g)).bfloat16()

    def post_norm(p, n):
        around_one(p + f"norm{n}", d)
        mat(p + f"norm{n}.b", d, s=0.3)
        out[p + f"ls{n}"] = (0.3 + 0.7 * torch.rand(d, generator=g)).bfloat16()

    mat("embed", cfg["vocab"], d, s=1.0)
    mat("head", cfg["vocab"], d)
    around_one("final.norm", d)
    mat("final.norm.b", d, s=0.3)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        post_norm(p, 1)
        H = m["heads"]
        if layer["type"] == "attention":
            G = m["kv_heads"]
            mat(p + "mix.q", H * m["dim"], d, s=2 * std)
            mat(p + "mix.k", G * m["dim"], d, s=2 * std)
            mat(p + "mix.v", G * m["vdim"], d)
            around_one(p + "mix.q.norm", m["dim"])
            around_one(p + "mix.k.norm", m["dim"])
            out[p + "mix.q.norm"] = (out[p + "mix.q.norm"].float() * 2.0).bfloat16()     # scores that matter
            mat(p + "mix.sink", H, s=1.5)
            if m.get("v_mix"):
                out[p + "mix.vmix"] = (0.3 + 0.4 * torch.rand((), generator=g)).bfloat16()
            mat(p + "mix.o", d, H * m["vdim"])
        elif layer["type"] == "latent_attention":
            r = m["kv_rank"]
            mat(p + "mix.q", H * m["dim"], d, s=2 * std)
            mat(p + "mix.dkv", r, d)
            around_one(p + "mix.dkv.norm", r)
            mat(p + "mix.uk", H * m["dim"], r, s=3 * std)
            mat(p + "mix.uv", H * m["vdim"], r)
            mat(p + "mix.sink", H, s=1.5)
            mat(p + "mix.g", H, d, s=3 * std)
            mat(p + "mix.o", d, H * m["vdim"])
        else:
            G = m["kv_heads"]
            hk, hv, T = G * m["dim"], H * m["vdim"], m["conv"]
            for n, rows in (("q", hk), ("k", hk), ("v", hv)):
                mat(p + "mix." + n, rows, d, s=2 * std)
                mat(p + f"mix.{n}.conv", rows, T, s=0.6)
            mat(p + "mix.b", H, d, s=3 * std)
            mat(p + "mix.a", H, d, s=3 * std)
            out[p + "mix.A_log"] = (torch.rand(H, generator=g) * 3.0 - 2.5).bfloat16()
            out[p + "mix.dt_bias"] = (torch.randn(H, generator=g) - 1.0).bfloat16()
            mat(p + "mix.g", hv, d, s=2 * std)
            around_one(p + "mix.norm", m["vdim"])
            mat(p + "mix.o", d, hv)
        f = layer["mlp"]
        if f:
            post_norm(p, 2)
            if f["kind"] == "dense":
                mat(p + "mlp.up", f["ff"], d)
                mat(p + "mlp.down", d, f["ff"])
            else:
                # clear preferences, but logits that stay where a sigmoid still tells them apart
                mat(p + "mlp.router", f["router"]["experts"], d, s=4 * std * 8.0 / d ** 0.5)
                for e in range(f["router"]["experts"]):
                    mat(p + f"mlp.e{e}.gate", f["expert"]["ff"], d)
                    mat(p + f"mlp.e{e}.up", f["expert"]["ff"], d)
                    mat(p + f"mlp.e{e}.down", d, f["expert"]["ff"])
    return out


def make_folder(tmp, name, tensors_edit=None, cfg=None, seed=None):
    if cfg is None:
        cfg, seed = CONFIGS[name]
    folder = os.path.join(str(tmp), "fugavik_" + name)
    if not os.path.isdir(folder):
        os.makedirs(folder)
        tensors = random_tensors(cfg, seed, STD.get(name, 0.15))
        if tensors_edit:
            tensors_edit(tensors)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg, f)
        save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return folder


FP32_TOL = 2e-4           # on logits of order one to ten
# bfloat16, against the plain implementation run exactly, as fractions of the request's largest |logit|.  Every
# part's output is normed before it joins the stream, which carries the rounding of a small output over at full
# size: the plain implementation itself, rounding where a 16-bit path stores an activation, moves by 1 to 2 % on
# average and by up to 15 % at single ill-conditioned positions.  A wrong mechanism (a sink left out, a lost state,
# a missing gate, values not blended) moves most positions by a tenth of the largest logit or more.
BF16_MEAN_TOL = 2.0 ** -5     # the mean over a request's positions (requests of 20 positions or more)
BF16_EACH_TOL = 2.0 ** -2     # any single position
BF16_REL_TOL = 2.0 ** -5      # for comparisons of the engine with itself
# An expert chosen although the exact run scores another higher: in float32 the scores must lie within 1e-4; in
# bfloat16 the router's logits within an eighth of the layer's largest, for all but 3 % of the tokens (at least one).
BF16_GAP_TOL = 2.0 ** -3


def as_bfloat16(x):
    return x.bfloat16().to(x.dtype)


def moe_layers(cfg):
    return [i for i, l in enumerate(cfg["layers"]) if l["mlp"] and l["mlp"]["kind"] == "moe"]


class Recorder:
    """Collects the experts the engine chose, per layer with experts, in the order the tokens were fed."""

    def __init__(self, engine):
        self.engine, self.rec = engine, []
        engine.recorder = self

    def __call__(self, name, run, t):
        if name == "moe.topk_idx":
            self.rec.append((run, t.cpu()))

    def take(self):
        out = {}
        for run, t in self.rec:
            out.setdefault(run, []).append(t)
        self.rec = []
        return {run: torch.cat(ts) for run, ts in out.items()}


def check_request(cfg, tensors, tokens, got_rows, dtype, label="", routes=None, floor=False):
    """got_rows: {position: logits row of the engine}.  routes: {layer: [len(tokens), top]} the engine's experts, or
    None.  The plain run is forced to the engine's experts; where they differ from its own choice, the gap between
    the scores of the last chosen and of the engine's pick must be within the rounding of the path.  ``floor``: for
    models drawn at random, whose conditioning nobody chose: the bfloat16 rules are no tighter than twice (the mean)
    and two and a half times (any position) what the plain implementation itself loses when it rounds where a
    16-bit path stores, the float32 rule no tighter than three times what it loses when it computes in 32-bit."""
    choices = None if routes is None else {l: (r.long(), None) for l, r in routes.items()}
    scores = {}
    ref = FP.forward(cfg, tensors, tokens, choices=choices, scores_out=scores)
    if routes is not None:
        for l, r in routes.items():
            k = r.shape[1]
            if dtype == "float32":
                z, tol = scores[l], 1e-4
            else:
                z = torch.logit(scores[l].clamp(1e-12, 1 - 1e-12))
                tol = BF16_GAP_TOL * float(z.abs().max())
            kept = torch.topk(z, k, dim=-1).values[:, -1]              # what an expert needs to be chosen
            took = torch.gather(z, 1, r.long()).min(dim=-1).values
            over = int(((kept - took) > tol).sum())
            allowed = 0 if dtype == "float32" else max(1, (3 * len(tokens)) // 100)
            assert over <= allowed, f"{label}: layer {l}: {over} tokens took an expert over a clear gap " \
                                    f"(worst {float((kept - took).max()):.3e}, rule {tol:.3e})"
    top = float(ref.abs().max())
    tol = FP32_TOL * max(1.0, top / 10.0) if dtype == "float32" else BF16_EACH_TOL * top
    mean_tol = BF16_MEAN_TOL * top
    if floor and dtype == "bfloat16":
        lost = (FP.forward(cfg, tensors, tokens, store=as_bfloat16, choices=choices) - ref).abs().max(dim=1).values
        tol, mean_tol = max(tol, 2.5 * float(lost.max())), max(mean_tol, 2.0 * float(lost.mean()))
    if floor and dtype == "float32":
        # three times what the plain implementation itself loses when it computes in 32-bit
        single = FP.forward(cfg, {k: v.float() if v.is_floating_point() else v for k, v in tensors.items()}, tokens,
                            choices=choices)
        tol = max(tol, 3.0 * float((single.double() - ref).abs().max()))
    worst, total = 0.0, 0.0
    for pos, row in sorted(got_rows.items()):
        diff = float((torch.as_tensor(row).double() - ref[pos]).abs().max())
        worst, total = max(worst, diff), total + diff
        assert diff <= tol, f"{label}: position {pos} (first wrong of the request): |diff| {diff:.3e} > {tol:.3e}"
    if dtype == "bfloat16" and len(got_rows) >= 20:
        mean = total / len(got_rows)
        assert mean <= mean_tol, f"{label}: mean |diff| {mean:.3e} > {mean_tol:.3e}"
    return worst


def run_cuts(engine, tokens, cuts, graphs=False, record=True):
    """One request through the engine in steps of the given sizes (the rest one token at a time); returns
    ({position: logits} for every position, {layer: experts [len(tokens), top]} or None)."""
    engine.use_graphs = graphs
    rec = Recorder(engine) if record and not graphs else None
    try:
        slot = engine.open()
        rows, at = {}, 0
        sizes = list(cuts) + [1] * (len(tokens) - sum(cuts))
        for n in sizes:
            lg = engine.step([slot], [tokens[at:at + n]], [list(range(n))]).cpu()
            for i in range(n):
                rows[at + i] = lg[i].clone()
            at += n
        engine.close(slot)
        engine.check_kernels()
    finally:
        engine.recorder = None
    routes = rec.take() if rec is not None else None
    return rows, (routes or None)
