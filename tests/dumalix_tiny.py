"""Small Dumalix configurations, random model folders in the design's own tensor names, and the comparison of the
engine with the plain implementation (tests/plain/dumalix_plain.py)."""
import json
import os

import torch
from safetensors.torch import save_file

from plain import dumalix_plain as DP


def rot(base, dims, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling is not None:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def attention(heads, kv_heads, dim, vdim, conv=3, chunk=None, dims=None, base=10000.0, scaling=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "rot": rot(base, dim if dims is None else dims, scaling), "scale": dim ** -0.5 if scale is None else scale}
    if conv is not None:        # absent: no convolution on the projections; 1: a weight per channel
        m["conv"] = conv
    if chunk is not None:
        m["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": m}


def latent(heads, dim, rot_dim, vdim, kv_rank, base=10000.0, scaling=None, scale=None):
    return {"type": "latent_attention", "mixer": {
        "heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
        "rot": rot(base, rot_dim, scaling), "scale": (dim + rot_dim) ** -0.5 if scale is None else scale}}


def dense(ff, limit=1.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def config(vocab, width, layers, eps=1e-6, taps=3, loop=None):
    out = {"architecture": "Dumalix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "max_context": 1024,
           "layers": [dict(l[0], mlp=l[1]) for l in layers]}
    if taps:
        out["canon"] = {"taps": taps}
    if loop is not None:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


# Sizes differ from one another wherever the design lets them: query and key heads, the two head sizes, groups of
# one and of several, a rotation of a part of the head and of all of it, rescaled frequencies with the ramp inside
# the head, chunks shorter than a page and across page borders or none, one to five taps or no convolution, layers with and without
# a feed-forward, a repeated group at the start, in the middle and up to the end, three passes, one, or no loop.
MIXED = config(101, 64, [
    (latent(3, 16, 8, 12, 24, base=5000.0, scaling=(4.0, 64, 8.0, 1.0), scale=0.2), dense(48, 0.8)),
    (attention(4, 2, 16, 24, conv=3, chunk=40, dims=8, scaling=(8.0, 32, 4.0, 0.5), scale=0.3), dense(40, 2.0)),
    (attention(3, 3, 12, 8, conv=2, dims=12, base=300.0), None),
    (latent(2, 32, 16, 32, 32, scaling=(2.0, 128, 16.0, 2.0)), dense(24, 1.5)),
], eps=1e-5, taps=4, loop=(1, 3, 2))
ONLY_ATTENTION = config(64, 48, [(attention(4, 2, 16, 8, conv=4, chunk=6, dims=8, scaling=(3.0, 16, 2.0, 0.25)), None)],
                        taps=0)
ONLY_LATENT = config(64, 48, [(latent(4, 8, 8, 16, 16, scaling=(5.0, 32, 4.0, 1.0), scale=0.4), None)], taps=0)
ONLY_DENSE = config(64, 48, [(attention(1, 1, 8, 8, conv=1), dense(56, 0.5))], taps=2, loop=(0, 1, 1))
# head sizes the tensor-core kernels take, chunks across several pages
WIDE = config(128, 128, [
    (attention(4, 2, 64, 64, conv=4, chunk=100, dims=32, scaling=(3.0, 256, 8.0, 1.0)), dense(96)),
    (latent(4, 64, 32, 64, 64, scaling=(4.0, 256, 16.0, 1.0)), None),
    (attention(8, 2, 128, 64, conv=2, chunk=64, dims=64, base=5e5), dense(96, 3.0)),
    (attention(2, 2, 32, 32, conv=None, dims=32), None),
    (latent(8, 32, 16, 32, 96), dense(64)),
], taps=2, loop=(2, 5, 2))
# sizes that are multiples of nothing: every vectorized or tensor-core form refuses them
ODD = config(77, 50, [
    (attention(5, 1, 10, 6, conv=5, chunk=7, dims=6, scaling=(2.0, 16, 2.0, 0.5)), dense(22, 0.7)),
    (latent(3, 10, 6, 14, 20, base=77.0), None),
    (attention(6, 2, 18, 22, conv=2, chunk=130, dims=18), dense(30)),
], eps=1e-4, taps=5, loop=(0, 2, 3))
CONFIGS = {"mixed": (MIXED, 1), "attention": (ONLY_ATTENTION, 2), "latent": (ONLY_LATENT, 3), "dense": (ONLY_DENSE, 4),
           "wide": (WIDE, 5), "odd": (ODD, 6)}
STD = {"wide": 0.08}


def random_tensors(cfg, seed, std=0.15):
    """Every tensor of a model file, by the design's names; norm weights around zero where the design adds one,
    around one elsewhere, temperatures and sinks that matter."""
    g = torch.Generator().manual_seed(seed)
    d = cfg["width"]
    out = {}

    def mat(name, *shape, s=std):
        out[name] = (torch.randn(*shape, generator=g) * s).bfloat16()

    def around(name, n, mid):
        out[name] = (mid + 0.3 * torch.randn(n, generator=g)).bfloat16()

    mat("embed", cfg["vocab"], d, s=1.0)
    mat("head", cfg["vocab"], d)
    around("final.norm", d, 0.0)
    if cfg.get("loop"):
        mat("loop.in", d, 2 * d, s=1.0 / (2 * d) ** 0.5)
    taps = (cfg.get("canon") or {}).get("taps", 0)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        around(p + "norm1", d, 0.0)
        if taps:
            mat(p + "canon1", d, taps, s=0.4)
        H = m["heads"]
        if layer["type"] == "attention":
            G, T = m["kv_heads"], m.get("conv", 0)
            for n, rows in (("q", H * m["dim"]), ("k", G * m["dim"]), ("v", G * m["vdim"])):
                mat(p + "mix." + n, rows, d, s=2 * std)
                if T:
                    mat(p + f"mix.{n}.conv", rows, T, s=0.6)
            around(p + "mix.q.norm", m["dim"], 1.3)          # scores that matter, and that bfloat16 can still carry
            around(p + "mix.k.norm", m["dim"], 1.0)
            out[p + "mix.temp"] = (0.5 + torch.rand(H, generator=g)).bfloat16()
            out[p + "mix.sink"] = (torch.randn(H, generator=g) * 2.0).bfloat16()
            mat(p + "mix.o", d, H * m["vdim"])
        else:
            mat(p + "mix.q", H * (m["dim"] + m["rot_dim"]), d, s=1.5 * std)
            mat(p + "mix.dkv", m["kv_rank"] + m["rot_dim"], d, s=2 * std)
            around(p + "mix.dkv.norm", m["kv_rank"], 1.0)
            mat(p + "mix.uk", H * m["dim"], m["kv_rank"], s=0.25)
            mat(p + "mix.uv", H * m["vdim"], m["kv_rank"], s=0.3)
            mat(p + "mix.o", d, H * m["vdim"])
        f = layer["mlp"]
        if f:
            around(p + "norm2", d, 0.0)
            mat(p + "mlp.gate", f["ff"], d, s=2 * std)        # some pairs reach the limit
            mat(p + "mlp.up", f["ff"], d, s=2 * std)
            mat(p + "mlp.down", d, f["ff"])
    return out


def make_folder(tmp, name, tensors_edit=None):
    cfg, seed = CONFIGS[name]
    folder = os.path.join(str(tmp), "dumalix_" + name)
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
# The 16-bit path is measured against what 16-bit storage itself costs in this model: the plain implementation run
# exactly and run again rounding where the 16-bit path stores an activation.  The largest difference of the two over
# a position's logits, its maximum and its mean over the request's positions, is the floor.  No position of the
# engine may be further from the exact logits than twice the floor's maximum, and the positions on average not
# further than one and a half times its mean: the engine rounds at the same places, so it sits at the floor (both
# ratios were between 1.0 and 1.2 whichever kernels ran), while a wrong mechanism (a chunk one token off, a lost
# state, a missing sink) moves most positions by several floors.  The 32-bit path holds every position to FP32_TOL.
BF16_MAX_FLOORS = 2.0
BF16_MEAN_FLOORS = 1.5
BF16_REL_TOL = 2.0 ** -4  # two runs of the 16-bit path against one another, as a part of the largest |logit|


def as_bfloat16(x):
    return x.bfloat16().to(x.dtype)


def check_request(cfg, tensors, tokens, got_rows, dtype, label=""):
    """got_rows: {position: logits row of the engine}.  Every position must be within the rule of the path."""
    ref = DP.forward(cfg, tensors, tokens)
    if dtype == "float32":
        tol = FP32_TOL * max(1.0, float(ref.abs().max()) / 10.0)
    else:
        floor = (DP.forward(cfg, tensors, tokens, store=as_bfloat16) - ref).abs().max(dim=1).values
        # a request of a few positions has a floor of a few samples: never below 2^-5 of the largest |logit|
        tol = max(BF16_MAX_FLOORS * float(floor.max()), 2.0 ** -5 * float(ref.abs().max()))
    worst, total = 0.0, 0.0
    for pos, row in sorted(got_rows.items()):
        diff = float((torch.as_tensor(row).double() - ref[pos]).abs().max())
        worst = max(worst, diff)
        total += diff
        assert diff <= tol, f"{label}: position {pos} (first wrong of the request): |diff| {diff:.3e} > {tol:.3e}"
    if dtype == "bfloat16" and len(got_rows) >= 16:
        mean, most = total / len(got_rows), BF16_MEAN_FLOORS * float(floor.mean())
        assert mean <= most, f"{label}: mean |diff| over the positions {mean:.3e} > {most:.3e}"
    return worst


def run_cuts(engine, tokens, cuts, graphs=False):
    """One request through the engine in steps of the given sizes (the rest one token at a time); returns
    {position: logits} for every position."""
    engine.use_graphs = graphs
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
    return rows
