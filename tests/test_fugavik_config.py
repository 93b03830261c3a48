"""The Fugavik design without a GPU: its configuration, model spec and tensor plan, and the plain implementation's
own invariants."""
import copy
import math

import pytest
import torch

import fugavik_tiny as T
from plain import fugavik_plain as FP


def _typed(cfg):
    from transformer_b200.api import _typed
    return _typed(cfg)


def test_configuration_reads_every_size_and_round_trips():
    arch, meta = _typed(T.MIXED)
    assert arch.name == "fugavik"
    assert len(meta.layers) == 7 and meta.eps == 1e-5 and meta.vocab == 101 and meta.width == 64
    a = meta.layers[0].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.rot_dims, a.rot_factor, a.v_mix) == (4, 2, 16, 24, 8, 2.5, False)
    b = meta.layers[4].mixer
    assert b.rot_dims == 0 and b.v_mix and meta.first_v_mix() == 2
    lat = meta.layers[3].mixer
    assert (lat.heads, lat.dim, lat.vdim, lat.kv_rank, lat.scale) == (4, 16, 24, 32, 0.3)
    f = meta.layers[3].mlp
    assert (f.ff, f.experts, f.top) == (16, 3, 3) and meta.layers[2].mlp is None and meta.layers[0].mlp.ff == 40
    d = meta.layers[5].mixer
    assert (d.heads, d.kv_heads, d.dim, d.vdim, d.conv) == (2, 2, 24, 8, 2)
    assert type(meta).from_dict(meta.to_dict()) == meta


def test_model_spec_names_one_source_of_values_and_its_blenders():
    arch, meta = _typed(T.MIXED)
    spec = arch.build_spec(meta)
    spec.validate()
    mixes = [dict(l.mixer.params).get("value_mix") for l in spec.layers if l.mixer.kind == "attention"]
    assert mixes == [None, "source", "blend", "blend"]
    assert all(l.arrangement == "sandwich" and l.mixer_norm.kind == "none" for l in spec.layers)
    assert spec.final_norm.kind == "layernorm" and dict(spec.layers[0].extra)["mixer_post_norm"].kind == "layernorm"
    kinds = [None if l.feed_forward is None else l.feed_forward.kind for l in spec.layers]
    assert kinds == ["mlp", "moe", None, "moe", "mlp", None, "moe"]


@pytest.mark.parametrize("bad", [
    lambda c: c["layers"][0]["mixer"].update(kv_heads=3),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18),
    lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(factor=0.0),
    lambda c: c["layers"][4]["mixer"].update(vdim=16),             # cannot be blended with the source's values
    lambda c: c["layers"][2]["mixer"].update(v_mix="yes"),
    lambda c: c["layers"][3]["mixer"].pop("kv_rank"),
    lambda c: c["layers"][1]["mlp"]["router"].update(top=6),
    lambda c: c["layers"][1].update(type="mlstm"),
    lambda c: c["layers"][0]["mlp"].update(kind="glu"),
    lambda c: c["layers"][5]["mixer"].update(conv=0),
    lambda c: c["norm"].pop("eps"),
])
def test_configuration_errors_are_named(bad):
    from transformer_b200.config.registry import ConfigError
    cfg = copy.deepcopy(T.MIXED)
    bad(cfg)
    with pytest.raises(ConfigError):
        _typed(cfg)


@pytest.mark.parametrize("name", list(T.CONFIGS))
def test_tensor_plan_names_every_tensor_of_a_model_file(name):
    from transformer_b200.weights.loader import check_rules
    cfg, seed = T.CONFIGS[name]
    arch, meta = _typed(cfg)
    tensors = T.random_tensors(cfg, seed)
    present = {n: (tuple(t.shape), "BF16") for n, t in tensors.items()}
    chosen = check_rules(arch.tensor_plan(meta), present, name)
    assert all(v is not None for v in chosen.values())


def test_random_model_folder_has_the_design_s_tensor_names(tmp_path):
    import random
    import transformer_b200 as tb
    from transformer_b200.weights.loader import check_rules, open_tensors
    for cfg in (T.MIXED, T.random_config(random.Random(5), True), T.random_config(random.Random(6), False)):
        folder = tb.write_random_model(str(tmp_path / f"m{cfg['width']}_{cfg['vocab']}"), cfg, seed=1)
        arch, meta = _typed(cfg)
        files = open_tensors(folder)
        present = {n: files.shape_dtype(n) for n in files.names()}
        check_rules(arch.tensor_plan(meta), present, folder)
        read, tensors = FP.read_folder(folder)
        assert _typed(read)[1] == meta
        assert FP.forward(read, tensors, [1, 2, 3]).shape == (3, cfg["vocab"])


def test_a_blending_number_that_nothing_reads_may_be_there_or_not():
    """The first blending layer does not use its number, a layer that does not blend has none: a file may carry
    either all the same; only a later blending layer's number is asked for."""
    from transformer_b200.weights.loader import WeightError, check_rules
    cfg, seed = T.CONFIGS["mixed"]
    arch, meta = _typed(cfg)
    rules = arch.tensor_plan(meta)
    tensors = T.random_tensors(cfg, seed)
    present = {n: (tuple(t.shape), "BF16") for n, t in tensors.items()}
    assert "l2.mix.vmix" in present and "l0.mix.vmix" not in present      # layer 2 is the source, layer 0 does not blend
    check_rules(rules, present, "as written")
    check_rules(rules, dict(present, **{"l0.mix.vmix": ((), "BF16")}), "one more")
    check_rules(rules, {n: v for n, v in present.items() if n != "l2.mix.vmix"}, "one fewer")
    with pytest.raises(WeightError):
        check_rules(rules, {n: v for n, v in present.items() if n != "l4.mix.vmix"}, "a blender without its number")


def test_plain_layer_norm_and_sink_softmax():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(4, 10, generator=g, dtype=torch.float64) * 3 + 1
    w, b = torch.randn(10, generator=g, dtype=torch.float64), torch.randn(10, generator=g, dtype=torch.float64)
    ref = torch.nn.functional.layer_norm(x, (10,), w, b, 1e-3)
    assert float((FP.layer_norm(x, w, b, 1e-3) - ref).abs().max()) < 1e-12
    s = torch.tensor([0.5, -1.0, 2.0], dtype=torch.float64)
    p = FP.sink_softmax(s, 1.0)
    full = torch.softmax(torch.cat([s, torch.tensor([1.0], dtype=torch.float64)]), 0)
    assert float((p - full[:3]).abs().max()) < 1e-12 and float(p.sum()) < 1.0
    assert float(FP.sink_softmax(s, 200.0).sum()) < 1e-80          # a sink far above the scores takes everything
    assert abs(float(FP.sink_softmax(s, -200.0).sum()) - 1.0) < 1e-12


def test_plain_rotation_of_halves():
    f = FP.rotary_frequencies(8, 100.0, {"factor": 4.0})
    assert all(abs(f[i] - 100.0 ** (-2.0 * i / 8) / 4.0) < 1e-15 for i in range(4))
    v = torch.arange(12, dtype=torch.float64)
    r = FP.rotate_halves(v, 3, f)
    assert torch.equal(r[8:], v[8:])                                # what lies behind the rotated entries passes
    for i in range(4):
        a = 3 * f[i]
        assert abs(float(r[i]) - (float(v[i]) * math.cos(a) - float(v[i + 4]) * math.sin(a))) < 1e-12
        assert abs(float(r[i + 4]) - (float(v[i + 4]) * math.cos(a) + float(v[i]) * math.sin(a))) < 1e-12
    # scores depend on the distance alone
    q, k = torch.randn(8, dtype=torch.float64), torch.randn(8, dtype=torch.float64)
    s1 = FP.rotate_halves(q, 9, f) @ FP.rotate_halves(k, 4, f)
    s2 = FP.rotate_halves(q, 25, f) @ FP.rotate_halves(k, 20, f)
    assert abs(float(s1 - s2)) < 1e-12


def test_plain_convolution_is_causal_and_matches_conv1d():
    g = torch.Generator().manual_seed(0)
    u, w = torch.randn(12, 5, generator=g, dtype=torch.float64), torch.randn(5, 4, generator=g, dtype=torch.float64)
    y = FP.causal_conv(u, w)
    ref = torch.nn.functional.conv1d(torch.nn.functional.pad(u.T[None], (3, 0)), w[:, None, :], groups=5)[0].T
    assert float((y - ref).abs().max()) < 1e-12


def test_plain_delta_rule_writes_reads_back_and_fades():
    """One head, no convolution to speak of (one tap of weight one): a value written with beta = 1 under a unit key
    is read back by that key, and fades by the decays of the tokens after it."""
    d, dim, vdim = 6, 4, 3
    m = {"heads": 1, "kv_heads": 1, "dim": dim, "vdim": vdim, "conv": 1}
    z = lambda *s: torch.zeros(*s, dtype=torch.float64)
    w = {"q": z(dim, d), "k": z(dim, d), "v": z(vdim, d), "q.conv": torch.ones(dim, 1, dtype=torch.float64),
         "k.conv": torch.ones(dim, 1, dtype=torch.float64), "v.conv": torch.ones(vdim, 1, dtype=torch.float64),
         "b": z(1, d), "a": z(1, d), "A_log": z(1), "dt_bias": z(1), "g": z(vdim, d), "norm": torch.ones(vdim, dtype=torch.float64),
         "o": torch.eye(vdim, dtype=torch.float64)}
    w["k"][0, 0] = w["q"][0, 0] = 50.0          # input channel 0 makes key and query entry 0
    w["v"][:, 1] = torch.tensor([10.0, 20.0, 30.0], dtype=torch.float64)
    w["b"][0, 2] = 1.0                          # channel 2 sets beta
    w["g"][:, 3] = 1.0                          # channel 3 opens the gate
    h = z(3, d)
    h[0, 0], h[0, 1], h[0, 2] = 1.0, 1.0, 100.0
    h[1, 2] = h[2, 2] = -100.0                  # nothing is written afterwards
    h[2, 0], h[2, 3] = 1.0, 5.0
    out = FP.delta_mixer(h, w, m, 1e-12)
    g = math.exp(-math.log(2.0))                # exp(-exp(0) softplus(0)) per token
    v = torch.nn.functional.silu(torch.tensor([10.0, 20.0, 30.0], dtype=torch.float64)) * g * g * dim ** -0.5
    want = v / torch.sqrt((v * v).mean() + 1e-12) * (5.0 / (1 + math.exp(-5.0)))
    assert float((out[2] - want).abs().max()) < 1e-6


def test_plain_experts_weight_what_they_read():
    cfg, seed = T.CONFIGS["experts"]
    t = {k: v.double() for k, v in T.random_tensors(cfg, seed).items()}
    f = cfg["layers"][0]["mlp"]
    w = FP.sub(t, "l0.mlp.")
    g = torch.Generator().manual_seed(3)
    h = torch.randn(5, cfg["width"], generator=g, dtype=torch.float64)
    experts, weights = FP.router_choice(h, w["router"], f["router"]["top"])
    s = torch.sigmoid(h @ w["router"].T)
    assert torch.equal(experts, torch.topk(s, 2).indices) and float(weights.sum(1).max()) != 1.0
    out = FP.moe_ff(h, w, f)
    want = torch.zeros_like(out)
    for tkn in range(5):
        for e, a in zip(experts[tkn].tolist(), weights[tkn]):
            x = a * h[tkn]
            want[tkn] += (FP.silu(x @ w[f"e{e}.gate"].T) * (x @ w[f"e{e}.up"].T)) @ w[f"e{e}.down"].T
    assert float((out - want).abs().max()) < 1e-12
    # not the same as weighting what the expert returns
    other = torch.zeros_like(out)
    for tkn in range(5):
        for e, a in zip(experts[tkn].tolist(), weights[tkn]):
            other[tkn] += a * ((FP.silu(h[tkn] @ w[f"e{e}.gate"].T) * (h[tkn] @ w[f"e{e}.up"].T)) @ w[f"e{e}.down"].T)
    assert float((out - other).abs().max()) > 1e-3


def test_plain_later_tokens_do_not_change_earlier_logits():
    cfg, seed = T.CONFIGS["mixed"]
    t = {k: v.double() for k, v in T.random_tensors(cfg, seed).items()}
    a = FP.forward(cfg, t, [5, 9, 33, 2, 71, 8, 8, 40])
    b = FP.forward(cfg, t, [5, 9, 33, 2, 71, 1, 2, 3])
    assert float((a[:5] - b[:5]).abs().max()) < 1e-12 and float((a[5:] - b[5:]).abs().max()) > 1e-3


def test_mechanisms_left_out_would_show():
    """The test weights are made so that every mechanism matters: the plain implementation with one of them switched
    off moves the logits far beyond the tolerances above."""
    cfg, seed = T.CONFIGS["mixed"]
    tensors = {k: v.double() for k, v in T.random_tensors(cfg, seed).items()}
    tokens = torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(3)).tolist()
    ref = FP.forward(cfg, tensors, tokens)
    rule = T.BF16_MEAN_TOL * float(ref.abs().max())      # what the mean over a request's positions is held to

    def moved(edit):
        t = dict(tensors)
        edit(t)
        return float((FP.forward(cfg, t, tokens) - ref).abs().max(dim=1).values.mean())

    def every(suffix, value):
        def edit(t):
            for k in t:
                if k.endswith(suffix):
                    t[k] = torch.full_like(t[k], value)
        return edit
    assert moved(every("mix.sink", -100.0)) > 2 * rule              # no sink
    assert moved(every("mix.vmix", 0.0)) > 2 * rule                 # values not blended
    assert moved(every(".ls1", 1.0)) > 2 * rule                     # no layer scale
    assert moved(every("norm1.b", 0.0)) > 2 * rule                  # no bias in the norm
    assert moved(every("l3.mix.g", 0.0)) > 2 * rule                 # every head's gate at one half
    assert moved(every("mix.dt_bias", 10.0)) > 2 * rule             # a delta rule that forgets at once
