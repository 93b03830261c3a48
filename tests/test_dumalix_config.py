"""The Dumalix design without a GPU: its configuration, run order and tensor plan, and the plain implementation's
own invariants."""
import math

import pytest
import torch

import dumalix_tiny as T
from plain import dumalix_plain as DP


def _typed(cfg):
    from transformer_b200.api import _typed
    return _typed(cfg)


def test_configuration_reads_every_size_and_round_trips():
    arch, meta = _typed(T.MIXED)
    assert arch.name == "dumalix"
    assert meta.canon_taps == 4 and meta.loop.times == 2 and len(meta.layers) == 4
    a = meta.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.conv, a.chunk, a.rot_dims) == (4, 2, 16, 24, 3, 40, 8)
    assert a.rot_ramp.as_tuple() == (8.0, 32.0, 4.0, 0.5)
    assert meta.layers[2].mlp is None and meta.layers[2].mixer.chunk == 0
    again = type(meta).from_dict(meta.to_dict())
    assert again == meta


def test_run_order_repeats_the_group_with_a_joint_before_every_pass():
    arch, meta = _typed(T.MIXED)
    assert meta.run_order() == [(0, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    spec = arch.build_spec(meta)
    spec.validate()
    assert [(e.layer, e.joint) for e in spec.order] == [(0, None), (1, 0), (2, None), (1, 0), (2, None), (3, None)]
    assert meta.run_order() == DP.run_order(T.MIXED)
    _, odd = _typed(T.ODD)
    assert [i for i, _ in odd.run_order()] == [0, 1, 0, 1, 0, 1, 2]
    _, flat = _typed(T.ONLY_LATENT)
    assert flat.run_order() == [(0, False)] and not arch.build_spec(flat).joints


@pytest.mark.parametrize("bad", [
    lambda c: c["layers"][1]["mixer"].update(kv_heads=3),
    lambda c: c["layers"][1]["mixer"].update(vdim=23),
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18),
    lambda c: c["loop"].update(stop=9),
    lambda c: c["layers"][0].update(type="mlstm"),
    lambda c: c["layers"][0]["mlp"].update(kind="moe"),
    lambda c: c["norm"].pop("eps"),
])
def test_configuration_errors_are_named(bad):
    import copy
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


def test_plain_convolution_is_causal_and_matches_conv1d():
    g = torch.Generator().manual_seed(0)
    u, w = torch.randn(12, 5, generator=g, dtype=torch.float64), torch.randn(5, 4, generator=g, dtype=torch.float64)
    y = DP.causal_conv(u, w)
    ref = torch.nn.functional.conv1d(torch.nn.functional.pad(u.T[None], (3, 0)), w[:, None, :], groups=5)[0].T
    assert float((y - ref).abs().max()) < 1e-12
    u2 = u.clone()
    u2[7:] += 1.0
    assert torch.equal(DP.causal_conv(u2, w)[:7], y[:7])


def test_plain_frequency_ramp():
    f, mult = DP.rescaled_frequencies(16, 10000.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0})
    plain, one = DP.rescaled_frequencies(16, 10000.0, None)
    assert one == 1.0 and abs(mult - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    lo = max(math.floor(16 * math.log(64 / (2 * math.pi * 8.0)) / (2 * math.log(10000.0))), 0)
    hi = min(math.ceil(16 * math.log(64 / (2 * math.pi * 1.0)) / (2 * math.log(10000.0))), 15)
    assert all(abs(f[i] - plain[i]) < 1e-15 for i in range(lo + 1))                   # fast turns are kept
    assert all(abs(f[i] - plain[i] / 4.0) < 1e-15 for i in range(hi, 8))              # slow ones divided
    assert any(plain[i] / 4.0 < f[i] < plain[i] for i in range(8)) or hi - lo <= 1


def test_plain_chunks_and_sink():
    assert DP.chunk_visible(40, 40, 40) and not DP.chunk_visible(40, 39, 40) and DP.chunk_visible(79, 40, 40)
    assert not DP.chunk_visible(3, 4, None) and DP.chunk_visible(500, 0, None)
    # a rotation turned back is the identity; rotated values summed and turned back are a rotation by the distance
    g = torch.Generator().manual_seed(1)
    x = torch.randn(6, 2, 8, generator=g, dtype=torch.float64)
    f, _ = DP.rescaled_frequencies(8, 100.0, None)
    pos = torch.arange(6)
    assert float((DP.rotate_adjacent(DP.rotate_adjacent(x, pos, f), pos, f, sign=-1.0) - x).abs().max()) < 1e-12


def test_latent_attention_equals_attention_with_keys_and_values_per_head():
    """The latent form against explicit per-head keys and values, which the plain implementation builds."""
    cfg, seed = T.CONFIGS["latent"]
    t = {k: v.double() for k, v in T.random_tensors(cfg, seed).items()}
    m = cfg["layers"][0]["mixer"]
    g = torch.Generator().manual_seed(2)
    h = torch.randn(9, cfg["width"], generator=g, dtype=torch.float64)
    out = DP.latent_attention(h, t, "l0.mix.", m, 1e-6)
    # a later token does not change an earlier output
    h2 = h.clone()
    h2[5:] += 1.0
    assert float((DP.latent_attention(h2, t, "l0.mix.", m, 1e-6)[:5] - out[:5]).abs().max()) < 1e-12
