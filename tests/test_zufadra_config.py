"""The Zufadra design without a GPU: its configuration, its tensor plan, and the plain implementation's own
invariants (what a window sees, the frequency bands, the delta rule's algebra, the convolution, the pair hash)."""
import math

import pytest
import torch

import zufadra_tiny as T
from plain import zufadra_plain as ZP
from transformer_b200.api import _typed
from transformer_b200.config.registry import ConfigError
from transformer_b200.weights.loader import check_rules


def _typed_with_shapes(cfg, tensors):
    arch, meta = _typed(T.file_config(cfg))
    return arch, arch.refine(meta, {k: tuple(v.shape) for k, v in tensors.items()})


@pytest.mark.parametrize("name", sorted(T.CONFIGS))
def test_plan_names_every_tensor_of_a_model_file(name):
    cfg, seed = T.CONFIGS[name]
    tensors = T.random_tensors(cfg, seed)
    arch, meta = _typed_with_shapes(cfg, tensors)
    rules = arch.tensor_plan(meta)
    present = {k: (tuple(v.shape), "BF16") for k, v in tensors.items()}
    chosen = check_rules(rules, present, name)              # raises on missing, unexpected or misshaped tensors
    assert len(chosen) == len(rules)
    spec = arch.build_spec(meta)
    spec.validate()
    assert len(spec.order) == len(cfg["layers"])
    for ls, layer in zip(spec.layers, cfg["layers"]):
        assert ls.arrangement == "sandwich" and ls.mixer_norm.kind == "none"
        assert (ls.feed_forward is None) == (layer["mlp"] is None)
        assert ls.mixer.kind == layer["type"]


def test_configuration_round_trip_and_what_it_reads():
    arch, meta = _typed_with_shapes(T.MIXED, T.random_tensors(T.MIXED, 1))
    again = type(meta).from_dict(meta.to_dict())
    assert again == meta
    a = meta.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.keep_first, a.rot_dims) == (4, 2, 32, 16, 70, 5, 16)
    assert a.softcap == 30.0 and a.scale == 0.2 and a.rot_scaling.as_tuple() == (8.0, 1.0, 4.0, 64.0)
    assert meta.layers[2].mixer.softcap == 0.0 and meta.layers[2].mixer.rot_scaling is None
    assert meta.layers[4].mixer.window == 0                   # no mask: plain causal
    d = meta.layers[0].mixer
    assert (d.conv, d.decay_rank, d.gate_rank) == (3, 8, 12)  # the ranks came from the tensors' shapes
    assert (meta.residual_mult, meta.logit_scale, meta.embedding_scale) == (0.6, 0.3, 3.0)
    assert (meta.bigram.buckets, meta.bigram.mul_prev, meta.bigram.mul_cur) == (37, 31, 7)


def test_what_a_configuration_may_leave_out():
    import copy
    cfg = copy.deepcopy(T.file_config(T.ONLY_ATTENTION))
    mix = cfg["layers"][0]["mixer"]
    heads, dim = mix["heads"], mix["dim"]
    for k in ("kv_heads", "vdim", "scale", "softcap", "mask"):
        mix.pop(k, None)
    mix["rot"]["scaling"] = None
    cfg["embedding"].pop("bigram")
    cfg.pop("residual_mult")
    _, meta = _typed(cfg)
    a = meta.layers[0].mixer
    assert (a.kv_heads, a.vdim, a.scale, a.softcap, a.window, a.keep_first) == (heads, dim, dim ** -0.5, 0.0, 0, 0)
    assert a.rot_scaling is None and meta.bigram is None and meta.residual_mult == 1.0


def test_ranks_must_come_from_somewhere():
    arch, meta = _typed(T.file_config(T.ONLY_DELTA))
    with pytest.raises(ConfigError, match="ranks"):
        arch.tensor_plan(meta)
    cfg = T.file_config(T.ONLY_DELTA)
    cfg["layers"][0]["mixer"].update(decay_rank=6, gate_rank=10)
    arch, meta = _typed(cfg)
    assert len(arch.tensor_plan(meta)) > 5


@pytest.mark.parametrize("edit, what", [
    (lambda c: c["layers"][1]["mixer"].update(heads=5), "share"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=34), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(conv=0), "conv"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][1]["mlp"].update(kind="moe"), "dense"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), "buckets"),
    (lambda c: c.pop("vocab"), "vocab"),
])
def test_faulty_configurations_are_refused(edit, what):
    import copy
    cfg = copy.deepcopy(T.file_config(T.MIXED))
    edit(cfg)
    with pytest.raises(ConfigError, match=what):
        _typed(cfg)


def test_a_window_sees_exactly_its_tokens():
    for window, keep in [(1, 0), (5, 0), (5, 3), (70, 5), (3, 10)]:
        for i in range(0, 90, 7):
            seen = [j for j in range(100) if ZP.visible(i, j, window, keep)]
            want = sorted(set(range(max(0, i - window + 1), i + 1)) | set(range(min(keep, i + 1))))
            assert seen == want, (window, keep, i)


def test_frequency_bands():
    base, dims = 10000.0, 32
    plain = ZP.rotary_frequencies(dims, base, None)
    assert plain[0] == 1.0 and math.isclose(plain[-1], base ** (-(dims - 2) / dims))
    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    scaled = ZP.rotary_frequencies(dims, base, sc)
    bands = set()
    for f, s in zip(plain, scaled):
        wave = 2 * math.pi / f
        if wave < 64 / 4.0:
            assert s == f
            bands.add("kept")
        elif wave > 64 / 1.0:
            assert math.isclose(s, f / 8.0)
            bands.add("divided")
        else:
            assert f / 8.0 <= s <= f
            bands.add("between")
    assert bands == {"kept", "divided", "between"}
    # the rotation keeps lengths and turns pair i by position * f_i
    v = torch.arange(1.0, 9.0, dtype=torch.float64)
    r = ZP.rotate_pairs(v, 3, [0.5, 0.25])
    assert torch.allclose(r[4:], v[4:]) and math.isclose(float(r[:4].norm()), float(v[:4].norm()))
    assert math.isclose(float(r[0]), 1.0 * math.cos(1.5) - 2.0 * math.sin(1.5))


def test_convolution_is_causal_and_its_last_tap_is_the_present():
    g = torch.Generator().manual_seed(0)
    x, taps = torch.randn(9, 5, generator=g, dtype=torch.float64), torch.randn(5, 4, generator=g, dtype=torch.float64)
    y = ZP.causal_conv(x, taps)
    ref = torch.nn.functional.conv1d(torch.nn.functional.pad(x.T[None], (3, 0)), taps[:, None, :], groups=5)[0].T
    assert torch.allclose(y, ref)
    only_now = torch.zeros(5, 4, dtype=torch.float64)
    only_now[:, -1] = 2.0
    assert torch.allclose(ZP.causal_conv(x, only_now), 2.0 * x)


def test_delta_rule_writes_reads_and_forgets():
    """With unit keys, beta = 1 and no decay a written value is read back exactly and a second write to the same key
    replaces it; with a decay the memory fades by the product of the decays."""
    dim, vdim = 6, 4
    e = torch.eye(dim, dtype=torch.float64)
    S = torch.zeros(dim, vdim, dtype=torch.float64)

    def step(S, g, k, v, beta):
        S = g[:, None] * S
        u = beta * (v - S.T @ k)
        return S + torch.outer(k, u)
    v1, v2 = torch.tensor([1.0, 2.0, 3.0, 4.0], dtype=torch.float64), torch.tensor([-1.0, 0.5, 0.0, 2.0], dtype=torch.float64)
    one = torch.ones(dim, dtype=torch.float64)
    S = step(S, one, e[2], v1, 1.0)
    assert torch.allclose(S.T @ e[2], v1)
    S = step(S, one, e[4], v2, 1.0)
    assert torch.allclose(S.T @ e[2], v1) and torch.allclose(S.T @ e[4], v2)
    S = step(S, one, e[2], v2, 1.0)
    assert torch.allclose(S.T @ e[2], v2)
    g = torch.full((dim,), 0.5, dtype=torch.float64)
    S = step(S, g, e[0], torch.zeros(vdim, dtype=torch.float64), 0.0)
    assert torch.allclose(S.T @ e[2], 0.5 * v2)


def test_pair_hash_and_first_token():
    assert ZP.bigram_row(None, 5, 31, 7, 37) == 37
    assert ZP.bigram_row(4, 5, 31, 7, 37) == (4 * 31 + 5 * 7) % 37
    table, pairs = torch.eye(4, dtype=torch.float64), torch.arange(12.0, dtype=torch.float64).view(6, 2).repeat(1, 2)
    x = ZP.embedding(table, pairs, [1, 3, 3], 2.0, {"buckets": 5, "mul_prev": 2, "mul_cur": 1})
    assert torch.allclose(x[0], 2.0 * table[1] + pairs[5])
    assert torch.allclose(x[1], 2.0 * table[3] + pairs[(1 * 2 + 3) % 5])
    assert torch.allclose(x[2], 2.0 * table[3] + pairs[(3 * 2 + 3) % 5])


def test_both_attention_forms_of_the_plain_implementation_agree():
    cfg, seed = T.CONFIGS["mixed"]
    tensors = {k: v.double() for k, v in T.random_tensors(cfg, seed).items()}
    tokens = [int(t) for t in torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(3))]
    a = ZP.forward(T.file_config(cfg), tensors, tokens, fast=True)
    b = ZP.forward(T.file_config(cfg), tensors, tokens, fast=False)
    assert float((a - b).abs().max()) < 1e-9
