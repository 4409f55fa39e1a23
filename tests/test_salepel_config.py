"""The Salepel configuration, its tensor plan and the plain implementation's own invariants (no GPU)."""
import copy

import pytest
import torch

import salepel_tiny as T
from plain import salepel_plain as SP
from transformer_b200.architectures import salepel as arch
from transformer_b200.config.registry import ConfigError, architecture_for
from transformer_b200.config.salepel import LatentMeta, MlstmMeta, SalepelMeta


def test_the_registry_finds_the_design_by_its_name():
    a = architecture_for(T.MIXED)
    assert a.name == "salepel"
    meta = a.config_cls.from_dict(T.MIXED)
    assert isinstance(meta.layers[0].mixer, LatentMeta) and isinstance(meta.layers[1].mixer, MlstmMeta)
    assert meta.layers[2].mlp is None and meta.layers[2].mixer.kv_from == 0
    assert meta.embedding_scale == 3.0 and meta.eps == 1e-5
    assert SalepelMeta.from_dict(meta.to_dict()) == meta


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "earlier"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "no latent"),
    (lambda c: c["layers"][5]["mixer"].update(kv_from=2), "no latent"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=16), "differ"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "positive"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][1].update(type="conv"), "type"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][1]["mixer"].pop("gate_cap"), "gate_cap"),
])
def test_bad_configurations_are_refused_by_name(edit, word):
    cfg = copy.deepcopy(T.MIXED)
    edit(cfg)
    with pytest.raises(ConfigError, match=word):
        SalepelMeta.from_dict(cfg)


def test_the_plan_names_every_tensor_of_a_file_once():
    meta = SalepelMeta.from_dict(T.MIXED)
    names = [n for rule in arch.tensor_plan(meta) for n in rule.canonical.names]
    assert sorted(names) == sorted(T.random_tensors(T.MIXED, 0))
    spec = arch.build_spec(meta)
    spec.validate()
    assert [e.cache_of for e in spec.order] == [None, None, 0, None, None, 4]
    assert spec.layers[2].feed_forward is None and spec.layers[0].arrangement == "sandwich"


def _double(tensors):
    return {k: v.double() for k, v in tensors.items()}


def test_plain_window_sees_exactly_its_tokens():
    """Changing a token just outside the window leaves a position's mixer output alone; just inside changes it."""
    cfg = T.ONLY_LATENT
    m = cfg["layers"][0]["mixer"]
    w = SP.sub(_double(T.random_tensors(cfg, 7)), "l0.mix.")
    g = torch.Generator().manual_seed(0)
    h = torch.randn(12, cfg["width"], generator=g, dtype=torch.float64)
    base = SP.latent_attention_mixer(h, w, m, 1e-6, SP.latent_of(h, w, m, 1e-6))
    W, t = m["mask"]["size"], 10
    for j, seen in ((t - W, False), (t - W + 1, True)):
        h2 = h.clone()
        h2[j] += 1.0
        out = SP.latent_attention_mixer(h2, w, m, 1e-6, SP.latent_of(h2, w, m, 1e-6))
        assert (float((out[t] - base[t]).abs().max()) > 1e-9) == seen


def test_plain_matrix_memory_equals_its_closed_form():
    """The recurrence with its running maximum equals the unstabilized sums it stands for."""
    cfg = T.ONLY_MEMORY
    m = cfg["layers"][0]["mixer"]
    w = SP.sub(_double(T.random_tensors(cfg, 3)), "l0.mix.")
    g = torch.Generator().manual_seed(1)
    h = torch.randn(9, cfg["width"], generator=g, dtype=torch.float64)
    got = SP.mlstm_mixer(h, w, m, 1e-6)
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    n = h.shape[0]
    q = (h @ w["q"].T).view(n, H, dk) * dk ** -0.5
    k, v = (h @ w["k"].T).view(n, H, dk), (h @ w["v"].T).view(n, H, dv)
    ig = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    F = torch.cumsum(fg, 0)
    o = torch.zeros(n, H, dv, dtype=torch.float64)
    for a in range(H):
        for t in range(n):
            logw = F[t, a] - F[:t + 1, a] + ig[:t + 1, a]               # weight of token j in the state at t
            mt = max(float(F[t, a]), float(logw.max()))                   # the running maximum, started at zero
            wts = torch.exp(logw - mt)
            num = (wts * (k[:t + 1, a] @ q[t, a])) @ v[:t + 1, a]
            den = max(abs(float(wts @ (k[:t + 1, a] @ q[t, a]))), float(torch.exp(torch.tensor(-mt)))) + 1e-6
            o[t, a] = num / den
    o = SP.rms_norm(o, None, 1e-6).reshape(n, H * dv) * w["norm"]
    want = (o * torch.sigmoid(h @ w["g"].T)) @ w["o"].T
    assert float((got - want).abs().max()) < 1e-9


def test_plain_router_rules():
    w = {"router": torch.eye(4, dtype=torch.float64), "correction": torch.tensor([0.0, 0.0, 0.9, 0.0], dtype=torch.float64)}
    h = torch.tensor([[2.0, 1.0, 0.0, 0.5]], dtype=torch.float64)
    idx, wt, s = SP.route(h, w, 2)
    assert idx.tolist() == [[2, 0]]                         # the correction moves the choice ...
    assert torch.allclose(wt, s[0, [2, 0]][None])           # ... but not the weights, which are not renormalized
    assert float(wt.sum()) < 1.0
    f = {"router": {"experts": 2, "identity": 2, "top": 2}, "expert": {"ff": 3, "limit": 1.0}}
    w.update({f"e{e}.{n}": torch.zeros(3 if n != "down" else 4, 4 if n != "down" else 3, dtype=torch.float64)
              for e in range(2) for n in ("gate", "up", "down")})
    out = SP.moe(h, w, f)                                   # expert 2 hands h through, expert 0 gives zero
    assert torch.allclose(out, s[0, 2] * h)
