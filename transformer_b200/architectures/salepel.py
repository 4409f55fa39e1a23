"""The Salepel decoder: layers of two kinds of mixer (attention through a cached latent with a sliding window;
a matrix memory with exponential gates), each followed by a mixture of experts, in blocks that norm their
parts' outputs as well as their inputs.

Everything particular to the design lives here: how its configuration becomes a :class:`ModelSpec`, and which
file tensors fill which parameters.  Tensor names of a model file (linear weights [out, in]):

    embed [vocab, width]      final.norm [width]      head [vocab, width]
    l<i>.norm1, .norm1b, .norm2, .norm2b [width]      norms before / after the mixer, before / after the feed-forward
    latent attention:  l<i>.mix.dq [q_rank, width]  .dq.norm [q_rank]  .uq [heads (dim + rot_dim), q_rank]
                       .dkv [kv_rank + rot_dim, width]  .dkv.norm [kv_rank]      (absent with kv_from)
                       .uk [heads dim, kv_rank]  .uv [heads vdim, kv_rank]  .o [width, heads vdim]
    matrix memory:     l<i>.mix.q, .k [heads dim, width]  .v, .g [heads vdim, width]  .o [width, heads vdim]
                       .norm [heads vdim]  .i, .f [heads, width]  .i.b, .f.b [heads]
    experts:           l<i>.mlp.router [experts + identity, width]  .correction [experts + identity]
                       l<i>.mlp.e<j>.gate, .up [ff, width]  .down [width, ff]
"""
from __future__ import annotations

from typing import List

from ..config.registry import Architecture, register_architecture
from ..config.salepel import LatentMeta, SalepelMeta
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..weights.plan import Source, TensorRule, single

GLU_ALPHA = 1.702      # the experts' gate: g * sigmoid(GLU_ALPHA g)


def build_spec(m: SalepelMeta) -> ModelSpec:
    norm = PartSpec.of("rmsnorm", width=m.width, eps=m.eps)
    layers, order = [], []
    for i, layer in enumerate(m.layers):
        x = layer.mixer
        if isinstance(x, LatentMeta):
            rope = PartSpec.of("rope", dh=x.rot_dims, theta=x.rot_base, pairing="half", positions=m.max_context)
            mixer = PartSpec.of("latent_attention", width=m.width, heads=x.heads, dim=x.dim, rot_dim=x.rot_dim,
                                vdim=x.vdim, kv_rank=x.kv_rank, q_rank=x.q_rank, window=x.window, scale=x.scale,
                                eps=m.eps, own_latent=x.kv_from is None, position=rope)
            order.append(RunEntry(i, cache_of=x.kv_from))
        else:
            mixer = PartSpec.of("mlstm", width=m.width, heads=x.heads, dim=x.dim, vdim=x.vdim, gate_cap=x.gate_cap,
                                eps=m.eps)
            order.append(RunEntry(i))
        extra = [("mixer_post_norm", norm)]
        ff = None
        if layer.mlp is not None:
            f = layer.mlp
            ff = PartSpec.of("moe", width=m.width, di=f.ff, nexp=f.experts, nexp_use=f.top, identity=f.identity,
                             scoring="all", correction=True, glu_alpha=GLU_ALPHA, glu_limit=f.limit)
            extra.append(("feed_forward_post_norm", norm))
        layers.append(LayerSpec(mixer=mixer, feed_forward=ff, mixer_norm=norm,
                                feed_forward_norm=norm if ff is not None else None, arrangement="sandwich",
                                extra=tuple(extra)))
    return ModelSpec(
        width=m.width, vocab=m.vocab, max_context=m.max_context, layers=tuple(layers), order=tuple(order),
        embedding=PartSpec.of("lookup", vocab=m.vocab, width=m.width, scale=m.embedding_scale),
        final_norm=norm, head=PartSpec.of("linear", vocab=m.vocab, width=m.width, tied=False),
        stop_tokens=tuple(m.eos),
    )


def tensor_plan(m: SalepelMeta) -> List[TensorRule]:
    d = m.width
    rules = [TensorRule(("embedding", "table"), (m.vocab, d), "matrix", (single("embed", (m.vocab, d)),))]
    for i, layer in enumerate(m.layers):
        p, L = f"l{i}.", ("layers", i)

        def norm(part, name):
            rules.append(TensorRule(L + (part, "weight"), (d,), "norm", (single(p + name, (d,)),), init="ones"))

        norm("mixer_norm", "norm1")
        norm("mixer_post_norm", "norm1b")
        x, mx = layer.mixer, L + ("mixer",)
        if isinstance(x, LatentMeta):
            hq, r = x.heads * (x.dim + x.rot_dim), x.kv_rank
            if x.kv_from is None:
                rules.append(TensorRule(mx + ("wdown",), (x.q_rank + r + x.rot_dim, d), "matrix", (
                    Source((p + "mix.dq", p + "mix.dkv"), ((x.q_rank, d), (r + x.rot_dim, d)), "cat0"),)))
                rules.append(TensorRule(mx + ("c_norm",), (r,), "norm", (single(p + "mix.dkv.norm", (r,)),),
                                        init="ones"))
            else:
                rules.append(TensorRule(mx + ("wdown",), (x.q_rank, d), "matrix", (single(p + "mix.dq", (x.q_rank, d)),)))
            rules.append(TensorRule(mx + ("q_norm",), (x.q_rank,), "norm", (single(p + "mix.dq.norm", (x.q_rank,)),),
                                    init="ones"))
            rules.append(TensorRule(mx + ("uq",), (hq, x.q_rank), "matrix", (single(p + "mix.uq", (hq, x.q_rank)),)))
            rules.append(TensorRule(mx + ("uk",), (x.heads * x.dim, r), "matrix",
                                    (single(p + "mix.uk", (x.heads * x.dim, r)),)))
            rules.append(TensorRule(mx + ("uv",), (x.heads * x.vdim, r), "matrix",
                                    (single(p + "mix.uv", (x.heads * x.vdim, r)),)))
            rules.append(TensorRule(mx + ("wo",), (d, x.heads * x.vdim), "matrix",
                                    (single(p + "mix.o", (d, x.heads * x.vdim)),)))
        else:
            hk, hv, H = x.heads * x.dim, x.heads * x.vdim, x.heads
            rules.append(TensorRule(mx + ("wqkvg",), (2 * hk + 2 * hv, d), "matrix", (
                Source((p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g"), ((hk, d), (hk, d), (hv, d), (hv, d)),
                       "cat0"),)))
            rules.append(TensorRule(mx + ("wif",), (2 * H, d), "matrix", (
                Source((p + "mix.i", p + "mix.f"), ((H, d), (H, d)), "cat0"),)))
            rules.append(TensorRule(mx + ("bif",), (2 * H,), "norm", (
                Source((p + "mix.i.b", p + "mix.f.b"), ((H,), (H,)), "cat0"),)))
            rules.append(TensorRule(mx + ("norm",), (hv,), "norm", (single(p + "mix.norm", (hv,)),), init="ones"))
            rules.append(TensorRule(mx + ("wo",), (d, hv), "matrix", (single(p + "mix.o", (d, hv)),)))
        f = layer.mlp
        if f is None:
            continue
        norm("feed_forward_norm", "norm2")
        norm("feed_forward_post_norm", "norm2b")
        ff, R, E = L + ("feed_forward",), f.experts + f.identity, f.experts
        rules.append(TensorRule(ff + ("router",), (R, d), "matrix", (single(p + "mlp.router", (R, d)),)))
        rules.append(TensorRule(ff + ("correction",), (R,), "norm", (single(p + "mlp.correction", (R,)),)))
        rules.append(TensorRule(ff + ("wgu",), (E, 2 * f.ff, d), "matrix", (
            Source(tuple(p + f"mlp.e{e}.{which}" for e in range(E) for which in ("gate", "up")),
                   ((f.ff, d),) * (2 * E), "stack0_of_row_pairs"),)))
        rules.append(TensorRule(ff + ("wd",), (E, d, f.ff), "matrix", (
            Source(tuple(p + f"mlp.e{e}.down" for e in range(E)), ((d, f.ff),) * E, "stack0"),)))
    rules.append(TensorRule(("final_norm", "weight"), (d,), "norm", (single("final.norm", (d,)),), init="ones"))
    rules.append(TensorRule(("head", "weight"), (m.vocab, d), "matrix", (single("head", (m.vocab, d)),)))
    return rules


SALEPEL = register_architecture(Architecture(
    name="salepel",
    config_cls=SalepelMeta,
    build_spec=build_spec,
    tensor_plan=tensor_plan,
    names=("salepel", "Salepel"),
))
