"""The Zufadra decoder: layers of two kinds of mixer (grouped-query attention with a sliding window that keeps the
first tokens, capped scores, a norm over the whole query / key projection and an output gate; a gated delta rule
with a decay per key channel), some followed by a dense gated feed-forward with biases, in blocks that read the
residual stream as it is and norm only what their parts produce, times a fixed multiplier.  Token embeddings are
joined by a hashed embedding of the (previous, current) token pair.

Everything particular to the design lives here: how its configuration becomes a :class:`ModelSpec`, and which
file tensors fill which parameters.  Tensor names of a model file (linear weights [out, in]):

    embed [vocab, width]    bigram [buckets + 1, width]    final.norm [width]    head [vocab, width]
    l<i>.norm1, .norm2 [width]         norms of the mixer's and of the feed-forward's output
    attention:      l<i>.mix.q [heads dim, width]  .k [kv_heads dim, width]  .v [kv_heads vdim, width]
                    .q.norm [heads dim]  .k.norm [kv_heads dim]  .g [heads vdim, width]  .o [width, heads vdim]
    channel_delta:  l<i>.mix.q, .k [kv_heads dim, width]  .v [heads vdim, width]  .q.conv, .k.conv, .v.conv [rows, taps]
                    .b [heads, width]  .A_log [heads]  .a1 [r, width]  .a2 [heads dim, r]  .dt_bias [heads dim]
                    .g1 [r', width]  .g2 [heads vdim, r']  .norm [vdim]  .o [width, heads vdim]
    feed-forward:   l<i>.mlp.gate, .up [ff, width]  .gate.b, .up.b [ff]  .down [width, ff]  .down.b [width]
"""
from __future__ import annotations

from typing import List

from ..config.registry import Architecture, ConfigError, register_architecture
from ..config.zufadra import AttentionMeta, ZufadraMeta
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..weights.plan import Source, TensorRule, single


def _ranks(x, where):
    if x.decay_rank is None or x.gate_rank is None:
        raise ConfigError(f"{where}: the ranks of the decay's and the gate's projections are known neither from the "
                          f"configuration (decay_rank, gate_rank) nor from a weight file")
    return x.decay_rank, x.gate_rank


def build_spec(m: ZufadraMeta) -> ModelSpec:
    read = PartSpec.of("none", width=m.width)                                   # the parts read the stream as it is
    post = PartSpec.of("rmsnorm", width=m.width, eps=m.eps, mult=m.residual_mult)
    layers, order = [], []
    for i, layer in enumerate(m.layers):
        x = layer.mixer
        if isinstance(x, AttentionMeta):
            rope = PartSpec.of("rope", dh=x.rot_dims, theta=x.rot_base, pairing="adjacent", positions=m.max_context,
                               scaling=None if x.rot_scaling is None else x.rot_scaling.as_tuple())
            mixer = PartSpec.of("attention", width=m.width, nh=x.heads, nkvh=x.kv_heads, dh=x.dim, dv=x.vdim,
                                scale=x.scale, softcap=x.softcap, window=x.window, keep_first=x.keep_first,
                                qk_norm="whole", eps=m.eps, gate=True, position=rope if x.rot_dims else None)
        else:
            ra, rg = _ranks(x, f"layers[{i}].mixer")
            mixer = PartSpec.of("channel_delta", width=m.width, heads=x.heads, kv_heads=x.kv_heads, dim=x.dim,
                                vdim=x.vdim, taps=x.conv, decay_rank=ra, gate_rank=rg, eps=m.eps)
        order.append(RunEntry(i))
        extra = [("mixer_post_norm", post)]
        ff = None
        if layer.mlp is not None:
            ff = PartSpec.of("swiglu", width=m.width, di=layer.mlp.ff, bias=True)
            extra.append(("feed_forward_post_norm", post))
        layers.append(LayerSpec(mixer=mixer, feed_forward=ff, mixer_norm=read,
                                feed_forward_norm=read if ff is not None else None, arrangement="sandwich",
                                extra=tuple(extra)))
    if m.bigram is not None:
        b = m.bigram
        embedding = PartSpec.of("bigram_lookup", vocab=m.vocab, width=m.width, scale=m.embedding_scale,
                                buckets=b.buckets, mul_prev=b.mul_prev, mul_cur=b.mul_cur)
    else:
        embedding = PartSpec.of("lookup", vocab=m.vocab, width=m.width, scale=m.embedding_scale)
    return ModelSpec(
        width=m.width, vocab=m.vocab, max_context=m.max_context, layers=tuple(layers), order=tuple(order),
        embedding=embedding, final_norm=PartSpec.of("rmsnorm", width=m.width, eps=m.eps),
        head=PartSpec.of("linear", vocab=m.vocab, width=m.width, tied=False, scale=m.logit_scale),
        stop_tokens=tuple(m.eos),
    )


def tensor_plan(m: ZufadraMeta) -> List[TensorRule]:
    d = m.width
    rules = [TensorRule(("embedding", "table"), (m.vocab, d), "matrix", (single("embed", (m.vocab, d)),))]
    if m.bigram is not None:
        n = m.bigram.buckets + 1
        rules.append(TensorRule(("embedding", "pairs"), (n, d), "matrix", (single("bigram", (n, d)),)))
    for i, layer in enumerate(m.layers):
        p, L = f"l{i}.", ("layers", i)
        mx = L + ("mixer",)

        def vec(dest, name, n, init="normal"):
            rules.append(TensorRule(dest, (n,), "norm", (single(p + name, (n,)),), init=init))

        def mat(dest, name, shape):
            rules.append(TensorRule(dest, tuple(shape), "matrix", (single(p + name, shape),)))

        vec(L + ("mixer_post_norm", "weight"), "norm1", d, "ones")
        x = layer.mixer
        if isinstance(x, AttentionMeta):
            hq, hk, hv, ho = x.heads * x.dim, x.kv_heads * x.dim, x.kv_heads * x.vdim, x.heads * x.vdim
            rules.append(TensorRule(mx + ("wqkv",), (hq + hk + hv + ho, d), "matrix", (
                Source((p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g"), ((hq, d), (hk, d), (hv, d), (ho, d)),
                       "cat0"),)))
            vec(mx + ("q_norm",), "mix.q.norm", hq, "ones")
            vec(mx + ("k_norm",), "mix.k.norm", hk, "ones")
            mat(mx + ("wo",), "mix.o", (d, ho))
        else:
            ra, rg = _ranks(x, f"layers[{i}].mixer")
            hk, hv, hd, T = x.kv_heads * x.dim, x.heads * x.vdim, x.heads * x.dim, x.conv
            rules.append(TensorRule(mx + ("win",), (2 * hk + hv + ra + rg, d), "matrix", (
                Source((p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.a1", p + "mix.g1"),
                       ((hk, d), (hk, d), (hv, d), (ra, d), (rg, d)), "cat0"),)))
            rules.append(TensorRule(mx + ("conv",), (2 * hk + hv, T), "norm", (
                Source((p + "mix.q.conv", p + "mix.k.conv", p + "mix.v.conv"), ((hk, T), (hk, T), (hv, T)), "cat0"),)))
            mat(mx + ("wb",), "mix.b", (x.heads, d))
            mat(mx + ("a2",), "mix.a2", (hd, ra))
            mat(mx + ("g2",), "mix.g2", (hv, rg))
            vec(mx + ("dt_bias",), "mix.dt_bias", hd)
            vec(mx + ("A_log",), "mix.A_log", x.heads)
            vec(mx + ("norm",), "mix.norm", x.vdim, "ones")
            mat(mx + ("wo",), "mix.o", (d, hv))
        f = layer.mlp
        if f is None:
            continue
        vec(L + ("feed_forward_post_norm", "weight"), "norm2", d, "ones")
        ff = L + ("feed_forward",)
        rules.append(TensorRule(ff + ("wgu",), (2 * f.ff, d), "matrix", (
            Source((p + "mlp.gate", p + "mlp.up"), ((f.ff, d), (f.ff, d)), "cat0"),)))
        rules.append(TensorRule(ff + ("bgu",), (2 * f.ff,), "norm", (
            Source((p + "mlp.gate.b", p + "mlp.up.b"), ((f.ff,), (f.ff,)), "cat0"),)))
        mat(ff + ("wd",), "mlp.down", (d, f.ff))
        vec(ff + ("bd",), "mlp.down.b", d)
    rules.append(TensorRule(("final_norm", "weight"), (d,), "norm", (single("final.norm", (d,)),), init="ones"))
    rules.append(TensorRule(("head", "weight"), (m.vocab, d), "matrix", (single("head", (m.vocab, d)),)))
    return rules


def refine(m: ZufadraMeta, shapes) -> ZufadraMeta:
    """Sizes that only the weight file gives."""
    return m.with_tensor_shapes(shapes)


ZUFADRA = register_architecture(Architecture(
    name="zufadra",
    config_cls=ZufadraMeta,
    build_spec=build_spec,
    tensor_plan=tensor_plan,
    names=("zufadra", "Zufadra"),
    refine=refine,
))
