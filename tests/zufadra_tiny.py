"""Small Zufadra configurations, random model folders in the design's own tensor names, and the comparison of the
engine with the plain implementation (tests/plain/zufadra_plain.py)."""
import json
import os

import torch
from safetensors.torch import save_file

from plain import zufadra_plain as ZP


def attention(heads, kv_heads, dim, vdim, window=None, keep_first=0, dims=None, base=10000.0, scaling=None,
              scale=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "rot": {"base": base, "dims": dim if dims is None else dims}, "scale": dim ** -0.5 if scale is None else scale}
    if window is not None:
        m["mask"] = {"size": window, "keep_first": keep_first}
    if scaling is not None:
        m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    if softcap is not None:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m}


def delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank):
    # the two ranks are sizes of tensors only; they ride along here for the writer of the random tensors
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                               "conv": conv}, "ranks": (decay_rank, gate_rank)}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(vocab, width, layers, eps=1e-6, scale=1.0, mult=1.0, logit_scale=1.0, bigram=None):
    emb = {"scale": scale}
    if bigram is not None:
        emb["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))
    return {"architecture": "Zufadra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "logit_scale": logit_scale, "embedding": emb, "max_context": 1024,
            "layers": [dict(l[0], mlp=l[1]) for l in layers]}


# Sizes differ from one another wherever the design lets them: query and key heads, the two head sizes, groups of
# one and of several, windows shorter than a page and across page borders, kept first tokens or none, no window at
# all, a rotation of a part of the head, of all of it and of nothing, scaled frequencies with all three bands in
# use, capped and uncapped scores, one to five taps, layers with and without a feed-forward.
MIXED = config(101, 64, [
    (delta(4, 2, 16, 24, 3, 8, 12), None),
    (attention(4, 2, 32, 16, window=70, keep_first=5, dims=16, scaling=(8.0, 1.0, 4.0, 64), scale=0.2, softcap=30.0),
     dense(48)),
    (attention(3, 3, 16, 16, window=5), None),
    (delta(2, 2, 24, 8, 2, 4, 4), dense(40)),
    (attention(2, 1, 48, 80, dims=0, softcap=8.0), dense(24)),
], eps=1e-5, scale=3.0, mult=0.6, logit_scale=0.3, bigram=(37, 31, 7))
ONLY_ATTENTION = config(64, 48, [(attention(4, 2, 16, 32, window=6, keep_first=2, dims=8, softcap=20.0), None)],
                        scale=2.0, mult=0.8, bigram=(11, 3, 5))
ONLY_DELTA = config(64, 48, [(delta(4, 2, 12, 20, 4, 6, 10), None)], scale=2.0, mult=0.8)
ONLY_DENSE = config(64, 48, [(delta(1, 1, 8, 8, 2, 4, 4), dense(56))], scale=2.0, logit_scale=0.5, bigram=(64, 1, 1))
# head sizes the tensor-core kernels take, windows across several pages
WIDE = config(128, 128, [
    (attention(4, 2, 64, 64, window=100, keep_first=10, dims=32, scaling=(3.0, 1.0, 8.0, 256), softcap=40.0), dense(96)),
    (delta(2, 1, 64, 64, 4, 16, 16), None),
    (attention(8, 2, 128, 128, window=64, keep_first=64, dims=64, base=5e5), dense(96)),
    (attention(2, 2, 64, 128, window=129, keep_first=1, dims=64), None),
    (delta(2, 2, 128, 128, 4, 16, 16), None),
], scale=4.0, mult=0.9, logit_scale=0.75, bigram=(251, 61, 13))
# sizes that are multiples of nothing: every vectorized or tensor-core form refuses them
ODD = config(77, 50, [
    (attention(3, 1, 10, 6, window=1, keep_first=3, dims=6, softcap=3.0), dense(22)),
    (delta(3, 3, 10, 7, 1, 3, 5), None),
    (delta(6, 2, 36, 33, 5, 5, 3), dense(30)),
    (attention(5, 5, 12, 20, window=200, keep_first=0, dims=12, scaling=(2.0, 0.5, 2.0, 16)), None),
], eps=1e-4, scale=0.5, mult=1.3, logit_scale=2.0, bigram=(5, 1, 0))
CONFIGS = {"mixed": (MIXED, 1), "attention": (ONLY_ATTENTION, 2), "delta": (ONLY_DELTA, 3), "dense": (ONLY_DENSE, 4),
           "wide": (WIDE, 5), "odd": (ODD, 6)}
STD = {"wide": 0.08}


def file_config(cfg):
    """What goes into config.json: without the ranks, which only the tensors carry."""
    out = dict(cfg)
    out["layers"] = [{k: v for k, v in l.items() if k != "ranks"} for l in cfg["layers"]]
    return out


def random_tensors(cfg, seed, std=0.15):
    """Every tensor of a model file, by the design's names; norms around one, biases and decays not trivial."""
    g = torch.Generator().manual_seed(seed)
    d = cfg["width"]
    out = {}

    def mat(name, *shape, s=std):
        out[name] = (torch.randn(*shape, generator=g) * s).bfloat16()

    def around_one(name, n):
        out[name] = (1.0 + 0.3 * torch.randn(n, generator=g)).bfloat16()

    mat("embed", cfg["vocab"], d, s=1.0)
    bg = cfg["embedding"].get("bigram")
    if bg:
        mat("bigram", bg["buckets"] + 1, d, s=2.0)
    mat("head", cfg["vocab"], d)
    around_one("final.norm", d)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        around_one(p + "norm1", d)
        H, G = m["heads"], m["kv_heads"]
        if layer["type"] == "attention":
            mat(p + "mix.q", H * m["dim"], d, s=2 * std)
            mat(p + "mix.k", G * m["dim"], d, s=2 * std)
            mat(p + "mix.v", G * m["vdim"], d)
            mat(p + "mix.g", H * m["vdim"], d, s=3 * std)
            around_one(p + "mix.q.norm", H * m["dim"])
            around_one(p + "mix.k.norm", G * m["dim"])
            out[p + "mix.q.norm"] = (out[p + "mix.q.norm"].float() * 2.0).bfloat16()     # scores that matter
            mat(p + "mix.o", d, H * m["vdim"])
        else:
            ra, rg = layer["ranks"]
            hk, hv, T = G * m["dim"], H * m["vdim"], m["conv"]
            for n, rows in (("q", hk), ("k", hk), ("v", hv)):
                mat(p + "mix." + n, rows, d, s=2 * std)
                mat(p + f"mix.{n}.conv", rows, T, s=0.6)
            mat(p + "mix.b", H, d, s=3 * std)
            out[p + "mix.A_log"] = (torch.rand(H, generator=g) * 3.0 - 2.5).bfloat16()
            mat(p + "mix.a1", ra, d, s=2 * std)
            mat(p + "mix.a2", H * m["dim"], ra, s=0.5)
            out[p + "mix.dt_bias"] = (torch.randn(H * m["dim"], generator=g) - 1.0).bfloat16()
            mat(p + "mix.g1", rg, d, s=2 * std)
            mat(p + "mix.g2", hv, rg, s=0.5)
            around_one(p + "mix.norm", m["vdim"])
            mat(p + "mix.o", d, hv)
        f = layer["mlp"]
        if f:
            around_one(p + "norm2", d)
            mat(p + "mlp.gate", f["ff"], d)
            mat(p + "mlp.up", f["ff"], d)
            mat(p + "mlp.down", d, f["ff"])
            mat(p + "mlp.gate.b", f["ff"], s=0.5)
            mat(p + "mlp.up.b", f["ff"], s=0.5)
            mat(p + "mlp.down.b", d, s=0.5)
    return out


def make_folder(tmp, name, tensors_edit=None):
    cfg, seed = CONFIGS[name]
    folder = os.path.join(str(tmp), "zufadra_" + name)
    if not os.path.isdir(folder):
        os.makedirs(folder)
        tensors = random_tensors(cfg, seed, STD.get(name, 0.15))
        if tensors_edit:
            tensors_edit(tensors)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(file_config(cfg), f)
        save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return folder


FP32_TOL = 2e-4           # on logits of order one to ten
# of the largest |logit| of the request, against the plain implementation rounding where the 16-bit path stores an
# activation.  Every part's output is normed before it joins the stream, which carries the rounding of a small
# output over at full size; a wrong mechanism (a window one token off, a lost state, a missing gate) moves the
# logits by a tenth of their size or more.
BF16_REL_TOL = 2.0 ** -5


def as_bfloat16(x):
    return x.bfloat16().to(x.dtype)


def check_request(cfg, tensors, tokens, got_rows, dtype, label=""):
    """got_rows: {position: logits row of the engine}.  Every position must be within the rule of the path."""
    ref = ZP.forward(cfg, tensors, tokens, store=as_bfloat16 if dtype == "bfloat16" else None)
    tol = FP32_TOL * max(1.0, float(ref.abs().max()) / 10.0) if dtype == "float32" else BF16_REL_TOL * float(ref.abs().max())
    worst = 0.0
    for pos, row in sorted(got_rows.items()):
        diff = float((torch.as_tensor(row).double() - ref[pos]).abs().max())
        worst = max(worst, diff)
        assert diff <= tol, f"{label}: position {pos} (first wrong of the request): |diff| {diff:.3e} > {tol:.3e}"
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
