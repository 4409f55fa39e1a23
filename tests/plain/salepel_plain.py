"""A plain, slow implementation of the Salepel decoder: one function per mechanism, whole sequences,
no cache, loops where loops are clearest.  It shares no code with the package under test, reads
``config.json`` and ``model.safetensors`` by itself and works on CPU tensors (float64 by default).

The design in short (n tokens of one sequence, positions 0 .. n-1, width d):

    x_0 = E[token] * embedding.scale
    every layer:  x <- x + N1b(mixer(N1(x)));  x <- x + N2b(ff(N2(x)))      (a layer may have no ff)
    logits = head . Nf(x)
    N(x) = x / sqrt(mean(x^2) + eps) * w

Mixers: a matrix memory with exponential gates ("mlstm"), and attention through a low-rank latent
with a sliding window and a shared rotated key part ("latent_attention"), which may read the latent
that an earlier layer cached instead of making one.  The feed-forward is a mixture of experts whose
router takes a softmax over all outputs, chooses with a correction added, weighs without it, and
counts a few outputs as experts that hand their input through.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch
from safetensors import safe_open

GLU_ALPHA = 1.702      # the experts' gate is g * sigmoid(GLU_ALPHA * g)
DENOM_FLOOR = 1e-6     # added to the matrix memory's denominator


def read_folder(folder: str, dtype=torch.float64):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            t = f.get_tensor(name)
            tensors[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, tensors


# ----------------------------------------------------------------------------------------------
# small parts
# ----------------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) [* w], over the last axis."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def embedding(table: torch.Tensor, tokens: Sequence[int], scale: float) -> torch.Tensor:
    return torch.stack([table[int(t)] for t in tokens]) * scale


def rotate_halves(v: torch.Tensor, position: int, base: float, dims: int) -> torch.Tensor:
    """Rotate the first ``dims`` entries of the vector(s) v [..., >= dims]: entry i pairs with entry
    i + dims/2, angle = position * base^(-2i/dims); the rest passes."""
    out = v.clone()
    half = dims // 2
    for i in range(half):
        ang = position * base ** (-2.0 * i / dims)
        c, s = math.cos(ang), math.sin(ang)
        a, b = v[..., i], v[..., i + half]
        out[..., i] = a * c - b * s
        out[..., i + half] = b * c + a * s
    return out


# ----------------------------------------------------------------------------------------------
# matrix memory with exponential gates
# ----------------------------------------------------------------------------------------------
def soft_cap(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def mlstm_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, store=None) -> torch.Tensor:
    """h [n, d] -> [n, d].  Per head, with S [dim, vdim], n [dim], m scalar, all zero at the start:

        i_t = cap(Wi h + bi),  f_t = logsigmoid(cap(Wf h + bf))
        m_t = max(f_t + m_{t-1}, i_t)
        S_t = e^{f_t + m_{t-1} - m_t} S_{t-1} + e^{i_t - m_t} k_t v_t^T        (n_t alike with k_t alone)
        o_t = S_t^T q_t / (max(|n_t . q_t|, e^{-m_t}) + DENOM_FLOOR),  q scaled by dim^-1/2

    then each head's o is divided by its root mean square, all heads times ``norm``, times
    sigmoid(Wg h), then Wo.  ``store`` rounds the projections as a 16-bit path would store them."""
    st = store or (lambda z: z)
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    n = h.shape[0]
    q = st(h @ w["q"].T).view(n, H, dk) * dk ** -0.5
    k = st(h @ w["k"].T).view(n, H, dk)
    v = st(h @ w["v"].T).view(n, H, dv)
    gate = torch.sigmoid(st(h @ w["g"].T))
    ig = soft_cap(h @ w["i"].T + w["i.b"], cap)                                     # [n, H]
    fg = torch.nn.functional.logsigmoid(soft_cap(h @ w["f"].T + w["f.b"], cap))
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    for a in range(H):
        S = torch.zeros(dk, dv, dtype=h.dtype)
        nn = torch.zeros(dk, dtype=h.dtype)
        mm = torch.zeros((), dtype=h.dtype)
        for t in range(n):
            m_new = torch.maximum(fg[t, a] + mm, ig[t, a])
            keep, take = torch.exp(fg[t, a] + mm - m_new), torch.exp(ig[t, a] - m_new)
            S = keep * S + take * torch.outer(k[t, a], v[t, a])
            nn = keep * nn + take * k[t, a]
            mm = m_new
            den = torch.maximum((nn @ q[t, a]).abs(), torch.exp(-mm)) + DENOM_FLOOR
            out[t, a] = (S.T @ q[t, a]) / den
    out = rms_norm(out, None, eps).reshape(n, H * dv) * w["norm"]
    return st(out * gate) @ w["o"].T


# ----------------------------------------------------------------------------------------------
# attention through a latent
# ----------------------------------------------------------------------------------------------
def latent_of(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, store=None):
    """What a layer keeps of every token: the normed latent c [n, kv_rank] and the rotated shared key part
    [n, rot_dim]."""
    st = store or (lambda z: z)
    r, rd = m["kv_rank"], m["rot_dim"]
    rot = m["rot"]
    kv = h @ w["dkv"].T                                    # [n, kv_rank + rot_dim]
    c = st(rms_norm(kv[:, :r], w["dkv.norm"], eps))
    kr = torch.stack([rotate_halves(kv[t, r:], t, rot["base"], rot["dims"]) for t in range(h.shape[0])])
    return c, st(kr)


def latent_attention_mixer(h, w, m: dict, eps: float, latent, store=None) -> torch.Tensor:
    """h [n, d] -> [n, d] with ``latent`` = (c, rotated key part) of this layer or of the layer it reads.

        q = Wuq N(Wdq h) per head [dim plain | rot_dim rotated];   k_plain = Wuk c,  v = Wuv c  per head
        score(t, j) = (q_plain . k_plain_j + q_rot . k_rot_j) * scale,  j visible iff 0 <= t - j < window
        out = Wo concat_heads(softmax(score) v)
    """
    st = store or (lambda z: z)
    H, dk, rd, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    window, scale, rot = m["mask"]["size"], m["scale"], m["rot"]
    n = h.shape[0]
    c, kr = latent
    cq = st(rms_norm(h @ w["dq"].T, w["dq.norm"], eps))
    q = st(cq @ w["uq"].T).view(n, H, dk + rd)
    kp = (c @ w["uk"].T).view(n, H, dk)
    v = (c @ w["uv"].T).view(n, H, dv)
    o = torch.zeros(n, H, dv, dtype=h.dtype)
    for t in range(n):
        lo = max(0, t - window + 1)
        for a in range(H):
            qr = rotate_halves(q[t, a, dk:], t, rot["base"], rot["dims"])
            s = (kp[lo:t + 1, a] @ q[t, a, :dk] + kr[lo:t + 1] @ qr) * scale
            o[t, a] = torch.softmax(s, dim=0) @ v[lo:t + 1, a]
    return st(o.reshape(n, H * dv)) @ w["o"].T


# ----------------------------------------------------------------------------------------------
# mixture of experts
# ----------------------------------------------------------------------------------------------
def route(h: torch.Tensor, w: Dict[str, torch.Tensor], top: int):
    """Scores s = softmax(Wr h) over all outputs; the ``top`` largest of s + correction are chosen (ties to the
    lower index); the weights are their s, as they are.  Returns (index [n, top], weight [n, top], s)."""
    s = torch.softmax(h @ w["router"].T, dim=-1)
    choice = s + w["correction"]
    idx = torch.zeros(h.shape[0], top, dtype=torch.long)
    for t in range(h.shape[0]):
        order = sorted(range(choice.shape[1]), key=lambda e: (-float(choice[t, e]), e))
        idx[t] = torch.tensor(order[:top])
    return idx, torch.gather(s, 1, idx), s


def expert(h: torch.Tensor, gate_w, up_w, down_w, limit: float, store=None) -> torch.Tensor:
    st = store or (lambda z: z)
    g = torch.clamp(h @ gate_w.T, max=limit)
    u = torch.clamp(h @ up_w.T, min=-limit, max=limit)
    return st(g * torch.sigmoid(GLU_ALPHA * g) * (u + 1.0)) @ down_w.T


def moe(h: torch.Tensor, w: Dict[str, torch.Tensor], f: dict, store=None, forced=None, margins_out=None) -> torch.Tensor:
    """h [n, d] -> [n, d].  Outputs E .. E + identity - 1 of the router stand for experts whose output is h.
    ``forced`` [n, top]: the experts to use instead of the free choice; ``margins_out`` then receives, per token,
    (free choice, gap between the last chosen and the first left-out choice score)."""
    st = store or (lambda z: z)
    E, ident, top = f["router"]["experts"], f["router"].get("identity", 0), f["router"]["top"]
    limit = float(f["expert"]["limit"])
    idx, wt, s = route(h, w, top)
    if margins_out is not None:
        choice = torch.sort(s + w["correction"], dim=-1, descending=True).values
        gaps = choice[:, top - 1] - choice[:, top] if choice.shape[1] > top else torch.full((h.shape[0],), 1e9)
        margins_out.append([(sorted(int(e) for e in idx[t]), float(gaps[t])) for t in range(h.shape[0])])
    if forced is not None:
        idx = forced
        wt = torch.gather(s, 1, idx)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            if e >= E:
                y = h[t]
            else:
                y = st(expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], limit, store)[0])
            out[t] += wt[t, j] * y
    return out


# ----------------------------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------------------------
def sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: Sequence[int], store=None, layers_out=None,
            routes=None, margins_out=None) -> torch.Tensor:
    """Logits [n, vocab] of one whole sequence.  ``layers_out``: a list that receives the stream after every
    layer; ``routes``: {layer: index [n, top]} forces the experts' choice; ``margins_out``: a dict that receives
    {layer: [(free choice, gap) per token]}."""
    eps = cfg["norm"]["eps"]
    x = embedding(tensors["embed"], tokens, cfg["embedding"]["scale"])
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = rms_norm(x, tensors[p + "norm1"], eps)
        h = store(h) if store else h
        wm = sub(tensors, p + "mix.")
        if layer["type"] == "mlstm":
            y = mlstm_mixer(h, wm, m, eps, store)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_of(h, wm, m, eps, store)
                src = i
            y = latent_attention_mixer(h, wm, m, eps, latents[src], store)
        else:
            raise ValueError(layer["type"])
        y = store(y) if store else y
        x = x + rms_norm(y, tensors[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = rms_norm(x, tensors[p + "norm2"], eps)
            h = store(h) if store else h
            margins = None
            if margins_out is not None:
                margins = []
            y = moe(h, sub(tensors, p + "mlp."), layer["mlp"], store, None if routes is None else routes.get(i),
                    margins)
            if margins_out is not None:
                margins_out[i] = margins[0]
            x = x + rms_norm(y, tensors[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    xn = rms_norm(x, tensors["final.norm"], eps)
    xn = store(xn) if store else xn
    return xn @ tensors["head"].T


def greedy_generate(cfg, tensors, prompt: Sequence[int], steps: int) -> List[int]:
    toks = list(prompt)
    out = []
    for _ in range(steps):
        nxt = int(torch.argmax(forward(cfg, tensors, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
