"""A plain, slow implementation of the Zufadra decoder: one function per mechanism, whole sequences,
no cache, loops where loops are clearest.  It shares no code with the package under test, reads
``config.json`` and ``model.safetensors`` by itself and works on CPU tensors (float64 by default).

The design in short (n tokens of one sequence, positions 0 .. n-1, width d, m = residual_mult):

    x_0[t] = E[tok_t] * scale + B[(tok_{t-1} * mul_prev + tok_t * mul_cur) mod buckets]     (t = 0: the last row of B)
    every layer:  x <- x + m * N1(mixer(x));  x <- x + m * N2(ff(x))       (a layer may have no ff; no norm on the way in)
    logits = head . Nf(x) * logit_scale
    N(u) = u / sqrt(mean(u^2) + eps) * w

Mixers: grouped-query attention with a norm over the whole query / key projection, a partial rotary
encoding with scaled frequencies, capped scores, a sliding window that keeps the first tokens and a
sigmoid gate on its output ("attention"); and a gated delta rule with a decay per key channel, short
causal convolutions and a low-rank output gate ("channel_delta").  The feed-forward is a dense
silu-gated pair with biases.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, Optional, Sequence

import torch
from safetensors import safe_open

UNIT_EPS = 1e-6        # added under the root when queries and keys of the delta rule are made unit vectors


def read_folder(folder: str, dtype=torch.float64):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            t = f.get_tensor(name)
            tensors[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, tensors


def _keep(x, store):
    """``store``: what a 16-bit path does where it writes an activation to memory (round and come back)."""
    return x if store is None else store(x)


# ----------------------------------------------------------------------------------------------
# small parts
# ----------------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def bigram_row(prev: Optional[int], cur: int, mul_prev: int, mul_cur: int, buckets: int) -> int:
    return buckets if prev is None else (int(prev) * mul_prev + int(cur) * mul_cur) % buckets


def embedding(table, bigram, tokens: Sequence[int], scale: float, rule: Optional[dict]) -> torch.Tensor:
    rows = []
    for t, tok in enumerate(tokens):
        x = table[int(tok)] * scale
        if rule is not None:
            prev = None if t == 0 else tokens[t - 1]
            x = x + bigram[bigram_row(prev, tok, rule["mul_prev"], rule["mul_cur"], rule["buckets"])]
        rows.append(x)
    return torch.stack(rows)


def silu(z):
    return z * torch.sigmoid(z)


# ----------------------------------------------------------------------------------------------
# rotary encoding with scaled frequencies
# ----------------------------------------------------------------------------------------------
def rotary_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """f_i = base^(-2i/dims), i < dims/2; with scaling, long wavelengths are divided by ``factor``, short ones
    kept, and those between blended linearly in original/wavelength."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave < orig / high:
                pass
            elif wave > orig / low:
                f = f / factor
            else:
                s = (orig / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate_pairs(v: torch.Tensor, position: int, freqs) -> torch.Tensor:
    """Entries (2i, 2i+1) of the vector(s) v [..., >= 2 len(freqs)] turn by position * freqs[i]; the rest passes."""
    out = v.clone()
    for i, f in enumerate(freqs):
        ang = position * f
        c, s = math.cos(ang), math.sin(ang)
        a, b = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


# ----------------------------------------------------------------------------------------------
# attention
# ----------------------------------------------------------------------------------------------
def visible(i: int, j: int, window: int, keep_first: int) -> bool:
    return j <= i and (i - j < window or j < keep_first)


def _mask(m: dict, n: int):
    """(window, keep_first); a mixer without a mask sees every earlier token."""
    mask = m.get("mask")
    return (n + 1, 0) if mask is None else (mask["size"], mask.get("keep_first", 0))


def cap_scores(s: torch.Tensor, m: dict) -> torch.Tensor:
    cap = m.get("softcap")
    return s if not cap else float(cap) * torch.tanh(s / float(cap))


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, store=None) -> torch.Tensor:
    n = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot, (window, keep_first) = m["rot"], _mask(m, n)
    freqs = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    q = _keep(h @ w["q"].T, store)
    k = _keep(h @ w["k"].T, store)
    v = _keep(h @ w["v"].T, store)
    gate = _keep(h @ w["g"].T, store)
    q = rms_norm(q, w["q.norm"], eps).view(n, H, dim)
    k = rms_norm(k, w["k.norm"], eps).view(n, G, dim)
    v = v.view(n, G, vdim)
    q = _keep(torch.stack([rotate_pairs(q[t], t, freqs) for t in range(n)]), store)
    k = _keep(torch.stack([rotate_pairs(k[t], t, freqs) for t in range(n)]), store)
    out = torch.zeros(n, H, vdim, dtype=h.dtype)
    for t in range(n):
        js = [j for j in range(t + 1) if visible(t, j, window, keep_first)]
        for hd in range(H):
            g = hd // (H // G)
            s = torch.stack([(q[t, hd] * k[j, g]).sum() for j in js]) * m["scale"]
            p = torch.softmax(cap_scores(s, m), dim=0)
            out[t, hd] = sum(p[a] * v[j, g] for a, j in enumerate(js))
    o = out.reshape(n, H * vdim) * torch.sigmoid(gate)
    return _keep(_keep(o, store) @ w["o"].T, store)


def attention_mixer_fast(h, w, m, eps, store=None):
    """The same as :func:`attention_mixer` with the scores of all pairs at once (for long sequences)."""
    n = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot, (window, keep_first) = m["rot"], _mask(m, n)
    freqs = torch.tensor(rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling")), dtype=torch.float64)
    q = _keep(h @ w["q"].T, store)
    k = _keep(h @ w["k"].T, store)
    v = _keep(h @ w["v"].T, store).view(n, G, vdim)
    gate = _keep(h @ w["g"].T, store)
    q = rms_norm(q, w["q.norm"], eps).view(n, H, dim)
    k = rms_norm(k, w["k.norm"], eps).view(n, G, dim)
    ang = torch.arange(n, dtype=torch.float64)[:, None] * freqs[None, :]
    c, s = torch.cos(ang).to(h.dtype)[:, None, :], torch.sin(ang).to(h.dtype)[:, None, :]

    def turn(x):
        r = rot["dims"]
        a, b = x[..., 0:r:2], x[..., 1:r:2]
        y = x.clone()
        y[..., 0:r:2] = a * c - b * s
        y[..., 1:r:2] = b * c + a * s
        return y
    q, k = _keep(turn(q), store), _keep(turn(k), store)
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    see = (j <= i) & ((i - j < window) | (j < keep_first))
    out = torch.zeros(n, H, vdim, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        sc = (q[:, hd] @ k[:, g].T) * m["scale"]
        sc = cap_scores(sc, m).masked_fill(~see, float("-inf"))
        out[:, hd] = torch.softmax(sc, dim=-1) @ v[:, g]
    o = out.reshape(n, H * vdim) * torch.sigmoid(gate)
    return _keep(_keep(o, store) @ w["o"].T, store)


# ----------------------------------------------------------------------------------------------
# gated delta rule with a decay per key channel
# ----------------------------------------------------------------------------------------------
def causal_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [n, channels], taps [channels, T]: y_t = sum_j taps[:, j] * x_{t - (T - 1 - j)}, zeros before the start."""
    n, T = x.shape[0], taps.shape[1]
    y = torch.zeros_like(x)
    for t in range(n):
        for j in range(T):
            src = t - (T - 1 - j)
            if src >= 0:
                y[t] = y[t] + taps[:, j] * x[src]
    return y


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + UNIT_EPS)


def channel_delta_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, store=None) -> torch.Tensor:
    """Per head, with S [dim, vdim] zero at the start:
        S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t"""
    n = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(_keep(h @ w["q"].T, store), w["q.conv"])).view(n, G, dim)
    k = silu(causal_conv(_keep(h @ w["k"].T, store), w["k.conv"])).view(n, G, dim)
    v = silu(causal_conv(_keep(h @ w["v"].T, store), w["v.conv"])).view(n, H, vdim)
    q = unit(q) * dim ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ w["b"].T)                                       # [n, H]
    a = _keep(h @ w["a1"].T, store) @ w["a2"].T + w["dt_bias"]               # [n, H * dim]
    rate = torch.exp(w["A_log"])                                             # [H]
    g = torch.exp(-rate[None, :, None] * torch.nn.functional.softplus(a.view(n, H, dim)))
    gate = torch.sigmoid(_keep(_keep(h @ w["g1"].T, store) @ w["g2"].T, store)).view(n, H, vdim)
    out = torch.zeros(n, H, vdim, dtype=h.dtype)
    for hd in range(H):
        kv = hd // (H // G)
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        for t in range(n):
            S = g[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            out[t, hd] = S.T @ q[t, kv]
    o = rms_norm(out, w["norm"], eps) * gate
    return _keep(_keep(o.reshape(n, H * vdim), store) @ w["o"].T, store)


# ----------------------------------------------------------------------------------------------
# feed-forward
# ----------------------------------------------------------------------------------------------
def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], store=None) -> torch.Tensor:
    a = silu(_keep(h @ w["gate"].T, store) + w["gate.b"]) * (_keep(h @ w["up"].T, store) + w["up.b"])
    return _keep(_keep(a, store) @ w["down"].T + w["down.b"], store)


# ----------------------------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------------------------
def sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: Sequence[int], store=None, layers_out=None,
            fast: bool = True) -> torch.Tensor:
    """Logits [n, vocab] of one sequence from its first token.  ``layers_out``: a list that receives the stream
    after every layer."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    emb = cfg["embedding"]
    x = embedding(tensors["embed"], tensors.get("bigram"), tokens, emb["scale"], emb.get("bigram"))
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = _keep(x, store)
        if layer["type"] == "attention":
            fn = attention_mixer_fast if fast else attention_mixer
            y = fn(h, sub(tensors, p + "mix."), layer["mixer"], eps, store)
        elif layer["type"] == "channel_delta":
            y = channel_delta_mixer(h, sub(tensors, p + "mix."), layer["mixer"], eps, store)
        else:
            raise ValueError(layer["type"])
        x = x + mult * rms_norm(y, tensors[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            y = dense_ff(_keep(x, store), sub(tensors, p + "mlp."), store)
            x = x + mult * rms_norm(y, tensors[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    xn = _keep(rms_norm(x, tensors["final.norm"], eps), store)
    return (xn @ tensors["head"].T) * cfg["logit_scale"]
