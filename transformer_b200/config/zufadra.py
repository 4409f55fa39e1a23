"""Typed configuration of the Zufadra decoder.

``config.json`` of this design is nested; every size and every constant that may differ between models is
read from it (or, for the two low ranks of the delta-rule mixer, from the shapes of the model's tensors):

    architecture: "Zufadra"     vocab, width     norm: {eps}     residual_mult     logit_scale
    embedding: {scale, bigram: {buckets, mul_prev, mul_cur}}          (no "bigram": a plain scaled lookup)
    layers: [ {type, mixer: {...}, mlp: {kind: "dense", ff} | null}, ... ]
      type "attention":     mixer {heads, kv_heads, dim, vdim, scale, softcap, mask: {size, keep_first},
                                   rot: {base, dims, scaling: {factor, low, high, original}}}
                            (softcap absent or 0: none; mask absent: plain causal; rot.scaling absent: none)
      type "channel_delta": mixer {heads, kv_heads, dim, vdim, conv}    (+ decay_rank, gate_rank when no weight
                            file is at hand to read them from: random models)
    max_context (optional): the longest sequence, default 32768.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, replace
from typing import Any, Mapping, Optional, Tuple

from .registry import ConfigError
from .salepel import _num, _sub

DEFAULT_CONTEXT = 32768


@dataclass(frozen=True)
class RotScaling:
    factor: float
    low: float
    high: float
    original: float

    def as_tuple(self):
        return (self.factor, self.low, self.high, self.original)


@dataclass(frozen=True)
class AttentionMeta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float          # 0: the scores are not capped
    window: int             # 0: every earlier token is visible
    keep_first: int
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[RotScaling] = None

    @classmethod
    def from_dict(cls, m, where):
        rot = _sub(m, "rot", where)
        mask = m.get("mask")
        if mask is not None and not isinstance(mask, Mapping):
            raise ConfigError(f"{where}.mask must be an object")
        window = keep = 0
        if mask is not None:
            window = _num(mask, "size", where + ".mask")
            keep = _num({"keep_first": mask.get("keep_first", 0)}, "keep_first", where + ".mask")
        sc = rot.get("scaling")
        scaling = None
        if sc is not None:
            w = where + ".rot.scaling"
            scaling = RotScaling(_num(sc, "factor", w, float), _num(sc, "low", w, float), _num(sc, "high", w, float),
                                 _num(sc, "original", w, float))
        cap = m.get("softcap")
        heads, dim = _num(m, "heads", where), _num(m, "dim", where)
        # what a file may leave out: key heads (as many as query heads), the value size (the key's), the multiplier
        m = dict(m, kv_heads=m.get("kv_heads", heads), vdim=m.get("vdim", dim), scale=m.get("scale", dim ** -0.5))
        return cls(heads, _num(m, "kv_heads", where), dim, _num(m, "vdim", where),
                   _num(m, "scale", where, float), 0.0 if cap is None else _num(m, "softcap", where, float),
                   window, keep, _num(rot, "base", where + ".rot", float), _num(rot, "dims", where + ".rot"), scaling)

    def to_dict(self):
        rot = {"base": self.rot_base, "dims": self.rot_dims}
        if self.rot_scaling is not None:
            s = self.rot_scaling
            rot["scaling"] = {"factor": s.factor, "low": s.low, "high": s.high, "original": s.original}
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
               "rot": rot}
        if self.softcap:
            out["softcap"] = self.softcap
        if self.window:
            out["mask"] = {"size": self.window, "keep_first": self.keep_first}
        return out


@dataclass(frozen=True)
class DeltaMeta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: Optional[int] = None     # rows of the decay's first projection; from the tensors when a file is read
    gate_rank: Optional[int] = None      # rows of the output gate's first projection

    @classmethod
    def from_dict(cls, m, where):
        opt = lambda k: None if m.get(k) is None else _num(m, k, where)
        heads, dim = _num(m, "heads", where), _num(m, "dim", where)
        m = dict(m, kv_heads=m.get("kv_heads", heads), vdim=m.get("vdim", dim))
        return cls(heads, _num(m, "kv_heads", where), dim, _num(m, "vdim", where),
                   _num(m, "conv", where), opt("decay_rank"), opt("gate_rank"))

    def to_dict(self):
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}
        if self.decay_rank is not None:
            out["decay_rank"] = self.decay_rank
        if self.gate_rank is not None:
            out["gate_rank"] = self.gate_rank
        return out


@dataclass(frozen=True)
class DenseMeta:
    ff: int

    @classmethod
    def from_dict(cls, m, where):
        if m.get("kind") != "dense":
            raise ConfigError(f"{where}.kind must be 'dense', got {m.get('kind')!r}")
        return cls(_num(m, "ff", where))

    def to_dict(self):
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class BigramMeta:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class ZufadraLayer:
    type: str                     # "attention" | "channel_delta"
    mixer: Any                    # AttentionMeta | DeltaMeta
    mlp: Optional[DenseMeta]


_MIXERS = {"attention": AttentionMeta, "channel_delta": DeltaMeta}


@dataclass(frozen=True)
class ZufadraMeta:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    logit_scale: float
    embedding_scale: float
    bigram: Optional[BigramMeta]
    layers: Tuple[ZufadraLayer, ...]
    max_context: int = DEFAULT_CONTEXT
    eos: tuple = ()

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "ZufadraMeta":
        layers_in = cfg.get("layers")
        if not isinstance(layers_in, (list, tuple)) or not layers_in:
            raise ConfigError("config.json lacks the list 'layers'")
        layers = []
        for i, entry in enumerate(layers_in):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping):
                raise ConfigError(f"{where} must be an object")
            kind = entry.get("type")
            if kind not in _MIXERS:
                raise ConfigError(f"{where}.type must be one of {sorted(_MIXERS)}, got {kind!r}")
            mixer = _MIXERS[kind].from_dict(_sub(entry, "mixer", where), where + ".mixer")
            mlp = entry.get("mlp")
            if mlp is not None and not isinstance(mlp, Mapping):
                raise ConfigError(f"{where}.mlp must be an object or null")
            layers.append(ZufadraLayer(kind, mixer, None if mlp is None else DenseMeta.from_dict(mlp, where + ".mlp")))
        eos = cfg.get("eos_token_id", ())
        if isinstance(eos, bool) or not isinstance(eos, (int, list, tuple)):
            raise ConfigError(f"eos_token_id must be an integer or a list of integers, got {eos!r}")
        eos = (eos,) if isinstance(eos, int) else tuple(int(e) for e in eos)
        emb = cfg.get("embedding") or {}
        bg = emb.get("bigram")
        bigram = None
        if bg is not None:
            w = "embedding.bigram"
            bigram = BigramMeta(_num(bg, "buckets", w), _num(bg, "mul_prev", w), _num(bg, "mul_cur", w))
        meta = cls(_num(cfg, "vocab", "config"), _num(cfg, "width", "config"),
                   _num(_sub(cfg, "norm", "config"), "eps", "norm", float),
                   _num({"residual_mult": cfg.get("residual_mult", 1.0)}, "residual_mult", "config", float),
                   _num({"logit_scale": cfg.get("logit_scale", 1.0)}, "logit_scale", "config", float),
                   _num({"scale": emb.get("scale", 1.0)}, "scale", "embedding", float), bigram, tuple(layers),
                   _num({"max_context": cfg.get("max_context", DEFAULT_CONTEXT)}, "max_context", "config"), eos)
        meta.validate()
        return meta

    @classmethod
    def from_folder(cls, folder: str) -> "ZufadraMeta":
        with open(os.path.join(folder, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def with_tensor_shapes(self, shapes: Mapping[str, Tuple[int, ...]]) -> "ZufadraMeta":
        """The sizes that only the model's tensors give (the delta-rule mixers' two low ranks), filled in from
        ``shapes`` (file tensor name -> shape) where the configuration left them open."""
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if isinstance(m, DeltaMeta):
                a1, g1 = shapes.get(f"l{i}.mix.a1"), shapes.get(f"l{i}.mix.g1")
                if m.decay_rank is None and a1 is not None and len(a1) == 2:
                    m = replace(m, decay_rank=int(a1[0]))
                if m.gate_rank is None and g1 is not None and len(g1) == 2:
                    m = replace(m, gate_rank=int(g1[0]))
                layer = replace(layer, mixer=m)
            layers.append(layer)
        return replace(self, layers=tuple(layers))

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or self.max_context <= 0:
            raise ConfigError("vocab, width and max_context must be positive")
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.eps}")
        if self.bigram is not None:
            b = self.bigram
            if b.buckets <= 0 or b.mul_prev < 0 or b.mul_cur < 0:
                raise ConfigError("embedding.bigram: buckets must be positive, the multipliers not negative")
            if (self.vocab - 1) * (b.mul_prev + b.mul_cur) >= 2 ** 62:
                raise ConfigError("embedding.bigram: the multipliers are too large for this vocabulary")
        for i, layer in enumerate(self.layers):
            m, where = layer.mixer, f"layers[{i}].mixer"
            for n in ("heads", "kv_heads", "dim", "vdim"):
                if getattr(m, n) <= 0:
                    raise ConfigError(f"{where}.{n} must be positive, got {getattr(m, n)}")
            if m.heads % m.kv_heads:
                raise ConfigError(f"{where}: {m.heads} heads cannot share {m.kv_heads} key heads")
            if isinstance(m, AttentionMeta):
                if m.rot_dims < 0 or m.rot_dims > m.dim or m.rot_dims % 2:
                    raise ConfigError(f"{where}.rot.dims must be even and at most dim ({m.rot_dims}, {m.dim})")
                if not m.rot_base > 0:
                    raise ConfigError(f"{where}.rot.base must be positive, got {m.rot_base}")
                if m.window < 0 or m.keep_first < 0 or m.softcap < 0:
                    raise ConfigError(f"{where}: mask.size, mask.keep_first and softcap must not be negative")
                s = m.rot_scaling
                if s is not None and (not s.factor > 0 or not s.original > 0 or not s.low > 0 or not s.high > s.low):
                    raise ConfigError(f"{where}.rot.scaling: factor, original and low must be positive, high above low")
            else:
                if m.conv < 1:
                    raise ConfigError(f"{where}.conv must be at least 1, got {m.conv}")
                for n in ("decay_rank", "gate_rank"):
                    if getattr(m, n) is not None and getattr(m, n) <= 0:
                        raise ConfigError(f"{where}.{n} must be positive, got {getattr(m, n)}")
            if layer.mlp is not None and layer.mlp.ff <= 0:
                raise ConfigError(f"layers[{i}].mlp.ff must be positive")
        for e in self.eos:
            if not (0 <= e < self.vocab):
                raise ConfigError(f"eos token {e} lies outside the vocabulary of {self.vocab}")

    def to_dict(self) -> dict:
        emb: dict = {"scale": self.embedding_scale}
        if self.bigram is not None:
            emb["bigram"] = {"buckets": self.bigram.buckets, "mul_prev": self.bigram.mul_prev,
                             "mul_cur": self.bigram.mul_cur}
        out = {"architecture": "Zufadra", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "residual_mult": self.residual_mult, "logit_scale": self.logit_scale, "embedding": emb,
               "max_context": self.max_context,
               "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                          for l in self.layers]}
        if self.eos:
            out["eos_token_id"] = list(self.eos)
        return out
