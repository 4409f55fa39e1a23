"""Typed configuration of the Salepel decoder.

``config.json`` of this design is nested; every size and every constant that may differ between models is
read from it, nothing stands in code:

    architecture: "Salepel"        vocab, width        norm: {eps}        embedding: {scale}
    layers: [ {type, mixer: {...}, mlp: {...} | null}, ... ]
      type "latent_attention": mixer {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, mask: {size},
                                      rot: {base, dims}, kv_from (optional: the layer whose cached latent it reads)}
      type "mlstm":            mixer {heads, dim, vdim, gate_cap}
      mlp: {kind: "moe", router: {experts, identity, top}, expert: {ff, limit}}
    max_context (optional): the longest sequence, default 32768.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .registry import ConfigError

DEFAULT_CONTEXT = 32768


def _num(d: Mapping[str, Any], key: str, where: str, cast=int):
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise ConfigError(f"config.json lacks {where}.{key}")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{where}.{key} must be a number, got {v!r}")
    if cast is int and int(v) != v:
        raise ConfigError(f"{where}.{key} must be an integer, got {v!r}")
    return cast(v)


def _sub(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key) if isinstance(d, Mapping) else None
    if not isinstance(v, Mapping):
        raise ConfigError(f"config.json lacks the section {where}.{key}")
    return v


@dataclass(frozen=True)
class LatentMeta:
    heads: int
    dim: int            # unrotated query/key entries per head
    rot_dim: int        # rotated entries per head (the key's are shared by all heads)
    vdim: int
    kv_rank: int
    q_rank: int
    window: int
    scale: float
    rot_base: float
    rot_dims: int       # how many of the rotated part's entries rotate (the rest pass)
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, m, where):
        rot, mask = _sub(m, "rot", where), _sub(m, "mask", where)
        kv_from = m.get("kv_from")
        if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int)):
            raise ConfigError(f"{where}.kv_from must be a layer index, got {kv_from!r}")
        return cls(_num(m, "heads", where), _num(m, "dim", where), _num(m, "rot_dim", where), _num(m, "vdim", where),
                   _num(m, "kv_rank", where), _num(m, "q_rank", where), _num(mask, "size", where + ".mask"),
                   _num(m, "scale", where, float), _num(rot, "base", where + ".rot", float),
                   _num(rot, "dims", where + ".rot"), kv_from)

    def to_dict(self):
        out = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
               "kv_rank": self.kv_rank, "q_rank": self.q_rank, "scale": self.scale, "mask": {"size": self.window},
               "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class MlstmMeta:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, m, where):
        return cls(_num(m, "heads", where), _num(m, "dim", where), _num(m, "vdim", where),
                   _num(m, "gate_cap", where, float))

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}


@dataclass(frozen=True)
class MoeMeta:
    experts: int
    identity: int
    top: int
    ff: int
    limit: float

    @classmethod
    def from_dict(cls, m, where):
        if m.get("kind") != "moe":
            raise ConfigError(f"{where}.kind must be 'moe', got {m.get('kind')!r}")
        r, e = _sub(m, "router", where), _sub(m, "expert", where)
        identity = r.get("identity", 0)
        return cls(_num(r, "experts", where + ".router"), _num({"identity": identity}, "identity", where + ".router"),
                   _num(r, "top", where + ".router"), _num(e, "ff", where + ".expert"),
                   _num(e, "limit", where + ".expert", float))

    def to_dict(self):
        return {"kind": "moe", "router": {"experts": self.experts, "identity": self.identity, "top": self.top},
                "expert": {"ff": self.ff, "limit": self.limit}}


@dataclass(frozen=True)
class SalepelLayer:
    type: str                     # "latent_attention" | "mlstm"
    mixer: Any                    # LatentMeta | MlstmMeta
    mlp: Optional[MoeMeta]


_MIXERS = {"latent_attention": LatentMeta, "mlstm": MlstmMeta}


@dataclass(frozen=True)
class SalepelMeta:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: Tuple[SalepelLayer, ...]
    max_context: int = DEFAULT_CONTEXT
    eos: tuple = ()

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "SalepelMeta":
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
            layers.append(SalepelLayer(kind, mixer, None if mlp is None else MoeMeta.from_dict(mlp, where + ".mlp")))
        eos = cfg.get("eos_token_id", ())
        if isinstance(eos, bool) or not isinstance(eos, (int, list, tuple)):
            raise ConfigError(f"eos_token_id must be an integer or a list of integers, got {eos!r}")
        eos = (eos,) if isinstance(eos, int) else tuple(int(e) for e in eos)
        emb = cfg.get("embedding") or {}
        meta = cls(_num(cfg, "vocab", "config"), _num(cfg, "width", "config"),
                   _num(_sub(cfg, "norm", "config"), "eps", "norm", float),
                   _num({"scale": emb.get("scale", 1.0)}, "scale", "embedding", float), tuple(layers),
                   _num({"max_context": cfg.get("max_context", DEFAULT_CONTEXT)}, "max_context", "config"), eos)
        meta.validate()
        return meta

    @classmethod
    def from_folder(cls, folder: str) -> "SalepelMeta":
        with open(os.path.join(folder, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or self.max_context <= 0:
            raise ConfigError("vocab, width and max_context must be positive")
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.eps}")
        for i, layer in enumerate(self.layers):
            m, where = layer.mixer, f"layers[{i}].mixer"
            if isinstance(m, LatentMeta):
                for n in ("heads", "dim", "vdim", "kv_rank", "q_rank", "window"):
                    if getattr(m, n) <= 0:
                        raise ConfigError(f"{where}.{n} must be positive, got {getattr(m, n)}")
                if m.rot_dim < 0 or m.rot_dims < 0 or m.rot_dims > m.rot_dim or m.rot_dims % 2:
                    raise ConfigError(f"{where}: rot.dims must be even and at most rot_dim ({m.rot_dims}, {m.rot_dim})")
                if not m.rot_base > 0:
                    raise ConfigError(f"{where}.rot.base must be positive, got {m.rot_base}")
                if m.kv_from is not None:
                    if not (0 <= m.kv_from < i):
                        raise ConfigError(f"{where}.kv_from = {m.kv_from} must name an earlier layer")
                    src = self.layers[m.kv_from].mixer
                    if not isinstance(src, LatentMeta) or src.kv_from is not None:
                        raise ConfigError(f"{where}.kv_from = {m.kv_from}: that layer makes no latent of its own")
                    if (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) != (m.kv_rank, m.rot_dim, m.rot_base,
                                                                                 m.rot_dims):
                        raise ConfigError(f"{where}.kv_from = {m.kv_from}: the two layers' latents differ in size or "
                                          f"rotation")
            else:
                for n in ("heads", "dim", "vdim"):
                    if getattr(m, n) <= 0:
                        raise ConfigError(f"{where}.{n} must be positive, got {getattr(m, n)}")
                if not m.gate_cap > 0:
                    raise ConfigError(f"{where}.gate_cap must be positive, got {m.gate_cap}")
            f = layer.mlp
            if f is not None:
                if f.experts <= 0 or f.identity < 0 or f.ff <= 0 or not f.limit > 0:
                    raise ConfigError(f"layers[{i}].mlp: experts and ff must be positive, identity not negative, "
                                      f"limit positive")
                if not (0 < f.top <= f.experts + f.identity):
                    raise ConfigError(f"layers[{i}].mlp.router.top = {f.top} must lie in 1..{f.experts + f.identity}")
        for e in self.eos:
            if not (0 <= e < self.vocab):
                raise ConfigError(f"eos token {e} lies outside the vocabulary of {self.vocab}")

    def to_dict(self) -> dict:
        out = {"architecture": "Salepel", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "embedding": {"scale": self.embedding_scale}, "max_context": self.max_context,
               "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                          for l in self.layers]}
        if self.eos:
            out["eos_token_id"] = list(self.eos)
        return out
