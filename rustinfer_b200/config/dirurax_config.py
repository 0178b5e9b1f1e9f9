"""Typed configuration of the Dirurax decoder, read from config.json's own keys.

config.json names the width, the vocabulary, the norms' eps and a list of layers; every layer
names its mixer (`type`), the mixer's sizes and constants (`mixer`) and its feed-forward (`mlp`,
null for none).  Each kind of mixer and feed-forward has a record of its own here, so a size or a
constant that config.json gives is a field that code reads; an unknown mixer type or feed-forward kind
is an error, a key the engine does not know is named in a warning.  The rank of a mixer's low-rank decay projection is not in
config.json: it is the shape of the tensors (`rank` may be given for random-weights models).
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from .model_config import ConfigError, _eos_ids, _need


def _only(d: Mapping[str, Any], known, where: str) -> None:
    """Keys the engine does not know are named in a warning: they may be notes of whoever wrote the file,
    and they may be constants of a variant this engine does not compute."""
    extra = sorted(set(d) - set(known))
    if extra:
        warnings.warn(f"config.json: {where} has keys the engine does not know and does not use: {extra}")


def _rank(d: Mapping[str, Any]) -> Optional[int]:
    return int(d["rank"]) if d.get("rank") else None


@dataclass(frozen=True)
class GlaMixerConfig:
    """Gated linear attention: `heads` heads with keys of `dim` and values of `vdim`; the decay is
    sigmoid(.)^(1/tau)."""
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "GlaMixerConfig":
        _only(d, ("heads", "dim", "vdim", "tau", "rank"), "a gla mixer")
        c = cls(_need(d, "heads"), _need(d, "dim"), _need(d, "vdim"), _need(d, "tau", float), _rank(d))
        if min(c.heads, c.dim, c.vdim) <= 0 or not c.tau > 0:
            raise ConfigError("config.json: a gla mixer needs positive heads, dim, vdim and tau")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.rank:
            d["rank"] = self.rank
        return d


@dataclass(frozen=True)
class BlockAttentionConfig:
    """Softmax attention without rotation whose queries see only the keys of their own block of
    `mask_size` positions; q and k normed per head, values of unit root mean square."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    mask_size: int

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BlockAttentionConfig":
        _only(d, ("heads", "kv_heads", "dim", "vdim", "scale", "mask"), "an attention mixer")
        mask = d.get("mask")
        if not isinstance(mask, Mapping):
            raise ConfigError("config.json: an attention mixer needs 'mask': {'size': n}")
        _only(mask, ("size",), "an attention mask")
        c = cls(_need(d, "heads"), _need(d, "kv_heads"), _need(d, "dim"), _need(d, "vdim"),
                _need(d, "scale", float), _need(mask, "size"))
        if min(c.heads, c.kv_heads, c.dim, c.vdim, c.mask_size) <= 0 or c.heads % c.kv_heads:
            raise ConfigError("config.json: an attention mixer needs positive sizes and heads a multiple of kv_heads")
        return c

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                "scale": self.scale, "mask": {"size": self.mask_size}}


@dataclass(frozen=True)
class DeltaMixerConfig:
    """Delta rule with a per-channel decay: `heads` heads of `dim` (keys and values alike)."""
    heads: int
    dim: int
    rank: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "DeltaMixerConfig":
        _only(d, ("heads", "dim", "rank"), "a delta-rule mixer")
        c = cls(_need(d, "heads"), _need(d, "dim"), _rank(d))
        if min(c.heads, c.dim) <= 0:
            raise ConfigError("config.json: a delta-rule mixer needs positive heads and dim")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "dim": self.dim}
        if self.rank:
            d["rank"] = self.rank
        return d


@dataclass(frozen=True)
class ParallelMixerConfig:
    """Attention (`left`) beside a delta rule (`right`), summed with the two scales."""
    left: BlockAttentionConfig
    right: DeltaMixerConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ParallelMixerConfig":
        _only(d, ("left", "right", "left_scale", "right_scale"), "a parallel mixer")
        for side in ("left", "right"):
            if not isinstance(d.get(side), Mapping):
                raise ConfigError(f"config.json: a parallel mixer needs '{side}'")
        return cls(BlockAttentionConfig.from_dict(d["left"]), DeltaMixerConfig.from_dict(d["right"]),
                   _need(d, "left_scale", float), _need(d, "right_scale", float))

    def to_dict(self) -> Dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict(),
                "left_scale": self.left_scale, "right_scale": self.right_scale}


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "DenseMlpConfig":
        _only(d, ("ff", "kind"), "a feed-forward")
        if d.get("kind") != "dense":
            raise ConfigError(f"config.json: feed-forward kind {d.get('kind')!r} is not built; known: 'dense'")
        c = cls(_need(d, "ff"))
        if c.ff <= 0:
            raise ConfigError("config.json: ff must be positive")
        return c

    def to_dict(self) -> Dict[str, Any]:
        return {"ff": self.ff, "kind": "dense"}


_MIXERS = {"gla": GlaMixerConfig, "parallel": ParallelMixerConfig}


@dataclass(frozen=True)
class DiruraxLayer:
    type: str
    mixer: Union[GlaMixerConfig, ParallelMixerConfig]
    mlp: Optional[DenseMlpConfig]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], index: int) -> "DiruraxLayer":
        _only(d, ("type", "mixer", "mlp"), f"layer {index}")
        kind = d.get("type")
        if kind not in _MIXERS:
            raise ConfigError(f"config.json: layer {index} has mixer type {kind!r}; known: {sorted(_MIXERS)}")
        if not isinstance(d.get("mixer"), Mapping):
            raise ConfigError(f"config.json: layer {index} has no 'mixer'")
        mlp = d.get("mlp")
        if mlp is not None and not isinstance(mlp, Mapping):
            raise ConfigError(f"config.json: layer {index}: 'mlp' is a table or null")
        return cls(kind, _MIXERS[kind].from_dict(d["mixer"]), DenseMlpConfig.from_dict(mlp) if mlp is not None else None)

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


@dataclass(frozen=True)
class DiruraxConfig:
    width: int
    vocab: int
    norm_eps: float
    layers: Tuple[DiruraxLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Dirurax"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], generation: Optional[Mapping[str, Any]] = None) -> "DiruraxConfig":
        norm = d.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("config.json: required key 'norm' is missing")
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        vocab = _need(d, "vocab")
        cfg = cls(width=_need(d, "width"), vocab=vocab, norm_eps=_need(norm, "eps", float),
                  layers=tuple(DiruraxLayer.from_dict(l, i) for i, l in enumerate(layers)),
                  eos_token_ids=_eos_ids(d, generation, vocab),
                  architecture=str(d.get("architecture") or "Dirurax"))
        if cfg.width <= 0 or cfg.vocab <= 0 or not cfg.norm_eps > 0:
            raise ConfigError("config.json: width, vocab and norm.eps must be positive")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
                             "norm": {"eps": self.norm_eps}, "layers": [l.to_dict() for l in self.layers]}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
