"""Typed configuration of the Pikalix decoder, read from config.json's own keys.

config.json names the width, the vocabulary, the norms' eps, the number of residual streams and a
list of layers; every layer names its mixer (`type`: only `attention`), the mixer's sizes and
constants (`mixer`) and its feed-forward (`mlp`: `dense`, `moe`, or null for none).  Every size and
constant is a field here; what config.json leaves out does not exist in the model (no `mask`: every
earlier key is seen; no `rot`: no rotation; no `groups`: every expert can be chosen; no `shared`: no
expert that every token uses; no `streams`: one stream and the plain residual sum).  An unknown mixer
type or feed-forward kind is an error, a key the engine does not know is named in a warning.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from .dirurax_config import DenseMlpConfig, _only
from .model_config import ConfigError, _eos_ids, _need


def _table(d: Mapping[str, Any], key: str, where: str) -> Optional[Mapping[str, Any]]:
    v = d.get(key)
    if v is not None and not isinstance(v, Mapping):
        raise ConfigError(f"config.json: {where}: '{key}' is a table")
    return v


@dataclass(frozen=True)
class SinkAttentionConfig:
    """Grouped-query attention with biased projections, an RMS norm over the whole q and k
    projections, rotary pairs on the first `rot_dims` channels of a head, a sliding window of
    `mask_size` keys and a softmax whose denominator has one added.  `kv_from`: the layer whose keys
    and values this one reads instead of projecting its own."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    mask_size: Optional[int] = None
    rot_dims: int = 0
    rot_base: float = 10000.0
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "SinkAttentionConfig":
        _only(d, ("heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot", "kv_from"), "an attention mixer")
        mask, rot = _table(d, "mask", "an attention mixer"), _table(d, "rot", "an attention mixer")
        if mask is not None:
            _only(mask, ("size",), "an attention mask")
        if rot is not None:
            _only(rot, ("base", "dims"), "a rotation")
        c = cls(_need(d, "heads"), _need(d, "kv_heads"), _need(d, "dim"), _need(d, "vdim"), _need(d, "scale", float),
                _need(mask, "size") if mask is not None else None,
                _need(rot, "dims") if rot is not None else 0,
                _need(rot, "base", float) if rot is not None else 10000.0,
                int(d["kv_from"]) if d.get("kv_from") is not None else None)
        if min(c.heads, c.kv_heads, c.dim, c.vdim) <= 0 or c.heads % c.kv_heads:
            raise ConfigError("config.json: an attention mixer needs positive sizes and heads a multiple of kv_heads")
        if c.mask_size is not None and c.mask_size <= 0:
            raise ConfigError("config.json: mask.size must be positive")
        if c.rot_dims < 0 or c.rot_dims % 2 or c.rot_dims > c.dim or (c.rot_dims and not c.rot_base > 0):
            raise ConfigError("config.json: rot.dims is even and at most dim, rot.base positive")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.mask_size is not None:
            d["mask"] = {"size": self.mask_size}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class MoeMlpConfig:
    """`experts` gated feed-forwards of width `expert_ff`, of which a token uses `top`, chosen by
    sigmoid scores plus a correction within the best `groups_keep` of `groups_count` groups of
    neighbours; `shared_ff`: width of the expert every token uses (None: there is none)."""
    experts: int
    top: int
    expert_ff: int
    groups_count: Optional[int] = None
    groups_keep: Optional[int] = None
    shared_ff: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "MoeMlpConfig":
        _only(d, ("kind", "expert", "router", "shared"), "a feed-forward of experts")
        expert, router = _table(d, "expert", "a feed-forward"), _table(d, "router", "a feed-forward")
        if expert is None or router is None:
            raise ConfigError("config.json: a feed-forward of experts needs 'expert' and 'router'")
        _only(expert, ("ff",), "an expert")
        _only(router, ("experts", "top", "groups"), "a router")
        groups, shared = _table(router, "groups", "a router"), _table(d, "shared", "a feed-forward")
        if groups is not None:
            _only(groups, ("count", "keep"), "a router's groups")
        if shared is not None:
            _only(shared, ("ff",), "a shared expert")
        c = cls(_need(router, "experts"), _need(router, "top"), _need(expert, "ff"),
                _need(groups, "count") if groups is not None else None,
                _need(groups, "keep") if groups is not None else None,
                _need(shared, "ff") if shared is not None else None)
        if min(c.experts, c.top, c.expert_ff) <= 0 or c.top > c.experts:
            raise ConfigError("config.json: a router needs positive experts and top <= experts")
        if c.groups_count is not None:
            if c.groups_count <= 0 or c.experts % c.groups_count or not 0 < c.groups_keep <= c.groups_count:
                raise ConfigError("config.json: groups.count divides experts and 0 < groups.keep <= groups.count")
            if c.groups_keep * (c.experts // c.groups_count) < c.top:
                raise ConfigError("config.json: the groups that are kept hold fewer experts than a token uses")
        if c.shared_ff is not None and c.shared_ff <= 0:
            raise ConfigError("config.json: shared.ff must be positive")
        return c

    def to_dict(self) -> Dict[str, Any]:
        router: Dict[str, Any] = {"experts": self.experts, "top": self.top}
        if self.groups_count is not None:
            router["groups"] = {"count": self.groups_count, "keep": self.groups_keep}
        d: Dict[str, Any] = {"kind": "moe", "expert": {"ff": self.expert_ff}, "router": router}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff}
        return d


_MLPS = {"dense": DenseMlpConfig, "moe": MoeMlpConfig}


@dataclass(frozen=True)
class PikalixLayer:
    type: str
    mixer: SinkAttentionConfig
    mlp: Optional[Union[DenseMlpConfig, MoeMlpConfig]]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], index: int) -> "PikalixLayer":
        _only(d, ("type", "mixer", "mlp"), f"layer {index}")
        if d.get("type") != "attention":
            raise ConfigError(f"config.json: layer {index} has mixer type {d.get('type')!r}; known: ['attention']")
        if not isinstance(d.get("mixer"), Mapping):
            raise ConfigError(f"config.json: layer {index} has no 'mixer'")
        mlp = _table(d, "mlp", f"layer {index}")
        if mlp is not None and mlp.get("kind") not in _MLPS:
            raise ConfigError(f"config.json: layer {index}: feed-forward kind {mlp.get('kind')!r} is not built; "
                              f"known: {sorted(_MLPS)}")
        return cls("attention", SinkAttentionConfig.from_dict(d["mixer"]),
                   _MLPS[mlp["kind"]].from_dict(mlp) if mlp is not None else None)

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


@dataclass(frozen=True)
class PikalixConfig:
    width: int
    vocab: int
    norm_eps: float
    layers: Tuple[PikalixLayer, ...]
    streams: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Pikalix"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], generation: Optional[Mapping[str, Any]] = None) -> "PikalixConfig":
        norm = d.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("config.json: required key 'norm' is missing")
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        vocab = _need(d, "vocab")
        cfg = cls(width=_need(d, "width"), vocab=vocab, norm_eps=_need(norm, "eps", float),
                  layers=tuple(PikalixLayer.from_dict(l, i) for i, l in enumerate(layers)),
                  streams=int(d["streams"]) if d.get("streams") is not None else None,
                  eos_token_ids=_eos_ids(d, generation, vocab),
                  architecture=str(d.get("architecture") or "Pikalix"))
        if cfg.width <= 0 or cfg.vocab <= 0 or not cfg.norm_eps > 0:
            raise ConfigError("config.json: width, vocab and norm.eps must be positive")
        if cfg.streams is not None and not 1 <= cfg.streams <= 8:
            raise ConfigError("config.json: streams is between 1 and 8")
        for i, layer in enumerate(cfg.layers):
            m, src = layer.mixer, layer.mixer.kv_from
            if src is None:
                continue
            if not 0 <= src < i or cfg.layers[src].mixer.kv_from is not None:
                raise ConfigError(f"config.json: layer {i} reads the keys of layer {src}, which must be an earlier "
                                  f"layer with projections of its own")
            o = cfg.layers[src].mixer
            if (o.kv_heads, o.dim, o.vdim) != (m.kv_heads, m.dim, m.vdim):
                raise ConfigError(f"config.json: layer {i} reads the keys of layer {src}, whose head sizes differ")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
                             "norm": {"eps": self.norm_eps}, "layers": [l.to_dict() for l in self.layers]}
        if self.streams is not None:
            d["streams"] = self.streams
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
