"""The Pikalix decoder as a registry entry: configuration -> model spec.

A token embedding that is RMS-normed; layers in the order config.json lists them, every sublayer
behind a norm that reads a weighted sum of the residual streams and followed by an update that mixes
the streams and adds the sublayer's output to each with a weight of its own (the `hyper` arrangement);
one kind of mixer, grouped-query attention with biased projections, an RMS norm over the whole q and k
projections, interleaved rotary pairs on part of a head, a sliding window and a softmax with one added
to its denominator, some layers reading the keys and values an earlier layer cached; a dense tanh-GELU
feed-forward or routed experts beside a shared one; a last RMS norm over the sum of the streams and a
head of its own.  Nothing here computes: the spec names registered parts and hands them the numbers
of config.json.

Tensor names: `embed`, `embed.norm`, `final.norm`, `head`, and per layer i `l<i>.norm1`, `l<i>.norm2`,
`l<i>.hc1.{in,out,mix}`, `l<i>.hc2.{in,out,mix}`, `l<i>.mix.{q,k,v}` (bias with `.b`, norm weight with
`.norm` added), `l<i>.mix.o`, `l<i>.mlp.{up,down}` or `l<i>.mlp.e<j>.{gate,up,down}`, `l<i>.mlp.router`,
`l<i>.mlp.correction`, `l<i>.mlp.shared.{gate,up,down}`.
"""
from __future__ import annotations

from typing import Optional

from ..config.dirurax_config import DenseMlpConfig
from ..config.pikalix_config import MoeMlpConfig, PikalixConfig
from ..config.registry import ArchitectureFamily, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

_ATTENTION_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                    "q_proj.bias": "q.b", "k_proj.bias": "k.b", "v_proj.bias": "v.b",
                    "q_norm": "q.norm", "k_norm": "k.norm"}


def _kept_window(cfg: PikalixConfig, owner: int) -> Optional[int]:
    """Keys the cache of layer `owner` must keep: the widest window among the layers that read it
    (None as soon as one of them sees every key)."""
    sizes = [l.mixer.mask_size for i, l in enumerate(cfg.layers) if i == owner or l.mixer.kv_from == owner]
    return None if any(s is None for s in sizes) else max(sizes)


def _mixer_spec(cfg: PikalixConfig, i: int) -> PartSpec:
    m = cfg.layers[i].mixer
    rope = None
    if m.rot_dims:
        rope = PartSpec("rope", {"head_dim": m.dim, "rotary_dim": m.rot_dims, "theta": m.rot_base, "scaling": None,
                                 "layout": "interleaved"})
    owner = i if m.kv_from is None else m.kv_from
    return PartSpec("gqa_attention", {
        "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
        "value_dim": m.vdim, "scale": m.scale, "window": m.mask_size, "cache_window": _kept_window(cfg, owner),
        "position": rope, "own_kv": m.kv_from is None, "bias": True, "qk_norm": "whole",
        "qk_norm_eps": cfg.norm_eps, "sink": True, "output": "float32", "tensor_names": _ATTENTION_NAMES})


def _ffn_spec(cfg: PikalixConfig, mlp) -> PartSpec:
    if isinstance(mlp, DenseMlpConfig):
        return PartSpec("dense_mlp", {"hidden_size": cfg.width, "intermediate_size": mlp.ff, "activation": "gelu_tanh",
                                      "up_name": "up", "down_name": "down", "output": "float32"})
    if isinstance(mlp, MoeMlpConfig):
        return PartSpec("routed_experts", {
            "hidden_size": cfg.width, "expert_ff": mlp.expert_ff, "experts": mlp.experts, "top": mlp.top,
            "groups_count": mlp.groups_count, "groups_keep": mlp.groups_keep, "shared_ff": mlp.shared_ff,
            "score": "sigmoid", "correction": True, "renormalize": False})
    raise TypeError(f"no feed-forward for {type(mlp).__name__}")


def pikalix_model_spec(cfg: PikalixConfig) -> ModelSpec:
    streams = cfg.streams or 1
    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."

        def norm(q: int) -> PartSpec:
            # without `streams` in config.json there are no connection tensors: one stream, x += y
            return PartSpec("hyper_rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "streams": streams,
                                              "learned": cfg.streams is not None, "weight_name": f"norm{q}",
                                              "connection_prefix": f"hc{q}."})
        names = {"mixer": p + "mix.", "mixer_norm": p}
        ffn = None
        if layer.mlp is not None:
            ffn = _ffn_spec(cfg, layer.mlp)
            names.update({"ffn": p + "mlp.", "ffn_norm": p})
        layers.append(LayerSpec(mixer=_mixer_spec(cfg, i), mixer_norm=norm(1), ffn=ffn,
                                ffn_norm=norm(2) if ffn else None, names=names, arrangement="hyper"))
        order.append(RunEntry(i, layer.mixer.kv_from))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, layers=tuple(layers), run_order=tuple(order),
        final_norm=PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight_name": ""}),
        embed_name="embed", final_norm_name="final.norm", head_name="head",
        tie_head=False, eos_token_ids=cfg.eos_token_ids, streams=streams,
        embed=PartSpec("normed_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "eps": cfg.norm_eps,
                                            "weight_name": "", "norm_name": ".norm"}),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied": False,
                                      "weight_name": ""}))


PIKALIX = ArchitectureFamily(name="pikalix", parse_config=PikalixConfig.from_dict, model_spec=pikalix_model_spec)
register_architecture(["pikalix"], PIKALIX)
