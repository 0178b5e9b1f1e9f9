"""The Dirurax decoder as a registry entry: configuration -> model spec.

A token embedding plus a sinusoidal position vector; layers in the order config.json lists them,
each with a layer norm before and after every sublayer (the `sandwich` arrangement); two kinds of
mixer, gated linear attention (`gla`) and attention over the current block of positions beside a
delta-rule recurrence (`parallel`); a dense GELU feed-forward where the layer has one; a last layer
norm and a head tied to the embedding table.  Nothing here computes: the spec names registered
parts and hands them the numbers of config.json.

Tensor names: `embed`, `final.norm`, and per layer i `l<i>.norm1`, `l<i>.norm1b`, `l<i>.norm2`,
`l<i>.norm2b` (weight; bias with `.b` added), `l<i>.mix.*`, `l<i>.mlp.up`, `l<i>.mlp.down`.
"""
from __future__ import annotations

from ..config.dirurax_config import DiruraxConfig, GlaMixerConfig, ParallelMixerConfig
from ..config.registry import ArchitectureFamily, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _mixer_spec(cfg: DiruraxConfig, m) -> PartSpec:
    if isinstance(m, GlaMixerConfig):
        return PartSpec("gated_linear_attention", {
            "hidden_size": cfg.width, "num_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim,
            "tau": m.tau, "norm_eps": cfg.norm_eps, "decay_rank": m.rank})
    if isinstance(m, ParallelMixerConfig):
        a, r = m.left, m.right
        left = PartSpec("gqa_attention", {
            "hidden_size": cfg.width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
            "value_dim": a.vdim, "scale": a.scale, "window": None, "block": a.mask_size, "position": None,
            "qk_norm_eps": cfg.norm_eps, "value_norm_eps": cfg.norm_eps,
            "tensor_names": {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v",
                             "o_proj.weight": "o", "q_norm": "q.norm", "k_norm": "k.norm"}})
        right = PartSpec("delta_rule", {
            "hidden_size": cfg.width, "num_heads": r.heads, "key_dim": r.dim, "norm_eps": cfg.norm_eps,
            "decay_rank": r.rank})
        return PartSpec("parallel_mixers", {"left": left, "right": right, "left_scale": m.left_scale,
                                            "right_scale": m.right_scale})
    raise TypeError(f"no mixer for {type(m).__name__}")


def dirurax_model_spec(cfg: DiruraxConfig) -> ModelSpec:
    norm = PartSpec("layernorm", {"size": cfg.width, "eps": cfg.norm_eps, "bias": True})
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        names = {"mixer": p + "mix.", "mixer_norm": p + "norm1", "post_mixer_norm": p + "norm1b"}
        extra = {"post_mixer_norm": norm}
        ffn = None
        if layer.mlp is not None:
            ffn = PartSpec("dense_mlp", {"hidden_size": cfg.width, "intermediate_size": layer.mlp.ff,
                                         "activation": "gelu", "up_name": "up", "down_name": "down"})
            names.update({"ffn": p + "mlp.", "ffn_norm": p + "norm2", "post_ffn_norm": p + "norm2b"})
            extra["post_ffn_norm"] = norm
        layers.append(LayerSpec(mixer=_mixer_spec(cfg, layer.mixer), mixer_norm=norm, ffn=ffn,
                                ffn_norm=norm if ffn else None, names=names, arrangement="sandwich",
                                extra_norms=extra))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, layers=tuple(layers),
        run_order=tuple(RunEntry(i) for i in range(len(layers))),
        # the last norm's bias is used when the file has one
        final_norm=PartSpec("layernorm", {"size": cfg.width, "eps": cfg.norm_eps, "bias": None}),
        embed_name="embed", final_norm_name="final.norm", head_name="head.",
        tie_head=True, eos_token_ids=cfg.eos_token_ids,
        embed=PartSpec("sinusoid_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                              "base": 10000.0, "weight_name": ""}))


DIRURAX = ArchitectureFamily(name="dirurax", parse_config=DiruraxConfig.from_dict, model_spec=dirurax_model_spec)
register_architecture(["dirurax"], DIRURAX)
