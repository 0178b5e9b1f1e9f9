"""Shared by the Dirurax tests: small configurations that differ from one another in every size,
constant and layer order, weights that make faults show, model folders, the plain model's logits."""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Sequence

import torch

import plain_dirurax


def _gla(heads, dim, vdim, tau):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def _par(heads, kv, dim, vdim, scale, size, rheads, rdim, ls, rs):
    return {"left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}},
            "right": {"heads": rheads, "dim": rdim}, "left_scale": ls, "right_scale": rs}


def _layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": {"ff": ff, "kind": "dense"} if ff else None}


# X: attention first, values wider than keys, a block of 24 positions (one and a half pages of 16),
#    odd sizes everywhere, a gla layer with a feed-forward, rank 12 (not a multiple of 8)
# Y: keys and values of one size (the cache of equal sizes), block = page size, one kv head for six
#    query heads, a key size above 64 (eight lanes a column) that is not a multiple of 8
# Z: no attention at all (no paged cache group), one head, tau 1, key size 100
CONFIGS = {
    "X": {"architecture": "Dirurax", "width": 96, "vocab": 211, "norm": {"eps": 1e-5}, "rank": 12, "layers": [
        _layer("parallel", _par(4, 2, 16, 24, 0.3, 24, 3, 20, 0.8, 1.1), 136),
        _layer("gla", _gla(2, 24, 40, 8.0), 72),
        _layer("gla", _gla(3, 16, 16, 4.0))]},
    "Y": {"architecture": "Dirurax", "width": 128, "vocab": 300, "norm": {"eps": 1e-6}, "rank": 8, "layers": [
        _layer("gla", _gla(4, 32, 32, 16.0)),
        _layer("parallel", _par(2, 2, 32, 32, 0.2, 16, 2, 64, 1.0, 0.5), 256),
        _layer("parallel", _par(6, 1, 8, 16, 0.5, 50, 1, 76, 0.4, 1.3))]},
    "Z": {"architecture": "Dirurax", "width": 64, "vocab": 97, "norm": {"eps": 3e-6}, "rank": 5, "layers": [
        _layer("gla", _gla(1, 100, 8, 1.0), 64),
        _layer("gla", _gla(2, 8, 72, 32.0))]},
}


def config_json(name: str) -> dict:
    """What goes into config.json: the rank of the low-rank pairs is not a key of it."""
    cfg = json.loads(json.dumps(CONFIGS[name]))
    cfg.pop("rank")
    return cfg


def tensor_shapes(name: str) -> Dict[str, tuple]:
    """Names and shapes of a checkpoint, written out here so that the tests do not lean on the
    framework's own list."""
    cfg = CONFIGS[name]
    d, v, rank = cfg["width"], cfg["vocab"], cfg["rank"]
    s = {"embed": (v, d), "final.norm": (d,), "final.norm.b": (d,)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        norms = ["norm1", "norm1b"] + (["norm2", "norm2b"] if layer["mlp"] else [])
        for n in norms:
            s[p + n] = (d,)
            s[p + n + ".b"] = (d,)
        m = layer["mixer"]
        if layer["type"] == "gla":
            hk, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            s.update({p + "mix.q": (hk, d), p + "mix.k": (hk, d), p + "mix.v": (hv, d), p + "mix.g": (hv, d),
                      p + "mix.o": (d, hv), p + "mix.norm": (m["vdim"],), p + "mix.a1": (rank, d),
                      p + "mix.a2": (hk, rank), p + "mix.a2.b": (hk,)})
        else:
            a, r = m["left"], m["right"]
            q = p + "mix.left."
            s.update({q + "q": (a["heads"] * a["dim"], d), q + "k": (a["kv_heads"] * a["dim"], d),
                      q + "v": (a["kv_heads"] * a["vdim"], d), q + "q.norm": (a["dim"],), q + "k.norm": (a["dim"],),
                      q + "o": (d, a["heads"] * a["vdim"])})
            q = p + "mix.right."
            hd = r["heads"] * r["dim"]
            for n in ("r", "k", "v", "g", "a"):
                s[q + n] = (hd, d)
            s.update({q + "a.b": (hd,), q + "w1": (rank, d), q + "w2": (hd, rank), q + "w0": (hd,),
                      q + "norm": (hd,), q + "o": (d, hd)})
        if layer["mlp"]:
            s[p + "mlp.up"] = (layer["mlp"]["ff"], d)
            s[p + "mlp.down"] = (d, layer["mlp"]["ff"])
    return s


def sharp_weights(name: str, seed: int, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Matrices of size 1/sqrt(fan_in) (q, k, r twice that), norm weights spread around 1, biases
    around 0: activations are O(1), attention is peaked, decays spread over their range."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for n, shape in tensor_shapes(name).items():
        leaf = n.split(".")[-1]
        if len(shape) == 1:
            t = 0.3 * torch.randn(shape, generator=g)
            if leaf != "b" and leaf != "w0":
                t = t + 1.0
        elif n == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if leaf in ("q", "k", "r", "a2", "w2"):
                t = t * 2.0
        out[n] = t.to(dtype)
    return out


def write_model(folder: str, name: str, weights: Dict[str, torch.Tensor]) -> str:
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config_json(name), f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def make_sharp_model(folder: str, name: str, seed: int = 0) -> str:
    return write_model(folder, name, sharp_weights(name, seed))


class Plain:
    """The plain implementation over one model folder, with per-sequence memo."""

    def __init__(self, folder: str):
        self.cfg, self.w = plain_dirurax.read_model_folder(folder)
        self._memo = {}

    def logits(self, ids: Sequence[int]) -> torch.Tensor:
        key = tuple(ids)
        if key not in self._memo:
            self._memo[key] = plain_dirurax.forward_logits(self.cfg, self.w, list(ids))
        return self._memo[key]

    def greedy(self, prompt: Sequence[int], n: int) -> List[int]:
        ids, out = list(prompt), []
        for _ in range(n):
            t = int(torch.argmax(self.logits(ids)[-1]))
            out.append(t)
            ids.append(t)
        return out
