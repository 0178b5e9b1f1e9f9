"""Shared by the Pikalix tests: small configurations that differ from one another in every size, constant
and layer order, weights that make faults show, model folders, the plain model's logits."""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Sequence

import torch

import plain_pikalix


def _att(heads, kv, dim, vdim, scale, mask=None, rot=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if mask:
        m["mask"] = {"size": mask}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, groups=None, shared=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _layer(mixer, mlp=None):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


# P: three streams; values wider than keys; a window of 20 (a page and a quarter) read by its own layer and a
#    window of 37 by the layer that borrows its cache (the cache must keep the wider one); a layer that sees
#    every key and rotates whole heads, with one kv head for six query heads; a layer without a feed-forward;
#    experts in groups with a shared one, and experts without groups or a shared one
# Q: one stream with learned connections; keys and values of one size (the cache of equal sizes; heads of 64
#    take the tensor-core kernel for prompt portions in bfloat16); a window equal to the page; a layer without
#    rotation; one expert a token out of two groups of which one is kept; sixteen experts of which four are used
# R: no `streams` key (the plain residual sum); one head of an odd size with rotation on half of it and no mask;
#    as many experts used as there are; a window of 9 inside one page
CONFIGS = {
    "P": {"architecture": "Pikalix", "width": 96, "vocab": 211, "norm": {"eps": 1e-5}, "streams": 3, "layers": [
        _layer(_att(4, 2, 16, 24, 0.3, mask=20, rot=(8, 10000.0)), _dense(136)),
        _layer(_att(4, 2, 16, 24, 0.25, mask=37, rot=(8, 10000.0), kv_from=0), _moe(8, 3, 40, groups=(4, 2), shared=56)),
        _layer(_att(6, 1, 8, 16, 0.4, rot=(8, 300.0)), _moe(6, 2, 24)),
        _layer(_att(6, 1, 8, 16, 0.4, mask=50, rot=(8, 300.0), kv_from=2))]},
    "Q": {"architecture": "Pikalix", "width": 128, "vocab": 300, "norm": {"eps": 1e-6}, "streams": 1, "layers": [
        _layer(_att(2, 2, 32, 32, 0.2, mask=16, rot=(16, 500.0)), _dense(256)),
        _layer(_att(2, 1, 64, 64, 0.15, mask=100), _moe(4, 1, 48, groups=(2, 1), shared=64)),
        _layer(_att(2, 1, 64, 64, 0.15, mask=30, kv_from=1), _moe(16, 4, 24, groups=(4, 2)))]},
    "R": {"architecture": "Pikalix", "width": 64, "vocab": 97, "norm": {"eps": 3e-6}, "layers": [
        _layer(_att(1, 1, 40, 8, 0.2, rot=(20, 1e6)), _moe(3, 3, 20, shared=32)),
        _layer(_att(3, 3, 20, 36, 0.35, mask=9, rot=(20, 50.0)), _dense(72))]},
}


def tensor_shapes(name: str) -> Dict[str, tuple]:
    """Names and shapes of a checkpoint, written out here so that the tests do not lean on the framework's own list."""
    cfg = CONFIGS[name]
    d, v, n = cfg["width"], cfg["vocab"], cfg.get("streams")
    s = {"embed": (v, d), "embed.norm": (d,), "final.norm": (d,), "head": (v, d)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        q, kv, vv = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
        s.update({p + "norm1": (d,), p + "mix.q": (q, d), p + "mix.q.b": (q,), p + "mix.q.norm": (q,),
                  p + "mix.o": (d, m["heads"] * m["vdim"])})
        if "kv_from" not in m:
            s.update({p + "mix.k": (kv, d), p + "mix.k.b": (kv,), p + "mix.k.norm": (kv,), p + "mix.v": (vv, d),
                      p + "mix.v.b": (vv,)})
        subs = [1]
        mlp = layer["mlp"]
        if mlp:
            subs.append(2)
            s[p + "norm2"] = (d,)
            if mlp["kind"] == "dense":
                s[p + "mlp.up"], s[p + "mlp.down"] = (mlp["ff"], d), (d, mlp["ff"])
            else:
                ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
                for e in range(E):
                    s.update({f"{p}mlp.e{e}.gate": (ff, d), f"{p}mlp.e{e}.up": (ff, d), f"{p}mlp.e{e}.down": (d, ff)})
                s[p + "mlp.router"], s[p + "mlp.correction"] = (E, d), (E,)
                if "shared" in mlp:
                    sf = mlp["shared"]["ff"]
                    s.update({p + "mlp.shared.gate": (sf, d), p + "mlp.shared.up": (sf, d), p + "mlp.shared.down": (d, sf)})
        if n:
            for q_ in subs:
                s.update({f"{p}hc{q_}.in": (n,), f"{p}hc{q_}.out": (n,), f"{p}hc{q_}.mix": (n, n)})
    return s


def sharp_weights(name: str, seed: int, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Matrices of size 1/sqrt(fan_in) (q, k and the router several times that), norm weights spread around 1,
    biases and corrections around 0 (some choice scores go negative), stream weights that are far from the
    plain residual sum: activations are O(1), attention is peaked, the router's choices are mostly clear."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for n, shape in tensor_shapes(name).items():
        leaf = n.split(".")[-1]
        if leaf == "mix" and len(shape) == 2 and ".hc" in n:
            t = torch.eye(shape[0]) * 0.8 + 0.25 * torch.randn(shape, generator=g)
        elif leaf in ("in", "out") and ".hc" in n:
            t = 0.7 + 0.4 * torch.randn(shape, generator=g)
        elif leaf == "correction":
            t = 0.4 * torch.randn(shape, generator=g) - 0.3
        elif len(shape) == 1:
            t = 0.3 * torch.randn(shape, generator=g)
            if leaf != "b":
                t = t + 1.0
        elif n == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if leaf in ("q", "k"):
                t = t * 2.0
            if leaf == "router":
                t = t * 3.0
        out[n] = t.to(dtype)
    return out


def write_model(folder: str, name: str, weights: Dict[str, torch.Tensor]) -> str:
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(CONFIGS[name], f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def make_sharp_model(folder: str, name: str, seed: int = 0) -> str:
    return write_model(folder, name, sharp_weights(name, seed))


class Plain:
    """The plain implementation over one model folder, with per-sequence memo."""

    def __init__(self, folder: str):
        self.cfg, self.w = plain_pikalix.read_model_folder(folder)
        self._memo = {}

    def logits(self, ids: Sequence[int]) -> torch.Tensor:
        key = tuple(ids)
        if key not in self._memo:
            self._memo[key] = plain_pikalix.forward(self.cfg, self.w, list(ids))
        return self._memo[key]

    def greedy(self, prompt: Sequence[int], n: int) -> List[int]:
        ids, out = list(prompt), []
        for _ in range(n):
            t = int(torch.argmax(self.logits(ids)[-1]))
            out.append(t)
            ids.append(t)
        return out
