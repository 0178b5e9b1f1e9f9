"""Plain, slow statement of the Dirurax decoder: whole sequences, no cache, one function per
mechanism, float64 on the CPU.  It shares no code with ``rustinfer_b200``: the configuration
is a raw dict, the weights a name -> tensor map.

Notation.  x[t] is the residual stream, h the input of a sublayer, W.y a weight stored
[out, in] applied to y.  A layer is

    x <- x + LN_1b(mixer(LN_1(x)));   x <- x + LN_2b(ff(LN_2(x)))      (the second only with a feed-forward)

with LN the layer norm (mean and variance over the width, weight and bias).  Mixers:

  gla       S_t = diag(alpha_t) S_{t-1} + k_t v_t^T,  o_t = S_t^T q_t,  alpha = sigmoid(z)^(1/tau)
  parallel  c_l * attention(h) + c_r * delta(h)
    attention  grouped-query softmax attention without rotation, q and k RMS-normed per head with a
               shared weight, v divided by its RMS, keys visible only inside the query's own block of
               `mask.size` positions (and not after the query)
    delta      S_t = diag(w_t) S_{t-1} - (a_t * u_t)(u_t^T S_{t-1}) + k_t v_t^T,  o_t = S_t^T r_t,
               u = k / sqrt(|k|^2 + 1e-6)
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Sequence

import torch

F64 = torch.float64


def read_model_folder(folder: str):
    from safetensors import safe_open
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            w[name] = f.get_tensor(name).to(F64)
    return cfg, w


# ---------------------------------------------------------------------------- small parts
def rms_divide(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, w: torch.Tensor, b, eps: float) -> torch.Tensor:
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    y = (x - mu) / torch.sqrt(var + eps) * w
    return y if b is None else y + b


def sinusoid_positions(positions: Sequence[int], width: int) -> torch.Tensor:
    """Entry 2i: sin(p * 10000^(-2i/width)); entry 2i+1: cos of the same angle."""
    out = torch.zeros((len(positions), width), dtype=F64)
    for r, p in enumerate(positions):
        for i in range((width + 1) // 2):
            ang = p * 10000.0 ** (-2.0 * i / width)
            out[r, 2 * i] = math.sin(ang)
            if 2 * i + 1 < width:
                out[r, 2 * i + 1] = math.cos(ang)
    return out


def embed(table: torch.Tensor, ids: Sequence[int], pos0: int = 0) -> torch.Tensor:
    x = table[torch.tensor(list(ids), dtype=torch.long)]
    return x + sinusoid_positions(range(pos0, pos0 + len(ids)), table.shape[1])


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def dense_ff(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return gelu_erf(h @ up.T) @ down.T


# --------------------------------------------------------------------------------- mixers
def gla_scan(q, k, v, alpha):
    """q, k, alpha [T, H, dk]; v [T, H, dv] -> o [T, H, dv]; state from zero."""
    T, H, dk = k.shape
    S = torch.zeros((H, dk, v.shape[-1]), dtype=q.dtype)
    out = []
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, q[t]))
    return torch.stack(out)


def gla_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    H, dk, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    T = h.shape[0]
    q = (h @ w[p + "q"].T * dk ** -0.5).view(T, H, dk)
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / tau).view(T, H, dk)
    o = gla_scan(q, k, v, alpha)
    o = rms_divide(o, eps) * w[p + "norm"]
    g = h @ w[p + "g"].T
    return (o.reshape(T, H * dv) * (g * torch.sigmoid(g))) @ w[p + "o"].T


def block_attention(q, k, v, scale: float, block: int, pos0: int = 0):
    """q [T, H, d], k [T, G, d], v [T, G, dv].  Query at position i sees key j <= i when both lie
    in the same block of `block` positions counted from 0."""
    T, H, _ = q.shape
    G = k.shape[1]
    pos = torch.arange(pos0, pos0 + T)
    seen = (pos[None, :] <= pos[:, None]) & ((pos[None, :] // block) == (pos[:, None] // block))
    out = []
    for hq in range(H):
        g = hq // (H // G)
        s = (q[:, hq] @ k[:, g].T) * scale
        s = s.masked_fill(~seen, float("-inf"))
        out.append(torch.softmax(s, dim=-1) @ v[:, g])
    return torch.stack(out, dim=1)


def attention_mixer(h, w, p: str, m: dict, eps: float) -> torch.Tensor:
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rms_divide((h @ w[p + "q"].T).view(T, H, d), eps) * w[p + "q.norm"]
    k = rms_divide((h @ w[p + "k"].T).view(T, G, d), eps) * w[p + "k.norm"]
    v = rms_divide((h @ w[p + "v"].T).view(T, G, dv), eps)
    o = block_attention(q, k, v, float(m["scale"]), int(m["mask"]["size"]))
    return o.reshape(T, H * dv) @ w[p + "o"].T


def delta_scan(r, k, v, decay, rate):
    """All [T, H, d].  u = k / sqrt(|k|^2 + 1e-6); both state terms read the old state."""
    T, H, d = k.shape
    S = torch.zeros((H, d, d), dtype=r.dtype)
    out = []
    for t in range(T):
        u = k[t] / torch.sqrt((k[t] * k[t]).sum(dim=-1, keepdim=True) + 1e-6)
        uS = torch.einsum("hk,hkv->hv", u, S)
        S = decay[t][:, :, None] * S - (rate[t] * u)[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, r[t]))
    return torch.stack(out)


def delta_mixer(h, w, p: str, m: dict, eps: float) -> torch.Tensor:
    H, d = m["heads"], m["dim"]
    T = h.shape[0]
    r = (h @ w[p + "r"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, H, d)
    v = (h @ w[p + "v"].T).view(T, H, d)
    z = torch.tanh(h @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(z)).view(T, H, d)
    rate = torch.sigmoid(h @ w[p + "a"].T + w[p + "a.b"]).view(T, H, d)
    o = rms_divide(delta_scan(r, k, v, decay, rate), eps).reshape(T, H * d) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel_mixer(h, w, p: str, m: dict, eps: float) -> torch.Tensor:
    return (float(m["left_scale"]) * attention_mixer(h, w, p + "left.", m["left"], eps)
            + float(m["right_scale"]) * delta_mixer(h, w, p + "right.", m["right"], eps))


MIXERS = {"gla": gla_mixer, "parallel": parallel_mixer}


# ---------------------------------------------------------------------------------- model
def forward_layers(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int]) -> List[torch.Tensor]:
    """The stream after the embedding and after every layer."""
    eps = float(cfg["norm"]["eps"])
    ln = lambda x, name: layer_norm(x, w[name], w.get(name + ".b"), eps)
    x = embed(w["embed"], ids)
    seen = [x]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + ln(MIXERS[layer["type"]](ln(x, p + "norm1"), w, p + "mix.", layer["mixer"], eps), p + "norm1b")
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"feed-forward kind {layer['mlp']['kind']!r}")
            x = x + ln(dense_ff(ln(x, p + "norm2"), w[p + "mlp.up"], w[p + "mlp.down"]), p + "norm2b")
        seen.append(x)
    return seen


def forward_logits(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int]) -> torch.Tensor:
    x = forward_layers(cfg, w, ids)[-1]
    eps = float(cfg["norm"]["eps"])
    return layer_norm(x, w["final.norm"], w.get("final.norm.b"), eps) @ w["embed"].T
