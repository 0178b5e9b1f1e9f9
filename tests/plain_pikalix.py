"""A plain, slow statement of the Pikalix decoder in float64 on the CPU: one function per mechanism,
whole sequences at once, no cache, no batching.  It shares no code with the package; the tests hold the
engine to it.

    embedding -> RMS norm -> `streams` copies of the stream
    per layer, per sublayer q (mixer, feed-forward):
        u = sum_s a_q[s] X_s;  y = sublayer(rmsnorm(u));  X_t <- sum_s M_q[s, t] X_s + b_q[t] y
    sum of the streams -> RMS norm -> head

Mixer: grouped-query attention with biased projections, an RMS norm over the whole q (and k) projection,
interleaved rotary pairs on the first `rot.dims` channels of every head, a sliding window, a softmax whose
denominator has one added, values of a size of their own, and optionally the keys and values of an earlier
layer.  Feed-forward: a tanh-GELU pair of matrices, or sigmoid-routed experts chosen within the best groups,
plus an expert every token uses.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional, Tuple

import torch

F64 = torch.float64


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: channels (2i, 2i+1), i < dims/2, turn by the angle p * base^(-2i/dims)."""
    if not dims:
        return x
    out = x.clone()
    i = torch.arange(dims // 2, dtype=F64)
    ang = positions.to(F64)[:, None] * base ** (-2.0 * i / dims)[None, :]       # [T, dims/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def keys_and_values(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping, eps: float,
                    positions: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """What a layer with projections of its own keeps: k [T, G, d] normed and rotated, v [T, G, dv]."""
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = h @ w["k"].T + w["k.b"]
    v = h @ w["v"].T + w["v.b"]
    k = rms_norm(k, w["k.norm"], eps).view(-1, G, d)
    rot = m.get("rot") or {}
    k = rotate_pairs(k, positions, int(rot.get("dims", 0)), float(rot.get("base", 1.0)))
    return k, v.view(-1, G, dv)


def sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int],
                   sink: bool = True) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] of positions 0..T-1 -> [T, H, dv].  Query i sees keys j with
    0 <= i - j < window (every j <= i without a window); weights exp(s_j) / (1 + sum exp(s_j)): the one in
    the denominator is a key of score 0 that has no value (left out when `sink` is False)."""
    T, H, _ = q.shape
    G, dv = k.shape[1], v.shape[2]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (j <= i)
    if window:
        seen = seen & (i - j < window)
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head, :].to(F64) @ k[:, g, :].to(F64).T) * scale
        s = s - (0.0 if sink else s.masked_fill(~seen, -math.inf).max(dim=-1, keepdim=True).values)
        e = torch.where(seen, torch.exp(s), torch.zeros_like(s))
        p = e / ((1.0 if sink else 0.0) + e.sum(dim=-1, keepdim=True))
        out[:, head, :] = p @ v[:, g, :].to(F64)
    return out


def attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping, eps: float, positions: torch.Tensor,
              kv: Tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
    """h [T, width] -> [T, width]; kv: the keys and values it reads (its own or an earlier layer's)."""
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rms_norm(h @ w["q"].T + w["q.b"], w["q.norm"], eps).view(T, H, d)
    rot = m.get("rot") or {}
    q = rotate_pairs(q, positions, int(rot.get("dims", 0)), float(rot.get("base", 1.0)))
    out = sink_attention(q, kv[0], kv[1], m["scale"], (m.get("mask") or {}).get("size"))
    return out.reshape(T, H * dv) @ w["o"].T


def dense_ff(h: torch.Tensor, w: Mapping[str, torch.Tensor]) -> torch.Tensor:
    return gelu_tanh(h @ w["up"].T) @ w["down"].T


def gated_expert(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str) -> torch.Tensor:
    return (silu(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def route(h: torch.Tensor, w: Mapping[str, torch.Tensor], r: Mapping) -> Tuple[torch.Tensor, torch.Tensor]:
    """(chosen experts [T, top], their weights [T, top])."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ w["router"].T)                        # [T, E]
    choice = s + w["correction"] if "correction" in w else s.clone()
    groups = r.get("groups")
    if groups:
        n, keep = groups["count"], groups["keep"]
        per = choice.view(-1, n, E // n)
        score = per.topk(min(2, E // n), dim=-1).values.sum(dim=-1)            # [T, n]
        best = score.topk(keep, dim=-1).indices
        allowed = torch.zeros_like(score, dtype=torch.bool).scatter_(1, best, True)
        choice = torch.where(allowed[:, :, None].expand_as(per), per, torch.full_like(per, -math.inf)).reshape(-1, E)
    chosen = choice.topk(top, dim=-1).indices
    return chosen, s.gather(1, chosen)


def moe_ff(h: torch.Tensor, w: Mapping[str, torch.Tensor], mlp: Mapping) -> torch.Tensor:
    chosen, weight = route(h, w, mlp["router"])
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weight[t]):
            out[t] += a * gated_expert(h[t:t + 1], w, f"e{e}.")[0]
    if mlp.get("shared"):
        out += gated_expert(h, w, "shared.")
    return out


def connected(X: List[torch.Tensor], a: torch.Tensor, M: torch.Tensor, b: torch.Tensor, fn) -> List[torch.Tensor]:
    """One sublayer over n streams: u = sum_s a[s] X_s, y = fn(u), X_t <- sum_s M[s, t] X_s + b[t] y."""
    n = len(X)
    y = fn(sum(a[s] * X[s] for s in range(n)))
    return [sum(M[s, t] * X[s] for s in range(n)) + b[t] * y for t in range(n)]


def read_model_folder(folder: str):
    """(config.json as a dict, tensors by name) of a model folder."""
    import json
    import os
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, load_file(os.path.join(folder, "model.safetensors"))


def _sub(w: Mapping[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(config: Mapping, weights: Mapping[str, torch.Tensor], tokens: List[int],
            after_layers: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  `after_layers`, if a list, gets the sum of the streams
    after every layer."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    S = config.get("streams")
    T = len(tokens)
    positions = torch.arange(T)
    x = rms_norm(w["embed"][torch.tensor(tokens)], w["embed.norm"], eps)
    X = [x.clone() for _ in range(S or 1)]
    kept: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}

    def sublayer(X, q: int, p: str, fn):
        norm = lambda u: rms_norm(u, w[f"{p}norm{q}"], eps)
        if not S:                                             # one stream: the plain residual sum
            return [X[0] + fn(norm(X[0]))]
        return connected(X, w[f"{p}hc{q}.in"], w[f"{p}hc{q}.mix"], w[f"{p}hc{q}.out"], lambda u: fn(norm(u)))

    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        mw = _sub(w, p + "mix.")

        def mixer(h, i=i, m=m, mw=mw):
            src = m.get("kv_from")
            if src is None:
                kept[i] = keys_and_values(h, mw, m, eps, positions)
                src = i
            return attention(h, mw, m, eps, positions, kept[src])

        X = sublayer(X, 1, p, mixer)
        mlp = layer.get("mlp")
        if mlp is not None:
            fw = _sub(w, p + "mlp.")
            X = sublayer(X, 2, p, (lambda h: dense_ff(h, fw)) if mlp["kind"] == "dense" else (lambda h: moe_ff(h, fw, mlp)))
        if after_layers is not None:
            after_layers.append(sum(X))
    return rms_norm(sum(X), w["final.norm"], eps) @ w["head"].T
