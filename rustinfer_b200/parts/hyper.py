"""Several residual streams joined to the sublayers by learned weights (hyper-connections).

Instead of one stream x there are n streams X_1 .. X_n, all equal to the embedding's output at the
start.  A sublayer with read weights a [n], mixing matrix M [n, n] (indexed [from, to]) and write
weights b [n] runs as

    u = sum_s a[s] X_s;   y = sublayer(rmsnorm(u) * w);   X_t <- sum_s M[s, t] X_s + b[t] y   (all t at once)

and the model's last norm reads the plain sum of the streams.  With n = 1, a = b = M = 1 this is the
usual residual sum.  `hyper_rmsnorm` is the norm in front of a sublayer together with the sublayer's
three connection tensors; a sublayer's output stays pending (`HyperPending`) and the next read of the
streams applies it, so that update, weighted sum and norm are one kernel over the streams, as the
residual add rides on the next RMSNorm in the `pre_norm` arrangement.  Streams, weights, sums and the
norm are fp32.  The reference engine has one stream (crates/infer-core/src/component.rs:8-27).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import kernels as K
from .base import Norm, ParamDecl, register_norm


@dataclass
class HyperPending:
    """A sublayer's output y [T, hidden] that is not yet in the streams, with the norm part that holds
    the sublayer's mixing matrix and write weights."""
    y: torch.Tensor
    owner: "HyperRMSNorm"


@register_norm("hyper_rmsnorm")
class HyperRMSNorm(Norm):
    """params: size, eps, streams, learned (False: no connection tensors, every weight is 1; only with
    one stream), weight_name (local name of the norm's weight, default "weight"), connection_prefix
    (local prefix of the tensors `in` [n], `out` [n], `mix` [n, n]; default "hc.")."""

    def __init__(self, params):
        super().__init__(params)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.streams = int(params.get("streams", 1))
        self.learned = bool(params.get("learned", True))
        self.weight_name = str(params.get("weight_name", "weight"))
        self.prefix = str(params.get("connection_prefix", "hc."))
        if not 1 <= self.streams <= K.HYPER_MAX_STREAMS:
            raise ValueError(f"{self.streams} streams: the kernel takes 1 to {K.HYPER_MAX_STREAMS}")
        if not self.learned and self.streams != 1:
            raise ValueError("several streams need their connection tensors")
        self.weight: Optional[torch.Tensor] = None
        self.read: Optional[torch.Tensor] = None           # a [n] fp32
        self.mix: Optional[torch.Tensor] = None            # M [n, n] fp32
        self.write: Optional[torch.Tensor] = None          # b [n] fp32

    def param_decls(self) -> Dict[str, ParamDecl]:
        d = {self.weight_name: ParamDecl((self.size,), init="ones")}
        if self.learned:
            n = self.streams
            d[self.prefix + "in"] = ParamDecl((n,), init="ones")
            d[self.prefix + "out"] = ParamDecl((n,), init="ones")
            d[self.prefix + "mix"] = ParamDecl((n, n), init="identity")
        return d

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()
        dev, n = self.weight.device, self.streams
        if self.learned:
            self.read = tensors[self.prefix + "in"].to(torch.float32).contiguous()
            self.write = tensors[self.prefix + "out"].to(torch.float32).contiguous()
            self.mix = tensors[self.prefix + "mix"].to(torch.float32).contiguous()
        else:
            self.read = torch.ones(n, dtype=torch.float32, device=dev)
            self.write = torch.ones(n, dtype=torch.float32, device=dev)
            self.mix = torch.eye(n, dtype=torch.float32, device=dev)

    def collect(self, hidden) -> torch.Tensor:
        """Apply what is pending to the streams, then return rmsnorm(sum_s a[s] X_s) * w [T, size]."""
        out = torch.empty((hidden.stream.shape[1], self.size), dtype=self.ctx.dtype, device=hidden.stream.device)
        _run(hidden, self.read, self.weight, self.eps, out, None)
        return out

    def add_norm(self, h, delta, rows=None):
        raise TypeError("hyper_rmsnorm reads several streams: it runs in the `hyper` block arrangement")


def _run(hidden, read, weight, eps, out, rows) -> None:
    p = hidden.pending
    K.hyper_collect(hidden.stream, hidden.fresh, p.y if p is not None else None,
                    p.owner.mix if p is not None else None, p.owner.write if p is not None else None,
                    read, weight, eps, out, rows)
    if rows is None and p is not None:
        hidden.fresh = False                 # every stream has been written
    if rows is None:
        hidden.pending = None


def finish(hidden, final_norm, rows: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The model's last norm over the plain sum of the streams, at `rows` only (the streams themselves
    are left as they are): rmsnorm(sum_t X_t) * w with what is pending applied on the way."""
    out = torch.empty((rows.numel(), final_norm.size), dtype=dtype, device=hidden.stream.device)
    _run(hidden, None, final_norm.weight, final_norm.eps, out, rows)
    return out


def stream_sum(hidden) -> torch.Tensor:
    """sum_t X_t [T, hidden] fp32 with what is pending applied (and written back): what a one-stream
    model would call its residual stream at this point."""
    out = torch.empty(hidden.stream.shape[1:], dtype=torch.float32, device=hidden.stream.device)
    _run(hidden, None, None, 0.0, out, None)
    return out
