"""Grouped-query attention over the paged cache
(crates/infer-worker/src/components/attention.rs:21-37,83-179): fused q,k,v projection,
rotary encoding of q and k, write of k and v into the request's pages, attention of every
new token over the keys it may see, output projection.  The residual add and the norm
before it belong to the block, not to this part.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from ..ops import kernels as K
from ..ops import library as L
from .base import (BuildContext, Mixer, PagedKV, PagedLayerCache, ParamDecl, POSITIONS, StepContext,
                   register_mixer, single_token_entries, token_tiles)
from .linear import Linear
from .spec import PartSpec


@register_mixer("gqa_attention")
class GQAAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, scale, window (None: all keys),
    position (PartSpec of a rotary encoding, or None), own_kv (False: the layer projects no
    keys or values and reads the cache another layer wrote).

    Further options, each None or absent by default: `value_dim` (size of a value and of a head's
    output where it is not head_dim), `block` (a query sees only keys of its own block of that
    many positions, counted from position 0 of the request), `qk_norm_eps` (q and k of every head
    are divided by their root mean square over head_dim and multiplied by the weights
    `q_norm` / `k_norm` [head_dim], shared by the heads), `value_norm_eps` (v of every head is divided
    by its root mean square; it is cached so), `tensor_names` (local name -> name in the file, for
    checkpoints that call q_proj.weight and the others something else), `bias` (q, k and v have biases
    `q_proj.bias` and so on, added in the projection), `qk_norm` ("head", the default; "whole": one RMS norm
    over all heads of q, and one over all of k, with weights of that size, before the rotation), `sink` (the
    softmax's denominator has one added: a key of score 0 that has no value), `cache_window` (keys the cache
    keeps where that is more than `window`: other layers with wider windows read this layer's cache),
    `output` ("float32": the sublayer's output leaves the output projection in 32-bit).  A mixer with any
    of these but the last two runs on the fp32-arithmetic attention kernels in both precisions: scores,
    softmax weights and the weighted sum of values are 32-bit there.  With `position`, the rotary part's
    `layout` says which channels pair up."""

    graph_safe = True
    adds_to_residual = True
    MAX_SPLITS = 16

    def __init__(self, params):
        super().__init__(params)
        p = params
        self.hidden = int(p["hidden_size"])
        self.Hq, self.Hkv, self.hd = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        self.scale = float(p["scale"])
        self.window = int(p["window"]) if p.get("window") else None
        self.own_kv = bool(p.get("own_kv", True))
        self.vd = int(p.get("value_dim") or self.hd)
        self.block = int(p["block"]) if p.get("block") else None
        self.qk_norm_eps = float(p["qk_norm_eps"]) if p.get("qk_norm_eps") is not None else None
        self.value_norm_eps = float(p["value_norm_eps"]) if p.get("value_norm_eps") is not None else None
        self.tensor_names = dict(p.get("tensor_names") or {})
        self.bias = bool(p.get("bias", False))
        self.qk_norm = str(p.get("qk_norm", "head"))
        if self.qk_norm not in ("head", "whole"):
            raise ValueError(f"qk_norm {self.qk_norm!r}: known are 'head' and 'whole'")
        self.sink = bool(p.get("sink", False))
        self.cache_window = (int(p["cache_window"]) if p.get("cache_window") else None) if "cache_window" in p else self.window
        if self.window is None and self.cache_window is not None:
            raise ValueError("a mixer that sees every key cannot read a cache that keeps a window")
        if self.window and self.cache_window and self.cache_window < self.window:
            raise ValueError(f"the cache keeps {self.cache_window} keys, the mask wants {self.window}")
        self.out_fp32 = str(p.get("output", "")) == "float32"
        whole = self.qk_norm_eps is not None and self.qk_norm == "whole"
        # options only the plain kernels serve
        self.general = (self.vd != self.hd or self.block is not None or self.qk_norm_eps is not None
                        or self.value_norm_eps is not None or self.bias or self.sink)
        # q, k, v leave the projection in 32-bit and one kernel adds biases, norms, rotates and writes the cache
        self.prepared = self.general and (self.bias or whole or self.sink or p.get("position") is not None
                                          or not self.own_kv)
        if self.prepared and self.value_norm_eps is not None:
            raise ValueError("values of unit root mean square are built for mixers without biases, rotation or a sink")
        if self.Hq % self.Hkv:
            raise ValueError(f"{self.Hq} heads are not a multiple of {self.Hkv} kv heads")
        if self.general:
            if not (1 <= self.hd <= 512 and 1 <= self.vd <= 512):
                raise ValueError(f"head sizes {self.hd}, {self.vd}: the attention kernel takes sizes up to 512")
            if self.qk_norm_eps is not None and self.value_norm_eps is not None and self.qk_norm_eps != self.value_norm_eps:
                raise ValueError("the norms of q, k and of v share one eps")
        elif self.hd % 16 or not 16 <= self.hd <= 512:
            raise ValueError(f"head_dim {self.hd}: the attention kernels take multiples of 16 up to 512")
        pos = p.get("position")
        self.position_spec: Optional[PartSpec] = pos
        self.position = None
        self.qkv: Optional[Linear] = None
        self.o: Optional[Linear] = None

    def _name(self, local: str) -> str:
        return self.tensor_names.get(local, local)

    def param_decls(self) -> Dict[str, ParamDecl]:
        q, kv = self.Hq * self.hd, self.Hkv * self.hd
        d = {self._name("q_proj.weight"): ParamDecl((q, self.hidden)),
             self._name("o_proj.weight"): ParamDecl((self.hidden, self.Hq * self.vd))}
        if self.own_kv:
            d[self._name("k_proj.weight")] = ParamDecl((kv, self.hidden))
            d[self._name("v_proj.weight")] = ParamDecl((self.Hkv * self.vd, self.hidden))
        if self.qk_norm_eps is not None:
            whole = self.qk_norm == "whole"
            d[self._name("q_norm")] = ParamDecl((q if whole else self.hd,), init="ones")
            if self.own_kv:
                d[self._name("k_norm")] = ParamDecl((kv if whole else self.hd,), init="ones")
        if self.bias:
            d[self._name("q_proj.bias")] = ParamDecl((q,), init="zeros")
            if self.own_kv:
                d[self._name("k_proj.bias")] = ParamDecl((kv,), init="zeros")
                d[self._name("v_proj.bias")] = ParamDecl((self.Hkv * self.vd,), init="zeros")
        return d

    def cache_need(self):
        return PagedKV(self.Hkv, self.hd, self.cache_window, value_dim=self.vd if self.vd != self.hd else None,
                       block=self.block)

    def prepare(self, ctx: BuildContext) -> None:
        super().prepare(ctx)
        # bf16 runs on the tensor-core kernels (head sizes up to 256); fp32, and larger heads,
        # on the plain fp32-arithmetic kernel
        self.use_mma = ctx.dtype == torch.bfloat16 and self.hd <= L.MMA_MAX_HEAD_DIM and not self.general
        # steps of 512 tokens or more: rotary encoding and cache write inside the q,k,v product
        self.fuse_rope = (ctx.dtype == torch.bfloat16 and self.hd in (64, 128)
                          and os.environ.get("RUSTINFER_B200_FUSE_ROPE", "1") != "0")
        # prompt portions: the tcgen05 kernel where it takes the geometry, else the mma.sync one
        self.use_tc = (self.use_mma and os.environ.get("RUSTINFER_B200_PREFILL_ATTENTION", "tc") != "mma"
                       and K.tc_attention_supports(self.Hq, self.Hkv, self.hd, ctx.page_size))
        if self.use_mma:
            self.tokens_per_tile = (K.tc_tokens_per_tile(self.Hq, self.Hkv) if self.use_tc
                                    else K.mma_tokens_per_tile(self.Hq, self.Hkv))
            # entries of one token go to the split-KV kernel, the others are cut into tiles
            self._single = single_token_entries()
            self._tiles = token_tiles(self.tokens_per_tile, skip_single_token=True)
            key = ("decode_scratch", self.Hq, self.hd)
            if key not in ctx.shared:
                no, nl = K.decode_scratch_floats(ctx.max_batch_seqs, self.Hq, self.hd, self.MAX_SPLITS)
                ctx.shared[key] = (torch.empty(no, dtype=torch.float32, device=ctx.device),
                                   torch.empty(nl, dtype=torch.float32, device=ctx.device))
            self.part_o, self.part_lse = ctx.shared[key]
            lib = L.attention_mma(self.hd)
            # the kernel that fetches keys and values by TMA where it is built for this geometry
            self.decode_ctas_per_sm = (int(lib.ri_attention_decode_tma_ctas_per_sm(ctx.page_size))
                                       or int(lib.ri_attention_decode_ctas_per_sm()))
            self.decode_tile_keys = int(lib.ri_attention_decode_tile_keys())
        else:
            self._single = None
            self._tiles = token_tiles(16, skip_single_token=False)
        # a mixer with the further options in bfloat16: entries of one token go to the kernel that reads a kv
        # head's keys once for all its query heads; prompt portions run on the tensor-core kernel with fp32
        # softmax weights (three bf16 pieces each) where keys and values have one size it is built for, else
        # on the fp32-arithmetic kernel.  The 32-bit engine keeps the one kernel whose sums do not depend on the cut.
        fast = (self.general and ctx.dtype == torch.bfloat16
                and os.environ.get("RUSTINFER_B200_BLOCK_ATTENTION", "fast") != "plain")
        self.precise_mma = (fast and self.vd == self.hd and self.hd % 16 == 0 and 16 <= self.hd <= L.MMA_MAX_HEAD_DIM)
        self.fast_single = fast and K.attention_single_supports(self.Hq, self.Hkv, self.hd, self.vd)
        if self.fast_single:
            key = ("single_scratch", self.Hq, self.vd)
            if key not in ctx.shared:
                n = K.attention_single_scratch_floats(ctx.max_batch_seqs, self.Hq, self.vd, self.MAX_SPLITS)
                ctx.shared[key] = torch.empty(n, dtype=torch.float32, device=ctx.device)
            self.single_part = ctx.shared[key]
        if self.precise_mma or self.fast_single:
            self._single = single_token_entries()
            rows = K.mma_tokens_per_tile(self.Hq, self.Hkv) if self.precise_mma else 16
            self._tiles = token_tiles(rows, skip_single_token=True)
            key = ("zero_tile_starts", ctx.max_batch_seqs)
            if key not in ctx.shared:
                ctx.shared[key] = torch.zeros(ctx.max_batch_seqs + 4, dtype=torch.int32, device=ctx.device)
            self._zeros = ctx.shared[key]
        if self.position_spec is not None:
            key = ("position", self.position_spec.key(), ctx.max_model_len)
            if key not in ctx.shared:
                part = POSITIONS.build(self.position_spec)
                part.prepare(ctx)
                ctx.shared[key] = part
            self.position = ctx.shared[key]

    def step_indices(self):
        return [self._tiles] if self._single is None else [self._single, self._tiles]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        # q, k, v fused by rows into one matrix, gate rows first
        # (crates/infer-worker/src/models/loader.rs:419-454)
        parts = [tensors[self._name("q_proj.weight")]]
        if self.own_kv:
            parts += [tensors[self._name("k_proj.weight")], tensors[self._name("v_proj.weight")]]
        dt = torch.float32 if any(t.dtype == torch.float32 for t in parts) else parts[0].dtype
        self.qkv = Linear(torch.cat([t.to(dt) for t in parts], dim=0), self.ctx.num_sms)
        self.o = Linear(tensors[self._name("o_proj.weight")], self.ctx.num_sms)
        self.q_norm = self.k_norm = None
        if self.qk_norm_eps is not None:
            self.q_norm = tensors[self._name("q_norm")].contiguous()
            if self.own_kv:
                self.k_norm = tensors[self._name("k_norm")].to(self.q_norm.dtype).contiguous()
        self.qkv_bias = None
        if self.bias:
            names = ["q_proj.bias"] + (["k_proj.bias", "v_proj.bias"] if self.own_kv else [])
            self.qkv_bias = torch.cat([tensors[self._name(n)].to(torch.float32) for n in names]).contiguous()

    def _project_out(self, out: torch.Tensor, residual: Optional[torch.Tensor]):
        if residual is not None and self.o.add_into(out, residual):
            return None
        return self.o(out, out_dtype=torch.float32 if self.out_fp32 else self.ctx.dtype)

    def _prepared_forward(self, x: torch.Tensor, step: StepContext, cache: PagedLayerCache, writes: bool):
        """q, k, v in 32-bit out of the projection; one kernel adds the biases, norms q and k, rotates them,
        rounds q to the activation dtype and writes k and v into their pages."""
        g = step.groups[cache.group]
        qkv = self.qkv(x, out_dtype=torch.float32)
        q = torch.empty((x.shape[0], self.Hq * self.hd), dtype=self.ctx.dtype, device=x.device)
        pos = self.position
        K.qkv_prepare(qkv, self.qkv_bias, self.q_norm, self.k_norm,
                      0 if self.qk_norm_eps is None else 2 if self.qk_norm == "whole" else 1,
                      self.qk_norm_eps or 0.0, step.positions, pos.cos if pos else None, pos.sin if pos else None,
                      pos.rotary_dim if pos else 0, bool(pos and pos.layout == "interleaved"),
                      g.slot_of_token if writes else None, cache.kv if writes else None, q,
                      self.Hq, self.Hkv, self.hd, self.vd, self.own_kv)
        return q

    def forward(self, x: torch.Tensor, step: StepContext, cache: PagedLayerCache,
                residual: Optional[torch.Tensor] = None):
        """Returns the sublayer's output, or None when it was added into `residual`."""
        g = step.groups[cache.group]
        writes = self.own_kv and cache.writes
        # many tokens: the product rotates q and k and writes keys and values into their pages in
        # its own epilogue (no pass over q, k, v in between)
        if (self.fuse_rope and self.position is not None and self.position.rotary_dim == self.hd
                and x.shape[0] >= 512 and (writes or not self.own_kv) and self.qkv.tensor_core):
            q = torch.empty((x.shape[0], self.Hq * self.hd), dtype=torch.bfloat16, device=x.device)
            if K.gemm_tc_rope(x, self.qkv.weight, q, step.positions, self.position.cos, self.position.sin,
                              g.slot_of_token if writes else None, cache.kv if writes else None,
                              self.Hq, self.Hkv if writes else 0, self.hd):
                return self._project_out(self.attend(q, step, cache), residual)
        if self.prepared:
            q = self._prepared_forward(x, step, cache, writes)
            return self._project_out(self.attend(q, step, cache), residual)
        qkv = self.qkv(x, out_dtype=self.ctx.dtype)
        if self.general:
            if self.position is not None or not self.own_kv:
                raise NotImplementedError("head norms, a value size of its own and the block mask are built "
                                          "for mixers without rotation that project their own keys")
            # per-head norms of q, k, v in fp32, then keys and values into their pages
            K.head_norm_scatter(qkv, self.q_norm, self.k_norm, self.value_norm_eps is not None,
                                self.qk_norm_eps if self.qk_norm_eps is not None else (self.value_norm_eps or 0.0),
                                g.slot_of_token if writes else None, cache.kv if writes else None,
                                self.Hq, self.Hkv, self.hd, self.vd)
            return self._project_out(self.attend(qkv[:, : self.Hq * self.hd], step, cache), residual)
        if self.position is not None:
            # a layer that reads another's cache has only the q projection: qkv is q alone
            K.rope_scatter(qkv, step.positions, self.position.cos,
                           self.position.sin, g.slot_of_token if writes else None,
                           cache.kv if writes else None, self.Hq, self.Hkv if writes else 0, self.hd,
                           self.position.rotary_dim)
        elif writes:
            # no position encoding inside the mixer: keys and values go into their pages as they are
            K.rope_scatter(qkv, step.positions, None, None, g.slot_of_token, cache.kv, self.Hq, self.Hkv,
                           self.hd, 0)
        return self._project_out(self.attend(qkv[:, : self.Hq * self.hd], step, cache), residual)

    def unmerged_ranges(self, step: StepContext) -> int:
        """Key ranges a step of single tokens only is cut into when its caller merges them itself
        (`attend(..., merge=False)`); 0 when there is nothing to merge (another kind of step, one
        range, or the kernel without ranges)."""
        if not self.use_mma or not step.decode_only:
            return 0
        splits = self._splits(step.num_tokens, step.max_kv_len)
        return splits if splits > 1 else 0

    def attend(self, q: torch.Tensor, step: StepContext, cache: PagedLayerCache,
               out: Optional[torch.Tensor] = None, merge: bool = True) -> torch.Tensor:
        """Attention of the rotated queries q [T, Hq*hd] (unit column stride) over the cache, whose
        pages already hold this step's keys and values: [T, Hq*hd] (into `out` if given).  With
        `merge` False in a step for which `unmerged_ranges` is not 0, the key ranges' partial
        results stay in `self.part_o` / `self.part_lse` and `out` is not written."""
        T = step.num_tokens
        g = step.groups[cache.group]
        if out is None:
            out = torch.empty((T, self.Hq * self.vd), dtype=self.ctx.dtype, device=q.device)
        if self.general and self._single is not None:
            (single,) = step.index(self._single)
            if single.numel() and self.fast_single:
                K.attention_single(q, out, cache.kv, g.block_table, step.cu_q, step.kv_len, single, self.Hq, self.Hkv,
                                   self.hd, self.scale, self.window, self.block, self.vd, sink=self.sink,
                                   splits=self._single_splits(single.numel(), step.max_kv_len), part=self.single_part)
            elif single.numel():                      # every single token is a tile of one row
                K.attention_plain(q, out, cache.kv, g.block_table, step.cu_q, step.kv_len, single,
                                  self._zeros[: single.numel()], self.Hq, self.Hkv, self.hd, self.scale,
                                  self.window, self.block, self.vd, sink=self.sink)
            tile_entry, tile_tok0 = step.index(self._tiles)
            if tile_entry.numel() and self.precise_mma:
                K.attention_prefill_bf16(q, out, cache.kv, g.block_table, step.cu_q, step.kv_len, tile_entry,
                                         tile_tok0, self.Hq, self.Hkv, self.hd, self.scale, self.window,
                                         self.block, precise=True, sink=self.sink)
            elif tile_entry.numel():
                K.attention_plain(q, out, cache.kv, g.block_table, step.cu_q, step.kv_len, tile_entry, tile_tok0,
                                  self.Hq, self.Hkv, self.hd, self.scale, self.window, self.block, self.vd,
                                  sink=self.sink)
            return out
        if not self.use_mma:
            tile_entry, tile_q0 = step.index(self._tiles)
            K.attention_plain(q, out, cache.kv, g.block_table, step.cu_q, step.kv_len, tile_entry, tile_q0,
                              self.Hq, self.Hkv, self.hd, self.scale, self.window, self.block, self.vd, sink=self.sink)
            return out
        (single,) = step.index(self._single)
        if single.numel():
            splits = self._splits(single.numel(), step.max_kv_len)
            K.attention_decode_bf16(q, out, cache.kv, g.block_table, step.cu_q, step.kv_len,
                                    single, single.numel(), self.Hq, self.Hkv, self.hd,
                                    self.scale, self.window, splits, self.part_o, self.part_lse,
                                    merge=merge or not step.decode_only)
        tile_entry, tile_tok0 = step.index(self._tiles)
        if tile_entry.numel():
            prefill = K.attention_prefill_tc if self.use_tc else K.attention_prefill_bf16
            prefill(q, out, cache.kv, g.block_table, step.cu_q, step.kv_len, tile_entry, tile_tok0,
                    self.Hq, self.Hkv, self.hd, self.scale, self.window)
        return out

    def _single_splits(self, n_single: int, max_kv_len: int) -> int:
        """Ranges the fp32-arithmetic kernel for single tokens cuts an entry's keys into: enough CTAs for four
        an SM, no range shorter than 128 keys.  A CTA walks its keys in order, so few CTAs with many keys
        each are bound by the latency of that walk (64 entries of 4 kv heads at 1,024 keys: 114 us in one
        range, 70 in two, 67 in four, 74 in eight)."""
        span = max_kv_len
        if self.window:
            span = min(span, self.window)
        if self.block:
            span = min(span, self.block)
        want = -(-4 * self.ctx.num_sms // max(1, n_single * self.Hkv))
        return max(1, min(want, -(-span // 128), self.MAX_SPLITS))

    def _splits(self, n_decode: int, max_kv_len: int) -> int:
        """Ranges each decoding request's keys are cut into.  A few CTAs sit on an SM (the
        kernel says how many).  A grid that fits one wave is best filled as far as it goes; a
        grid of several waves pays for every wave's start and end, so it is scored by how
        full its last wave is, at a discount.  Measured on B200 at 4,096 keys with 5 CTAs per
        SM: batch 8, 11 ranges (704 CTAs, one wave) 20.6 us, 13 ranges (a second wave) 26.1 us;
        batch 64, 4 ranges 107 us, 1 range 138 us.  Never more ranges than tiles of keys."""
        chunks = (self.Hq // self.Hkv + 15) // 16
        ctas = n_decode * self.Hkv * chunks
        span = min(max_kv_len, self.window) if self.window else max_kv_len
        tiles = max(1, -(-span // self.decode_tile_keys))
        slots = self.decode_ctas_per_sm * self.ctx.num_sms
        best, best_score = 1, -1.0
        for s in range(1, min(tiles, self.MAX_SPLITS) + 1):
            waves = ctas * s / slots
            score = waves if waves <= 1.0 else 0.85 * waves / float(-(-ctas * s // slots))
            if score > best_score + 0.02:
                best, best_score = s, score
        return best
