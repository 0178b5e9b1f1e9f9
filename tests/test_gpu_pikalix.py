"""The Pikalix family on the GPU against the plain implementation: every new kernel alone, then the engine
under every way of cutting the work (whole prompts, a decoded tail, portions down to two tokens, mixed batches
with pages and state slots used again), in true 32-bit and in bfloat16, on small configurations that differ in
every size; greedy generation through `Engine`; the trace replay command."""
import json
import math
import os
import subprocess

import pytest
import torch

import plain_pikalix as P
from helpers import random_ids, rel_err
from pikalix_helpers import CONFIGS, Plain, make_sharp_model

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"
F64 = torch.float64
# max |engine - plain| / max |plain| over the compared logits.  fp32 sums a few hundred products per output
# against float64; in bfloat16 projections and activations are rounded to 8 bits.
TOL = {"float32": 3e-5, "bfloat16": 6e-2}
DTYPES = ["float32", "bfloat16"]
NAMES = sorted(CONFIGS)


def K():
    from rustinfer_b200.ops import kernels
    return kernels


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float32) * scale


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# =============================================================================== kernels alone
@pytest.mark.parametrize("d", [83, 96])
def test_embed_rmsnorm(d):
    table = rnd(50, d, seed=1).to(torch.bfloat16)
    w = (1.0 + 0.3 * rnd(d, seed=2)).to(torch.bfloat16)
    ids = [3, 49, 0, 3, 17]
    out = torch.empty((len(ids), d), dtype=torch.float32, device=DEV)
    K().embed_rmsnorm(i32(ids), table.to(DEV), w.to(DEV), 1e-3, out)
    ref = P.rms_norm(table.to(F64)[ids], w.to(F64), 1e-3)
    assert rel_err(out, ref) < 1e-6


@pytest.mark.parametrize("S", [1, 3, 4])
@pytest.mark.parametrize("ydtype", [torch.float32, torch.bfloat16])
def test_stream_update_sum_and_norm(S, ydtype):
    """One launch applies the last sublayer's output to every stream, forms the weighted sum and norms it;
    fresh streams (only the first written), rows picked for the last norm, the plain sum without a norm."""
    T, d, eps = 7, 83, 1e-4
    x0 = rnd(T, d, seed=1)
    y = rnd(T, d, seed=2).to(ydtype)
    a, b, M = rnd(S, seed=3), rnd(S, seed=4), rnd(S, S, seed=5)
    w = (1.0 + 0.3 * rnd(d, seed=6))
    X = torch.zeros(S, T, d)
    X[0] = x0
    Xd = X.to(DEV)
    out = torch.empty((T, d), dtype=torch.float32, device=DEV)
    # first read: nothing pending, every stream is the first
    K().hyper_collect(Xd, True, None, None, None, a.to(DEV), w.to(DEV), eps, out)
    ref = P.rms_norm(float(a.sum()) * x0.to(F64), w.to(F64), eps)
    assert rel_err(out, ref) < 1e-5
    assert torch.equal(Xd.cpu(), X)                                     # nothing written yet
    # second read: the update of all streams from the old ones, then the sum with other weights
    a2 = rnd(S, seed=7)
    K().hyper_collect(Xd, True, y.to(DEV), M.to(DEV), b.to(DEV), a2.to(DEV), w.to(DEV), eps, out)
    new = P.connected([x0.to(F64)] * S, a.to(F64), M.to(F64), b.to(F64), lambda u: y.to(F64))
    assert rel_err(Xd, torch.stack(new)) < 1e-6
    assert rel_err(out, P.rms_norm(sum(a2[s].to(F64) * new[s] for s in range(S)), w.to(F64), eps)) < 1e-5
    # third: not fresh any more; rows picked, streams left alone, plain sum
    y2 = rnd(T, d, seed=8).to(ydtype)
    before = Xd.clone()
    rows = [5, 0, 5]
    picked = torch.empty((3, d), dtype=torch.bfloat16, device=DEV)
    K().hyper_collect(Xd, False, y2.to(DEV), M.to(DEV), b.to(DEV), None, w.to(DEV), eps, picked, i32(rows))
    new2 = P.connected(new, a2.to(F64), M.to(F64), b.to(F64), lambda u: y2.to(F64))
    assert torch.equal(Xd, before)
    assert rel_err(picked, P.rms_norm(sum(new2), w.to(F64), eps)[rows]) < 1e-2
    total = torch.empty((T, d), dtype=torch.float32, device=DEV)
    K().hyper_collect(Xd, False, y2.to(DEV), M.to(DEV), b.to(DEV), None, None, 0.0, total)
    assert rel_err(total, sum(new2)) < 1e-6 and rel_err(Xd, torch.stack(new2)) < 1e-6


def plain_prepare(qkv, bias, qw, kw, mode, eps, pos, rot, base, interleaved, H, G, dk, dv):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] as the attention reads them (float64)."""
    T = qkv.shape[0]
    x = qkv.to(F64) + bias.to(F64)
    q, k, v = x[:, : H * dk], x[:, H * dk: (H + G) * dk], x[:, (H + G) * dk:]
    if mode == 2:
        q, k = P.rms_norm(q, qw.to(F64), eps), P.rms_norm(k, kw.to(F64), eps)
    q, k = q.reshape(T, H, dk), k.reshape(T, G, dk)
    if mode == 1:
        q, k = P.rms_norm(q, qw.to(F64), eps), P.rms_norm(k, kw.to(F64), eps)
    if rot and interleaved:
        q, k = P.rotate_pairs(q, pos, rot, base), P.rotate_pairs(k, pos, rot, base)
    elif rot:                                  # channel i with channel i + rot/2: the same turn after a shuffle
        perm = [c // 2 if c % 2 == 0 else rot // 2 + c // 2 for c in range(rot)]      # interleaved slot -> half slot
        def half(t):
            t = t.clone()
            inter = t[..., perm]
            t[..., perm] = P.rotate_pairs(inter, pos, rot, base)
            return t
        q, k = half(q), half(k)
    return q, k, v.reshape(T, G, dv)


@pytest.mark.parametrize("mode,interleaved,rot", [(2, True, 8), (2, True, 12), (1, False, 12), (0, True, 0), (2, False, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_qkv_prepare(mode, interleaved, rot, dtype):
    """Bias, the norm over the whole projection (or per head, or none), the rotation of part of every head in both
    pairings, far positions, q rounded once, k and v into scrambled pages (and nothing where the slot is -1)."""
    T, H, G, dk, dv, page, eps, base = 9, 4, 2, 12, 20, 4, 1e-3, 700.0
    qkv = rnd(T, H * dk + G * (dk + dv), seed=1)
    bias = rnd(qkv.shape[1], seed=2, scale=0.5)
    n = {0: (1, 1), 1: (dk, dk), 2: (H * dk, G * dk)}[mode]
    qw, kw = 1.0 + 0.3 * rnd(n[0], seed=3), 1.0 + 0.3 * rnd(n[1], seed=4)
    pos = torch.tensor([0, 1, 2, 1000, 1001, 4095, 7, 8, 9])
    f = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=F64) if rot else None
    ang = pos.to(F64)[:, None] * f[None, :] if rot else None
    cos = torch.zeros(4096, max(rot // 2, 1)); sin = torch.zeros(4096, max(rot // 2, 1))
    if rot:
        cos[pos], sin[pos] = torch.cos(ang).float(), torch.sin(ang).float()
    slots = [13, 2, 7, 0, -1, 22, 9, 5, 30]
    pages = 9
    cache = torch.full((pages, G * page * (dk + dv)), 77.0, dtype=dtype, device=DEV)
    q_out = torch.empty((T, H * dk), dtype=dtype, device=DEV)
    K().qkv_prepare(qkv.to(DEV), bias.to(DEV), qw.to(DEV) if mode else None, kw.to(DEV) if mode else None, mode, eps,
                    i32(pos.tolist()), cos.to(DEV) if rot else None, sin.to(DEV) if rot else None, rot, interleaved,
                    i32(slots), cache, q_out, H, G, dk, dv, True)
    q, k, v = plain_prepare(qkv, bias, qw, kw, mode, eps, pos, rot, base, interleaved, H, G, dk, dv)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    assert rel_err(q_out, q.reshape(T, H * dk)) < tol
    c = cache.float().cpu()
    for t, slot in enumerate(slots):
        if slot < 0:
            continue
        pg, off = slot // page, slot % page
        for g in range(G):
            got_k = c[pg, (g * page + off) * dk: (g * page + off + 1) * dk]
            b0 = G * page * dk + (g * page + off) * dv
            assert rel_err(got_k, k[t, g]) < tol and rel_err(c[pg, b0: b0 + dv], v[t, g]) < tol
    used = sum(1 for s in slots if s >= 0) * G * (dk + dv)
    assert int((c != 77.0).sum()) <= used and int((c == 77.0).sum()) >= c.numel() - used
    # a layer that reads another's keys: q alone, nothing written
    q_only = torch.empty_like(q_out)
    K().qkv_prepare(qkv[:, : H * dk].contiguous().to(DEV), bias[: H * dk].contiguous().to(DEV), qw.to(DEV) if mode else None,
                    None, mode, eps, i32(pos.tolist()), cos.to(DEV) if rot else None, sin.to(DEV) if rot else None, rot,
                    interleaved, None, None, q_only, H, G, dk, dv, False)
    assert torch.equal(q_only, q_out)


def paged(keys, vals, page, table, dtype):
    """A cache [pages, Hkv*page*(dk+dv)] (or [pages, 2, Hkv, page, d] when the sizes are equal) that holds keys
    [n, G, dk] and vals [n, G, dv] of one request in the pages `table` names; the rest is poison."""
    n, G, dk = keys.shape
    dv = vals.shape[2]
    pages = max(table) + 2
    c = torch.full((pages, G * page * (dk + dv)), 1e4, dtype=torch.float32)
    for t in range(n):
        pg, off = table[t // page], t % page
        for g in range(G):
            c[pg, (g * page + off) * dk: (g * page + off + 1) * dk] = keys[t, g]
            b = G * page * dk + (g * page + off) * dv
            c[pg, b: b + dv] = vals[t, g]
    c = c.to(dtype).to(DEV)
    return c.view(pages, 2, G, page, dk) if dk == dv else c


@pytest.mark.parametrize("dk,dv,window", [(16, 24, 20), (32, 32, 16), (40, 8, 33), (20, 36, None)])
def test_sink_attention_edges_and_far_keys(dk, dv, window):
    """One key stands out for every query: its score is 0, like the sink's, and every other score is at least
    30 lower.  So the output is half that key's value when the key is inside the window, and nearly nothing when
    it is outside (the sink takes the weight).  Keys just inside and just outside the window, in prompt portions
    and for single tokens, with the window's edge inside a page and at a page's edge, the pages scrambled and
    poisoned outside; without a window, a key hundreds of tokens back among hundreds of others.  The same inputs
    through the plain model give the numbers.  (Keys are unit vectors with a channel of 1 appended, queries the
    looked-for key times a gain with -gain appended: q . k = gain * (cos - 1).)"""
    page, H, G, n = 8, 4, 2, 330
    table = torch.randperm(48, generator=torch.Generator().manual_seed(5)).tolist()[: (n + page - 1) // page]
    unit = torch.nn.functional.normalize(rnd(n, dk, seed=2), dim=-1)
    cosm = unit @ unit.T - 2.0 * torch.eye(n)
    gain = 30.0 / (1.0 - float(cosm.max()))
    keys = torch.cat([unit, torch.ones(n, 1)], dim=-1)[:, None, :].repeat(1, G, 1)
    vals = rnd(n, G, dv, seed=1)
    d1 = dk + 1
    cache = paged(keys, vals, page, table, torch.float32)
    bt = i32([table])

    def queries(targets):
        q = torch.zeros(len(targets), H, d1)
        for i, tgt in enumerate(targets):
            q[i, :, :dk] = unit[tgt] * gain
            q[i, :, dk] = -gain
        return q

    def plain_rows(first, targets):
        T = first + len(targets)
        q = torch.zeros(T, H, d1)
        q[first:] = queries(targets)
        return P.sink_attention(q, keys[:T], vals[:T], 1.0, window)[first:]

    def attend(first, targets):
        count = len(targets)
        out = torch.empty((count, H * dv), dtype=torch.float32, device=DEV)
        tiles = list(range(0, count, 16))
        K().attention_plain(queries(targets).reshape(count, H * d1).to(DEV), out, cache, bt, i32([0, count]),
                            i32([first + count]), i32([0] * len(tiles)), i32(tiles), H, G, d1, 1.0, window, None, dv, sink=True)
        return out.cpu().view(count, H, dv)

    def attend_single(pos, tgt, splits=1):
        """The kernel for entries of one token; with `splits`, the keys in that many ranges joined by a second launch."""
        out = torch.empty((1, H * dv), dtype=torch.float32, device=DEV)
        part = torch.full((K().attention_single_scratch_floats(1, H, dv, splits),), float("nan"), device=DEV)
        K().attention_single(queries([tgt]).reshape(1, H * d1).to(DEV), out, cache, bt, i32([0, 1]), i32([pos + 1]),
                             i32([0]), H, G, d1, 1.0, window, None, dv, sink=True, splits=splits, part=part)
        return out.cpu().view(H, dv)

    w = window or 10 ** 9
    first, count = 45, 70
    for shift in ((0, 1, w - 1, w, w + 1) if window else (0, 1, 40, 100)):
        targets = [max(0, p - shift) for p in range(first, first + count)]
        got, ref = attend(first, targets), plain_rows(first, targets)
        assert float((got.to(F64) - ref).abs().max()) < 2e-4, shift
        seen = shift < w
        lead = ref[-1, 0] - 0.5 * vals[targets[-1], 0].to(F64)
        assert (float(lead.abs().max()) < 1e-3) == seen
        assert seen or float(ref[-1].abs().max()) < 1e-6
    if window:
        singles = [(p, t) for p in (w - 1, w, w + 1, 2 * w + 3, n - 1) for t in (p, p - w + 1, p - w, 0) if 0 <= t <= p]
    else:
        singles = [(n - 1, 3), (n - 1, n - 1), (300, 0), (64, 63), (7, 0)]
    for p, tgt in singles:
        ref = plain_rows(p, [tgt])[0]
        assert float((attend(p, [tgt])[0].to(F64) - ref).abs().max()) < 2e-4, (p, tgt)
        if K().attention_single_supports(H, G, d1, dv):
            for splits in (1, 2, 5):                       # with 5, ranges of 64 keys: some are empty
                assert float((attend_single(p, tgt, splits).to(F64) - ref).abs().max()) < 2e-4, (p, tgt, splits)


@pytest.mark.parametrize("hd,H,G,window", [(32, 4, 2, 24), (64, 6, 1, 50), (16, 2, 2, None)])
def test_sink_attention_on_tensor_cores(hd, H, G, window):
    """Prompt portions of the bfloat16 engine where keys and values have one size: scores from the tensor cores,
    softmax weights in fp32, the sink's one in the denominator and the window's lower bound.  Two requests in one
    launch, one starting in the middle of its sequence, against the plain model on the same bf16 inputs."""
    page = 16
    lens, firsts = [70, 33], [0, 27]
    tables = [[3, 0, 5, 2, 7], [1, 4, 6, 8]]
    cache = torch.full((10, 2, G, page, hd), 1e4, dtype=torch.bfloat16)
    qs, refs, kept = [], [], []
    for r, (n, first) in enumerate(zip(lens, firsts)):
        total = first + n
        k = rnd(total, G, hd, seed=10 + r).to(torch.bfloat16)
        v = rnd(total, G, hd, seed=20 + r).to(torch.bfloat16)
        q = rnd(total, H, hd, seed=30 + r, scale=2.0).to(torch.bfloat16)
        for t in range(total):
            cache[tables[r][t // page], 0, :, t % page] = k[t]
            cache[tables[r][t // page], 1, :, t % page] = v[t]
        refs.append(P.sink_attention(q, k, v, 0.3, window)[first:])
        kept.append((q, k, v))
        qs.append(q[first:].reshape(n, H * hd))
    q = torch.cat(qs).to(DEV)
    out = torch.empty_like(q)
    rows = K().mma_tokens_per_tile(H, G)
    te, t0 = [], []
    for r, n in enumerate(lens):
        for a in range(0, n, rows):
            te.append(r)
            t0.append(a)
    bt = torch.zeros(2, 5, dtype=torch.int32)
    for r in range(2):
        bt[r, : len(tables[r])] = torch.tensor(tables[r])
    K().attention_prefill_bf16(q, out, cache.to(DEV), bt.to(DEV), i32([0, lens[0], sum(lens)]),
                               i32([f + n for f, n in zip(firsts, lens)]), i32(te), i32(t0), H, G, hd, 0.3, window,
                               precise=True, sink=True)
    ref = torch.cat([x.reshape(x.shape[0], H * hd) for x in refs])
    assert float((out.cpu().to(F64) - ref).abs().max()) <= 2.0 ** -8 * float(ref.abs().max()) * 1.01
    # the test can tell: without the sink the same rows are further away than that
    nosink = torch.cat([P.sink_attention(*kv, 0.3, window, sink=False)[f:].reshape(-1, H * hd) for kv, f in zip(kept, firsts)])
    assert float((nosink - ref).abs().max()) > 0.05 * float(ref.abs().max())


@pytest.mark.parametrize("E,top,groups", [(8, 3, (4, 2)), (6, 2, None), (64, 8, (8, 4)), (3, 3, None), (40, 5, (40, 7)),
                                          (16, 4, (4, 4))])
def test_router_choice(E, top, groups):
    T = 200
    z = rnd(T, E, seed=E, scale=2.0)
    corr = rnd(E, seed=E + 1, scale=0.6) - 0.4                            # choice scores go negative
    ids = torch.empty((T, top), dtype=torch.int32, device=DEV)
    wts = torch.empty((T, top), dtype=torch.float32, device=DEV)
    counts = torch.zeros(E, dtype=torch.int32, device=DEV)
    K().moe_route(z.to(DEV), corr.to(DEV), top, groups[0] if groups else 0, groups[1] if groups else 0, False, ids, wts, counts)
    r = {"experts": E, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    chosen, weight = P.route(z.to(F64), {"router": torch.eye(E, dtype=F64), "correction": corr.to(F64)}, r)
    got = ids.cpu().long()
    assert torch.equal(got.sort(dim=1).values, chosen.sort(dim=1).values)
    assert torch.equal(got, chosen)                                       # in the order of their choice scores
    assert rel_err(wts, weight) < 1e-6
    assert torch.equal(counts.cpu().long(), torch.bincount(chosen.reshape(-1), minlength=E))
    # the same from the router's input: the kernel forms the logits itself, in fp32 from a bf16 input
    d = 83
    x = rnd(T, d, seed=7).to(torch.bfloat16)
    rw = rnd(E, d, seed=8, scale=0.5)
    counts.zero_()
    K().moe_route(None, corr.to(DEV), top, groups[0] if groups else 0, groups[1] if groups else 0, False, ids, wts, counts,
                  x=x.to(DEV), router=rw.to(DEV))
    chosen, weight = P.route(x.to(F64), {"router": rw.to(F64), "correction": corr.to(F64)}, r)
    same = (ids.cpu().long().sort(dim=1).values == chosen.sort(dim=1).values).all(dim=1)
    assert float(same.double().mean()) > 0.97                   # a close call may fall the other way in fp32
    assert rel_err(wts[same.to(DEV)], weight[same]) < 1e-5


@pytest.mark.parametrize("T,E,top,d,ff", [(150, 8, 3, 96, 40), (5, 6, 2, 83, 24), (700, 4, 1, 64, 72), (1, 3, 3, 64, 20),
                                          (600, 5, 2, 320, 136)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_sort_products_and_sum(T, E, top, d, ff, dtype):
    """Pairs sorted by expert keep their order; every row meets its own expert's matrices; the weighted sum comes
    back per token; the counters are left at zero.  Some experts get no token, some many."""
    g = torch.Generator().manual_seed(T + E)
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)])
    if E > 3:
        ids[ids == 1] = 0 if top == 1 else ids[ids == 1]                  # an expert without tokens where that keeps rows distinct
    wts = torch.rand(T, top, generator=g)
    x = rnd(T, d, seed=1).to(dtype)
    gate_up = (rnd(E, 2 * ff, d, seed=2) / math.sqrt(d)).to(dtype)
    down = (rnd(E, d, ff, seed=3) / math.sqrt(ff)).to(dtype)
    shared = rnd(T, d, seed=4)
    N = T * top
    counts = torch.bincount(ids.reshape(-1), minlength=E).to(torch.int32).to(DEV)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    order = torch.empty(N, dtype=torch.int32, device=DEV)
    place = torch.empty(N, dtype=torch.int32, device=DEV)
    ids32 = ids.to(torch.int32).to(DEV)
    K().moe_sort(ids32, counts, offsets, order, place)
    flat = ids.reshape(-1)
    want_order = torch.sort(flat, stable=True).indices
    assert torch.equal(order.cpu().long(), want_order)
    assert torch.equal(place.cpu().long()[want_order], torch.arange(N))
    assert offsets.cpu().tolist() == [0] + torch.cumsum(torch.bincount(flat, minlength=E), 0).tolist()
    mid = torch.empty((N, ff), dtype=dtype, device=DEV)
    laced = torch.stack([gate_up[:, :ff], gate_up[:, ff:]], dim=2).reshape(E, 2 * ff, d).contiguous()   # gate_j, up_j, ...
    K().moe_product(x.to(DEV), laced.to(DEV), mid, offsets, order, top, gated=True)
    Y = torch.empty((N, d), dtype=torch.float32, device=DEV)
    K().moe_product(mid, down.to(DEV), Y, offsets, None, top, gated=False)
    if dtype == torch.bfloat16 and d % 8 == 0 and ff % 8 == 0:
        # the same on tcgen05: rows gathered into expert order, tiles of 128 rows, groups that end inside a tile
        xs = torch.empty((N, d), dtype=dtype, device=DEV)
        K().moe_gather(x.to(DEV), order, top, xs)
        assert torch.equal(xs.cpu(), x[order.cpu().long() // top])
        mid2 = torch.full((N, ff), float("nan"), dtype=dtype, device=DEV)
        K().gemm_tc_grouped(xs, laced.to(DEV), mid2, offsets, K().EPI_SILU)
        Y2 = torch.full((N, d), float("nan"), dtype=torch.float32, device=DEV)
        K().gemm_tc_grouped(mid2, down.to(DEV), Y2, offsets, K().EPI_F32)
        torch.cuda.synchronize()
        assert K().gemm_tc_error(torch.device(DEV)) == 0
        assert rel_err(mid2, mid) < 1e-2 and rel_err(Y2, Y) < 1e-2
    out = torch.empty((T, d), dtype=torch.float32, device=DEV)
    K().moe_combine(Y, place, wts.to(DEV), shared.to(DEV), out, counts)
    assert int(counts.abs().sum()) == 0
    ref = shared.to(F64).clone()
    xf, gu, dn = x.to(F64), gate_up.to(F64), down.to(F64)
    mids = {}
    for t in range(T):
        for j in range(top):
            e = int(ids[t, j])
            m = P.silu(gu[e, :ff] @ xf[t]) * (gu[e, ff:] @ xf[t])
            mids[(t, j)] = m
            ref[t] += float(wts[t, j]) * (dn[e] @ (m.to(dtype).to(F64)))
    got_mid = mid.cpu().to(F64)[place.cpu().long()].view(T, top, ff)
    want_mid = torch.stack([torch.stack([mids[(t, j)] for j in range(top)]) for t in range(T)])
    assert rel_err(got_mid, want_mid) < (2e-6 if dtype == torch.float32 else 1e-2)
    assert rel_err(out, ref) < (3e-6 if dtype == torch.float32 else 2e-3)


def test_grouped_products_follow_the_sort():
    """The tcgen05 products find their tiles in offsets that the sort before them writes, in buffers that are used
    again step after step: launched back to back (every kernel may start while its predecessor drains), each round's
    products must see that round's offsets and no earlier ones."""
    T, E, top, d, ff = 400, 6, 2, 128, 64
    g = torch.Generator().manual_seed(3)
    x = rnd(T, d, seed=1).to(torch.bfloat16).to(DEV)
    laced = (rnd(E, 2 * ff, d, seed=2) / math.sqrt(d)).to(torch.bfloat16).to(DEV)
    down = (rnd(E, d, ff, seed=3) / math.sqrt(ff)).to(torch.bfloat16).to(DEV)
    N = T * top
    offsets = torch.zeros(E + 1, dtype=torch.int32, device=DEV)
    order = torch.zeros(N, dtype=torch.int32, device=DEV)
    place = torch.zeros(N, dtype=torch.int32, device=DEV)
    xs = torch.empty((N, d), dtype=torch.bfloat16, device=DEV)
    rounds = []
    for r in range(6):
        # very uneven and different every round: most pairs on one expert, which moves
        ids = torch.full((T, top), r % E, dtype=torch.int64)
        ids[:, 1] = (r + 1 + torch.randint(0, E - 1, (T,), generator=g)) % E
        ids[torch.rand(T, generator=g) < 0.3, 0] = (r + 3) % E
        rounds.append(ids)
    outs, refs = [], []
    for ids in rounds:
        counts = torch.bincount(ids.reshape(-1), minlength=E).to(torch.int32).to(DEV)
        K().moe_sort(ids.to(torch.int32).to(DEV), counts, offsets, order, place)
        K().moe_gather(x, order, top, xs)
        mid = torch.empty((N, ff), dtype=torch.bfloat16, device=DEV)
        K().gemm_tc_grouped(xs, laced, mid, offsets, K().EPI_SILU)
        Y = torch.empty((N, d), dtype=torch.float32, device=DEV)
        K().gemm_tc_grouped(mid, down, Y, offsets, K().EPI_F32)
        outs.append((Y, place.clone()))
    torch.cuda.synchronize()
    assert K().gemm_tc_error(torch.device(DEV)) == 0
    for ids, (Y, pl) in zip(rounds, outs):
        counts = torch.bincount(ids.reshape(-1), minlength=E).to(torch.int32).to(DEV)
        o2, or2, pl2 = torch.empty_like(offsets), torch.empty_like(order), torch.empty_like(place)
        K().moe_sort(ids.to(torch.int32).to(DEV), counts, o2, or2, pl2)
        mid = torch.empty((N, ff), dtype=torch.bfloat16, device=DEV)
        K().moe_product(x, laced, mid, o2, or2, top, gated=True)
        want = torch.empty((N, d), dtype=torch.float32, device=DEV)
        K().moe_product(mid, down, want, o2, None, top, gated=False)
        torch.cuda.synchronize()
        assert torch.equal(pl, pl2)
        assert rel_err(Y, want) < 1e-2


# ============================================================================ the engine
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("pikalix")
    out = {}
    for n in NAMES:
        folder = make_sharp_model(str(root / n), n, seed=31 + ord(n))
        out[n] = (folder, Plain(folder))
    return out


def close(got, ref, dtype):
    """Whether engine logits match the plain model's.  In 32-bit every row is held.  In bfloat16 nine rows of
    ten are: where two experts' choice scores lie closer than the rounding of the router's input, the engine
    may take the other expert, which changes that row by more than rounding does (the 32-bit engine and the
    router test above hold the choice itself)."""
    if dtype == "float32":
        return rel_err(got, ref) <= TOL[dtype]
    got, ref = got.double().cpu(), ref.double().cpu()
    rows = (got - ref).abs().amax(dim=1) / ref.abs().max()
    return float((rows <= TOL[dtype]).double().mean()) >= 0.9 and float(rows.median()) <= TOL[dtype] / 2


def runner(folder, dtype, max_tokens=512, page=16, seqs=4, pages=None, capture=None):
    from rustinfer_b200.engine.runner import ModelRunner
    return ModelRunner(folder, dtype=dtype, max_model_len=max_tokens, page_size=page,
                       num_pages=pages if pages is not None else max_tokens // page,
                       max_batch_seqs=seqs, max_batch_tokens=max_tokens, capture_sizes=capture)


def run_cuts(r, rid, ids, cuts):
    from rustinfer_b200.engine.runner import StepEntry
    r.open(rid)
    outs, at = [], 0
    for c in cuts:
        outs.append(r.step([StepEntry(rid, ids[at: at + c], list(range(c)))]))
        at += c
    assert at == len(ids)
    r.close(rid)
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_layers_one_by_one(models, name, dtype):
    """The sum of the streams after every layer against the plain model's."""
    from rustinfer_b200.engine.runner import StepEntry
    from rustinfer_b200.parts import hyper
    folder, plain = models[name]
    ids = random_ids(50, CONFIGS[name]["vocab"], 7)
    want = []
    P.forward(plain.cfg, plain.w, ids, want)
    r = runner(folder, dtype)
    taps = []
    r.model.layer_tap = lambda i, hidden: taps.append(hyper.stream_sum(hidden).cpu())
    r.open("a")
    r.step([StepEntry("a", ids, [0])])
    assert len(taps) == len(want)
    for i, (g, w) in enumerate(zip(taps, want)):
        assert close(g, w, dtype), i


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_tail_and_portions(models, name, dtype):
    folder, plain = models[name]
    V = CONFIGS[name]["vocab"]
    r = runner(folder, dtype, page=8 if name == "Q" else 16)
    for n, seed in [(130, 1), (61, 2), (1, 3), (3, 4)]:
        ids = random_ids(n, V, seed)
        ref = plain.logits(ids)
        assert close(run_cuts(r, "w", ids, [n]), ref, dtype)                   # the first tokens included
        if n < 40:
            continue
        tail = run_cuts(r, "t", ids, [n - 45] + [1] * 45)                      # windows pass over decoded tokens
        assert close(tail, ref, dtype)
        cuts, left, sizes = [], n, [2, 7, 1, 16, 2, 33, 24, 5, 2, 64]
        while left:
            c = min(sizes[len(cuts) % len(sizes)], left)
            cuts.append(c)
            left -= c
        assert close(run_cuts(r, "p", ids, cuts), ref, dtype)
        assert close(run_cuts(r, "two", ids[:40], [2] * 20), ref[:40], dtype)
        assert close(run_cuts(r, "one", ids[:40], [1] * 40), ref[:40], dtype)  # token by token from the start
    r.cache.check_invariants()
    torch.cuda.synchronize()
    r.check_kernel_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_batches_reuse_pages_and_slots(models, name, dtype):
    """Three state slots and a pool that holds far less than the requests' sum: requests come and go, portions
    of prompts run beside single tokens, and every request's logits are those it has alone."""
    from rustinfer_b200.engine.runner import StepEntry
    folder, plain = models[name]
    V = CONFIGS[name]["vocab"]
    r = runner(folder, dtype, max_tokens=256, page=16, seqs=3, pages=20)
    lens = {"a": 150, "b": 37, "c": 90, "d": 2, "e": 120, "f": 64}
    ids = {k: random_ids(n, V, 100 + i) for i, (k, n) in enumerate(lens.items())}
    at = {k: 0 for k in ids}
    got = {k: [] for k in ids}
    waiting = list(ids)
    live = []
    portion = {"a": [33, 1, 1, 50, 2], "b": [5, 1, 1], "c": [64, 1, 25], "d": [1], "e": [2, 100, 1], "f": [16, 47, 1]}
    turn = 0
    while waiting or live:
        while waiting and len(live) < 3:
            k = waiting.pop(0)
            r.open(k)
            live.append(k)
        entries = []
        for k in live:
            if (turn + ord(k)) % 4 == 3 and len(live) > 1 and len(entries) + 1 < len(live):
                continue                                         # a request sits a step out now and then
            plan = portion[k]
            n = min(plan[min(len(got[k]), len(plan) - 1)], lens[k] - at[k])
            entries.append(StepEntry(k, ids[k][at[k]: at[k] + n], list(range(n))))
        if not entries:
            turn += 1
            continue
        lg = r.step(entries)
        row = 0
        for e in entries:
            n = len(e.tokens)
            got[e.request_id].append(lg[row: row + n])
            row += n
            at[e.request_id] += n
            if at[e.request_id] == lens[e.request_id]:
                r.close(e.request_id)
                live.remove(e.request_id)
        r.cache.check_invariants()
        turn += 1
    for k in ids:
        assert close(torch.cat(got[k]), plain.logits(ids[k]), dtype), k
    torch.cuda.synchronize()
    r.check_kernel_errors()


def test_fp32_logits_do_not_depend_on_the_cut(models):
    """Attention, the experts' products and the stream sums add in an order that the cut does not change."""
    folder, _ = models["P"]
    r = runner(folder, "float32")
    ids = random_ids(90, CONFIGS["P"]["vocab"], 9)
    whole = run_cuts(r, "w", ids, [90])
    assert torch.equal(run_cuts(r, "p", ids, [31, 2, 1, 24, 32]), whole)
    assert torch.equal(run_cuts(r, "t", ids, [60] + [1] * 30), whole)


@pytest.mark.parametrize("name", ["P", "Q"])
def test_long_decoding_and_graphs(models, name):
    """300 single tokens after a short prompt, eager and from captured steps: windows pass, their pages are
    given back (the pool is smaller than the sequence where every layer has a window), and the logits stay
    those of the plain model."""
    from rustinfer_b200.engine.runner import StepEntry
    folder, plain = models[name]
    ids = random_ids(310, CONFIGS[name]["vocab"], 5)
    ref = plain.logits(ids)
    for capture in (None, [1, 2]):
        r = runner(folder, "float32", max_tokens=320, page=16, seqs=2, pages=20 if name == "P" else 9, capture=capture)
        r.open("a")
        out = [r.step([StepEntry("a", ids[:10], list(range(10)))])]
        for t in range(10, 310):
            out.append(r.step([StepEntry("a", ids[t: t + 1], [0])]))
        assert rel_err(torch.cat(out), ref) <= TOL["float32"]
        if capture:
            assert r.graph_replays == 300
        r.close("a")
        r.cache.check_invariants()


@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_engine(models, name):
    """`Engine.generate`: scheduler, chunked prefill, continuous batching, device argmax, decode graphs."""
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.sampling.params import SamplingParams
    folder, plain = models[name]
    V = CONFIGS[name]["vocab"]
    prompts = [random_ids(n, V, 50 + n) for n in (45, 3, 70, 1, 26)]
    want = [plain.greedy(p, 12) for p in prompts]
    eng = Engine(folder, dtype="float32", max_batch_seqs=3, max_model_len=128, paged_block_size=16,
                 num_blocks=24, max_batch_tokens=64, chunked_prefill_size=32)
    got = [res.tokens for res in eng.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))]
    assert got == want
    eng16 = Engine(folder, dtype="bfloat16", max_batch_seqs=3, max_model_len=128, paged_block_size=16,
                   num_blocks=24, max_batch_tokens=64, chunked_prefill_size=32)
    got16 = [res.tokens for res in eng16.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))]
    same = sum(a == b for g, w in zip(got16, want) for a, b in zip(g, w))
    assert same >= 0.5 * 12 * len(prompts), (got16, want)


def test_trace_replay_command(models, tmp_path):
    folder, plain = models["Q"]
    V = CONFIGS["Q"]["vocab"]
    a, b = random_ids(70, V, 1), random_ids(20, V, 2)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:33], "want": [0, 32]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[33:69], "want": []}, {"id": "b", "tokens": b[:19], "want": [18]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[19:], "want": [0]}, {"id": "a", "tokens": a[69:], "want": [0]}], "end": ["a", "b"]},
    ]
    out = tmp_path / "out"
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    import numpy as np
    ra, rb = plain.logits(a), plain.logits(b)
    g0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4")).view(2, V)
    assert rel_err(g0, ra[[0, 32]]) <= TOL["float32"]
    g1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4")).view(1, V)
    assert rel_err(g1, rb[[18]]) <= TOL["float32"]
    g2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4")).view(2, V)
    assert rel_err(g2, torch.stack([rb[19], ra[69]])) <= TOL["float32"]


def test_command_line_and_sampler_serve_a_pikalix_folder(models, tmp_path):
    """`bin/rustinfer --config run.toml` on a Pikalix folder: greedy tokens are the plain model's.  Through `Engine`
    with temperature, top-k and top-p: a seeded request gives the same tokens twice, and every drawn token is among
    the most likely at its place."""
    import sys
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.sampling.params import SamplingParams
    folder, plain = models["R"]
    V = CONFIGS["R"]["vocab"]
    prompt = random_ids(21, V, 8)
    (tmp_path / "run.toml").write_text(f"""
model = "{folder}"
dtype = "float32"
max_batch_tokens = 64
max_batch_seqs = 3
max_model_len = 96
paged_block_size = 16
chunked_prefill_size = 8
num_blocks = 18
ignore_eos = true
capture_sizes = [1, 2, 4]

[sampling]
temperature = 0.0
max_tokens = 7

[[request]]
prompt_ids = {prompt}

[[request]]
prompt_ids = {prompt[:5]}
""")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "rustinfer"), "--config", str(tmp_path / "run.toml")],
                       capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-3000:]
    lines = [json.loads(l) for l in p.stdout.splitlines() if l.strip()]
    assert [l["request"] for l in lines] == [0, 1]
    assert lines[0]["tokens"] == plain.greedy(prompt, 7) and lines[1]["tokens"] == plain.greedy(prompt[:5], 7)
    eng = Engine(folder, dtype="float32", max_batch_seqs=3, max_model_len=96, paged_block_size=16, num_blocks=18,
                 max_batch_tokens=64, chunked_prefill_size=8)
    sp = SamplingParams(temperature=0.9, top_k=12, top_p=0.8, seed=11, max_tokens=7, ignore_eos=True)
    first = [r.tokens for r in eng.generate([prompt[:5], prompt], sp)]
    again = [r.tokens for r in eng.generate([prompt[:5], prompt], sp)]
    assert first == again and all(len(t) == 7 for t in first)
    ids = list(prompt[:5])
    for tok in first[0]:
        assert tok in torch.topk(plain.logits(ids)[-1], 12).indices.tolist()
        ids.append(tok)
