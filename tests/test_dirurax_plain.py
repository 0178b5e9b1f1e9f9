"""No GPU: the plain Dirurax model's mechanisms against closed forms and against other ways to
write them, and the framework's host side for this family (configuration, registry, declared
tensors, cache layout, pages given back as a block of positions passes, random-weights mode)."""
import json
import math
import os

import pytest
import torch

import plain_dirurax as P
from dirurax_helpers import CONFIGS, config_json, make_sharp_model, tensor_shapes

F64 = torch.float64


def rnd(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=F64)


# ------------------------------------------------------------------- the plain model itself
def test_sinusoid_entries():
    s = P.sinusoid_positions([0, 1, 7, 1000], 10)
    assert torch.equal(s[0], torch.tensor([0, 1] * 5, dtype=F64))
    assert abs(float(s[2, 0]) - math.sin(7.0)) < 1e-15 and abs(float(s[2, 1]) - math.cos(7.0)) < 1e-15
    f = 10000.0 ** (-2.0 * 3 / 10)
    assert abs(float(s[3, 6]) - math.sin(1000 * f)) < 1e-12 and abs(float(s[3, 7]) - math.cos(1000 * f)) < 1e-12
    odd = P.sinusoid_positions([3], 7)                  # an odd width ends on a sine
    assert odd.shape == (1, 7) and abs(float(odd[0, 6]) - math.sin(3 * 10000.0 ** (-6.0 / 7))) < 1e-15


def test_norms_and_activations_against_torch():
    x, w, b = rnd(5, 12), rnd(12, seed=1), rnd(12, seed=2)
    ref = torch.nn.functional.layer_norm(x, (12,), w, b, eps=1e-3)
    assert torch.allclose(P.layer_norm(x, w, b, 1e-3), ref, atol=1e-13)
    assert torch.allclose(P.gelu_erf(x), torch.nn.functional.gelu(x), atol=1e-14)
    r = P.rms_divide(x, 0.0)
    assert torch.allclose((r * r).mean(-1), torch.ones(5, dtype=F64), atol=1e-13)
    big = P.rms_divide(torch.zeros(1, 4, dtype=F64), 1e-6)      # eps sits inside the root
    assert torch.equal(big, torch.zeros(1, 4, dtype=F64))


def test_gated_scan_closed_form():
    """o_t = sum_{s<=t} (prod_{s<u<=t} alpha_u * k_s) . q_t  v_s."""
    T, H, dk, dv = 9, 2, 3, 4
    q, k, v = rnd(T, H, dk), rnd(T, H, dk, seed=1), rnd(T, H, dv, seed=2)
    alpha = torch.sigmoid(rnd(T, H, dk, seed=3))
    o = P.gla_scan(q, k, v, alpha)
    for t in (0, 4, 8):
        want = torch.zeros(H, dv, dtype=F64)
        for s in range(t + 1):
            decay = torch.ones(H, dk, dtype=F64)
            for u in range(s + 1, t + 1):
                decay = decay * alpha[u]
            want += ((decay * k[s] * q[t]).sum(-1))[:, None] * v[s]
        assert torch.allclose(o[t], want, atol=1e-12)


def test_delta_scan_as_matrices():
    """Per head S_t = (diag(w) - (a*u) u^T) S_{t-1} + k v^T with both terms on the old state."""
    T, d = 7, 5
    r, k, v = rnd(T, 1, d), rnd(T, 1, d, seed=1), rnd(T, 1, d, seed=2)
    w, a = torch.sigmoid(rnd(T, 1, d, seed=3)), torch.sigmoid(rnd(T, 1, d, seed=4))
    o = P.delta_scan(r, k, v, w, a)
    S = torch.zeros(d, d, dtype=F64)
    for t in range(T):
        u = k[t, 0] / torch.sqrt((k[t, 0] ** 2).sum() + 1e-6)
        S = (torch.diag(w[t, 0]) - torch.outer(a[t, 0] * u, u)) @ S + torch.outer(k[t, 0], v[t, 0])
        assert torch.allclose(o[t, 0], S.T @ r[t, 0], atol=1e-12)
    # removal rate 1 and no decay: writing the same unit key twice leaves only the second value
    k1 = torch.zeros(2, 1, d, dtype=F64); k1[:, 0, 2] = 1.0
    vals = rnd(2, 1, d, seed=5)
    one = torch.ones(2, 1, d, dtype=F64)
    out = P.delta_scan(k1, k1, vals, one, one)
    assert torch.allclose(out[1, 0], vals[1, 0], atol=1e-5)


def test_block_attention_sees_its_own_block_only():
    T, H, G, d, dv, block = 23, 4, 2, 6, 3, 5
    q, k, v = rnd(T, H, d), rnd(T, G, d, seed=1), rnd(T, G, dv, seed=2)
    o = P.block_attention(q, k, v, 0.7, block)
    for i in (0, 4, 5, 9, 10, 22):
        lo = i // block * block
        for h in (0, 3):
            g = h // (H // G)
            s = torch.softmax((k[lo:i + 1, g] @ q[i, h]) * 0.7, dim=0)
            assert torch.allclose(o[i, h], s @ v[lo:i + 1, g], atol=1e-13)
    assert torch.allclose(o[5, 0], v[5, 0], atol=1e-13)           # the first position of a block sees itself alone
    # a prompt that starts in the middle of a block still counts blocks from position 0
    part = P.block_attention(q[7:], k[7:], v[7:], 0.7, block, pos0=7)
    assert torch.allclose(part[3:], o[10:], atol=1e-13)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_plain_model_prefix_property(name, tmp_path):
    """Logits at position t do not depend on later tokens; the stream has one entry per layer."""
    folder = make_sharp_model(str(tmp_path / name), name, seed=3)
    cfg, w = P.read_model_folder(folder)
    ids = [(7 * i + 3) % cfg["vocab"] for i in range(40)]
    full = P.forward_logits(cfg, w, ids)
    assert torch.allclose(P.forward_logits(cfg, w, ids[:17]), full[:17], atol=1e-10)
    assert len(P.forward_layers(cfg, w, ids[:5])) == len(cfg["layers"]) + 1


# ----------------------------------------------------------------- the framework's host side
def test_config_registry_and_declared_tensors():
    from rustinfer_b200.config.dirurax_config import DiruraxConfig
    from rustinfer_b200.config.model_config import ConfigError
    from rustinfer_b200.config.registry import resolve_architecture
    from rustinfer_b200.models.decoder import Decoder
    for name in CONFIGS:
        raw = config_json(name)
        fam = resolve_architecture(raw)
        assert fam.name == "dirurax"
        typed = fam.parse_config(raw, None)
        assert isinstance(typed, DiruraxConfig) and typed.to_dict() == raw
        decls = Decoder(fam.model_spec(typed)).param_decls()
        want = tensor_shapes(name)
        assert set(want) <= set(decls) and all(decls[n].optional for n in set(decls) - set(want))
        for n, shape in want.items():
            assert all(a == b or a == -1 for a, b in zip(decls[n].shape, shape)), n
    bad = config_json("X")
    bad["layers"][0]["mixer"]["left"]["mask"] = {"span": 3}
    with pytest.raises(ConfigError), pytest.warns(UserWarning, match="span"):
        resolve_architecture(bad).parse_config(bad, None)
    bad = config_json("X")
    bad["layers"][1]["type"] = "mamba"
    with pytest.raises(ConfigError):
        resolve_architecture(bad).parse_config(bad, None)
    bad = config_json("X")
    bad["layers"][1]["mlp"]["kind"] = "experts"
    with pytest.raises(ConfigError):
        resolve_architecture(bad).parse_config(bad, None)
    odd = config_json("Z")
    odd["layers"][0]["mixer"]["note"] = "a key nobody reads"
    with pytest.warns(UserWarning, match="note"):
        resolve_architecture(odd).parse_config(odd, None)


def test_cache_layout_of_mixed_layers():
    """A layer with attention beside a recurrence holds a page group and a state group; layers of
    one kind and size share a group; a model without attention has no page pool."""
    from rustinfer_b200.cache.manager import CacheLayout, CacheManager
    from rustinfer_b200.config.registry import resolve_architecture
    from rustinfer_b200.models.decoder import Decoder
    from rustinfer_b200.parts.base import FixedState, PagedKV

    def layout(name):
        raw = config_json(name)
        fam = resolve_architecture(raw)
        return CacheLayout.from_needs(Decoder(fam.model_spec(fam.parse_config(raw, None))).cache_needs())

    lx = layout("X")
    assert isinstance(lx.entry_cache[0], list) and len(lx.entry_cache[0]) == 2
    kinds = [type(lx.groups[g].need) for g, _ in lx.entry_cache[0]]
    assert kinds == [PagedKV, FixedState]
    need = lx.groups[lx.entry_cache[0][0][0]].need
    assert (need.head_dim, need.v_dim, need.block, need.window) == (16, 24, 24, None)
    assert lx.groups[lx.entry_cache[0][1][0]].need.shape == (3, 20, 32)      # 20 key channels kept as 4 lanes of 8
    assert len(lx.paged_groups()) == 1
    ly = layout("Y")
    assert len(ly.paged_groups()) == 2                 # two attentions of different sizes
    lz = layout("Z")
    assert lz.paged_groups() == []
    m = CacheManager(lz, [], 16, 2)
    m.open("a")
    with m.lease([("a", 40)]):
        pass
    assert m.length("a") == 40
    m.close("a")
    m.check_invariants()


def test_pages_of_passed_blocks_are_given_back():
    from rustinfer_b200.cache.manager import CacheLayout, CacheManager
    from rustinfer_b200.parts.base import PagedKV
    lay = CacheLayout.from_needs([(0, PagedKV(1, 8, None, value_dim=4, block=24), None)])
    m = CacheManager(lay, [6], 8, 2)
    m.open("a")
    held = []
    for n in (5, 18, 1, 1, 30, 1, 17, 24):              # lengths 5, 23, 24, 25, 55, 56, 73, 97
        with m.lease([("a", n)]):
            pass
        length = m.length("a")
        first = (length // 24 * 24) // 8               # page of the first key the next token sees
        table = m.block_table("a", 0)
        assert all(p == -1 for p in table[:first]) and all(p >= 0 for p in table[first:])
        held.append(m.pages_held("a")[0])
        m.check_invariants()
    assert max(held) <= 4 and m.length("a") == 97       # 97 tokens went through a pool of 6 pages of 8
    m.close("a")
    assert m.free_pages()[0] == 6


def test_random_weights_mode(tmp_path):
    from rustinfer_b200.weights.random_init import write_random_model
    from rustinfer_b200.weights.safetensors_io import SafetensorsReader
    folder = write_random_model(str(tmp_path / "m"), config_json("Y"), seed=5, std=0.1, norm_std=0.1)
    with open(os.path.join(folder, "config.json")) as f:
        assert json.load(f)["layers"] == config_json("Y")["layers"]
    r = SafetensorsReader(folder)
    assert tuple(r.shape("l1.mix.right.w2"))[0] == 2 * 64 and "head.weight" not in r.names()
    cfg, w = P.read_model_folder(folder)
    assert torch.isfinite(P.forward_logits(cfg, w, [1, 2, 3])).all()
