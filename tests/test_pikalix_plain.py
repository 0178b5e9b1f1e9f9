"""The Pikalix family without a GPU: the plain implementation's mechanisms against closed forms, the
configuration reader, the registry, declared tensors, the cache layout of layers that share keys, the
random-weights mode."""
import json
import math

import pytest
import torch

import plain_pikalix as P
from pikalix_helpers import CONFIGS, tensor_shapes

F64 = torch.float64


def rnd(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=F64)


# ------------------------------------------------------------------- the plain mechanisms
def test_sink_softmax_weights_sum_to_less_than_one():
    """With one key of score s the weight is e^s / (1 + e^s): 1/2 at s = 0; without the sink it is 1."""
    q = torch.zeros(1, 1, 4, dtype=F64)
    k = rnd(1, 1, 4)
    v = torch.ones(1, 1, 3, dtype=F64)
    assert torch.allclose(P.sink_attention(q, k, v, 1.0, None), torch.full((1, 1, 3), 0.5, dtype=F64))
    assert torch.allclose(P.sink_attention(q, k, v, 1.0, None, sink=False), torch.ones(1, 1, 3, dtype=F64))
    q = k.clone()
    s = float((k * k).sum())
    assert torch.allclose(P.sink_attention(q, k, v, 1.0, None), torch.full((1, 1, 3), math.exp(s) / (1 + math.exp(s)), dtype=F64))


def test_window_keeps_exactly_its_size():
    """Query i sees i - w + 1 .. i: a value placed w - 1 back is seen, w back is not."""
    T, w = 12, 5
    q, k = torch.zeros(T, 1, 2, dtype=F64), torch.zeros(T, 1, 2, dtype=F64)
    for back, seen in ((w - 1, True), (w, False)):
        v = torch.zeros(T, 1, 1, dtype=F64)
        v[T - 1 - back] = 1.0
        out = P.sink_attention(q, k, v, 1.0, w)[T - 1, 0, 0]
        assert (float(out) > 0) == seen
        if seen:
            assert abs(float(out) - 1.0 / (1 + w)) < 1e-12          # w keys of weight 1 and the sink


def test_rotation_turns_pairs_and_leaves_the_rest():
    x = rnd(6, 2, 10)
    pos = torch.arange(6) * 7
    y = P.rotate_pairs(x, pos, 4, 100.0)
    assert torch.equal(y[..., 4:], x[..., 4:])
    assert torch.allclose(y[..., 0] ** 2 + y[..., 1] ** 2, x[..., 0] ** 2 + x[..., 1] ** 2)
    a = pos.to(F64) * 100.0 ** (-2.0 / 4)                              # pair 1 turns by p * base^(-2/4)
    assert torch.allclose(y[:, 0, 2], x[:, 0, 2] * torch.cos(a) - x[:, 0, 3] * torch.sin(a))
    # relative: the product of a rotated query and key depends on the distance only
    q, k = rnd(1, 1, 4, seed=1), rnd(1, 1, 4, seed=2)
    d1 = (P.rotate_pairs(q, torch.tensor([9]), 4, 50.0) * P.rotate_pairs(k, torch.tensor([4]), 4, 50.0)).sum()
    d2 = (P.rotate_pairs(q, torch.tensor([105]), 4, 50.0) * P.rotate_pairs(k, torch.tensor([100]), 4, 50.0)).sum()
    assert abs(float(d1 - d2)) < 1e-9


def test_router_groups_by_hand():
    """Eight experts in four groups of two, two groups kept, three experts used.  Choice scores (sigmoid of
    the logit plus the correction) are set so that the best single expert sits in a group that loses."""
    z = torch.tensor([[2.0, -9.0, 1.0, 1.0, 0.5, 0.9, -9.0, -9.0]], dtype=F64)
    w = {"router": torch.eye(8, dtype=F64), "correction": torch.zeros(8, dtype=F64)}
    r = {"experts": 8, "top": 3, "groups": {"count": 4, "keep": 2}}
    chosen, weight = P.route(z, w, r)
    # group sums: (0,1) .88, (2,3) 1.46, (4,5) 1.33, (6,7) ~0: groups 1 and 2 are kept, expert 0 is not eligible
    assert sorted(chosen[0].tolist()) == [2, 3, 5]
    assert torch.allclose(weight[0].sort().values, torch.sigmoid(torch.tensor([0.9, 1.0, 1.0], dtype=F64)))
    # the correction moves the choice but not the weights
    w["correction"] = torch.tensor([5.0, 5.0, 0, 0, 0, 0, 0, 0], dtype=F64)
    chosen, weight = P.route(z, w, r)
    assert set(chosen[0].tolist()) >= {0, 1}
    assert abs(float(weight[0][chosen[0].tolist().index(1)]) - 1.0 / (1.0 + math.exp(9.0))) < 1e-12
    # negative choice scores: experts outside the kept groups lose to negative ones inside
    w["correction"] = torch.tensor([-3.0, -3.0, -2.0, -2.5, -2.2, -2.7, 0.0, 0.0], dtype=F64)
    z2 = torch.full((1, 8), -20.0, dtype=F64)
    r2 = {"experts": 8, "top": 4, "groups": {"count": 4, "keep": 2}}
    chosen, _ = P.route(z2, w, r2)
    assert sorted(chosen[0].tolist()) == [2, 3, 6, 7]               # groups 3 (sum 0) and 1 (-4.5) win


def test_streams_reduce_to_the_residual_sum():
    X = [rnd(5, 7)]
    fn = lambda u: u * 2.0 + 1.0
    one = torch.ones(1, dtype=F64)
    (Y,) = P.connected(X, one, one.view(1, 1), one, fn)
    assert torch.allclose(Y, X[0] + fn(X[0]))
    # every stream from the old ones at once
    X = [rnd(3, 4, seed=1), rnd(3, 4, seed=2)]
    a, b = torch.tensor([0.5, -1.0], dtype=F64), torch.tensor([2.0, 0.0], dtype=F64)
    M = torch.tensor([[0.0, 1.0], [1.0, 0.0]], dtype=F64)              # the streams swap
    Y = P.connected(X, a, M, b, lambda u: u)
    assert torch.allclose(Y[0], X[1] + 2.0 * (0.5 * X[0] - X[1]))
    assert torch.allclose(Y[1], X[0])


def test_gelu_and_norm():
    z = rnd(100)
    assert torch.allclose(P.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"))
    x, w = rnd(4, 9), rnd(9, seed=1)
    assert torch.allclose(P.rms_norm(x, w, 0.5), x / torch.sqrt((x ** 2).mean(-1, keepdim=True) + 0.5) * w)


# --------------------------------------------------------------------- configuration, registry
def test_registry_and_declared_tensors():
    import rustinfer_b200  # noqa: F401
    from rustinfer_b200.config.registry import resolve_architecture
    from rustinfer_b200.models.decoder import Decoder
    for name, cfg in CONFIGS.items():
        fam = resolve_architecture(cfg)
        assert fam.name == "pikalix"
        typed = fam.parse_config(cfg, None)
        assert typed.to_dict() == cfg
        spec = fam.model_spec(typed)
        decls = Decoder(spec).param_decls()
        want = tensor_shapes(name)
        assert {n: tuple(d.shape) for n, d in decls.items()} == want
        assert [e.cache_of for e in spec.run_order] == [l["mixer"].get("kv_from") for l in cfg["layers"]]


def test_cache_layout_of_shared_keys():
    """A layer that reads another's keys owns no cache; the owner's cache keeps the widest window among its
    readers (every key as soon as one of them sees every key)."""
    import rustinfer_b200  # noqa: F401
    from rustinfer_b200.cache.manager import CacheLayout
    from rustinfer_b200.config.registry import resolve_architecture
    from rustinfer_b200.models.decoder import Decoder
    fam = resolve_architecture(CONFIGS["P"])
    dec = Decoder(fam.model_spec(fam.parse_config(CONFIGS["P"], None)))
    needs = dec.cache_needs()
    assert needs[0][1].window == 37 and needs[2][1].window is None
    assert dec.blocks[0].mixer.window == 20 and dec.blocks[1].mixer.window == 37 and dec.blocks[3].mixer.window == 50
    layout = CacheLayout.from_needs(needs)
    assert len(layout.groups) == 2 and layout.entry_writes == [True, False, True, False]
    assert layout.entry_cache[1] == layout.entry_cache[0] and layout.entry_cache[3] == layout.entry_cache[2]


@pytest.mark.parametrize("change,needle", [
    (lambda c: c["layers"][0].__setitem__("type", "gla"), "mixer type"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "glu"), "feed-forward kind"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 1), "reads the keys"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 2), "reads the keys"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("dim", 32), "head sizes differ"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("count", 3), "groups.count"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 5), "fewer experts"),
    (lambda c: c.__setitem__("streams", 0), "streams"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configuration_errors(change, needle):
    from rustinfer_b200.config.model_config import ConfigError
    from rustinfer_b200.config.pikalix_config import PikalixConfig
    cfg = json.loads(json.dumps(CONFIGS["P"]))
    change(cfg)
    with pytest.raises(ConfigError, match=needle):
        PikalixConfig.from_dict(cfg)


def test_unknown_keys_are_named():
    from rustinfer_b200.config.pikalix_config import PikalixConfig
    cfg = json.loads(json.dumps(CONFIGS["R"]))
    cfg["layers"][0]["mixer"]["taper"] = 3
    with pytest.warns(UserWarning, match="taper"):
        PikalixConfig.from_dict(cfg)


def test_random_weights_mode(tmp_path):
    import rustinfer_b200  # noqa: F401
    from rustinfer_b200.weights.random_init import write_random_model
    folder = write_random_model(str(tmp_path / "m"), CONFIGS["P"], seed=3, norm_std=0.1)
    cfg, w = P.read_model_folder(folder)
    assert {n: tuple(t.shape) for n, t in w.items()} == tensor_shapes("P")
    assert cfg["streams"] == 3 and cfg["layers"][1]["mixer"]["kv_from"] == 0
    mix = w["l0.hc1.mix"].float()
    assert float((mix - torch.eye(3)).abs().max()) < 0.6 and float(mix.diagonal().mean()) > 0.6
    logits = P.forward(cfg, w, [1, 5, 9, 200])
    assert logits.shape == (4, 211) and bool(torch.isfinite(logits).all())
