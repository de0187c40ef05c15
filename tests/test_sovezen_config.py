"""Sovezen without a GPU: the configuration and its checks, the model description (parts, run order, tensor names),
the cache layout of one-plane pages, and properties of the plain implementation that the GPU tests lean on."""
import copy
import math

import pytest
import torch

import plain_sovezen as plain
from sovezen_models import CONFIGS, make_weights, owner, tensor_shapes

from sandyrt_b200.config.base import ConfigError, config_from_normalised
from sandyrt_b200.config.sovezen import SovezenConfig


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_description_names_every_tensor_with_its_shape(name):
    from sandyrt_b200.models.model import build_model

    cfg = config_from_normalised(CONFIGS[name])
    assert isinstance(cfg, SovezenConfig) and cfg.vocab_size == CONFIGS[name]["vocab"]
    cfg.validate()
    got = {k: list(v.shape) for k, v in build_model(cfg).tensor_requests().items()}
    assert got == tensor_shapes(CONFIGS[name])


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_run_order_and_shared_tensors(name):
    """A layer that uses another layer's tensors is a second call of that layer's parts, with a cache entry of its own."""
    from sandyrt_b200.models.model import describe

    raw = CONFIGS[name]
    spec = describe(config_from_normalised(raw))
    owners = [owner(raw, i) for i in range(len(raw["layers"]))]
    own = sorted(set(owners))
    assert len(spec.layers) == len(own)
    assert [c.layer for c in spec.schedule] == [own.index(o) for o in owners]
    assert [c.cache for c in spec.schedule] == list(range(len(raw["layers"])))
    assert spec.max_positions is None and not spec.remixes
    for l, i in zip(spec.layers, own):
        src = raw["layers"][i]
        assert l.block == "parallel_branches" and l.mixer.kind == "latent_attention"
        assert l.feed_forward.kind == {None: "none", "dense": "gated_mlp", "moe": "routed_experts"}[src["mlp"] and src["mlp"]["kind"]]
        assert sorted(l.norms) == (["feed_forward_scale", "input", "mixer_scale"] if src["mlp"] else ["input", "mixer_scale"])
    assert spec.head.params["tied"] is True and spec.head.params["logit_scale"] == raw["logit_scale"]


def test_config_round_trip_and_constants_reach_the_parts():
    from sandyrt_b200.models.model import describe

    raw = CONFIGS["B"]
    cfg = SovezenConfig.from_dict(raw)
    assert SovezenConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.to_dict()["layers"] == raw["layers"]
    spec = describe(cfg)
    p, m = spec.layers[0].mixer.params, raw["layers"][0]["mixer"]
    assert (p["n_heads"], p["qk_dim"], p["rot_dim"], p["v_dim"], p["kv_rank"], p["q_rank"]) == (1, 20, 6, 12, 20, 0)
    assert p["rot_dims"] == m["rot"]["dims"] == 4 and p["rot_base"] == m["rot"]["base"] and p["scale"] == m["scale"]
    assert p["sink"] is True and p["eps"] == raw["norm"]["eps"]
    q = spec.layers[1].mixer.params
    assert q["q_rank"] == 10 and q["rot_dim"] == 0 and q["sink"] is False
    f = spec.layers[2].feed_forward.params
    assert (f["n_experts"], f["top"], f["inner"]) == (3, 1, 20)


def _broken(path, value):
    raw = copy.deepcopy(CONFIGS["A"])
    node = raw
    for k in path[:-1]:
        node = node[k]
    if value is KeyError:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return raw


@pytest.mark.parametrize("path,value,message", [
    (("layers", 0, "type"), "attention", "unknown layer type"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "even"),
    (("layers", 0, "mixer", "rot", "dims"), 10, "at most"),
    (("layers", 0, "mixer", "kv_rank"), 640, "at most 640"),
    (("layers", 1, "mixer", "q_rank"), KeyError, "q_rank"),
    (("layers", 1, "mlp", "router", "top"), 9, "top"),
    (("layers", 1, "mlp", "kind"), "routed", "dense"),
    (("layers", 2, "weights_of"), 2, "another layer"),
    (("layers", 2, "weights_of"), 1, "that layer's type"),
    (("layers", 2, "mixer", "heads"), 3, "that layer's type"),
    (("logit_scale",), KeyError, "logit_scale"),
    (("norm",), KeyError, "norm"),
    (("layers", 4, "mixer", "vdim"), "8", "int"),
])
def test_configurations_that_are_refused(path, value, message):
    with pytest.raises(ConfigError, match=message):
        SovezenConfig.from_dict(_broken(path, value)).validate()


def test_one_plane_pages_have_groups_of_their_own():
    from sandyrt_b200.cache.pages import BlockAllocator, CacheLayout
    from sandyrt_b200.parts.base import PagedKVSpec

    one = PagedKVSpec(1, 32, planes=1)
    layout = CacheLayout.from_specs([one, PagedKVSpec(1, 32), one, PagedKVSpec(1, 64, planes=1)], 16)
    assert [g.caches for g in layout.groups] == [[0, 2], [1], [3]]
    al = BlockAllocator(layout, [4, 4, 4], max_requests=2)
    al.admit("a")
    al.reserve("a", 40)
    assert all(len(al.block_list("a", g)) == 3 for g in range(3))
    al.commit("a", 40)
    al.release("a")
    al.check()


# ---- the plain implementation --------------------------------------------------------------------------------
def test_plain_rotation_pairs_neighbours_and_keeps_lengths():
    x = torch.randn(5, 2, 10, dtype=torch.float64)
    pos = torch.tensor([0, 1, 7, 100, 1000])
    y = plain.rotate_pairs(x, pos, 6, 100.0)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 6:], x[..., 6:])
    for i in range(3):
        assert torch.allclose(y[..., 2 * i] ** 2 + y[..., 2 * i + 1] ** 2, x[..., 2 * i] ** 2 + x[..., 2 * i + 1] ** 2)
    a = 7 * 100.0 ** (-2.0 / 6)
    assert torch.allclose(y[2, 0, 2], x[2, 0, 2] * math.cos(a) - x[2, 0, 3] * math.sin(a))


def test_plain_sink_only_joins_the_denominator():
    q, k, v = (torch.randn(6, 2, 4, dtype=torch.float64) for _ in range(3))
    free = plain.causal_softmax_attention(q, k, v, 0.5, None)
    sunk = plain.causal_softmax_attention(q, k, v, 0.5, torch.tensor([-40.0, 0.3]))
    assert torch.allclose(sunk[:, 0], free[:, 0])
    s0 = float((q[0, 1] @ k[0, 1]) * 0.5)
    assert torch.allclose(sunk[0, 1], v[0, 1] * math.exp(s0) / (math.exp(s0) + math.exp(0.3)))


def test_plain_routing_weights_are_a_softmax_over_the_chosen():
    cfg = CONFIGS["B"]
    w = {k: v.to(torch.float64) for k, v in make_weights(cfg, 3).items()}
    h = torch.randn(4, cfg["width"], dtype=torch.float64)
    every = plain.routed_ff(cfg["layers"][0]["mlp"], w, "l0.mlp.", h)           # every expert chosen
    z = h @ w["l0.mlp.router"].t() + w["l0.mlp.router.b"]
    g = torch.softmax(z, -1)
    want = sum(g[:, e:e + 1] * (torch.relu(h @ w[f"l0.mlp.e{e}.up"].t()) ** 2 @ w[f"l0.mlp.e{e}.down"].t()) for e in range(5))
    assert torch.allclose(every, want)
    one = plain.routed_ff(cfg["layers"][2]["mlp"], w, "l2.mlp.", h)             # one expert: weight 1
    z = h @ w["l2.mlp.router"].t() + w["l2.mlp.router.b"]
    for t in range(4):
        e = int(z[t].argmax())
        assert torch.allclose(one[t], torch.relu(w[f"l2.mlp.e{e}.up"] @ h[t]) ** 2 @ w[f"l2.mlp.e{e}.down"].t())


def test_plain_model_is_causal_and_every_mechanism_matters():
    cfg = CONFIGS["A"]
    w = make_weights(cfg, 1)
    ids = list(range(3, 40))
    full = plain.forward(cfg, w, ids)
    assert torch.allclose(plain.forward(cfg, w, ids[:20]), full[:20])
    for name in ("l0.mix.sink", "l0.ls1", "l1.ls2", "l1.mlp.router.b", "l4.mix.dkv.norm", "l1.mix.dq.norm"):
        w2 = dict(w)
        w2[name] = w[name] + torch.linspace(0.5, 3.0, w[name].numel()).view_as(w[name])     # not a constant: a router ignores one
        assert (plain.forward(cfg, w2, ids) - full).abs().max() > 1e-3, name
    two, four = copy.deepcopy(cfg), copy.deepcopy(cfg)                        # the layers on shared tensors do run
    two["layers"], four["layers"] = cfg["layers"][:2], cfg["layers"][:4]
    assert (plain.forward(two, w, ids) - plain.forward(four, w, ids)).abs().max() > 1e-3
