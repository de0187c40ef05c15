"""Panupel without a GPU: the configuration and its checks, the model description (parts, run order, tensor
names), the cache layout of a mixer that wants pages and a state, and properties of the plain implementation
that the GPU tests lean on."""
import copy
import math

import pytest
import torch

import plain_panupel as plain
from panupel_models import CONFIGS, SCALING, tensor_shapes

from sandyrt_b200.config.base import ConfigError, config_from_normalised
from sandyrt_b200.config.panupel import PanupelConfig


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_description_names_every_tensor_with_its_shape(name):
    from sandyrt_b200.models.model import build_model

    cfg = config_from_normalised(CONFIGS[name])
    assert isinstance(cfg, PanupelConfig) and cfg.vocab_size == CONFIGS[name]["vocab"]
    cfg.validate()
    got = {k: list(v.shape) for k, v in build_model(cfg).tensor_requests().items()}
    assert got == tensor_shapes(CONFIGS[name])


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_run_order_follows_the_loop(name):
    from sandyrt_b200.models.model import describe

    raw = CONFIGS[name]
    spec = describe(config_from_normalised(raw))
    want = plain.run_order(raw)
    assert [c.layer for c in spec.schedule] == [i for i, _ in want]
    assert [c.remix is not None for c in spec.schedule] == [m for _, m in want]
    assert [c.cache for c in spec.schedule] == list(range(len(want)))          # every pass has a cache of its own
    assert len(spec.remixes) == (1 if raw.get("loop") else 0)
    assert spec.max_positions is None
    kinds = {"parallel": "attention_beside_matrix_memory", "delta": "gated_delta"}
    assert [l.mixer.kind for l in spec.layers] == [kinds[l["type"]] for l in raw["layers"]]
    assert [l.feed_forward.kind for l in spec.layers] == ["gated_mlp" if l["mlp"] else "none" for l in raw["layers"]]
    assert all(l.block == "sandwich_norm" and l.block_params["residual_mult"] == raw["residual_mult"] for l in spec.layers)


def test_config_round_trip_and_constants_reach_the_parts():
    from sandyrt_b200.models.model import describe

    raw = CONFIGS["A"]
    cfg = PanupelConfig.from_dict(raw)
    again = PanupelConfig.from_dict(cfg.to_dict())
    assert again == cfg
    spec = describe(cfg)
    p = spec.layers[1].mixer.params
    left = raw["layers"][1]["mixer"]["left"]
    assert p["left.rot_dims"] == left["rot"]["dims"] and p["left.rot_base"] == left["rot"]["base"]
    assert p["left.rot_scaling"] == SCALING and p["left.scale"] == left["scale"]
    assert p["right.gate_cap"] == raw["layers"][1]["mixer"]["right"]["gate_cap"] and p["eps"] == raw["norm"]["eps"]
    assert "left.rot_base" not in describe(PanupelConfig.from_dict(CONFIGS["C"])).layers[0].mixer.params   # no rotary there
    d = spec.layers[0].mixer.params
    assert (d["n_heads"], d["n_qk_heads"], d["qk_dim"], d["v_dim"], d["conv_taps"]) == (4, 2, 16, 8, 4)


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
    (("layers", 1, "mixer", "left", "kv_heads"), 3, "do not divide"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 7, "even"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 18, "at most"),
    (("layers", 0, "type"), "conv", "unknown layer type"),
    (("layers", 0, "mlp", "kind"), "routed", "dense"),
    (("layers", 0, "mixer", "conv"), 0, "taps"),
    (("layers", 1, "mixer", "right", "gate_cap"), 0.0, "gate_cap"),
    (("loop", "stop"), 9, "loop"),
    (("loop", "times"), 0, "times"),
    (("width",), KeyError, "width"),
    (("norm",), KeyError, "norm"),
    (("layers", 2, "mixer", "vdim"), "8", "int"),
])
def test_configurations_that_are_refused(path, value, message):
    with pytest.raises(ConfigError, match=message):
        PanupelConfig.from_dict(_broken(path, value)).validate()


def test_a_mixer_may_hold_pages_and_a_state():
    from sandyrt_b200.cache.pages import BlockAllocator, CacheLayout
    from sandyrt_b200.parts.base import PagedKVSpec, PagedStateSpec, StateSpec

    both = PagedStateSpec(2, 48, (1234,))
    layout = CacheLayout.from_specs([StateSpec((7,)), both, PagedKVSpec(2, 48), both, PagedKVSpec(2, 32)], 16)
    assert [g.caches for g in layout.groups] == [[1, 2, 3], [4]]           # equal page needs share a group, state or not
    assert sorted(layout.state_of_cache) == [0, 1, 3]
    al = BlockAllocator(layout, [4, 4], max_requests=2)
    al.admit("a")
    al.reserve("a", 40)
    assert len(al.block_list("a", 0)) == 3 and len(al.block_list("a", 1)) == 3
    al.commit("a", 40)
    al.release("a")
    al.check()


# ---- the plain implementation itself ---------------------------------------------------------------
def test_rotary_frequency_rescaling_has_three_regimes():
    base, dims = 100.0, 16
    plain_f = plain.rotary_frequencies(dims, base, None)
    assert plain_f == [base ** (-2.0 * i / dims) for i in range(8)]
    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    got = plain.rotary_frequencies(dims, base, sc)
    seen = set()
    for f, g in zip(plain_f, got):
        wavelength = 2 * math.pi / f
        if wavelength < 64 / 4.0:
            assert g == f
            seen.add("kept")
        elif wavelength > 64 / 1.0:
            assert g == f / 8.0
            seen.add("divided")
        else:
            assert f / 8.0 < g < f
            seen.add("blended")
    assert seen == {"kept", "divided", "blended"}


def test_a_sink_takes_weight_and_gives_nothing():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(9, 2, 4, generator=g, dtype=torch.float64) for _ in range(3))
    none = plain.sink_attention(q, k, v, 0.5, None)
    far = plain.sink_attention(q, k, v, 0.5, torch.tensor([-1e9, -1e9], dtype=torch.float64))
    assert torch.allclose(none, far)
    big = plain.sink_attention(q, k, v, 0.5, torch.tensor([0.0, 30.0], dtype=torch.float64))
    assert big[:, 1].abs().max() < 1e-6                  # head 1's weights all went to the sink
    # one key, score s: the weight is exp(s) / (exp(s) + exp(sink))
    s = (q[0, 0] @ k[0, 0]) * 0.5
    assert torch.allclose(big[0, 0], v[0, 0] * torch.exp(s) / (torch.exp(s) + 1.0))


def test_recurrences_carry_their_state_across_portions():
    g = torch.Generator().manual_seed(1)
    T, d, e = 23, 6, 5
    q, k = torch.randn(T, d, generator=g, dtype=torch.float64), torch.randn(T, d, generator=g, dtype=torch.float64)
    v = torch.randn(T, e, generator=g, dtype=torch.float64)
    a, b = torch.randn(T, generator=g, dtype=torch.float64), torch.randn(T, generator=g, dtype=torch.float64)
    whole, _ = plain.matrix_memory(q, k, v, a, plain.log_sigmoid(b + 2))
    part1, st = plain.matrix_memory(q[:9], k[:9], v[:9], a[:9], plain.log_sigmoid(b[:9] + 2))
    part2, _ = plain.matrix_memory(q[9:], k[9:], v[9:], a[9:], plain.log_sigmoid(b[9:] + 2), st)
    assert torch.allclose(torch.cat([part1, part2]), whole, atol=1e-12)
    kn = plain.unit(k)
    beta, decay = torch.sigmoid(a), torch.sigmoid(b + 2)
    whole, _ = plain.delta_rule(q, kn, v, beta, decay)
    part1, S = plain.delta_rule(q[:9], kn[:9], v[:9], beta[:9], decay[:9])
    part2, _ = plain.delta_rule(q[9:], kn[9:], v[9:], beta[9:], decay[9:], S)
    assert torch.allclose(torch.cat([part1, part2]), whole, atol=1e-12)
    # with beta = 1 and no decay, writing a unit key stores its value exactly: the read-out of the same key returns it
    S0 = torch.zeros(d, e, dtype=torch.float64)
    o, _ = plain.delta_rule(kn[:1], kn[:1], v[:1], torch.ones(1, dtype=torch.float64), torch.ones(1, dtype=torch.float64), S0)
    assert torch.allclose(o[0], v[0] * (kn[0] @ kn[0]))


def test_short_convolution_is_causal_and_ends_on_the_current_token():
    x = torch.arange(12, dtype=torch.float64).reshape(6, 2) + 1
    taps = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=torch.float64)
    y = plain.short_conv(x, taps)
    assert torch.equal(y[:, 0], x[:, 0])                                       # last column: the current token
    assert torch.equal(y[:, 1], torch.cat([torch.zeros(2, dtype=torch.float64), x[:-2, 1]]))   # first column: two tokens back
