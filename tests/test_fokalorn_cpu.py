"""Fokalorn without a GPU: configuration, tensor names, what the cache manager is asked for, and the
plain implementation's own consistency (its recurrences carried over a cut equal the uncut run)."""

from __future__ import annotations

import pytest
import torch

import fokalorn_configs
import fokalorn_plain as plain
from mlx_omnia_b200.cache import CacheManager
from mlx_omnia_b200.config.hydrate import ConfigError
from mlx_omnia_b200.parts.base import KVSpec
from mlx_omnia_b200.parts.model import DecoderModel
from mlx_omnia_b200.registry import resolve_architecture
from mlx_omnia_b200.weights.loader import DictSource


def build(name):
    raw = fokalorn_configs.config(name)
    architecture = resolve_architecture(raw)
    weights = fokalorn_configs.tensors(name)
    source = DictSource(weights)
    config = architecture.sizes_from_tensors(architecture.parse(raw),
                                             lambda n: source.shape(n) if n in weights else None)
    return raw, architecture, config, weights, DecoderModel(architecture.model_spec(config))


@pytest.mark.parametrize("name", ["X", "Y", "Z"])
def test_tensor_names_and_shapes_match_the_random_checkpoint(name):
    raw, architecture, config, weights, model = build(name)
    wanted = model.tensors()
    assert {architecture.tensor_name(k) for k in weights} == set(wanted)
    for k, t in weights.items():
        assert tuple(t.shape) == tuple(wanted[architecture.tensor_name(k)].shape), k


def test_schedule_and_cache_needs_follow_the_loop():
    raw, architecture, config, weights, model = build("X")
    assert config.schedule() == [0, 1, 2, 1, 2, 1, 2, 3] == plain.schedule(raw)
    needs = model.cache_needs()
    assert len(needs) == 8
    assert [n.kv for n in needs] == [KVSpec(((1, 48),)), None, None, None, None, None, None, KVSpec(((1, 64),))]
    assert needs[1].state["S"].shape == (4, 24, 40) and needs[1].state["conv"].shape == (3, 2 * 2 * 24 + 4 * 40)
    assert all(n.block_state["shift"].shape == (96,) for n in needs)
    cache = CacheManager(needs, page_size=4, pages_per_group=8, max_requests=3, device="cpu", dtype=torch.float32)
    # Every run of a looped layer has state of its own; a slot's state is cleared for a new request.
    assert cache.state[1]["S"].data_ptr() != cache.state[3]["S"].data_ptr()
    cache.state[3]["S"][1] = 5.0
    cache.block_state[0]["shift"][1] = 2.0
    cache.reset_slots([1])
    assert float(cache.state[3]["S"][1].abs().max()) == 0.0 and float(cache.block_state[0]["shift"][1].abs().max()) == 0.0


def test_sizes_that_only_tensors_give():
    raw = fokalorn_configs.config("X")
    for layer in raw["layers"]:
        layer["mixer"].pop("decay_rank", None), layer["mixer"].pop("gate_rank", None)
    architecture = resolve_architecture(raw)
    parsed = architecture.parse(raw)
    with pytest.raises(ConfigError):
        architecture.model_spec(parsed)
    weights = fokalorn_configs.tensors("X")
    del weights["l2.shift"]
    filled = architecture.sizes_from_tensors(parsed, lambda n: tuple(weights[n].shape) if n in weights else None)
    assert filled.layers[1].m("decay_rank") == 8 and filled.layers[1].m("gate_rank") == 12
    assert [layer.shift for layer in filled.layers] == [True, True, False, True]
    assert "l2.shift" not in DecoderModel(architecture.model_spec(filled)).tensors()


def test_bad_configurations_are_named():
    raw = fokalorn_configs.config("Y")
    raw["layers"][0]["type"] = "something_else"
    with pytest.raises(ConfigError, match="unknown type"):
        resolve_architecture(raw).parse(raw)
    raw = fokalorn_configs.config("X")
    raw["loop"]["stop"] = 9
    with pytest.raises(ConfigError, match="loop"):
        resolve_architecture(raw).parse(raw)
    raw = fokalorn_configs.config("X")
    del raw["layers"][3]["mixer"]["kv_rank"]
    with pytest.raises(ConfigError, match="kv_rank"):
        resolve_architecture(raw).parse(raw)


def test_plain_recurrences_carry_over_a_cut():
    g = torch.Generator().manual_seed(3)
    T, dk, dv = 11, 6, 5
    q, k = torch.randn(T, dk, generator=g, dtype=torch.float64), torch.randn(T, dk, generator=g, dtype=torch.float64)
    v, beta = torch.randn(T, dv, generator=g, dtype=torch.float64), torch.rand(T, generator=g, dtype=torch.float64)
    decay = torch.rand(T, dk, generator=g, dtype=torch.float64)
    whole, S = plain.delta_rule(q, k, v, beta, decay)
    first, S1 = plain.delta_rule(q[:4], k[:4], v[:4], beta[:4], decay[:4])
    second, S2 = plain.delta_rule(q[4:], k[4:], v[4:], beta[4:], decay[4:], S1)
    assert torch.allclose(torch.cat([first, second]), whole) and torch.allclose(S2, S)
    h, mu = torch.randn(T, 7, generator=g, dtype=torch.float64), torch.rand(7, generator=g, dtype=torch.float64)
    assert torch.allclose(torch.cat([plain.token_shift(h[:4], mu), plain.token_shift(h[4:], mu, h[3])]),
                          plain.token_shift(h, mu))
    # with a decay of one, beta of one and orthonormal keys the rule stores and returns values exactly
    eye = torch.eye(dk, dtype=torch.float64)
    out, _ = plain.delta_rule(eye[:dv], eye[:dv], v[:dv], torch.ones(dv, dtype=torch.float64),
                              torch.ones(dv, dk, dtype=torch.float64))
    assert torch.allclose(out, v[:dv])


def test_plain_rotation_and_grouped_norm():
    x = torch.arange(12, dtype=torch.float64).reshape(1, 12) + 1
    n = plain.grouped_rms_norm(x, torch.ones(12, dtype=torch.float64), 0.0, 3)
    assert torch.allclose(n.reshape(3, 4).pow(2).mean(-1), torch.ones(3, dtype=torch.float64))
    v = torch.tensor([[1.0, 0.0, 0.0, 2.0, 5.0, 6.0]], dtype=torch.float64)
    turned = plain.rotate_interleaved(v, torch.tensor([1]), 4, 1.0)  # both pairs by one radian
    c, s = torch.cos(torch.tensor(1.0, dtype=torch.float64)), torch.sin(torch.tensor(1.0, dtype=torch.float64))
    assert torch.allclose(turned, torch.stack([c, s, -2 * s, 2 * c, v[0, 4], v[0, 5]])[None])
