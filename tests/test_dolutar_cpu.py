"""Dolutar without a GPU: configuration, tensor names, what the cache manager is asked for and
how it keeps a window's first pages, and the plain implementation against itself."""

from __future__ import annotations

import pytest
import torch

import dolutar_configs as dc
import dolutar_plain as plain
from mlx_omnia_b200.cache.manager import CacheManager
from mlx_omnia_b200.config.hydrate import ConfigError
from mlx_omnia_b200.parts.base import KVSpec
from mlx_omnia_b200.parts.model import CacheNeed, DecoderModel
from mlx_omnia_b200.registry import resolve_architecture

F64 = torch.float64


def _model(name):
    raw = dc.config(name)
    architecture = resolve_architecture(raw)
    return raw, architecture, DecoderModel(architecture.model_spec(architecture.parse(raw)))


@pytest.mark.parametrize("name", sorted(dc.CONFIGS))
def test_tensor_names_and_shapes(name):
    raw, architecture, model = _model(name)
    wanted = {k: tuple(v.shape) for k, v in model.tensors().items()}
    drawn = {architecture.tensor_name(k): tuple(t.shape) for k, t in dc.tensors(name).items()}
    assert wanted == drawn
    for i, layer in enumerate(raw["layers"]):
        reads = layer["mixer"].get("kv_from") is not None
        assert (f"l{i}.mix.k" in wanted) != reads and (f"l{i}.mix.k.norm" in wanted) != reads
        assert f"l{i}.mix.sink" in wanted and f"l{i}.mix.q.b" in wanted
        assert (f"l{i}.norm2.weight" in wanted) == (layer["mlp"] is not None)


def test_a_reader_widens_its_owners_cache():
    _, _, model = _model("P")
    needs = model.cache_needs()
    assert needs[1].kv is None and needs[1].reads == 0
    assert needs[0].kv == KVSpec(((2, 16), (2, 24)), 11, keep_first=3)  # the owner's window is the wider one
    assert needs[2].kv == KVSpec(((1, 24), (1, 8)), 19, keep_first=0)
    assert model.model_state() is not None and "prev" in model.model_state()
    raw = dc.config("P")
    raw["layers"][1]["mixer"]["mask"] = {"size": 40, "keep_first": 9}
    architecture = resolve_architecture(raw)
    widened = DecoderModel(architecture.model_spec(architecture.parse(raw))).cache_needs()[0].kv
    assert (widened.window, widened.keep_first) == (40, 9)


def test_configuration_errors_are_named():
    for change, text in [(lambda r: r["layers"][1]["mixer"].update(kv_from=1), "does not run before"),
                         (lambda r: r["layers"][0].update(type="conv"), "unknown type"),
                         (lambda r: r["layers"][0]["mlp"].update(kind="sparse"), "unknown kind"),
                         (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
                         (lambda r: r["layers"][0]["mixer"].pop("vdim"), "lacks the key 'vdim'"),
                         (lambda r: r["layers"][2]["mixer"].update(kv_from=1), "none of its own"),
                         (lambda r: r["layers"][3]["mixer"].update(kv_from=0), "differ in key/value sizes")]:
        raw = dc.config("P")
        change(raw)
        with pytest.raises(ConfigError, match=text):
            resolve_architecture(raw).parse(raw)


def test_pages_of_the_first_positions_outlive_the_window():
    spec = KVSpec(((1, 8), (1, 8)), window=10, keep_first=5)
    cache = CacheManager([CacheNeed(spec, None, None)], page_size=4, pages_per_group=16, max_requests=2, allocate=False)
    request = cache.open("a")
    cache.grow(request, 30)
    cache.release_behind_window(request)
    # positions 0..4 live in pages 0 and 1; positions below 30 - 10 + 1 = 21 are dead: pages 2, 3, 4
    assert request.tables[0][:2] == [0, 1] and request.tables[0][2:5] == [-1, -1, -1] and request.tables[0][5] >= 0
    cache.grow(request, 9)
    cache.release_behind_window(request)
    assert request.tables[0][:2] == [0, 1] and all(p < 0 for p in request.tables[0][2:7]) and request.tables[0][7] >= 0
    cache.check()
    cache.close("a")
    assert cache.groups[0].pool.free == 16
    with pytest.raises(ValueError):
        KVSpec(((1, 8), (1, 8)), window=None, keep_first=2)


def test_visibility_rule():
    see = plain.visible(12, 4, 2)
    assert see[9].tolist() == [True, True, False, False, False, False, True, True, True, True, False, False]
    assert see[3].tolist()[:5] == [True, True, True, True, False]
    assert plain.visible(5, 9, 0).tolist() == torch.ones(5, 5).tril().bool().tolist()


def test_the_sink_only_takes_weight():
    """With a sink of minus infinity the attention is an ordinary softmax; a large sink empties the output."""
    raw, W = dc.config("Q"), dc.tensors("Q")
    m, p = raw["layers"][1]["mixer"], "l1.mix."
    h = torch.randn(9, raw["width"], dtype=F64)
    kv = plain.keys_and_values(h, W, p, m, 1e-6)
    W = dict(W)
    W[p + "sink"] = torch.full((m["heads"],), -1e30)
    without = plain.attention(h, W, p, m, 1e-6, kv)
    W[p + "sink"] = torch.full((m["heads"],), 60.0)
    assert plain.attention(h, W, p, m, 1e-6, kv).abs().max() < 1e-12 * without.abs().max()
    W[p + "sink"] = torch.zeros(m["heads"])
    # one key of score s and a sink of 0: the key's weight is e^s / (e^s + 1)
    q = (h[:1] @ W[p + "q"].double().T + W[p + "q.b"].double()).view(1, m["heads"], m["dim"])
    q = plain.rotate(plain.rms(q, 1e-6, W[p + "q.norm"].double()), torch.arange(1), m["rot"]["dims"], m["rot"]["base"])
    s = (q[0, 0] * kv[0][0, 0]).sum() * m["scale"]
    want = torch.sigmoid(s) * kv[1][0, 0]
    W2 = dict(W)
    W2[p + "o"] = torch.eye(m["heads"] * m["vdim"])  # heads * vdim equals the width here: the heads come out as they are
    out = plain.attention(h[:1], W2, p, m, 1e-6, (kv[0][:1], kv[1][:1]))
    assert torch.allclose(out[0, : m["vdim"]], want, atol=1e-12)


def test_identity_experts_and_unnormalised_weights():
    raw, W = dc.config("P"), dc.tensors("P")
    router, p = raw["layers"][1]["mlp"]["router"], "l1.mlp."
    h = torch.randn(40, raw["width"], dtype=F64)
    chosen, weights = plain.route(h, W, p, router["top"])
    assert chosen.shape == (40, 2) and (chosen >= router["experts"]).any() and (chosen < router["experts"]).any()
    assert (weights.sum(-1) < 1.0).all()  # scores of all outputs sum to one; the chosen ones to less
    W2 = dict(W)
    W2[p + "correction"] = torch.tensor([0.0] * router["experts"] + [9.0] * router["identity"])
    y = plain.moe_ff(h, W2, p, router)  # every token is sent to the two identity experts
    s = torch.softmax(h @ W[p + "router"].double().T, -1)[:, router["experts"]:].sum(-1, keepdim=True)
    assert torch.allclose(y, s * h, atol=1e-12)


def test_clamped_unit():
    W = {"m.gate": torch.eye(3), "m.up": torch.eye(3), "m.down": torch.eye(3)}
    h = torch.tensor([[5.0, -5.0, 0.5]], dtype=F64)
    y = plain.dense_ff(h, W, "m.", 2.0)
    want = [2.0 * torch.sigmoid(torch.tensor(1.702 * 2.0)) * 3.0, -5.0 * torch.sigmoid(torch.tensor(1.702 * -5.0)) * -1.0,
            0.5 * torch.sigmoid(torch.tensor(1.702 * 0.5)) * 1.5]
    assert torch.allclose(y[0], torch.stack(want).double(), atol=1e-12)


def test_pair_rows():
    raw, W = dc.config("P"), dc.tensors("P")
    tokens = [5, 150, 5, 5]
    x = plain.embedding(tokens, W, raw, F64)
    e = raw["embedding"]
    rows = [61, (5 * 13 + 150 * 5) % 61, (150 * 13 + 5 * 5) % 61, (5 * 13 + 5 * 5) % 61]
    want = W["embed"].double()[tokens] * e["scale"] + W["bigram"].double()[rows]
    assert torch.equal(x, want)


@pytest.mark.parametrize("name", sorted(dc.CONFIGS))
def test_a_prefix_of_a_sequence_gives_the_same_logits(name):
    """Causality of the whole plain model: a longer sequence does not change earlier positions."""
    raw, W = dc.config(name), dc.tensors(name)
    tokens = dc.prompt(60, raw["vocab"], 1)
    full = plain.forward(tokens, W, raw)
    assert torch.allclose(plain.forward(tokens[:23], W, raw), full[:23], atol=1e-9, rtol=1e-9)
