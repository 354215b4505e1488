"""Dolutar as configuration, parts and tensor names.

A decoder of attention layers only, each with a sliding window that keeps the request's first
positions visible, a softmax sink per head, biased projections, weighted per-head norms of queries
and keys and a rotation of part of the head; a layer may have no key/value tensors and read an
earlier layer's cache instead (`kv_from`). Norms sit on the branches' outputs only, the branches read
the residual itself. The feed-forward is a clamped gated unit or a routed mixture of small experts
(some of them identity experts without tensors). The embedding adds a hashed row for the pair
(token before, token); the logits are scaled. Everything here is data for the generic engine.

config.json keys: `architecture` ("Dolutar"), `vocab`, `width`, `logit_scale`, `norm.eps`,
`embedding.scale`, `embedding.bigram` {buckets, mul_prev, mul_cur}, and `layers`: a list of
{`type`: "attention", `mixer` {heads, kv_heads, dim, vdim, scale, rot {base, dims}, mask {size,
keep_first}, kv_from?}, `mlp`: null | {kind: "dense", ff, limit} | {kind: "moe", expert {ff}, router
{experts, identity, top}}}.
Tensor names: `embed`, `bigram`, `head`, `final.norm`, and per layer i `l<i>.norm1`, `l<i>.norm2`,
`l<i>.mix.q|k|v` (+ `.b`, and `.norm` for q and k), `l<i>.mix.sink`, `l<i>.mix.o`, `l<i>.mlp.gate|up|down`
or `l<i>.mlp.router`, `l<i>.mlp.correction`, `l<i>.mlp.e<j>.gate|up|down`.
"""

from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Any

import torch

from mlx_omnia_b200.config.hydrate import ConfigError
from mlx_omnia_b200.parts.base import PartSpec
from mlx_omnia_b200.parts.model import LayerSpec, ModelSpec, ScheduleEntry
from mlx_omnia_b200.registry import Architecture, register_architecture

GLU_SLOPE = 1.702  # of the sigmoid in the dense feed-forward's gated unit


@dataclass(frozen=True)
class DolutarMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float
    window: int | None  # None: every earlier position is visible
    keep_first: int
    kv_from: int | None


@dataclass(frozen=True)
class DolutarFeedForward:
    kind: str  # "dense" or "moe"
    ff: int
    limit: float = 0.0  # dense
    experts: int = 0  # moe: experts with tensors
    identity: int = 0
    top: int = 0


@dataclass(frozen=True)
class DolutarConfig:
    vocab: int
    width: int
    embedding_scale: float
    bigram: tuple[int, int, int] | None  # (buckets, mul_prev, mul_cur)
    norm_eps: float
    logit_scale: float
    mixers: tuple[DolutarMixer, ...]
    feed_forwards: tuple[DolutarFeedForward | None, ...]


def _need(raw: dict, key: str, where: str):
    if not isinstance(raw, dict) or key not in raw:
        raise ConfigError(f"Dolutar: {where} lacks the key {key!r}")
    return raw[key]


def _mixer(raw: dict, where: str, index: int) -> DolutarMixer:
    rot = _need(raw, "rot", where)
    mask = raw.get("mask")
    kv_from = raw.get("kv_from")
    if kv_from is not None and not 0 <= int(kv_from) < index:
        raise ConfigError(f"Dolutar: {where}.kv_from names layer {kv_from}, which does not run before layer {index}")
    heads, kv_heads = int(_need(raw, "heads", where)), int(_need(raw, "kv_heads", where))
    if kv_heads < 1 or heads % kv_heads:
        raise ConfigError(f"Dolutar: {where}: {heads} heads do not divide into {kv_heads} key/value heads")
    dim = int(_need(raw, "dim", where))
    dims = int(_need(rot, "dims", where + ".rot"))
    if dims % 2 or not 0 <= dims <= dim:
        raise ConfigError(f"Dolutar: {where}.rot.dims must be even and at most dim = {dim}, got {dims}")
    return DolutarMixer(heads, kv_heads, dim, int(_need(raw, "vdim", where)), float(_need(raw, "scale", where)), dims,
                        float(_need(rot, "base", where + ".rot")),
                        None if mask is None else int(_need(mask, "size", where + ".mask")),
                        0 if mask is None else int(mask.get("keep_first", 0)),
                        None if kv_from is None else int(kv_from))


def _feed_forward(raw: dict | None, where: str) -> DolutarFeedForward | None:
    if raw is None:
        return None
    kind = _need(raw, "kind", where)
    if kind == "dense":
        return DolutarFeedForward("dense", int(_need(raw, "ff", where)), limit=float(_need(raw, "limit", where)))
    if kind == "moe":
        router = _need(raw, "router", where)
        return DolutarFeedForward("moe", int(_need(_need(raw, "expert", where), "ff", where + ".expert")),
                                  experts=int(_need(router, "experts", where + ".router")),
                                  identity=int(router.get("identity", 0)), top=int(_need(router, "top", where + ".router")))
    raise ConfigError(f"Dolutar: {where} has the unknown kind {kind!r}")


def parse(raw: dict[str, Any]) -> DolutarConfig:
    if raw.get("architecture") != "Dolutar":
        raise ConfigError(f"expected architecture 'Dolutar', got {raw.get('architecture')!r}")
    mixers, feed_forwards = [], []
    for index, layer in enumerate(_need(raw, "layers", "config.json")):
        where = f"layers[{index}]"
        if _need(layer, "type", where) != "attention":
            raise ConfigError(f"Dolutar: {where} has the unknown type {layer['type']!r}")
        mixers.append(_mixer(_need(layer, "mixer", where), where + ".mixer", index))
        feed_forwards.append(_feed_forward(layer.get("mlp"), where + ".mlp"))
    if not mixers:
        raise ConfigError("Dolutar: no layers")
    for index, mixer in enumerate(mixers):
        if mixer.kv_from is None:
            continue
        owner = mixers[mixer.kv_from]
        if owner.kv_from is not None:
            raise ConfigError(f"Dolutar: layers[{index}] reads the cache of layer {mixer.kv_from}, which has none of its own")
        if (owner.kv_heads, owner.dim, owner.vdim) != (mixer.kv_heads, mixer.dim, mixer.vdim):
            raise ConfigError(f"Dolutar: layers[{index}] and the layer whose cache it reads differ in key/value sizes")
    embedding = raw.get("embedding", {})
    bigram = embedding.get("bigram")
    if bigram is not None:
        bigram = (int(_need(bigram, "buckets", "embedding.bigram")), int(_need(bigram, "mul_prev", "embedding.bigram")),
                  int(_need(bigram, "mul_cur", "embedding.bigram")))
    return DolutarConfig(vocab=int(_need(raw, "vocab", "config.json")), width=int(_need(raw, "width", "config.json")),
                         embedding_scale=float(embedding.get("scale", 1.0)), bigram=bigram,
                         norm_eps=float(_need(_need(raw, "norm", "config.json"), "eps", "norm")),
                         logit_scale=float(raw.get("logit_scale", 1.0)), mixers=tuple(mixers),
                         feed_forwards=tuple(feed_forwards))


def _norm(config: DolutarConfig) -> PartSpec:
    return PartSpec("rms_norm", {"size": config.width, "eps": config.norm_eps, "weight": "plain"})


def model_spec(config: DolutarConfig) -> ModelSpec:
    layers = []
    for index, (m, f) in enumerate(zip(config.mixers, config.feed_forwards)):
        position = PartSpec("rotary", {"dims": m.rot_dims, "theta": m.rot_base}) if m.rot_dims else None
        mixer = PartSpec("sink_window_attention", {
            "hidden": config.width, "heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim,
            "scale": m.scale, "window": m.window, "keep_first": m.keep_first, "norm_eps": config.norm_eps,
            "position": position, "bias": True, "sink": True, "own_kv": m.kv_from is None})
        if f is None:
            feed_forward = None
        elif f.kind == "dense":
            feed_forward = PartSpec("clamped_glu_mlp", {"hidden": config.width, "inner": f.ff, "limit": f.limit,
                                                        "alpha": GLU_SLOPE})
        else:
            feed_forward = PartSpec("routed_experts", {"hidden": config.width, "inner": f.ff, "experts": f.experts,
                                                       "identity": f.identity, "top": f.top})
        norms = {"norm1": _norm(config)} if feed_forward is None else {"norm1": _norm(config), "norm2": _norm(config)}
        layers.append(LayerSpec(PartSpec("branch_norm", {"mixer": mixer, "feed_forward": feed_forward, "norms": norms}),
                                f"l{index}"))
    if config.bigram is not None:
        buckets, mul_prev, mul_cur = config.bigram
        embedding = PartSpec("pair_hash_embedding", {"vocab": config.vocab, "hidden": config.width, "buckets": buckets,
                                                     "mul_prev": mul_prev, "mul_cur": mul_cur,
                                                     "scale": config.embedding_scale})
    else:
        embedding = PartSpec("token_embedding", {"vocab": config.vocab, "hidden": config.width,
                                                 "scale": config.embedding_scale})
    return ModelSpec(
        embedding=embedding,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i, m.kv_from) for i, m in enumerate(config.mixers)),
        final_norm=_norm(config),
        head=PartSpec("lm_head", {"vocab": config.vocab, "hidden": config.width, "multiplier": config.logit_scale}),
        embedding_prefix="embed", final_norm_prefix="final.norm", head_prefix="head",
    )


_WEIGHT_SUFFIXED = re.compile(r"^(embed|head|final\.norm|l\d+\.norm[12])$")


def tensor_name(file_name: str) -> str:
    """The file's names are the model's, but for the parts that call their one tensor `weight` and
    for the pair table, which belongs to the embedding."""
    if file_name == "bigram":
        return "embed.pairs"
    return file_name + ".weight" if _WEIGHT_SUFFIXED.match(file_name) else file_name


def random_tensors(config: DolutarConfig, seed: int) -> dict[str, torch.Tensor]:
    """Float32 tensors under the checkpoint's names, drawn on the CPU in a fixed order from one
    generator: matrices N(0, gain / sqrt(fan_in)), norm weights 1 + N(0, 0.1), biases, sinks and
    router corrections of a size at which each of them matters."""
    g = torch.Generator().manual_seed(seed)

    def normal(*shape: int, std: float = 1.0) -> torch.Tensor:
        return torch.randn(*shape, generator=g, dtype=torch.float32) * std

    def matrix(rows: int, cols: int, gain: float = 1.0) -> torch.Tensor:
        return normal(rows, cols, std=gain * cols ** -0.5)

    D = config.width
    out = {"embed": normal(config.vocab, D, std=1.0 / max(config.embedding_scale, 1e-6))}
    if config.bigram is not None:
        out["bigram"] = normal(config.bigram[0] + 1, D, std=0.5)
    for i, (m, f) in enumerate(zip(config.mixers, config.feed_forwards)):
        p = f"l{i}."
        out[p + "norm1"] = 1.0 + normal(D, std=0.1)
        names = [("q", m.heads * m.dim)]
        if m.kv_from is None:
            names += [("k", m.kv_heads * m.dim), ("v", m.kv_heads * m.vdim)]
        for name, rows in names:
            out[p + f"mix.{name}"] = matrix(rows, D, gain=2.0)
            out[p + f"mix.{name}.b"] = normal(rows, std=0.3)
            if name != "v":
                out[p + f"mix.{name}.norm"] = 1.0 + normal(m.dim, std=0.2)
        out[p + "mix.sink"] = normal(m.heads, std=1.0)
        out[p + "mix.o"] = matrix(D, m.heads * m.vdim)
        if f is None:
            continue
        out[p + "norm2"] = 1.0 + normal(D, std=0.1)
        if f.kind == "dense":
            out[p + "mlp.gate"], out[p + "mlp.up"] = matrix(f.ff, D, gain=2.0), matrix(f.ff, D, gain=2.0)
            out[p + "mlp.down"] = matrix(D, f.ff)
        else:
            for e in range(f.experts):
                out[p + f"mlp.e{e}.gate"], out[p + f"mlp.e{e}.up"] = matrix(f.ff, D, gain=2.0), matrix(f.ff, D, gain=2.0)
                out[p + f"mlp.e{e}.down"] = matrix(D, f.ff)
            out[p + "mlp.router"] = matrix(f.experts + f.identity, D, gain=2.0)
            out[p + "mlp.correction"] = normal(f.experts + f.identity, std=0.05)
    out["final.norm"] = 1.0 + normal(D, std=0.1)
    out["head"] = matrix(config.vocab, D)
    return out


ARCHITECTURE = Architecture(
    name="dolutar",
    config_class=DolutarConfig,
    parse=parse,
    model_spec=model_spec,
    tensor_name=tensor_name,
    random_tensors=random_tensors,
)

register_architecture(ARCHITECTURE, "Dolutar", "dolutar")
