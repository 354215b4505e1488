"""Fokalorn as configuration, parts and tensor names.

A decoder whose layers alternate, in any order the configuration lists, between a recurrent mixer
(`channel_delta`: a gated delta rule with a decay per key channel behind short convolutions) and
an attention over a low-rank latent cache (`latent_attention`, with a softmax sink and a gate per
head). Around them: a scaled embedding, RMS norms taken in groups, a token shift in front of every
mixer, a residual kept as several streams (hyper-connections), a dense feed-forward with a squared
ReLU (a layer may have none), and a span of layers that runs several times with the same weights,
each run with a cache and state of its own. Everything here is data for the generic engine.

config.json keys: `architecture` ("Fokalorn"), `vocab`, `width`, `embedding.scale`, `norm.eps`,
`norm.groups`, `streams` (absent: one ordinary residual), `loop` {start, stop, times} (absent: none),
and `layers`: a list of {`type`, `mixer` {sizes}, `mlp` {`ff`, `kind`: "dense"} or null}.
Tensor names: `embed`, `head`, `final.norm`, and per layer i `l<i>.norm1`, `l<i>.norm2`,
`l<i>.shift`, `l<i>.hc<q>.in|out|mix`, `l<i>.mix.*`, `l<i>.mlp.up|down`.
Two inner widths (the ranks of the decay's and the output gate's low-rank maps) are in no key: they
are read from the shapes of `l<i>.mix.a1` and `l<i>.mix.g1`; a configuration may name them
(`decay_rank`, `gate_rank` in `mixer`) for the random-weights mode.
"""

from __future__ import annotations

import dataclasses
import re
from dataclasses import dataclass
from typing import Any, Callable

import torch

from mlx_omnia_b200.config.hydrate import ConfigError
from mlx_omnia_b200.parts.base import PartSpec
from mlx_omnia_b200.parts.model import LayerSpec, ModelSpec, ScheduleEntry
from mlx_omnia_b200.registry import Architecture, register_architecture

DELTA = "channel_delta"
LATENT = "latent_attention"


@dataclass(frozen=True)
class FokalornLayer:
    type: str
    mixer: tuple[tuple[str, Any], ...]  # the mixer's keys, as sorted items (hashable)
    ff: int | None  # None: the layer has no feed-forward
    activation: str = "relu2"
    shift: bool = True

    def m(self, key: str, default: Any = None) -> Any:
        return dict(self.mixer).get(key, default)


@dataclass(frozen=True)
class FokalornConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    norm_groups: int
    streams: int | None
    layers: tuple[FokalornLayer, ...]
    loop: tuple[int, int, int] | None  # (start, stop, times)

    def schedule(self) -> list[int]:
        """Layer indices in the order they run."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))


_DELTA_KEYS = ("heads", "kv_heads", "dim", "vdim", "conv")
_LATENT_KEYS = ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot")


def _need(raw: dict, key: str, where: str):
    if key not in raw:
        raise ConfigError(f"Fokalorn: {where} lacks the key {key!r}")
    return raw[key]


def parse(raw: dict[str, Any]) -> FokalornConfig:
    if raw.get("architecture") != "Fokalorn":
        raise ConfigError(f"expected architecture 'Fokalorn', got {raw.get('architecture')!r}")
    layers = []
    for index, layer in enumerate(_need(raw, "layers", "config.json")):
        where = f"layers[{index}]"
        kind, mixer = _need(layer, "type", where), dict(_need(layer, "mixer", where))
        if kind not in (DELTA, LATENT):
            raise ConfigError(f"Fokalorn: {where} has the unknown type {kind!r}")
        for key in (_DELTA_KEYS if kind == DELTA else _LATENT_KEYS):
            _need(mixer, key, f"{where}.mixer")
        if kind == LATENT:
            rot = dict(mixer["rot"])
            _need(rot, "base", f"{where}.mixer.rot"), _need(rot, "dims", f"{where}.mixer.rot")
            mixer["rot"] = tuple(sorted(rot.items()))
        mlp = layer.get("mlp")
        if mlp is not None and mlp.get("kind", "dense") != "dense":
            raise ConfigError(f"Fokalorn: {where}.mlp has the unknown kind {mlp.get('kind')!r}")
        layers.append(FokalornLayer(kind, tuple(sorted(mixer.items())), None if mlp is None else int(_need(mlp, "ff", where + ".mlp")),
                                    "relu2" if mlp is None else mlp.get("act", "relu2")))
    loop = raw.get("loop")
    if loop is not None:
        loop = (int(_need(loop, "start", "loop")), int(_need(loop, "stop", "loop")), int(_need(loop, "times", "loop")))
        if not (0 <= loop[0] <= loop[1] <= len(layers)) or loop[2] < 1:
            raise ConfigError(f"Fokalorn: loop {loop} does not fit {len(layers)} layers")
    norm = _need(raw, "norm", "config.json")
    streams = raw.get("streams")
    width = int(_need(raw, "width", "config.json"))
    groups = int(norm.get("groups", 1))
    if groups < 1 or width % groups:
        raise ConfigError(f"Fokalorn: a width of {width} does not divide into {groups} norm groups")
    if not layers:
        raise ConfigError("Fokalorn: no layers")
    return FokalornConfig(vocab=int(_need(raw, "vocab", "config.json")), width=width,
                          embedding_scale=float(raw.get("embedding", {}).get("scale", 1.0)),
                          norm_eps=float(_need(norm, "eps", "norm")), norm_groups=groups,
                          streams=None if streams is None else int(streams), layers=tuple(layers), loop=loop)


def sizes_from_tensors(config: FokalornConfig, shape_of: Callable[[str], tuple[int, ...] | None]) -> FokalornConfig:
    """Fill in what only the checkpoint's tensors say: the two low-rank widths of a recurrent mixer
    (rows of `a1` and `g1`), and whether a layer has the token shift's tensor."""
    layers = []
    for index, layer in enumerate(config.layers):
        mixer = dict(layer.mixer)
        if layer.type == DELTA:
            for key, tensor in (("decay_rank", "a1"), ("gate_rank", "g1")):
                shape = shape_of(f"l{index}.mix.{tensor}")
                if shape is not None:
                    mixer[key] = int(shape[0])
        else:
            mixer["sink"] = shape_of(f"l{index}.mix.sink") is not None
            mixer["gated"] = shape_of(f"l{index}.mix.g") is not None
        layers.append(dataclasses.replace(layer, mixer=tuple(sorted(mixer.items())),
                                          shift=shape_of(f"l{index}.shift") is not None))
    return dataclasses.replace(config, layers=tuple(layers))


def _norm(config: FokalornConfig) -> PartSpec:
    return PartSpec("rms_norm", {"size": config.width, "eps": config.norm_eps, "weight": "plain",
                                 "groups": config.norm_groups})


def _mixer(config: FokalornConfig, layer: FokalornLayer, index: int) -> PartSpec:
    if layer.type == DELTA:
        for key in ("decay_rank", "gate_rank"):
            if layer.m(key) is None:
                raise ConfigError(f"Fokalorn: layers[{index}].mixer.{key} is in neither the configuration nor a tensor's shape")
        return PartSpec(DELTA, {"hidden": config.width, "heads": layer.m("heads"), "kv_heads": layer.m("kv_heads"),
                                "dim": layer.m("dim"), "vdim": layer.m("vdim"), "conv": layer.m("conv"),
                                "decay_rank": layer.m("decay_rank"), "gate_rank": layer.m("gate_rank"),
                                "norm_eps": config.norm_eps})
    rot = dict(layer.m("rot"))
    position = PartSpec("rotary", {"dims": int(rot["dims"]), "theta": float(rot["base"]), "pairing": "interleaved"})
    return PartSpec(LATENT, {"hidden": config.width, "heads": layer.m("heads"), "dim": layer.m("dim"),
                             "rot_dim": layer.m("rot_dim"), "vdim": layer.m("vdim"), "kv_rank": layer.m("kv_rank"),
                             "scale": float(layer.m("scale")), "norm_eps": config.norm_eps, "position": position,
                             "sink": layer.m("sink", True), "gated": layer.m("gated", True),
                             "window": layer.m("window")})


def model_spec(config: FokalornConfig) -> ModelSpec:
    layers = []
    for index, layer in enumerate(config.layers):
        feed_forward = None if layer.ff is None else PartSpec("dense_mlp", {
            "hidden": config.width, "inner": layer.ff, "activation": layer.activation})
        norms = {"norm1": _norm(config)} if feed_forward is None else {"norm1": _norm(config), "norm2": _norm(config)}
        block = PartSpec("hyper_pre_norm", {"hidden": config.width, "mixer": _mixer(config, layer, index),
                                            "feed_forward": feed_forward, "norms": norms, "streams": config.streams,
                                            "shift": layer.shift})
        layers.append(LayerSpec(block, f"l{index}"))
    return ModelSpec(
        embedding=PartSpec("token_embedding", {"vocab": config.vocab, "hidden": config.width,
                                               "scale": config.embedding_scale, "copies": config.streams or 1}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in config.schedule()),
        final_norm=_norm(config),
        head=PartSpec("lm_head", {"vocab": config.vocab, "hidden": config.width}),
        embedding_prefix="embed", final_norm_prefix="final.norm", head_prefix="head",
    )


_WEIGHT_SUFFIXED = re.compile(r"^(embed|head|final\.norm|l\d+\.norm[12])$")


def tensor_name(file_name: str) -> str:
    """The file's names are the model's, but for the parts that call their one tensor `weight`."""
    return file_name + ".weight" if _WEIGHT_SUFFIXED.match(file_name) else file_name


def random_tensors(config: FokalornConfig, seed: int) -> dict[str, torch.Tensor]:
    """Float32 tensors under the checkpoint's names, drawn on the CPU in a fixed order from one
    generator: matrices N(0, 1/sqrt(fan_in)); norm weights 1 + N(0, 0.1); the stream-mixing matrices
    near the identity; decays, gates and sinks in ranges where every term matters."""
    g = torch.Generator().manual_seed(seed)

    def normal(*shape: int, std: float = 1.0) -> torch.Tensor:
        return torch.randn(*shape, generator=g, dtype=torch.float32) * std

    def matrix(rows: int, cols: int, gain: float = 1.0) -> torch.Tensor:
        return normal(rows, cols, std=gain * cols ** -0.5)

    D = config.width
    out = {"embed": normal(config.vocab, D, std=1.0 / max(config.embedding_scale, 1e-6))}
    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        out[p + "norm1"] = 1.0 + normal(D, std=0.1)
        if layer.shift:
            out[p + "shift"] = torch.rand(D, generator=g) * 0.8
        branches = ["hc1"]
        if layer.ff is not None:
            out[p + "norm2"] = 1.0 + normal(D, std=0.1)
            out[p + "mlp.up"], out[p + "mlp.down"] = matrix(layer.ff, D), matrix(D, layer.ff)
            branches.append("hc2")
        if config.streams is not None:
            n = config.streams
            for hc in branches:
                out[p + hc + ".in"] = 1.0 / n + normal(n, std=0.2)
                out[p + hc + ".out"] = 1.0 + normal(n, std=0.3)
                out[p + hc + ".mix"] = torch.eye(n) * 0.8 + normal(n, n, std=0.15)
        H = layer.m("heads")
        if layer.type == DELTA:
            G, dk, dv, K = layer.m("kv_heads"), layer.m("dim"), layer.m("vdim"), layer.m("conv")
            ra, rg = layer.m("decay_rank"), layer.m("gate_rank")
            if ra is None or rg is None:
                raise ConfigError(f"Fokalorn: layers[{i}].mixer needs decay_rank and gate_rank for random weights")
            for name, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                out[p + f"mix.{name}"] = matrix(rows, D)
                out[p + f"mix.{name}.conv"] = normal(rows, K, std=0.5) + torch.eye(K)[-1] * 0.7
            out[p + "mix.b"] = matrix(H, D)
            out[p + "mix.A_log"] = normal(H, std=0.5) - 1.0
            out[p + "mix.a1"], out[p + "mix.a2"] = matrix(ra, D), matrix(H * dk, ra)
            out[p + "mix.dt_bias"] = normal(H * dk, std=1.0) - 1.0
            out[p + "mix.g1"], out[p + "mix.g2"] = matrix(rg, D), matrix(H * dv, rg)
            out[p + "mix.norm"] = 1.0 + normal(dv, std=0.1)
            out[p + "mix.o"] = matrix(D, H * dv)
        else:
            dn, dr, dv, rank = layer.m("dim"), layer.m("rot_dim"), layer.m("vdim"), layer.m("kv_rank")
            out[p + "mix.q"] = matrix(H * (dn + dr), D, gain=2.0)
            out[p + "mix.dkv"] = matrix(rank + dr, D, gain=2.0)
            out[p + "mix.dkv.norm"] = 1.0 + normal(rank, std=0.1)
            out[p + "mix.uk"], out[p + "mix.uv"] = matrix(H * dn, rank, gain=2.0), matrix(H * dv, rank)
            if layer.m("sink", True):
                out[p + "mix.sink"] = normal(H, std=1.0)
            if layer.m("gated", True):
                out[p + "mix.g"] = matrix(H, D)
            out[p + "mix.o"] = matrix(D, H * dv)
    out["final.norm"] = 1.0 + normal(D, std=0.1)
    out["head"] = matrix(config.vocab, D)
    return out


ARCHITECTURE = Architecture(
    name="fokalorn",
    config_class=FokalornConfig,
    parse=parse,
    model_spec=model_spec,
    tensor_name=tensor_name,
    random_tensors=random_tensors,
    sizes_from_tensors=sizes_from_tensors,
)

register_architecture(ARCHITECTURE, "Fokalorn", "fokalorn")
