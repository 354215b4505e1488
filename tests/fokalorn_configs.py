"""Tiny Fokalorn configurations for the tests, and their random weights as a checkpoint would
hold them (matrices rounded to bfloat16)."""

from __future__ import annotations

import copy

import torch

from mlx_omnia_b200.registry import resolve_architecture


def _latent(heads, dim, rot_dim, dims, vdim, rank, scale, base=100.0, **more):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim,
                                                   "kv_rank": rank, "scale": scale, "rot": {"base": base, "dims": dims},
                                                   **more}}


def _delta(heads, kv_heads, dim, vdim, conv, decay_rank=8, gate_rank=12):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                                "conv": conv, "decay_rank": decay_rank, "gate_rank": gate_rank}}


def _with_mlp(layer, ff):
    layer["mlp"] = None if ff is None else {"ff": ff, "kind": "dense"}
    return layer


CONFIGS = {
    # three value heads to a key head, a rotation over part of the rotated dims, a layer without a
    # feed-forward, a looped span in the middle, two streams, three norm groups
    "X": {"architecture": "Fokalorn", "vocab": 211, "width": 96, "embedding": {"scale": 4.0},
          "norm": {"eps": 1e-5, "groups": 3}, "streams": 2, "loop": {"start": 1, "stop": 3, "times": 3},
          "layers": [_with_mlp(_latent(3, 24, 8, 4, 16, 40, 0.2), 160), _with_mlp(_delta(4, 2, 24, 40, 4), None),
                     _with_mlp(_delta(2, 2, 16, 24, 2), 128), _with_mlp(_latent(2, 16, 16, 16, 32, 48, 0.17), 96)]},
    # the ordinary residual, one norm group, no loop, a convolution of one tap, one head
    "Y": {"architecture": "Fokalorn", "vocab": 130, "width": 64, "embedding": {"scale": 1.0},
          "norm": {"eps": 1e-6, "groups": 1},
          "layers": [_with_mlp(_delta(1, 1, 8, 8, 1, 4, 4), 64), _with_mlp(_latent(1, 8, 4, 4, 8, 16, 0.3), 80)]},
    # a single stream that still mixes, the whole model looped, five taps
    "Z": {"architecture": "Fokalorn", "vocab": 97, "width": 48, "embedding": {"scale": 7.0},
          "norm": {"eps": 1e-5, "groups": 2}, "streams": 1, "loop": {"start": 0, "stop": 2, "times": 2},
          "layers": [_with_mlp(_delta(3, 3, 12, 20, 5, 6, 6), 72), _with_mlp(_latent(4, 12, 6, 6, 10, 24, 0.25), None)]},
}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def tensors(name_or_raw, seed: int = 0) -> dict[str, torch.Tensor]:
    raw = config(name_or_raw) if isinstance(name_or_raw, str) else name_or_raw
    architecture = resolve_architecture(raw)
    drawn = architecture.random_tensors(architecture.parse(raw), seed)
    return {k: (t if t.dim() < 2 else t.to(torch.bfloat16).float()) for k, t in drawn.items()}


def prompt(length: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(500 + seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()
