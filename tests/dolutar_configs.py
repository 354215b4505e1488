"""Tiny Dolutar configurations for the tests, and their random weights as a checkpoint would hold
them (matrices rounded to bfloat16). Their sizes are unlike one another on purpose."""

from __future__ import annotations

import copy
import json
from pathlib import Path

import torch

from mlx_omnia_b200.registry import resolve_architecture


def _attention(heads, kv_heads, dim, vdim, dims, window, keep, scale, base=300.0, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
             "rot": {"base": base, "dims": dims}, "mask": {"size": window, "keep_first": keep}}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer}


def _dense(layer, ff, limit):
    layer["mlp"] = {"kind": "dense", "ff": ff, "limit": limit}
    return layer


def _moe(layer, ff, experts, identity, top):
    layer["mlp"] = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}
    return layer


def _bare(layer):
    layer["mlp"] = None
    return layer


CONFIGS = {
    # values wider than keys (the generic attention kernel in both precisions), two key/value heads,
    # a rotation over half of a head, a window that is no multiple of anything, a reader whose window
    # and kept positions are smaller than its owner's, a layer without a feed-forward
    "P": {"architecture": "Dolutar", "vocab": 157, "width": 96, "logit_scale": 0.5, "norm": {"eps": 1e-5},
          "embedding": {"scale": 3.0, "bigram": {"buckets": 61, "mul_prev": 13, "mul_cur": 5}},
          "layers": [_dense(_attention(4, 2, 16, 24, 8, 11, 3, 0.25), 80, 0.9),
                     _moe(_attention(4, 2, 16, 24, 8, 7, 2, 0.3, kv_from=0), 24, 5, 2, 2),
                     _bare(_attention(2, 1, 24, 8, 24, 19, 0, 0.2)),
                     _moe(_attention(6, 3, 8, 8, 4, 5, 5, 0.35), 40, 3, 0, 1)]},
    # keys and values of one width (the tensor-core kernels in bfloat16), six query heads to a key
    # head, one query head to a key head, a whole-head rotation, kept positions that outnumber the window
    "Q": {"architecture": "Dolutar", "vocab": 211, "width": 64, "logit_scale": 2.0, "norm": {"eps": 1e-6},
          "embedding": {"scale": 6.0, "bigram": {"buckets": 97, "mul_prev": 3, "mul_cur": 11}},
          "layers": [_moe(_attention(6, 1, 16, 16, 16, 9, 14, 0.25), 32, 4, 1, 3),
                     _dense(_attention(2, 2, 32, 32, 16, 33, 4, 0.18), 48, 2.0),
                     _dense(_attention(2, 2, 32, 32, 16, 33, 4, 0.18, kv_from=1), 96, 0.5)]},
    # wider windows for long prompts: edges of tiles (64), of decode chunks (128) and of pages
    "R": {"architecture": "Dolutar", "vocab": 120, "width": 64, "logit_scale": 1.0, "norm": {"eps": 1e-5},
          "embedding": {"scale": 5.0, "bigram": {"buckets": 53, "mul_prev": 7, "mul_cur": 9}},
          "layers": [_dense(_attention(4, 2, 16, 16, 8, 150, 70, 0.25), 64, 1.5),
                     _moe(_attention(4, 1, 24, 24, 12, 64, 33, 0.2), 32, 6, 2, 2)]},
    # heads of 64 and pages of 16: in bfloat16 the prompts' attention runs on the tcgen05 kernel
    "S": {"architecture": "Dolutar", "vocab": 180, "width": 128, "logit_scale": 0.7, "norm": {"eps": 1e-5},
          "embedding": {"scale": 4.0, "bigram": {"buckets": 89, "mul_prev": 5, "mul_cur": 3}},
          "layers": [_dense(_attention(4, 2, 64, 64, 32, 70, 9, 0.125), 96, 1.2),
                     _moe(_attention(4, 2, 64, 64, 32, 33, 70, 0.125, kv_from=0), 48, 4, 1, 2),
                     _dense(_attention(3, 1, 64, 64, 64, 130, 0, 0.125), 64, 3.0)]},
    # nothing a multiple of eight: a width of 100, heads of 20 with values of 12, feed-forwards of 30 and
    # 20, a window of one token, one kept position, a rotation over four dims, three of four experts
    "O": {"architecture": "Dolutar", "vocab": 101, "width": 100, "logit_scale": 1.5, "norm": {"eps": 1e-5},
          "embedding": {"scale": 2.0, "bigram": {"buckets": 7, "mul_prev": 1000003, "mul_cur": 999983}},
          "layers": [_moe(_attention(3, 3, 20, 12, 4, 1, 1, 0.22), 20, 4, 0, 3),
                     _dense(_attention(3, 3, 20, 12, 4, 6, 1, 0.22, kv_from=0), 30, 0.8),
                     _bare(_attention(5, 1, 36, 36, 0, 13, 2, 0.17)),
                     _moe(_attention(3, 3, 20, 12, 4, 2, 0, 0.22, kv_from=0), 12, 1, 3, 2)]},
}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def tensors(name_or_raw, seed: int = 0) -> dict[str, torch.Tensor]:
    raw = config(name_or_raw) if isinstance(name_or_raw, str) else name_or_raw
    architecture = resolve_architecture(raw)
    drawn = architecture.random_tensors(architecture.parse(raw), seed)
    return {k: t.to(torch.bfloat16).float() for k, t in drawn.items()}


def prompt(length: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(900 + seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


def write_folder(folder: Path, raw: dict, weights: dict[str, torch.Tensor]) -> None:
    """A model folder as the loader reads it: config.json and bfloat16 tensors."""
    from safetensors.torch import save_file

    folder.mkdir(parents=True, exist_ok=True)
    save_file({k: t.to(torch.bfloat16).contiguous() for k, t in weights.items()}, str(folder / "model.safetensors"))
    (folder / "config.json").write_text(json.dumps(raw))
