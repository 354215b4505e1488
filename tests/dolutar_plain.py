"""Dolutar, written out plainly: one function per mechanism, whole sequences, no cache, float64
unless told otherwise. It shares nothing with the package; the engine is compared with it.

Notation: a sequence is T tokens; D the model width; H query heads in G key/value groups;
dk the query/key size of a head, dv its value size; tensors are a dict by checkpoint name.
"""

from __future__ import annotations

import math

import torch


def rms(x: torch.Tensor, eps: float, w: torch.Tensor | None = None) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, times w."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def embedding(tokens: list[int], W: dict, cfg: dict, dtype) -> torch.Tensor:
    """Token rows times the scale, plus one row of the pair table: the row of (previous, current)
    hashed into the buckets, or the extra last row for a sequence's first token."""
    e = cfg["embedding"]
    x = W["embed"].to(dtype)[tokens] * e["scale"]
    pair = e.get("bigram")
    if pair is not None:
        rows = [pair["buckets"]] + [(a * pair["mul_prev"] + b * pair["mul_cur"]) % pair["buckets"]
                                    for a, b in zip(tokens[:-1], tokens[1:])]
        x = x + W["bigram"].to(dtype)[rows]
    return x


def rotate(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: the first `dims` dims turn, dim i with dim i + dims/2, by position * base^(-2i/dims)."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None, None] * freq
    c, s = torch.cos(angle), torch.sin(angle)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def visible(T: int, size: int, keep_first: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j when j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def keys_and_values(h: torch.Tensor, W: dict, p: str, m: dict, eps: float):
    """The keys (normed, rotated) and values a layer with projections of its own makes: [T, G, dk], [T, G, dv]."""
    T, G, dk, dv = h.shape[0], m["kv_heads"], m["dim"], m["vdim"]
    dt = h.dtype
    k = (h @ W[p + "k"].to(dt).T + W[p + "k.b"].to(dt)).view(T, G, dk)
    v = (h @ W[p + "v"].to(dt).T + W[p + "v.b"].to(dt)).view(T, G, dv)
    k = rms(k, eps, W[p + "k.norm"].to(dt))
    k = rotate(k, torch.arange(T), m["rot"]["dims"], m["rot"]["base"])
    return k, v


def attention(h: torch.Tensor, W: dict, p: str, m: dict, eps: float, kv) -> torch.Tensor:
    """Softmax attention over `kv` = (keys, values) with a sliding window that keeps the first
    tokens and one extra term exp(sink_h) in every head's denominator."""
    T, H, G, dk, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    dt = h.dtype
    q = (h @ W[p + "q"].to(dt).T + W[p + "q.b"].to(dt)).view(T, H, dk)
    q = rms(q, eps, W[p + "q.norm"].to(dt))
    q = rotate(q, torch.arange(T), m["rot"]["dims"], m["rot"]["base"])
    k, v = kv
    see = visible(T, m["mask"]["size"], m["mask"]["keep_first"])
    sink = W[p + "sink"].to(dt)
    out = torch.zeros(T, H, dv, dtype=dt)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~see, -math.inf)
        top = torch.maximum(s.max(-1, keepdim=True).values, sink[head])
        e = torch.exp(s - top)
        weights = e / (e.sum(-1, keepdim=True) + torch.exp(sink[head] - top))
        out[:, head] = weights @ v[:, g]
    return out.reshape(T, H * dv) @ W[p + "o"].to(dt).T


def dense_ff(h: torch.Tensor, W: dict, p: str, limit: float) -> torch.Tensor:
    """g = min(gate h, limit), u = clamp(up h, -limit, limit); down(g sigmoid(1.702 g) (u + 1))."""
    dt = h.dtype
    g = torch.clamp(h @ W[p + "gate"].to(dt).T, max=limit)
    u = torch.clamp(h @ W[p + "up"].to(dt).T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].to(dt).T


def route(h: torch.Tensor, W: dict, p: str, top: int):
    """Which experts each token uses and with what weights: softmax over every router output;
    the choice is by score + correction, the weight is the score itself, not renormalised."""
    dt = h.dtype
    s = torch.softmax(h @ W[p + "router"].to(dt).T, dim=-1)
    chosen = torch.topk(s + W[p + "correction"].to(dt), top, dim=-1).indices
    return chosen, torch.gather(s, 1, chosen)


def moe_ff(h: torch.Tensor, W: dict, p: str, router: dict) -> torch.Tensor:
    """The weighted sum of the chosen experts; the last `identity` router outputs name experts
    that hand their input back."""
    dt = h.dtype
    E = router["experts"]
    chosen, weights = route(h, W, p, router["top"])
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weights[t]):
            if e >= E:
                y[t] += w * h[t]
            else:
                q = f"{p}e{e}."
                a = h[t] @ W[q + "gate"].to(dt).T
                y[t] += w * ((a * torch.sigmoid(a) * (h[t] @ W[q + "up"].to(dt).T)) @ W[q + "down"].to(dt).T)
    return y


def forward(tokens: list[int], W: dict, cfg: dict, dtype=torch.float64, layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence. `layers_out`, when a list, receives the residual after every layer."""
    eps = cfg["norm"]["eps"]
    x = embedding(tokens, W, cfg, dtype)
    held: dict[int, tuple] = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] != "attention":
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        if m.get("kv_from") is None:
            held[i] = keys_and_values(x, W, p + "mix.", m, eps)
            kv = held[i]
        else:
            kv = held[m["kv_from"]]
        x = x + rms(attention(x, W, p + "mix.", m, eps, kv), eps, W[p + "norm1"].to(dtype))
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                y = dense_ff(x, W, p + "mlp.", mlp["limit"])
            elif mlp["kind"] == "moe":
                y = moe_ff(x, W, p + "mlp.", mlp["router"])
            else:
                raise ValueError(f"layer {i}: unknown feed-forward {mlp['kind']!r}")
            x = x + rms(y, eps, W[p + "norm2"].to(dtype))
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms(x, eps, W["final.norm"].to(dtype))
    return (x @ W["head"].to(dtype).T) * cfg.get("logit_scale", 1.0)
