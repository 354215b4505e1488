"""A plain, slow Fokalorn: whole sequences on the CPU, no cache, no batching, one function per
mechanism. It shares nothing with the package (it reads the raw config.json object and a dict of
tensors under the checkpoint's names) and exists to be compared with it.

Notation: T tokens, D model width, S residual streams, H heads; every function takes and returns
tensors of the dtype it is given (float64 for a tight oracle, float32 otherwise).
"""

from __future__ import annotations

import math

import torch


def grouped_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, groups: int = 1) -> torch.Tensor:
    """The last axis cut into `groups` equal runs; each run divided by sqrt(mean(run^2) + eps); then * weight."""
    parts = x.reshape(*x.shape[:-1], groups, x.shape[-1] // groups)
    parts = parts / torch.sqrt(parts.pow(2).mean(-1, keepdim=True) + eps)
    return parts.reshape(x.shape) * weight


def token_shift(h: torch.Tensor, mu: torch.Tensor, before: torch.Tensor | None = None) -> torch.Tensor:
    """h_t + (h_{t-1} - h_t) * mu with h_{-1} = `before` (zeros when None); h is [T, D] and unshifted."""
    first = torch.zeros_like(h[:1]) if before is None else before.reshape(1, -1)
    previous = torch.cat([first, h[:-1]], dim=0)
    return h + (previous - h) * mu


def short_conv_silu(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """Causal depth-wise convolution over time, then SiLU. x [T, C]; taps [C, K], the last column
    multiplying the current token, the one before it the previous token, zeros before the start."""
    T, K = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, x.shape[1], dtype=x.dtype), x], dim=0)
    out = torch.zeros_like(x)
    for j in range(K):
        out = out + padded[j: j + T] * taps[:, j]
    return out * torch.sigmoid(out)


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).sum(-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, beta, decay, state=None):
    """One head of the gated delta rule with a decay per key channel.
    q, k, decay [T, dk]; v [T, dv]; beta [T]; state [dk, dv] (zeros when None).
    Per token: S = decay[:, None] * S; u = beta * (v - S^T k); S = S + k u^T; o = S^T q."""
    T, dk = q.shape
    S = torch.zeros(dk, v.shape[1], dtype=q.dtype) if state is None else state.clone()
    out = []
    for t in range(T):
        S = decay[t][:, None] * S
        u = beta[t] * (v[t] - S.t() @ k[t])
        S = S + torch.outer(k[t], u)
        out.append(S.t() @ q[t])
    return torch.stack(out), S


def channel_delta(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """The recurrent mixer on a whole sequence. `w` holds its tensors by local name, `m` its sizes."""
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = unit(short_conv_silu(h @ w["q"].t(), w["q.conv"]).reshape(T, G, dk)) * dk ** -0.5
    k = unit(short_conv_silu(h @ w["k"].t(), w["k.conv"]).reshape(T, G, dk))
    v = short_conv_silu(h @ w["v"].t(), w["v.conv"]).reshape(T, H, dv)
    beta = torch.sigmoid(h @ w["b"].t())  # [T, H]
    step = torch.nn.functional.softplus((h @ w["a1"].t()) @ w["a2"].t() + w["dt_bias"]).reshape(T, H, dk)
    decay = torch.exp(-torch.exp(w["A_log"]).reshape(1, H, 1) * step)
    gate = torch.sigmoid((h @ w["g1"].t()) @ w["g2"].t()).reshape(T, H, dv)
    heads = []
    for head in range(H):
        g = head // (H // G)
        o, _ = delta_rule(q[:, g], k[:, g], v[:, head], beta[:, head], decay[:, head])
        o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps) * w["norm"]
        heads.append(o * gate[:, head])
    return torch.cat(heads, dim=-1) @ w["o"].t()


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Rotary encoding of the first `dims` entries of the last axis, entry 2i paired with 2i + 1;
    x [T, ..., d]; angle = position * base^(-2i/dims)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    angle = positions.to(torch.float64)[:, None] * base ** (-2.0 * i / dims)  # [T, dims/2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = angle.cos().to(x.dtype).reshape(shape), angle.sin().to(x.dtype).reshape(shape)
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([even * cos - odd * sin, odd * cos + even * sin], dim=-1).flatten(-2)
    return torch.cat([turned, x[..., dims:]], dim=-1)


def latent_attention(h: torch.Tensor, w: dict, m: dict, eps: float, positions: torch.Tensor) -> torch.Tensor:
    """Attention whose keys and values are expanded from one low-rank row per token, with one
    rotated key part shared by the heads, a sink in the softmax's denominator and a gate per head."""
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    q = (h @ w["q"].t()).reshape(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate_interleaved(q[..., dn:], positions, m["rot"]["dims"], m["rot"]["base"])
    down = h @ w["dkv"].t()
    latent = grouped_rms_norm(down[:, :rank], w["dkv.norm"], eps)
    k_rot = rotate_interleaved(down[:, rank:], positions, m["rot"]["dims"], m["rot"]["base"])  # [T, dr]
    k_plain = (latent @ w["uk"].t()).reshape(T, H, dn)
    value = (latent @ w["uv"].t()).reshape(T, H, dv)
    scores = (torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thd,sd->hts", q_rot, k_rot)) * m["scale"]
    hidden = torch.ones(T, T, dtype=torch.bool).triu(1)
    scores = scores.masked_fill(hidden, -math.inf)
    if m.get("window"):
        scores = scores.masked_fill(torch.ones(T, T, dtype=torch.bool).tril(-m["window"]), -math.inf)
    sink = w["sink"].reshape(H, 1, 1)
    top = torch.maximum(scores.max(-1, keepdim=True).values, sink)
    weights = torch.exp(scores - top)
    weights = weights / (weights.sum(-1, keepdim=True) + torch.exp(sink - top))
    out = torch.einsum("hts,shd->thd", weights, value)
    out = out * torch.sigmoid(h @ w["g"].t())[:, :, None]
    return out.reshape(T, H * dv) @ w["o"].t()


ACTIVATIONS = {
    "relu2": lambda z: torch.relu(z) ** 2,
    "gelu_tanh": lambda z: 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))),
    "silu": lambda z: z * torch.sigmoid(z),
}


def dense_mlp(h: torch.Tensor, w: dict, act: str = "relu2") -> torch.Tensor:
    return ACTIVATIONS[act](h @ w["up"].t()) @ w["down"].t()


def sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def schedule(config: dict) -> list[int]:
    """Layer indices in the order they run: the looped span repeated in place."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    span = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + span * loop["times"] + list(range(loop["stop"], n))


def forward(config: dict, tensors: dict, ids, dtype=torch.float64, layer_outputs: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence `ids`. With `layer_outputs` (a list), the sum of the
    residual streams after every layer run is appended to it."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps, groups = config["norm"]["eps"], config["norm"].get("groups", 1)
    ids = torch.as_tensor(ids, dtype=torch.long)
    positions = torch.arange(ids.shape[0])
    x = w["embed"][ids] * config["embedding"]["scale"]
    streams = config.get("streams")
    xs = [x.clone() for _ in range(streams)] if streams else None

    def sublayer(which: str, lw: dict, run):
        nonlocal x, xs
        if xs is None:
            x = x + run(x)
            return
        hc = sub(lw, which + ".")
        y = run(sum(hc["in"][s] * xs[s] for s in range(streams)))
        xs = [sum(hc["mix"][s, t] * xs[s] for s in range(streams)) + hc["out"][t] * y for t in range(streams)]

    for index in schedule(config):
        layer, lw = config["layers"][index], sub(w, f"l{index}.")
        m = layer["mixer"]

        def mix(u):
            h = grouped_rms_norm(u, lw["norm1"], eps, groups)
            if "shift" in lw:
                h = token_shift(h, lw["shift"])
            if layer["type"] == "channel_delta":
                return channel_delta(h, sub(lw, "mix."), m, eps)
            if layer["type"] == "latent_attention":
                return latent_attention(h, sub(lw, "mix."), m, eps, positions)
            raise ValueError(layer["type"])

        sublayer("hc1", lw, mix)
        if layer.get("mlp"):
            sublayer("hc2", lw, lambda u: dense_mlp(grouped_rms_norm(u, lw["norm2"], eps, groups), sub(lw, "mlp."),
                                                    layer["mlp"].get("act", "relu2")))
        if layer_outputs is not None:
            layer_outputs.append(sum(xs) if xs is not None else x.clone())
    if xs is not None:
        x = sum(xs)
    return grouped_rms_norm(x, w["final.norm"], eps, groups) @ w["head"].t()
