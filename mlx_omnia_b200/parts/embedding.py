"""The two ends of a decoder: token embedding and language-model head.

Reference: the embedding is a lookup followed by a weightless RMS norm
(src/mlx_omnia/engine/models/muse_glimmer/model.py:62-63); the head is
tanh(lm_head(n) * output_multiplier / cap) * cap
(src/mlx_omnia/engine/models/muse_glimmer/model.py:79-82). A tied head reads the
embedding table, as the reference's dense model does
(src/mlx_omnia/engine/core/attention.py:792-796).
"""

from __future__ import annotations

import torch

from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import Embedding, Part, StateSpec, TensorSpec, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    """x = table[ids], RMS-normalised without a weight when `norm_eps` is given, or multiplied by
    `scale`; with `copies` n the row is written n times side by side (the start of a residual
    kept as n streams). The output is the float32 residual stream."""

    def __init__(self, vocab: int, hidden: int, norm_eps: float | None = None, scale: float = 1.0,
                 copies: int = 1) -> None:
        if norm_eps is not None and (scale != 1.0 or copies != 1):
            raise ValueError("a normed embedding is neither scaled nor copied")
        self.vocab, self.hidden, self.norm_eps, self.scale, self.copies = vocab, hidden, norm_eps, float(scale), copies

    def tensors(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab, self.hidden))}

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        self.weight = tensors["weight"].contiguous()

    def forward(self, token_ids: torch.Tensor, positions: torch.Tensor | None = None) -> torch.Tensor:
        if self.scale != 1.0 or self.copies != 1:
            return ops.embed_streams(token_ids, self.weight, self.scale, self.copies)
        return ops.embed_rmsnorm(token_ids, self.weight, self.norm_eps)


@register_head("lm_head")
class LMHead(Part):
    """float32 logits = cap * tanh((h @ W^T) * multiplier / cap) for the rows given.

    tied:       read the embedding table instead of a tensor of its own
    multiplier: scales the product; softcap: the cap, None for none
    """

    def __init__(self, vocab: int, hidden: int, tied: bool = False, multiplier: float = 1.0,
                 softcap: float | None = None) -> None:
        self.vocab, self.hidden, self.tied = vocab, hidden, tied
        self.multiplier, self.softcap = float(multiplier), softcap

    def tensors(self) -> dict[str, TensorSpec]:
        return {} if self.tied else {"weight": TensorSpec((self.vocab, self.hidden))}

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        self.weight = None if self.tied else tensors["weight"].contiguous()

    def bind(self, table: torch.Tensor) -> None:
        """Give a tied head the embedding table."""
        if self.tied:
            self.weight = table

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return ops.linear_softcap(h, self.weight, self.multiplier, self.softcap)


@register_embedding("pair_hash_embedding")
class PairHashEmbedding(Embedding):
    """x = table[id] * scale + pairs[(id_before * mul_prev + id * mul_cur) mod buckets]: beside its own
    row a token gets a row that its pair with the token before it is hashed to. `pairs` has
    buckets + 1 rows; the extra last row is the one of a request's first token. The token before a
    portion's first token is per-request state (`prev`, one int32 a slot). float32 out.

    Tensors: `weight` [vocab, hidden], `pairs` [buckets + 1, hidden]."""

    def __init__(self, vocab: int, hidden: int, buckets: int, mul_prev: int, mul_cur: int, scale: float = 1.0) -> None:
        if buckets < 1 or mul_prev < 0 or mul_cur < 0:
            raise ValueError(f"pair_hash_embedding: {buckets} buckets, multipliers {mul_prev} and {mul_cur}")
        self.vocab, self.hidden, self.buckets = vocab, hidden, buckets
        self.mul_prev, self.mul_cur, self.scale = int(mul_prev), int(mul_cur), float(scale)

    def tensors(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab, self.hidden)), "pairs": TensorSpec((self.buckets + 1, self.hidden))}

    def state_spec(self):
        return {"prev": StateSpec((), torch.int32)}

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        self.weight, self.pairs = tensors["weight"].contiguous(), tensors["pairs"].contiguous()

    def forward(self, token_ids: torch.Tensor, positions: torch.Tensor, step=None) -> torch.Tensor:
        if step is None or not step.model_state:
            raise RuntimeError("pair_hash_embedding needs the step and its per-request state")
        return ops.embed_pair(step, self.weight, self.pairs, step.model_state["prev"], self.scale, self.mul_prev,
                              self.mul_cur)
