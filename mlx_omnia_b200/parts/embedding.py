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
from mlx_omnia_b200.parts.base import Embedding, Part, TensorSpec, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    """x = table[ids], RMS-normalised without a weight when `norm_eps` is given.
    The output is the float32 residual stream."""

    def __init__(self, vocab: int, hidden: int, norm_eps: float | None = None) -> None:
        self.vocab, self.hidden, self.norm_eps = vocab, hidden, norm_eps

    def tensors(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab, self.hidden))}

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        self.weight = tensors["weight"].contiguous()

    def forward(self, token_ids: torch.Tensor, positions: torch.Tensor | None = None) -> torch.Tensor:
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
