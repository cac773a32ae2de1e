"""Norms. `rms_norm` covers the three conventions one trunk can mix: a plain weight,
a centred weight stored as `w` and applied as `1 + w`, and no weight at all.

Reference: the four block norms are centred and folded at load
(src/mlx_omnia/engine/models/muse_glimmer/checkpoint.py:85-93), `model.norm` is plain
(src/mlx_omnia/engine/models/muse_glimmer/layers/block.py:39), and the QK and embedding
norms carry no weight (src/mlx_omnia/engine/models/muse_glimmer/layers/attention.py:8-17).
"""

from __future__ import annotations

import torch

from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import Norm, TensorSpec, register_norm


@register_norm("rms_norm")
class RMSNorm(Norm):
    """h = x * rsqrt(mean(x^2) + eps) * scale over the last axis.

    size:    length of the normalised axis
    eps:     added to the mean square
    weight:  "plain" (scale = w), "centred" (scale = 1 + w, the sum taken in float32
             at load) or "none" (no tensor in the checkpoint)
    """

    def __init__(self, size: int, eps: float, weight: str = "plain") -> None:
        if weight not in ("plain", "centred", "none"):
            raise ValueError(f"rms_norm weight convention {weight!r}")
        self.size, self.eps, self.convention = size, float(eps), weight
        self.weight = None

    def tensors(self) -> dict[str, TensorSpec]:
        return {} if self.convention == "none" else {"weight": TensorSpec((self.size,), "vector")}

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        if self.convention != "none":
            w = tensors["weight"].to(torch.float32)
            self.weight = (w + 1.0).contiguous() if self.convention == "centred" else w.contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, self.runtime.dtype)
