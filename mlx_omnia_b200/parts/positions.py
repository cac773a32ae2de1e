"""Position encodings. A position part owns a float32 table of inverse frequencies
that the rotation kernel multiplies by each token's position; no table means the
layer sees no positions at all (NoPE).

Reference: per-layer base with 0 = no rotation
(src/mlx_omnia/engine/models/muse_glimmer/layers/attention.py:39-40); half-split pairing
(i, i + d/2), angle pos * theta^(-2i/d), scale 1
(src/mlx_omnia/engine/core/attention.py:587-599,
src/mlx_omnia/engine/core/kernels/qkv_rope/epilogue.py:56-63).
"""

from __future__ import annotations

import torch

from mlx_omnia_b200.parts.base import Position, register_position


_TABLES: dict[tuple[int, float, str], torch.Tensor] = {}


@register_position("rotary")
class Rotary(Position):
    """Half-split rotary embedding over the first `dims` dims of each head.

    theta: the base; inverse frequency i is theta^(-2i/dims), computed in float64 and
           rounded once to float32, so every consumer multiplies the same constants.
    """

    def __init__(self, dims: int, theta: float) -> None:
        if dims % 2 or dims <= 0:
            raise ValueError(f"rotary dims must be even and positive, got {dims}")
        if theta <= 0:
            raise ValueError(f"rotary theta must be positive, got {theta}")
        self.dims, self.theta = dims, float(theta)
        self._table = None

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        # Layers of one base share one tensor: what kernels make from a table once per pass over the
        # layers (the angles of a step's positions) is then made once, not once per layer.
        key = (self.dims, self.theta, str(runtime.device))
        if key not in _TABLES:
            exponent = torch.arange(self.dims // 2, dtype=torch.float64) * (2.0 / self.dims)
            inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -exponent)
            _TABLES[key] = inv.to(torch.float32).to(runtime.device)
        self._table = _TABLES[key]

    def table(self) -> torch.Tensor | None:
        return self._table


@register_position("none")
class NoPosition(Position):
    """The layer is not told where a token is."""

    def __init__(self) -> None:
        pass

    def table(self) -> None:
        return None
