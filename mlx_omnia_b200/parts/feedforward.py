"""Feed-forward parts.

Reference: SwiGLU with gate and up fused on the output axis at load
(src/mlx_omnia/engine/core/layers.py:253-272, src/mlx_omnia/engine/checkpoint.py:333-347).
"""

from __future__ import annotations

import torch

from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import FeedForward, TensorSpec, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    """down(silu(gate(h)) * up(h)), no biases.

    hidden, inner: widths. The checkpoint's `gate_proj` and `up_proj` are stacked into
    one [2 * inner, hidden] operand at load so the step runs one product for both.
    """

    takes_pending = True

    def __init__(self, hidden: int, inner: int) -> None:
        self.hidden, self.inner = hidden, inner

    def tensors(self) -> dict[str, TensorSpec]:
        return {
            "gate_proj.weight": TensorSpec((self.inner, self.hidden)),
            "up_proj.weight": TensorSpec((self.inner, self.hidden)),
            "down_proj.weight": TensorSpec((self.hidden, self.inner)),
        }

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        self.gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0).contiguous()
        self.down = tensors["down_proj.weight"].contiguous()

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        return ops.linear(ops.linear_swiglu(h, self.gate_up), self.down)
