"""Blocks: how a mixer, a feed-forward and norms sit around the residual stream.

The residual stream `x` is float32 [tokens, hidden] and is updated in place. A block
is handed `h`, its own entry norm already applied to `x` (the previous block's last
kernel produced it), and the norm that whatever runs next wants applied on the way
out, so each residual update is one fused pass: add the (normed) branch, then norm.
In a step of few rows that pass need not be a kernel of its own: where the part that
takes its result says `takes_pending`, the block hands it an `ops.PendingStep` instead
of `h`, the part's first product runs the step in front of itself, and the block then
picks up the new residual with `ops.residual_after`.

Reference: sandwich arrangement x + post(attn(input_ln(x))), then + post(mlp(pre_ff(.)))
(src/mlx_omnia/engine/models/muse_glimmer/layers/block.py:11-26).
"""

from __future__ import annotations

import torch

from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import (FEED_FORWARDS, MIXERS, NORMS, Block, Norm, PartSpec, TensorSpec,
                                       register_block)
from mlx_omnia_b200.parts.norms import RMSNorm


def residual_step(x: torch.Tensor, branch: torch.Tensor, branch_norm: Norm | None, out_norm: Norm | None,
                  may_pend: bool = False):
    """x += branch_norm(branch); return out_norm(x) (None without an out_norm).
    RMS norms take the fused kernel; any other norm class is applied by its own forward.
    With `may_pend` (whoever takes the result says it `takes_pending`) a step of few rows is
    not run here but handed on as an `ops.PendingStep`, for the taker's first product to run."""
    fused_b = branch_norm is None or isinstance(branch_norm, RMSNorm)
    fused_o = out_norm is None or isinstance(out_norm, RMSNorm)
    if may_pend and fused_b and fused_o and out_norm is not None and ops.pending_supported(x, branch):
        return ops.PendingStep(x, branch, None if branch_norm is None else branch_norm.weight,
                               None if branch_norm is None else branch_norm.eps, out_norm.weight, out_norm.eps)
    if not fused_b:
        branch = branch_norm.forward(branch.float())
        branch_norm = None
    h = ops.add_rmsnorm(x, branch,
                        None if branch_norm is None else branch_norm.weight,
                        None if branch_norm is None else branch_norm.eps,
                        out_norm.weight if (fused_o and out_norm is not None) else None,
                        out_norm.eps if (fused_o and out_norm is not None) else None)
    if not fused_o:
        h = out_norm.forward(x)
    return h


class _TwoBranchBlock(Block):
    norm_names: tuple[str, ...] = ()

    def __init__(self, mixer: PartSpec, feed_forward: PartSpec, norms: dict[str, PartSpec],
                 mixer_name: str = "self_attn", feed_forward_name: str = "mlp") -> None:
        missing = set(self.norm_names) - set(norms)
        if missing:
            raise ValueError(f"{type(self).__name__} needs the norms {sorted(missing)}")
        self.mixer = MIXERS.build(mixer)
        self.feed_forward = FEED_FORWARDS.build(feed_forward)
        self.norms = {name: NORMS.build(norms[name]) for name in self.norm_names}
        self.mixer_name, self.feed_forward_name = mixer_name, feed_forward_name
        self.entry_norm = self.norms[self.norm_names[0]]

    def _mix(self, h, ctx):
        """The mixer's branch; `h` may be the block before's pending step, which a mixer that does
        not take such gets settled."""
        return self.mixer.forward(h if getattr(self.mixer, "takes_pending", False) else ops.settle(h), ctx)

    def children(self):
        yield self.mixer_name, self.mixer
        yield self.feed_forward_name, self.feed_forward
        yield from self.norms.items()

    def tensors(self) -> dict[str, TensorSpec]:
        return {f"{name}.{local}": spec for name, part in self.children() for local, spec in part.tensors().items()}

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        for name, part in self.children():
            prefix = name + "."
            part.load({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}, runtime)


@register_block("sandwich")
class SandwichBlock(_TwoBranchBlock):
    """Four norms: one before and one after each branch; the after-norm is on the branch."""

    norm_names = ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm",
                  "post_feedforward_layernorm")

    def forward(self, x, h, ctx, exit_norm):
        n = self.norms
        a = self._mix(h, ctx)
        x = ops.residual_after(h, x)
        h2 = residual_step(x, a, n["post_attention_layernorm"], n["pre_feedforward_layernorm"],
                           getattr(self.feed_forward, "takes_pending", False))
        m = self.feed_forward.forward(h2, ctx)
        x = ops.residual_after(h2, x)
        return x, residual_step(x, m, n["post_feedforward_layernorm"], exit_norm, ctx.exit_may_pend)


@register_block("pre_norm")
class PreNormBlock(_TwoBranchBlock):
    """Two norms, one before each branch; branches are added as they are."""

    norm_names = ("input_layernorm", "post_attention_layernorm")

    def forward(self, x, h, ctx, exit_norm):
        a = self._mix(h, ctx)
        x = ops.residual_after(h, x)
        h2 = residual_step(x, a, None, self.norms["post_attention_layernorm"],
                           getattr(self.feed_forward, "takes_pending", False))
        m = self.feed_forward.forward(h2, ctx)
        x = ops.residual_after(h2, x)
        return x, residual_step(x, m, None, exit_norm, ctx.exit_may_pend)
