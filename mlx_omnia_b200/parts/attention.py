"""Attention mixers over the paged cache.

Reference: separate q/k/v projections, per-head norm before rotation, keys cached after
rotation, grouped-query softmax attention, a full-width sigmoid gate computed from the
same input as q, output projection (src/mlx_omnia/engine/core/attention.py:618-682);
Muse-Glimmer's choice of options
(src/mlx_omnia/engine/models/muse_glimmer/layers/attention.py:20-47).
"""

from __future__ import annotations

import torch

from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import POSITIONS, KVSpec, Mixer, PartSpec, TensorSpec, register_mixer


@register_mixer("gqa_attention")
class GQAAttention(Mixer):
    """Grouped-query causal attention.

    hidden, heads, kv_heads, head_dim: sizes (heads * head_dim need not equal hidden)
    scale:     multiplies q.k before the softmax
    window:    None, or how many latest positions (the query's own included) are visible
    qk_norm_eps: None, or the eps of a weightless RMS norm of every q and k head
    gated:     multiply the attention output by sigmoid(gate_proj(h)), full width
    position:  PartSpec of the position encoding applied to q and k
    own_kv:    False for a layer that only reads another layer's cache (no k/v weights)
    """

    graph_safe = True  # no host-side work per request: a decode step can be captured
    graph_safe_mixed = True  # nor in a step of any other shape: repeated mixed steps can be captured too
    takes_pending = True  # h goes to the in-projection and nowhere else

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, scale: float,
                 window: int | None = None, qk_norm_eps: float | None = None, gated: bool = False,
                 position: PartSpec | None = None, own_kv: bool = True) -> None:
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads do not divide into {kv_heads} groups")
        if head_dim % 2 or head_dim > 256:
            raise ValueError(f"head_dim must be even and at most 256, got {head_dim}")
        self.hidden, self.heads, self.kv_heads, self.head_dim = hidden, heads, kv_heads, head_dim
        self.scale, self.window, self.qk_norm_eps, self.gated, self.own_kv = scale, window, qk_norm_eps, gated, own_kv
        self.position = POSITIONS.build(position or PartSpec("none"))

    def kv_spec(self) -> KVSpec:
        return KVSpec.keys_and_values(self.kv_heads, self.head_dim, self.window)

    def tensors(self) -> dict[str, TensorSpec]:
        q, kv = self.heads * self.head_dim, self.kv_heads * self.head_dim
        specs = {"q_proj.weight": TensorSpec((q, self.hidden)), "o_proj.weight": TensorSpec((self.hidden, q))}
        if self.gated:
            specs["gate_proj.weight"] = TensorSpec((q, self.hidden))
        if self.own_kv:
            specs["k_proj.weight"] = TensorSpec((kv, self.hidden))
            specs["v_proj.weight"] = TensorSpec((kv, self.hidden))
        return specs

    def load(self, tensors, runtime) -> None:
        super().load(tensors, runtime)
        self.position.load({}, runtime)
        q, kv = self.heads * self.head_dim, self.kv_heads * self.head_dim
        # One operand [q | gate | k | v] so the step runs a single input projection.
        rows, self.q_col, col = [tensors["q_proj.weight"]], 0, q
        self.gate_col = self.k_col = self.v_col = 0
        if self.gated:
            rows.append(tensors["gate_proj.weight"])
            self.gate_col, col = col, col + q
        if self.own_kv:
            rows += [tensors["k_proj.weight"], tensors["v_proj.weight"]]
            self.k_col, self.v_col = col, col + kv
        self.in_proj = torch.cat(rows, dim=0).contiguous()
        self.o_proj = tensors["o_proj.weight"].contiguous()

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        if ctx.kv is None:
            raise RuntimeError("an attention mixer needs cache pages")
        if ctx.kv.writes and not self.own_kv:
            raise RuntimeError("a mixer without k/v projections cannot own a cache entry")
        inv_freq = self.position.table()
        # Many rows: the product's epilogue normalises, rotates and stores (only the gate's columns of
        # the projected rows are then written).
        made = ops.linear_qkv(h, self.in_proj, self.q_col, self.k_col, self.v_col, self.heads,
                              self.kv_heads if self.own_kv else 0, self.head_dim, self.qk_norm_eps, inv_freq, ctx.step,
                              ctx.kv if self.own_kv else None)
        if made is not None:
            proj, q = made
            out = ops.paged_attention(q, ctx.kv, ctx.step, self.scale, gate=proj if self.gated else None,
                                      gate_col=self.gate_col)
            return ops.linear(out, self.o_proj)
        proj = ops.linear(h, self.in_proj)
        gate = proj if self.gated else None
        if self.own_kv and ops.decode_fusable(proj, self.heads, self.kv_heads, self.head_dim, inv_freq, ctx.kv,
                                              ctx.step):
            # Single tokens only: the attention kernel normalises, rotates and stores by itself.
            rows = ops.Projection(proj, self.q_col, self.k_col, self.v_col, self.heads, self.head_dim,
                                  self.qk_norm_eps, inv_freq)
            out = ops.paged_attention(None, ctx.kv, ctx.step, self.scale, gate=gate, gate_col=self.gate_col,
                                      projection=rows)
        else:
            q = ops.qk_norm_rope_store(proj, self.q_col, self.k_col, self.v_col, self.heads, self.kv_heads,
                                       self.head_dim, self.qk_norm_eps, inv_freq, ctx.step.positions,
                                       ctx.kv if self.own_kv else None)
            out = ops.paged_attention(q, ctx.kv, ctx.step, self.scale, gate=gate, gate_col=self.gate_col)
        return ops.linear(out, self.o_proj)
