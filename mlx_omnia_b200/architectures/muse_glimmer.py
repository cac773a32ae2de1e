"""Muse-Glimmer's text trunk as configuration, parts and tensor names.

Everything here is data for the generic engine: the configuration mirrors the
checkpoint's `text_config` keys (src/mlx_omnia/engine/models/muse_glimmer/config.py:13-48),
`model_spec` turns it into parts layer by layer
(src/mlx_omnia/engine/models/muse_glimmer/layers/block.py:11-39,
src/mlx_omnia/engine/models/muse_glimmer/layers/attention.py:20-47,
src/mlx_omnia/engine/models/muse_glimmer/model.py:42-106), and `tensor_name` maps the
file's names to the model's (src/mlx_omnia/engine/models/muse_glimmer/checkpoint.py:48-53,72-82).
The vision tower, the DFlash drafter and quantised files are outside this engine.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from mlx_omnia_b200.config.hydrate import ConfigError, hydrate
from mlx_omnia_b200.parts.base import PartSpec
from mlx_omnia_b200.parts.model import LayerSpec, ModelSpec, ScheduleEntry
from mlx_omnia_b200.registry import Architecture, register_architecture

SLIDING = "sliding_attention"
FULL = "full_attention"


@dataclass(frozen=True)
class MuseGlimmerRoPE:
    rope_theta: float
    rope_type: str = "default"


@dataclass(frozen=True)
class MuseGlimmerTextConfig:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    post_norm_eps: float
    sliding_window: int
    qk_scale_factor: float
    output_multiplier: float
    final_logit_softcapping: float
    layer_types: tuple[str, ...]
    layer_rope_theta: tuple[float, ...]  # per layer; 0 switches rotation off for that layer
    rope_parameters: MuseGlimmerRoPE | None = None
    eos_token_id: int | tuple[int, ...] = ()
    tie_word_embeddings: bool = False
    max_position_embeddings: int | None = None

    def __post_init__(self) -> None:
        problems = []
        unknown = set(self.layer_types) - {SLIDING, FULL}
        if unknown:
            problems.append(f"unknown layer types {sorted(unknown)}")
        if len(self.layer_types) != self.num_hidden_layers:
            problems.append(f"layer_types has {len(self.layer_types)} entries for {self.num_hidden_layers} layers")
        if len(self.layer_rope_theta) != len(self.layer_types):
            problems.append("layer_rope_theta and layer_types disagree on layer count")
        if self.num_key_value_heads <= 0 or self.num_attention_heads % max(self.num_key_value_heads, 1):
            problems.append(f"{self.num_attention_heads} query heads do not divide into "
                            f"{self.num_key_value_heads} key/value heads")
        if self.head_dim % 2 or self.head_dim <= 0:
            problems.append(f"head_dim {self.head_dim} must be even and positive")
        if any(theta < 0 for theta in self.layer_rope_theta):
            problems.append("layer_rope_theta holds a negative base")
        if self.rope_parameters is not None and self.rope_parameters.rope_type != "default":
            problems.append(f"rope_type {self.rope_parameters.rope_type!r} is not supported")
        if self.rms_norm_eps <= 0 or self.post_norm_eps <= 0:
            problems.append("norm eps must be positive")
        if self.final_logit_softcapping <= 0:
            problems.append("final_logit_softcapping must be positive")
        if SLIDING in self.layer_types and self.sliding_window < 1:
            problems.append("sliding_window must be at least 1")
        for name in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "vocab_size"):
            if getattr(self, name) <= 0:
                problems.append(f"{name} must be positive")
        if problems:
            raise ConfigError("muse_glimmer text_config: " + "; ".join(problems))

    @property
    def eos(self) -> tuple[int, ...]:
        return self.eos_token_id if isinstance(self.eos_token_id, tuple) else (self.eos_token_id,)


@dataclass(frozen=True)
class MuseGlimmerConfig:
    text_config: MuseGlimmerTextConfig
    image_token_id: int = -1

    @property
    def tie_word_embeddings(self) -> bool:
        return self.text_config.tie_word_embeddings


def parse(raw: dict[str, Any]) -> MuseGlimmerConfig:
    """Read config.json. The reference requires the nested `text_config`
    (src/mlx_omnia/engine/models/muse_glimmer/config.py:79-85); a flat file with the
    same keys at the top level is accepted as well."""
    if raw.get("model_type") not in (None, "muse_glimmer"):
        raise ConfigError(f"expected model_type 'muse_glimmer', got {raw.get('model_type')!r}")
    if "text_config" in raw:
        return hydrate(MuseGlimmerConfig, raw)
    return MuseGlimmerConfig(text_config=hydrate(MuseGlimmerTextConfig, raw))


def model_spec(config: MuseGlimmerConfig) -> ModelSpec:
    c = config.text_config
    layers = []
    for index, (kind, theta) in enumerate(zip(c.layer_types, c.layer_rope_theta)):
        position = PartSpec("rotary", {"dims": c.head_dim, "theta": theta}) if theta else PartSpec("none")
        mixer = PartSpec("gqa_attention", {
            "hidden": c.hidden_size, "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
            "head_dim": c.head_dim, "scale": c.qk_scale_factor * c.head_dim ** -0.5,
            "window": c.sliding_window if kind == SLIDING else None, "qk_norm_eps": c.rms_norm_eps,
            "gated": True, "position": position})
        feed_forward = PartSpec("gated_mlp", {"hidden": c.hidden_size, "inner": c.intermediate_size})
        pre = PartSpec("rms_norm", {"size": c.hidden_size, "eps": c.rms_norm_eps, "weight": "centred"})
        post = PartSpec("rms_norm", {"size": c.hidden_size, "eps": c.post_norm_eps, "weight": "centred"})
        block = PartSpec("sandwich", {"mixer": mixer, "feed_forward": feed_forward, "norms": {
            "input_layernorm": pre, "post_attention_layernorm": post,
            "pre_feedforward_layernorm": pre, "post_feedforward_layernorm": post}})
        layers.append(LayerSpec(block, f"model.layers.{index}"))
    return ModelSpec(
        embedding=PartSpec("token_embedding", {"vocab": c.vocab_size, "hidden": c.hidden_size,
                                               "norm_eps": c.rms_norm_eps}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rms_norm", {"size": c.hidden_size, "eps": c.rms_norm_eps, "weight": "plain"}),
        head=PartSpec("lm_head", {"vocab": c.vocab_size, "hidden": c.hidden_size, "tied": c.tie_word_embeddings,
                                  "multiplier": c.output_multiplier, "softcap": c.final_logit_softcapping}),
    )


_TRUNK_PREFIX = "model.language_model."
_IGNORED_PREFIXES = ("model.vision_tower.", "model.vision_adapter.", "model.vision_projection.",
                     "visual.", "vision_adapter.", "vision_projection.")


def tensor_name(file_name: str) -> str | None:
    if file_name.startswith(_IGNORED_PREFIXES):
        return None
    if file_name.startswith(_TRUNK_PREFIX):
        return "model." + file_name[len(_TRUNK_PREFIX):]
    return file_name


def random_tensors(config: MuseGlimmerConfig, seed: int) -> dict[str, torch.Tensor]:
    """Float32 tensors under the checkpoint's own names: matrices N(0, 0.02); the
    centred block norms store w = N(0, 0.01) (so they multiply by 1 + w); the final
    norm stores 1 + N(0, 0.01). Drawn on the CPU in a fixed order from one generator."""
    c = config.text_config
    g = torch.Generator().manual_seed(seed)

    def normal(*shape: int, std: float) -> torch.Tensor:
        return torch.randn(*shape, generator=g, dtype=torch.float32) * std

    q, kv = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim
    out = {_TRUNK_PREFIX + "embed_tokens.weight": normal(c.vocab_size, c.hidden_size, std=0.02)}
    for i in range(c.num_hidden_layers):
        p = f"{_TRUNK_PREFIX}layers.{i}."
        out[p + "self_attn.q_proj.weight"] = normal(q, c.hidden_size, std=0.02)
        out[p + "self_attn.k_proj.weight"] = normal(kv, c.hidden_size, std=0.02)
        out[p + "self_attn.v_proj.weight"] = normal(kv, c.hidden_size, std=0.02)
        out[p + "self_attn.gate_proj.weight"] = normal(q, c.hidden_size, std=0.02)
        out[p + "self_attn.o_proj.weight"] = normal(c.hidden_size, q, std=0.02)
        out[p + "mlp.gate_proj.weight"] = normal(c.intermediate_size, c.hidden_size, std=0.02)
        out[p + "mlp.up_proj.weight"] = normal(c.intermediate_size, c.hidden_size, std=0.02)
        out[p + "mlp.down_proj.weight"] = normal(c.hidden_size, c.intermediate_size, std=0.02)
        for norm in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm",
                     "post_feedforward_layernorm"):
            out[p + norm + ".weight"] = normal(c.hidden_size, std=0.01)
    out[_TRUNK_PREFIX + "norm.weight"] = 1.0 + normal(c.hidden_size, std=0.01)
    if not c.tie_word_embeddings:
        out["lm_head.weight"] = normal(c.vocab_size, c.hidden_size, std=0.02)
    return out


ARCHITECTURE = Architecture(
    name="muse_glimmer",
    config_class=MuseGlimmerConfig,
    parse=parse,
    model_spec=model_spec,
    tensor_name=tensor_name,
    random_tensors=random_tensors,
    stop_tokens=lambda config: config.text_config.eos,
    dropped_tensors=lambda config: ("lm_head.weight",) if config.tie_word_embeddings else (),
    max_context=lambda config: config.text_config.max_position_embeddings,
)

register_architecture(ARCHITECTURE, "muse_glimmer", "MuseGlimmerForConditionalGeneration", "MuseGlimmerForCausalLM")
