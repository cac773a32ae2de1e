"""Parts a decoder is put together from, and the registries they are found in."""

from mlx_omnia_b200.parts import attention, blocks, embedding, feedforward, norms, positions  # noqa: F401 (register)
from mlx_omnia_b200.parts.base import (KVSpec, KVView, LayerContext, PartSpec, Runtime, StateSpec, StepContext,
                                       TensorSpec, register_block, register_embedding, register_feed_forward,
                                       register_head, register_mixer, register_norm, register_position)
from mlx_omnia_b200.parts.model import CacheNeed, DecoderModel, LayerSpec, ModelSpec, ScheduleEntry

__all__ = ["CacheNeed", "DecoderModel", "KVSpec", "KVView", "LayerContext", "LayerSpec", "ModelSpec", "PartSpec",
           "Runtime", "ScheduleEntry", "StateSpec", "StepContext", "TensorSpec", "register_block",
           "register_embedding", "register_feed_forward", "register_head", "register_mixer", "register_norm",
           "register_position"]
